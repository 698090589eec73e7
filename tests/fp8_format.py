"""FP8 formats written out from their bit layouts, independent of ml_dtypes and of the library under test.

e4m3fn: 1 sign, 4 exponent (bias 7), 3 mantissa bits; no infinity; S.1111.111 is NaN; largest finite 448.
e5m2:   1 sign, 5 exponent (bias 15), 2 mantissa bits; S.11111.00 is infinity, S.11111.{01,10,11} NaN; largest finite 57344.

The float -> FP8 rule checked against is the one itex/core/utils/float8.h:651-766 states for its default
(kSaturate = true, kTruncate = false): round to nearest, ties to the even code; a finite value that rounds
beyond the largest finite code saturates to it; NaN stays NaN; an infinite input gives numeric_limits::infinity()
of the target, which is NaN for e4m3fn (float8.h:313-315) and +-infinity for e5m2 (float8.h:400).
"""
import numpy as np

FORMATS = {"E4M3": dict(ebits=4, mbits=3, bias=7), "E5M2": dict(ebits=5, mbits=2, bias=15)}


def decode(code: int, fmt: str) -> float:
    """Value of one 8-bit code, from the bit layout."""
    f = FORMATS[fmt]
    mb, eb, bias = f["mbits"], f["ebits"], f["bias"]
    sign = -1.0 if code & 0x80 else 1.0
    e = (code >> mb) & ((1 << eb) - 1)
    m = code & ((1 << mb) - 1)
    if fmt == "E4M3":
        if e == 15 and m == 7:
            return float("nan")
    else:
        if e == 31:
            return sign * float("inf") if m == 0 else float("nan")
    if e == 0:
        return sign * m * 2.0 ** (1 - bias - mb)
    return sign * (1.0 + m / float(1 << mb)) * 2.0 ** (e - bias)


def table(fmt: str) -> np.ndarray:
    """All 256 decoded values as float64 (exact: every FP8 value is a float32)."""
    return np.array([decode(c, fmt) for c in range(256)], np.float64)


def finite_positive_codes(fmt: str):
    """(codes, values) of the non-negative finite codes in increasing order of value."""
    codes = [c for c in range(128) if np.isfinite(decode(c, fmt))]
    vals = [decode(c, fmt) for c in codes]
    assert vals == sorted(vals)
    return codes, vals


def encode(x: float, fmt: str) -> int:
    """float -> code by exhaustive nearest search over the finite codes (ties to the even code), saturating."""
    x = float(np.float32(x))
    if np.isnan(x):
        return 0x7F
    sign = 0x80 if np.signbit(x) else 0
    if np.isinf(x):
        return sign | (0x7F if fmt == "E4M3" else 0x7C)
    codes, vals = finite_positive_codes(fmt)
    a = abs(x)
    if a >= vals[-1]:
        return sign | codes[-1]
    hi = int(np.searchsorted(vals, a, side="left"))   # vals[hi-1] < a <= vals[hi]
    if vals[hi] == a:
        return sign | codes[hi]
    lo = hi - 1
    dl, dh = a - vals[lo], vals[hi] - a              # exact in float64
    if dl < dh:
        return sign | codes[lo]
    if dh < dl:
        return sign | codes[hi]
    return sign | (codes[lo] if codes[lo] % 2 == 0 else codes[hi])


def probe_inputs(fmt: str) -> np.ndarray:
    """float32 inputs that exercise every rounding decision: each finite value, each midpoint between neighbours
    (a tie), the float32 neighbours of each midpoint, values around and far beyond the largest finite code,
    infinities, NaN and signed zeros; all with both signs."""
    _, vals = finite_positive_codes(fmt)
    xs = []
    for i, v in enumerate(vals):
        xs.append(v)
        if i + 1 < len(vals):
            mid = np.float32((v + vals[i + 1]) / 2.0)
            assert float(mid) == (v + vals[i + 1]) / 2.0
            xs += [mid, np.nextafter(mid, np.float32(0)), np.nextafter(mid, np.float32(np.inf))]
    top = vals[-1]
    step = top - vals[-2]
    xs += [top + step / 2, np.nextafter(np.float32(top + step / 2), np.float32(0)), top + step, top * 2, top * 1000, 3.0e38,
           vals[1] / 2, vals[1] / 4, np.nextafter(np.float32(vals[1] / 2), np.float32(1)), 1e-30, 0.0]
    xs = np.array(xs, np.float32)
    return np.concatenate([xs, -xs, np.array([np.inf, -np.inf, np.nan], np.float32)])


def encode_many(xs, fmt: str) -> np.ndarray:
    return np.array([encode(v, fmt) for v in np.asarray(xs, np.float32)], np.uint8)


def same_codes(got: np.ndarray, want: np.ndarray, fmt: str) -> bool:
    """Equality of codes, except that any NaN code equals any other NaN code."""
    got, want = np.asarray(got, np.uint8), np.asarray(want, np.uint8)
    t = table(fmt)
    gn, wn = np.isnan(t[got]), np.isnan(t[want])
    return bool(np.array_equal(gn, wn) and np.array_equal(got[~gn], want[~wn]))
