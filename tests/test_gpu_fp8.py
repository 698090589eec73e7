"""GPU parity of Fp8Quantize / Fp8Dequantize / Fp8Matmul and the delayed-scaling update.
The reference has no FP8 test: parity here is against the CPU restatement only (unpinned)."""
import importlib

import numpy as np
import pytest
import torch

import itex_oracle as o
from gpu_util import dev, host, modules

pytestmark = pytest.mark.gpu


def test_quantize_dequantize_bit_exact():
    itex, K, ops = modules()
    rng = np.random.default_rng(21)
    for dt in (torch.float32, torch.bfloat16, torch.float16):
        x = torch.from_numpy((rng.standard_normal((257, 129)) * 3).astype(np.float32)).to(dt).cuda()
        x[0, 0] = 1000.0   # saturates to 448
        x[0, 1] = -1e5
        x[0, 2] = 0.0
        amax = torch.zeros((16, 3), device="cuda")
        scale = torch.tensor([1.0, 8.0, 0.5], device="cuda")
        for idx in (0, 1, 2):
            y = ops.Fp8Quantize(x, amax[0], scale, idx, "E4M3")
            ref_amax = np.zeros(3, np.float32)
            ref = o.fp8_quantize(host(x), ref_amax, host(scale), idx, "E4M3")
            np.testing.assert_array_equal(host(y).view(np.uint8), ref)
            assert float(amax[0, idx]) == float(ref_amax[idx])
        yd = ops.Fp8Dequantize(y, 1.0 / scale, 2, "E4M3", out_dtype="bfloat16" if dt == torch.bfloat16 else "float")
        refd = o.fp8_dequantize(ref, host(1.0 / scale), 2, "E4M3", "bfloat16" if dt == torch.bfloat16 else "float")
        np.testing.assert_array_equal(host(yd), refd)
    # e5m2 and NaN stay NaN; amax is a running maximum
    x = torch.tensor([1.0, float("nan"), 70000.0, -3.0], device="cuda")
    amax = torch.tensor([5.0], device="cuda")
    y = ops.Fp8Quantize(x, amax, torch.ones(1, device="cuda"), 0, "E5M2")
    back = o.fp8_to_f32(host(y).view(np.uint8), "E5M2")
    assert back[0] == 1.0 and np.isnan(back[1]) and back[2] == 57344.0 and back[3] == -3.0


@pytest.mark.parametrize("m,k,n", [(256, 512, 384), (100, 144, 72), (64, 4096, 256)])
@pytest.mark.parametrize("sum_dtype", ["float", "bfloat16"])
def test_fp8_matmul_vs_oracle(m, k, n, sum_dtype):
    """1e-2 relative against the restated dequantize->matmul path; and no further from an exact f64 sum
    than that restatement is."""
    itex, K, ops = modules()
    rng = np.random.default_rng(m + n)
    A = rng.standard_normal((m, k)).astype(np.float32)
    W = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    scale = np.array([64.0, 4096.0, 16.0], np.float32)
    sinv = (1.0 / scale).astype(np.float32)
    amax = np.zeros(3, np.float32)
    qa = o.fp8_quantize(A, amax, scale, 0)
    qw = o.fp8_quantize(W, amax, scale, 1)
    tdt = torch.bfloat16 if sum_dtype == "bfloat16" else torch.float32
    b_t = torch.from_numpy(bias).to(tdt).cuda()
    bias_r = host(b_t)
    dsinv, dscale = dev(sinv), dev(scale)
    damax = torch.zeros(3, device="cuda")
    dummy = torch.zeros(1, dtype=tdt, device="cuda")
    for tb in (False, True):
        wq = qw.T.copy() if tb else qw
        out = ops.Fp8Matmul(dev(qa).view(torch.int8), dev(wq).view(torch.int8), b_t, dummy, dsinv, dsinv, damax, dscale, 0, 1,
                            transpose_b=tb, use_bias=True, sum_dtype=sum_dtype, out_dtype=sum_dtype)
        ref = o.fp8_matmul(qa, wq, bias_r, None, sinv, sinv, None, None, transpose_b=tb, use_bias=True, sum_dtype=sum_dtype,
                           out_dtype=sum_dtype)
        got = host(out)
        denom = np.abs(ref).max()
        assert np.abs(got - ref).max() / denom < 1e-2
        exact = (o.fp8_to_f32(qa).astype(np.float64) * sinv[0]) @ (o.fp8_to_f32(qw).astype(np.float64) * sinv[1]) + bias_r
        assert np.abs(got - exact).max() <= np.abs(ref - exact).max() * 1.5 + 1e-6 * denom
    # fp8 output with amax, and post_add
    pa = torch.from_numpy(rng.standard_normal((m, n)).astype(np.float32)).to(tdt).cuda()
    out = ops.Fp8Matmul(dev(qa).view(torch.int8), dev(qw).view(torch.int8), b_t, pa, dsinv, dsinv, damax, dscale, 0, 1, 2,
                        use_bias=True, has_post_add=True, sum_dtype=sum_dtype, out_dtype="int8", fp8_dtype_c="E4M3")
    ref_amax = np.zeros(3, np.float32)
    ref = o.fp8_matmul(qa, qw, bias_r, host(pa), sinv, sinv, ref_amax, scale, fp8_meta_index_c=2, use_bias=True, has_post_add=True,
                       sum_dtype=sum_dtype, out_dtype="int8")
    got = o.fp8_to_f32(host(out).view(np.uint8))
    want = o.fp8_to_f32(ref)
    # accumulation order differs, so a value may land on the neighbouring e4m3 code: allow one code of distance
    assert np.abs(got - want).max() <= np.abs(want).max() * 2 ** -3 and (got != want).mean() < 0.02
    assert abs(float(damax[2]) - float(ref_amax[2])) <= 1e-2 * float(ref_amax[2])


def test_delayed_scaling_20_steps_matches_oracle():
    """DelayedScaling(margin=0, amax_history_len=16, 'max'): 20 steps with fresh inputs, scale lags one step."""
    itex, K, ops = modules()
    fp8 = importlib.import_module("itex_b200.fp8")
    rng = np.random.default_rng(1239)
    k, n, m = 256, 192, 128
    W = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
    layer = fp8.Fp8Dense(torch.from_numpy(W).to(torch.bfloat16).cuda(), recipe=fp8.DelayedScaling(amax_history_len=16), out_dtype="bfloat16")
    Wb = host(layer.kernel)
    hist = np.zeros((16, 3), np.float32)
    scale = np.ones(3, np.float32)
    for step in range(20):
        A = (rng.standard_normal((m, k)) * (1.0 + step)).astype(np.float32)
        At = torch.from_numpy(A).to(torch.bfloat16).cuda()
        out = layer(At)
        hist, scale, sinv = o.fp8_amax_and_scale_update(hist, scale, 448.0, 0, "max")
        qa = o.fp8_quantize(host(At), hist[0], scale, 0)
        qw = o.fp8_quantize(Wb, hist[0], scale, 1)
        ref = o.fp8_matmul(qa, qw, None, None, sinv, sinv, None, None, sum_dtype="bfloat16", out_dtype="bfloat16")
        np.testing.assert_array_equal(host(layer.meta.scale), scale)
        np.testing.assert_array_equal(host(layer.meta.scale_inv), sinv)
        np.testing.assert_array_equal(host(layer.meta.amax_history), hist)
        got = host(out)
        assert np.abs(got - ref).max() / np.abs(ref).max() < 1e-2
    assert scale[0] < 64 and scale[1] >= 1024  # scales moved away from 1 in both directions
    sd = layer.meta.state_dict()
    layer.meta.amax_history.zero_()
    layer.meta.load_state_dict(sd)
    np.testing.assert_array_equal(host(layer.meta.amax_history), hist)
    for algo in ("max", "most_recent"):
        h = np.abs(rng.standard_normal((16, 5))).astype(np.float32) * np.array([1, 0, 1000, 1e-6, 448], np.float32)
        h[3, 2] = np.inf
        s = np.array([2.0, 4.0, 8.0, 16.0, 32.0], np.float32)
        dh, ds, dsi = dev(h), dev(s), torch.zeros(5, device="cuda")
        K.fp8_amax_and_scale_update(dh, ds, dsi, 448.0, 0.0, algo)
        rh, rs, rsi = o.fp8_amax_and_scale_update(h, s, 448.0, 0, algo)
        np.testing.assert_array_equal(host(dh), rh)
        np.testing.assert_array_equal(host(ds), rs)
        np.testing.assert_array_equal(host(dsi), rsi)


def test_column_parallel_shards_reassemble_the_full_product():
    """Column-parallel FP8 linear: the [M, N/g] results of g weight shards (each with the shared, max-combined
    scaling state) concatenated along N equal the unsharded [M, N] result bit for bit."""
    itex, K, ops = modules()
    fp8 = importlib.import_module("itex_b200.fp8")
    rng = np.random.default_rng(5)
    m, k, n, g = 128, 256, 384, 4
    W = torch.from_numpy((rng.standard_normal((n, k)) * 0.02).astype(np.float32)).to(torch.bfloat16).cuda()   # [N, K]
    full = fp8.Fp8Dense(W, recipe=fp8.DelayedScaling(amax_history_len=4), out_dtype="bfloat16", weight_layout="nk")
    shards = [fp8.Fp8Dense(W[r * (n // g):(r + 1) * (n // g)].contiguous(), recipe=fp8.DelayedScaling(amax_history_len=4),
                           out_dtype="bfloat16", weight_layout="nk") for r in range(g)]
    for step in range(6):
        A = torch.from_numpy((rng.standard_normal((m, k)) * (1 + step)).astype(np.float32)).to(torch.bfloat16).cuda()
        ref = full(A)
        outs = [sh(A) for sh in shards]
        amax = torch.stack([sh.meta.amax_history[0] for sh in shards]).amax(dim=0)   # what all_reduce(MAX) leaves on every rank
        for sh in shards:
            sh.meta.amax_history[0].copy_(amax)
        assert bool((torch.cat(outs, dim=1) == ref).all())
        assert bool((shards[0].meta.amax_history == full.meta.amax_history).all())
        assert bool((shards[-1].meta.scale == full.meta.scale).all())


def test_fp8_gelu_and_layernorm():
    """Fp8Gelu and Fp8LayerNorm against the restatement: FP8 outputs within one FP8 step (1e-2 relative is the bar; the
    device's tanh / rsqrt and fp32 summation order differ from the float64 restatement in the last bits, which can move a
    value across an FP8 rounding boundary), real outputs and the row statistics at 1e-5."""
    itex, K, ops = modules()
    rng = np.random.default_rng(33)
    x = (rng.standard_normal((300, 1000)) * 2).astype(np.float32)
    for dt in (torch.float32, torch.bfloat16):
        X = torch.from_numpy(x).to(dt).cuda()
        amax = torch.zeros(3, device="cuda")
        scale = torch.tensor([1.0, 16.0, 0.5], device="cuda")
        y = ops.Fp8Gelu(X, amax, scale, 1, "E4M3")
        ref_amax = np.zeros(3, np.float32)
        ref = o.fp8_gelu(host(X), ref_amax, host(scale), 1, "E4M3")
        got_f, ref_f = o.fp8_to_f32(host(y).view(np.uint8), "E4M3"), o.fp8_to_f32(ref, "E4M3")
        assert (host(y).view(np.uint8) != ref).mean() < 2e-3
        np.testing.assert_allclose(got_f, ref_f, rtol=0.13, atol=2e-3)        # at most the neighbouring FP8 value
        np.testing.assert_allclose(float(amax[1]), float(ref_amax[1]), rtol=1e-6)
        assert float(amax[0]) == 0.0 and float(amax[2]) == 0.0
    gamma = (1 + 0.1 * rng.standard_normal(1000)).astype(np.float32)
    beta = (0.1 * rng.standard_normal(1000)).astype(np.float32)
    X, G, B = dev(x), dev(gamma), dev(beta)
    z, mu, rs = ops.Fp8LayerNorm(X, G, B, torch.zeros(1, device="cuda"), torch.ones(1, device="cuda"), 0, epsilon=1e-5, out_dtype="float")
    zr, mur, rsr = o.fp8_layernorm(x, gamma, beta, None, None, 0, epsilon=1e-5, out_dtype="float")
    np.testing.assert_allclose(host(mu), mur, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(host(rs), rsr, rtol=1e-5)
    np.testing.assert_allclose(host(z), zr, rtol=1e-5, atol=1e-5)
    amax = torch.zeros(2, device="cuda")
    scale = torch.tensor([1.0, 32.0], device="cuda")
    z8, mu, rs = ops.Fp8LayerNorm(X.to(torch.bfloat16), G, B, amax, scale, 1, epsilon=1e-5, fp8_dtype="E4M3")
    ref_amax = np.zeros(2, np.float32)
    z8r, _, _ = o.fp8_layernorm(host(X.to(torch.bfloat16)), gamma, beta, ref_amax, host(scale), 1, epsilon=1e-5)
    assert z8.dtype == torch.int8 and (host(z8).view(np.uint8) != z8r).mean() < 2e-3
    np.testing.assert_allclose(o.fp8_to_f32(host(z8).view(np.uint8), "E4M3"), o.fp8_to_f32(z8r, "E4M3"), rtol=0.13, atol=2e-3)
    np.testing.assert_allclose(float(amax[1]), float(ref_amax[1]), rtol=1e-5)
