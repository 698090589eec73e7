"""Per-node parity of the INT8 BERT-shaped encoder: every quantize + int8 matmul node against the oracle."""
import importlib

import numpy as np
import pytest
import torch

import itex_oracle as o
from gpu_util import host, modules

pytestmark = pytest.mark.gpu


def test_encoder_nodes_match_oracle_and_graph_replay_matches_eager():
    itex, K, ops = modules()
    bert = importlib.import_module("itex_b200.bert_int8")
    enc = bert.BertInt8Encoder(layers=2, hidden=128, heads=4, ffn=512, seed=11)
    batch, seq = 4, 64
    gen = torch.Generator(device="cuda")
    gen.manual_seed(12)
    x = torch.randn((batch * seq, 128), generator=gen, device="cuda").to(torch.bfloat16)
    trace = []
    y = enc.forward(x, batch, seq, trace=trace)
    torch.cuda.synchronize()
    assert len(trace) == 8 and bool(torch.isfinite(y.float()).all())
    for lin, xin, q, range3, out in trace:
        xf = host(xin).astype(np.float32)
        # dynamic per-tensor range, reduced on the device, then QuantizeV2 SCALED / HALF_TO_EVEN to qint8
        qr, omin, omax = o.quantize_v2(xf, xf.min(), xf.max(), T="qint8", mode="SCALED", round_mode="HALF_TO_EVEN")
        r3 = host(range3)
        assert (r3[1], r3[2]) == (omin, omax)
        np.testing.assert_array_equal(host(q), qr)
        rw = host(lin.weight_range)
        fused = ["BiasAdd", "GeluApproximate"] if lin.gelu else ["BiasAdd"]
        ref, _, _ = o.quantized_fused_matmul(qr, host(lin.w_kn), host(lin.bias), omin, omax, -rw, rw, fused_ops=fused, t1="qint8",
                                             toutput="bfloat16", scaled_bias_mode="intended")
        got = host(out)
        if lin.gelu:  # transcendental post-op: a result within an ulp of a bf16 rounding tie may land on the neighbour
            np.testing.assert_allclose(got, ref, rtol=2.0 ** -7, atol=1e-6)
            assert (got != ref).mean() < 1e-2
        else:
            np.testing.assert_array_equal(got, ref)
    g, y_static = enc.capture(enc.forward, x, batch, seq)
    g.replay()
    torch.cuda.synchronize()
    np.testing.assert_array_equal(host(y_static), host(y))
    assert enc.int8_ops_per_token() == 2 * 2 * (128 * 384 + 128 * 128 + 128 * 512 + 512 * 128)


@pytest.mark.parametrize("name,k,n,gelu", [("qkv", 1024, 3072, False), ("attn_out", 1024, 1024, False), ("ffn_up", 1024, 4096, True),
                                           ("ffn_down", 4096, 1024, False)])
def test_bert_large_nodes_at_full_size(name, k, n, gelu):
    """The four int8 matmul nodes of a BERT-large layer at their real sizes (32 x 384 = 12288 tokens, hidden 1024, FFN
    4096): dynamic per-tensor range over the whole activation, QuantizeV2 to qint8, fused int8 matmul with per-channel
    scales, bias, (GELU,) bf16 output.  The quantized activation is compared in full, the matmul output on two 128-row
    slabs (one straddling a tile boundary, one at the end) against the oracle."""
    itex, K, ops = modules()
    bert = importlib.import_module("itex_b200.bert_int8")
    tokens = 32 * 384
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1238 + n)
    lin = bert.Int8Linear(name, k, n, gen, torch.device("cuda"), gelu=gelu)
    x = (torch.randn((tokens, k), generator=gen, device="cuda") * (1.5 if k == 4096 else 1.0)).to(torch.bfloat16)
    trace = []
    y = lin(x, trace)
    torch.cuda.synchronize()
    _, xin, q, range3, out = trace[0]
    xf = host(xin).astype(np.float32)
    qr, omin, omax = o.quantize_v2(xf, xf.min(), xf.max(), T="qint8", mode="SCALED", round_mode="HALF_TO_EVEN")
    r3 = host(range3)
    assert (r3[1], r3[2]) == (omin, omax)
    np.testing.assert_array_equal(host(q), qr)
    rw = host(lin.weight_range)
    fused = ["BiasAdd", "GeluApproximate"] if gelu else ["BiasAdd"]
    w_kn, bias = host(lin.w_kn), host(lin.bias)
    for rows in (slice(4032, 4160), slice(tokens - 128, tokens)):
        ref, _, _ = o.quantized_fused_matmul(qr[rows], w_kn, bias, omin, omax, -rw, rw, fused_ops=fused, t1="qint8", toutput="bfloat16",
                                             scaled_bias_mode="intended")
        got = host(out[rows])
        if gelu:  # transcendental post-op: a result within an ulp of a bf16 rounding tie may land on the neighbour
            np.testing.assert_allclose(got, ref, rtol=2.0 ** -7, atol=1e-6)
            assert (got != ref).mean() < 1e-2
        else:
            np.testing.assert_array_equal(got, ref)
    assert bool(torch.isfinite(y.float()).all())
