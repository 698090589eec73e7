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
