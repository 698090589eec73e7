"""INT8 ResNet-50 v1.5 graph runner: every node's output is bit-identical to the oracle's result for the
same inputs (small image so the NumPy oracle finishes in seconds), and a CUDA-graph replay equals eager."""
import importlib

import numpy as np
import pytest
import torch

import itex_oracle as o
from gpu_util import host, modules

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("image", [64, 224])
def test_every_node_matches_the_oracle_and_graph_replay_matches_eager(image):
    """image 64: a small case; image 224: the configuration's real resolution (batch 2), where the layers meet the tile
    counts, the 256-byte-pitch stem patches and the multi-wave tile walk of the full-size graph."""
    itex, K, ops = modules()
    rn = importlib.import_module("itex_b200.resnet50")
    net = rn.ResNet50Int8(device="cuda", seed=1237, num_classes=100)
    assert 4.0e9 < net.macs_per_image(224) < 4.2e9     # from the layer table: 53 convolutions + the classifier
    assert sum(1 for _ in net.conv_nodes()) == 53
    x = torch.randint(0, 256, (2, image, image, 3), dtype=torch.uint8, device="cuda", generator=torch.Generator("cuda").manual_seed(3))
    net.forward(x, calibrate=True)
    trace = []
    logits = net.forward(x, trace=trace)
    assert logits.shape == (2, 100) and bool(torch.isfinite(logits).all())
    n_conv = n_sum_u8 = n_sum_s8 = 0
    for node, inp, out in trace:
        if node == "maxpool":
            continue
        if node == "avgpool":
            q, mn, mx = inp
            ref = o.quantized_pool2d(host(q), (1, q.shape[1], q.shape[2], 1), (1, q.shape[1], q.shape[2], 1), "VALID", avg=True)
            np.testing.assert_array_equal(host(out[0]), ref)
            assert (out[1], out[2]) == (mn, mx)
            continue
        if node == "fc":
            feat, mn, mx = inp
            ref, _, _ = o.quantized_matmul_with_bias(host(feat), host(net.fc_w), host(net.fc_b), mn, mx, net.fc_range[0], net.fc_range[1],
                                                     0.0, 0.0, toutput="float", input_quant_mode="SCALED", scaled_bias_mode="intended")
            np.testing.assert_array_equal(host(out), ref)
            continue
        q, mn, mx, sm, smn, smx = inp
        ref, rmn, rmx = o.quantized_conv2d(host(q), host(node.filter), host(node.bias), mn, mx, node.min_filter, node.max_filter,
                                           node.min_out, node.max_out, strides=(1, node.stride, node.stride, 1), padding="SAME",
                                           out_type=node.out_type, relu=node.relu, summand=None if sm is None else host(sm),
                                           min_summand=smn, max_summand=smx)
        np.testing.assert_array_equal(host(out[0]), ref, err_msg=node.name)
        assert (out[1], out[2]) == (rmn, rmx)
        n_conv += 1
        n_sum_u8 += int(sm is not None and sm.dtype == torch.uint8)
        n_sum_s8 += int(sm is not None and sm.dtype == torch.int8)
        frac_sat = float((out[0] == (255 if node.relu else 127)).float().mean())
        assert frac_sat < 0.02, (node.name, frac_sat)     # calibrated ranges are neither saturated ...
    assert (n_conv, n_sum_u8, n_sum_s8) == (53, 12, 4)     # identity shortcuts are u8 summands, projections s8
    # max-pool node against the oracle
    stem_out = trace[0][2]
    mp = [t for t in trace if t[0] == "maxpool"][0][2]
    np.testing.assert_array_equal(host(mp[0]), o.quantized_pool2d(host(stem_out[0]), (1, 3, 3, 1), (1, 2, 2, 1), "SAME"))
    # the whole forward in one CUDA graph gives the same logits
    g, static_out = net.capture(x)
    g.replay()
    torch.cuda.synchronize()
    assert bool((static_out == logits).all())


def test_pooling_ops_match_oracle_on_odd_shapes():
    itex, K, ops = modules()
    rng = np.random.default_rng(4)
    for (n, h, w, c, k, s, pad, avg, dt) in ((2, 11, 9, 32, 3, 2, "SAME", False, np.uint8), (1, 7, 7, 48, 7, 7, "VALID", True, np.uint8),
                                             (2, 10, 10, 5, 2, 2, "VALID", False, np.int8), (1, 9, 9, 16, 3, 1, "SAME", True, np.int8),
                                             (2, 8, 12, 32, 3, 2, "SAME", False, np.int8),      # signed max, 16 channels per thread
                                             (1, 12, 13, 16, 11, 1, "VALID", True, np.uint8),    # window rows longer than one batch of loads
                                             (1, 12, 13, 16, 11, 2, "SAME", False, np.int8)):
        x = rng.integers(0, 256, (n, h, w, c)).astype(np.uint8) if dt == np.uint8 else rng.integers(-128, 128, (n, h, w, c)).astype(np.int8)
        op = ops.Op("_ITEXQuantizedAvgPool" if avg else "_ITEXQuantizedMaxPool", T="quint8" if dt == np.uint8 else "qint8",
                    ksize=[1, k, k, 1], strides=[1, s, s, 1], padding=pad)
        out, mn, mx = op(torch.from_numpy(x).cuda(), -1.5, 2.5)
        np.testing.assert_array_equal(host(out), o.quantized_pool2d(x, (1, k, k, 1), (1, s, s, 1), pad, avg=avg))
        assert (mn, mx) == (-1.5, 2.5)
