"""CPU: the FFW4 / OPSC2 producer (fastface_b200/producer.py) against golden vectors made by the
reference's own Python functions, fold identities on single layers, and a round trip of a produced
model through this library's loader, the oracle and (where it can run) the unmodified reference,
whose int8 embedding must agree with the fp32 network the files were produced from."""
import os
import struct

import numpy as np
import pytest

from conftest import GOLDEN
import fastface_b200 as ff
from fastface_b200 import producer as P
from fastface_b200 import synth
from oracle import ffo


def test_quantiser_and_percentile_match_the_reference_functions():
    g = np.load(os.path.join(GOLDEN, "producer_golden.npz"))
    w_int, scales = P.quantize_per_channel_int8(g["w"])
    assert w_int.dtype == np.int8 and scales.dtype == np.float32
    assert np.array_equal(w_int, g["w_int"]) and np.array_equal(scales.view(np.uint32), g["scales"].view(np.uint32))
    for p in (99.9, 99.0, 50.0):
        got = P.percentile_scales(g["absmax"], p)
        assert np.array_equal(got.view(np.uint32), g[f"pct_{p}"].view(np.uint32)), p


def test_conv_fold_moves_the_input_scale_into_the_weights():
    """y = conv(w, x_q * S_a) in fp32 must equal (sum x_q * w_int) * scale[oc] up to the weight rounding:
    the fold multiplies by S_a[ci] (prepare_weights_v3.py:206-217), so the run-time input scale is 1."""
    rng = np.random.default_rng(1)
    cout, cin = 8, 6
    w = (rng.standard_normal((cout, cin, 3, 3)) * 0.2).astype(np.float32)
    s_a = rng.uniform(0.005, 0.05, cin).astype(np.float32)
    xq = rng.integers(-127, 128, size=(5, 5, cin)).astype(np.float32)
    w_int, scales = P.fold_conv(w, s_a)
    y_ref = P._conv_nhwc(xq * s_a, w, np.zeros(cout, np.float32), 1, 1)
    y_q = P._conv_nhwc(xq, w_int.astype(np.float32), np.zeros(cout, np.float32), 1, 1) * scales
    bound = 0.5 * scales * np.abs(xq).sum() + 1e-4         # half a quantisation step per weight, worst case
    assert np.all(np.abs(y_ref - y_q) <= bound)
    assert np.abs(y_ref - y_q).max() < 0.05 * np.abs(y_ref).max()
    # without a per-channel scale of the right length the weights stay unfolded (the reference's fallback)
    w_int2, scales2 = P.fold_conv(w, None)
    assert np.array_equal(w_int2, P.quantize_per_channel_int8(w)[0])


def test_gemm_fold_uses_the_flatten_order_and_the_trailing_bn():
    rng = np.random.default_rng(2)
    c, spatial, n = 8, 4, 5
    w = (rng.standard_normal((n, c * spatial)) * 0.1).astype(np.float32)
    b = (rng.standard_normal(n) * 0.1).astype(np.float32)
    s_c = rng.uniform(0.01, 0.05, c).astype(np.float32)
    bn = (rng.uniform(0.5, 1.5, n).astype(np.float32), (rng.standard_normal(n) * 0.1).astype(np.float32))
    aq = rng.integers(-127, 128, size=(c * spatial,)).astype(np.float32)     # int8 activations in k = c*spatial + hw order
    w_int, scales, b_eff = P.fold_gemm(w, b, s_c, bn)
    want = (w @ (aq * np.repeat(s_c, spatial)) + b) * bn[0] + bn[1]
    got = (w_int.astype(np.float32) @ aq) * scales + b_eff
    assert np.abs(want - got).max() < 0.02 * np.abs(want).max() + 1e-3


@pytest.fixture(scope="module")
def produced(tmp_path_factory):
    root = str(tmp_path_factory.mktemp("produced"))
    ops = P.synth_float_model(seed=7)
    calib = synth.faces(3, seed=900)
    path = P.write_model(root, ops, calib, percentile=99.9)
    return root, path, ops


def test_produced_files_have_the_reference_layout(produced):
    root, path, ops = produced
    d = open(path, "rb").read()
    assert d[:4] == b"FFW4" and struct.unpack_from("<I", d, 4)[0] == 177
    assert d[8] == synth.OP_CONV and struct.unpack_from("<6H", d, 9) == (3, 64, 3, 3, 1, 1)
    assert len(d) == 43723361                          # the size of any FFW4 file of this 177-op architecture
    v2 = open(os.path.join(root, "models", "op_scales_v2.bin"), "rb").read()
    assert v2[:5] == b"OPSC2" and struct.unpack_from("<II", v2, 5) == (177, 3)
    v1 = open(os.path.join(root, "models", "op_scales.bin"), "rb").read()
    assert v1[:4] == b"OPSC" and struct.unpack_from("<I", v1, 4)[0] == 177 and len(v1) == 12 + 4 * 177


def test_produced_model_loads_and_agrees_with_its_fp32_source(built_lib, produced):
    """The produced files go through this library's loader and planner (fastface_create gets as far as
    looking for a GPU), the oracle runs them, and the int8 embedding agrees with the fp32 network they
    were produced from: a wrong fold (scale on the wrong side, wrong flatten order, BN not folded)
    would leave the cosine near zero."""
    root, path, ops = produced
    lib = ff.load_library()
    old = os.getcwd()
    os.chdir(root)
    try:
        h = lib.fastface_create(path.encode())
        err = lib.fastface_last_error().decode()
        if h:
            lib.fastface_destroy(h)
    finally:
        os.chdir(old)
    assert h or "no CUDA device" in err, err          # parsed and planned; only the device is missing here
    orc = ffo.Oracle(path, os.path.join(root, "models", "op_scales.bin"), os.path.join(root, "models", "op_scales_v2.bin"))
    faces = synth.faces(2, seed=901)
    emb_q = orc.forward(faces, ffo.CONTRACT)
    for k in range(2):
        emb_f = P.float_forward(ops, faces[k])
        cos = float(np.dot(emb_q[k], emb_f) / (np.linalg.norm(emb_q[k]) * np.linalg.norm(emb_f)))
        assert cos > 0.95, cos
    if ffo.ref_available():
        ref = ffo.RefLib(root, path)
        want = ref.embed(faces[0])
        ref.close()
        assert np.array_equal(want, emb_q[0])          # the unmodified reference accepts the files and agrees bit for bit
