"""CPU: the oracle restatement is pinned against outputs of the unmodified reference.

Golden vectors (tests/golden/, made by make_golden.py from the reference compiled from
its own sources) travel with the repo; the live comparison against oracle/_ref runs
wherever that build exists and the host has AVX-VNNI.
"""
import os
import sys
import zlib

import numpy as np
import pytest

from conftest import GOLDEN, read_trace
from fastface_b200 import synth
from oracle import ffo

sys.path.insert(0, GOLDEN)
import make_golden  # noqa: E402


@pytest.mark.parametrize("mode,tag", [(ffo.CONTRACT, "contract"), (ffo.STRICT, "strict")])
def test_oracle_matches_reference_trace(oracle, mode, tag):
    """Every int32 accumulator tensor, int8 activation tensor and embedding of the
    reference's batched driver, by CRC, for B=2."""
    faces = synth.faces(2, seed=1)
    emb, recs = oracle.forward_crc(faces, mode)
    gold = read_trace(os.path.join(GOLDEN, f"ref_trace_b2_{tag}.txt"))
    assert len(gold) == 1 + 53 + 53 + 25 + 2
    assert recs == gold
    assert np.array_equal(emb, np.load(os.path.join(GOLDEN, f"ref_emb_b2_{tag}.npy")))


def test_oracle_per_tensor_fallback(oracle_per_tensor):
    """No OPSC2 file: per-tensor scales exactly as libfastface.c:240,383-384 falls back."""
    assert not oracle_per_tensor.has_per_channel
    e = oracle_per_tensor.forward(synth.faces(2, seed=1)[:1], ffo.CONTRACT)
    assert np.array_equal(e[0], np.load(os.path.join(GOLDEN, "ref_emb_b1_per_tensor.npy")))


def test_oracle_batch_independence(oracle):
    """Reference property: a batched run equals per-face runs bit for bit."""
    faces = synth.faces(3, seed=5)
    whole = oracle.forward(faces)
    for b in range(3):
        assert np.array_equal(whole[b], oracle.forward(faces[b:b + 1])[0])


@pytest.mark.parametrize("mode,tag", [(ffo.CONTRACT, "contract"), (ffo.STRICT, "strict")])
def test_oracle_single_layer_conv56(mode, tag):
    """The reference's single-layer benchmark case (conv3x3 64->64, 56x56, batch 8) against the reference's
    conv2d_i8_nhwc_batched + fused_epilogue_int8 CRCs."""
    import ctypes as C
    ffo.build()
    lib = C.CDLL(os.path.join(ffo.HERE, "libffo.so"))
    c = make_golden.conv56_case()
    x, w = c["x"], c["w"]
    B, H, W, Cin = x.shape
    Cout = w.shape[0]
    acc = np.zeros((B, H, W, Cout), np.int32)
    lib.ffo_conv_i32(x.ctypes.data_as(C.c_void_p), B, Cin, H, W, w.ctypes.data_as(C.c_void_p), Cout, 3, 3, 1, 1, H, W,
                     acc.ctypes.data_as(C.c_void_p))
    gold = {}
    for line in open(os.path.join(GOLDEN, f"ref_conv56_{tag}.txt")):
        if not line.startswith("#"):
            name, n, crc = line.split()
            gold[name] = (int(n), int(crc, 16))
    assert (acc.size, zlib.crc32(acc.tobytes())) == gold["acc"]
    lib.ffo_epilogue.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_void_p, C.c_void_p, C.c_void_p,
                                 C.c_void_p, C.c_float, C.c_void_p, C.c_void_p, C.c_float, C.c_int, C.c_void_p]
    for name, slope, res in (("prelu", c["slope"], None), ("add", None, c["res"])):
        o = np.zeros((B, H, W, Cout), np.int8)
        lib.ffo_epilogue(acc.ctypes.data, B * H * W, Cout, 1.0, c["ws"].ctypes.data, c["bias"].ctypes.data,
                         None if slope is None else slope.ctypes.data, None if res is None else res.ctypes.data, 0.0,
                         None if res is None else c["res_scale"].ctypes.data, c["inv_out"].ctypes.data, 1.0, mode,
                         o.ctypes.data)
        assert (o.size, zlib.crc32(o.tobytes())) == gold[name], name


@pytest.mark.skipif(not ffo.ref_available(), reason="oracle/_ref not built here or host lacks avx_vnni")
@pytest.mark.parametrize("strict", [False, True])
def test_oracle_matches_live_reference(oracle, model_root, ffw4, strict):
    """Fresh inputs (not the golden ones) through the compiled reference CLI, B=3."""
    faces = synth.faces(3, seed=11)
    emb_r, recs_r = ffo.run_ref_trace(model_root, ffw4, faces, strict=strict)
    emb_o, recs_o = oracle.forward_crc(faces, ffo.STRICT if strict else ffo.CONTRACT)
    assert recs_o == recs_r
    assert np.array_equal(emb_o, emb_r)


def test_requant_edge_cases():
    """Rounding is half AWAY from zero via +/-0.5 then truncation, clamp [-128,127];
    a product beyond int32 range lands on -128 like x86 cvttps2dq (int8_epilogue.c:80-87)."""
    import ctypes as C
    ffo.build()
    lib = C.CDLL(os.path.join(ffo.HERE, "libffo.so"))
    lib.ffo_epilogue.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_void_p, C.c_void_p, C.c_void_p,
                                 C.c_void_p, C.c_float, C.c_void_p, C.c_void_p, C.c_float, C.c_int, C.c_void_p]
    acc = np.array([1, -1, 3, -3, 5, 1000, -1000, 0], np.int32)   # x0.5 -> 0.5,-0.5,1.5,-1.5,2.5,...
    ws = np.full(8, 0.5, np.float32); bias = np.zeros(8, np.float32); inv = np.ones(8, np.float32)
    out = np.zeros(8, np.int8)
    lib.ffo_epilogue(acc.ctypes.data, 1, 8, 1.0, ws.ctypes.data, bias.ctypes.data, None, None, 0.0, None,
                     inv.ctypes.data, 1.0, ffo.STRICT, out.ctypes.data)
    assert out.tolist() == [1, -1, 2, -2, 3, 127, -128, 0]
    inv_big = np.full(8, 1e9, np.float32)
    lib.ffo_epilogue(acc.ctypes.data, 1, 8, 1.0, ws.ctypes.data, bias.ctypes.data, None, None, 0.0, None,
                     inv_big.ctypes.data, 1.0, ffo.STRICT, out.ctypes.data)
    assert out.tolist() == [127, -128, 127, -128, -128, -128, -128, 0]   # 2.5e9 overflows -> INT_MIN -> -128
