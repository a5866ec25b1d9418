"""GPU parity: the CUDA path, called through the C-ABI, against the oracle and against the
golden vectors of the unmodified reference.  Integer tensors and the fp32 embedding are
compared bit for bit (tolerance 0)."""
import ctypes as C
import os
import sys
import zlib

import numpy as np
import pytest

from conftest import GOLDEN, read_trace
import fastface_b200 as ff
from fastface_b200 import synth
from oracle import ffo

sys.path.insert(0, GOLDEN)
import make_golden  # noqa: E402

pytestmark = pytest.mark.gpu


def _libffo():
    ffo.build()
    lib = C.CDLL(os.path.join(ffo.HERE, "libffo.so"))
    lib.ffo_epilogue.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_void_p, C.c_void_p, C.c_void_p,
                                 C.c_void_p, C.c_float, C.c_void_p, C.c_void_p, C.c_float, C.c_int, C.c_void_p]
    return lib


def oracle_conv(x, w, ws, bias, inv_out, stride, pad, slope, res, res_scale, mode):
    lib = _libffo()
    B, H, W, Cin = x.shape
    Cout, _, Kh, Kw = w.shape
    Ho = (H + 2 * pad - Kh) // stride + 1
    Wo = (W + 2 * pad - Kw) // stride + 1
    acc = np.zeros((B, Ho, Wo, Cout), np.int32)
    lib.ffo_conv_i32(x.ctypes.data_as(C.c_void_p), B, Cin, H, W, w.ctypes.data_as(C.c_void_p), Cout, Kh, Kw,
                     stride, pad, Ho, Wo, acc.ctypes.data_as(C.c_void_p))
    out = np.zeros((B, Ho, Wo, Cout), np.int8)
    lib.ffo_epilogue(acc.ctypes.data, B * Ho * Wo, Cout, 1.0, ws.ctypes.data, bias.ctypes.data,
                     None if slope is None else slope.ctypes.data, None if res is None else res.ctypes.data, 0.0,
                     None if res is None else res_scale.ctypes.data, inv_out.ctypes.data, 1.0, mode, out.ctypes.data)
    return acc, out


def describe_mismatch(name, got, want):
    bad = np.argwhere(got != want)
    if bad.size == 0:
        return ""
    lines = [f"{name}: {len(bad)}/{got.size} elements differ ({100.0 * len(bad) / got.size:.3f}%)"]
    for idx in bad[:6]:
        t = tuple(int(i) for i in idx)
        lines.append(f"  at {t}: got {got[t]} want {want[t]}")
    for ax, nm in enumerate(("b", "h", "w", "c")[:got.ndim]):
        u = np.unique(bad[:, ax])
        lines.append(f"  bad {nm}: {u[:16].tolist()}{'...' if len(u) > 16 else ''} ({len(u)} distinct)")
    return "\n".join(lines)


def random_layer(rng, B, H, Cin, Cout, k, stride, with_slope, with_res):
    pad = 1 if k == 3 else 0
    x = rng.integers(-127, 128, size=(B, H, H, Cin), dtype=np.int8)
    w = np.clip(np.rint(rng.standard_normal((Cout, Cin, k, k)) * 40.0), -127, 127).astype(np.int8)
    ws = np.exp(rng.uniform(np.log(1e-5), np.log(1e-3), Cout)).astype(np.float32)
    bias = (rng.standard_normal(Cout) * 0.1).astype(np.float32)
    inv = (np.float32(1) / (rng.uniform(0.005, 0.05, Cout).astype(np.float32) + np.float32(1e-9))).astype(np.float32)
    Ho = (H + 2 * pad - k) // stride + 1
    slope = rng.uniform(0, 0.25, Cout).astype(np.float32) if with_slope else None
    res = rng.integers(-127, 128, size=(B, Ho, Ho, Cout), dtype=np.int8) if with_res else None
    rs = rng.uniform(0.002, 0.02, Cout).astype(np.float32) if with_res else None
    return dict(x=x, w=w, ws=ws, bias=bias, inv=inv, stride=stride, pad=pad, slope=slope, res=res, rs=rs)


def force_wide_tiles(monkeypatch, Cout):
    """Small test batches would get the narrow column tiles of the latency configuration; the kernel
    variants under test here are the ones large batches run, so pin the widest tile."""
    monkeypatch.setenv("FF_TC_BN", "wide")


LAYER_CASES = [
    # name, B, H, Cin, Cout, k, stride, slope, res
    ("s1_64_64_56_prelu", 2, 56, 64, 64, 3, 1, True, False),
    ("s1_64_64_112_oddB", 1, 112, 64, 64, 3, 1, True, False),
    ("s1_64_64_56_add", 3, 56, 64, 64, 3, 1, False, True),
    ("s1_64_128_56_prelu", 3, 56, 64, 128, 3, 1, True, False),
    ("s1_128_128_28_add", 3, 28, 128, 128, 3, 1, False, True),
    ("s1_128_256_28_prelu", 2, 28, 128, 256, 3, 1, True, False),
    ("s1_256_256_14_add", 5, 14, 256, 256, 3, 1, False, True),
    ("s1_256_512_14_prelu", 2, 14, 256, 512, 3, 1, True, False),
    ("s1_512_512_7_add", 9, 7, 512, 512, 3, 1, False, True),
    ("s2_64_64_112", 2, 112, 64, 64, 3, 2, False, False),
    ("s2_128_128_56", 3, 56, 128, 128, 3, 2, False, False),
    ("s2_256_256_28", 2, 28, 256, 256, 3, 2, False, False),
    ("s2_512_512_14", 3, 14, 512, 512, 3, 2, False, False),
    ("sc_64_64_112_add", 2, 112, 64, 64, 1, 2, False, True),
    ("sc_64_128_56_add", 3, 56, 64, 128, 1, 2, False, True),
    ("sc_128_256_28_add", 2, 28, 128, 256, 1, 2, False, True),
    ("sc_256_512_14_add", 3, 14, 256, 512, 1, 2, False, True),
]


@pytest.mark.parametrize("case", LAYER_CASES, ids=[c[0] for c in LAYER_CASES])
@pytest.mark.parametrize("impl", ["tc", "tc_wide", "simt"])
def test_single_layer_vs_oracle(built_lib, case, impl, monkeypatch):
    """impl "tc": the tile width the library picks for this (small) batch, i.e. the narrow column tiles of
    the latency configuration; "tc_wide": the widest tile (FF_TC_BN), which is what large batches run."""
    name, B, H, Cin, Cout, k, stride, sl, rs = case
    if impl == "tc_wide":
        monkeypatch.setenv("FF_TC_BN", "wide")
        impl = "tc"
    rng = np.random.default_rng(zlib.crc32(name.encode()))
    L = random_layer(rng, B, H, Cin, Cout, k, stride, sl, rs)
    for mode in (ff.EPILOGUE_CONTRACT, ff.EPILOGUE_STRICT):
        acc, out = ff.conv_once(L["x"], L["w"], L["ws"], L["bias"], L["inv"], stride=stride, pad=L["pad"],
                                slope=L["slope"], res=L["res"], res_scale=L["rs"], mode=mode, impl=impl)
        acc_o, out_o = oracle_conv(L["x"], L["w"], L["ws"], L["bias"], L["inv"], stride, L["pad"], L["slope"],
                                   L["res"], L["rs"], mode)
        msg = describe_mismatch("int32 accumulators", acc, acc_o)
        assert not msg, msg
        msg = describe_mismatch(f"int8 output (mode {mode})", out, out_o)
        assert not msg, msg



# Row geometries and tile counts that only large batches reach.  The 128-pixel row tile is
# {TW, TH, TB} = 16x8x1 on 112x112, 8x8x2 on 56x56, 4x4x8 on 28x28, 2x2x32 on 14x14 and 1x1x128 on
# 7x7 once the batch is large enough, and a CTA (or CTA pair) then walks many tiles: more than
# twice its accumulator ring, with the stage ring's phase flipping many times on the way.
BIG_LAYER_CASES = [
    # name, B, H, Cin, Cout, k, stride, slope, res
    ("big_s1_512_512_7_add_B128", 128, 7, 512, 512, 3, 1, False, True),
    ("big_s1_256_256_14_prelu_B64", 64, 14, 256, 256, 3, 1, True, False),
    ("big_s1_256_256_14_add_B392", 392, 14, 256, 256, 3, 1, False, True),
    ("big_s1_256_512_14_prelu_B64", 64, 14, 256, 512, 3, 1, True, False),
    ("big_s1_256_256_14_add_B33", 33, 14, 256, 256, 3, 1, False, True),
    ("big_s1_128_128_28_add_B16", 16, 28, 128, 128, 3, 1, False, True),
    ("big_s1_128_128_28_prelu_B200", 200, 28, 128, 128, 3, 1, True, False),
    ("big_s1_128_128_28_add_B37", 37, 28, 128, 128, 3, 1, False, True),
    ("big_s1_128_256_28_prelu_B40", 40, 28, 128, 256, 3, 1, True, False),
    ("big_s1_64_64_56_prelu_B100", 100, 56, 64, 64, 3, 1, True, False),
    ("big_s1_64_64_56_add_B37", 37, 56, 64, 64, 3, 1, False, True),
    ("big_s1_64_128_56_prelu_B24", 24, 56, 64, 128, 3, 1, True, False),
    ("big_s1_64_64_112_prelu_B24", 24, 112, 64, 64, 3, 1, True, False),
    ("big_s2_64_64_112_B20", 20, 112, 64, 64, 3, 2, False, False),
    ("big_s2_128_128_56_B33", 33, 56, 128, 128, 3, 2, False, False),
    ("big_s2_256_256_28_B64", 64, 28, 256, 256, 3, 2, False, False),
    ("big_s2_512_512_14_B130", 130, 14, 512, 512, 3, 2, False, False),
    ("big_sc_64_64_112_add_B20", 20, 112, 64, 64, 1, 2, False, True),
    ("big_sc_64_128_56_add_B33", 33, 56, 64, 128, 1, 2, False, True),
    ("big_sc_128_256_28_add_B64", 64, 28, 128, 256, 1, 2, False, True),
    ("big_sc_256_512_14_add_B130", 130, 14, 256, 512, 1, 2, False, True),
]


@pytest.mark.parametrize("case", BIG_LAYER_CASES, ids=[c[0] for c in BIG_LAYER_CASES])
def test_single_layer_large_batch_vs_oracle(built_lib, case):
    """The kernels and tilings large batches run (no override: the library picks them from the batch),
    with the fused BN second output on the residual layers as in the network."""
    name, B, H, Cin, Cout, k, stride, sl, rs = case
    rng = np.random.default_rng(zlib.crc32(name.encode()))
    L = random_layer(rng, B, H, Cin, Cout, k, stride, sl, rs)
    bn2 = None
    if rs:
        in_scale = (np.float32(1) / L["inv"]).astype(np.float32)
        bn_s = rng.uniform(0.5, 1.5, Cout).astype(np.float32)
        bn_o = (rng.standard_normal(Cout) * 0.1).astype(np.float32)
        bn_inv = (np.float32(1) / (rng.uniform(0.005, 0.05, Cout).astype(np.float32) + np.float32(1e-9))).astype(np.float32)
        bn2 = (in_scale, bn_s, bn_o, bn_inv)
    got = ff.conv_once(L["x"], L["w"], L["ws"], L["bias"], L["inv"], stride=stride, pad=L["pad"],
                       slope=L["slope"], res=L["res"], res_scale=L["rs"], impl="tc", bn2=bn2)
    acc_o, out_o = oracle_conv(L["x"], L["w"], L["ws"], L["bias"], L["inv"], stride, L["pad"], L["slope"],
                               L["res"], L["rs"], ffo.CONTRACT)
    msg = describe_mismatch("int32 accumulators", got[0], acc_o)
    assert not msg, msg
    msg = describe_mismatch("int8 output", got[1], out_o)
    assert not msg, msg
    if bn2:
        lib = _libffo()
        want2 = np.zeros_like(out_o)
        lib.ffo_bn_requant.argtypes = [C.c_void_p, C.c_float, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                       C.c_float, C.c_void_p, C.c_int, C.c_int]
        lib.ffo_bn_requant(out_o.ctypes.data, 1.0, bn2[0].ctypes.data, bn2[1].ctypes.data, bn2[2].ctypes.data, None,
                           bn2[3].ctypes.data, 1.0, want2.ctypes.data, out_o.size // Cout, Cout)
        msg = describe_mismatch("fused BN output", got[2], want2)
        assert not msg, msg


@pytest.mark.parametrize("case", LAYER_CASES, ids=[c[0] for c in LAYER_CASES])
@pytest.mark.parametrize("wide", [False, True], ids=["narrow", "wide"])
def test_single_layer_specialised_epilogues(built_lib, case, wide, monkeypatch):
    """Without an accumulator dump a layer takes the specialised epilogue variant of its kernel (the ones the
    forward runs; a dump forces the general variant).  int8 output and fused BN output against the oracle,
    both evaluation orders."""
    name, B, H, Cin, Cout, k, stride, sl, rs = case
    if wide:
        force_wide_tiles(monkeypatch, Cout)
    rng = np.random.default_rng(zlib.crc32(name.encode()) + 7)
    L = random_layer(rng, B, H, Cin, Cout, k, stride, sl, rs)
    in_scale = (np.float32(1) / L["inv"]).astype(np.float32)
    bn_s = rng.uniform(0.5, 1.5, Cout).astype(np.float32)
    bn_o = (rng.standard_normal(Cout) * 0.1).astype(np.float32)
    bn_inv = (np.float32(1) / (rng.uniform(0.005, 0.05, Cout).astype(np.float32) + np.float32(1e-9))).astype(np.float32)
    lib = _libffo()
    lib.ffo_bn_requant.argtypes = [C.c_void_p, C.c_float, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                   C.c_float, C.c_void_p, C.c_int, C.c_int]
    for mode in (ffo.CONTRACT, ffo.STRICT):
        _, out_o = oracle_conv(L["x"], L["w"], L["ws"], L["bias"], L["inv"], stride, L["pad"], L["slope"], L["res"], L["rs"], mode)
        _, out = ff.conv_once(L["x"], L["w"], L["ws"], L["bias"], L["inv"], stride=stride, pad=L["pad"], slope=L["slope"],
                              res=L["res"], res_scale=L["rs"], mode=mode, impl="tc", want_acc=False)
        msg = describe_mismatch(f"int8 output (mode {mode})", out, out_o)
        assert not msg, msg
        if rs or sl:                       # the forward's fused-BN layers: residual + BN, and PReLU + BN in the stem
            want2 = np.zeros_like(out_o)
            lib.ffo_bn_requant(out_o.ctypes.data, 1.0, in_scale.ctypes.data, bn_s.ctypes.data, bn_o.ctypes.data, None,
                               bn_inv.ctypes.data, 1.0, want2.ctypes.data, out_o.size // Cout, Cout)
            _, out, out2 = ff.conv_once(L["x"], L["w"], L["ws"], L["bias"], L["inv"], stride=stride, pad=L["pad"], slope=L["slope"],
                                        res=L["res"], res_scale=L["rs"], mode=mode, impl="tc", want_acc=False,
                                        bn2=(in_scale, bn_s, bn_o, bn_inv))
            assert np.array_equal(out, out_o)
            msg = describe_mismatch(f"fused BN output (mode {mode})", out2, want2)
            assert not msg, msg


@pytest.mark.parametrize("wval,xval,proved", [(56, -128, True), (56, 127, True), (127, 127, False), (-127, -128, False)])
def test_accumulator_to_float_near_and_beyond_22_bits(built_lib, wval, xval, proved):
    """The 64-input-channel kernels convert the accumulator to float with an integer add and a float add where the
    host has proved |accumulator| < 2^22 from the weights (128 * sum|w|), and take the general variant otherwise.
    All-equal weights and activations drive the accumulator to the largest magnitude the weights allow: 576 * 56 *
    128 = 4 128 768 is just inside the bound (proved: the add-based conversion runs at its edge), 576 * 127 * 127 is
    twice beyond it (not proved: the layer must fall back).  Random tensors with the same weights ride along."""
    rng = np.random.default_rng(1000 + wval + xval)
    B, H, Cin, Cout = 2, 16, 64, 64
    w = np.full((Cout, Cin, 3, 3), wval, np.int8)
    assert (128 * np.abs(w.astype(np.int64)).reshape(Cout, -1).sum(1).max() < (1 << 22)) == proved
    ws = np.exp(rng.uniform(np.log(5e-6), np.log(1.2e-5), Cout)).astype(np.float32)
    bias = (rng.standard_normal(Cout) * 0.1).astype(np.float32)
    inv = np.full(Cout, 1.0, np.float32)
    slope = rng.uniform(0, 0.25, Cout).astype(np.float32)
    res = rng.integers(-128, 128, size=(B, H, H, Cout), dtype=np.int8)
    rs = rng.uniform(0.2, 2.0, Cout).astype(np.float32)
    for x in (np.full((B, H, H, Cin), xval, np.int8), rng.integers(-128, 128, size=(B, H, H, Cin), dtype=np.int8)):
        for mode in (ffo.CONTRACT, ffo.STRICT):
            for sl, r, rsc in ((slope, None, None), (None, res, rs)):
                acc_o, out_o = oracle_conv(x, w, ws, bias, inv, 1, 1, sl, r, rsc, mode)
                _, out = ff.conv_once(x, w, ws, bias, inv, stride=1, pad=1, slope=sl, res=r, res_scale=rsc, mode=mode,
                                      impl="tc", want_acc=False)
                msg = describe_mismatch(f"w={wval} x={xval} mode {mode} {'PReLU' if sl is not None else 'residual'}", out, out_o)
                assert not msg, msg
        if x.min() == x.max():
            assert (np.abs(acc_o).max() >= (1 << 22)) == (not proved)


@pytest.mark.parametrize("impl", ["tc", "simt"])
def test_requant_out_of_range_matches_x86_conversion(built_lib, impl):
    """With a requant scale so large that t * inv leaves the int32 range, the reference's
    cvttps2dq yields INT_MIN (-> -128) for both signs (kernels/int8_epilogue.c:80-87).  The
    library may only take its unchecked conversion path when the weights and tables prove
    that cannot happen; here it can, so the checked path must reproduce the reference bytes."""
    rng = np.random.default_rng(77)
    L = random_layer(rng, 2, 56, 64, 64, 3, 1, True, False)
    inv = L["inv"].copy()
    inv[::2] = np.float32(3e10)                      # every other channel overflows for most pixels
    for mode in (ff.EPILOGUE_CONTRACT, ff.EPILOGUE_STRICT):
        acc, out = ff.conv_once(L["x"], L["w"], L["ws"], L["bias"], inv, stride=1, pad=L["pad"],
                                slope=L["slope"], mode=mode, impl=impl)
        acc_o, out_o = oracle_conv(L["x"], L["w"], L["ws"], L["bias"], inv, 1, L["pad"], L["slope"], None, None, mode)
        assert (out_o[..., ::2] == -128).mean() > 0.7        # the case does exercise the overflow
        msg = describe_mismatch(f"int8 output (mode {mode})", out, out_o)
        assert not msg, msg


@pytest.mark.parametrize("case", [LAYER_CASES[0], LAYER_CASES[2], LAYER_CASES[4], LAYER_CASES[6], LAYER_CASES[8], LAYER_CASES[14]],
                         ids=lambda c: c[0])
@pytest.mark.parametrize("impl", ["tc", "simt"])
def test_fused_bn_second_output(built_lib, case, impl, monkeypatch):
    """The BN pass that follows a conv rides along as a second epilogue output; it must equal
    bn_prelu_requant_int8 (kernels/int8_epilogue.c:253-318) applied to the conv's int8 output."""
    name, B, H, Cin, Cout, k, stride, sl, rs = case
    force_wide_tiles(monkeypatch, Cout)
    rng = np.random.default_rng(zlib.crc32(name.encode()) + 1)
    L = random_layer(rng, B, H, Cin, Cout, k, stride, sl, rs)
    in_scale = (np.float32(1) / L["inv"]).astype(np.float32)
    bn_s = rng.uniform(0.5, 1.5, Cout).astype(np.float32)
    bn_o = (rng.standard_normal(Cout) * 0.1).astype(np.float32)
    bn_inv = (np.float32(1) / (rng.uniform(0.005, 0.05, Cout).astype(np.float32) + np.float32(1e-9))).astype(np.float32)
    acc, out, out2 = ff.conv_once(L["x"], L["w"], L["ws"], L["bias"], L["inv"], stride=stride, pad=L["pad"],
                                  slope=L["slope"], res=L["res"], res_scale=L["rs"], impl=impl,
                                  bn2=(in_scale, bn_s, bn_o, bn_inv))
    acc_o, out_o = oracle_conv(L["x"], L["w"], L["ws"], L["bias"], L["inv"], stride, L["pad"], L["slope"],
                               L["res"], L["rs"], ffo.CONTRACT)
    lib = _libffo()
    want2 = np.zeros_like(out_o)
    lib.ffo_bn_requant.argtypes = [C.c_void_p, C.c_float, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                   C.c_float, C.c_void_p, C.c_int, C.c_int]
    lib.ffo_bn_requant(out_o.ctypes.data, 1.0, in_scale.ctypes.data, bn_s.ctypes.data, bn_o.ctypes.data, None,
                       bn_inv.ctypes.data, 1.0, want2.ctypes.data, out_o.size // Cout, Cout)
    assert np.array_equal(out, out_o)
    msg = describe_mismatch("fused BN output", out2, want2)
    assert not msg, msg


def test_unfused_plan_agrees(built_lib, model_root, ffw4, oracle, monkeypatch):
    """FF_FUSE_BN=0 / FF_FUSE_STEM=0 (separate BN passes, separate quantise + stem conv) give
    the same bytes as the fused default."""
    faces = synth.faces(3, seed=41)
    want = oracle.forward(faces, ffo.CONTRACT)
    with ff.FastFace(ffw4, cwd=model_root, max_batch=3) as e:
        assert np.array_equal(e.embed_batch(faces), want)
        n_fused = e.launches_per_forward
    monkeypatch.setenv("FF_FUSE_BN", "0")
    monkeypatch.setenv("FF_FUSE_STEM", "0")
    with ff.FastFace(ffw4, cwd=model_root, max_batch=3) as e:
        assert np.array_equal(e.embed_batch(faces), want)
        # fused: 1 stem launch, 52 convs (the four stride-2 conv + shortcut pairs one launch each at this batch), 1 FC;
        # unfused: 1 quantise, 53 convs (same four pairs fused), 25 BN passes, 1 FC
        assert e.launches_per_forward == 80 - 4 and n_fused == 54 - 4


@pytest.mark.parametrize("case", LAYER_CASES[:4], ids=lambda c: c[0])
def test_64ch_layers_on_the_per_tap_kernel(built_lib, case, monkeypatch):
    """FF_TC_WS=0 routes the 64-input-channel layers through the generic per-tap kernel
    instead of the weight-stationary one; both must give the same bytes."""
    monkeypatch.setenv("FF_TC_WS", "0")
    name, B, H, Cin, Cout, k, stride, sl, rs = case
    force_wide_tiles(monkeypatch, Cout)
    rng = np.random.default_rng(zlib.crc32(name.encode()))
    L = random_layer(rng, B, H, Cin, Cout, k, stride, sl, rs)
    acc, out = ff.conv_once(L["x"], L["w"], L["ws"], L["bias"], L["inv"], stride=stride, pad=L["pad"],
                            slope=L["slope"], res=L["res"], res_scale=L["rs"], impl="tc")
    acc_o, out_o = oracle_conv(L["x"], L["w"], L["ws"], L["bias"], L["inv"], stride, L["pad"], L["slope"],
                               L["res"], L["rs"], ffo.CONTRACT)
    assert np.array_equal(acc, acc_o) and np.array_equal(out, out_o)


@pytest.mark.parametrize("case", [LAYER_CASES[2], LAYER_CASES[4], LAYER_CASES[6]], ids=lambda c: c[0])
def test_fused_bn_by_arithmetic(built_lib, case, monkeypatch):
    """FF_TC_BNLUT_MAX=0 computes the fused BN output arithmetically in the epilogue instead of through
    the per-channel byte table; both must equal bn_prelu_requant_int8 (kernels/int8_epilogue.c:253-318)."""
    monkeypatch.setenv("FF_TC_BNLUT_MAX", "0")
    name, B, H, Cin, Cout, k, stride, sl, rs = case
    force_wide_tiles(monkeypatch, Cout)
    rng = np.random.default_rng(zlib.crc32(name.encode()) + 9)
    L = random_layer(rng, B, H, Cin, Cout, k, stride, sl, rs)
    in_scale = (np.float32(1) / L["inv"]).astype(np.float32)
    bn_s = rng.uniform(0.5, 1.5, Cout).astype(np.float32)
    bn_o = (rng.standard_normal(Cout) * 0.1).astype(np.float32)
    bn_inv = (np.float32(1) / (rng.uniform(0.005, 0.05, Cout).astype(np.float32) + np.float32(1e-9))).astype(np.float32)
    acc, out, out2 = ff.conv_once(L["x"], L["w"], L["ws"], L["bias"], L["inv"], stride=stride, pad=L["pad"],
                                  slope=L["slope"], res=L["res"], res_scale=L["rs"], impl="tc",
                                  bn2=(in_scale, bn_s, bn_o, bn_inv))
    acc_o, out_o = oracle_conv(L["x"], L["w"], L["ws"], L["bias"], L["inv"], stride, L["pad"], L["slope"],
                               L["res"], L["rs"], ffo.CONTRACT)
    lib = _libffo()
    want2 = np.zeros_like(out_o)
    lib.ffo_bn_requant.argtypes = [C.c_void_p, C.c_float, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                   C.c_float, C.c_void_p, C.c_int, C.c_int]
    lib.ffo_bn_requant(out_o.ctypes.data, 1.0, in_scale.ctypes.data, bn_s.ctypes.data, bn_o.ctypes.data, None,
                       bn_inv.ctypes.data, 1.0, want2.ctypes.data, out_o.size // Cout, Cout)
    assert np.array_equal(out, out_o)
    msg = describe_mismatch("fused BN output (arithmetic)", out2, want2)
    assert not msg, msg


@pytest.mark.parametrize("case", [c for c in LAYER_CASES if c[3] >= 128], ids=lambda c: c[0])
def test_wide_layers_on_the_single_cta_kernel(built_lib, case, monkeypatch):
    """FF_TC_PAIR=0 routes the >=128-input-channel layers through the one-CTA kernel instead of
    the CTA-pair (cta_group::2) one; both must give the same bytes."""
    monkeypatch.setenv("FF_TC_PAIR", "0")
    name, B, H, Cin, Cout, k, stride, sl, rs = case
    force_wide_tiles(monkeypatch, Cout)
    rng = np.random.default_rng(zlib.crc32(name.encode()))
    L = random_layer(rng, B, H, Cin, Cout, k, stride, sl, rs)
    acc, out = ff.conv_once(L["x"], L["w"], L["ws"], L["bias"], L["inv"], stride=stride, pad=L["pad"],
                            slope=L["slope"], res=L["res"], res_scale=L["rs"], impl="tc")
    acc_o, out_o = oracle_conv(L["x"], L["w"], L["ws"], L["bias"], L["inv"], stride, L["pad"], L["slope"],
                               L["res"], L["rs"], ffo.CONTRACT)
    assert np.array_equal(acc, acc_o) and np.array_equal(out, out_o)


@pytest.mark.parametrize("shape", [(8, 56, 64, 64), (3, 112, 64, 64), (2, 56, 64, 128), (5, 24, 128, 128), (2, 8, 16, 64)],
                         ids=lambda s: "B%d_H%d_%dto%d" % s)
def test_integer_winograd_f23_equals_four_times_direct(built_lib, shape):
    """The exact-integer Winograd F(2,3) kernel (the measured alternative for the 3x3 stride-1 layers): its
    int32 output must equal 4 x the direct convolution's accumulators, the property the reference's own
    Winograd self-test checks (kernels/winograd_int8_ref.c:237-259); the first shape is the single-layer
    case of the benchmark configuration, 56x56 64->64 batch 8, with full-range int8 operands."""
    B, H, Cin, Cout = shape
    rng = np.random.default_rng(B * 1000 + H + Cin)
    x = rng.integers(-127, 128, size=(B, H, H, Cin), dtype=np.int8)
    w = rng.integers(-127, 128, size=(Cout, Cin, 3, 3), dtype=np.int8)
    lib = _libffo()
    acc = np.zeros((B, H, H, Cout), np.int32)
    lib.ffo_conv_i32(x.ctypes.data_as(C.c_void_p), B, Cin, H, H, w.ctypes.data_as(C.c_void_p), Cout, 3, 3, 1, 1, H, H,
                     acc.ctypes.data_as(C.c_void_p))
    y4, ms = ff.winograd_f23(x, w, iters=2)
    msg = describe_mismatch("Winograd output vs 4 x direct", y4, acc * 4)
    assert not msg, msg
    assert ms > 0


def test_layer_microbench_reports_both_kernels(built_lib):
    """python -m fastface_b200.layer_bench: the single-layer case (56x56, 64->64, batch 8) on the tensor-core
    implicit GEMM with the Winograd kernel timed beside it on the same tensors."""
    from fastface_b200 import layer_bench
    line = layer_bench.run("conv56", 8, 5, False, True)
    assert line["winograd_f23"]["equals_4x_direct"] is True
    assert line["ms_per_launch"] > 0 and line["winograd_f23"]["ms_per_launch"] > 0


def test_network_microbench_single_face(built_lib):
    """`layer_bench --forward` at batch 1: the small-batch launch list (stem, layer chains, one-launch FC) through
    the public call; the similarity matrix of an embedding with itself has a unit diagonal."""
    from fastface_b200 import layer_bench
    line = layer_bench.run_forward(1, 3, 4)
    assert line["launches_per_forward"] == 22 and line["device_ms_per_forward"] > 0
    assert abs(line["cos_sim_matrix"]["diag_min"] - 1.0) < 1e-6


@pytest.mark.parametrize("case", [c for c in BIG_LAYER_CASES if (c[2], c[3], c[4], c[6]) == (28, 128, 128, 1)] + [LAYER_CASES[4]],
                         ids=lambda c: c[0])
def test_128_channel_layers_on_the_per_tap_pair_kernel(built_lib, case, monkeypatch):
    """FF_TC_WSP=0 routes the 128 -> 128 3x3 layers through the per-tap CTA-pair kernel instead of the
    flat-pitch weight-stationary one; both must give the oracle's bytes."""
    monkeypatch.setenv("FF_TC_WSP", "0")
    monkeypatch.setenv("FF_TC_BN", "wide")
    name, B, H, Cin, Cout, k, stride, sl, rs = case
    rng = np.random.default_rng(zlib.crc32(name.encode()) + 3)
    L = random_layer(rng, B, H, Cin, Cout, k, stride, sl, rs)
    acc, out = ff.conv_once(L["x"], L["w"], L["ws"], L["bias"], L["inv"], stride=stride, pad=L["pad"],
                            slope=L["slope"], res=L["res"], res_scale=L["rs"], impl="tc")
    acc_o, out_o = oracle_conv(L["x"], L["w"], L["ws"], L["bias"], L["inv"], stride, L["pad"], L["slope"],
                               L["res"], L["rs"], ffo.CONTRACT)
    assert np.array_equal(acc, acc_o) and np.array_equal(out, out_o)


def test_stem_conv_simt_vs_oracle(built_lib):
    """Cin=3 stem (K=27): CUDA-core dp4a kernel."""
    rng = np.random.default_rng(3)
    L = random_layer(rng, 2, 112, 3, 64, 3, 1, True, False)
    acc, out = ff.conv_once(L["x"], L["w"], L["ws"], L["bias"], L["inv"], slope=L["slope"], impl="simt")
    acc_o, out_o = oracle_conv(L["x"], L["w"], L["ws"], L["bias"], L["inv"], 1, 1, L["slope"], None, None, ffo.CONTRACT)
    assert np.array_equal(acc, acc_o) and np.array_equal(out, out_o)


@pytest.mark.parametrize("mode,tag", [(ff.EPILOGUE_CONTRACT, "contract"), (ff.EPILOGUE_STRICT, "strict")])
@pytest.mark.parametrize("impl", ["tc", "simt"])
def test_conv56_microbench_vs_reference_golden(built_lib, mode, tag, impl):
    """The reference's single-layer benchmark case: int32 and int8 CRCs of the reference's own kernels."""
    c = make_golden.conv56_case()
    gold = {}
    for line in open(os.path.join(GOLDEN, f"ref_conv56_{tag}.txt")):
        if not line.startswith("#"):
            nm, n, crc = line.split()
            gold[nm] = (int(n), int(crc, 16))
    for nm, slope, res in (("prelu", c["slope"], None), ("add", None, c["res"])):
        acc, out = ff.conv_once(c["x"], c["w"], c["ws"], c["bias"], c["inv_out"], slope=slope, res=res,
                                res_scale=None if res is None else c["res_scale"], mode=mode, impl=impl)
        assert (acc.size, zlib.crc32(acc.tobytes())) == gold["acc"]
        assert (out.size, zlib.crc32(out.tobytes())) == gold[nm], nm


@pytest.fixture(scope="module")
def engine(built_lib, model_root, ffw4):
    e = ff.FastFace(ffw4, cwd=model_root, max_batch=8)
    yield e
    e.close()


def gpu_crc_trace(engine, faces):
    recs, counts = [], {}
    B = faces.shape[0]

    def fn(op, kind, arr):
        if kind == "F":
            for b in range(B):
                i = counts.get(kind, 0); counts[kind] = i + 1
                row = arr.reshape(B, -1)[b]
                recs.append((kind, i, row.size, zlib.crc32(row.tobytes())))
            return
        i = counts.get(kind, 0); counts[kind] = i + 1
        recs.append((kind, i, arr.size, zlib.crc32(arr.tobytes())))

    emb = engine.trace(faces, fn)
    return emb, recs


@pytest.mark.parametrize("mode,tag", [(ff.EPILOGUE_CONTRACT, "contract"), (ff.EPILOGUE_STRICT, "strict")])
def test_network_trace_vs_reference_golden(engine, mode, tag):
    """Every dump point of the reference's batched driver (int32 accumulators and int8
    activations after every layer, embeddings), B=2, by CRC."""
    engine.set_epilogue_mode(mode)
    try:
        emb, recs = gpu_crc_trace(engine, synth.faces(2, seed=1))
    finally:
        engine.set_epilogue_mode(ff.EPILOGUE_CONTRACT)
    gold = read_trace(os.path.join(GOLDEN, f"ref_trace_b2_{tag}.txt"))
    bad = [(g, r) for g, r in zip(gold, recs) if g != r]
    assert len(recs) == len(gold) and not bad, f"first mismatching dump points (want, got): {bad[:4]}"
    want = np.load(os.path.join(GOLDEN, f"ref_emb_b2_{tag}.npy"))
    assert np.array_equal(emb, want), f"max abs diff {np.abs(emb - want).max()}"


@pytest.mark.parametrize("B", [1, 3, 8])
def test_network_layers_vs_oracle(engine, oracle, B):
    faces = synth.faces(B, seed=20 + B)
    want = {}
    oracle.forward(faces, ffo.CONTRACT, lambda op, kind, arr: want.__setitem__((op, ffo.KIND_LETTER[kind]), arr.copy()))
    first = []

    def fn(op, kind, arr):
        w = want[(op, kind)]
        if not np.array_equal(arr, w) and len(first) < 3:
            first.append(f"op {op} kind {kind}: {(arr != w).sum()}/{arr.size} differ")

    emb = engine.trace(faces, fn)
    assert not first, "; ".join(first)
    assert np.array_equal(emb, oracle.forward(faces, ffo.CONTRACT))


def _spread(n, k=40):
    """Indices over a batch of n: the ends, both sides of every 128-face boundary, and a seeded sample."""
    idx = {0, 1, n - 2, n - 1}
    for b in range(128, n, 128):
        idx.update((b - 1, b))
    rng = np.random.default_rng(n)
    idx.update(int(i) for i in rng.integers(0, n, size=k))
    return sorted(i for i in idx if 0 <= i < n)


@pytest.mark.parametrize("B", [64, 256, 1024])
def test_network_at_the_benchmark_batches(built_lib, model_root, ffw4, oracle, B):
    """The launch lists the benchmark times: a context created for batch 64 / 256 / 1024 with no override, so
    the row tile, the column tile, the tensor-core FC and the CUDA-graph replay are the ones those batches
    get.  Embeddings bit for bit against the unmodified reference's batched CLI where it can run (every
    face), else against the C port on faces spread over the batch (the reference treats the faces of a
    batch independently, arcface_forward_int8_batched.c:402-410)."""
    faces = synth.faces(B, seed=300 + B)
    with ff.FastFace(ffw4, cwd=model_root, max_batch=B) as e:
        first = e.embed_batch(faces)            # eager launches
        e.embed_batch(faces)                    # second call on the other slot
        got = e.embed_batch(faces)              # third call: the captured graph
        part = e.embed_batch(faces[:B - 7])     # a ragged batch through the same context
    assert np.array_equal(first, got)
    assert np.array_equal(part, got[:B - 7])
    if ffo.ref_available():
        want = ffo.ref_embed_many(model_root, ffw4, faces, batch=32)
        bad = np.flatnonzero((got != want).any(axis=1))
        assert bad.size == 0, f"{bad.size} of {B} faces differ from the reference, first {bad[:8].tolist()}"
    else:
        idx = _spread(B)
        want = oracle.forward(faces[idx], ffo.CONTRACT)
        bad = [i for j, i in enumerate(idx) if not np.array_equal(got[i], want[j])]
        assert not bad, f"faces {bad[:8]} differ from the oracle"


SWEEP_BATCHES = [3, 6, 12, 16, 17, 24, 31, 32, 33, 47, 48, 63, 65, 96, 127, 128, 129, 160, 192, 255, 257, 320, 384, 511, 512, 640]


@pytest.mark.parametrize("bn", ["auto", "64", "128", "wide"])
def test_network_batch_sweep_against_the_small_batch_launch_list(built_lib, model_root, ffw4, oracle, monkeypatch, bn):
    """Tile shape, column-tile width, kernel family, fused launches and graph replay all depend on the batch of
    the call; the reference treats the faces of a batch independently (arcface_forward_int8_batched.c:402-410).
    So every batch size must give, face for face, the bytes of the batch-8 launch list (which the tests above
    pin against the reference): 26 sizes around the tile-batch multiples (16 / 32 / 128), each in a context
    created for exactly that batch and again as a call of that size inside one batch-640 context.  Then the same with
    the column tile pinned (FF_TC_BN): 64 puts every down-sampling block on the fused stride-2 + shortcut launch and
    every layer on the one-CTA kernels at many tiles per CTA, 128 / wide put small batches on the CTA-pair kernels."""
    nmax = max(SWEEP_BATCHES)
    faces = synth.faces(nmax, seed=77)
    with ff.FastFace(ffw4, cwd=model_root, max_batch=8) as small:
        want = small.embed_batch(faces)
    if bn != "auto":
        monkeypatch.setenv("FF_TC_BN", bn)
    idx = [0, 7, 8, nmax - 1]
    assert np.array_equal(want[idx], oracle.forward(faces[idx], ffo.CONTRACT))
    failures = []
    with ff.FastFace(ffw4, cwd=model_root, max_batch=nmax) as big:
        for B in SWEEP_BATCHES:
            with ff.FastFace(ffw4, cwd=model_root, max_batch=B) as e:
                for rep in range(2):
                    got = e.embed_batch(faces[:B])
                    bad = np.flatnonzero((got != want[:B]).any(axis=1))
                    if bad.size:
                        failures.append(f"context of batch {B}, call {rep}: {bad.size} faces differ, first {bad[:8].tolist()}")
            got = big.embed_batch(faces[nmax - B:])          # the last B faces: another offset into the same buffers
            bad = np.flatnonzero((got != want[nmax - B:]).any(axis=1))
            if bad.size:
                failures.append(f"batch-{nmax} context, call of {B}: {bad.size} faces differ, first {bad[:8].tolist()}")
    assert not failures, "\n".join(failures)


def test_single_layer_random_cases(built_lib, monkeypatch):
    """Sixty seeded random single-layer cases over the network's layer shapes: 3x3 / 1x1, stride 1 / 2, PReLU or
    residual or neither, batch 1..400 (bounded by 1.5 GMAC per case, a third at powers of two), a third with the
    widest column tile pinned; int32 accumulators and int8 outputs against the oracle in both epilogue orders."""
    rng = np.random.default_rng(2024)
    shapes = [(112, 64, 64), (56, 64, 64), (56, 64, 128), (56, 128, 128), (28, 128, 128), (28, 128, 256), (28, 256, 256),
              (14, 256, 256), (14, 256, 512), (14, 512, 512), (7, 512, 512)]
    done = 0
    while done < 60:
        H, Cin, Cout = shapes[int(rng.integers(len(shapes)))]
        k, stride = [(3, 1), (3, 2), (1, 2), (1, 1)][int(rng.integers(4))]
        if k == 1 and Cin == Cout and stride == 1:
            continue
        bmax = max(1, int(1.5e9 / ((H // stride) ** 2 * Cin * Cout * k * k)))
        B = int(rng.integers(1, min(bmax, 400) + 1))
        if rng.random() < 0.3:
            B = int(rng.choice([b for b in (1, 2, 8, 16, 32, 64, 128) if b <= bmax] or [1]))
        sl = rng.random() < 0.5
        rs = (not sl) and rng.random() < 0.7
        L = random_layer(rng, B, H, Cin, Cout, k, stride, sl, rs)
        if rng.random() < 0.3:
            monkeypatch.setenv("FF_TC_BN", "wide")
        else:
            monkeypatch.delenv("FF_TC_BN", raising=False)
        for mode in (ff.EPILOGUE_CONTRACT, ff.EPILOGUE_STRICT):
            acc, out = ff.conv_once(L["x"], L["w"], L["ws"], L["bias"], L["inv"], stride=stride, pad=L["pad"],
                                    slope=L["slope"], res=L["res"], res_scale=L["rs"], mode=mode, impl="tc")
            acc_o, out_o = oracle_conv(L["x"], L["w"], L["ws"], L["bias"], L["inv"], stride, L["pad"], L["slope"],
                                       L["res"], L["rs"], mode)
            tag = f"B={B} H={H} {Cin}->{Cout} k{k} s{stride} slope={sl} res={rs} mode={mode}"
            msg = describe_mismatch("int32 accumulators, " + tag, acc, acc_o) or describe_mismatch("int8 output, " + tag, out, out_o)
            assert not msg, msg
        done += 1


def test_random_call_sequence_in_one_context(built_lib, model_root, ffw4):
    """300 calls of random size (1..300 faces, weighted towards 1-8 and the tile-batch multiples), random offset
    into the face set, random entry point (fastface_embed, fastface_embed_batch, fastface_embed_batch_u8) and an
    epilogue-order switch now and then, all through ONE context: the latency path and the three-stream pipeline
    alternate, graphs are captured and replayed per (size, order, slot), plans and tile geometries are made on
    first use.  Every result must equal the batch-8 launch list's for the same faces (8-bit pixels and their
    normalised floats give the same bits)."""
    N = 300
    rng = np.random.default_rng(11)
    pix = rng.integers(0, 256, size=(N, 112, 112, 3), dtype=np.uint8)
    faces = ((pix.astype(np.float32) - np.float32(127.5)) / np.float32(127.5)).astype(np.float32)
    want = {}
    with ff.FastFace(ffw4, cwd=model_root, max_batch=8) as small:
        for mode in (ff.EPILOGUE_CONTRACT, ff.EPILOGUE_STRICT):
            small.set_epilogue_mode(mode)
            want[mode] = small.embed_batch(faces)
    fails = []
    with ff.FastFace(ffw4, cwd=model_root, max_batch=N) as e:
        mode = ff.EPILOGUE_CONTRACT
        for it in range(300):
            r = rng.random()
            if r < 0.3:
                n = int(rng.integers(1, 9))
            elif r < 0.5:
                n = int(rng.choice([16, 17, 31, 32, 33, 64, 128, 129, 256, 300]))
            else:
                n = int(rng.integers(1, N + 1))
            off = int(rng.integers(0, N - n + 1))
            if rng.random() < 0.15:
                mode = ff.EPILOGUE_STRICT if mode == ff.EPILOGUE_CONTRACT else ff.EPILOGUE_CONTRACT
                e.set_epilogue_mode(mode)
            u8 = rng.random() < 0.4
            if n == 1 and not u8 and rng.random() < 0.5:
                got = e.embed(faces[off])[None]
            elif u8:
                got = e.embed_batch_u8(pix[off:off + n])
            else:
                got = e.embed_batch(faces[off:off + n])
            bad = np.flatnonzero((got != want[mode][off:off + n]).any(axis=1))
            if bad.size:
                fails.append((it, n, off, mode, u8, bad[:6].tolist()))
    assert not fails, fails[:10]


@pytest.mark.parametrize("mode,strict", [(ff.EPILOGUE_CONTRACT, False), (ff.EPILOGUE_STRICT, True)])
def test_network_trace_at_batch_64(built_lib, model_root, ffw4, oracle, mode, strict):
    """Every dump point (int32 accumulators, int8 activations, embeddings) at batch 64, in both epilogue
    orders, against the reference's traced driver run on the same faces (the C port where it cannot run)."""
    faces = synth.faces(64, seed=64)
    with ff.FastFace(ffw4, cwd=model_root, max_batch=64) as e:
        e.set_epilogue_mode(mode)
        emb, recs = gpu_crc_trace(e, faces)
    if ffo.ref_available():
        want, gold = ffo.run_ref_trace(model_root, ffw4, faces, strict=strict)
    else:
        want, gold = oracle.forward_crc(faces, mode)
    bad = [(g, r) for g, r in zip(gold, recs) if g != r]
    assert len(recs) == len(gold) and not bad, f"first mismatching dump points (want, got): {bad[:4]}"
    assert np.array_equal(emb, want)


@pytest.mark.parametrize("seed", [1, 2])
def test_network_other_model_seeds(built_lib, tmp_path_factory, seed):
    """Synthetic models of seeds 1 and 2 (other weights, scales and calibration tables): every dump
    point at batch 3 against the C port, embeddings at batch 8 and 40 against port and live reference, single faces
    (the layer-chain launch list) against the batch."""
    root = str(tmp_path_factory.mktemp(f"ffmodel_seed{seed}"))
    path = synth.materialize(root, seed)
    orc = ffo.Oracle(path, os.path.join(root, "models", "op_scales.bin"), os.path.join(root, "models", "op_scales_v2.bin"))
    faces = synth.faces(40, seed=500 + seed)
    want = {}
    orc.forward(faces[:3], ffo.CONTRACT, lambda op, kind, arr: want.__setitem__((op, ffo.KIND_LETTER[kind]), arr.copy()))
    first = []

    def fn(op, kind, arr):
        if not np.array_equal(arr, want[(op, kind)]) and len(first) < 3:
            first.append(f"op {op} kind {kind}: {(arr != want[(op, kind)]).sum()}/{arr.size} differ")

    with ff.FastFace(path, cwd=root, max_batch=40) as e:
        e.trace(faces[:3], fn)
        assert not first, "; ".join(first)
        got8 = e.embed_batch(faces[:8])
        got40 = e.embed_batch(faces)
        got1 = [e.embed(faces[i]) for i in (0, 5, 0, 5)]        # single faces: layer chains, eager then captured
    assert np.array_equal(got8, orc.forward(faces[:8], ffo.CONTRACT))
    assert all(np.array_equal(g, got8[i]) for g, i in zip(got1, (0, 5, 0, 5)))
    assert np.array_equal(got40[:8], got8)
    if ffo.ref_available():
        assert np.array_equal(got40, ffo.ref_embed_many(root, path, faces, batch=8))
    else:
        assert np.array_equal(got40[32:], orc.forward(faces[32:], ffo.CONTRACT))


def test_model_from_the_weight_producer(built_lib, tmp_path_factory):
    """A model written by fastface_b200.producer (fp32 network -> calibration -> folds -> FFW4 + OPSC2 + OPSC)
    runs through the CUDA path with the oracle's bytes: real calibrated scales (not the synthetic
    generator's) reach every epilogue and table."""
    from fastface_b200 import producer as P
    root = str(tmp_path_factory.mktemp("produced_gpu"))
    path = P.write_model(root, P.synth_float_model(seed=11), synth.faces(2, seed=910))
    orc = ffo.Oracle(path, os.path.join(root, "models", "op_scales.bin"), os.path.join(root, "models", "op_scales_v2.bin"))
    faces = synth.faces(6, seed=911)
    with ff.FastFace(path, cwd=root, max_batch=6) as e:
        got = e.embed_batch(faces)
        one = [e.embed(faces[2]) for _ in range(3)]              # the single-face launch list on real calibrated scales
    want = orc.forward(faces, ffo.CONTRACT)
    assert np.array_equal(got, want)
    assert all(np.array_equal(o, want[2]) for o in one)


def test_default_context_picks_the_tiling_from_the_call(built_lib, model_root, ffw4, oracle):
    """fastface_create's default context (room for 256 faces) must give one face, eight faces and a full
    batch each the tiling of that batch; results stay those of the oracle whichever plan runs."""
    faces = synth.faces(70, seed=17)
    want = oracle.forward(faces[:9], ffo.CONTRACT)
    with ff.FastFace(ffw4, cwd=model_root, max_batch=256) as e:
        assert np.array_equal(e.embed(faces[0]), want[0])
        assert np.array_equal(e.embed_batch(faces[:9]), want)
        big = e.embed_batch(faces)
        assert np.array_equal(big[:9], want)
        for _ in range(3):                       # batch 1 again, now from its captured graph
            assert np.array_equal(e.embed(faces[4]), want[4])


@pytest.mark.parametrize("mode", [ffo.CONTRACT, ffo.STRICT], ids=["contract", "strict"])
def test_single_face_layer_chains(built_lib, model_root, ffw4, oracle, monkeypatch, mode):
    """One face: the 26 same-shape convolutions of the 14x14 stage and the 4 of the 7x7 stage go out as ONE
    launch each (activations resident in the shared memory of a cluster of eight CTAs).  Same bytes as the
    per-layer launches (FF_CHAIN=0) and as the oracle: eager call, graph capture and replays, both epilogue
    orders, several faces through one context."""
    faces = synth.faces(4, seed=77)
    want = oracle.forward(faces, mode)
    counts = {}
    for flag in ("1", "0"):
        monkeypatch.setenv("FF_CHAIN", flag)
        with ff.FastFace(ffw4, cwd=model_root, max_batch=4) as e:
            e.set_epilogue_mode(mode)
            for rep in range(3):                 # eager, captured, replayed
                for i in range(4):
                    got = e.embed(faces[i])
                    assert np.array_equal(got, want[i]), f"FF_CHAIN={flag} rep {rep} face {i}"
            counts[flag] = e.launches_per_forward
            assert np.array_equal(e.embed_batch(faces), want)      # batch 4: per-layer launches in the same context
    assert counts["0"] == 54 - 4 and counts["1"] == 54 - 4 - 26 - 4 + 2, counts


@pytest.mark.parametrize("B", [1, 5, 32, 40, 64, 300])
def test_stride2_conv_and_shortcut_in_one_launch(built_lib, model_root, ffw4, oracle, monkeypatch, B):
    """A down-sampling block's 3x3 stride-2 convolution and its 1x1 stride-2 shortcut (ADD and the next block's BN
    fused) run as ONE launch where the call's column tile is 64 channels wide: all four blocks at small batch, the
    112x112 one at any batch.  Same bytes as the two launches (FF_FUSE_SC=0) for every face, and as the oracle on a
    sample, both epilogue orders.  Batches 32 and 64 give the 14x14 block tiles of 2 x 2 pixels x 32 faces and more
    tiles than CTAs: there a shortcut output sharing a buffer with the 3x3 conv's input (legal as two launches) is
    overwritten before later tiles have read it; batch 64 with the column tile pinned to 64 fuses all four blocks
    at several tiles per CTA."""
    if B == 64:
        monkeypatch.setenv("FF_TC_BN", "64")
    faces = synth.faces(B, seed=300 + B)
    sample = sorted(set([0, B // 2, B - 1]))
    want = {m: oracle.forward(faces[sample], m) for m in (ffo.CONTRACT, ffo.STRICT)}
    counts, full = {}, {}
    for flag in ("1", "0"):
        monkeypatch.setenv("FF_FUSE_SC", flag)
        with ff.FastFace(ffw4, cwd=model_root, max_batch=B) as e:
            for mode in (ffo.CONTRACT, ffo.STRICT):
                e.set_epilogue_mode(mode)
                for rep in range(2):
                    got = e.embed_batch(faces) if B > 1 else e.embed(faces[0])[None, :]
                    assert np.array_equal(got[sample], want[mode]), f"FF_FUSE_SC={flag} mode {mode} rep {rep}"
                    if flag == "1":
                        full[(mode, rep)] = got
                    else:
                        bad = np.nonzero((got != full[(mode, rep)]).any(axis=1))[0]
                        assert bad.size == 0, f"mode {mode} rep {rep}: faces {bad[:16].tolist()} differ between one and two launches"
            counts[flag] = e.launches_per_forward
    fused_pairs = counts["0"] - counts["1"]                 # the wider the batch, the fewer blocks keep 64-column tiles
    assert fused_pairs == 4 if (B <= 5 or B == 64) else 1 <= fused_pairs <= 4, counts


def test_bounded_wait_runs_out_and_the_device_stays_usable(built_lib):
    """The timeout path of the tensor-core kernels, exercised without faulting anything: the test hook
    makes the TMA producer of ONE one-CTA launch leave out a K step, and shortens the issuer's wait for
    that step to two million cycles (about a millisecond).  The wait must give up, every role must leave
    its loop, tensor memory must be freed and the call must return 1000 + FFCU_ERR_TMA_TIMEOUT (1); the
    same call, not armed, must then be bit-exact."""
    lib = ff.load_library()
    lib.ffcu_test_arm_timeout.restype = None
    lib.ffcu_test_arm_timeout.argtypes = [C.c_int, C.c_longlong]
    rng = np.random.default_rng(4242)
    L = random_layer(rng, 1, 8, 64, 64, 3, 1, True, False)     # 64 pixels x 64 channels: one tile, one CTA
    acc_o, out_o = oracle_conv(L["x"], L["w"], L["ws"], L["bias"], L["inv"], 1, 1, L["slope"], None, None, ffo.CONTRACT)
    lib.ffcu_test_arm_timeout(1, 2_000_000)
    with pytest.raises(RuntimeError) as ei:
        ff.conv_once(L["x"], L["w"], L["ws"], L["bias"], L["inv"], stride=1, pad=1, slope=L["slope"], impl="tc")
    assert "rc=1001" in str(ei.value), str(ei.value)
    for _ in range(2):                                          # the hook disarmed itself; the device is fine
        acc, out = ff.conv_once(L["x"], L["w"], L["ws"], L["bias"], L["inv"], stride=1, pad=1, slope=L["slope"], impl="tc")
        assert np.array_equal(acc, acc_o) and np.array_equal(out, out_o)


def test_layer_chain_bounded_waits_run_out_and_the_device_stays_usable(built_lib, model_root, ffw4, oracle):
    """The timeout path of the cluster-resident layer chain, exercised without faulting anything: the test hook makes
    CTA 0's weight producer leave out one ring step of the next chain launch and limits every barrier wait of that
    launch to two million cycles (about a millisecond).  CTA 0's issuer must give up, then the seven peers that wait
    for CTA 0's results, all eight must meet at the final cluster barrier and return; the call reports 1000 + the
    error word.  The same context must then serve the same face bit-exactly (eager, captured, replayed)."""
    lib = ff.load_library()
    lib.ffcu_test_arm_chain_timeout.restype = None
    lib.ffcu_test_arm_chain_timeout.argtypes = [C.c_int, C.c_longlong]
    faces = synth.faces(2, seed=5)
    want = oracle.forward(faces, ffo.CONTRACT)
    with ff.FastFace(ffw4, cwd=model_root, max_batch=2) as e:
        lib.ffcu_test_arm_chain_timeout(12, 2_000_000)          # layer 1, fourth tap
        with pytest.raises(RuntimeError) as ei:
            e.embed(faces[0])
        # 1000 + the code of whichever wait ran out first: the issuer's for the missing stage (TMA, 1) or the epilogue
        # warps' for the accumulator that stage belongs to (4): both started about together, with the same limit
        assert "rc=1001" in str(ei.value) or "rc=1004" in str(ei.value), str(ei.value)
        for _ in range(3):
            assert np.array_equal(e.embed(faces[0]), want[0])
            assert np.array_equal(e.embed(faces[1]), want[1])
        assert e.launches_per_forward == 22


def test_embed_and_embed_batch_agree_with_oracle(engine, oracle):
    faces = synth.faces(8, seed=99)
    want = oracle.forward(faces, ffo.CONTRACT)
    got = engine.embed_batch(faces)
    assert np.array_equal(got, want), f"max abs diff {np.abs(got - want).max()}"
    one = engine.embed(faces[3])
    assert np.array_equal(one, want[3])
    # tolerance stated by the spec (met with margin, since the match is exact)
    assert np.abs(got - want).max() <= 1e-5
    assert ff.FastFace.cos_sim(got[0], want[0]) >= 0.99999


def test_cos_sim_matrix_matches_pairwise(engine):
    """fastface_cos_sim_matrix gives, for every pair, the bits of fastface_cos_sim (float64 accumulation in
    index order, go/fastface/fastface.go:157-168), including a zero vector (-> 0) and odd sizes."""
    rng = np.random.default_rng(5)
    a = rng.standard_normal((19, 512)).astype(np.float32)
    b = rng.standard_normal((37, 512)).astype(np.float32) * np.float32(3.0)
    b[5] = 0
    b[6] = a[3]
    got = engine.cos_sim_matrix(a, b)
    want = np.array([[ff.FastFace.cos_sim(x, y) for y in b] for x in a], np.float32)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert got[3, 6] == np.float32(1.0) and np.all(got[:, 5] == 0)


def test_uint8_pixel_entry_point(engine, oracle):
    """fastface_embed_batch_u8 normalises 8-bit pixels on the device exactly as the reference's wrapper
    does on the host ((p - 127.5) / 127.5 in fp32, fastface.py:11): the embeddings must be bit for bit
    those of the fp32 entry on the normalised floats, and of the oracle."""
    rng = np.random.default_rng(11)
    pix = rng.integers(0, 256, size=(5, 112, 112, 3), dtype=np.uint8)
    pix[0, :2] = 0
    pix[0, 2:4] = 255                                   # the range ends
    x = ((pix.astype(np.float32) - np.float32(127.5)) / np.float32(127.5)).astype(np.float32)
    e_u8 = engine.embed_batch_u8(pix)
    e_f32 = engine.embed_batch(x)
    assert np.array_equal(e_u8.view(np.uint32), e_f32.view(np.uint32))
    want = oracle.forward(x, ffo.CONTRACT)
    assert np.array_equal(e_u8.view(np.uint32), want.view(np.uint32))
    one = engine.embed_batch_u8(pix[3:4])               # batch 1 goes through the CUDA-graph path on its third call
    for _ in range(3):
        one = engine.embed_batch_u8(pix[3:4])
    assert np.array_equal(one[0].view(np.uint32), e_u8[3].view(np.uint32))


def test_stem_on_cuda_cores_agrees(built_lib, model_root, ffw4, oracle, monkeypatch):
    """FF_STEM_TC=0 runs the stem as the fused dp4a kernel instead of the pack pass + K = 32 tensor-core
    GEMM; both give the oracle's bytes, from fp32 and from 8-bit pixel input."""
    faces = synth.faces(3, seed=21)
    want = oracle.forward(faces, ffo.CONTRACT)
    pix = np.random.default_rng(3).integers(0, 256, size=(3, 112, 112, 3), dtype=np.uint8)
    x = ((pix.astype(np.float32) - np.float32(127.5)) / np.float32(127.5)).astype(np.float32)
    want_u8 = oracle.forward(x, ffo.CONTRACT)
    for flag in ("1", "0"):
        monkeypatch.setenv("FF_STEM_TC", flag)
        with ff.FastFace(ffw4, cwd=model_root, max_batch=3) as e:
            assert np.array_equal(e.embed_batch(faces), want), f"FF_STEM_TC={flag}"
            assert np.array_equal(e.embed_batch_u8(pix), want_u8), f"FF_STEM_TC={flag}, uint8 input"
            assert e.launches_per_forward == 54 - 4


def test_network_with_the_large_batch_tiling(built_lib, model_root, ffw4, oracle, monkeypatch):
    """A small batch picks narrow column tiles; FF_TC_BN=wide pins the column tiling large batches get
    (CTA-pair kernels at BN = 256 / 128, weight-stationary kernel at 64 -> 128), here checked end to end."""
    monkeypatch.setenv("FF_TC_BN", "wide")
    faces = synth.faces(5, seed=31)
    want = oracle.forward(faces, ffo.CONTRACT)
    with ff.FastFace(ffw4, cwd=model_root, max_batch=5) as e:
        assert np.array_equal(e.embed_batch(faces), want)


def test_fc_paths(built_lib, model_root, ffw4, oracle, monkeypatch):
    """The FC runs as a split-K CUDA-core kernel for a handful of faces (up to 4 by default, up to 16 with
    FF_FC_SMALL_MAX) and on the tensor cores above; all match the reference's matvec, FF_FC_SMALL=0 sends a small
    batch down the large path, FF_FC_SPLITK=0 takes the one-CTA-per-tile tensor-core form."""
    faces = synth.faces(20, seed=61)
    want = oracle.forward(faces, ffo.CONTRACT)
    with ff.FastFace(ffw4, cwd=model_root, max_batch=20) as e:
        assert np.array_equal(e.embed_batch(faces), want)            # tensor-core FC
        for n in (5, 3, 3, 16, 4):                                   # tensor-core and CUDA-core FC in turn, scratch left clean
            assert np.array_equal(e.embed_batch(faces[:n]), want[:n]), n
    monkeypatch.setenv("FF_FC_SMALL_MAX", "16")
    with ff.FastFace(ffw4, cwd=model_root, max_batch=20) as e:
        for n in (5, 16, 9, 20, 16):                                 # CUDA-core FC up to 16 faces
            assert np.array_equal(e.embed_batch(faces[:n]), want[:n]), n
    monkeypatch.delenv("FF_FC_SMALL_MAX")
    monkeypatch.setenv("FF_FC_SMALL", "0")
    with ff.FastFace(ffw4, cwd=model_root, max_batch=5) as e:
        assert np.array_equal(e.embed_batch(faces[:5]), want[:5])
        assert np.array_equal(e.embed_batch(faces[:2]), want[:2])
    monkeypatch.setenv("FF_FC_SPLITK", "0")
    with ff.FastFace(ffw4, cwd=model_root, max_batch=20) as e:
        assert np.array_equal(e.embed_batch(faces), want)
        assert np.array_equal(e.embed_batch(faces[:2]), want[:2])


def test_fc_split_k_on_tensor_cores(built_lib, model_root, ffw4, oracle, monkeypatch):
    """Above 16 faces the FC runs as a split-K tensor-core GEMM: each (128-face, 64-output) tile is cut into K
    ranges, one CTA each; the CTAs add int32 partial sums into a scratch array and the one that takes a tile's last
    ticket writes the floats and leaves sums and ticket zero.  Same bytes as the one-CTA-per-tile form
    (FF_FC_SPLITK=0) for every face and as the oracle on a sample, in both epilogue orders, at batches that give one
    row tile, a ragged second one, several row tiles (fewer K ranges), and repeated calls (clean scratch), also
    inside a larger context (rows of other faces in the tile) and after a single face and a small batch."""
    nmax = 700
    faces = synth.faces(nmax, seed=71)
    sample = [0, 16, 17, 127, 128, 129, 299, nmax - 1]
    want = {m: oracle.forward(faces[sample], m) for m in (ffo.CONTRACT, ffo.STRICT)}
    ref = {}
    monkeypatch.setenv("FF_FC_SPLITK", "0")
    with ff.FastFace(ffw4, cwd=model_root, max_batch=nmax) as e:
        for mode in (ffo.CONTRACT, ffo.STRICT):
            e.set_epilogue_mode(mode)
            ref[mode] = e.embed_batch(faces)
            assert np.array_equal(ref[mode][sample], want[mode])
    monkeypatch.delenv("FF_FC_SPLITK")
    with ff.FastFace(ffw4, cwd=model_root, max_batch=nmax) as e:
        for mode in (ffo.CONTRACT, ffo.STRICT):
            e.set_epilogue_mode(mode)
            for B in (17, 32, 128, 129, 130, 256, 300, 700, 1, 5, 33, 700):
                for rep in range(2):
                    got = e.embed_batch(faces[nmax - B:]) if B > 1 else e.embed(faces[nmax - 1])[None, :]
                    bad = np.flatnonzero((got != ref[mode][nmax - B:]).any(axis=1))
                    assert bad.size == 0, f"mode {mode} batch {B} call {rep}: faces {bad[:8].tolist()} differ"
    for B in (17, 128, 200):
        with ff.FastFace(ffw4, cwd=model_root, max_batch=B) as e:
            got = e.embed_batch(faces[:B])
            assert np.array_equal(got, ref[ffo.CONTRACT][:B]), B


def test_fc_split_k_bounded_waits_run_out_and_the_device_stays_usable(built_lib, model_root, ffw4):
    """The timeout path of the split-K FC kernel, without faulting anything: the hook makes every CTA's producer leave
    out the activation box of one K step of ONE launch and limits that launch's waits to two million cycles.  Every
    CTA gives up, takes no ticket and returns; the call reports 1000 + an error word, the library clears the scratch
    sums, and the next calls are bit-exact."""
    lib = ff.load_library()
    lib.ffcu_test_arm_fc_timeout.restype = None
    lib.ffcu_test_arm_fc_timeout.argtypes = [C.c_int, C.c_longlong]
    faces = synth.faces(40, seed=72)
    with ff.FastFace(ffw4, cwd=model_root, max_batch=8) as small:
        want = small.embed_batch(faces)
    with ff.FastFace(ffw4, cwd=model_root, max_batch=40) as e:
        assert np.array_equal(e.embed_batch(faces), want)
        lib.ffcu_test_arm_fc_timeout(1, 2_000_000)
        with pytest.raises(RuntimeError) as ei:
            e.embed_batch(faces)
        assert any(f"rc={1000 + k}" in str(ei.value) for k in (1, 2, 3, 4)), str(ei.value)
        for _ in range(2):
            assert np.array_equal(e.embed_batch(faces), want)
        assert np.array_equal(e.embed_batch(faces[:3]), want[:3])


def test_chunking_and_determinism(built_lib, model_root, ffw4, oracle):
    """n larger than max_batch is split into steps; repeated runs give identical bytes."""
    faces = synth.faces(11, seed=7)
    with ff.FastFace(ffw4, cwd=model_root, max_batch=4) as e:
        a = e.embed_batch(faces)
        b = e.embed_batch(faces)
    assert np.array_equal(a, b)
    assert np.array_equal(a, oracle.forward(faces, ffo.CONTRACT))


def test_per_tensor_fallback(built_lib, model_root, ffw4, oracle_per_tensor, monkeypatch):
    """Without an OPSC2 file the per-tensor scales are used (libfastface.c:240)."""
    monkeypatch.setenv("OPSC2_PATH", os.path.join(model_root, "no_such_file.bin"))
    faces = synth.faces(2, seed=1)
    with ff.FastFace(ffw4, cwd=model_root, max_batch=2) as e:
        got = e.embed_batch(faces)
    assert np.array_equal(got[0], np.load(os.path.join(GOLDEN, "ref_emb_b1_per_tensor.npy")))
    assert np.array_equal(got, oracle_per_tensor.forward(faces, ffo.CONTRACT))


def test_simt_and_tensor_core_paths_agree(built_lib, model_root, ffw4, monkeypatch):
    faces = synth.faces(3, seed=5)
    with ff.FastFace(ffw4, cwd=model_root, max_batch=3) as e:
        a = e.embed_batch(faces)
    monkeypatch.setenv("FF_CONV_IMPL", "simt")
    with ff.FastFace(ffw4, cwd=model_root, max_batch=3) as e:
        b = e.embed_batch(faces)
    assert np.array_equal(a, b)


@pytest.mark.skipif(not ffo.ref_available(), reason="oracle/_ref not built here or host lacks avx_vnni")
def test_against_live_reference_library(engine, model_root, ffw4):
    face = synth.faces(1, seed=31)[0]
    ref = ffo.RefLib(model_root, ffw4)
    want = ref.embed(face)
    ref.close()
    assert np.array_equal(engine.embed(face), want)


def test_multi_device_context_shards_the_batch(built_lib, model_root, ffw4, oracle):
    """A context that owns two devices splits a batch into contiguous chunks (one host thread
    per device, no exchange between devices); the result equals the single-device one."""
    lib = ff.load_library()
    if lib.ffcu_device_count() < 2:
        pytest.skip("needs 2 GPUs")
    faces = synth.faces(9, seed=123)
    want = oracle.forward(faces, ffo.CONTRACT)
    with ff.FastFace(ffw4, cwd=model_root, devices=[0, 1], max_batch=4) as e:
        got = e.embed_batch(faces)          # 5 + 4 faces, in steps of at most 4 per device
    assert np.array_equal(got, want)


def test_cli_file_and_server_modes(built_lib, model_root, ffw4, oracle):
    """The reference-compatible CLI (arcface_forward_int8_batched.c:523-553): --in/--out dumps and
    the --server stdin/stdout protocol its Python / Go wrappers speak."""
    import subprocess
    from fastface_b200 import build as _b
    exe = _b.CLI
    faces = synth.faces(4, seed=88)
    want = oracle.forward(faces, ffo.CONTRACT)
    inp, outp = os.path.join(model_root, "_cli_in.bin"), os.path.join(model_root, "_cli_out.bin")
    faces.tofile(inp)
    r = subprocess.run([exe, ffw4, "--batch", "4", "--in", inp, "--out", outp], cwd=model_root, capture_output=True, timeout=300)
    assert r.returncode == 0, r.stderr.decode()[-500:]
    assert np.array_equal(np.fromfile(outp, np.float32).reshape(4, 512), want)
    p = subprocess.Popen([exe, ffw4, "--batch", "2", "--server"], cwd=model_root, stdin=subprocess.PIPE,
                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL)
    try:
        for k in (0, 2):
            p.stdin.write(faces[k:k + 2].tobytes()); p.stdin.flush()
            raw = p.stdout.read(2 * 512 * 4)
            assert np.array_equal(np.frombuffer(raw, np.float32).reshape(2, 512), want[k:k + 2])
        p.stdin.write(b"\0" * 100); p.stdin.close()          # partial batch: abort with exit code 4
        assert p.wait(timeout=60) == 4
    finally:
        if p.poll() is None:
            p.kill()
