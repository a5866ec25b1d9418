"""Regenerate the golden vectors in this directory from the UNMODIFIED reference.

Run in a container where the reference sources are mounted (oracle/Makefile builds
them into oracle/_ref/):

    python tests/golden/make_golden.py

Writes, for the seed-0 synthetic model and faces(2, seed=1):
  ref_trace_b2_{contract,strict}.txt   one line per kernel call of the reference's batched
                                       driver: kind, call#, n_elems, CRC-32 of the tensor
                                       (Q input int8, A conv int32 accumulators, O conv int8
                                       output, B BN int8 output, F one face's f32 embedding)
  ref_emb_b2_{contract,strict}.npy     the [2,512] f32 embeddings
  ref_emb_b1_per_tensor.npy            face 0 through the b=1 library with no OPSC2 file
  ref_conv56_*                         the 64->64 3x3 56x56 batch-8 single-layer case:
                                       CRCs of the reference's int32 accumulators and of its
                                       int8 epilogue output (PReLU and residual variants)
"""
import ctypes as C
import os
import sys
import tempfile
import zlib

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from fastface_b200 import synth   # noqa: E402
from oracle import ffo            # noqa: E402


def conv56_case(seed=0):
    """The reference's single-layer benchmark case: conv3x3 s1 p1 64->64, 56x56 NHWC, batch 8."""
    rng = np.random.Generator(np.random.PCG64(4242 + seed))
    x = rng.integers(-127, 128, size=(8, 56, 56, 64), dtype=np.int8)
    w = np.clip(np.rint(rng.standard_normal((64, 64, 3, 3)) * 40.0), -127, 127).astype(np.int8)
    ws = np.exp(rng.uniform(np.log(1e-5), np.log(1e-3), 64)).astype(np.float32)
    bias = (rng.standard_normal(64) * 0.1).astype(np.float32)
    slope = rng.uniform(0, 0.25, 64).astype(np.float32)
    out_scale = rng.uniform(0.005, 0.02, 64).astype(np.float32)
    inv_out = (np.float32(1.0) / (out_scale + np.float32(1e-9))).astype(np.float32)
    res = rng.integers(-127, 128, size=(8, 56, 56, 64), dtype=np.int8)
    res_scale = rng.uniform(0.002, 0.02, 64).astype(np.float32)
    return dict(x=x, w=w, ws=ws, bias=bias, slope=slope, inv_out=inv_out, res=res, res_scale=res_scale)


def ref_conv56(strict):
    """The reference's own conv + epilogue on the conv56 case, through its shared library."""
    lib = C.CDLL(os.path.join(ffo.REF_DIR, "libfastface_ref_strict.so" if strict else "libfastface_ref.so"))
    c = conv56_case()
    x, w = c["x"], c["w"]
    B, H, W, Cin = x.shape; Cout = w.shape[0]; K = Cin * 9
    wrow = np.zeros(K * Cout, np.int8); wpk = np.zeros(K * Cout, np.int8); cs = np.zeros(Cout, np.int32)
    lib.pack_conv_weight_nhwc(w.ctypes.data_as(C.c_void_p), Cout, Cin, 3, 3, K, wrow.ctypes.data_as(C.c_void_p),
                              wpk.ctypes.data_as(C.c_void_p), cs.ctypes.data_as(C.c_void_p))
    acc = np.zeros((B, H, W, Cout), np.int32)
    scratch = np.zeros(B * H * W * K + 64, np.uint8)
    lib.fastface_conv2d_i8_nhwc_batched(x.ctypes.data_as(C.c_void_p), B, Cin, H, W, Cout, 3, 3, 1, 1,
                                        wpk.ctypes.data_as(C.c_void_p), cs.ctypes.data_as(C.c_void_p), H, W,
                                        acc.ctypes.data_as(C.c_void_p), scratch.ctypes.data_as(C.c_void_p))
    lib.fused_epilogue_int8.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_void_p, C.c_void_p, C.c_void_p,
                                        C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_void_p, C.c_void_p,
                                        C.c_float, C.c_void_p]
    outs = {}
    for name, slope, res in (("prelu", c["slope"], None), ("add", None, c["res"])):
        o = np.zeros((B, H, W, Cout), np.int8)
        lib.fused_epilogue_int8(acc.ctypes.data, B * H * W, Cout, 1.0, c["ws"].ctypes.data, c["bias"].ctypes.data,
                                None, None, None if slope is None else slope.ctypes.data,
                                None if res is None else res.ctypes.data, 0.0,
                                None if res is None else c["res_scale"].ctypes.data, c["inv_out"].ctypes.data, 1.0,
                                o.ctypes.data)
        outs[name] = o
    return acc, outs


def main():
    ffo.build()
    assert ffo.ref_available(), "reference build unavailable"
    with tempfile.TemporaryDirectory() as root:
        ffw4 = synth.materialize(root, 0)
        faces = synth.faces(2, seed=1)
        for strict in (False, True):
            tag = "strict" if strict else "contract"
            emb, recs = ffo.run_ref_trace(root, ffw4, faces, strict=strict)
            np.save(os.path.join(HERE, f"ref_emb_b2_{tag}.npy"), emb)
            with open(os.path.join(HERE, f"ref_trace_b2_{tag}.txt"), "w") as f:
                f.write("# kind call n_elems crc32 -- reference fastface_int8_batched, seed-0 synthetic model, faces(2, seed=1)\n")
                for k, i, n, crc in recs:
                    f.write(f"{k} {i} {n} {crc:08x}\n")
            acc, outs = ref_conv56(strict)
            with open(os.path.join(HERE, f"ref_conv56_{tag}.txt"), "w") as f:
                f.write("# name n_elems crc32 -- reference conv2d_i8_nhwc_batched + fused_epilogue_int8 on conv56_case()\n")
                f.write(f"acc {acc.size} {zlib.crc32(acc.tobytes()):08x}\n")
                for name, o in outs.items():
                    f.write(f"{name} {o.size} {zlib.crc32(o.tobytes()):08x}\n")
        # b=1 library, per-tensor fallback (no OPSC2 file)
        ref = ffo.RefLib(root, ffw4, strict=False, opsc2_path=os.path.join(root, "does_not_exist.bin"))
        np.save(os.path.join(HERE, "ref_emb_b1_per_tensor.npy"), ref.embed(faces[0]))
        ref.close()
        # b=1 library with per-channel scales must equal row 0 of the batched run
        ref = ffo.RefLib(root, ffw4, strict=False)
        e = ref.embed(faces[0]); ref.close()
        assert np.array_equal(e, np.load(os.path.join(HERE, "ref_emb_b2_contract.npy"))[0])
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main()
