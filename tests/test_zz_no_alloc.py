"""GPU: the FC entry point that allocates nothing (ffcu_fc_small_noalloc).

Some callers hold device buffers but may not allocate: a serving loop that cannot afford the
device-wide synchronisation of cudaMalloc, a plug-in handed buffers but no allocator, a process
with a fixed memory budget.  For them the library carries the split-K accumulator of the
small-batch FC as a fixed 32 KiB array in its own device image.  This test plays such a caller:
it owns every input / output buffer (torch tensors here) and checks the entry point, called
twice in a row through the C-ABI, against the regular path (the FC inside fastface_trace_batch,
whose accumulator the context allocated with cudaMalloc) and against the CPU oracle's embeddings,
bit for bit, the tolerance all parity tests of this repository use.  Arguments the kernel could
not read safely (an unaligned slice, a K that is not a multiple of 16) must be refused on the
host.  The file sorts last so a failure here cannot hide another test.
"""
import ctypes as C
import os

import numpy as np
import pytest

import fastface_b200 as ff
from fastface_b200 import synth
from oracle import ffo

pytestmark = pytest.mark.gpu

N, K = 512, 25088


def _fc_tables(ffw4_path):
    """FC weights of the FFW4 file (its last op), K axis permuted from the file's CHW order
    (k = c*49 + hw) to the HWC order activations are stored in (k' = hw*512 + c)."""
    tail = 1 + 8 + N * K + 8 * N
    with open(ffw4_path, "rb") as f:
        f.seek(-tail, os.SEEK_END)
        d = f.read()
    assert d[0] == synth.OP_GEMM and np.frombuffer(d, "<u4", 2, 1).tolist() == [N, K]
    w = np.frombuffer(d, np.int8, N * K, 9).reshape(N, 512, 49)
    scale = np.frombuffer(d, "<f4", N, 9 + N * K).copy()
    bias = np.frombuffer(d, "<f4", N, 9 + N * K + 4 * N).copy()
    return np.ascontiguousarray(w.transpose(0, 2, 1)).reshape(N, K), scale, bias


def test_fc_small_noalloc_matches_regular_path(built_lib, model_root, ffw4, oracle):
    torch = pytest.importorskip("torch")
    lib = ff.load_library()
    lib.ffcu_fc_small_noalloc.restype = C.c_int
    lib.ffcu_fc_small_noalloc.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                          C.c_int, C.c_void_p, C.c_void_p]
    faces = synth.faces(3, seed=77)
    rec = {}
    with ff.FastFace(ffw4, cwd=model_root, max_batch=3) as eng:
        eng.trace(faces, lambda op, kind, arr: rec.__setitem__((op, kind), arr.copy()))
    act = rec[(174, "B")].reshape(3, K)          # int8 output of the last BN = FC input, HWC order
    want = rec[(176, "F")].reshape(3, N)         # embeddings from the regular (allocating) path
    want_cpu = oracle.forward(faces, ffo.CONTRACT)   # and from the CPU oracle: the checker proper
    assert np.array_equal(want, want_cpu)
    w, scale, bias = _fc_tables(ffw4)

    dev = torch.device("cuda:0")
    torch.cuda.set_device(0)
    d_w = torch.from_numpy(w).to(dev)
    d_scale, d_bias = torch.from_numpy(scale).to(dev), torch.from_numpy(bias).to(dev)
    d_act = torch.from_numpy(act).to(dev)
    d_out = torch.full((3, N), float("nan"), dtype=torch.float32, device=dev)
    torch.cuda.synchronize()

    # first call: all three faces (this call also resolves the built-in array's address)
    rc = lib.ffcu_fc_small_noalloc(d_act.data_ptr(), d_w.data_ptr(), d_scale.data_ptr(), d_bias.data_ptr(),
                                   3, N, K, ff.EPILOGUE_CONTRACT, d_out.data_ptr(), None)
    assert rc == 0, lib.ffcu_last_error().decode()
    torch.cuda.synchronize()
    assert np.array_equal(d_out.cpu().numpy(), want)
    assert np.array_equal(d_out.cpu().numpy(), want_cpu)

    # second call right after, different batch: the shared array must not leak the first call's sums
    d_out2 = torch.full((2, N), float("nan"), dtype=torch.float32, device=dev)
    rc = lib.ffcu_fc_small_noalloc(d_act[1:].contiguous().data_ptr(), d_w.data_ptr(), d_scale.data_ptr(),
                                   d_bias.data_ptr(), 2, N, K, ff.EPILOGUE_CONTRACT, d_out2.data_ptr(), None)
    assert rc == 0, lib.ffcu_last_error().decode()
    torch.cuda.synchronize()
    assert np.array_equal(d_out2.cpu().numpy(), want_cpu[1:])

    # beyond the built-in accumulator: refused with a clear message, nothing launched
    rc = lib.ffcu_fc_small_noalloc(d_act.data_ptr(), d_w.data_ptr(), d_scale.data_ptr(), d_bias.data_ptr(),
                                   17, N, K, ff.EPILOGUE_CONTRACT, d_out.data_ptr(), None)
    assert rc == -2 and b"batch <= 16" in lib.ffcu_last_error()

    # arguments the kernel's 16-byte loads could not take: refused on the host, nothing launched
    d_act_pad = torch.zeros(3 * K + 16, dtype=torch.int8, device=dev)
    rc = lib.ffcu_fc_small_noalloc(d_act_pad.data_ptr() + 1, d_w.data_ptr(), d_scale.data_ptr(), d_bias.data_ptr(),
                                   3, N, K, ff.EPILOGUE_CONTRACT, d_out.data_ptr(), None)
    assert rc == -1 and b"16-byte aligned" in lib.ffcu_last_error()
    rc = lib.ffcu_fc_small_noalloc(d_act.data_ptr(), d_w.data_ptr(), d_scale.data_ptr(), d_bias.data_ptr(),
                                   3, N, K - 8, ff.EPILOGUE_CONTRACT, d_out.data_ptr(), None)
    assert rc == -1 and b"multiple of 16" in lib.ffcu_last_error()
    rc = lib.ffcu_fc_small_noalloc(d_act.data_ptr(), d_w.data_ptr(), d_scale.data_ptr(), d_bias.data_ptr(),
                                   3, N, 0, ff.EPILOGUE_CONTRACT, d_out.data_ptr(), None)
    assert rc == -1
    torch.cuda.synchronize()
    # the refused calls launched nothing: the last good output is untouched
    assert np.array_equal(d_out.cpu().numpy(), want_cpu)
