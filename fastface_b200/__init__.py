"""fastface_b200 -- ctypes view of libfastface_b200.so (the C API in include/fastface.h).

The product is the C library; this module exists so tests and the benchmark can
drive it, and it mirrors the reference's Python wrapper (fastface.py:32-121):
``FastFace(...).embed(arr)``, ``.embed_batch(arrs)``, ``FastFace.cos_sim(a, b)``,
``.close()``, context-manager use.  Where the reference wrapper talks to a
``--server`` subprocess, this one calls the library in-process.

There is no fallback: if the shared library is missing (not built) or no
sm_100 GPU is present, construction raises.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Callable, List, Optional, Sequence, Tuple

import numpy as np

_PKG = os.path.dirname(os.path.abspath(__file__))
# $FASTFACE_B200_LIB names another build of the same library (for side-by-side comparisons of two builds)
LIB_PATH = os.environ.get("FASTFACE_B200_LIB") or os.path.join(_PKG, "libfastface_b200.so")

FACE_SHAPE = (112, 112, 3)
FACE_NELEMS = 112 * 112 * 3
EMB_DIM = 512

EPILOGUE_STRICT, EPILOGUE_CONTRACT = 0, 1

_TRACE_FN = C.CFUNCTYPE(None, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_ulonglong)
_lib = None


class FfcuLayer(C.Structure):
    """struct ffcu_layer of include/ff_cuda.h."""
    _fields_ = [("kind", C.c_int), ("op_index", C.c_int), ("src_buf", C.c_int), ("dst_buf", C.c_int),
                ("res_buf", C.c_int), ("Cin", C.c_int), ("Cout", C.c_int), ("Kh", C.c_int), ("Kw", C.c_int),
                ("stride", C.c_int), ("pad", C.c_int), ("H", C.c_int), ("W", C.c_int), ("Ho", C.c_int),
                ("Wo", C.c_int), ("w", C.c_void_p), ("w_bytes", C.c_size_t), ("Cin_pad", C.c_int),
                ("w_scale", C.c_void_p), ("bias", C.c_void_p), ("slope", C.c_void_p),
                ("res_scale", C.c_void_p), ("inv_out", C.c_void_p), ("in_scale", C.c_void_p),
                ("bn_scale", C.c_void_p), ("bn_offset", C.c_void_p),
                ("bn2_dst_buf", C.c_int), ("bn2_op_index", C.c_int), ("bn2_in_scale", C.c_void_p),
                ("bn2_scale", C.c_void_p), ("bn2_offset", C.c_void_p), ("bn2_inv_out", C.c_void_p),
                ("bn2_lut", C.c_void_p)]


def load_library() -> C.CDLL:
    """dlopen the in-tree library and declare its prototypes (no CUDA call is made)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(f"{LIB_PATH} is missing: run `python -m fastface_b200.build` (there is no fallback)")
    L = C.CDLL(LIB_PATH)
    L.fastface_create.restype = C.c_void_p
    L.fastface_create.argtypes = [C.c_char_p]
    L.fastface_create_ex.restype = C.c_void_p
    L.fastface_create_ex.argtypes = [C.c_char_p, C.POINTER(C.c_int), C.c_int, C.c_int]
    L.fastface_embed.restype = C.c_int
    L.fastface_embed.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
    L.fastface_embed_batch.restype = C.c_int
    L.fastface_embed_batch.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
    L.fastface_cos_sim_matrix.restype = C.c_int
    L.fastface_cos_sim_matrix.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p]
    L.fastface_embed_batch_u8.restype = C.c_int
    L.fastface_embed_batch_u8.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
    L.fastface_destroy.restype = None
    L.fastface_destroy.argtypes = [C.c_void_p]
    L.fastface_cos_sim.restype = C.c_float
    L.fastface_cos_sim.argtypes = [C.c_void_p, C.c_void_p]
    L.fastface_set_epilogue_mode.restype = C.c_int
    L.fastface_set_epilogue_mode.argtypes = [C.c_void_p, C.c_int]
    L.fastface_trace_batch.restype = C.c_int
    L.fastface_trace_batch.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, _TRACE_FN, C.c_void_p]
    L.fastface_bench_resident.restype = C.c_int
    L.fastface_bench_resident.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_float)]
    L.fastface_launches_per_forward.restype = C.c_int
    L.fastface_launches_per_forward.argtypes = [C.c_void_p]
    L.fastface_last_error.restype = C.c_char_p
    L.fastface_layer_count.restype = C.c_int
    L.fastface_layer_count.argtypes = [C.c_void_p]
    L.fastface_layer_desc.restype = C.c_int
    L.fastface_layer_desc.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_int)]
    L.fastface_bench_layers.restype = C.c_int
    L.fastface_bench_layers.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_float), C.c_int]
    L.ffcu_device_count.restype = C.c_int
    L.ffcu_conv_once.restype = C.c_int
    L.ffcu_conv_once.argtypes = [C.c_int, C.POINTER(FfcuLayer), C.c_int, C.c_int, C.c_int,
                                 C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    L.ffcu_conv_bench.restype = C.c_int
    L.ffcu_conv_bench.argtypes = [C.c_int, C.POINTER(FfcuLayer), C.c_int, C.c_int, C.c_int,
                                  C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.POINTER(C.c_float)]
    L.ffcu_winograd_f23_once.restype = C.c_int
    L.ffcu_winograd_f23_once.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                         C.c_int, C.c_void_p, C.POINTER(C.c_float)]
    L.ffcu_last_error.restype = C.c_char_p
    _lib = L
    return L


def _ptr(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


class FastFace:
    """In-process counterpart of the reference's ``fastface.FastFace``.

    ``weights`` is an FFW4 file; ``models/op_scales.bin`` (and optionally
    ``models/op_scales_v2.bin``) are looked up relative to ``cwd`` exactly as
    the reference binary does relative to its working directory.
    """

    def __init__(self, weights: str, batch: int = 1, devices: Optional[Sequence[int]] = None,
                 cwd: Optional[str] = None, max_batch: Optional[int] = None):
        self.lib = load_library()
        self.batch = int(batch)
        devs = list(devices) if devices is not None else [0]
        arr = (C.c_int * len(devs))(*devs)
        mb = int(max_batch) if max_batch else max(1, self.batch)
        old = os.getcwd()
        wpath = os.path.abspath(weights)
        try:
            if cwd:
                os.chdir(cwd)
            self.h = self.lib.fastface_create_ex(wpath.encode(), arr, len(devs), mb)
        finally:
            os.chdir(old)
        if not self.h:
            raise RuntimeError("fastface_create failed: " + self.lib.fastface_last_error().decode())
        self.max_batch = mb
        self.n_devices = len(devs)
        self.device0 = devs[0]

    # -- reference wrapper surface -------------------------------------------------
    def embed(self, arr: np.ndarray) -> np.ndarray:
        if arr.dtype != np.float32 or arr.size != FACE_NELEMS:
            raise ValueError(f"arr must be float32 with {FACE_NELEMS} elements, got {arr.dtype}/{arr.size}")
        a = np.ascontiguousarray(arr)
        out = np.empty(EMB_DIM, np.float32)
        rc = self.lib.fastface_embed(self.h, _ptr(a), _ptr(out))
        if rc != 0:
            raise RuntimeError(f"fastface_embed rc={rc}: " + self.lib.fastface_last_error().decode())
        return out

    def embed_batch(self, arrs) -> np.ndarray:
        a = np.ascontiguousarray(np.asarray(arrs, dtype=np.float32)).reshape(-1, *FACE_SHAPE)
        out = np.empty((a.shape[0], EMB_DIM), np.float32)
        self.embed_into(a, out)
        return out

    def embed_into(self, faces: np.ndarray, out: np.ndarray) -> None:
        """faces [n,112,112,3] f32 -> out [n,512] f32, no copies on the Python side
        (either array may live in pinned host memory)."""
        n = faces.shape[0]
        rc = self.lib.fastface_embed_batch(self.h, _ptr(faces), n, _ptr(out))
        if rc != 0:
            raise RuntimeError(f"fastface_embed_batch rc={rc}: " + self.lib.fastface_last_error().decode())

    def embed_batch_u8(self, pixels) -> np.ndarray:
        """8-bit pixels [n,112,112,3] -> [n,512]; same embeddings as embed_batch((p - 127.5) / 127.5)."""
        a = np.ascontiguousarray(np.asarray(pixels, dtype=np.uint8)).reshape(-1, *FACE_SHAPE)
        out = np.empty((a.shape[0], EMB_DIM), np.float32)
        self.embed_into_u8(a, out)
        return out

    def embed_into_u8(self, pixels: np.ndarray, out: np.ndarray) -> None:
        n = pixels.shape[0]
        rc = self.lib.fastface_embed_batch_u8(self.h, _ptr(pixels), n, _ptr(out))
        if rc != 0:
            raise RuntimeError(f"fastface_embed_batch_u8 rc={rc}: " + self.lib.fastface_last_error().decode())

    def cos_sim_matrix(self, a: np.ndarray, b: np.ndarray) -> np.ndarray:
        """[n,512] x [m,512] -> [n,m] cosine similarities, the values cos_sim gives pair by pair."""
        a = np.ascontiguousarray(a, dtype=np.float32).reshape(-1, EMB_DIM)
        b = np.ascontiguousarray(b, dtype=np.float32).reshape(-1, EMB_DIM)
        out = np.empty((a.shape[0], b.shape[0]), np.float32)
        rc = self.lib.fastface_cos_sim_matrix(self.h, _ptr(a), a.shape[0], _ptr(b), b.shape[0], _ptr(out))
        if rc != 0:
            raise RuntimeError(f"fastface_cos_sim_matrix rc={rc}: " + self.lib.fastface_last_error().decode())
        return out

    @staticmethod
    def cos_sim(a: np.ndarray, b: np.ndarray) -> float:
        a = np.ascontiguousarray(a, dtype=np.float32)
        b = np.ascontiguousarray(b, dtype=np.float32)
        return float(load_library().fastface_cos_sim(_ptr(a), _ptr(b)))

    def close(self):
        if getattr(self, "h", None):
            self.lib.fastface_destroy(self.h)
            self.h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- additions -----------------------------------------------------------------
    def set_epilogue_mode(self, mode: int) -> None:
        if self.lib.fastface_set_epilogue_mode(self.h, mode) != 0:
            raise RuntimeError("fastface_set_epilogue_mode failed")

    def trace(self, faces: np.ndarray, fn: Callable[[int, str, np.ndarray], None]) -> np.ndarray:
        """Forward with dump points: fn(op_index, kind, array) per record, kinds as in
        include/fastface.h ('Q','A','O','B','F')."""
        a = np.ascontiguousarray(np.asarray(faces, dtype=np.float32)).reshape(-1, *FACE_SHAPE)
        out = np.empty((a.shape[0], EMB_DIM), np.float32)
        dt = {"Q": np.int8, "A": np.int32, "O": np.int8, "B": np.int8, "F": np.float32}

        def _cb(user, op_index, kind, data, n):
            k = chr(kind)
            nbytes = n * np.dtype(dt[k]).itemsize
            buf = np.ctypeslib.as_array(C.cast(data, C.POINTER(C.c_uint8)), shape=(nbytes,))
            fn(op_index, k, buf.view(dt[k]))

        cb = _TRACE_FN(_cb)
        rc = self.lib.fastface_trace_batch(self.h, _ptr(a), a.shape[0], _ptr(out), cb, None)
        if rc != 0:
            raise RuntimeError(f"fastface_trace_batch rc={rc}: " + self.lib.fastface_last_error().decode())
        return out

    def bench_resident(self, faces: np.ndarray, iters: int) -> float:
        """Milliseconds (CUDA events) for ``iters`` forwards over device-resident faces."""
        a = np.ascontiguousarray(np.asarray(faces, dtype=np.float32)).reshape(-1, *FACE_SHAPE)
        ms = C.c_float(0)
        rc = self.lib.fastface_bench_resident(self.h, _ptr(a), a.shape[0], iters, C.byref(ms))
        if rc != 0:
            raise RuntimeError(f"fastface_bench_resident rc={rc}: " + self.lib.fastface_last_error().decode())
        return float(ms.value)

    def layers(self) -> List[dict]:
        """Static launch list: one dict per kernel launch of a forward pass."""
        keys = ("kind", "op_index", "Cin", "Cout", "Kh", "Kw", "stride", "H", "W", "Ho", "Wo", "tensor_core")
        out = []
        for k in range(self.lib.fastface_layer_count(self.h)):
            d = (C.c_int * 12)()
            if self.lib.fastface_layer_desc(self.h, k, d) != 0:
                raise RuntimeError("fastface_layer_desc failed")
            out.append(dict(zip(keys, list(d))))
        return out

    def bench_layers(self, faces: np.ndarray, iters: int) -> List[float]:
        """Per-layer CUDA-event milliseconds (total over ``iters`` launches of each layer)."""
        a = np.ascontiguousarray(np.asarray(faces, dtype=np.float32)).reshape(-1, *FACE_SHAPE)
        n = self.lib.fastface_layer_count(self.h)
        ms = (C.c_float * n)()
        rc = self.lib.fastface_bench_layers(self.h, _ptr(a), a.shape[0], iters, ms, n)
        if rc != n:
            raise RuntimeError(f"fastface_bench_layers rc={rc}: " + self.lib.fastface_last_error().decode())
        return list(ms)

    @property
    def launches_per_forward(self) -> int:
        return int(self.lib.fastface_launches_per_forward(self.h))


def conv_once(x: np.ndarray, w_oihw: np.ndarray, w_scale: np.ndarray, bias: np.ndarray,
              inv_out: np.ndarray, stride: int = 1, pad: int = 1, slope: Optional[np.ndarray] = None,
              res: Optional[np.ndarray] = None, res_scale: Optional[np.ndarray] = None,
              mode: int = EPILOGUE_CONTRACT, impl: str = "tc", device: int = 0,
              bn2: Optional[Tuple[np.ndarray, np.ndarray, np.ndarray, np.ndarray]] = None,
              want_acc: bool = True, bench_iters: int = 0):
    """One conv layer through the C-ABI (ffcu_conv_once): x int8 [B,H,W,Cin],
    w int8 [Cout,Cin,Kh,Kw] -> (int32 accumulators, int8 output), both [B,Ho,Wo,Cout].
    bench_iters > 0 goes through ffcu_conv_bench instead and returns (ms per launch, int8 output[, BN output])."""
    lib = load_library()
    B, H, W, Cin = x.shape
    Cout, _, Kh, Kw = w_oihw.shape
    Cp = (Cin + 3) & ~3
    Ho = (H + 2 * pad - Kh) // stride + 1
    Wo = (W + 2 * pad - Kw) // stride + 1
    xp = np.zeros((B, H, W, Cp), np.int8); xp[..., :Cin] = x
    wp = np.zeros((Cout, Kh, Kw, Cp), np.int8); wp[..., :Cin] = np.transpose(w_oihw, (0, 2, 3, 1))
    keep = [np.ascontiguousarray(a, dtype=np.float32) if a is not None else None
            for a in (w_scale, bias, slope, res_scale, inv_out)]
    L = FfcuLayer()
    L.kind = 1; L.op_index = 0; L.src_buf = 0; L.dst_buf = 1; L.res_buf = -1 if res is None else 2
    L.Cin, L.Cout, L.Kh, L.Kw, L.stride, L.pad = Cin, Cout, Kh, Kw, stride, pad
    L.H, L.W, L.Ho, L.Wo = H, W, Ho, Wo
    L.w = wp.ctypes.data; L.w_bytes = wp.size; L.Cin_pad = Cp
    L.w_scale, L.bias, L.slope, L.res_scale, L.inv_out = [None if a is None else a.ctypes.data for a in keep]
    L.bn2_dst_buf = -1
    out2 = None
    if bn2 is not None:
        keep2 = [np.ascontiguousarray(a, dtype=np.float32) for a in bn2]
        L.bn2_dst_buf = 3
        L.bn2_in_scale, L.bn2_scale, L.bn2_offset, L.bn2_inv_out = [a.ctypes.data for a in keep2]
        out2 = np.empty((B, Ho, Wo, Cout), np.int8)
    acc = np.empty((B, Ho, Wo, Cout), np.int32) if want_acc else None
    out = np.empty((B, Ho, Wo, Cout), np.int8)
    r = None if res is None else np.ascontiguousarray(res, dtype=np.int8)
    if bench_iters > 0:
        ms = C.c_float(0)
        rc = lib.ffcu_conv_bench(device, C.byref(L), B, mode, 0 if impl == "tc" else 1, _ptr(xp), _ptr(r), _ptr(out), _ptr(out2),
                                 bench_iters, C.byref(ms))
        if rc != 0:
            raise RuntimeError(f"ffcu_conv_bench rc={rc}: " + lib.ffcu_last_error().decode())
        return (float(ms.value), out, out2) if bn2 is not None else (float(ms.value), out)
    rc = lib.ffcu_conv_once(device, C.byref(L), B, mode, 0 if impl == "tc" else 1, _ptr(xp), _ptr(r), _ptr(acc), _ptr(out), _ptr(out2))
    if rc != 0:
        raise RuntimeError(f"ffcu_conv_once rc={rc}: " + lib.ffcu_last_error().decode())
    if bn2 is not None:
        return acc, out, out2
    return acc, out


def winograd_f23(x: np.ndarray, w_oihw: np.ndarray, iters: int = 1, device: int = 0):
    """3x3 stride-1 pad-1 conv by exact-integer Winograd F(2,3) on the CUDA cores (ffcu_winograd_f23_once):
    x int8 [B,H,W,Cin], w int8 [Cout,Cin,3,3] -> (int32 [B,H,W,Cout] = 4 x the direct accumulators, ms per run)."""
    lib = load_library()
    B, H, W, Cin = x.shape
    Cout = w_oihw.shape[0]
    xc = np.ascontiguousarray(x, dtype=np.int8)
    wc = np.ascontiguousarray(w_oihw, dtype=np.int8)
    out = np.empty((B, H, W, Cout), np.int32)
    ms = C.c_float(0)
    rc = lib.ffcu_winograd_f23_once(device, _ptr(xc), _ptr(wc), B, H, W, Cin, Cout, iters, _ptr(out), C.byref(ms))
    if rc != 0:
        raise RuntimeError(f"ffcu_winograd_f23_once rc={rc}: " + lib.ffcu_last_error().decode())
    return out, float(ms.value)
