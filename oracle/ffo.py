"""ctypes access to the test oracle (TEST INFRASTRUCTURE -- never imported by the library).

* ``Oracle``   : the plain-C restatement in oracle/libffo.so (ff_oracle.c).
* ``RefLib``   : the reference's own libfastface, compiled from its sources into
                 oracle/_ref/ by oracle/Makefile (needs an AVX-VNNI host CPU).
* ``run_ref_trace`` : runs the reference's batched CLI linked with the ld --wrap
                 shim and returns its per-call CRC records.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
import zlib
from typing import Callable, List, Optional, Tuple

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")

STRICT, CONTRACT = 0, 1
TRACE_INPUT_I8, TRACE_CONV_ACC, TRACE_CONV_OUT, TRACE_BN_OUT, TRACE_FC_OUT = range(5)
KIND_LETTER = {TRACE_INPUT_I8: "Q", TRACE_CONV_ACC: "A", TRACE_CONV_OUT: "O", TRACE_BN_OUT: "B", TRACE_FC_OUT: "F"}
KIND_DTYPE = {TRACE_INPUT_I8: np.int8, TRACE_CONV_ACC: np.int32, TRACE_CONV_OUT: np.int8,
              TRACE_BN_OUT: np.int8, TRACE_FC_OUT: np.float32}

_TRACE_CB = C.CFUNCTYPE(None, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_size_t)


def host_has_avx_vnni() -> bool:
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    return " avx_vnni" in line
    except OSError:
        pass
    return False


def build(force: bool = False) -> None:
    """Compile libffo.so and, when the reference sources are present, oracle/_ref/."""
    if force or not os.path.exists(os.path.join(HERE, "libffo.so")) or \
            os.path.getmtime(os.path.join(HERE, "libffo.so")) < os.path.getmtime(os.path.join(HERE, "ff_oracle.c")):
        subprocess.run(["make", "-C", HERE, "port"], check=True, capture_output=True)
    subprocess.run(["make", "-C", HERE, "ref"], check=True, capture_output=True)


def _fp(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


class Oracle:
    def __init__(self, ffw4: str, opsc: str, opsc2: Optional[str]):
        build()
        self.lib = C.CDLL(os.path.join(HERE, "libffo.so"))
        L = self.lib
        L.ffo_load.restype = C.c_void_p
        L.ffo_load.argtypes = [C.c_char_p, C.c_char_p, C.c_char_p]
        L.ffo_free.argtypes = [C.c_void_p]
        L.ffo_forward.restype = C.c_int
        L.ffo_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, _TRACE_CB, C.c_void_p]
        L.ffo_n_ops.argtypes = [C.c_void_p]
        L.ffo_has_per_channel.argtypes = [C.c_void_p]
        self.h = L.ffo_load(ffw4.encode(), opsc.encode(), opsc2.encode() if opsc2 else None)
        if not self.h:
            raise RuntimeError("ffo_load failed")

    def close(self):
        if self.h:
            self.lib.ffo_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def has_per_channel(self) -> bool:
        return bool(self.lib.ffo_has_per_channel(self.h))

    def forward(self, faces: np.ndarray, mode: int = CONTRACT,
                trace: Optional[Callable[[int, int, np.ndarray], None]] = None) -> np.ndarray:
        faces = np.ascontiguousarray(faces, dtype=np.float32).reshape(-1, 112, 112, 3)
        B = faces.shape[0]
        out = np.empty((B, 512), np.float32)

        def _cb(user, op_index, kind, data, n):
            arr = np.ctypeslib.as_array(C.cast(data, C.POINTER(C.c_uint8)),
                                        shape=(n * np.dtype(KIND_DTYPE[kind]).itemsize,))
            trace(op_index, kind, arr.view(KIND_DTYPE[kind]))

        cb = _TRACE_CB(_cb) if trace else C.cast(None, _TRACE_CB)
        rc = self.lib.ffo_forward(self.h, _fp(faces), B, _fp(out), mode, cb, None)
        if rc != 0:
            raise RuntimeError(f"ffo_forward rc={rc}")
        return out

    def forward_crc(self, faces: np.ndarray, mode: int = CONTRACT) -> Tuple[np.ndarray, List[Tuple[str, int, int, int]]]:
        """Forward + the same (kind, call#, n, crc32) records the reference shim writes."""
        recs: List[Tuple[str, int, int, int]] = []
        counts = {}
        B = np.asarray(faces).reshape(-1, 112, 112, 3).shape[0]

        def tr(op_index, kind, arr):
            k = KIND_LETTER[kind]
            if k == "F":      # the reference calls the matvec once per face
                for b in range(B):
                    i = counts.get(k, 0); counts[k] = i + 1
                    row = arr.reshape(B, -1)[b]
                    recs.append((k, i, row.size, zlib.crc32(row.tobytes())))
                return
            i = counts.get(k, 0); counts[k] = i + 1
            recs.append((k, i, arr.size, zlib.crc32(arr.tobytes())))

        out = self.forward(faces, mode, tr)
        return out, recs


def calibrate(ffw4: str, faces: np.ndarray, percentile: float, opsc_out: str, opsc2_out: str) -> None:
    build()
    lib = C.CDLL(os.path.join(HERE, "libffo.so"))
    lib.ffo_calibrate.restype = C.c_int
    lib.ffo_calibrate.argtypes = [C.c_char_p, C.c_void_p, C.c_int, C.c_double, C.c_char_p, C.c_char_p]
    faces = np.ascontiguousarray(faces, dtype=np.float32).reshape(-1, 112, 112, 3)
    rc = lib.ffo_calibrate(ffw4.encode(), _fp(faces), faces.shape[0], percentile,
                           opsc_out.encode(), opsc2_out.encode())
    if rc != 0:
        raise RuntimeError(f"ffo_calibrate rc={rc}")


def ref_available() -> bool:
    return host_has_avx_vnni() and os.path.exists(os.path.join(REF_DIR, "libfastface_ref.so"))


class RefLib:
    """The reference's fastface_create/embed/destroy (fastface.h:27-42), b=1.

    The reference opens models/op_scales.bin relative to the working directory
    (libfastface.c:236), so create() runs with cwd=model_root.
    """

    def __init__(self, model_root: str, ffw4: str, strict: bool = False, opsc2_path: Optional[str] = None):
        if not ref_available():
            raise RuntimeError("reference library unavailable (not built, or host lacks avx_vnni)")
        name = "libfastface_ref_strict.so" if strict else "libfastface_ref.so"
        self.lib = C.CDLL(os.path.join(REF_DIR, name))
        self.lib.fastface_create.restype = C.c_void_p
        self.lib.fastface_create.argtypes = [C.c_char_p]
        self.lib.fastface_embed.restype = C.c_int
        self.lib.fastface_embed.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        self.lib.fastface_destroy.argtypes = [C.c_void_p]
        cwd = os.getcwd()
        old = os.environ.get("OPSC2_PATH")
        try:
            os.chdir(model_root)
            if opsc2_path is not None:
                os.environ["OPSC2_PATH"] = opsc2_path
            self.h = self.lib.fastface_create(os.path.abspath(ffw4).encode())
        finally:
            os.chdir(cwd)
            if opsc2_path is not None:
                if old is None:
                    os.environ.pop("OPSC2_PATH", None)
                else:
                    os.environ["OPSC2_PATH"] = old
        if not self.h:
            raise RuntimeError("reference fastface_create failed")

    def embed(self, face: np.ndarray) -> np.ndarray:
        face = np.ascontiguousarray(face, dtype=np.float32).reshape(112, 112, 3)
        out = np.empty(512, np.float32)
        rc = self.lib.fastface_embed(self.h, _fp(face), _fp(out))
        if rc != 0:
            raise RuntimeError(f"reference fastface_embed rc={rc}")
        return out

    def close(self):
        if self.h:
            self.lib.fastface_destroy(self.h)
            self.h = None


def ref_embed_many(model_root: str, ffw4: str, faces: np.ndarray, batch: int = 32, threads: Optional[int] = None) -> np.ndarray:
    """Embeddings of any number of faces from the reference's batched CLI through its --server
    protocol (arcface_forward_int8_batched.c:531-553), `batch` faces per request; the last
    request is padded with copies of the last face.  The reference treats the faces of a batch
    independently, so the batch size of the requests does not change a face's result."""
    exe = os.path.join(REF_DIR, "fastface_int8_batched")
    faces = np.ascontiguousarray(faces, dtype=np.float32).reshape(-1, 112, 112, 3)
    n = faces.shape[0]
    env = dict(os.environ)
    env.pop("OPSC2_PATH", None)
    if threads:
        env["OMP_NUM_THREADS"] = str(threads)
    p = subprocess.Popen([exe, os.path.abspath(ffw4), "--batch", str(batch), "--server"], cwd=model_root, env=env,
                         stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, bufsize=0)
    out = np.empty((n, 512), np.float32)
    try:
        for k in range(0, n, batch):
            chunk = faces[k:k + batch]
            if chunk.shape[0] < batch:
                chunk = np.concatenate([chunk, np.repeat(chunk[-1:], batch - chunk.shape[0], 0)])
            p.stdin.write(chunk.tobytes())
            p.stdin.flush()
            need, buf = batch * 512 * 4, b""
            while len(buf) < need:
                part = p.stdout.read(need - len(buf))
                if not part:
                    raise RuntimeError("reference server closed its pipe")
                buf += part
            emb = np.frombuffer(buf, np.float32).reshape(batch, 512)
            out[k:k + batch] = emb[:min(batch, n - k)]
    finally:
        try:
            p.stdin.close()
            p.wait(timeout=30)
        except Exception:
            p.kill()
    return out


def run_ref_trace(model_root: str, ffw4: str, faces: np.ndarray, strict: bool = False,
                  dump_dir: Optional[str] = None, threads: Optional[int] = None):
    """Run the traced reference CLI on the given faces (arcface_forward_int8_batched.c
    --in/--out mode).  Returns (embeddings [B,512], [(kind, call#, n_elems, crc32)])."""
    exe = os.path.join(REF_DIR, "fastface_int8_batched_trace" + ("_strict" if strict else ""))
    faces = np.ascontiguousarray(faces, dtype=np.float32).reshape(-1, 112, 112, 3)
    B = faces.shape[0]
    tag = f"{os.getpid()}_{'s' if strict else 'c'}"
    in_path = os.path.join(model_root, f"_trace_in_{tag}.bin")
    out_path = os.path.join(model_root, f"_trace_out_{tag}.bin")
    log_path = os.path.join(model_root, f"_trace_log_{tag}.txt")
    faces.tofile(in_path)
    env = dict(os.environ, FF_TRACE_OUT=log_path)
    env.pop("OPSC2_PATH", None)
    if dump_dir:
        env["FF_TRACE_DUMP_DIR"] = dump_dir
    if threads:
        env["OMP_NUM_THREADS"] = str(threads)
    r = subprocess.run([exe, os.path.abspath(ffw4), "--batch", str(B), "--in", in_path, "--out", out_path],
                       cwd=model_root, env=env, capture_output=True, timeout=1800)
    if r.returncode != 0:
        raise RuntimeError(f"reference CLI failed rc={r.returncode}: {r.stderr.decode()[-500:]}")
    emb = np.fromfile(out_path, np.float32).reshape(B, 512)
    recs = []
    with open(log_path) as f:
        for line in f:
            k, i, n, crc = line.split()
            recs.append((k, int(i), int(n), int(crc, 16)))
    for p in (in_path, out_path, log_path):
        os.remove(p)
    return emb, recs
