"""Seeded synthetic IR-ResNet50 model files in the reference's on-disk formats.

The reference's shipped weight file (models/w600k_r50_ffw4.bin) is not
redistributable, so tests and the benchmark run on a random-init network of
the same architecture: the 177-op sequence the reference's loader walks
(kernels/ffw2_loader.c:94-157), written as FFW4 (writer side:
prepare_weights_v3.py:280-307), plus the OPSC / OPSC2 activation-scale files
(libfastface.c:133-204).

Weights: int8 = clip(round(N(0, 40)), +-127); per-output-channel scale
log-uniform in [1e-3, 1e-1]; folded bias ~ N(0, 0.1); BN scale U[0.5, 1.5],
BN offset N(0, 0.1); PReLU slope U[0, 0.25].

Activation scales come from a committed calibration table
(fastface_b200/data/synth_seed<seed>.opsc2): per-channel p99.9 of the seeded
run, produced once by oracle/calibrate_synth.py.  Writing the model never
runs any forward pass.
"""
from __future__ import annotations

import os
import struct
from typing import List, Tuple

import numpy as np

OP_CONV, OP_BN, OP_PRELU, OP_ADD, OP_GEMM, OP_FLATTEN, OP_SAVE_ID, OP_BLOCK_START = range(1, 9)

STAGE_CHANNELS = (64, 128, 256, 512)
STAGE_BLOCKS = (3, 4, 14, 3)

_DATA_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "data")


def op_sequence() -> List[Tuple]:
    """The 177 ops of the IR-ResNet50 export, as (type, *params)."""
    ops: List[Tuple] = [(OP_CONV, 3, 64, 3, 1, 1), (OP_PRELU, 64)]
    cin = 64
    for c, nb in zip(STAGE_CHANNELS, STAGE_BLOCKS):
        for b in range(nb):
            if b == 0:
                ops += [(OP_BLOCK_START,), (OP_BN, cin), (OP_CONV, cin, c, 3, 1, 1), (OP_PRELU, c),
                        (OP_CONV, c, c, 3, 2, 1), (OP_SAVE_ID,), (OP_CONV, cin, c, 1, 2, 0), (OP_ADD,)]
            else:
                ops += [(OP_SAVE_ID,), (OP_BLOCK_START,), (OP_BN, c), (OP_CONV, c, c, 3, 1, 1),
                        (OP_PRELU, c), (OP_CONV, c, c, 3, 1, 1), (OP_ADD,)]
            cin = c
    ops += [(OP_BN, 512), (OP_FLATTEN,), (OP_GEMM, 512, 25088)]
    assert len(ops) == 177
    return ops


def _int8_weights(rng: np.random.Generator, n: int) -> np.ndarray:
    w = np.rint(rng.standard_normal(n, dtype=np.float32) * np.float32(40.0))
    return np.clip(w, -127, 127).astype(np.int8)


def _log_uniform(rng: np.random.Generator, n: int, lo: float, hi: float) -> np.ndarray:
    u = rng.random(n, dtype=np.float64)
    return np.exp(np.log(lo) + u * (np.log(hi) - np.log(lo))).astype(np.float32)


def write_ffw4(path: str, seed: int = 0) -> None:
    """Write the seeded synthetic network as an FFW4 file (about 43.7 MB)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    ops = op_sequence()
    with open(path, "wb") as f:
        f.write(b"FFW4")
        f.write(struct.pack("<I", len(ops)))
        for op in ops:
            t = op[0]
            f.write(struct.pack("<B", t))
            if t == OP_CONV:
                _, cin, cout, k, stride, pad = op
                f.write(struct.pack("<6H", cin, cout, k, k, stride, pad))
                f.write(_int8_weights(rng, cout * cin * k * k).tobytes())
                f.write(_log_uniform(rng, cout, 1e-3, 1e-1).tobytes())
                f.write((rng.standard_normal(cout, dtype=np.float32) * np.float32(0.1)).tobytes())
            elif t == OP_BN:
                n = op[1]
                f.write(struct.pack("<H", n))
                f.write((0.5 + rng.random(n, dtype=np.float32)).astype(np.float32).tobytes())
                f.write((rng.standard_normal(n, dtype=np.float32) * np.float32(0.1)).tobytes())
            elif t == OP_PRELU:
                n = op[1]
                f.write(struct.pack("<H", n))
                f.write((rng.random(n, dtype=np.float32) * np.float32(0.25)).astype(np.float32).tobytes())
            elif t == OP_GEMM:
                _, n, k = op
                f.write(struct.pack("<II", n, k))
                f.write(_int8_weights(rng, n * k).tobytes())
                f.write(_log_uniform(rng, n, 1e-3, 1e-1).tobytes())
                f.write((rng.standard_normal(n, dtype=np.float32) * np.float32(0.1)).tobytes())


def faces(n: int, seed: int = 0) -> np.ndarray:
    """n seeded faces, float32 HWC [n,112,112,3], uniform in [-1, 1]."""
    rng = np.random.Generator(np.random.PCG64(1000003 + seed))
    return (rng.random((n, 112, 112, 3), dtype=np.float32) * np.float32(2.0) - np.float32(1.0))


def scale_table_path(seed: int = 0) -> str:
    return os.path.join(_DATA_DIR, f"synth_seed{seed}.opsc2")


def write_opsc_from_opsc2(opsc2_path: str, opsc_path: str) -> None:
    """Per-tensor OPSC whose scalar for each op is the largest per-channel scale."""
    d = open(opsc2_path, "rb").read()
    assert d[:5] == b"OPSC2"
    n_ops, n_in = struct.unpack_from("<II", d, 5)
    in_scale = np.frombuffer(d, "<f4", n_in, 13)
    p = 13 + 4 * n_in
    scal = np.zeros(n_ops, np.float32)
    for i in range(n_ops):
        (nch,) = struct.unpack_from("<I", d, p)
        p += 4
        if nch:
            scal[i] = np.frombuffer(d, "<f4", nch, p).max()
            p += 4 * nch
    with open(opsc_path, "wb") as f:
        f.write(b"OPSC")
        f.write(struct.pack("<I", n_ops))
        f.write(struct.pack("<f", float(in_scale.max())))
        f.write(scal.astype("<f4").tobytes())


def materialize(root: str, seed: int = 0) -> str:
    """Create <root>/models/{synth_ffw4.bin, op_scales.bin, op_scales_v2.bin}.

    The directory layout mirrors what fastface_create expects relative to the
    working directory (libfastface.c:236-240).  Returns the FFW4 path.
    """
    mdir = os.path.join(root, "models")
    os.makedirs(mdir, exist_ok=True)
    ffw4 = os.path.join(mdir, f"synth_seed{seed}_ffw4.bin")
    if not os.path.exists(ffw4):
        tmp = ffw4 + f".tmp{os.getpid()}"
        write_ffw4(tmp, seed)
        os.replace(tmp, ffw4)
    table = scale_table_path(seed)
    if not os.path.exists(table):
        raise FileNotFoundError(f"missing calibration table {table}; run oracle/calibrate_synth.py")
    v2 = os.path.join(mdir, "op_scales_v2.bin")
    with open(table, "rb") as src, open(v2 + f".tmp{os.getpid()}", "wb") as dst:
        dst.write(src.read())
    os.replace(v2 + f".tmp{os.getpid()}", v2)
    v1 = os.path.join(mdir, "op_scales.bin")
    write_opsc_from_opsc2(v2, v1 + f".tmp{os.getpid()}")
    os.replace(v1 + f".tmp{os.getpid()}", v1)
    return ffw4
