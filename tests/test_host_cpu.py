"""CPU: the C-ABI library loads, exports what include/*.h declares, and its host-side
logic (file parsing, error returns, cos_sim) behaves like the reference's. No GPU work."""
import ctypes as C
import os
import re
import struct

import numpy as np
import pytest

from conftest import ROOT
import fastface_b200 as ff


def _declared_symbols():
    names = set()
    for h in ("fastface.h", "ff_cuda.h"):
        src = open(os.path.join(ROOT, "include", h)).read()
        src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
        names |= set(re.findall(r"\b((?:fastface|ffcu)_[a-z0-9_]+)\s*\(", src))
    return names - {"fastface_trace_fn", "ffcu_trace_fn"}


def test_library_exports_every_declared_symbol(built_lib):
    lib = C.CDLL(built_lib)
    declared = _declared_symbols()
    assert {"fastface_create", "fastface_embed", "fastface_destroy", "fastface_embed_batch",
            "fastface_embed_batch_u8", "fastface_cos_sim", "fastface_cos_sim_matrix", "ffcu_cos_sim_matrix", "ffcu_submit", "ffcu_submit_u8", "ffcu_conv_once"} <= declared
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in include/ but not exported"


def test_null_arguments(built_lib):
    lib = ff.load_library()
    buf = np.zeros(ff.FACE_NELEMS, np.float32)
    out = np.zeros(512, np.float32)
    # reference: embed returns -1 on NULL arguments (libfastface.c:313), destroy(NULL) is a no-op (:473)
    assert lib.fastface_embed(None, buf.ctypes.data, out.ctypes.data) == -1
    assert lib.fastface_embed_batch(None, buf.ctypes.data, 1, out.ctypes.data) == -1
    assert lib.fastface_embed_batch_u8(None, buf.ctypes.data, 1, out.ctypes.data) == -1
    lib.fastface_destroy(None)
    assert lib.fastface_create(None) is None


def test_cos_sim_matches_go_wrapper_semantics(built_lib):
    rng = np.random.default_rng(0)
    a = rng.standard_normal(512).astype(np.float32)
    b = rng.standard_normal(512).astype(np.float32)
    want = np.float32(np.dot(a.astype(np.float64), b.astype(np.float64)) /
                      (np.sqrt(np.dot(a.astype(np.float64), a.astype(np.float64))) *
                       np.sqrt(np.dot(b.astype(np.float64), b.astype(np.float64)))))
    assert ff.FastFace.cos_sim(a, b) == pytest.approx(float(want), abs=1e-7)
    assert ff.FastFace.cos_sim(a, a) == pytest.approx(1.0, abs=1e-6)
    assert ff.FastFace.cos_sim(a, np.zeros(512, np.float32)) == 0.0   # zero norm -> 0 (fastface.go:164-166)


def _create_in(tmp, weights_bytes, opsc=True, n_ops=1):
    os.makedirs(os.path.join(tmp, "models"), exist_ok=True)
    w = os.path.join(tmp, "w.bin")
    open(w, "wb").write(weights_bytes)
    if opsc:
        with open(os.path.join(tmp, "models", "op_scales.bin"), "wb") as f:
            f.write(b"OPSC" + struct.pack("<If", n_ops, 1.0 / 127) + struct.pack(f"<{n_ops}f", *([0.01] * n_ops)))
    lib = ff.load_library()
    old = os.getcwd()
    os.chdir(tmp)
    try:
        h = lib.fastface_create(w.encode())
        err = lib.fastface_last_error().decode()
    finally:
        os.chdir(old)
    return h, err


def test_create_failures_return_null(built_lib, tmp_path):
    """fastface_create returns NULL on unreadable file, bad magic, old format versions,
    truncated payload, missing op_scales.bin and op-count mismatch (libfastface.c:233-237)."""
    lib = ff.load_library()
    assert lib.fastface_create(str(tmp_path / "missing.bin").encode()) is None
    h, err = _create_in(str(tmp_path / "a"), b"XXXX" + struct.pack("<I", 1))
    assert h is None and "magic" in err
    h, err = _create_in(str(tmp_path / "b"), b"FFW3" + struct.pack("<I", 1) + b"\x06")
    assert h is None and "FFW4" in err
    conv_hdr = b"\x01" + struct.pack("<6H", 64, 64, 3, 3, 1, 1)
    h, err = _create_in(str(tmp_path / "c"), b"FFW4" + struct.pack("<I", 1) + conv_hdr + b"\x00" * 100)
    assert h is None and "truncated" in err
    h, err = _create_in(str(tmp_path / "d"), b"FFW4" + struct.pack("<I", 1) + b"\x63")
    assert h is None and "bad op type" in err
    h, err = _create_in(str(tmp_path / "e"), b"FFW4" + struct.pack("<I", 1) + b"\x06", opsc=False)
    assert h is None and "op_scales" in err
    h, err = _create_in(str(tmp_path / "f"), b"FFW4" + struct.pack("<I", 1) + b"\x06", n_ops=2)
    assert h is None and "mismatch" in err


def test_plan_rejects_shape_mismatch(built_lib, tmp_path):
    """A conv whose Cin does not match the running tensor is refused at create."""
    conv = b"\x01" + struct.pack("<6H", 5, 8, 1, 1, 1, 0) + b"\x00" * 40 + b"\x00" * 64
    h, err = _create_in(str(tmp_path / "g"), b"FFW4" + struct.pack("<I", 1) + conv)
    assert h is None and "input channels" in err


def test_synth_model_is_the_177_op_sequence():
    from fastface_b200 import synth
    ops = synth.op_sequence()
    kinds = [o[0] for o in ops]
    assert len(ops) == 177
    assert kinds.count(synth.OP_CONV) == 53 and kinds.count(synth.OP_BN) == 25
    assert kinds.count(synth.OP_SAVE_ID) == 24 and kinds.count(synth.OP_BLOCK_START) == 24
    assert kinds.count(synth.OP_ADD) == 24 and kinds.count(synth.OP_PRELU) == 25
    macs, H = 0, 112
    cur_h = {0: 112}
    # work per face: 6.3093 GMAC
    h = 112
    for o in ops:
        if o[0] == synth.OP_CONV:
            _, cin, cout, k, s, p = o
            hin = h if not (k == 1) else h * 2      # shortcut reads the block input (pre-downsample)
            ho = (hin + 2 * p - k) // s + 1
            macs += ho * ho * cin * cout * k * k
            h = ho
    macs += 25088 * 512
    assert abs(macs / 1e9 - 6.3093) < 1e-3


def test_launch_list_never_writes_a_buffer_the_same_launch_reads(model_root, ffw4, tmp_path):
    """Activation buffers are reused by reference count.  No launch may write (output or fused-BN second output) a
    buffer it reads (input, residual).  A down-sampling block's [conv 3x3 stride 2][conv 1x1 stride 2 + ADD] pair can
    go out as ONE launch that reads both layers' inputs while it writes the second layer's outputs, tile by tile: for
    that pair the union counts, although as two launches the first conv's input is dead when the second one writes.
    (With the shortcut's output in the 3x3 conv's input buffer, a 32-face batch came back with faces 0-7 wrong.)"""
    import subprocess
    exe = str(tmp_path / "plan_buffers")
    host = os.path.join(ROOT, "fastface_b200", "csrc", "host")
    subprocess.run(["gcc", "-std=c11", "-O1", "-I" + os.path.join(ROOT, "include"), "-I" + host,
                    os.path.join(ROOT, "tests", "plan_buffers.c"), os.path.join(host, "ff_model.c"),
                    os.path.join(host, "ff_plan.c"), "-lm", "-o", exe], check=True)
    mdir = os.path.join(model_root, "models")
    out = subprocess.run([exe, ffw4, os.path.join(mdir, "op_scales.bin"), os.path.join(mdir, "op_scales_v2.bin")],
                         check=True, capture_output=True, text=True).stdout
    layers = []
    for line in out.splitlines():
        if line.startswith("L "):
            f = line.split()
            layers.append({f[k]: int(f[k + 1]) for k in range(2, len(f), 2)})
    assert len(layers) == 55                                   # input quantise + 53 convs + FC
    pairs = 0
    for i, l in enumerate(layers):
        reads = {l["src"], l["res"]} - {-1}
        writes = {l["dst"], l["bn2"]} - {-1}
        assert not (reads & writes), (i, l)
        if i and l["kind"] == 1 and l["k"] == 1 and l["stride"] == 2:
            m = layers[i - 1]
            assert m["k"] == 3 and m["stride"] == 2 and l["res"] == m["dst"], (i, m, l)
            pairs += 1
            assert not (({m["src"], l["src"]}) & (writes | {m["dst"]})), (i, m, l)
    assert pairs == 4
    n_bufs = int(out.split("N_BUFS")[1])
    assert n_bufs == 5


def _rss_kb():
    try:
        C.CDLL("libc.so.6").malloc_trim(0)      # hand free heap pages back first: what stays is what is still allocated
    except OSError:
        pass
    for line in open("/proc/self/status"):
        if line.startswith("VmRSS:"):
            return int(line.split()[1])
    return 0


def test_failing_create_does_not_leak(built_lib, tmp_path):
    """fastface_create that fails late (whole model parsed and planned, then no usable device, or a model
    refused by the planner) must hand back everything it allocated: a loop of failures leaves the
    resident set where it was.  The 43.7 MB synthetic model makes a leak of the model or the plan visible
    after a few rounds."""
    from fastface_b200 import synth
    root = str(tmp_path / "leak")
    ffw4 = synth.materialize(root, 0)
    lib = ff.load_library()
    have_gpu = lib.ffcu_device_count() > 0
    old = os.getcwd()
    os.chdir(root)
    try:
        env_old = os.environ.get("FASTFACE_DEVICES")
        os.environ["FASTFACE_DEVICES"] = "63"            # no such ordinal: fails after load + plan on any host
        for _ in range(3):
            assert lib.fastface_create(ffw4.encode()) is None
        base = _rss_kb()
        for _ in range(12):
            assert lib.fastface_create(ffw4.encode()) is None
        grown = _rss_kb() - base
    finally:
        os.chdir(old)
        if env_old is None:
            os.environ.pop("FASTFACE_DEVICES", None)
        else:
            os.environ["FASTFACE_DEVICES"] = env_old
    # one leaked model would be >= 43 MB per round (516 MB over the loop); allow allocator noise
    assert grown < 40 * 1024, f"resident set grew by {grown} kB over 12 failing creates (gpu present: {have_gpu})"
