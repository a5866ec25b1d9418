"""FFW4 / OPSC2 / OPSC producer: fp32 IR-ResNet weights + calibration faces -> the three model files.

Restates, in numpy as the reference does, the arithmetic of the reference's export scripts:

* per-output-channel symmetric int8 quantisation, ``scale = absmax / 127``, ``round(w / scale)``
  with numpy's round-half-to-even (prepare_weights_v3.py:37-43);
* BN folding to (scale, offset): ``gamma / sqrt(var + eps)``, ``beta - mean * scale`` (:221-229);
* the FFW4 conv fold: weights pre-multiplied by the per-input-channel activation scale of the
  tensor the conv reads, so the run-time input scale is 1.0 (:206-217);
* the FFW4 FC fold: weights pre-multiplied by the pre-flatten per-channel scale in the C
  driver's flatten order ``k = c * spatial + hw``, and by the BN that trails the Gemm, whose
  offset goes into the bias (:245-267);
* the FFW4 writer (:280-307), the OPSC2 writer (export_op_scales_v2.py:153-164) and the
  per-tensor OPSC file (export_op_scales.py:109-113);
* percentile calibration: per image the per-channel absmax of every tensor, then the given
  percentile over images, ``/ 127``, zero replaced by 1e-6 (calibrate_percentile_int8.py:105-118).

What is NOT here is the reference's ONNX graph walk (extract_onnx.py + the node loop of
prepare_weights_v3.py:184-278): the ONNX model the reference exports from is not
redistributable, so the input of this module is the network already in FFW4 op order with fp32
parameters (``FloatOp`` list; ``synth_float_model`` makes a seeded one of the IR-ResNet50
shape).  Real-weights path unpinned: ONNX model absent.

Nothing here runs on the GPU or is needed at inference time; it is the tool that makes the
files ``fastface_create`` loads.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from .synth import (OP_ADD, OP_BLOCK_START, OP_BN, OP_CONV, OP_FLATTEN, OP_GEMM, OP_PRELU, OP_SAVE_ID, op_sequence)


@dataclass
class FloatOp:
    """One FFW4 op with fp32 parameters (arrays are float32)."""
    kind: int
    w: Optional[np.ndarray] = None        # conv [Cout, Cin, Kh, Kw] / gemm [N, K]
    bias: Optional[np.ndarray] = None     # conv / gemm
    stride: int = 1
    pad: int = 0
    gamma: Optional[np.ndarray] = None    # BN (also: the BN trailing the gemm, folded into it)
    beta: Optional[np.ndarray] = None
    mean: Optional[np.ndarray] = None
    var: Optional[np.ndarray] = None
    eps: float = 1e-5
    slope: Optional[np.ndarray] = None    # PReLU
    extra: dict = field(default_factory=dict)


def quantize_per_channel_int8(w: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """int8 weights and fp32 per-output-channel scales (prepare_weights_v3.py:37-43)."""
    w = np.asarray(w, np.float32)
    co = w.shape[0]
    absmax = np.abs(w.reshape(co, -1)).max(axis=1)
    scales = absmax / 127.0
    safe = np.where(scales > 0, scales, 1.0)
    w_int = np.round(w / safe.reshape((-1,) + (1,) * (w.ndim - 1))).astype(np.int8)
    return w_int, scales.astype(np.float32)


def fold_bn(gamma, beta, mean, var, eps) -> Tuple[np.ndarray, np.ndarray]:
    """BN as y = x * scale + offset (prepare_weights_v3.py:221-229)."""
    scale = gamma / np.sqrt(var + eps)
    offset = beta - mean * scale
    return scale.astype(np.float32), offset.astype(np.float32)


def fold_conv(w: np.ndarray, in_scale: Optional[np.ndarray]) -> Tuple[np.ndarray, np.ndarray]:
    """FFW4 conv weights: W[oc, ci] * S_a[ci], then per-Cout quantisation (prepare_weights_v3.py:206-217)."""
    w = np.asarray(w, np.float32)
    cin = w.shape[1]
    if in_scale is not None and in_scale.shape == (cin,):
        w = w * in_scale.reshape(1, cin, 1, 1)
    return quantize_per_channel_int8(w)


def fold_gemm(w: np.ndarray, b: np.ndarray, pre_flatten_scale: np.ndarray,
              trailing_bn: Optional[Tuple[np.ndarray, np.ndarray]]) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """FFW4 FC: W[n, k] * S_c[k // spatial] (flatten order k = c * spatial + hw), times the trailing BN's
    scale, its offset into the bias (prepare_weights_v3.py:245-267)."""
    w = np.asarray(w, np.float32)
    n, k = w.shape
    spatial = k // len(pre_flatten_scale)
    assert k == spatial * len(pre_flatten_scale)
    s_flat = np.repeat(pre_flatten_scale, spatial).astype(np.float32)
    w_eff = w * s_flat[None, :]
    b_eff = np.asarray(b, np.float32).copy()
    if trailing_bn is not None:
        g, o = trailing_bn
        w_eff = w_eff * g[:, None]
        b_eff = b_eff * g + o
    w_int, scales = quantize_per_channel_int8(w_eff.reshape(n, k, 1, 1))
    return w_int.reshape(n, k), scales, b_eff.astype(np.float32)


def percentile_scales(per_image_absmax: np.ndarray, percentile: float) -> np.ndarray:
    """[n_images, C] per-image absmax -> per-channel scale (calibrate_percentile_int8.py:105-118)."""
    pc = np.percentile(per_image_absmax, percentile, axis=0).astype(np.float32)
    pc = np.where(pc > 0, pc, 1e-6).astype(np.float32)
    return pc / 127.0


# ---------------------------------------------------------------------------
# fp32 evaluation of the op list (calibration, and the accuracy check of the produced files)
# ---------------------------------------------------------------------------
def _conv_nhwc(x: np.ndarray, w: np.ndarray, bias: np.ndarray, stride: int, pad: int) -> np.ndarray:
    """x [H, W, Cin] f32, w [Cout, Cin, Kh, Kw] -> [Ho, Wo, Cout] by im2col + one matmul."""
    h, wd, cin = x.shape
    cout, _, kh, kw = w.shape
    xp = np.pad(x, ((pad, pad), (pad, pad), (0, 0)))
    ho = (h + 2 * pad - kh) // stride + 1
    wo = (wd + 2 * pad - kw) // stride + 1
    sh, sw, sc = xp.strides
    cols = np.lib.stride_tricks.as_strided(xp, (ho, wo, kh, kw, cin), (sh * stride, sw * stride, sh, sw, sc))
    a = cols.reshape(ho * wo, kh * kw * cin)
    b = np.transpose(w, (2, 3, 1, 0)).reshape(kh * kw * cin, cout)
    return (a @ b + bias).reshape(ho, wo, cout).astype(np.float32)


def float_forward(ops: Sequence[FloatOp], face: np.ndarray, record: Optional[Dict[int, np.ndarray]] = None) -> np.ndarray:
    """fp32 forward of one face [112,112,3] through the op list with the data flow of the reference's
    driver (libfastface.c:349-466): BLOCK_START snapshots the block input, a conv that follows SAVE_ID
    reads that snapshot (the shortcut), ADD adds the saved tensor.  record[i] receives the per-channel
    absmax of op i's output (the tensor the exporter attaches a scale to)."""
    a = np.asarray(face, np.float32).reshape(112, 112, 3)
    block_in = a
    saved = None
    for i, op in enumerate(ops):
        if op.kind == OP_BLOCK_START:
            block_in = a
            continue
        if op.kind == OP_SAVE_ID:
            saved = a
            continue
        if op.kind == OP_CONV:
            src = block_in if (i > 0 and ops[i - 1].kind == OP_SAVE_ID) else a
            a = _conv_nhwc(src, op.w, op.bias, op.stride, op.pad)
        elif op.kind == OP_BN:
            s, o = fold_bn(op.gamma, op.beta, op.mean, op.var, op.eps)
            a = (a * s + o).astype(np.float32)
        elif op.kind == OP_PRELU:
            a = np.where(a < 0, a * op.slope, a).astype(np.float32)
        elif op.kind == OP_ADD:
            a = (a + saved).astype(np.float32)
        elif op.kind == OP_FLATTEN:
            a = np.transpose(a, (2, 0, 1)).reshape(-1)          # NCHW flatten: k = c * 49 + h * 7 + w
        elif op.kind == OP_GEMM:
            a = (op.w @ a + op.bias).astype(np.float32)
            if op.gamma is not None:                            # the BN that trails the Gemm
                s, o = fold_bn(op.gamma, op.beta, op.mean, op.var, op.eps)
                a = (a * s + o).astype(np.float32)
        if record is not None:
            v = np.abs(a)
            record[i] = v.reshape(-1, v.shape[-1]).max(axis=0) if v.ndim == 3 else v
    return a


def calibrate(ops: Sequence[FloatOp], faces: np.ndarray, percentile: float = 99.9) -> Tuple[np.ndarray, Dict[int, np.ndarray]]:
    """Per-channel activation scales: (input scale [3], {op index: scale of its output})."""
    faces = np.asarray(faces, np.float32).reshape(-1, 112, 112, 3)
    per_op: Dict[int, List[np.ndarray]] = {}
    for f in faces:
        rec: Dict[int, np.ndarray] = {}
        float_forward(ops, f, rec)
        for i, v in rec.items():
            per_op.setdefault(i, []).append(v)
    in_absmax = np.abs(faces).reshape(faces.shape[0], -1, 3).max(axis=1)
    return percentile_scales(in_absmax, percentile), {i: percentile_scales(np.stack(v), percentile) for i, v in per_op.items()}


# ---------------------------------------------------------------------------
# writers
# ---------------------------------------------------------------------------
def build_files(ops: Sequence[FloatOp], in_scale: np.ndarray, out_scales: Dict[int, np.ndarray]) -> Tuple[bytes, bytes, bytes]:
    """(FFW4, OPSC2, OPSC) for the op list with the given activation scales."""
    ffw4 = [b"FFW4", struct.pack("<I", len(ops))]
    cur_scale: Optional[np.ndarray] = np.asarray(in_scale, np.float32)   # scale of the running tensor
    block_scale = cur_scale
    pre_flatten: Optional[np.ndarray] = None
    for i, op in enumerate(ops):
        ffw4.append(struct.pack("<B", op.kind))
        if op.kind == OP_BLOCK_START:
            block_scale = cur_scale
        elif op.kind == OP_CONV:
            src_scale = block_scale if (i > 0 and ops[i - 1].kind == OP_SAVE_ID) else cur_scale
            w_int, scales = fold_conv(op.w, src_scale)
            cout, cin, kh, kw = op.w.shape
            ffw4 += [struct.pack("<6H", cin, cout, kh, kw, op.stride, op.pad), w_int.tobytes(), scales.tobytes(),
                     np.asarray(op.bias, np.float32).tobytes()]
            cur_scale = out_scales.get(i)
        elif op.kind == OP_BN:
            s, o = fold_bn(op.gamma, op.beta, op.mean, op.var, op.eps)
            ffw4 += [struct.pack("<H", s.size), s.tobytes(), o.tobytes()]
            cur_scale = out_scales.get(i)
        elif op.kind == OP_PRELU:
            ffw4 += [struct.pack("<H", op.slope.size), np.asarray(op.slope, np.float32).tobytes()]
            cur_scale = out_scales.get(i)
        elif op.kind == OP_ADD:
            cur_scale = out_scales.get(i)
        elif op.kind == OP_FLATTEN:
            pre_flatten = cur_scale
        elif op.kind == OP_GEMM:
            tb = fold_bn(op.gamma, op.beta, op.mean, op.var, op.eps) if op.gamma is not None else None
            w_int, scales, b_eff = fold_gemm(op.w, op.bias, pre_flatten, tb)
            n, k = op.w.shape
            ffw4 += [struct.pack("<II", n, k), w_int.tobytes(), scales.tobytes(), b_eff.tobytes()]
    # OPSC2: "OPSC2", n_ops, n_in, in_scale, then per op nch + scales (0 for markers)
    v2 = [b"OPSC2", struct.pack("<II", len(ops), len(in_scale)), np.asarray(in_scale, np.float32).tobytes()]
    scal = np.zeros(len(ops), np.float32)
    for i, op in enumerate(ops):
        s = None if op.kind in (OP_BLOCK_START, OP_SAVE_ID) else out_scales.get(i)
        if s is None:
            v2.append(struct.pack("<I", 0))
        else:
            s = np.asarray(s, np.float32).reshape(-1)
            v2 += [struct.pack("<I", s.size), s.tobytes()]
            scal[i] = s.max()
    # OPSC (per tensor): the largest per-channel scale stands for the tensor
    v1 = [b"OPSC", struct.pack("<I", len(ops)), struct.pack("<f", float(np.max(in_scale))), scal.astype("<f4").tobytes()]
    return b"".join(ffw4), b"".join(v2), b"".join(v1)


def synth_float_model(seed: int = 0, weight_std: float = 1.0) -> List[FloatOp]:
    """A seeded fp32 network of the IR-ResNet50 shape (the 177-op sequence), He-style conv weights so that
    activations keep a sane range through 50 layers."""
    rng = np.random.Generator(np.random.PCG64(seed))
    ops: List[FloatOp] = []

    def bn(n):
        return dict(gamma=(0.8 + 0.4 * rng.random(n)).astype(np.float32), beta=(0.05 * rng.standard_normal(n)).astype(np.float32),
                    mean=(0.05 * rng.standard_normal(n)).astype(np.float32), var=(0.8 + 0.4 * rng.random(n)).astype(np.float32))

    for spec in op_sequence():
        t = spec[0]
        if t == OP_CONV:
            _, cin, cout, k, stride, pad = spec
            std = weight_std * np.sqrt(1.0 / (cin * k * k))
            ops.append(FloatOp(OP_CONV, w=(rng.standard_normal((cout, cin, k, k)) * std).astype(np.float32),
                               bias=(0.02 * rng.standard_normal(cout)).astype(np.float32), stride=stride, pad=pad))
        elif t == OP_BN:
            ops.append(FloatOp(OP_BN, **bn(spec[1])))
        elif t == OP_PRELU:
            ops.append(FloatOp(OP_PRELU, slope=(0.25 * rng.random(spec[1])).astype(np.float32)))
        elif t == OP_GEMM:
            _, n, k = spec
            ops.append(FloatOp(OP_GEMM, w=(rng.standard_normal((n, k)) * np.sqrt(1.0 / k)).astype(np.float32),
                               bias=(0.02 * rng.standard_normal(n)).astype(np.float32), **bn(n)))
        else:
            ops.append(FloatOp(t))
    return ops


def write_model(root: str, ops: Sequence[FloatOp], calib_faces: np.ndarray, percentile: float = 99.9,
                name: str = "produced_ffw4.bin") -> str:
    """Calibrate, fold, quantise and write <root>/models/{name, op_scales_v2.bin, op_scales.bin}; returns the FFW4 path."""
    import os
    in_scale, out_scales = calibrate(ops, calib_faces, percentile)
    ffw4, v2, v1 = build_files(ops, in_scale, out_scales)
    mdir = os.path.join(root, "models")
    os.makedirs(mdir, exist_ok=True)
    path = os.path.join(mdir, name)
    for p, data in ((path, ffw4), (os.path.join(mdir, "op_scales_v2.bin"), v2), (os.path.join(mdir, "op_scales.bin"), v1)):
        with open(p, "wb") as f:
            f.write(data)
    return path
