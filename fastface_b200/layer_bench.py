"""Single-layer microbenchmark: one INT8 convolution through the C-ABI, timed on the device.

    python -m fastface_b200.layer_bench [--case conv56] [--batch 8] [--iters 50] [--winograd]

Cases are layer shapes of the IR-ResNet50 (name: Cin, Cout, H, kernel, stride).  The default,
conv56 at batch 8, is the reference's own single-layer case (bench_batched_conv.c: 3x3 stride 1
pad 1, 64 -> 64 channels, 56 x 56, batch 8).  Activations are int8 uniform in [-127, 127],
weights int8 ~ round(N(0, 40)) clipped to +-127, per-channel fp32 scales and bias, PReLU
(or residual + fused BN with --residual).  Prints one JSON line: mean CUDA-event milliseconds
per launch of the tensor-core implicit GEMM, its int8 output's checksum and, with --winograd,
the exact-integer Winograd F(2,3) kernel on the same tensors (checked equal to 4 x the direct
int32 accumulators) with its time beside it.

    python -m fastface_b200.layer_bench --forward [--batch 1] [--iters 10]

runs the whole network instead (seeded synthetic model, seeded faces) through the public
embed / embed_batch call --iters times and prints the launch count, the device time per forward and
the wall-clock latency per call; at batch 1 the launch list is the small-batch one (layer chains,
one-launch FC), so this is also the command the profiler captures those kernels under.  With
--cos-sim N it ends with one N x N similarity matrix of the last embeddings.
"""
from __future__ import annotations

import argparse
import json
import zlib

import numpy as np

import fastface_b200 as ff

CASES = {
    # name: (Cin, Cout, H, k, stride)
    "conv112": (64, 64, 112, 3, 1),
    "conv56": (64, 64, 56, 3, 1),
    "conv56_128": (64, 128, 56, 3, 1),
    "conv28": (128, 128, 28, 3, 1),
    "conv14": (256, 256, 14, 3, 1),
    "conv7": (512, 512, 7, 3, 1),
    "down112": (64, 64, 112, 3, 2),
    "down56": (128, 128, 56, 3, 2),
    "down28": (256, 256, 28, 3, 2),
    "shortcut112": (64, 64, 112, 1, 2),
    "shortcut56": (64, 128, 56, 1, 2),
    "conv14_512": (256, 512, 14, 3, 1),
    "down14": (512, 512, 14, 3, 2),
}


def make_case(name: str, batch: int, residual: bool, seed: int = 0):
    cin, cout, h, k, stride = CASES[name]
    rng = np.random.default_rng(seed)
    pad = 1 if k == 3 else 0
    ho = (h + 2 * pad - k) // stride + 1
    c = dict(
        x=rng.integers(-127, 128, size=(batch, h, h, cin), dtype=np.int8),
        w=np.clip(np.rint(rng.standard_normal((cout, cin, k, k)) * 40.0), -127, 127).astype(np.int8),
        ws=np.exp(rng.uniform(np.log(1e-5), np.log(1e-3), cout)).astype(np.float32),
        bias=(rng.standard_normal(cout) * 0.1).astype(np.float32),
        inv=(np.float32(1) / (rng.uniform(0.005, 0.05, cout).astype(np.float32) + np.float32(1e-9))).astype(np.float32),
        stride=stride, pad=pad, slope=None, res=None, rs=None, bn2=None)
    if residual:
        c["res"] = rng.integers(-127, 128, size=(batch, ho, ho, cout), dtype=np.int8)
        c["rs"] = rng.uniform(0.002, 0.02, cout).astype(np.float32)
        c["bn2"] = ((np.float32(1) / c["inv"]).astype(np.float32), rng.uniform(0.5, 1.5, cout).astype(np.float32),
                    (rng.standard_normal(cout) * 0.1).astype(np.float32),
                    (np.float32(1) / (rng.uniform(0.005, 0.05, cout).astype(np.float32) + np.float32(1e-9))).astype(np.float32))
    else:
        c["slope"] = rng.uniform(0, 0.25, cout).astype(np.float32)
    return c


def run(name: str, batch: int, iters: int, residual: bool, winograd: bool, impl: str = "tc") -> dict:
    cin, cout, h, k, stride = CASES[name]
    c = make_case(name, batch, residual)
    r = ff.conv_once(c["x"], c["w"], c["ws"], c["bias"], c["inv"], stride=stride, pad=c["pad"], slope=c["slope"],
                     res=c["res"], res_scale=c["rs"], bn2=c["bn2"], impl=impl, bench_iters=iters)
    ms, out = r[0], r[1]
    ho = out.shape[1]
    macs = batch * ho * ho * cout * cin * k * k
    line = {"case": name, "batch": batch, "shape": {"Cin": cin, "Cout": cout, "H": h, "k": k, "stride": stride},
            "epilogue": "residual + fused BN" if residual else "PReLU", "impl": impl,
            "ms_per_launch": round(ms, 5), "tops": round(2.0 * macs / (ms * 1e-3) / 1e12, 1),
            "out_crc32": f"{zlib.crc32(out.tobytes()):08x}", "iters": iters}
    if winograd:
        if k != 3 or stride != 1:
            raise SystemExit("--winograd needs a 3x3 stride-1 case")
        acc, _ = ff.conv_once(c["x"], c["w"], c["ws"], c["bias"], c["inv"], stride=1, pad=1, slope=c["slope"],
                              res=c["res"], res_scale=c["rs"], impl=impl)
        y4, wms = ff.winograd_f23(c["x"], c["w"], iters=iters)
        line["winograd_f23"] = {"ms_per_launch": round(wms, 5), "equals_4x_direct": bool(np.array_equal(y4, acc * 4)),
                                "slower_than_implicit_gemm_by": round(wms / ms, 2),
                                "what": "exact-integer F(2,3), int16 transformed operands, CUDA cores; int32 output only "
                                        "(no epilogue), weight transform not timed"}
    return line


def run_forward(batch: int, iters: int, cos_sim: int) -> dict:
    import tempfile
    import time

    from fastface_b200 import synth

    root = tempfile.mkdtemp(prefix="ff_layer_bench_")
    ffw4 = synth.materialize(root, 0)
    faces = synth.faces(batch, seed=1)
    with ff.FastFace(ffw4, cwd=root, max_batch=batch) as e:
        out = None
        wall = []
        for _ in range(max(iters, 1)):
            t0 = time.perf_counter()
            out = e.embed(faces[0])[None, :] if batch == 1 else e.embed_batch(faces)
            wall.append((time.perf_counter() - t0) * 1e3)
        dev_ms = e.bench_resident(faces, max(iters, 1)) / max(iters, 1)
        line = {"forward": True, "batch": batch, "launches_per_forward": e.launches_per_forward,
                "device_ms_per_forward": round(dev_ms, 5), "call_ms_p50": round(sorted(wall)[len(wall) // 2], 5),
                "emb_crc32": f"{zlib.crc32(np.ascontiguousarray(out).tobytes()):08x}", "iters": iters}
        if cos_sim > 0:
            q = np.ascontiguousarray(np.resize(out, (cos_sim, out.shape[1])).astype(np.float32))
            m = e.cos_sim_matrix(q, q)
            line["cos_sim_matrix"] = {"n": cos_sim, "diag_min": float(np.min(np.diag(m)))}
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="conv56", choices=sorted(CASES))
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--residual", action="store_true", help="residual add + fused BN second output instead of PReLU")
    ap.add_argument("--winograd", action="store_true", help="also run the integer Winograd F(2,3) kernel on the same tensors")
    ap.add_argument("--impl", default="tc", choices=["tc", "simt"])
    ap.add_argument("--forward", action="store_true", help="time the whole network through embed / embed_batch instead of one layer")
    ap.add_argument("--cos-sim", type=int, default=0, help="with --forward: finish with an N x N similarity matrix")
    a = ap.parse_args()
    if a.forward:
        print(json.dumps(run_forward(a.batch, a.iters, a.cos_sim)), flush=True)
        return
    print(json.dumps(run(a.case, a.batch, a.iters, a.residual, a.winograd, a.impl)), flush=True)


if __name__ == "__main__":
    main()
