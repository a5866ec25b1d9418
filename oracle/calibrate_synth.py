"""Produce fastface_b200/data/synth_seed<seed>.opsc2 -- the committed activation-scale
table of the synthetic benchmark model (TEST INFRASTRUCTURE, run once, by hand).

Sequential calibration as the reference's export scripts do it
(export_op_scales_v2.py:121-164, calibrate_percentile_int8.py:105-118): run the
seeded network on N seeded faces and, at every requantisation point, set the
per-channel output scale to p99.9(|value|)/127 before quantising and moving on.

    python oracle/calibrate_synth.py [--seed 0] [--faces 8]
"""
import argparse
import os
import sys
import tempfile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from fastface_b200 import synth  # noqa: E402
from oracle import ffo           # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--faces", type=int, default=8)
    ap.add_argument("--percentile", type=float, default=99.9)
    a = ap.parse_args()
    with tempfile.TemporaryDirectory() as td:
        ffw4 = os.path.join(td, "m.bin")
        synth.write_ffw4(ffw4, a.seed)
        out2 = synth.scale_table_path(a.seed)
        os.makedirs(os.path.dirname(out2), exist_ok=True)
        ffo.calibrate(ffw4, synth.faces(a.faces, seed=a.seed + 7777), a.percentile,
                      os.path.join(td, "opsc.bin"), out2)
    print("wrote", out2, os.path.getsize(out2), "bytes")


if __name__ == "__main__":
    main()
