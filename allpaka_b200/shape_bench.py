"""Per-shape bandwidth of the dequant-matvec kernels at the benchmark shapes.

    python -m allpaka_b200.shape_bench [--layers 16] [--reps 3]

For each weight type (Q8_0, Q4_K) and batch (m = 1, 6, 8) a synthetic stack of
`--layers` Qwen3-32B-shaped layers is made resident (distinct device memory per
layer, so every launch streams HBM-cold weights) and the five matvec shapes are
timed with CUDA events, launched back to back over the layers.  Prints one JSON
line per (type, m): per shape the microseconds per launch, algorithmic GB/s and
the fraction of the measured HBM peak.  The shapes cover the stand-alone
configurations of the benchmark description: Q|K|V 10240x5120 with RMSNorm
prologue and RoPE epilogue; gate/up 2x25600x5120 with SwiGLU epilogue + down
5120x25600 at m = 6; Q4_K gate/up.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def main():
    import bench
    from allpaka_b200 import gpu as G

    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=16)
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--types", default="8,12")
    ap.add_argument("--ms", default="1,6,8")
    args = ap.parse_args()
    peak, kind = bench.measured_peak()
    for ty in [int(t) for t in args.types.split(",")]:
        for m in [int(v) for v in args.ms.split(",")]:
            g = G.Gpu(0)
            req, _, _, _, keep = bench.build_model(g, args.layers, set(), 0, ty=ty, m=m, head=False)
            g.decode_replay(req, 1)
            g.synth_release()
            prof = g.decode_profile(req, reps=args.reps)
            out = {"ty": "Q8_0" if ty == 8 else "Q4_K", "m": m, "layers": args.layers, "peak_gbs": peak, "peak_kind": kind}
            for k, v in prof.items():
                if k == "lm_head":
                    continue
                gbs = v["bytes"] / (v["ms"] * 1e-3) / 1e9
                out[k] = {"us": round(v["ms"] * 1e3, 2), "mb": round(v["bytes"] / 1e6, 2), "gbs": round(gbs, 1),
                          "frac": round(gbs / peak, 3)}
            ffn_b = prof["gate_up"]["bytes"] + prof["down"]["bytes"]
            ffn_t = prof["gate_up"]["ms"] + prof["down"]["ms"]
            out["ffn"] = {"us": round(ffn_t * 1e3, 2), "gbs": round(ffn_b / (ffn_t * 1e-3) / 1e9, 1),
                          "frac": round(ffn_b / (ffn_t * 1e-3) / 1e9 / peak, 3)}
            print(json.dumps(out), flush=True)
            g.close()
            del keep


if __name__ == "__main__":
    main()
