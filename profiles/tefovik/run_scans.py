"""Profiling driver: the two matrix-state scans alone on random inputs of a bench.py --design shape.  Usage:

    python profiles/tefovik/run_scans.py [--size 1b] [--tokens 2048] [--which delta|ssd|both] [--repeat 3]
"""
import argparse
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

import bench  # noqa: E402
from cold_compress_b200 import seq_ops  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--size", default="1b", choices=sorted(bench.DETATAR_SIZES))
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--which", default="both", choices=["delta", "ssd", "both"])
    ap.add_argument("--repeat", type=int, default=3)
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    cfg = bench._tefovik_config(bench.DESIGN_SIZES[a.size])
    P = a.tokens
    gen = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *s: torch.randn(*s, device=dev, generator=gen)
    if a.which in ("ssd", "both"):
        m = cfg["layers"][0]["mixer"]
        H, V, N = m["heads"], m["vdim"], m["state"]
        x, B, C, dt = rnd(P, H * V) * 0.1, rnd(P, N) * 0.1, rnd(P, N) * 0.1, rnd(P, H)
        z, o = torch.zeros(H, device=dev), torch.ones(H, device=dev)
        state, y = torch.zeros(H, N, V, device=dev), torch.empty(P, H * V, device=dev)
        for _ in range(a.repeat):
            seq_ops.ssd_scan(x, B, C, dt, z, z, o, state, y, H, 1, N, V)
    if a.which in ("delta", "both"):
        r = cfg["layers"][1]["mixer"]["right"]
        H, D, V = r["heads"], r["dim"], r["vdim"]
        q, k, v, ar, b = rnd(P, H * D), rnd(P, H * D), rnd(P, H * V) * 0.1, rnd(P, H * D), rnd(P, H)
        state, o = torch.zeros(H, D, V, device=dev), torch.empty(P, H * V, device=dev)
        for _ in range(a.repeat):
            seq_ops.delta_scan(q, k, v, b, ar, torch.zeros(H * D, device=dev), torch.zeros(H, device=dev), state, o, H, H, D, V, D ** -0.5)
    torch.cuda.synchronize()
    print("ok")


if __name__ == "__main__":
    main()
