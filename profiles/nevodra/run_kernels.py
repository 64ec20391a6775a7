"""Profiling driver: the Nevodra kernels alone on a small case (a few hundred MB on the device), so that a profiler
capture ends by itself.  Usage:

    python profiles/nevodra/run_kernels.py [--tokens 4096] [--width 2048]

Runs, once each after a warm-up: the sum + two norms + input convolutions of a layer over a prompt (three launches)
and for one token, the polynomial activation, the whole-row query / key norm, and windowed attention with kept first
positions, soft cap and distance penalty over a prompt and for one token."""
import argparse
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from cold_compress_b200 import seq_ops  # noqa: E402
from cold_compress_b200.cache import get_cache_constructor  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--width", type=int, default=2048)
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    P, E, taps = a.tokens, a.width, 4
    gen = torch.Generator(device=dev).manual_seed(0)
    x, sa, sb = (torch.randn(P, E, device=dev, generator=gen) for _ in range(3))
    gains = [torch.ones(E, device=dev) for _ in range(2)]
    convs = [torch.full((E, taps), 0.25, device=dev) for _ in range(2)]
    outs = [torch.empty(P, E, device=dev, dtype=torch.bfloat16) for _ in range(2)]
    tail, rinv = torch.zeros(taps - 1, E, device=dev), torch.empty(P, device=dev)
    spec = [(gains[i], convs[i], outs[i]) for i in range(2)]
    spec1 = [(gains[i], convs[i], outs[i][:1]) for i in range(2)]
    F = 4 * E
    up = torch.randn(P, F, device=dev, generator=gen)
    coef = torch.tensor([1.0, 0.3, 0.1, 0.0], device=dev)
    act = torch.empty(P, F, device=dev, dtype=torch.bfloat16)
    H, G, D, W, K = 16, 4, 128, 1024, 64
    q = torch.randn(P, H, D, device=dev, generator=gen)
    k, v = (torch.randn(P, G, D, device=dev, generator=gen).to(torch.bfloat16) for _ in range(2))
    y = torch.empty(P, H, D, device=dev, dtype=torch.bfloat16)
    da, db = torch.full((H,), 0.5, device=dev), torch.full((H,), 0.5, device=dev)
    ctor, _ = get_cache_constructor("recent_global")
    with torch.device(dev):
        cache = ctor(1, G, D, torch.bfloat16, max_cache_length=W + K, global_tokens=K, max_seq_length=2 * P, cache_bits=None)
    qkv = torch.randn(P, (H + 2 * G) * D, device=dev, generator=gen)
    wq, wk = torch.ones(H * D, device=dev), torch.ones(G * D, device=dev)
    qn = torch.empty(P, H * D, device=dev)
    kn, vn = torch.empty(P, G * D, device=dev, dtype=torch.bfloat16), torch.empty(P, G * D, device=dev, dtype=torch.bfloat16)
    x1 = torch.empty(1, E, device=dev)
    for _ in range(2):
        seq_ops.par_norm(x, spec, 1e-5, a=sa, b=sb, tail=tail, taps=taps, rinv=rinv)
        seq_ops.par_norm(x[:1], spec1, 1e-5, a=sa[:1], b=sb[:1], tail=tail, taps=taps, x_out=x1)
        seq_ops.poly_norm(up, coef, act, 1e-5)
        seq_ops.qk_row_norm(qkv, 0, H * D, H * D, G * D, (H + G) * D, G * D, wq, wk, qn, kn, vn, 1e-5)
        cache.reset()
        cache.sequence_step(q, k, v, torch.zeros(1, dtype=torch.int32, device=dev), y, window=W, scale=D ** -0.5, softcap=30.0, dist=(da, db))
        cache.sequence_step(q[:1], k[:1], v[:1], torch.tensor([P], dtype=torch.int32, device=dev), y[:1], window=W, scale=D ** -0.5,
                            softcap=30.0, dist=(da, db))
    torch.cuda.synchronize()
    print("ok")


if __name__ == "__main__":
    main()
