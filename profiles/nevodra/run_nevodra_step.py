"""Profiling driver: one prompt and a few single-token steps of a random-init Nevodra of a bench.py --design shape,
eager (no graph), so that a profiler sees every launch.  Usage:

    python profiles/nevodra/run_nevodra_step.py [--size 1b] [--prompt 1024] [--tokens 3]

The last single-token step is bracketed by two tiny `torch.zeros` fills that show up in a launch list."""
import argparse
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

import bench  # noqa: E402
from cold_compress_b200 import generation_utils as gu  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--size", default="1b", choices=sorted(bench.DETATAR_SIZES))
    ap.add_argument("--prompt", type=int, default=1024)
    ap.add_argument("--tokens", type=int, default=3)
    a = ap.parse_args()
    device = torch.device("cuda", 0)
    sz = dict(bench.DESIGN_SIZES[a.size], prompt=a.prompt)
    model = bench._nevodra_model(sz, bench.DETATAR_SIZES[a.size], device, torch.bfloat16)
    gu.setup_caches(model, None, device, a.prompt + 64, {})
    prompt = torch.randint(0, sz["vocab"], (a.prompt,), dtype=torch.int32, device=device)
    with torch.no_grad():
        tok, _ = gu.prefill(model, prompt.view(1, -1), torch.arange(a.prompt, device=device))
        pos = torch.tensor([a.prompt], dtype=torch.int32, device=device)
        for i in range(a.tokens):
            if i == a.tokens - 1:
                torch.zeros(7, device=device)      # marker before the last step
            tok, _ = gu.decode_one_token(model, tok.view(1, 1), pos)
            pos += 1
        torch.zeros(7, device=device)              # marker after it
    torch.cuda.synchronize()
    print("ok", int(tok))


if __name__ == "__main__":
    main()
