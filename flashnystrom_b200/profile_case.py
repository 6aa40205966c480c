"""One seeded forward + backward of the Nystrom attention path, for profilers.

    python -m flashnystrom_b200.profile_case [--heads 16] [--seq 65536] [--landmarks 64]
                                             [--iters 6] [--dtype fp16] [--repeat 2]

Runs `repeat` identical steps through the public API (the first warms up module loading and the
tensor-map cache), synchronises, checks the device status word and prints "ok".  Inputs are
N(0,1) draws from a fixed seed; nothing is timed here.
"""
import argparse

import torch

from . import _C, flash_nystrom_attention


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--seq", type=int, default=65536)
    ap.add_argument("--dim", type=int, default=64)
    ap.add_argument("--landmarks", type=int, default=64)
    ap.add_argument("--iters", type=int, default=6)
    ap.add_argument("--dtype", choices=("fp16", "bf16", "fp32"), default="fp16")
    ap.add_argument("--repeat", type=int, default=2)
    a = ap.parse_args(argv)
    dt = {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32}[a.dtype]
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev).manual_seed(1234)
    shape = (a.batch, a.heads, a.seq, a.dim)
    q, k, v, d_out = (torch.randn(shape, generator=gen, device=dev, dtype=torch.float32).to(dt)
                      for _ in range(4))
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
    for _ in range(a.repeat):
        q.grad = k.grad = v.grad = None
        out = flash_nystrom_attention(q, k, v, num_landmarks=a.landmarks, newton_iter=a.iters)
        out.backward(d_out)
    torch.cuda.synchronize(dev)
    _C.check_device_status()
    print("ok")


if __name__ == "__main__":
    main()
