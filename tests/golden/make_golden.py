"""Generate golden vectors from the reference project's own pure-PyTorch implementation.

Run in a container where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference/checkout

It imports flash_nystrom/reference.py from that checkout (the CUDA extension is not needed),
runs forward + autograd backward on seeded inputs and writes tests/golden/reference_vectors.npz.
Inputs are not stored: they are regenerated from the seed by oracle.nystrom_oracle.make_inputs
and pinned by a float64 checksum.  Large cases store every `stride`-th row plus checksums.
"""
import os
import sys
import warnings

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))

# name: (B, H, N, D, m, J, kappa_star, seed, input dtype, qk_scale, row stride, conv kernel size)
CASES = {
    "cfg1_cpu":      (1, 4, 1024, 64, 32, 6, 0.0, 0, "float32", 64 ** -0.25, 16, 0),
    "small_full":    (1, 2, 128, 64, 16, 6, 0.0, 1, "float32", 1.0, 1, 0),
    "ragged_m7":     (1, 2, 300, 64, 7, 6, 0.0, 2, "float32", 1.0, 2, 0),
    "n_equals_m":    (1, 1, 64, 64, 64, 6, 0.0, 3, "float32", 1.0, 1, 0),
    "single_lmk":    (1, 1, 100, 64, 1, 6, 0.0, 4, "float32", 1.0, 1, 0),
    "ridge_k1e3_j3": (1, 2, 130, 64, 8, 3, 1e3, 5, "float32", 1.0, 1, 0),
    "ridge_k5_m64":  (1, 1, 256, 64, 64, 8, 5.0, 6, "float32", 1.0, 1, 0),
    "fp16_valued":   (1, 2, 512, 64, 64, 6, 0.0, 7, "float16", 1.0, 8, 0),
    "d128_m32":      (1, 1, 256, 128, 32, 6, 0.0, 8, "float16", 1.0, 4, 0),
    "m128_ridge":    (1, 1, 512, 128, 128, 8, 5.0, 9, "float16", 1.0, 8, 0),
    "conv_k3":       (2, 2, 96, 64, 8, 6, 0.0, 10, "float32", 1.0, 1, 3),
}


def main(ref_root):
    sys.dont_write_bytecode = True
    sys.path.insert(0, ref_root)
    sys.path.insert(0, ROOT)
    warnings.filterwarnings("ignore")
    from flash_nystrom.reference import nystrom_attention_reference
    from oracle.nystrom_oracle import make_inputs

    torch.set_num_threads(1)  # one summation order, independent of the machine
    blob = {}
    for name, (B, H, N, D, m, J, kap, seed, dt, qks, stride, ks) in CASES.items():
        q, k, v, dO = make_inputs(B, H, N, D, seed=seed, dtype=getattr(torch, dt), qk_scale=qks)
        q, k, v, dO = (t.float() for t in (q, k, v, dO))
        w = None
        if ks:
            w = torch.randn(H, ks, generator=torch.Generator().manual_seed(seed + 100)) * 0.5
            blob[f"{name}/conv_weight"] = w.numpy()
        qq, kk, vv = (t.clone().requires_grad_(True) for t in (q, k, v))
        out = nystrom_attention_reference(qq, kk, vv, m, J, w, ks, kappa_star=kap)
        out.backward(dO)
        blob[f"{name}/in_checksum"] = np.array(
            [float(t.double().sum()) for t in (q, k, v, dO)]
            + [float(t.double().abs().sum()) for t in (q, k, v, dO)])
        for key, t in (("out", out.detach()), ("dq", qq.grad), ("dk", kk.grad), ("dv", vv.grad)):
            blob[f"{name}/{key}"] = t[:, :, ::stride].contiguous().numpy()
            blob[f"{name}/{key}_checksum"] = np.array(
                [float(t.double().sum()), float(t.double().abs().sum())])
    path = os.path.join(HERE, "reference_vectors.npz")
    np.savez_compressed(path, **blob)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: python make_golden.py <path to a checkout of the reference project>")
    main(sys.argv[1])
