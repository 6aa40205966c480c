"""Helpers shared by the parity tests: run the CUDA path through the public API / C ABI and
the CPU oracle on identical seeded inputs."""
import torch

from oracle import nystrom_oracle as O


def run_cuda(q, k, v, dO, m, J, kappa=0.0, device="cuda"):
    """Forward + backward through flashnystrom_b200._C (the ctypes face of the C ABI)."""
    from flashnystrom_b200 import _C
    qd, kd, vd, gd = (t.to(device).contiguous() for t in (q, k, v, dO))
    res = _C.forward(qd, kd, vd, m, J, kappa, False, True)
    grads = _C.backward(gd, *res[1:13], vd, res[0], m, J, True, kappa)
    names = ["out", "q_s", "k_s", "qt", "kt", "k2inv", "step2", "lse1", "lse2", "lse3",
             "iterates", "K2", "bmat"]
    d = {n: t for n, t in zip(names, res)}
    d.update(dq=grads[0], dk=grads[1], dv=grads[2])
    torch.cuda.synchronize()
    _C.check_device_status()   # a bounded device-side wait that expired fails the test
    return d


def run_oracle(q, k, v, dO, m, J, kappa=0.0, dtype=torch.float64):
    """Oracle on the same (already dtype-rounded) values, upcast to `dtype`."""
    q, k, v, dO = (t.to(dtype) for t in (q, k, v, dO))
    f = O.forward(q, k, v, m, J, kappa)
    b = O.backward(q, k, v, dO, m, J, kappa, fwd=f)
    f.update(b)
    return f


def errs(cu, ref, keys):
    return {key: O.rel_max(cu[key].detach().cpu(), ref[key]) for key in keys}
