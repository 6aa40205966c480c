"""torch.library registration of the forward and backward as custom operators, so that
torch.compile / torch.export trace through `flash_nystrom_attention` without a graph break (the
reference lists this as future work, README.md:387; its autograd.Function behind pybind breaks the
graph).

    torch.ops.flashnystrom_b200.nystrom_fwd(q, k, v, num_landmarks, newton_iter, kappa_star)
        -> (out, q_landmarks, k_landmarks, k2_inv, step2, lse1, lse2, lse3, ns_iterates, k2, bmat)
    torch.ops.flashnystrom_b200.nystrom_bwd(d_out, q, k, v, <the ten saved tensors>, ...)
        -> (dq, dk, dv)

Both have fake (meta) implementations, and nystrom_fwd has its autograd formula registered, so the
operators work under FakeTensorMode, AOT autograd and opcheck.  The eager path of the package keeps
using the plain autograd.Function (less dispatcher overhead per call); `flash_nystrom_attention`
switches to the operators while a compiler is tracing."""
from typing import Tuple

import torch

from . import _C

_LIB = "flashnystrom_b200"


@torch.library.custom_op(f"{_LIB}::nystrom_fwd", mutates_args=(), device_types="cuda")
def nystrom_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, num_landmarks: int, newton_iter: int,
                kappa_star: float) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor,
                                            torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor,
                                            torch.Tensor]:
    r = _C.forward(q.contiguous(), k.contiguous(), v.contiguous(), num_landmarks, newton_iter, kappa_star, False, True)
    # r = [out, q, k, qt, kt, k2inv, step2, lse1, lse2, lse3, iterates, k2, bmat]; q and k are the
    # caller's own tensors and an operator must not return its inputs
    return (r[0], r[3], r[4], r[5], r[6], r[7], r[8], r[9], r[10], r[11], r[12])


@nystrom_fwd.register_fake
def _(q, k, v, num_landmarks, newton_iter, kappa_star):
    B, H, N, D = q.shape
    m, J = num_landmarks, newton_iter
    f32 = dict(dtype=torch.float32, device=q.device)
    return (torch.empty_like(q, memory_format=torch.contiguous_format),
            torch.empty(B, H, m, D, **f32), torch.empty(B, H, m, D, **f32), torch.empty(B, H, m, m, **f32),
            torch.empty(B, H, m, D, **f32), torch.empty(B, H, N, **f32), torch.empty(B, H, m, **f32),
            torch.empty(B, H, m, **f32), torch.empty(B, H, J + 1, m, m, **f32), torch.empty(B, H, m, m, **f32),
            torch.empty(B, H, m, D, **f32))


@torch.library.custom_op(f"{_LIB}::nystrom_bwd", mutates_args=(), device_types="cuda")
def nystrom_bwd(d_out: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor,
                q_landmarks: torch.Tensor, k_landmarks: torch.Tensor, k2_inv: torch.Tensor, step2: torch.Tensor,
                lse1: torch.Tensor, lse2: torch.Tensor, lse3: torch.Tensor, ns_iterates: torch.Tensor,
                k2: torch.Tensor, bmat: torch.Tensor, num_landmarks: int, newton_iter: int,
                kappa_star: float) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    dq, dk, dv = _C.backward(d_out.contiguous(), q.contiguous(), k.contiguous(), q_landmarks, k_landmarks, k2_inv, step2,
                             lse1, lse2, lse3, ns_iterates, k2, bmat, v.contiguous(), out, num_landmarks, newton_iter,
                             True, kappa_star)
    return dq, dk, dv


@nystrom_bwd.register_fake
def _(d_out, q, k, v, out, q_landmarks, k_landmarks, k2_inv, step2, lse1, lse2, lse3, ns_iterates, k2, bmat,
      num_landmarks, newton_iter, kappa_star):
    c = torch.contiguous_format
    return (torch.empty_like(q, memory_format=c), torch.empty_like(k, memory_format=c),
            torch.empty_like(v, memory_format=c))


def _setup_context(ctx, inputs, output):
    q, k, v, m, J, kappa = inputs
    ctx.save_for_backward(q, k, v, *output)
    ctx.m, ctx.J, ctx.kappa = m, J, kappa


def _backward(ctx, d_out, *unused_saved_grads):
    q, k, v, out, qt, kt, k2inv, step2, lse1, lse2, lse3, iters, k2, bmat = ctx.saved_tensors
    dq, dk, dv = nystrom_bwd(d_out, q, k, v, out, qt, kt, k2inv, step2, lse1, lse2, lse3, iters, k2, bmat,
                             ctx.m, ctx.J, ctx.kappa)
    return dq, dk, dv, None, None, None


nystrom_fwd.register_autograd(_backward, setup_context=_setup_context)


def attention_via_ops(q, k, v, num_landmarks, newton_iter, kappa_star):
    """The attention output through the registered operators (differentiable, traceable)."""
    return nystrom_fwd(q, k, v, int(num_landmarks), int(newton_iter), float(kappa_star))[0]
