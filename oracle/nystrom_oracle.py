"""CPU oracle for Nystrom attention forward + exact backward.  TEST INFRASTRUCTURE ONLY.

This module is a checker, not a product path: only the test-suite, the smoke entry and the
CPU-baseline leg of the benchmark may import it.  The shipped package never does.

It restates, stage by stage and with every intermediate exposed, the algorithm of the
reference project's pure-PyTorch implementation:

  * forward ............ flash_nystrom/reference.py:49-144 (scale :70-72, landmarks :77-97,
                         three softmaxes :100-102, ridge :122-137, products :142-144)
  * pseudoinverse ...... flash_nystrom/reference.py:15-46 (Newton-Schulz, FP32 in the reference)
  * depthwise residual . flash_nystrom/reference.py:147-182
  * hand backward ...... the algebra the reference kernels implement:
                         csrc/kernels/backward/kernel1_bwd.cuh:65-115 (softmax-1 side),
                         csrc/kernels/backward/kernel3_bwd.cuh:93-156 (softmax-3 side),
                         csrc/kernels/backward/kernel2_inv_bwd.cu:32-51,208-228,794-971
                         (unrolled Newton-Schulz, Z0 norms, ridge wrap, softmax-2 Jacobian),
                         csrc/kernels/backward/landmark_bwd.cuh:53-70 (segment scatter).

Parity status: PINNED.  tests/golden/make_golden.py imports the reference's reference.py in
the build container and stores its outputs (and autograd gradients) as fixtures;
tests/test_oracle.py checks this restatement against them, and checks the hand backward
against autograd through `forward` itself.

Everything here is written with torch CPU ops in the dtype of the inputs (float32 to mirror
the reference, float64 for a tighter truth).  All matrices are per (b, h) slice, batched over
the leading two dimensions.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------------------
# helpers
# --------------------------------------------------------------------------------------
def segment_bounds(N: int, m: int):
    """Floor-division segments; the last one absorbs the remainder (reference.py:77-97)."""
    seg = N // m
    starts = [l * seg for l in range(m)]
    ends = [(l + 1) * seg for l in range(m - 1)] + [N]
    return seg, starts, ends


def landmark_index(N: int, m: int) -> torch.Tensor:
    """Row n -> landmark l(n) = min(n // seg, m-1)."""
    seg = N // m
    return torch.clamp(torch.arange(N) // seg, max=m - 1)


def segment_lengths(N: int, m: int, dtype=torch.float32) -> torch.Tensor:
    seg = N // m
    lens = torch.full((m,), seg, dtype=dtype)
    lens[m - 1] = N - seg * (m - 1)
    return lens


def pool_landmarks(x_s: torch.Tensor, m: int) -> torch.Tensor:
    """Segment means of the already-scaled rows, (B,H,N,D) -> (B,H,m,D)."""
    B, H, N, D = x_s.shape
    seg = N // m
    head = x_s[:, :, : seg * (m - 1)].reshape(B, H, m - 1, seg, D).mean(dim=3)
    tail = x_s[:, :, seg * (m - 1):].mean(dim=2, keepdim=True)
    return torch.cat([head, tail], dim=2)


def norms_1_inf(A: torch.Tensor):
    """(||A||_1 = max column abs-sum, argmax col, ||A||_inf = max row abs-sum, argmax row)."""
    absA = A.abs()
    n1, jc = absA.sum(dim=-2).max(dim=-1)
    ninf, ir = absA.sum(dim=-1).max(dim=-1)
    return n1, jc, ninf, ir


def newton_schulz(A: torch.Tensor, n_iter: int):
    """Third-order Newton-Schulz pseudoinverse; returns every iterate Z_0..Z_J
    (reference.py:15-46)."""
    m = A.shape[-1]
    n1, _, ninf, _ = norms_1_inf(A)
    c = (n1 * ninf).clamp(min=1e-12)[..., None, None]
    Z = A.transpose(-2, -1) / c
    I = torch.eye(m, dtype=A.dtype).expand_as(A)
    iterates = [Z]
    for _ in range(n_iter):
        M = A @ Z
        U = 7.0 * I - M
        V = 15.0 * I - M @ U
        T = 13.0 * I - M @ V
        Z = 0.25 * Z @ T
        iterates.append(Z)
    return iterates


def ridge_lambda(K2: torch.Tensor, kappa_star: float) -> torch.Tensor:
    """Detached Tikhonov scale lambda = ||K2||_1 ||K2||_inf / kappa* (reference.py:125-134)."""
    Kd = K2.detach()
    n1, _, ninf, _ = norms_1_inf(Kd)
    return (n1 * ninf / kappa_star)[..., None, None]


# --------------------------------------------------------------------------------------
# forward
# --------------------------------------------------------------------------------------
def forward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, num_landmarks: int,
            newton_iter: int = 6, kappa_star: float = 0.0) -> Dict[str, torch.Tensor]:
    """Stage-wise forward.  Built from differentiable torch ops, so autograd through
    result["out"] is the reference gradient.  Returned intermediates use the layout of the
    CUDA library's saved tensors (landmarks already scaled by D^-1/4, everything FP32/FP64)."""
    B, H, N, D = q.shape
    m = int(num_landmarks)
    if N < m:
        raise ValueError(f"seq_len ({N}) must be >= num_landmarks ({m})")
    s = D ** (-0.25)
    q_s, k_s = q * s, k * s
    qt, kt = pool_landmarks(q_s, m), pool_landmarks(k_s, m)

    S1 = q_s @ kt.transpose(-2, -1)
    S2 = qt @ kt.transpose(-2, -1)
    S3 = qt @ k_s.transpose(-2, -1)
    P1, K2, P3 = F.softmax(S1, -1), F.softmax(S2, -1), F.softmax(S3, -1)
    lse1, lse2, lse3 = (torch.logsumexp(S1, -1), torch.logsumexp(S2, -1),
                        torch.logsumexp(S3, -1))

    if kappa_star > 0.0:
        lam = ridge_lambda(K2, kappa_star)
        A = K2.transpose(-2, -1) @ K2 + lam * torch.eye(m, dtype=K2.dtype)
        iterates = newton_schulz(A, newton_iter)
        k2inv = iterates[-1] @ K2.transpose(-2, -1)
    else:
        A = K2
        iterates = newton_schulz(A, newton_iter)
        k2inv = iterates[-1]

    bmat = P3 @ v
    step2 = k2inv @ bmat
    out = P1 @ step2
    return dict(out=out, qt=qt, kt=kt, P1=P1, K2=K2, P3=P3, lse1=lse1, lse2=lse2, lse3=lse3,
                A=A, iterates=torch.stack(iterates, dim=2), k2inv=k2inv, bmat=bmat,
                step2=step2)


def depthwise_conv_residual(v: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """out[b,h,n,:] = sum_t w[h,t] * v[b,h,n+t-ks//2,:] with zero padding
    (reference.py:147-182; flash_nystrom/flash_nystrom.py:19-55)."""
    B, H, N, D = v.shape
    ks = weight.shape[1]
    pad = ks // 2
    vp = F.pad(v, (0, 0, pad, pad))
    out = torch.zeros_like(v)
    for t in range(ks):
        out = out + weight[:, t].to(v.dtype).view(1, H, 1, 1) * vp[:, :, t:t + N]
    return out


def attention(q, k, v, num_landmarks=64, newton_iter=6, conv_weight=None,
              conv_kernel_size=0, kappa_star=0.0):
    """Same call shape as the reference's nystrom_attention_reference."""
    out = forward(q, k, v, num_landmarks, newton_iter, kappa_star)["out"]
    if conv_weight is not None and conv_kernel_size > 0:
        out = out + depthwise_conv_residual(v, conv_weight)
    return out


# --------------------------------------------------------------------------------------
# hand-written backward (no autograd) with every intermediate exposed
# --------------------------------------------------------------------------------------
def ns_backward(A: torch.Tensor, iterates: torch.Tensor, dZ: torch.Tensor):
    """Backward through Z_0 = A^T/(||A||_1 ||A||_inf) and J unrolled iterations.
    iterates: (..., J+1, m, m); dZ = dL/dZ_J.  Returns dL/dA."""
    m = A.shape[-1]
    J = iterates.shape[-3] - 1
    I = torch.eye(m, dtype=A.dtype).expand_as(A)
    At = A.transpose(-2, -1)
    dA = torch.zeros_like(A)
    for j in range(J - 1, -1, -1):
        Z = iterates[..., j, :, :]
        M = A @ Z
        U = 7.0 * I - M
        V = 15.0 * I - M @ U
        T = 13.0 * I - M @ V
        Mt = M.transpose(-2, -1)
        dT = 0.25 * Z.transpose(-2, -1) @ dZ
        dZ_outer = 0.25 * dZ @ T.transpose(-2, -1)
        dM = -dT @ V.transpose(-2, -1)
        dV = -Mt @ dT
        dM = dM - dV @ U.transpose(-2, -1)
        dM = dM + Mt @ dV                     # dM_U = -dU = +M^T dV
        dA = dA + dM @ Z.transpose(-2, -1)
        dZ = dZ_outer + At @ dM
    # Z_0 = A^T / c
    n1, jc, ninf, ir = norms_1_inf(A)
    c = (n1 * ninf).clamp(min=1e-12)
    S = (dZ * At).sum(dim=(-2, -1))
    dA = dA + dZ.transpose(-2, -1) / c[..., None, None]
    col_term = (-S * ninf / (c * c))
    row_term = (-S * n1 / (c * c))
    sgn = torch.sign(A)
    col_mask = F.one_hot(jc, m).to(A.dtype)[..., None, :]       # (...,1,m): column jc
    row_mask = F.one_hot(ir, m).to(A.dtype)[..., :, None]       # (...,m,1): row ir
    dA = dA + sgn * col_mask * col_term[..., None, None]
    dA = dA + sgn * row_mask * row_term[..., None, None]
    return dA, dZ


def backward(q, k, v, dO, num_landmarks: int, newton_iter: int = 6,
             kappa_star: float = 0.0, fwd: Optional[dict] = None) -> Dict[str, torch.Tensor]:
    """Exact gradient of sum(out * dO) w.r.t. q, k, v, computed stage by stage."""
    with torch.no_grad():
        B, H, N, D = q.shape
        m = int(num_landmarks)
        s = D ** (-0.25)
        f = fwd if fwd is not None else forward(q, k, v, m, newton_iter, kappa_star)
        q_s, k_s = q * s, k * s
        qt, kt, P1, K2, P3 = f["qt"], f["kt"], f["P1"], f["K2"], f["P3"]
        k2inv, bmat, step2 = f["k2inv"], f["bmat"], f["step2"]

        # softmax-1 side
        dstep2 = P1.transpose(-2, -1) @ dO
        dP1 = dO @ step2.transpose(-2, -1)
        D1 = (P1 * dP1).sum(-1, keepdim=True)
        dS1 = P1 * (dP1 - D1)
        dq_s = dS1 @ kt
        dkt = dS1.transpose(-2, -1) @ q_s

        # middle
        dO3 = k2inv.transpose(-2, -1) @ dstep2
        dk2inv = dstep2 @ bmat.transpose(-2, -1)
        D3 = (bmat * dO3).sum(-1, keepdim=True)

        # softmax-3 side
        dV = P3.transpose(-2, -1) @ dO3
        dP3 = dO3 @ v.transpose(-2, -1)
        dS3 = P3 * (dP3 - D3)
        dk_s = dS3.transpose(-2, -1) @ qt
        dqt = dS3 @ k_s

        # pseudoinverse
        if kappa_star > 0.0:
            ZJ = f["iterates"][:, :, -1]
            dK2_a = dk2inv.transpose(-2, -1) @ ZJ
            dZJ = dk2inv @ K2
            dA, dZ0 = ns_backward(f["A"], f["iterates"], dZJ)
            dK2 = dK2_a + K2 @ (dA + dA.transpose(-2, -1))
        else:
            dA, dZ0 = ns_backward(f["A"], f["iterates"], dk2inv)
            dK2 = dA
        dS2 = K2 * (dK2 - (dK2 * K2).sum(-1, keepdim=True))
        dqt_ns = dS2 @ kt
        dkt_ns = dS2.transpose(-2, -1) @ qt
        dqt_tot = dqt + dqt_ns
        dkt_tot = dkt + dkt_ns

        # landmark scatter
        idx = landmark_index(N, m)
        lens = segment_lengths(N, m, q.dtype)
        dq_s = dq_s + (dqt_tot / lens[:, None])[:, :, idx]
        dk_s = dk_s + (dkt_tot / lens[:, None])[:, :, idx]
        return dict(dq=s * dq_s, dk=s * dk_s, dv=dV, dstep2=dstep2, dkt_a=dkt, dO3=dO3,
                    dk2inv=dk2inv, D3=D3.squeeze(-1), dqt_b=dqt, dA=dA, dK2=dK2, dS2=dS2,
                    dqt_ns=dqt_ns, dqt_tot=dqt_tot, dkt_tot=dkt_tot, D1=D1.squeeze(-1))


def forward_backward_autograd(q, k, v, dO, num_landmarks, newton_iter=6, kappa_star=0.0,
                              conv_weight=None, conv_kernel_size=0):
    """Forward + autograd backward; the reference's way of getting gradients."""
    q = q.detach().clone().requires_grad_(True)
    k = k.detach().clone().requires_grad_(True)
    v = v.detach().clone().requires_grad_(True)
    out = attention(q, k, v, num_landmarks, newton_iter, conv_weight, conv_kernel_size,
                    kappa_star)
    out.backward(dO)
    return out.detach(), q.grad, k.grad, v.grad


# --------------------------------------------------------------------------------------
# error metrics used by every parity test
# --------------------------------------------------------------------------------------
def rel_max(a: torch.Tensor, b: torch.Tensor) -> float:
    """max|a-b| / max|b| : the 'max relative error' the tolerances are quoted in."""
    a, b = a.detach().double(), b.detach().double()
    return float((a - b).abs().max() / b.abs().max().clamp(min=1e-300))


def rel_fro(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.detach().double(), b.detach().double()
    return float((a - b).norm() / b.norm().clamp(min=1e-300))


def make_inputs(B, H, N, D, seed=0, dtype=torch.float32, qk_scale=1.0, dO_scale=1.0):
    """Seeded synthetic inputs, drawn in FP32 in the order q, k, v, dO, then cast."""
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn(B, H, N, D, generator=g) * qk_scale).to(dtype)
    k = (torch.randn(B, H, N, D, generator=g) * qk_scale).to(dtype)
    v = torch.randn(B, H, N, D, generator=g).to(dtype)
    dO = (torch.randn(B, H, N, D, generator=g) * dO_scale).to(dtype)
    return q, k, v, dO
