"""Isolation tests of the Newton-Schulz pseudoinverse kernels through the C-ABI debug hooks,
against the oracle's restatement of the same algebra (the role of the reference's
tests/test_ns_bwd_kernel.py and tests/test_ns_bwd_graph.py)."""
import pytest
import torch

from oracle import nystrom_oracle as O

pytestmark = pytest.mark.gpu


def _softmax_matrix(BH, m, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.softmax(torch.randn(BH, m, m, generator=g) * 1.5, dim=-1)


def _oracle_pinv(k2, J, kappa):
    k2 = k2.double().unsqueeze(0)
    if kappa > 0:
        lam = O.ridge_lambda(k2, kappa)
        A = k2.transpose(-2, -1) @ k2 + lam * torch.eye(k2.shape[-1], dtype=k2.dtype)
        its = O.newton_schulz(A, J)
        inv = its[-1] @ k2.transpose(-2, -1)
    else:
        A = k2
        its = O.newton_schulz(A, J)
        inv = its[-1]
    return A, torch.stack(its, dim=2), inv


@pytest.mark.parametrize("m", [1, 7, 16, 33, 64, 100, 128])
@pytest.mark.parametrize("J,kappa", [(6, 0.0), (3, 1e3), (8, 5.0), (12, 0.0)])
def test_pinv_forward_and_backward(cuda_device, m, J, kappa):
    from flashnystrom_b200 import _C
    BH = 3
    k2 = _softmax_matrix(BH, m, seed=m + J)
    G = torch.randn(BH, m, m, generator=torch.Generator().manual_seed(99))
    iters, inv = _C.debug_pinv_forward(k2.cuda(), J, kappa)
    A, ref_its, ref_inv = _oracle_pinv(k2, J, kappa)
    assert O.rel_max(inv.cpu(), ref_inv[0]) < 2e-4, "k2_inv"
    assert O.rel_max(iters.cpu(), ref_its[0]) < 2e-4, "iterates"

    # backward: hand algebra of the oracle in float64 on the iterates the kernel itself saved
    dk2 = _C.debug_pinv_backward(k2.cuda(), iters, G.cuda(), kappa).cpu()
    its64 = iters.cpu().double().unsqueeze(0)
    k64, G64 = k2.double().unsqueeze(0), G.double().unsqueeze(0)
    if kappa > 0:
        ZJ = its64[:, :, -1]
        dA, _ = O.ns_backward(A, its64, G64 @ k64)
        ref = G64.transpose(-2, -1) @ ZJ + k64 @ (dA + dA.transpose(-2, -1))
    else:
        ref, _ = O.ns_backward(A, its64, G64)
    if kappa == 0:
        # K2 is row-stochastic, so its row sums tie at 1 and the argmax row of ||K2||_inf is
        # decided by round-off.  The term it steers is constant along a row and vanishes under
        # the softmax Jacobian that always follows, so compare after that projection.
        def jac(d):
            return k64[0] * (d - (d * k64[0]).sum(-1, keepdim=True))
        assert O.rel_max(jac(dk2.double()), jac(ref[0])) < 5e-4, "d_k2 (after softmax Jacobian)"
    else:
        assert O.rel_max(dk2, ref[0]) < 5e-4, "d_k2"


def test_pinv_same_call_twice_is_bit_identical(cuda_device):
    from flashnystrom_b200 import _C
    k2 = _softmax_matrix(4, 64, seed=1).cuda()
    a = _C.debug_pinv_forward(k2, 6, 5.0)
    b = _C.debug_pinv_forward(k2, 6, 5.0)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    G = torch.randn(4, 64, 64, device="cuda")
    assert torch.equal(_C.debug_pinv_backward(k2, a[0], G, 5.0), _C.debug_pinv_backward(k2, a[0], G, 5.0))
