"""The depthwise convolution residual as the library's own kernels (forward, transposed operator
for dV, weight gradient) against the oracle's restatement of the reference's F.conv1d formulation
(flash_nystrom/flash_nystrom.py:19-55), through the C ABI."""
import pytest
import torch

from oracle import nystrom_oracle as O

pytestmark = pytest.mark.gpu

TOL = {torch.float32: (2e-6, 2e-5), torch.float16: (1.5e-3, 3e-3), torch.bfloat16: (1.2e-2, 2.5e-2)}


def _inputs(B, H, N, D, ks, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    v = torch.randn(B, H, N, D, generator=g).to(dtype)
    base = torch.randn(B, H, N, D, generator=g).to(dtype)
    dout = torch.randn(B, H, N, D, generator=g).to(dtype)
    w = torch.randn(H, ks, generator=g) * 0.3
    return v, base, dout, w


def _split(t):
    """The same values as the head-split view of a contiguous (B, N, H*D) tensor."""
    return t.transpose(1, 2).contiguous().transpose(1, 2)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("B,H,N,D,ks", [(1, 2, 100, 64, 3), (2, 3, 257, 64, 5), (1, 2, 4096, 64, 33),
                                        (1, 1, 63, 16, 1), (2, 2, 130, 32, 7), (1, 4, 1000, 128, 33),
                                        (1, 1, 20, 64, 127)])
@pytest.mark.parametrize("split", [False, True])
def test_conv_residual_forward_backward(cuda_device, dtype, B, H, N, D, ks, split):
    from flashnystrom_b200 import _C
    v, base, dout, w = _inputs(B, H, N, D, ks, dtype, seed=N + ks)
    w32 = w.to(dtype).float()                      # the weights take part rounded to the tensors' dtype
    lay = _split if split else (lambda t: t)
    vd, bd, gd = lay(v.cuda()), lay(base.cuda()), lay(dout.cuda())
    out = _C.conv_residual(vd, w32.cuda(), base=bd)
    assert _C.layout_of(out) == _C.layout_of(vd)
    dv = _C.conv_residual(gd, w32.cuda(), transposed=True)
    dw = _C.conv_residual_dweight(vd, gd, ks)
    assert torch.equal(dw, _C.conv_residual_dweight(vd, gd, ks)), "the weight gradient is summed in a fixed order"
    # oracle in float64 on the identical rounded inputs
    v64, w64 = v.double().requires_grad_(True), w32.double().requires_grad_(True)
    ref = base.double() + O.depthwise_conv_residual(v64, w64)
    ref.backward(dout.double())
    t_out, t_grad = TOL[dtype]
    assert O.rel_max(out.cpu(), ref.detach()) <= t_out
    assert O.rel_max(dv.cpu(), v64.grad) <= t_grad
    assert O.rel_max(dw.cpu(), w64.grad) <= t_grad
    # without a base the result is the convolution alone
    alone = _C.conv_residual(vd, w32.cuda())
    assert O.rel_max(alone.cpu(), O.depthwise_conv_residual(v.double(), w32.double())) <= t_out


def test_conv_residual_through_the_public_entry(cuda_device):
    """flash_nystrom_attention with a conv kernel: the residual and all four gradients (q, k, v, w)
    against the oracle; fp16, ragged N, kernel longer than a tile's halo of the usual sizes."""
    from flashnystrom_b200 import flash_nystrom_attention
    q, k, v, dO = O.make_inputs(2, 4, 1000, 64, seed=4, dtype=torch.float16)
    w = torch.randn(4, 33, generator=torch.Generator().manual_seed(5)) * 0.1
    qd, kd, vd, wd = (t.cuda().requires_grad_(True) for t in (q, k, v, w))
    out = flash_nystrom_attention(qd, kd, vd, 32, 6, conv_weight=wd, conv_kernel_size=33)
    out.backward(dO.cuda())
    w_r = w.half().double().requires_grad_(True)
    q2, k2, v2 = (t.double().requires_grad_(True) for t in (q, k, v))
    ref = O.attention(q2, k2, v2, 32, 6, w_r, 33)
    ref.backward(dO.double())
    assert O.rel_max(out.detach().cpu(), ref.detach()) <= 2e-3
    assert O.rel_max(qd.grad.cpu(), q2.grad) <= 1e-2
    assert O.rel_max(kd.grad.cpu(), k2.grad) <= 1e-2
    assert O.rel_max(vd.grad.cpu(), v2.grad) <= 1e-2
    assert wd.grad.dtype == w.dtype and O.rel_max(wd.grad.cpu(), w_r.grad) <= 1e-2


def test_conv_residual_rejects_bad_arguments(cuda_device):
    from flashnystrom_b200 import _C, flash_nystrom_attention
    v = torch.randn(1, 2, 64, 64, device="cuda", dtype=torch.float16)
    with pytest.raises(RuntimeError, match="must be odd"):
        _C.conv_residual(v, torch.zeros(2, 4, device="cuda"))
    with pytest.raises(RuntimeError, match=r"\(heads, kernel_size\)"):
        _C.conv_residual(v, torch.zeros(3, 3, device="cuda"))
    with pytest.raises(RuntimeError, match="no CPU path"):
        _C.conv_residual(v.cpu(), torch.zeros(2, 3))
    with pytest.raises(ValueError, match="odd kernel_size"):
        flash_nystrom_attention(v, v, v, 16, 6, conv_weight=torch.zeros(2, 4, device="cuda"), conv_kernel_size=4)
