"""Public Python API: the reference's functional entry point, autograd Function and module
(flash_nystrom/flash_nystrom.py:19-292) on top of the sm_100a C-ABI library."""
import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _C
from .nystrom_config import NystromConfig

# The reference sets HAS_CUDA when its extension imports (flash_nystrom/__init__.py:38-46).  Here
# the library is the only implementation: the flag says whether it can run on this machine.
HAS_CUDA = bool(torch.cuda.is_available())


def _depthwise_conv_residual(v, weight):
    """Depthwise 1-D conv of V along the sequence, one kernel per head shared by its D
    channels, zero padding ks//2 (flash_nystrom/flash_nystrom.py:19-55), through F.conv1d as in the
    reference.  Only used while a compiler is tracing (it differentiates and traces this form);
    otherwise _ConvResidualFunction runs the library's kernel."""
    B, H, N, D = v.shape
    ks = weight.shape[1]
    if weight.dtype != v.dtype:
        weight = weight.to(v.dtype)
    v_in = v.permute(0, 1, 3, 2).contiguous().view(B, H * D, N)
    w = weight.unsqueeze(1).expand(H, D, ks).contiguous().view(H * D, 1, ks)
    out = F.conv1d(v_in, w, padding=ks // 2, groups=H * D)
    return out.view(B, H, D, N).permute(0, 1, 3, 2).contiguous()


class _ConvResidualFunction(torch.autograd.Function):
    """out + depthwise_conv(v, weight) as one streaming kernel in the tensors' own layout, with its
    backward (the reference's `out + _depthwise_conv_residual(v, conv_weight)`,
    flash_nystrom/flash_nystrom.py:19-55, makes two transposing copies around a grouped F.conv1d and
    leaves the backward to autograd).  The weights take part rounded to the tensors' dtype, as the
    reference's `weight.to(v.dtype)` has it."""

    @staticmethod
    def forward(ctx, out, v, weight):
        w32 = weight.detach().to(v.dtype).float()
        ctx.save_for_backward(v, w32)
        ctx.weight_dtype = weight.dtype
        return _C.conv_residual(v, w32, base=out)

    @staticmethod
    def backward(ctx, grad):
        v, w32 = ctx.saved_tensors
        d_v = _C.conv_residual(grad, w32, transposed=True) if ctx.needs_input_grad[1] else None
        d_w = None
        if ctx.needs_input_grad[2]:
            d_w = _C.conv_residual_dweight(v, grad, w32.shape[1]).to(ctx.weight_dtype)
        return grad, d_v, d_w


class FlashNystromFunction(torch.autograd.Function):
    """Autograd bridge (flash_nystrom/flash_nystrom.py:58-134): same eight positional
    arguments, same eight gradient slots."""

    @staticmethod
    def forward(ctx, q, k, v, num_landmarks, newton_iter, fast_dk2inv, kappa_star, use_tc_pinv):
        need_bwd = bool(q.requires_grad or k.requires_grad or v.requires_grad)
        results = _C.forward(q, k, v, num_landmarks, newton_iter, kappa_star, use_tc_pinv, need_bwd)
        output = results[0]
        saved = list(results[1:]) + [v, output]
        ctx.save_for_backward(*saved)
        ctx.num_landmarks = num_landmarks
        ctx.newton_iter = newton_iter
        ctx.fast_dk2inv = fast_dk2inv
        ctx.kappa_star = kappa_star
        return output

    @staticmethod
    def backward(ctx, grad_output):
        s = ctx.saved_tensors
        # (the shim brings grad_output to the layout of q: no copy when both are contiguous or both
        # are head-split views of (B, N, H*D) tensors, which is what the module below produces)
        dQ, dK, dV = _C.backward(grad_output, *s[0:12], s[12], s[13],
                                 ctx.num_landmarks, ctx.newton_iter, ctx.fast_dk2inv,
                                 ctx.kappa_star)
        return dQ, dK, dV, None, None, None, None, None


def flash_nystrom_attention(q, k, v, num_landmarks=64, newton_iter=6, conv_weight=None,
                            conv_kernel_size=0, fast_dk2inv=True, kappa_star=0.0,
                            use_tc_pinv=False):
    """Nystrom attention  softmax(Q Kt^T) pinv(softmax(Qt Kt^T)) softmax(Qt K^T) V  with
    segment-mean landmarks, forward and exact backward on the GPU
    (flash_nystrom/flash_nystrom.py:180-249).

    q, k, v: (B, H, N, D) CUDA tensors of one dtype (fp16 / bf16 / fp32), N >= num_landmarks,
    num_landmarks <= 128.  Every landmark count runs natively; there is no reference dispatch
    and no CPU path: CPU tensors raise."""
    if not (isinstance(q, torch.Tensor) and q.is_cuda):
        raise RuntimeError("flash_nystrom_attention: inputs must be CUDA tensors "
                           "(flashnystrom_b200 has no CPU path)")
    if torch.compiler.is_compiling():
        # registered custom operators (fake implementations + autograd formula): no graph break
        from . import _ops
        out = _ops.attention_via_ops(q, k, v, num_landmarks, newton_iter, kappa_star)
    else:
        out = FlashNystromFunction.apply(q, k, v, num_landmarks, newton_iter, fast_dk2inv,
                                         kappa_star, use_tc_pinv)
    if conv_weight is not None and conv_kernel_size > 0:
        if torch.compiler.is_compiling():
            out = out + _depthwise_conv_residual(v, conv_weight)      # traceable form
        else:
            if conv_weight.dim() != 2 or conv_weight.shape[1] % 2 == 0:
                raise ValueError("conv_weight must be (heads, kernel_size) with an odd kernel_size")
            out = _ConvResidualFunction.apply(out, v, conv_weight)
    return out


class FlashNystromAttention(nn.Module):
    """Multi-head self-attention block (flash_nystrom/flash_nystrom.py:252-292): bias-free
    q/k/v/out projections around flash_nystrom_attention, optional depthwise conv residual.
    Parameter names match the reference so its checkpoints load."""

    def __init__(self, dim, heads=8, config=None):
        super().__init__()
        if config is None:
            config = NystromConfig()
        assert dim % heads == 0
        self.dim, self.heads, self.head_dim = dim, heads, dim // heads
        self.config = config
        self.q_proj = nn.Linear(dim, dim, bias=False)
        self.k_proj = nn.Linear(dim, dim, bias=False)
        self.v_proj = nn.Linear(dim, dim, bias=False)
        self.out_proj = nn.Linear(dim, dim, bias=False)
        if config.use_conv_residual and config.conv_kernel_size > 0:
            self.conv_weight = nn.Parameter(torch.randn(heads, config.conv_kernel_size) * 0.02)
        else:
            self.conv_weight = None

    def forward(self, x):
        B, N, _ = x.shape
        H, D = self.heads, self.head_dim
        # Head-split views of the projection outputs, no transposing copies: where the tensor-core
        # kernels run they read this layout through strided tensor maps and write the output and the
        # gradients the same way; elsewhere the copies the reference always makes
        # (flash_nystrom/flash_nystrom.py:271-276) are made here.
        q = self.q_proj(x).view(B, N, H, D).transpose(1, 2)
        k = self.k_proj(x).view(B, N, H, D).transpose(1, 2)
        v = self.v_proj(x).view(B, N, H, D).transpose(1, 2)
        if not (q.is_cuda and _C.tc_eligible(q.dtype, D, self.config.num_landmarks)):
            q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        ks = self.config.conv_kernel_size if self.conv_weight is not None else 0
        out = flash_nystrom_attention(
            q, k, v, num_landmarks=self.config.num_landmarks, newton_iter=self.config.newton_iter,
            conv_weight=self.conv_weight, conv_kernel_size=ks,
            fast_dk2inv=self.config.fast_dk2inv, kappa_star=self.config.kappa_star,
            use_tc_pinv=self.config.use_tc_pinv)
        return self.out_proj(out.transpose(1, 2).reshape(B, N, self.dim))
