"""Sequence-parallel Nystrom attention: every (b,h) slice's sequence is cut into `world` equal
contiguous shards, one per rank (one process per GPU, torch.distributed / NCCL over NVLink).

Only landmark-sized data crosses ranks, four times per forward + backward:

    forward   all-reduce  raw landmark segment sums            2 * BH * m * D floats
              all-gather  softmax-3 partial (acc, max, sum)    BH * m * (D + 2) floats per rank
    backward  all-reduce  dstep2 and dKt partial sums          2 * BH * m * D floats
              all-reduce  dQt partial sums                     BH * m * D floats

Everything landmark-sized (K2, Newton-Schulz, its backward) is recomputed identically on every
rank; everything N-sized stays local.  The reference has no multi-GPU path; this follows the
split-N partial + combine algebra of its kernel3 (csrc/kernels/kernel3_output_fused.cuh:772-916)
across devices.  Requirements: num_landmarks % world == 0 and (world * N_local) % num_landmarks
== 0, so that every landmark segment lives on one rank.

The orchestration (`forward_collectives`, `backward_collectives`) only moves `xfer` buffers and
calls `stage(k)` on a backend context, so it runs unchanged on CPU ranks (gloo) with a stand-in
backend; `CudaContext` is the real one, three C-ABI calls per direction.
"""
import ctypes as C

import torch
import torch.distributed as dist

from . import _C, _lib


def xfer_floats(BH, m, D, world, backward, stage):
    md, mv = BH * m * D, BH * m
    if backward:
        return 2 * md if stage == 0 else md
    return 2 * md if stage == 0 else (md + 2 * mv if stage == 1 else world * (md + 2 * mv))


def forward_collectives(ctx, group=None):
    """Run the three forward stages of `ctx` with the two collectives between them."""
    world = dist.get_world_size(group)
    BH, m, D = ctx.BH, ctx.m, ctx.D
    n0, n1 = xfer_floats(BH, m, D, world, False, 0), xfer_floats(BH, m, D, world, False, 1)
    x = ctx.new_xfer(max(n0, n1))
    ctx.forward_stage(0, x)
    dist.all_reduce(x[:n0], group=group)
    ctx.forward_stage(1, x)
    gathered = ctx.new_xfer(world * n1)
    dist.all_gather_into_tensor(gathered, x[:n1].contiguous(), group=group)
    ctx.forward_stage(2, gathered)
    return ctx


def backward_collectives(ctx, group=None):
    """Run the three backward stages of `ctx` with the two all-reduces between them."""
    world = dist.get_world_size(group)
    BH, m, D = ctx.BH, ctx.m, ctx.D
    n0, n1 = xfer_floats(BH, m, D, world, True, 0), xfer_floats(BH, m, D, world, True, 1)
    x = ctx.new_xfer(n0)
    ctx.backward_stage(0, x)
    dist.all_reduce(x[:n0], group=group)
    ctx.backward_stage(1, x)
    dist.all_reduce(x[:n1], group=group)
    ctx.backward_stage(2, x)
    return ctx


class CudaContext:
    """One sequence-parallel forward (+ backward) of this rank's shard through the C ABI."""

    def __init__(self, q, k, v, num_landmarks, newton_iter, kappa_star, rank, world):
        for t, name in ((q, "q"), (k, "k"), (v, "v")):
            _C._check_big(t, name)
        B, H, N, D = q.shape
        self.q, self.k, self.v = q, k, v
        self.B, self.H, self.N, self.D = B, H, N, D
        self.BH, self.m, self.J = B * H, int(num_landmarks), int(newton_iter)
        self.kappa, self.rank, self.world = float(kappa_star), int(rank), int(world)
        self.dev = q.device
        self.lib = _lib.load()
        self.shape = _C._shape_struct(B, H, N, D, self.m, self.J, q.dtype, self.kappa)
        _lib.check(self.lib.fnb_check_shape(C.byref(self.shape)))
        f32 = dict(dtype=torch.float32, device=self.dev)
        m, J = self.m, self.J
        self.out = torch.empty_like(q)
        self.lse1 = torch.empty(B, H, N, **f32)
        self.qt, self.kt = torch.empty(B, H, m, D, **f32), torch.empty(B, H, m, D, **f32)
        self.k2, self.k2inv = torch.empty(B, H, m, m, **f32), torch.empty(B, H, m, m, **f32)
        self.lse2, self.lse3 = torch.empty(B, H, m, **f32), torch.empty(B, H, m, **f32)
        self.iters = torch.empty(B, H, J + 1, m, m, **f32)
        self.bmat, self.step2 = torch.empty(B, H, m, D, **f32), torch.empty(B, H, m, D, **f32)
        self.ws_f = _C._workspace(self.lib.fnb_fwd_workspace_bytes(C.byref(self.shape)), self.dev)
        self.ws_b = None

    def new_xfer(self, n):
        return torch.empty(n, dtype=torch.float32, device=self.dev)

    def _sp(self, stage, x):
        return _lib.SpInfo(self.rank, self.world, stage, self.world * self.N, x.data_ptr(), x.numel())

    def _stream(self):
        return C.c_void_p(torch.cuda.current_stream(self.dev).cuda_stream)

    def forward_stage(self, stage, x):
        p = _C._ptr
        with torch.cuda.device(self.dev):
            args = _lib.FwdArgs(self.shape, p(self.q), p(self.k), p(self.v), p(self.out), p(self.lse1), p(self.qt),
                                p(self.kt), p(self.k2), p(self.lse2), p(self.iters), p(self.k2inv), p(self.bmat),
                                p(self.lse3), p(self.step2), p(self.ws_f), self.ws_f.numel(), self.dev.index,
                                self._stream(), p(_C._status(self.dev)))
            sp = self._sp(stage, x)
            _lib.check(self.lib.fnb_sp_forward(C.byref(args), C.byref(sp)))

    def begin_backward(self, d_out):
        self.d_out = d_out.contiguous()
        self.dq, self.dk, self.dv = (torch.empty_like(self.q) for _ in range(3))
        self.ws_b = _C._workspace(self.lib.fnb_bwd_workspace_bytes(C.byref(self.shape)), self.dev)

    def backward_stage(self, stage, x):
        p = _C._ptr
        with torch.cuda.device(self.dev):
            args = _lib.BwdArgs(self.shape, p(self.q), p(self.k), p(self.v), p(self.d_out), p(self.lse1), p(self.qt),
                                p(self.kt), p(self.k2), p(self.iters), p(self.k2inv), p(self.bmat), p(self.lse3),
                                p(self.step2), p(self.dq), p(self.dk), p(self.dv), p(self.ws_b), self.ws_b.numel(),
                                self.dev.index, self._stream(), p(_C._status(self.dev)))
            sp = self._sp(stage, x)
            _lib.check(self.lib.fnb_sp_backward(C.byref(args), C.byref(sp)))


class _SeqParallelFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, num_landmarks, newton_iter, kappa_star, group):
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        c = CudaContext(q, k, v, num_landmarks, newton_iter, kappa_star, rank, world)
        forward_collectives(c, group)
        # The backward does not read the output.  Keeping it on the context would tie the returned
        # tensor to its own grad_fn (out -> grad_fn -> ctx -> context -> out): such a cycle is only
        # collected by the garbage collector, and every step would allocate fresh device memory.
        out, c.out = c.out, None
        c.ws_f = None
        ctx.sp, ctx.group = c, group
        return out

    @staticmethod
    def backward(ctx, grad_output):
        c = ctx.sp
        c.begin_backward(grad_output)
        backward_collectives(c, ctx.group)
        dq, dk, dv = c.dq, c.dk, c.dv
        c.dq = c.dk = c.dv = c.d_out = c.ws_b = None      # the context may outlive this call
        return dq, dk, dv, None, None, None, None


def seq_parallel_nystrom_attention(q, k, v, num_landmarks=64, newton_iter=6, kappa_star=0.0, group=None):
    """q, k, v: this rank's (B, H, N_local, D) CUDA shard of the sequence (rank r holds global rows
    [r * N_local, (r + 1) * N_local)).  Returns this rank's rows of the output; differentiable."""
    if not (dist.is_available() and dist.is_initialized()):
        raise RuntimeError("seq_parallel_nystrom_attention needs an initialised torch.distributed process group")
    return _SeqParallelFunction.apply(q, k, v, num_landmarks, newton_iter, kappa_star, group)
