"""Sequence-parallel kernels on one GPU: `world` virtual ranks run the staged C-ABI calls on their
shards one after another and the collectives are emulated by summing / concatenating the xfer
buffers, so the sharded geometry (row offsets, global segment lengths, strided merge of gathered
partials) is checked against the oracle without needing several GPUs."""
import pytest
import torch

from oracle import nystrom_oracle as O

pytestmark = pytest.mark.gpu


def _run_virtual_ranks(q, k, v, dO, m, J, kappa, world):
    from flashnystrom_b200 import seqpar, _C
    B, H, N, D = q.shape
    Nl = N // world
    shard = lambda t, r: t[:, :, r * Nl:(r + 1) * Nl].contiguous().cuda()
    ctxs = [seqpar.CudaContext(shard(q, r), shard(k, r), shard(v, r), m, J, kappa, r, world) for r in range(world)]
    BH = B * H
    n0, n1 = seqpar.xfer_floats(BH, m, D, world, False, 0), seqpar.xfer_floats(BH, m, D, world, False, 1)
    xs = [c.new_xfer(max(n0, n1)) for c in ctxs]
    for c, x in zip(ctxs, xs):
        c.forward_stage(0, x)
    tot = torch.stack([x[:n0] for x in xs]).sum(0)                 # all-reduce
    for c, x in zip(ctxs, xs):
        x[:n0] = tot
        c.forward_stage(1, x)
    gathered = torch.cat([x[:n1] for x in xs])                      # all-gather, rank-major
    for c in ctxs:
        c.forward_stage(2, gathered.clone())
    m0, m1 = seqpar.xfer_floats(BH, m, D, world, True, 0), seqpar.xfer_floats(BH, m, D, world, True, 1)
    ys = [c.new_xfer(m0) for c in ctxs]
    for r, (c, y) in enumerate(zip(ctxs, ys)):
        c.begin_backward(shard(dO, r))
        c.backward_stage(0, y)
    tot = torch.stack(ys).sum(0)
    for c, y in zip(ctxs, ys):
        y.copy_(tot)
        c.backward_stage(1, y)
    tot = torch.stack([y[:m1] for y in ys]).sum(0)
    for c, y in zip(ctxs, ys):
        y[:m1] = tot
        c.backward_stage(2, y)
    torch.cuda.synchronize()
    _C.check_device_status()
    cat = lambda name: torch.cat([getattr(c, name).cpu() for c in ctxs], dim=2)
    return cat("out"), cat("dq"), cat("dk"), cat("dv"), ctxs


@pytest.mark.parametrize("world", [1, 2, 4])
@pytest.mark.parametrize("dtype,shape", [
    (torch.float16, (1, 2, 2048, 64, 64, 6, 0.0)),
    (torch.float16, (2, 1, 1024, 64, 32, 6, 5.0)),
    (torch.float32, (1, 2, 512, 32, 16, 6, 0.0)),
    # more than 64 landmarks: the landmark-sized stages run as thread-block clusters
    (torch.float16, (1, 2, 2048, 128, 128, 6, 5.0)),
])
def test_virtual_ranks_match_oracle(cuda_device, world, dtype, shape):
    B, H, N, D, m, J, kappa = shape
    q, k, v, dO = O.make_inputs(B, H, N, D, seed=7, dtype=dtype)
    out, dq, dk, dv, ctxs = _run_virtual_ranks(q, k, v, dO, m, J, kappa, world)
    ref = O.forward_backward_autograd(q.double(), k.double(), v.double(), dO.double(), m, J, kappa)
    otol, gtol = (2e-3, 1e-2) if dtype == torch.float16 else (2e-4, 2e-3)
    e = [O.rel_max(a, b) for a, b in zip((out, dq, dk, dv), ref)]
    print(world, dtype, shape, [f"{x:.2e}" for x in e])
    assert e[0] <= otol and max(e[1:]) <= gtol, e
    # replicated saved tensors agree across ranks
    for c in ctxs[1:]:
        assert torch.equal(c.k2inv, ctxs[0].k2inv) and torch.equal(c.step2, ctxs[0].step2)


def test_world_one_equals_plain_call(cuda_device):
    from flashnystrom_b200 import _C
    q, k, v, dO = O.make_inputs(1, 2, 1024, 64, seed=1, dtype=torch.float16)
    out, dq, dk, dv, _ = _run_virtual_ranks(q, k, v, dO, 64, 6, 0.0, 1)
    res = _C.forward(q.cuda(), k.cuda(), v.cuda(), 64, 6)
    g = _C.backward(dO.cuda(), *res[1:13], v.cuda(), res[0], 64, 6)
    for a, b in ((out, res[0]), (dq, g[0]), (dk, g[1]), (dv, g[2])):
        assert O.rel_max(a, b.cpu()) < 2e-3


_NCCL_CHILD = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from flashnystrom_b200 import _C, flash_nystrom_attention
from flashnystrom_b200.seqpar import seq_parallel_nystrom_attention
os.environ["MASTER_ADDR"] = "127.0.0.1"
os.environ["MASTER_PORT"] = sys.argv[2]
torch.cuda.set_device(0)
dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
g = torch.Generator(device="cuda").manual_seed(3)
q, k, v = (torch.randn(1, 2, 4096, 64, device="cuda", dtype=torch.float16, generator=g).requires_grad_(True)
           for _ in range(3))
dO = torch.randn(1, 2, 4096, 64, device="cuda", dtype=torch.float16, generator=g)
def step():
    q.grad = k.grad = v.grad = None
    out = seq_parallel_nystrom_attention(q, k, v, 64, 6)
    out.backward(dO)
    return out
for _ in range(3):
    out = step()
torch.cuda.synchronize()
allocs = torch.cuda.memory_stats()["num_device_alloc"]
for _ in range(6):
    out = step()
torch.cuda.synchronize()
_C.check_device_status()
grew = torch.cuda.memory_stats()["num_device_alloc"] - allocs
sp = [t.detach().float().cpu() for t in (out, q.grad, k.grad, v.grad)]
q.grad = k.grad = v.grad = None
ref_out = flash_nystrom_attention(q, k, v, num_landmarks=64, newton_iter=6)
ref_out.backward(dO)
ref = [t.detach().float().cpu() for t in (ref_out, q.grad, k.grad, v.grad)]
err = max(float((a - b).abs().max() / b.abs().max()) for a, b in zip(sp, ref))
dist.destroy_process_group()
print("RESULT", grew, err)
"""


def test_nccl_world1_autograd_path(cuda_device, tmp_path):
    """The real torch.distributed (NCCL) path on one GPU, world size 1, in a child process: same
    results as the unsharded call, and steady-state steps allocate no new device memory (the
    autograd context must not keep the returned output alive through a reference cycle)."""
    import os
    import subprocess
    import sys
    script = tmp_path / "nccl_child.py"
    script.write_text(_NCCL_CHILD)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    port = str(29600 + os.getpid() % 300)
    res = subprocess.run([sys.executable, str(script), root, port], capture_output=True, text=True, timeout=240)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    line = [ln for ln in res.stdout.splitlines() if ln.startswith("RESULT")][-1].split()
    grew, err = int(line[1]), float(line[2])
    assert grew == 0, f"{grew} new device allocations over 6 steady-state steps"
    assert err <= 2e-3, f"sequence-parallel (world 1) vs unsharded rel_max {err}"
