"""Host side of the sequence-parallel path on CPU: two gloo ranks run the real orchestration
(flashnystrom_b200.seqpar.forward_collectives / backward_collectives: stage calls + all-reduce /
all-gather) with the torch stand-in backend, and must reproduce the single-process oracle."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, shape, kappa, ret):
    sys.path.insert(0, ROOT)
    from flashnystrom_b200 import seqpar
    from oracle import nystrom_oracle as O
    from tests._sp_backend import TorchContext
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, H, N, D, m, J = shape
        q, k, v, dO = O.make_inputs(B, H, N, D, seed=3, dtype=torch.float64)
        Nl = N // world
        sl = slice(rank * Nl, (rank + 1) * Nl)
        ctx = TorchContext(q[:, :, sl], k[:, :, sl], v[:, :, sl], m, J, kappa, rank, world)
        seqpar.forward_collectives(ctx)
        ctx.begin_backward(dO[:, :, sl])
        seqpar.backward_collectives(ctx)
        ref_out, rq, rk, rv = O.forward_backward_autograd(q, k, v, dO, m, J, kappa)
        errs = [O.rel_max(ctx.out, ref_out[:, :, sl]), O.rel_max(ctx.dq, rq[:, :, sl]),
                O.rel_max(ctx.dk, rk[:, :, sl]), O.rel_max(ctx.dv, rv[:, :, sl])]
        ret[rank] = errs
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("shape,kappa", [((1, 2, 256, 16, 8, 6), 0.0), ((2, 1, 192, 32, 16, 4), 5.0)])
def test_two_gloo_ranks_match_oracle(shape, kappa):
    world = 2
    port = 29500 + (os.getpid() % 2000)
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, shape, kappa, ret), nprocs=world, join=True)
    assert len(ret) == world
    for rank, errs in ret.items():
        # xfer buffers are FP32, everything else float64
        assert max(errs) < 5e-5, (rank, errs)


def test_xfer_sizes_match_c_abi():
    import ctypes as C
    from flashnystrom_b200 import _lib, seqpar
    lib = _lib.load()
    shp = _lib.Shape(2, 4, 512, 64, 32, 6, _lib.FNB_F16, 0.0, 0)
    for bwd in (0, 1):
        for stage in (0, 1, 2):
            assert lib.fnb_sp_xfer_floats(C.byref(shp), 4, bwd, stage) == seqpar.xfer_floats(8, 32, 64, 4, bool(bwd), stage)


def test_sp_argument_checks():
    import ctypes as C
    from flashnystrom_b200 import _lib
    lib = _lib.load()
    args = _lib.FwdArgs()
    args.shape = _lib.Shape(1, 1, 512, 64, 32, 6, _lib.FNB_F16, 0.0, 0)
    sp = _lib.SpInfo(0, 3, 0, 3 * 512, None, 0)
    assert lib.fnb_sp_forward(C.byref(args), C.byref(sp)) == -1 and "multiple of world" in _lib.last_error()
    sp = _lib.SpInfo(0, 2, 0, 999, None, 0)
    assert lib.fnb_sp_forward(C.byref(args), C.byref(sp)) == -1 and "seq_len_global" in _lib.last_error()
    sp = _lib.SpInfo(5, 2, 0, 1024, None, 0)
    assert lib.fnb_sp_forward(C.byref(args), C.byref(sp)) == -1 and "out of range" in _lib.last_error()
