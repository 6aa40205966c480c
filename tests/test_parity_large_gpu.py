"""Parity at the sizes the benchmark runs (run with -m gpu): every tensor-core kernel here walks
many 128-row tiles per CTA, so the staging rings wrap, the mbarrier parities flip, the TMEM
accumulators add up over tiles, the ping-pong groups take several turns and the parked
softmax-Jacobian tiles of different CTAs interleave in the dQ / dK buffers.

The GPU call always runs at the full shape (so the tile schedule is the benchmarked one); the
float64 oracle is evaluated on a few of the (b, h) slices, which are independent end to end.
Bars as in test_parity_gpu.py: rel_max = max|a-b| / max|b|; fp16 output <= 2e-3, gradients <= 1e-2.
Per-stage bars (saved tensors) are about three times what a B200 measures."""
import pytest
import torch

from oracle import nystrom_oracle as O
from tests._util import run_cuda, run_oracle

pytestmark = pytest.mark.gpu

STAGES = ["qt", "kt", "K2", "lse2", "k2inv", "bmat", "lse3", "step2", "lse1"]
# saved-tensor bars for 16-bit inputs (FP32 landmarks, FP32 Newton-Schulz, 16-bit MMA operands)
STAGE_TOL = {"qt": 2e-5, "kt": 2e-5, "K2": 2e-4, "lse2": 2e-5, "k2inv": 2e-3, "bmat": 2e-3,
             "lse3": 2e-5, "step2": 4e-3, "lse1": 2e-4}


def _check_slices(cu, q, k, v, dO, m, J, kappa, slices, out_tol, grad_tol, stage_scale=1.0):
    """Compare the listed flat (b*H + h) slices of a full-shape CUDA result with the oracle."""
    B, H = q.shape[:2]
    worst = {}
    for s in slices:
        b, h = divmod(s, H)
        sl = (slice(b, b + 1), slice(h, h + 1))
        ref = run_oracle(q[sl], k[sl], v[sl], dO[sl], m, J, kappa)
        for key in ["out", "dq", "dk", "dv"] + STAGES:
            got = cu[key][sl].detach().cpu()
            assert torch.isfinite(got).all(), (key, s)
            e = O.rel_max(got, ref[key])
            worst[key] = max(worst.get(key, 0.0), e)
    print({k_: f"{v_:.2e}" for k_, v_ in worst.items()})
    assert worst["out"] <= out_tol, worst
    for key in ("dq", "dk", "dv"):
        assert worst[key] <= grad_tol, worst
    for key in STAGES:
        assert worst[key] <= STAGE_TOL[key] * stage_scale, (key, worst)
    return worst


def test_config3_full_shape(cuda_device):
    """The benchmarked workload itself: B=1, H=16, N=65536, D=64, m=64, J=6, fp16 (29 tiles per
    CTA); four of the sixteen heads against the oracle."""
    B, H, N, D, m, J = 1, 16, 65536, 64, 64, 6
    q, k, v, dO = O.make_inputs(B, H, N, D, seed=0, dtype=torch.float16)
    cu = run_cuda(q, k, v, dO, m, J, 0.0)
    _check_slices(cu, q, k, v, dO, m, J, 0.0, [0, 5, 10, 15], 2e-3, 1e-2)


@pytest.mark.parametrize("N,dtype", [(262144, torch.float16), (131072, torch.float16),
                                     (131072, torch.bfloat16)])
def test_one_long_slice(cuda_device, N, dtype):
    """One slice, very long: softmax-3 probabilities are ~1/N (the 2^k shift of the column-pass
    backward sits at its cap) and one CTA walks the whole run of tiles of a 1/296th of the slice."""
    q, k, v, dO = O.make_inputs(1, 1, N, 64, seed=1, dtype=dtype)
    cu = run_cuda(q, k, v, dO, 64, 6, 0.0)
    bf = dtype == torch.bfloat16
    _check_slices(cu, q, k, v, dO, 64, 6, 0.0, [0], 8e-3 if bf else 2e-3, 4e-2 if bf else 1e-2,
                  stage_scale=8.0 if bf else 1.0)


def test_config4_full_shape(cuda_device):
    """Large-landmark configuration at full size: B=2, H=8, N=16384, D=128, m=128, J=8, ridge
    kappa* = 5, fp16; three of the sixteen slices against the oracle."""
    B, H, N, D, m, J, kap = 2, 8, 16384, 128, 128, 8, 5.0
    q, k, v, dO = O.make_inputs(B, H, N, D, seed=0, dtype=torch.float16)
    cu = run_cuda(q, k, v, dO, m, J, kap)
    _check_slices(cu, q, k, v, dO, m, J, kap, [0, 7, 12], 2e-3, 1e-2)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_head_dim_128_full_shape(cuda_device, dtype):
    """The shape of the reference's own latency tables: B=4, H=16, N=16384, D=128, m=64, J=6
    (tensor-core path with one CTA per SM, several tiles per CTA); three of the 64 slices."""
    B, H, N, D, m, J = 4, 16, 16384, 128, 64, 6
    q, k, v, dO = O.make_inputs(B, H, N, D, seed=4, dtype=dtype)
    cu = run_cuda(q, k, v, dO, m, J, 0.0)
    bf = dtype == torch.bfloat16
    _check_slices(cu, q, k, v, dO, m, J, 0.0, [0, 21, 63], 8e-3 if bf else 2e-3, 4e-2 if bf else 1e-2,
                  stage_scale=8.0 if bf else 1.0)


def test_head_dim_128_ragged_ridge(cuda_device):
    """head_dim 128 with a ragged sequence, 40 landmarks (padded to 64) and the ridge."""
    B, H, N, D, m, J, kap = 1, 3, 20011, 128, 40, 6, 5.0
    q, k, v, dO = O.make_inputs(B, H, N, D, seed=6, dtype=torch.float16)
    cu = run_cuda(q, k, v, dO, m, J, kap)
    _check_slices(cu, q, k, v, dO, m, J, kap, [0, 2], 2e-3, 1e-2)


def test_ragged_many_tiles(cuda_device):
    """N not a multiple of the tile, of the landmark count or of anything else; 33 landmarks
    (padded to 64 on the tensor-core path); seven slices; about ten tiles per CTA."""
    B, H, N, D, m, J = 1, 7, 50001, 64, 33, 6
    q, k, v, dO = O.make_inputs(B, H, N, D, seed=2, dtype=torch.float16)
    cu = run_cuda(q, k, v, dO, m, J, 0.0)
    _check_slices(cu, q, k, v, dO, m, J, 0.0, [0, 3, 6], 2e-3, 1e-2)


def test_many_slices_many_tiles_bf16(cuda_device):
    """More slices than a quarter of the SMs (the backward keeps the pseudoinverse on the main
    stream) and still several tiles per CTA, bf16."""
    B, H, N, D, m, J = 5, 8, 8192, 64, 64, 6
    q, k, v, dO = O.make_inputs(B, H, N, D, seed=3, dtype=torch.bfloat16)
    cu = run_cuda(q, k, v, dO, m, J, 0.0)
    _check_slices(cu, q, k, v, dO, m, J, 0.0, [0, 17, 39], 8e-3, 4e-2, stage_scale=8.0)


@pytest.mark.parametrize("D,m", [(64, 64), (128, 64)])
def test_more_slices_than_resident_ctas(cuda_device, D, m):
    """B*H = 512 slices: one CTA per slice and more CTAs than the GPU holds at once, so the grid of
    every tensor-core kernel runs in several waves (the first, the last and two middle slices
    against the oracle)."""
    q, k, v, dO = O.make_inputs(32, 16, 2048, D, seed=41, dtype=torch.float16)
    cu = run_cuda(q, k, v, dO, m, 6, 0.0)
    _check_slices(cu, q, k, v, dO, m, 6, 0.0, [0, 147, 300, 511], 2e-3, 1e-2)


def test_config2_module_full_shape(cuda_device):
    """The module configuration: dim 512, 8 heads (D = 64), B=4, N=4096, num_landmarks 64, conv
    residual k=3, fp16 weights and activations, y.sum().backward(); against the same module
    evaluated on the CPU in float64 (oracle in place of the kernels, same state_dict)."""
    from flashnystrom_b200 import FlashNystromAttention, NystromConfig
    torch.manual_seed(0)
    dim, heads, Bm, Nm = 512, 8, 4, 4096
    cfg = NystromConfig(num_landmarks=64, newton_iter=6, conv_kernel_size=3)
    mod = FlashNystromAttention(dim, heads=heads, config=cfg)
    mod.conv_weight.data = torch.randn(heads, 3) * 0.02
    x = torch.randn(Bm, Nm, dim)
    mod = mod.half()
    x16 = x.half()
    sd = {k_: v_.double() for k_, v_ in mod.state_dict().items()}

    def cpu_forward(xx):
        proj = lambda w: (xx @ w.t()).view(Bm, Nm, heads, dim // heads).transpose(1, 2)
        q, k, v = proj(sd["q_proj.weight"]), proj(sd["k_proj.weight"]), proj(sd["v_proj.weight"])
        o = O.attention(q, k, v, 64, 6, sd["conv_weight"], 3)
        return o.transpose(1, 2).reshape(Bm, Nm, dim) @ sd["out_proj.weight"].t()

    xc = x16.double().requires_grad_(True)
    yc = cpu_forward(xc)
    yc.sum().backward()
    modg = mod.cuda()
    xg = x16.cuda().requires_grad_(True)
    yg = modg(xg)
    yg.sum().backward()
    torch.cuda.synchronize()
    from flashnystrom_b200 import _C
    _C.check_device_status()
    e_y = O.rel_max(yg.detach().cpu(), yc.detach())
    e_x = O.rel_max(xg.grad.cpu(), xc.grad)
    print("config 2 module: y", f"{e_y:.2e}", "dx", f"{e_x:.2e}")
    # fp16 projections (cuBLAS, fp16 outputs) sit on both sides of the attention: 16-bit rounding
    # of q, k, v and of the attention output dominates
    assert e_y <= 4e-3 and e_x <= 2e-2, (e_y, e_x)
