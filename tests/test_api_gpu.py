"""Public Python API on the GPU: functional entry point, autograd Function, module, conv residual,
error behaviour.  Mirrors the reference's tests/test_flash_nystrom_cov.py and
tests/test_precision_config.py against the CPU oracle."""
import pytest
import torch

from oracle import nystrom_oracle as O

pytestmark = pytest.mark.gpu


def test_function_apply_eight_args_and_grads(cuda_device):
    from flashnystrom_b200 import FlashNystromFunction
    q, k, v, dO = O.make_inputs(1, 2, 384, 64, seed=0, dtype=torch.float16)
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    out = FlashNystromFunction.apply(qd, kd, vd, 32, 6, True, 0.0, False)
    out.backward(dO.cuda())
    ref = O.forward_backward_autograd(q.double(), k.double(), v.double(), dO.double(), 32, 6)
    assert O.rel_max(out.detach().cpu(), ref[0]) <= 2e-3
    for got, want in zip((qd.grad, kd.grad, vd.grad), ref[1:]):
        assert O.rel_max(got.cpu(), want) <= 1e-2


def test_conv_residual_matches_oracle(cuda_device):
    from flashnystrom_b200 import flash_nystrom_attention
    q, k, v, dO = O.make_inputs(2, 2, 200, 64, seed=1, dtype=torch.float32)
    w = torch.randn(2, 5, generator=torch.Generator().manual_seed(3)) * 0.3
    qd, kd, vd, wd = (t.cuda().requires_grad_(True) for t in (q, k, v, w))
    out = flash_nystrom_attention(qd, kd, vd, 16, 6, conv_weight=wd, conv_kernel_size=5)
    out.backward(dO.cuda())
    q2, k2, v2, w2 = (t.double().requires_grad_(True) for t in (q, k, v, w))
    ref = O.attention(q2, k2, v2, 16, 6, w2, 5)
    ref.backward(dO.double())
    assert O.rel_max(out.detach().cpu(), ref.detach()) <= 2e-4
    assert O.rel_max(vd.grad.cpu(), v2.grad) <= 2e-3
    assert O.rel_max(wd.grad.cpu(), w2.grad) <= 2e-3


def test_ridge_changes_output_and_matches(cuda_device):
    from flashnystrom_b200 import flash_nystrom_attention
    q, k, v, _ = O.make_inputs(1, 2, 1024, 64, seed=0, dtype=torch.float16)
    a = flash_nystrom_attention(q.cuda(), k.cuda(), v.cuda(), 64, 6, kappa_star=0.0)
    b = flash_nystrom_attention(q.cuda(), k.cuda(), v.cuda(), 64, 6, kappa_star=5.0)
    assert O.rel_max(a.cpu(), b.cpu()) > 1e-2
    ref = O.attention(q.double(), k.double(), v.double(), 64, 6, kappa_star=5.0)
    assert O.rel_max(b.cpu(), ref) <= 2e-3


def test_module_forward_backward_vs_cpu_module(cuda_device):
    """FlashNystromAttention (dim 128, 2 heads) against the same module evaluated on CPU in
    float64 with the oracle in place of the kernels and the same state_dict."""
    from flashnystrom_b200 import FlashNystromAttention, NystromConfig
    torch.manual_seed(0)
    cfg = NystromConfig(num_landmarks=16, newton_iter=6, conv_kernel_size=3)
    mod = FlashNystromAttention(128, heads=2, config=cfg)
    x = torch.randn(2, 256, 128)
    sd = {k_: v_.double() for k_, v_ in mod.state_dict().items()}

    def cpu_forward(xx):
        B, N, _ = xx.shape
        proj = lambda w: (xx @ w.t()).view(B, N, 2, 64).transpose(1, 2)
        q, k, v = proj(sd["q_proj.weight"]), proj(sd["k_proj.weight"]), proj(sd["v_proj.weight"])
        o = O.attention(q, k, v, 16, 6, sd["conv_weight"], 3)
        return o.transpose(1, 2).reshape(B, N, 128) @ sd["out_proj.weight"].t()

    xc = x.double().requires_grad_(True)
    yc = cpu_forward(xc)
    yc.sum().backward()
    modg = mod.cuda()
    xg = x.cuda().requires_grad_(True)
    yg = modg(xg)
    yg.sum().backward()
    assert O.rel_max(yg.detach().cpu(), yc.detach()) <= 1e-3
    assert O.rel_max(xg.grad.cpu(), xc.grad) <= 5e-3
    assert set(mod.state_dict()) == {"q_proj.weight", "k_proj.weight", "v_proj.weight", "out_proj.weight",
                                     "conv_weight"}


def test_module_fp16_runs(cuda_device):
    from flashnystrom_b200 import FlashNystromAttention
    mod = FlashNystromAttention(512, heads=8).cuda().half()
    x = torch.randn(2, 1024, 512, device="cuda", dtype=torch.float16, requires_grad=True)
    y = mod(x)
    y.sum().backward()
    assert torch.isfinite(y).all() and torch.isfinite(x.grad).all()


@pytest.mark.parametrize("bad,msg", [
    (dict(m=200), "num_landmarks must be in"),
    (dict(J=0), "newton_iter must be in"),
    (dict(kappa=-1.0), "kappa_star"),
    (dict(N=8, m=16), "must be >="),
])
def test_errors_are_runtime_errors(cuda_device, bad, msg):
    from flashnystrom_b200 import _C
    N, m, J, kappa = bad.get("N", 128), bad.get("m", 16), bad.get("J", 6), bad.get("kappa", 0.0)
    q = torch.zeros(1, 1, N, 64, device="cuda", dtype=torch.float16)
    with pytest.raises(RuntimeError, match=msg):
        _C.forward(q, q, q, m, J, kappa)
    with pytest.raises(RuntimeError, match="contiguous"):
        _C.forward(q.transpose(2, 3), q.transpose(2, 3), q.transpose(2, 3), 16, 6)
    with pytest.raises(RuntimeError, match="dtypes must match"):
        _C.forward(q, q.float(), q, 16, 6)


def test_backward_on_autograd_thread_and_no_status_error(cuda_device):
    from flashnystrom_b200 import flash_nystrom_attention, _C
    q, k, v, dO = O.make_inputs(1, 4, 2048, 64, seed=2, dtype=torch.bfloat16)
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    with torch.autograd.set_multithreading_enabled(False):
        flash_nystrom_attention(qd, kd, vd, 64, 6).backward(dO.cuda())
    torch.cuda.synchronize()
    _C.check_device_status()
    assert torch.isfinite(qd.grad).all()


def test_profile_lists_kernels(cuda_device):
    from flashnystrom_b200 import _C
    q, k, v, _ = O.make_inputs(1, 2, 512, 64, seed=0, dtype=torch.float16)
    _C.set_profiling(True)
    try:
        _C.forward(q.cuda(), k.cuda(), v.cuda(), 64, 6)
        prof = _C.last_profile()
    finally:
        _C.set_profiling(False)
    names = [n for n, _ in prof]
    assert "landmark_partial" in names and "tc_fwd_b" in names and "tc_fwd_c" in names
    assert all(ms >= 0 for _, ms in prof)
    caps = _C.query_sm_limits(0)
    assert caps["cc_major"] == 10 and caps["sm_count"] > 0


def test_cuda_graph_capture_and_replay(cuda_device):
    """A forward + backward captured once into a CUDA graph (the library allocates nothing, never
    synchronises and forks its side streams with events) replays to the same bits, also after the
    inputs were overwritten in place."""
    from flashnystrom_b200 import flash_nystrom_attention, _C
    q, k, v, dO = (t.cuda() for t in O.make_inputs(1, 4, 4096, 64, seed=12, dtype=torch.float16))
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)

    def step():
        q.grad = k.grad = v.grad = None
        out = flash_nystrom_attention(q, k, v, num_landmarks=64, newton_iter=6)
        out.backward(dO)
        return out

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            eager = step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    want = [eager.clone(), q.grad.clone(), k.grad.clone(), v.grad.clone()]
    g = torch.cuda.CUDAGraph()
    q.grad = k.grad = v.grad = None
    with torch.cuda.graph(g):
        gout = flash_nystrom_attention(q, k, v, num_landmarks=64, newton_iter=6)
        gout.backward(dO)
    g.replay()
    torch.cuda.synchronize()
    _C.check_device_status()
    for a, b in zip([gout, q.grad, k.grad, v.grad], want):
        assert torch.equal(a, b)
    # new data through the same graph: matches a fresh eager call
    with torch.no_grad():
        q.mul_(0.5)
        dO.mul_(2.0)
    g.replay()
    torch.cuda.synchronize()
    got = [gout.clone(), q.grad.clone(), k.grad.clone(), v.grad.clone()]
    eager = step()
    torch.cuda.synchronize()
    for a, b in zip(got, [eager, q.grad, k.grad, v.grad]):
        assert torch.equal(a, b)


def test_head_split_layout_matches_contiguous(cuda_device):
    """q, k, v given as head-split views of (B, N, H*D) tensors (what the projections of the module
    produce) go through strided tensor maps, without transposing copies: same bits as the contiguous
    call, and the output and the gradients come back in that layout too."""
    from flashnystrom_b200 import _C, flash_nystrom_attention
    B, H, N, D, m = 2, 3, 1500, 64, 48
    q, k, v, dO = (t.cuda() for t in O.make_inputs(B, H, N, D, seed=13, dtype=torch.float16))
    a = [t.clone().requires_grad_(True) for t in (q, k, v)]
    flash_nystrom_attention(*a, num_landmarks=m).backward(dO)
    want_out = flash_nystrom_attention(q, k, v, num_landmarks=m)
    # the same values stored as (B, N, H, D)
    b = [t.transpose(1, 2).contiguous().transpose(1, 2).detach().requires_grad_(True) for t in (q, k, v)]
    assert all(_C.layout_of(t) == 1 for t in b)
    out = flash_nystrom_attention(*b, num_landmarks=m)
    assert _C.layout_of(out) == 1 and torch.equal(out, want_out)
    out.backward(dO.transpose(1, 2).contiguous().transpose(1, 2))
    for x, y in zip(a, b):
        assert _C.layout_of(y.grad) == 1 and torch.equal(x.grad, y.grad)
    # head_dim 128 as well
    q, k, v, dO = (t.cuda() for t in O.make_inputs(1, 2, 700, 128, seed=14, dtype=torch.bfloat16))
    want = flash_nystrom_attention(q, k, v, num_landmarks=40)
    got = flash_nystrom_attention(*(t.transpose(1, 2).contiguous().transpose(1, 2) for t in (q, k, v)), num_landmarks=40)
    assert torch.equal(got, want)
    # fp32 (CUDA-core path): the view is accepted by the module only through a copy; the op itself refuses it
    with pytest.raises(RuntimeError, match="contiguous"):
        _C.forward(*(t.float().transpose(1, 2).contiguous().transpose(1, 2) for t in (q, k, v)), 40, 6)
