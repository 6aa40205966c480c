"""The torch.library custom operators: fake implementations, autograd registration (opcheck) and a
torch.compile trace of the public entry point without a graph break."""
import pytest
import torch

from oracle import nystrom_oracle as O

pytestmark = pytest.mark.gpu


def _inputs(dtype=torch.float16, N=512, m=32):
    q, k, v, dO = O.make_inputs(1, 2, N, 64, seed=9, dtype=dtype)
    return q.cuda(), k.cuda(), v.cuda(), dO.cuda(), m


def test_opcheck_forward_and_backward_ops(cuda_device):
    from flashnystrom_b200 import _ops
    q, k, v, dO, m = _inputs()
    qr, kr, vr = (t.clone().requires_grad_(True) for t in (q, k, v))
    # schema, fake tensor propagation, autograd registration, AOT dispatch
    torch.library.opcheck(_ops.nystrom_fwd, (qr, kr, vr, m, 6, 0.0),
                          test_utils=("test_schema", "test_faketensor", "test_autograd_registration"))
    res = _ops.nystrom_fwd(q, k, v, m, 6, 0.0)
    torch.library.opcheck(_ops.nystrom_bwd, (dO, q, k, v, *res, m, 6, 0.0),
                          test_utils=("test_schema", "test_faketensor"))


def test_ops_match_the_autograd_function(cuda_device):
    from flashnystrom_b200 import _ops, flash_nystrom_attention
    q, k, v, dO, m = _inputs()
    a = [t.clone().requires_grad_(True) for t in (q, k, v)]
    b = [t.clone().requires_grad_(True) for t in (q, k, v)]
    flash_nystrom_attention(*a, num_landmarks=m).backward(dO)
    _ops.attention_via_ops(*b, m, 6, 0.0).backward(dO)
    for x, y in zip(a, b):
        assert torch.equal(x.grad, y.grad)


def test_compile_traces_without_graph_break(cuda_device):
    from flashnystrom_b200 import flash_nystrom_attention
    q, k, v, dO, m = _inputs()

    def f(q_, k_, v_):
        return flash_nystrom_attention(q_ * 1.0, k_, v_, num_landmarks=m, newton_iter=6) + 0.0

    a = [t.clone().requires_grad_(True) for t in (q, k, v)]
    b = [t.clone().requires_grad_(True) for t in (q, k, v)]
    ref = f(*a)
    ref.backward(dO)
    # aot_eager: Dynamo + AOT autograd (fake tensors, functionalisation, the registered backward),
    # no code generation; fullgraph=True fails on any graph break
    cf = torch.compile(f, backend="aot_eager", fullgraph=True)
    got = cf(*b)
    got.backward(dO)
    assert torch.equal(got, ref)
    for x, y in zip(a, b):
        assert torch.equal(x.grad, y.grad)


def test_install_as_reference_package_name(cuda_device):
    import importlib
    import sys
    import flashnystrom_b200
    flashnystrom_b200.install_as("flash_nystrom")
    try:
        mod = importlib.import_module("flash_nystrom")
        from flash_nystrom import flash_nystrom_attention, NystromConfig, _C  # noqa: F401
        assert mod.HAS_CUDA and hasattr(_C, "forward") and hasattr(_C, "backward")
    finally:
        for name in [n for n in sys.modules if n == "flash_nystrom" or n.startswith("flash_nystrom.")]:
            del sys.modules[name]
