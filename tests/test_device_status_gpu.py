"""The device status word: what the host sees when a kernel could not finish its work the ordinary
way.  Nothing here faults, traps or hangs the GPU: the expiry test makes a bounded wait run out (one
CTA is told never to issue one copy, the wait limit is shortened to a few milliseconds) and the
kernel then leaves through its normal teardown; the range tests feed fp16 a softmax-3 so peaked (and a
dO so large) that a fixed scaling of the 16-bit dS' tiles would overflow: the kernel rescales per tile
and the gradients stay within the bars."""
import pytest
import torch

from oracle import nystrom_oracle as O
from tests._util import run_cuda, run_oracle, errs

pytestmark = pytest.mark.gpu


def test_bounded_wait_expires_and_the_context_stays_usable(cuda_device):
    from flashnystrom_b200 import _C
    q, k, v, dO = O.make_inputs(1, 2, 4096, 64, seed=11, dtype=torch.float16)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    _C.check_device_status()
    _C.set_wait_limit_ms(5)
    _C.set_test_drop_load(True)
    try:
        _C.forward(qd, kd, vd, 64, 6)          # returns: nothing in the call waits on the host side
        torch.cuda.synchronize()               # and the kernels return too, a few milliseconds later
        with pytest.raises(RuntimeError, match="wait timed out"):
            _C.check_device_status()
    finally:
        _C.set_test_drop_load(False)
        _C.set_wait_limit_ms(1500)
    _C.check_device_status()                   # the word was cleared by the failed check
    # tensor memory and shared memory were released: the same call now runs and is right
    cu = run_cuda(q, k, v, dO, 64, 6, 0.0)
    ref = run_oracle(q, k, v, dO, 64, 6, 0.0)
    e = errs(cu, ref, ["out", "dq", "dk", "dv"])
    assert e["out"] <= 2e-3 and max(e["dq"], e["dk"], e["dv"]) <= 1e-2, e


def _peaked_inputs(dtype, N=16384, m=16, D=64, seed=21, qmul=0.5, kmul=3.0):
    """Softmax-3 with a large share of a landmark's mass on one key: the queries of every segment
    share a direction (so the landmark has a component along it) and one key per segment points the
    same way.  With the defaults the score of that key is about 12 above the rest."""
    q, k, v, dO = O.make_inputs(1, 1, N, D, seed=seed, dtype=torch.float32)
    g = torch.Generator().manual_seed(seed + 1)
    seg = N // m
    for j in range(m):
        u = torch.sign(torch.randn(D, generator=g))
        q[0, 0, j * seg:(j + 1) * seg] += qmul * u
        k[0, 0, j * seg + 7] = kmul * u
    return tuple(t.to(dtype) for t in (q, k, v, dO))


@pytest.mark.parametrize("kmul", [2.0, 3.0, 4.0])
def test_peaked_softmax3_fp16(cuda_device, kmul):
    """fp16 at N = 16384 with 15 % .. 99.8 % of a landmark's softmax-3 mass on one key: the parked
    softmax-Jacobian tiles are rescaled on the fly (no clamp, no status) and the gradients hold the
    bar.  The bars are twice the N(0,1) ones: the large scores of this case amplify the rounding of
    the 16-bit landmark operands, in any implementation that feeds them to 16-bit MMAs."""
    q, k, v, dO = _peaked_inputs(torch.float16, kmul=kmul)
    cu = run_cuda(q, k, v, dO, 16, 6, 0.0)       # ends with check_device_status(): nothing reported
    ref = run_oracle(q, k, v, dO, 16, 6, 0.0)
    assert float(ref["P3"].max()) > 0.1, "the case is meant to be peaked"
    e = errs(cu, ref, ["out", "dq", "dk", "dv"])
    print(kmul, e)
    assert e["out"] <= 4e-3 and max(e["dq"], e["dk"], e["dv"]) <= 2e-2, e


@pytest.mark.parametrize("kmul", [2.0, 3.0])
def test_peaked_softmax3_bf16(cuda_device, kmul):
    """bf16 has the FP32 exponent range: no shift, no rescaling.  8-bit mantissas and this case's
    large scores: bars twice the usual bf16 ones."""
    q, k, v, dO = _peaked_inputs(torch.bfloat16, kmul=kmul)
    cu = run_cuda(q, k, v, dO, 16, 6, 0.0)
    ref = run_oracle(q, k, v, dO, 16, 6, 0.0)
    e = errs(cu, ref, ["out", "dq", "dk", "dv"])
    print(kmul, e)
    assert e["out"] <= 3e-2 and max(e["dq"], e["dk"], e["dv"]) <= 5e-2, e


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_large_incoming_gradient(cuda_device, dtype):
    """dO of magnitude ~ 2^12 (a loss-scaled gradient).  bf16 must simply be right; fp16 must be
    right or say that a 16-bit copy left its range - saturated gradients never come back silently."""
    from flashnystrom_b200 import _C
    q, k, v, dO = O.make_inputs(1, 2, 8192, 64, seed=31, dtype=torch.float32, dO_scale=4096.0)
    q, k, v, dO = (t.to(dtype) for t in (q, k, v, dO))
    _C.check_device_status()
    try:
        cu = run_cuda(q, k, v, dO, 64, 6, 0.0)
    except RuntimeError as exc:
        assert dtype == torch.float16 and "fp16 range" in str(exc), exc
        print("reported:", exc)
        return
    ref = run_oracle(q, k, v, dO, 64, 6, 0.0)
    e = errs(cu, ref, ["out", "dq", "dk", "dv"])
    print(dtype, e)
    bf = dtype == torch.bfloat16
    assert e["out"] <= (1.4e-2 if bf else 2e-3) and max(e["dq"], e["dk"], e["dv"]) <= (2.5e-2 if bf else 1e-2), e
