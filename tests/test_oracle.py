"""CPU tests of the oracle: it must reproduce the golden vectors produced by the reference's
own reference.py (tests/golden/make_golden.py), and its hand-written backward must agree with
autograd through its own forward."""
import os

import numpy as np
import pytest
import torch

from oracle import nystrom_oracle as O
from tests.golden.make_golden import CASES

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.npz")


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


def _inputs(case):
    B, H, N, D, m, J, kap, seed, dt, qks, stride, ks = CASES[case]
    q, k, v, dO = O.make_inputs(B, H, N, D, seed=seed, dtype=getattr(torch, dt), qk_scale=qks)
    return tuple(t.float() for t in (q, k, v, dO))


@pytest.mark.parametrize("case", sorted(CASES))
def test_oracle_matches_reference_golden(golden, case):
    B, H, N, D, m, J, kap, seed, dt, qks, stride, ks = CASES[case]
    q, k, v, dO = _inputs(case)
    chk = golden[f"{case}/in_checksum"]
    got = [float(t.double().sum()) for t in (q, k, v, dO)] + \
          [float(t.double().abs().sum()) for t in (q, k, v, dO)]
    assert np.allclose(chk, got, rtol=1e-12, atol=1e-9), "seeded inputs differ from the fixture"
    w = torch.from_numpy(golden[f"{case}/conv_weight"]) if ks else None
    torch.set_num_threads(1)
    out, dq, dk, dv = O.forward_backward_autograd(q, k, v, dO, m, J, kap, w, ks)
    for key, t in (("out", out), ("dq", dq), ("dk", dk), ("dv", dv)):
        ref = torch.from_numpy(golden[f"{case}/{key}"])
        # same ops in the same order as reference.py: FP32 round-off only
        assert O.rel_max(t[:, :, ::stride], ref) < 2e-5, (case, key)
        cs = golden[f"{case}/{key}_checksum"]
        assert abs(float(t.double().abs().sum()) - cs[1]) <= 1e-4 * abs(cs[1]), (case, key)


@pytest.mark.parametrize("shape", [(1, 2, 300, 16, 7, 6, 0.0), (1, 2, 256, 32, 16, 8, 5.0),
                                   (1, 1, 130, 16, 8, 3, 1e3), (1, 1, 64, 64, 64, 4, 0.0),
                                   (2, 1, 96, 16, 1, 6, 0.0)])
def test_hand_backward_matches_autograd_fp64(shape):
    B, H, N, D, m, J, kap = shape
    q, k, v, dO = O.make_inputs(B, H, N, D, seed=11, dtype=torch.float64)
    hb = O.backward(q, k, v, dO, m, J, kap)
    _, dq, dk, dv = O.forward_backward_autograd(q, k, v, dO, m, J, kap)
    assert O.rel_max(hb["dq"], dq) < 1e-12
    assert O.rel_max(hb["dk"], dk) < 1e-12
    assert O.rel_max(hb["dv"], dv) < 1e-12


def test_pinv_of_identity_and_spd():
    eye = torch.eye(8, dtype=torch.float64)[None, None]
    Z = O.newton_schulz(eye, 6)[-1]
    assert torch.allclose(Z, eye, atol=1e-12)
    g = torch.Generator().manual_seed(0)
    R = torch.randn(1, 1, 12, 12, generator=g, dtype=torch.float64)
    A = R @ R.transpose(-2, -1) + 0.5 * torch.eye(12, dtype=torch.float64)
    Z = O.newton_schulz(A, 30)[-1]
    assert O.rel_max(A @ Z @ A, A) < 1e-8


def test_segments_and_errors():
    seg, starts, ends = O.segment_bounds(300, 7)
    assert seg == 42 and starts[-1] == 252 and ends[-1] == 300
    assert O.landmark_index(300, 7)[-1] == 6 and O.landmark_index(300, 7)[293] == 6
    q = torch.zeros(1, 1, 4, 16)
    with pytest.raises(ValueError, match="must be >="):
        O.forward(q, q, q, 8)


def test_slices_independent():
    q, k, v, dO = O.make_inputs(2, 2, 64, 16, seed=1)
    full = O.forward(q, k, v, 8)["out"]
    part = O.forward(q[1:], k[1:], v[1:], 8)["out"]
    assert torch.allclose(full[1:], part, atol=1e-6)
