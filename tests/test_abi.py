"""The C-ABI library loads without a GPU and exports every symbol the header declares; the
host-side checks (shape validation, workspace sizing, error text) run on CPU."""
import ctypes as C
import os
import re

import pytest
import torch

from flashnystrom_b200 import _lib, _C

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "flashnystrom_b200.h")


@pytest.fixture(scope="module")
def lib():
    return _lib.load()


def test_every_declared_symbol_is_exported_and_bound(lib):
    text = open(HEADER).read()
    declared = set(re.findall(r"FNB_API\s+[\w\s\*]+?\b(fnb_\w+)\s*\(", text))
    assert len(declared) >= 12
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert declared == set(_lib.SIGNATURES), "ctypes binding and header disagree"
    assert lib.fnb_version() == 2


def _shape(B=1, H=2, N=256, D=64, m=32, J=6, dtype=_lib.FNB_F16, kappa=0.0):
    return _lib.Shape(B, H, N, D, m, J, dtype, kappa, 0)


@pytest.mark.parametrize("kw,msg", [
    (dict(N=16, m=32), "must be >="),
    (dict(m=0), "num_landmarks must be in"),
    (dict(m=129), "num_landmarks must be in"),
    (dict(D=48), "head_dim must be"),
    (dict(J=0), "newton_iter must be in"),
    (dict(J=21), "newton_iter must be in"),
    (dict(kappa=-1.0), "kappa_star must be finite"),
    (dict(kappa=float("inf")), "kappa_star must be finite"),
    (dict(B=0), "must be positive"),
    (dict(dtype=7), "Supported dtypes"),
])
def test_shape_validation_messages(lib, kw, msg):
    s = _shape(**kw)
    assert lib.fnb_check_shape(C.byref(s)) == -1
    assert msg in _lib.last_error()
    assert lib.fnb_fwd_workspace_bytes(C.byref(s)) == 0


def test_workspace_sizes_scale(lib):
    small, big = _shape(N=1024), _shape(N=65536, H=16, m=64)
    a, b = lib.fnb_fwd_workspace_bytes(C.byref(small)), lib.fnb_fwd_workspace_bytes(C.byref(big))
    assert 0 < a < b < 1 << 30
    assert lib.fnb_bwd_workspace_bytes(C.byref(big)) % 256 == 0


def test_null_and_workspace_errors(lib):
    assert lib.fnb_forward(None) == -1
    args = _lib.FwdArgs()
    args.shape = _shape()
    assert lib.fnb_forward(C.byref(args)) == -1 and "non-NULL" in _lib.last_error()
    assert lib.fnb_debug_pinv_workspace_bytes(4, 64) >= 4 * 12 * 64 * 64 * 4
    assert lib.fnb_debug_pinv_workspace_bytes(4, 300) == 0


def test_python_face_rejects_cpu_tensors():
    q = torch.zeros(1, 1, 64, 64)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        _C.forward(q, q, q, 16, 6)
    from flashnystrom_b200 import flash_nystrom_attention
    with pytest.raises(RuntimeError, match="no CPU path"):
        flash_nystrom_attention(q, q, q, 16)
    assert _C.reset_caches() is None


def test_kappa_validated_in_python_face():
    with pytest.raises(RuntimeError, match="kappa_star"):
        _C._shape_struct(1, 1, 64, 64, 16, 6, torch.float16, float("nan"))


def test_conv_residual_argument_checks(lib):
    """Shape and pointer checks of the convolution residual come before any device is touched."""
    a = _lib.ConvArgs(1, 2, 64, 64, 4, _lib.FNB_F16, 0, 16, None, 32, 48, 0, 0, None)
    assert lib.fnb_conv_residual(C.byref(a)) == -1 and "must be odd" in _lib.last_error()
    a = _lib.ConvArgs(1, 2, 64, 48, 3, _lib.FNB_F16, 0, 16, None, 32, 48, 0, 0, None)
    assert lib.fnb_conv_residual(C.byref(a)) == -1 and "head_dim must be" in _lib.last_error()
    a = _lib.ConvArgs(1, 2, 64, 64, 3, _lib.FNB_F16, 0, 16, None, 16, 48, 0, 0, None)
    assert lib.fnb_conv_residual(C.byref(a)) == -1 and "must not alias" in _lib.last_error()
    a = _lib.ConvArgs(1, 2, 64, 64, 3, _lib.FNB_F16, 0, 8, None, 32, 48, 0, 0, None)
    assert lib.fnb_conv_residual(C.byref(a)) == -1 and "16-byte aligned" in _lib.last_error()
    assert lib.fnb_conv_dweight_workspace_bytes(2, 4, 1000, 33) == 256 * ((4 * 2 * 4 * 16 * 33 + 255) // 256)
    assert lib.fnb_conv_dweight_workspace_bytes(2, 4, 1000, 0) == 0
    d = _lib.ConvDwArgs(2, 4, 1000, 64, 33, _lib.FNB_F16, 0, 16, 32, 48, 64, 16, 0, None)
    assert lib.fnb_conv_residual_dweight(C.byref(d)) != 0 and "workspace must be" in _lib.last_error()

