"""Host-side mirror of the reference's `flash_nystrom._C` extension module
(pybind signatures: csrc/flash_nystrom.cu:629-690), backed by the C-ABI library.

    forward(q, k, v, num_landmarks=64, newton_iter=6, kappa_star=0.0, use_tc_pinv=False,
            need_scaled_qk=True) -> [output, q_s, k_s, q_tilde, k_tilde, k2inv, step2, lse1, lse2,
                                     lse3, ns_iterates, k2_softmax, b_saved]
    backward(dO, q_s, k_s, q_tilde, k_tilde, kernel2_inv, step2, lse1, lse2, lse3, ns_iterates,
             k2_softmax, b_saved, v, output, num_landmarks, newton_iter, fast_dk2inv=True,
             kappa_star=0.0) -> [dQ, dK, dV]

Differences from the reference, all deliberate:
  * no scaled copies of Q and K are made: the q_s / k_s slots hold the caller's own q and k
    (the kernels fold the D^-1/4 scale in), so `need_scaled_qk` costs nothing either way;
  * the landmark-sized saved tensors (q_tilde, k_tilde, step2, b_saved) are FP32 whatever the
    input dtype;
  * num_landmarks up to 128 and head_dim 16/32/64/128 are native;
  * `use_tc_pinv` and `fast_dk2inv` are accepted and select nothing (FP32 always);
  * there is no CPU path: tensors must live on a CUDA device of compute capability 10.x.
All work is enqueued on torch's current stream of the inputs' device; nothing synchronises.
"""
import ctypes as C
import math
import os as _os

import torch

from . import _lib

_DTYPES = {torch.float32: _lib.FNB_F32, torch.float16: _lib.FNB_F16, torch.bfloat16: _lib.FNB_BF16}
_flags = 0


def set_force_generic(on: bool):
    """Route 16-bit inputs through the CUDA-core FP32 kernels too (verification aid)."""
    global _flags
    _flags = (_flags | _lib.FNB_FLAG_FORCE_GENERIC) if on else (_flags & ~_lib.FNB_FLAG_FORCE_GENERIC)


def set_test_drop_load(on: bool):
    """Tests only: make one CTA of the forward output pass skip the copy of its last tile, so that
    a bounded device-side wait runs out (see FNB_FLAG_TEST_DROP_LOAD)."""
    global _flags
    _flags = (_flags | _lib.FNB_FLAG_TEST_DROP_LOAD) if on else (_flags & ~_lib.FNB_FLAG_TEST_DROP_LOAD)


def set_wait_limit_ms(ms: int, device=0):
    """Tests only: time limit of the bounded device-side waits (default 1500 ms)."""
    _lib.check(_lib.load().fnb_debug_set_wait_limit_ms(int(device), int(ms)))


def layout_of(t):
    """FNB_LAYOUT_BHND for a contiguous (B, H, N, D) tensor, FNB_LAYOUT_BNHD for the head-split view
    of a contiguous (B, N, H * D) tensor (t.transpose(1, 2) is contiguous), None for anything else."""
    if t.dim() != 4:
        return None
    if t.is_contiguous():
        return _lib.FNB_LAYOUT_BHND
    B, H, N, D = t.shape
    if t.stride() == (N * H * D, D, H * D, 1):      # (strides alone: no view object is made)
        return _lib.FNB_LAYOUT_BNHD
    if t.transpose(1, 2).is_contiguous():           # sizes of 1 leave some strides arbitrary
        return _lib.FNB_LAYOUT_BNHD
    return None


def tc_eligible(dtype, D, m):
    """Shapes the tensor-core kernels cover (the only ones that take the (B, N, H, D) layout)."""
    if _flags & _lib.FNB_FLAG_FORCE_GENERIC or dtype not in (torch.float16, torch.bfloat16):
        return False
    return (D == 64 and m <= 64) or (D == 128 and m <= 128)


def _empty_like_layout(t, layout):
    """Uninitialised tensor of t's logical shape (B, H, N, D) in the given memory layout."""
    if layout == _lib.FNB_LAYOUT_BNHD:
        B, H, N, D = t.shape
        return torch.empty(B, N, H, D, dtype=t.dtype, device=t.device).transpose(1, 2)
    return torch.empty(t.shape, dtype=t.dtype, device=t.device)


def _to_layout(t, layout):
    """t in the given layout (a copy only if it is not already)."""
    if layout_of(t) == layout:
        return t
    if layout == _lib.FNB_LAYOUT_BNHD:
        return t.transpose(1, 2).contiguous().transpose(1, 2)
    return t.contiguous()


class _NoContext:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_CONTEXT = _NoContext()


def _on_device(dev):
    """Context that makes `dev` current for the allocations of a call; nothing when it already is
    (the library selects the device of its own work itself)."""
    return _NO_CONTEXT if torch.cuda.current_device() == dev.index else torch.cuda.device(dev)


def _shape_struct(B, H, N, D, m, J, dtype, kappa_star, layout=0):
    if dtype not in _DTYPES:
        raise RuntimeError("Supported dtypes: float32, float16, bfloat16")
    if not (isinstance(kappa_star, (int, float)) and math.isfinite(kappa_star) and kappa_star >= 0):
        raise RuntimeError(f"kappa_star must be finite and >= 0 (got {kappa_star}); "
                           "0 disables the Tikhonov ridge")
    return _lib.Shape(int(B), int(H), int(N), int(D), int(m), int(J), _DTYPES[dtype],
                      float(kappa_star), _flags, int(layout), 0)


def _check_big(t, name, shape=None, dtype=None, layout=None):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor (flashnystrom_b200 has no CPU path)")
    if layout is None:
        if not t.is_contiguous():
            raise RuntimeError(f"{name} must be contiguous")
    elif layout_of(t) != layout:
        raise RuntimeError(f"{name} must be contiguous (or, with q, k, v all laid out that way, the head-split "
                           f"view of a contiguous (B, N, H*D) tensor)")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise RuntimeError(f"{name} shape mismatch: expected {tuple(shape)}, got {tuple(t.shape)}")
    if dtype is not None and t.dtype != dtype:
        raise RuntimeError(f"{name} must be {dtype}, got {t.dtype}")


def _ptr(t):
    return C.c_void_p(t.data_ptr())


_status_words = {}


def _status(device):
    """Per-device int32 word the kernels write to when a bounded device-side wait expires."""
    t = _status_words.get(device.index)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _status_words[device.index] = t
    return t


def check_device_status(device=None):
    """Synchronise and raise if any kernel since the last check abandoned a bounded wait."""
    for idx, t in list(_status_words.items()):
        if device is not None and torch.device(device).index != idx:
            continue
        val = int(t.item())
        if val != 0:
            t.zero_()
            code = (val >> 24) & 0xff
            what = {1: "a device-side wait timed out",
                    2: "a kernel's shared-memory window was misaligned",
                    3: "a non-finite softmax-Jacobian value reached the backward column pass "
                       "(inf / NaN in the inputs or the incoming gradient)"}.get(code, "a kernel reported an error")
            raise RuntimeError(f"flashnystrom_b200: {what} on cuda:{idx} "
                               f"(status 0x{val & 0xffffffff:08x}); results of that call are invalid")


def _workspace(nbytes, device):
    return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)


def forward(q, k, v, num_landmarks=64, newton_iter=6, kappa_star=0.0, use_tc_pinv=False,
            need_scaled_qk=True):
    lib = _lib.load()
    if not all(isinstance(t, torch.Tensor) for t in (q, k, v)) or q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise RuntimeError("q, k, v must be 4D (B, H, N, D)")
    if not (q.dtype == k.dtype == v.dtype):
        raise RuntimeError("q, k, v dtypes must match")
    B, H, N, D = q.shape
    m, J = int(num_landmarks), int(newton_iter)
    # the head-split view of (B, N, H*D) projection outputs is taken as it is where the tensor-core
    # kernels run; everything else must be contiguous, as in the reference
    lay = layout_of(q)
    if lay != _lib.FNB_LAYOUT_BNHD or not tc_eligible(q.dtype, D, m) or layout_of(k) != lay or layout_of(v) != lay:
        lay = _lib.FNB_LAYOUT_BHND
    for t, name in ((q, "q"), (k, "k"), (v, "v")):
        _check_big(t, name, (B, H, N, D), layout=lay)
    shp = _shape_struct(B, H, N, D, m, J, q.dtype, kappa_star, lay)
    _lib.check(lib.fnb_check_shape(C.byref(shp)))
    dev = q.device
    f32 = dict(dtype=torch.float32, device=dev)
    with _on_device(dev):
        out = _empty_like_layout(q, lay)
        lse1 = torch.empty(B, H, N, **f32)
        qt = torch.empty(B, H, m, D, **f32)
        kt = torch.empty(B, H, m, D, **f32)
        k2 = torch.empty(B, H, m, m, **f32)
        lse2 = torch.empty(B, H, m, **f32)
        iters = torch.empty(B, H, J + 1, m, m, **f32)
        k2inv = torch.empty(B, H, m, m, **f32)
        bmat = torch.empty(B, H, m, D, **f32)
        lse3 = torch.empty(B, H, m, **f32)
        step2 = torch.empty(B, H, m, D, **f32)
        ws = _workspace(lib.fnb_fwd_workspace_bytes(C.byref(shp)), dev)
        args = _lib.FwdArgs(shp, _ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(lse1), _ptr(qt),
                            _ptr(kt), _ptr(k2), _ptr(lse2), _ptr(iters), _ptr(k2inv), _ptr(bmat),
                            _ptr(lse3), _ptr(step2), _ptr(ws), ws.numel(), dev.index,
                            C.c_void_p(torch.cuda.current_stream(dev).cuda_stream), _ptr(_status(dev)))
        _lib.check(lib.fnb_forward(C.byref(args)))
    return [out, q, k, qt, kt, k2inv, step2, lse1, lse2, lse3, iters, k2, bmat]


def backward(dO, q_s, k_s, q_tilde, k_tilde, kernel2_inv, step2, lse1, lse2, lse3, ns_iterates,
             k2_softmax, b_saved, v, output, num_landmarks, newton_iter, fast_dk2inv=True,
             kappa_star=0.0):
    lib = _lib.load()
    if not isinstance(dO, torch.Tensor) or dO.dim() != 4:
        raise RuntimeError(f"dO must be 4D (B, H, N, D), got {getattr(dO, 'dim', lambda: '?')()}D")
    B, H, N, D = dO.shape
    m, J = int(num_landmarks), int(newton_iter)
    dt = dO.dtype
    # q decides the layout of all eight (B, H, N, D) tensors; dO is brought to it if it differs
    lay = layout_of(q_s) if isinstance(q_s, torch.Tensor) else None
    if lay != _lib.FNB_LAYOUT_BNHD or not tc_eligible(dt, D, m):
        lay = _lib.FNB_LAYOUT_BHND
    if isinstance(dO, torch.Tensor) and dO.is_cuda:
        dO = _to_layout(dO, lay)
    _check_big(dO, "dO", layout=lay)
    shp = _shape_struct(B, H, N, D, m, J, dt, kappa_star, lay)
    _lib.check(lib.fnb_check_shape(C.byref(shp)))
    f32 = torch.float32
    _check_big(q_s, "q_s", (B, H, N, D), dt, layout=lay)
    _check_big(k_s, "k_s", (B, H, N, D), dt, layout=lay)
    _check_big(v, "v", (B, H, N, D), dt, layout=lay)
    _check_big(q_tilde, "q_tilde", (B, H, m, D), f32)
    _check_big(k_tilde, "k_tilde", (B, H, m, D), f32)
    _check_big(step2, "step2", (B, H, m, D), f32)
    _check_big(b_saved, "b_saved", (B, H, m, D), f32)
    _check_big(kernel2_inv, "kernel2_inv", (B, H, m, m), f32)
    _check_big(k2_softmax, "k2_softmax", (B, H, m, m), f32)
    _check_big(lse1, "softmax1_lse", (B, H, N), f32)
    _check_big(lse3, "softmax3_lse", (B, H, m), f32)
    _check_big(ns_iterates, "ns_iterates", (B, H, J + 1, m, m), f32)
    dev = dO.device
    with _on_device(dev):
        dq, dk, dv = (_empty_like_layout(dO, lay) for _ in range(3))
        ws = _workspace(lib.fnb_bwd_workspace_bytes(C.byref(shp)), dev)
        args = _lib.BwdArgs(shp, _ptr(q_s), _ptr(k_s), _ptr(v), _ptr(dO), _ptr(lse1),
                            _ptr(q_tilde), _ptr(k_tilde), _ptr(k2_softmax), _ptr(ns_iterates),
                            _ptr(kernel2_inv), _ptr(b_saved), _ptr(lse3), _ptr(step2), _ptr(dq),
                            _ptr(dk), _ptr(dv), _ptr(ws), ws.numel(), dev.index,
                            C.c_void_p(torch.cuda.current_stream(dev).cuda_stream), _ptr(_status(dev)))
        _lib.check(lib.fnb_backward(C.byref(args)))
    if _os.environ.get("FNB_BWD_DEBUG"):   # per-stage statistics, as FN_BWD_DEBUG does in the reference
        for name, st in tensor_stats(dO=dO, dQ=dq, dK=dk, dV=dv, step2=step2, k2inv=kernel2_inv).items():
            print(f"[FNB_BWD_DEBUG] {name}: absmax={st['absmax']:.4e} absmean={st['absmean']:.4e} "
                  f"nonfinite={st['nonfinite']}")
        check_device_status(dev)
    return [dq, dk, dv]


def reset_caches():
    """The reference drops its thread-local CUDA-graph and scratch caches here
    (csrc/flash_nystrom.cu:641-650).  This library keeps no caches; nothing to do."""
    return None


def debug_pinv_forward(k2, newton_iter, kappa_star=0.0):
    """(BH, m, m) softmax matrix -> (ns_iterates (BH, J+1, m, m), k2_inv (BH, m, m))."""
    lib = _lib.load()
    _check_big(k2, "k2", dtype=torch.float32)
    BH, m, _ = k2.shape
    J = int(newton_iter)
    dev = k2.device
    with _on_device(dev):
        iters = torch.empty(BH, J + 1, m, m, dtype=torch.float32, device=dev)
        k2inv = torch.empty_like(k2)
        ws = _workspace(lib.fnb_debug_pinv_workspace_bytes(BH, m), dev)
        _lib.check(lib.fnb_debug_pinv_forward(BH, m, J, float(kappa_star), _ptr(k2), _ptr(iters),
                                              _ptr(k2inv), _ptr(ws), ws.numel(), dev.index,
                                              C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)))
    return iters, k2inv


def debug_pinv_backward(k2, ns_iterates, d_k2_inv, kappa_star=0.0):
    """Gradient of the pseudoinverse w.r.t. the softmax matrix k2 (lambda detached)."""
    lib = _lib.load()
    _check_big(k2, "k2", dtype=torch.float32)
    BH, m, _ = k2.shape
    J = ns_iterates.shape[1] - 1
    _check_big(ns_iterates, "ns_iterates", (BH, J + 1, m, m), torch.float32)
    _check_big(d_k2_inv, "d_k2_inv", (BH, m, m), torch.float32)
    dev = k2.device
    with _on_device(dev):
        dk2 = torch.empty_like(k2)
        ws = _workspace(lib.fnb_debug_pinv_workspace_bytes(BH, m), dev)
        _lib.check(lib.fnb_debug_pinv_backward(BH, m, J, float(kappa_star), _ptr(k2),
                                               _ptr(ns_iterates), _ptr(d_k2_inv), _ptr(dk2),
                                               _ptr(ws), ws.numel(), dev.index,
                                               C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)))
    return dk2


def debug_ns_bwd_step(K2, Z_j, dZ_in):
    """One backward iteration of the Newton-Schulz unroll on the product's tensor-core kernel: the
    reference's debug_ns_bwd_step (csrc/flash_nystrom.cu:422-456).  (BH, m, m) FP32 tensors,
    m <= 64.  Returns [dZ_out, dK2_acc]: dL/dZ_j and this iteration's contribution to dL/dK2."""
    lib = _lib.load()
    for t, name in ((K2, "K2"), (Z_j, "Z_j"), (dZ_in, "dZ_in")):
        _check_big(t, name, dtype=torch.float32)
    if K2.dim() != 3 or K2.shape[1] != K2.shape[2] or Z_j.shape != K2.shape or dZ_in.shape != K2.shape:
        raise RuntimeError("K2, Z_j, dZ_in must all have shape (BH, m, m)")
    BH, m, _ = K2.shape
    dev = K2.device
    with _on_device(dev):
        dZ_out, dK2_acc = torch.empty_like(K2), torch.empty_like(K2)
        _lib.check(lib.fnb_debug_ns_bwd_step(BH, m, _ptr(K2), _ptr(Z_j), _ptr(dZ_in), _ptr(dZ_out), _ptr(dK2_acc),
                                             dev.index, C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)))
    return [dZ_out, dK2_acc]


def debug_ns_bwd_final(q_tilde, k_tilde, K2, dZ0, dK2_in):
    """The tail of the backward in isolation: the reference's debug_ns_bwd_final
    (csrc/flash_nystrom.cu:474-520).  q_tilde, k_tilde (BH, m, D); K2, dZ0, dK2_in (BH, m, m); FP32,
    m <= 64.  Returns [dQ_tilde, dK_tilde, dK2] with dK2 = dK2_in plus the Z0 terms."""
    lib = _lib.load()
    for t, name in ((q_tilde, "q_tilde"), (k_tilde, "k_tilde"), (K2, "K2"), (dZ0, "dZ0"), (dK2_in, "dK2_in")):
        _check_big(t, name, dtype=torch.float32)
    BH, m, D = q_tilde.shape
    dev = K2.device
    with _on_device(dev):
        dq, dk, dk2 = torch.empty_like(q_tilde), torch.empty_like(k_tilde), torch.empty_like(K2)
        zeros = torch.zeros(m, D, dtype=torch.float32, device=dev)
        _lib.check(lib.fnb_debug_ns_bwd_final(BH, m, D, _ptr(q_tilde), _ptr(k_tilde), _ptr(K2), _ptr(dZ0), _ptr(dK2_in),
                                              _ptr(zeros), _ptr(dq), _ptr(dk), _ptr(dk2), dev.index,
                                              C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)))
    return [dq, dk, dk2]


def probe_occupancy(device=0):
    """Registers, shared memory, spill bytes and resident CTAs per SM of the hot-path kernels, like
    the reference's probe_occupancy (csrc/occupancy_probe.h:89-142).  List of dicts."""
    lib = _lib.load()
    buf = (_lib.KernelInfo * 32)()
    n = lib.fnb_kernel_report(int(device), buf, 32)
    return [{f: (getattr(buf[i], f).decode() if f == "name" else getattr(buf[i], f)) for f, _ in _lib.KernelInfo._fields_}
            for i in range(n)]


def tensor_stats(**tensors):
    """abs-max, abs-mean and non-finite count per tensor (synchronises): what the reference prints
    with FN_BWD_DEBUG set (csrc/flash_nystrom.cu:392-408)."""
    out = {}
    for name, t in tensors.items():
        f = t.detach().float()
        out[name] = {"absmax": float(f.abs().max()), "absmean": float(f.abs().mean()),
                     "nonfinite": int((~torch.isfinite(f)).sum())}
    return out


def pinv_backward_noalloc(k2, ns_iterates, d_k2_inv, out, kappa_star=0.0):
    """Pseudoinverse gradient into the caller's `out` tensor through the entry point that
    allocates nothing (scratch is a fixed array inside the library).  For hosts that may not
    allocate device memory after start-up; at most 64 slices and num_landmarks <= 64 per call.
    Calls must not overlap on the GPU: they share the scratch."""
    lib = _lib.load()
    _check_big(k2, "k2", dtype=torch.float32)
    BH, m, _ = k2.shape
    J = ns_iterates.shape[1] - 1
    _check_big(ns_iterates, "ns_iterates", (BH, J + 1, m, m), torch.float32)
    _check_big(d_k2_inv, "d_k2_inv", (BH, m, m), torch.float32)
    _check_big(out, "out", (BH, m, m), torch.float32)
    dev = k2.device
    _lib.check(lib.fnb_pinv_backward_noalloc(BH, m, J, float(kappa_star), _ptr(k2), _ptr(ns_iterates),
                                             _ptr(d_k2_inv), _ptr(out), dev.index,
                                             C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)))
    return out


def query_sm_limits(device=0):
    """Device facts, like the reference's query_sm_limits (csrc/flash_nystrom.cu:693-726)."""
    lib = _lib.load()
    caps = _lib.Caps()
    _lib.check(lib.fnb_capabilities(int(device), C.byref(caps)))
    return {f: getattr(caps, f) for f, _ in _lib.Caps._fields_}


def set_profiling(on: bool):
    """Switch per-kernel CUDA-event timing on or off; returns the previous setting."""
    return bool(_lib.load().fnb_set_profiling(1 if on else 0))


def last_profile():
    """[(kernel name, milliseconds)] of the last forward or backward call on this thread."""
    lib = _lib.load()
    buf = (_lib.KernelTime * 32)()
    n = lib.fnb_last_profile(buf, 32)
    return [(buf[i].name.decode(), buf[i].ms) for i in range(n)]


# ---- depthwise convolution residual --------------------------------------------------------------
def _conv_geometry(v):
    if not isinstance(v, torch.Tensor) or not v.is_cuda or v.dim() != 4:
        raise RuntimeError("conv residual: v must be a 4-D CUDA tensor (flashnystrom_b200 has no CPU path)")
    if v.dtype not in _DTYPES:
        raise RuntimeError("Supported dtypes: float32, float16, bfloat16")
    layout = layout_of(v)
    if layout is None:
        v, layout = v.contiguous(), _lib.FNB_LAYOUT_BHND
    return v, layout


def conv_residual(v, weight, base=None, transposed=False):
    """base + depthwise_conv(v) (base may be None), or with transposed=True the same with the taps
    reversed (what the backward applies to the incoming gradient).  v, base: (B, H, N, D) in either
    layout; weight: (H, kernel_size) FP32 on the device.  Returns a new tensor in v's layout."""
    lib = _lib.load()
    v, layout = _conv_geometry(v)
    B, H, N, D = v.shape
    w = weight.detach().to(device=v.device, dtype=torch.float32).contiguous()
    if w.dim() != 2 or w.shape[0] != H:
        raise RuntimeError(f"conv weight must be (heads, kernel_size) = ({H}, ks), got {tuple(w.shape)}")
    if base is not None:
        if base.shape != v.shape or base.dtype != v.dtype:
            raise RuntimeError("conv residual: base must have the shape and dtype of v")
        base = _to_layout(base.detach(), layout)
    result = _empty_like_layout(v, layout)
    args = _lib.ConvArgs(B, H, N, D, int(w.shape[1]), _DTYPES[v.dtype], int(layout), v.data_ptr(),
                         base.data_ptr() if base is not None else None, result.data_ptr(), w.data_ptr(),
                         1 if transposed else 0, v.device.index, torch.cuda.current_stream(v.device).cuda_stream)
    with _on_device(v.device):
        _lib.check(lib.fnb_conv_residual(C.byref(args)))
    return result


def conv_residual_dweight(v, d_out, kernel_size):
    """Gradient of the convolution residual with respect to its (H, kernel_size) weights, FP32."""
    lib = _lib.load()
    v, layout = _conv_geometry(v)
    B, H, N, D = v.shape
    if d_out.shape != v.shape or d_out.dtype != v.dtype:
        raise RuntimeError("conv residual: d_out must have the shape and dtype of v")
    d_out = _to_layout(d_out.detach(), layout)
    dw = torch.empty(H, int(kernel_size), dtype=torch.float32, device=v.device)
    nbytes = lib.fnb_conv_dweight_workspace_bytes(B, H, N, int(kernel_size))
    ws = torch.empty(max(int(nbytes), 16), dtype=torch.uint8, device=v.device)
    args = _lib.ConvDwArgs(B, H, N, D, int(kernel_size), _DTYPES[v.dtype], int(layout), v.data_ptr(), d_out.data_ptr(),
                           dw.data_ptr(), ws.data_ptr(), ws.numel(), v.device.index,
                           torch.cuda.current_stream(v.device).cuda_stream)
    with _on_device(v.device):
        _lib.check(lib.fnb_conv_residual_dweight(C.byref(args)))
    return dw

