"""ctypes binding of libsso_b200.so (the C ABI declared in include/sso_b200.h).

There is no CPU or pure-torch fallback behind these wrappers: if the shared library is
missing or a call fails, a RuntimeError is raised.  Build it with
``python pytorch-sso_b200/build.py`` (needs nvcc; cross-compiles without a GPU).
"""
from __future__ import annotations

import ctypes as C
import os
import threading
from typing import Optional, Sequence

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, 'lib', 'libsso_b200.so')

F32, BF16, F16 = 0, 1, 2
IMPL_AUTO, IMPL_SIMT, IMPL_TCGEN05, IMPL_TMA = 0, 1, 2, 3
_DTYPES = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}

_lib = None
_lock = threading.Lock()

c_i64, c_i32, c_f32, c_vp, c_sz = C.c_int64, C.c_int, C.c_float, C.c_void_p, C.c_size_t


class TileTask(C.Structure):
    _fields_ = [('A', c_vp), ('B', c_vp), ('C', c_vp), ('C2', c_vp),
                ('lda', C.c_int32), ('ldb', C.c_int32), ('ldc', C.c_int32), ('ldc2', C.c_int32),
                ('m', C.c_int32), ('n', C.c_int32), ('k', C.c_int32), ('flags', C.c_uint32),
                ('alpha', c_f32), ('beta', c_f32)]


class DiagRec(C.Structure):
    _fields_ = [('L', c_vp), ('Linv', c_vp), ('ld_l', C.c_int32), ('ld_inv', C.c_int32),
                ('size', C.c_int32), ('mat', C.c_int32), ('row0', C.c_int32), ('info_slot', C.c_int32),
                ('LinvT', c_vp), ('ld_invt', C.c_int32), ('pad', C.c_int32)]


class CopyRec(C.Structure):
    _fields_ = [('src', c_vp), ('dst', c_vp), ('d', C.c_int32), ('row0', C.c_int32),
                ('nrows', C.c_int32), ('mat', C.c_int32), ('mode', C.c_int32), ('ld', C.c_int32)]


class Phase(C.Structure):
    _fields_ = [('kind', C.c_int32), ('first', C.c_int32), ('count', C.c_int32), ('reserved', C.c_int32)]


class FactorDesc(C.Structure):
    _fields_ = [('x', c_vp), ('dtype', C.c_int32), ('append_ones', C.c_int32),
                ('n', c_i64), ('c', c_i64), ('h', c_i64), ('w', c_i64),
                ('sn', c_i64), ('sc', c_i64), ('sh', c_i64), ('sw', c_i64),
                ('kh', C.c_int32), ('kw', C.c_int32), ('stride_h', C.c_int32), ('stride_w', C.c_int32),
                ('pad_h', C.c_int32), ('pad_w', C.c_int32), ('dil_h', C.c_int32), ('dil_w', C.c_int32),
                ('sample_weight', c_vp), ('alpha', c_f32), ('beta', c_f32), ('out', c_vp), ('ldo', c_i64)]


TRI_REC_DTYPE = np.dtype([('m', np.uint64), ('packed', np.uint64), ('n', np.int32), ('ld', np.int32),
                          ('row0', np.int32), ('nrows', np.int32)])

# name -> (restype, argtypes); every symbol include/sso_b200.h declares
SIGNATURES = {
    'sso_version': (c_i32, []),
    'sso_last_error': (C.c_char_p, []),
    'sso_launch_count': (C.c_uint64, []),
    'sso_configure': (c_i32, [C.c_char_p, c_i32]),
    'sso_factor_workspace_bytes': (c_sz, [c_i64, c_i64, c_i32]),
    'sso_factor_syrk_im2col': (c_i32, [c_vp, c_i32] + [c_i64] * 8 + [c_i32] * 8 +
                               [c_i32, c_vp, c_f32, c_f32, c_vp, c_i64, c_vp, c_sz, c_i32, c_vp]),
    'sso_factor_syrk': (c_i32, [c_vp, c_i32, c_i64, c_i64, c_i64, c_i64, c_i32, c_vp, c_f32, c_f32,
                                c_vp, c_i64, c_vp, c_sz, c_i32, c_vp]),
    'sso_factor_syrk_noalloc': (c_i32, [c_vp, c_i32, c_i64, c_i64, c_i64, c_i64, c_i32, c_vp, c_f32, c_f32,
                                        c_vp, c_i64, c_i32, c_vp]),
    'sso_factor_batch_workspace_bytes': (c_sz, [c_i32, c_vp]),
    'sso_factor_batch': (c_i32, [c_i32, c_vp, c_vp, c_sz, c_vp]),
    'sso_bn_plane_splits': (c_i32, [c_i32, c_i64, c_i64, c_i64, c_i64]),
    'sso_bn_plane_sums': (c_i32, [c_vp, c_vp, c_i32] + [c_i64] * 9 + [c_vp] * 4 + [c_i32, c_vp]),
    'sso_bn_diag_finish': (c_i32, [c_vp, c_vp, c_vp, c_i64, c_i64, c_i32, c_i32, c_f32, c_f32, c_vp, c_vp, c_vp]),
    'sso_ema_update': (c_i32, [c_vp, c_vp, c_i64, c_f32, c_i32, c_vp]),
    'sso_axpby': (c_i32, [c_vp, c_vp, c_i64, c_f32, c_f32, c_vp]),
    'sso_diag_inv_precondition': (c_i32, [c_vp, c_vp, c_vp, c_i64, c_f32, c_i32, c_i32, c_vp]),
    'sso_tri_pack': (c_i32, [c_vp, c_i32, c_f32, c_vp]),
    'sso_tri_unpack': (c_i32, [c_vp, c_i32, c_f32, c_i32, c_vp]),
    'sso_copy_segments': (c_i32, [c_vp, c_i32, c_f32, c_vp]),
    'sso_wire_absmax': (c_i32, [c_vp, c_vp, c_i32, c_vp, c_vp]),
    'sso_wire_encode': (c_i32, [c_vp, c_vp, c_i32, c_vp, c_vp, c_i32, c_vp]),
    'sso_wire_decode': (c_i32, [c_vp, c_vp, c_i32, c_vp, c_vp, c_i32, c_vp]),
    'sso_kron_plan_dev_bytes': (c_sz, [c_i32, c_vp, c_i32]),
    'sso_kron_plan_create': (c_i64, [c_i32, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_sz, c_i32, c_vp]),
    'sso_kron_plan_run': (c_i32, [c_i64, c_vp, c_vp, c_i32, c_i32, c_vp]),
    'sso_precond_plan_dev_bytes': (c_sz, [c_i32, c_vp, c_vp]),
    'sso_precond_plan_create': (c_i64, [c_i32] + [c_vp] * 8 + [c_sz, c_i32, c_vp, c_vp]),
    'sso_precond_plan_run': (c_i32, [c_i64, c_vp]),
    'sso_sample_plan_dev_bytes': (c_sz, [c_i32, c_vp, c_vp]),
    'sso_sample_plan_create': (c_i64, [c_i32] + [c_vp] * 9 + [c_sz, c_i32, c_vp, c_vp]),
    'sso_sample_plan_run': (c_i32, [c_i64, c_f32, c_vp]),
    'sso_plan_destroy': (c_i32, [c_i64]),
    'sso_plan_status': (c_i32, [c_i64]),
    'sso_plan_num_phases': (c_i32, [c_i64]),
    'sso_plan_get_phase': (c_i32, [c_i64, c_i32, c_vp]),
    'sso_plan_num_tasks': (c_i32, [c_i64]),
    'sso_plan_copy_tasks': (c_i32, [c_i64, c_vp, c_i32]),
    'sso_plan_num_diag_recs': (c_i32, [c_i64]),
    'sso_plan_copy_diag_recs': (c_i32, [c_i64, c_vp, c_i32]),
    'sso_plan_num_copy_recs': (c_i32, [c_i64]),
    'sso_plan_copy_copy_recs': (c_i32, [c_i64, c_vp, c_i32]),
    'sso_run_tile_tasks': (c_i32, [c_vp, c_i32, c_i32, c_vp]),
    'sso_optimizer_tail': (c_i32, [c_vp, c_i32, c_vp]),
    'sso_diag_sq_workspace_bytes': (c_sz, [c_i64, c_i64, c_i64]),
    'sso_diag_sq_im2col': (c_i32, [c_vp, c_vp, c_i32] + [c_i64] * 8 + [c_i64] * 5 + [c_i32] * 8 +
                           [c_vp, c_f32, c_f32, c_vp, c_vp, c_vp, c_sz, c_vp]),
}


def lib():
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(LIB_PATH):
                    raise RuntimeError(
                        'libsso_b200.so not found at %s: build it with '
                        '`python pytorch-sso_b200/build.py` (there is no fallback path)' % LIB_PATH)
                handle = C.CDLL(LIB_PATH)
                for name, (res, args) in SIGNATURES.items():
                    fn = getattr(handle, name)       # AttributeError if a symbol is missing
                    fn.restype, fn.argtypes = res, args
                _lib = handle
    return _lib


def _check(rc):
    if rc < 0:
        raise RuntimeError('sso_b200: %s (code %d)' % (lib().sso_last_error().decode(), rc))
    return rc


def _check_status(v):
    if v < 0:
        _check(v)
    return int(v)


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


# ---- optional side stream for the curvature kernels of the hooks -----------------------------
# When enabled, the factor / BatchNorm kernels that the forward and backward hooks launch go to a
# dedicated stream per device, so they overlap with the model's own kernels; whoever consumes
# curvature data joins the stream first (join_curvature_stream).
_curv_streams = {}
_curv_enabled = False
_curv_dirty = set()


def set_curvature_stream(enabled: bool):
    global _curv_enabled
    if not enabled:
        for dev in list(_curv_dirty):
            join_curvature_stream(torch.device('cuda', dev))
    _curv_enabled = bool(enabled)


def curvature_stream_enabled() -> bool:
    return _curv_enabled


def run_on_curvature_stream(fn, tensor: torch.Tensor):
    """fn(tensor) with its kernels on the side stream, ordered after everything already queued on
    the current stream.  `tensor` is kept alive for the side stream (record_stream)."""
    if not _curv_enabled or not tensor.is_cuda:
        return fn(tensor)
    idx = tensor.device.index if tensor.device.index is not None else torch.cuda.current_device()
    side = _curv_streams.get(idx)
    if side is None:
        side = _curv_streams[idx] = torch.cuda.Stream(device=idx)
    side.wait_stream(torch.cuda.current_stream(idx))
    tensor.record_stream(side)
    _curv_dirty.add(idx)
    with torch.cuda.stream(side):
        return fn(tensor)


def join_curvature_stream(device=None):
    """Make the current stream wait for the curvature kernels queued so far (factor problems that
    are still waiting for their batch are launched first)."""
    if _pending:
        flush_factors()
    if not _curv_dirty:
        return
    if device is None or device.index is None:
        idx = torch.cuda.current_device()
    else:
        idx = device.index
    if idx in _curv_dirty:
        torch.cuda.current_stream(idx).wait_stream(_curv_streams[idx])
        _curv_dirty.discard(idx)


def _require_cuda(t: torch.Tensor, what: str):
    if not t.is_cuda:
        raise RuntimeError('%s must live on a CUDA device: the K-FAC kernels have no CPU path' % what)


def configure(key: str, value: int):
    _check(lib().sso_configure(key.encode(), int(value)))


def launch_count() -> int:
    return int(lib().sso_launch_count())


# Optional per-call timing of the factor kernels: set to a list and every factor call appends
# (start_event, end_event, flops, bytes); the benchmark reads it after synchronising.
FACTOR_TIMING = None


def _timed_factor(fn, flops, nbytes):
    if FACTOR_TIMING is None:
        return fn()
    a = torch.cuda.Event(enable_timing=True)
    b = torch.cuda.Event(enable_timing=True)
    a.record()
    fn()
    b.record()
    FACTOR_TIMING.append((a, b, flops, nbytes))


_workspaces = {}
_retired_workspaces = []


def workspace(device, nbytes: int, which: str = '') -> Optional[torch.Tensor]:
    """Per-device scratch, grown on demand and reused (all launches are stream ordered).  A buffer
    that is outgrown is kept until the process ends: captured CUDA graphs hold its raw address.
    `which` names a separate buffer (the batched factor launches have their own)."""
    if nbytes == 0:
        return None
    key = (device.type, device.index) if not which else (device.type, device.index, which)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        if buf is not None:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError('the factor scratch would have to grow during stream capture: run the '
                                   'closure once eagerly before capturing it')
            _retired_workspaces.append(buf)
        buf = torch.empty(int(nbytes * 1.25) + 256, dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def _dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise RuntimeError('unsupported dtype %s (fp32, bf16, fp16 only)' % t.dtype)


def factor_im2col(x: torch.Tensor, kernel_size, stride, padding, dilation, append_ones: bool,
                  sample_weight: Optional[torch.Tensor], alpha: float, beta: float,
                  out: torch.Tensor, impl: int = IMPL_AUTO):
    """out <- alpha * sum_r w u_r u_r^T + beta * out for the im2col rows u_r of x [n,c,h,w]."""
    _require_cuda(x, 'factor input')
    n, c, h, w = x.shape
    kh, kw = kernel_size
    ho = (h + 2 * padding[0] - dilation[0] * (kh - 1) - 1) // stride[0] + 1
    wo = (w + 2 * padding[1] - dilation[1] * (kw - 1) - 1) // stride[1] + 1
    d = c * kh * kw + (1 if append_ones else 0)
    assert out.shape == (d, d) and out.dtype == torch.float32 and out.stride(1) == 1, (out.shape, d)
    rows = n * ho * wo
    L = lib()
    ws = workspace(x.device, L.sso_factor_workspace_bytes(rows, d, impl))
    sn, sc, sh, sw = x.stride()
    _timed_factor(lambda: _check(L.sso_factor_syrk_im2col(
        x.data_ptr(), _dtype_code(x), n, c, h, w, sn, sc, sh, sw, kh, kw, stride[0], stride[1],
        padding[0], padding[1], dilation[0], dilation[1], int(append_ones), _ptr(sample_weight),
        alpha, beta, out.data_ptr(), out.stride(0), _ptr(ws), 0 if ws is None else ws.numel(),
        impl, _stream())), 2.0 * rows * d * d, x.numel() * x.element_size() + 4 * d * d)


def factor_rows(x: torch.Tensor, append_ones: bool, row_weight: Optional[torch.Tensor],
                alpha: float, beta: float, out: torch.Tensor, impl: int = IMPL_AUTO):
    """out <- alpha * [x 1]^T diag(w) [x 1] + beta * out for a 2-D x [rows, cols]."""
    _require_cuda(x, 'factor input')
    rows, cols = x.shape
    d = cols + (1 if append_ones else 0)
    assert out.shape == (d, d) and out.dtype == torch.float32 and out.stride(1) == 1
    L = lib()
    ws = workspace(x.device, L.sso_factor_workspace_bytes(rows, d, impl))
    _timed_factor(lambda: _check(L.sso_factor_syrk(
        x.data_ptr(), _dtype_code(x), rows, cols, x.stride(0), x.stride(1), int(append_ones),
        _ptr(row_weight), alpha, beta, out.data_ptr(), out.stride(0), _ptr(ws),
        0 if ws is None else ws.numel(), impl, _stream())),
        2.0 * rows * d * d, x.numel() * x.element_size() + 4 * d * d)


class FactorOp:
    """A factor-construction call with everything that does not change between steps (geometry,
    strides, scratch size, output slot) resolved once; the hooks run it ~100 times per step, so
    the per-call Python work is kept to pointer look-ups and one foreign call."""

    __slots__ = ('fn', 'mid', 'out_ptr', 'ldo', 'nbytes', 'device', 'impl', 'flops', 'bytes')

    def __init__(self, x: torch.Tensor, kernel_size, stride, padding, dilation, append_ones: bool,
                 out: torch.Tensor, impl: int = IMPL_AUTO):
        _require_cuda(x, 'factor input')
        if x.dim() == 2:        # plain matrix [rows, cols]
            n, c, h, w = x.shape[0], x.shape[1], 1, 1
            sn, sc, sh, sw = x.stride(0), x.stride(1), 0, 0
        else:
            n, c, h, w = x.shape
            sn, sc, sh, sw = x.stride()
        kh, kw = kernel_size
        ho = (h + 2 * padding[0] - dilation[0] * (kh - 1) - 1) // stride[0] + 1
        wo = (w + 2 * padding[1] - dilation[1] * (kw - 1) - 1) // stride[1] + 1
        d = c * kh * kw + (1 if append_ones else 0)
        assert out.shape == (d, d) and out.dtype == torch.float32 and out.stride(1) == 1, (out.shape, d)
        rows = n * ho * wo
        L = lib()
        self.fn = L.sso_factor_syrk_im2col
        self.mid = (_dtype_code(x), n, c, h, w, sn, sc, sh, sw, kh, kw, stride[0], stride[1],
                    padding[0], padding[1], dilation[0], dilation[1], int(append_ones))
        self.out_ptr, self.ldo = out.data_ptr(), out.stride(0)
        self.nbytes = L.sso_factor_workspace_bytes(rows, d, impl)
        self.device, self.impl = x.device, impl
        self.flops = 2.0 * rows * d * d
        self.bytes = x.numel() * x.element_size() + 4 * d * d

    def run(self, x: torch.Tensor, weight: Optional[torch.Tensor], alpha: float, beta: float, defer: bool = True):
        if _batching and defer and weight is None:
            # wait for the other factors of this pass and go to the device with them in one launch
            if self.out_ptr in _pending_outs:
                flush_factors()
            _pending.append((self, x, alpha, beta))
            _pending_outs.add(self.out_ptr)
            return
        ws = workspace(self.device, self.nbytes)
        if FACTOR_TIMING is not None:
            a = torch.cuda.Event(enable_timing=True)
            b = torch.cuda.Event(enable_timing=True)
            a.record()
        rc = self.fn(x.data_ptr(), *self.mid, None if weight is None else weight.data_ptr(), alpha, beta,
                     self.out_ptr, self.ldo, None if ws is None else ws.data_ptr(),
                     0 if ws is None else ws.numel(), self.impl, torch.cuda.current_stream().cuda_stream)
        if rc < 0:
            _check(rc)
        if FACTOR_TIMING is not None:
            b.record()
            FACTOR_TIMING.append((a, b, self.flops, self.bytes))


# ---- batched factor construction -------------------------------------------------------------
# With batching on, the hooks only note their factor problems; flush_factors() sends everything that
# has been noted to the device as ONE call of sso_factor_batch (a persistent tcgen05 kernel over all
# problems plus one finishing kernel).  Flush points: the end of the forward pass and of every backward
# pass inside the Fisher closure, the first backward hook after a forward pass, and any consumer of
# curvature data (join_curvature_stream).  Inputs are kept alive until their batch has been issued; as
# with the curvature stream, the model must not modify a hooked layer's input or output in place.
_batching = False
_pending = []
_pending_outs = set()
_pending_phase = [None]
_batch_cache = {}


def set_factor_batching(enabled: bool):
    global _batching
    if not enabled and _pending:
        flush_factors()
    _batching = bool(enabled)


def factor_batching_enabled() -> bool:
    return _batching


def note_phase(phase: str):
    """Called by the hooks: a backward hook while forward-pass problems are still waiting means the
    forward pass is over, so they are sent off before this pass adds its own."""
    if _pending and _pending_phase[0] != phase:
        flush_factors()
    _pending_phase[0] = phase


def flush_factors():
    if not _pending:
        return
    items = list(_pending)
    _pending.clear()
    _pending_outs.clear()
    L = lib()
    key = tuple(id(op) for op, _, _, _ in items)
    ent = _batch_cache.get(key)
    if ent is None:
        arr = (FactorDesc * len(items))()
        for d, (op, x, alpha, beta) in zip(arr, items):
            (d.dtype, d.n, d.c, d.h, d.w, d.sn, d.sc, d.sh, d.sw, d.kh, d.kw, d.stride_h, d.stride_w,
             d.pad_h, d.pad_w, d.dil_h, d.dil_w, d.append_ones) = op.mid
            d.x, d.sample_weight, d.alpha, d.beta, d.out, d.ldo = x.data_ptr(), None, alpha, beta, op.out_ptr, op.ldo
        nbytes = L.sso_factor_batch_workspace_bytes(len(items), arr)
        if nbytes == 0:
            _check(-1)
        if len(_batch_cache) > 32:
            _batch_cache.pop(next(iter(_batch_cache)))
        ent = (arr, nbytes, [op for op, _, _, _ in items])       # the ops stay alive with their ids
        _batch_cache[key] = ent
    arr, nbytes = ent[0], ent[1]
    for d, (op, x, alpha, beta) in zip(arr, items):
        d.x, d.alpha, d.beta = x.data_ptr(), alpha, beta
    device = items[0][0].device

    def launch(_):
        ws = workspace(device, nbytes, 'batch')
        if FACTOR_TIMING is not None:
            a = torch.cuda.Event(enable_timing=True)
            b = torch.cuda.Event(enable_timing=True)
            a.record()
        _check(L.sso_factor_batch(len(items), arr, ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream))
        if FACTOR_TIMING is not None:
            b.record()
            FACTOR_TIMING.append((a, b, sum(op.flops for op, _, _, _ in items), sum(op.bytes for op, _, _, _ in items)))

    if _curv_enabled:
        idx = device.index if device.index is not None else torch.cuda.current_device()
        side = _curv_streams.get(idx)
        if side is None:
            side = _curv_streams[idx] = torch.cuda.Stream(device=idx)
        side.wait_stream(torch.cuda.current_stream(idx))
        for _, x, _, _ in items:
            x.record_stream(side)
        _curv_dirty.add(idx)
        with torch.cuda.stream(side):
            launch(None)
    else:
        launch(None)


def _plane_strides(t: torch.Tensor):
    """(n, c, hw) element strides of a [n,c] or [n,c,h,w] tensor whose (h,w) plane is
    addressable with one stride; returns None if it is not."""
    if t.dim() == 2:
        return t.stride(0), t.stride(1), 0
    n, c, h, w = t.shape
    sn, sc, sh, sw = t.stride()
    if h == 1 or sh == w * sw:
        return sn, sc, sw
    return None


def bn_plane_layout(t: torch.Tensor):
    """(tensor to pass, (n, c, hw) element strides, split count) for a [n,c] / [n,c,h,w] tensor."""
    st = _plane_strides(t)
    if st is None:
        t = t.contiguous()
        st = _plane_strides(t)
    n, c = t.shape[0], t.shape[1]
    hw = t.numel() // (n * c)
    splits = lib().sso_bn_plane_splits(_dtype_code(t), n, c, hw, st[1]) if hw > 1 else 1
    ok = (st[1] == 1 and t.data_ptr() % 16 == 0 and (st[0] * t.element_size()) % 16 == 0
          and (st[2] * t.element_size()) % 16 == 0)
    return t, st, (splits if ok else 1)


def bn_plane_sums(t: torch.Tensor, is_output: bool, scale, shift, out: torch.Tensor, layout=None) -> int:
    """out[n, splits, c] <- per-plane sums of squares of t (normalised with scale/shift when it
    is the layer output); returns the split count that was used."""
    _require_cuda(t, 'batch-norm tensor')
    t, st, splits = layout if layout is not None else bn_plane_layout(t)
    n, c = t.shape[0], t.shape[1]
    hw = t.numel() // (n * c)
    assert out.numel() >= n * splits * c
    if is_output:
        _check(lib().sso_bn_plane_sums(t.data_ptr(), None, _dtype_code(t), n, c, hw, *st, 0, 0, 0,
                                       _ptr(scale), _ptr(shift), out.data_ptr(), None, splits, _stream()))
    else:
        _check(lib().sso_bn_plane_sums(None, t.data_ptr(), _dtype_code(t), n, c, hw, 0, 0, 0, *st,
                                       None, None, None, out.data_ptr(), splits, _stream()))
    return splits


def bn_diag_finish(sx, sg, sample_weight, n, c, splits_x, splits_g, alpha, beta, w_out, b_out):
    _check(lib().sso_bn_diag_finish(sx.data_ptr(), sg.data_ptr(), _ptr(sample_weight), n, c, splits_x,
                                    splits_g, alpha, beta, w_out.data_ptr(), _ptr(b_out), _stream()))


def diag_sq(x: torch.Tensor, g: torch.Tensor, kernel_size, stride, padding, dilation,
            sample_weight: Optional[torch.Tensor], alpha: float, beta: float,
            out_w: torch.Tensor, out_b: Optional[torch.Tensor]):
    """out_w <- alpha * sum_b w_b (per-sample weight gradient of sample b)^2 + beta * out_w (and the
    same for the bias) for a convolution with input x [n,c,h,w] and output gradient g [n,oc,ho,wo];
    a Linear layer passes x [n,f_in], g [n,f_out]."""
    _require_cuda(x, 'layer input')
    if x.dim() == 2:
        x, g = x[:, :, None, None], g[:, :, None, None]
        kernel_size, stride, padding, dilation = (1, 1), (1, 1), (0, 0), (1, 1)
    if g.dtype != x.dtype:
        x, g = x.float(), g.float()
    n, c, h, w = x.shape
    oc = g.shape[1]
    d = c * kernel_size[0] * kernel_size[1]
    assert out_w.is_contiguous() and out_w.dtype == torch.float32 and out_w.numel() == oc * d
    assert out_b is None or (out_b.is_contiguous() and out_b.numel() == oc)
    assert sample_weight is None or (sample_weight.dtype == torch.float32 and sample_weight.is_contiguous()
                                     and sample_weight.numel() == n)
    L = lib()
    ws = workspace(x.device, L.sso_diag_sq_workspace_bytes(n, oc, d))
    _check(L.sso_diag_sq_im2col(x.data_ptr(), g.data_ptr(), _dtype_code(x), n, c, h, w, *x.stride(), oc,
                                *g.stride(), kernel_size[0], kernel_size[1], stride[0], stride[1],
                                padding[0], padding[1], dilation[0], dilation[1], _ptr(sample_weight),
                                alpha, beta, out_w.data_ptr(), _ptr(out_b), _ptr(ws),
                                0 if ws is None else ws.numel(), _stream()))


def ema_update(data: torch.Tensor, ema: torch.Tensor, beta: float, first: bool):
    _require_cuda(data, 'curvature data')
    assert data.is_contiguous() and ema.is_contiguous() and data.numel() == ema.numel()
    _check(lib().sso_ema_update(data.data_ptr(), ema.data_ptr(), data.numel(), beta, int(first), _stream()))


def axpby(src: torch.Tensor, dst: torch.Tensor, a: float, b: float):
    _require_cuda(src, 'tensor')
    assert src.is_contiguous() and dst.is_contiguous() and src.numel() == dst.numel()
    assert src.dtype == torch.float32 and dst.dtype == torch.float32
    _check(lib().sso_axpby(src.data_ptr(), dst.data_ptr(), src.numel(), a, b, _stream()))


def diag_inv_precondition(ema, inv, grad, damping: float, use_sqrt: bool, update_inv: bool):
    _require_cuda(inv, 'diagonal curvature')
    _check(lib().sso_diag_inv_precondition(_ptr(ema), inv.data_ptr(), _ptr(grad), inv.numel(), damping,
                                           int(use_sqrt), int(update_inv), _stream()))


def tri_records(mats: Sequence[torch.Tensor], packed: torch.Tensor, offsets: Sequence[int],
                rows_per_rec: int = 0) -> torch.Tensor:
    """Device table of row runs for sso_tri_pack / sso_tri_unpack."""
    recs = []
    for m, off in zip(mats, offsets):
        n = m.shape[0]
        step = rows_per_rec or max(1, 16384 // n)
        for r0 in range(0, n, step):
            recs.append((m.data_ptr(), packed.data_ptr() + 4 * off, n, m.stride(0), r0, min(step, n - r0)))
    arr = np.array(recs, dtype=TRI_REC_DTYPE)
    return torch.from_numpy(arr.view(np.uint8).copy()).to(packed.device)


def tri_pack(table: torch.Tensor, scale: float = 1.0):
    _check(lib().sso_tri_pack(table.data_ptr(), table.numel() // TRI_REC_DTYPE.itemsize, scale, _stream()))


def tri_unpack(table: torch.Tensor, scale: float = 1.0, symmetric: bool = True):
    _check(lib().sso_tri_unpack(table.data_ptr(), table.numel() // TRI_REC_DTYPE.itemsize, scale,
                                int(symmetric), _stream()))


SEG_REC_DTYPE = np.dtype([('src', np.uint64), ('dst', np.uint64), ('count', np.int64)])


def seg_records(pairs, device, chunk: int = 1 << 14) -> torch.Tensor:
    """Device table for sso_copy_segments from (src, dst) pairs of equal-sized flat fp32 tensors."""
    recs = []
    for src, dst in pairs:
        assert src.numel() == dst.numel() and src.is_contiguous() and dst.is_contiguous()
        assert src.dtype == torch.float32 and dst.dtype == torch.float32
        n = src.numel()
        for o in range(0, n, chunk):
            recs.append((src.data_ptr() + 4 * o, dst.data_ptr() + 4 * o, min(chunk, n - o)))
    arr = np.array(recs, dtype=SEG_REC_DTYPE)
    return torch.from_numpy(arr.view(np.uint8).copy()).to(device)


TAIL_REC_DTYPE = np.dtype([('p', np.uint64), ('g', np.uint64), ('mbuf', np.uint64), ('ebuf', np.uint64),
                           ('count', np.int64), ('add', np.float32), ('momentum', np.float32),
                           ('ema', np.float32), ('scale', np.float32), ('lr', np.float32), ('pad', np.int32)])


def tail_records(items, device, chunk: int = 1 << 15) -> torch.Tensor:
    """Device table for sso_optimizer_tail from (p, g, mbuf, ebuf, add, momentum, ema, scale, lr)
    tuples of flat, equally laid out fp32 tensors (mbuf / ebuf may be None)."""
    recs = []
    for p, g, mbuf, ebuf, add, momentum, ema, scale, lr in items:
        n = p.numel()
        for o in range(0, n, chunk):
            recs.append((p.data_ptr() + 4 * o, g.data_ptr() + 4 * o,
                         0 if mbuf is None else mbuf.data_ptr() + 4 * o,
                         0 if ebuf is None else ebuf.data_ptr() + 4 * o,
                         min(chunk, n - o), add, momentum, ema, scale, lr, 0))
    arr = np.array(recs, dtype=TAIL_REC_DTYPE)
    return torch.from_numpy(arr.view(np.uint8).copy()).to(device)


def optimizer_tail(table: torch.Tensor):
    _check(lib().sso_optimizer_tail(table.data_ptr(), table.numel() // TAIL_REC_DTYPE.itemsize, _stream()))


def copy_segments(table: torch.Tensor, scale: float = 1.0):
    _check(lib().sso_copy_segments(table.data_ptr(), table.numel() // SEG_REC_DTYPE.itemsize, scale, _stream()))


WIRE_REC_DTYPE = np.dtype([('offset', np.int64), ('count', np.int64), ('array', np.int32), ('pad', np.int32)])


def wire_records(offsets, counts, device, ids=None, chunk: int = 1 << 13) -> torch.Tensor:
    """Device table for the sso_wire_* kernels: array ids[i] (default i) occupies
    [offsets[i], offsets[i] + counts[i]) of the packed buffer."""
    recs = []
    for i, (off, n) in enumerate(zip(offsets, counts)):
        for o in range(0, n, chunk):
            recs.append((off + o, min(chunk, n - o), i if ids is None else ids[i], 0))
    arr = np.array(recs, dtype=WIRE_REC_DTYPE)
    return torch.from_numpy(arr.view(np.uint8).copy()).to(device)


def wire_absmax(buf: torch.Tensor, table: torch.Tensor, maxima: torch.Tensor):
    _check(lib().sso_wire_absmax(buf.data_ptr(), table.data_ptr(), table.numel() // WIRE_REC_DTYPE.itemsize,
                                 maxima.data_ptr(), _stream()))


def wire_encode(buf: torch.Tensor, table: torch.Tensor, sums: torch.Tensor, out16: torch.Tensor):
    _check(lib().sso_wire_encode(buf.data_ptr(), table.data_ptr(), table.numel() // WIRE_REC_DTYPE.itemsize,
                                 sums.data_ptr(), out16.data_ptr(), _dtype_code(out16), _stream()))


def wire_decode(in16: torch.Tensor, table: torch.Tensor, sums: torch.Tensor, out32: torch.Tensor):
    _check(lib().sso_wire_decode(in16.data_ptr(), table.data_ptr(), table.numel() // WIRE_REC_DTYPE.itemsize,
                                 sums.data_ptr(), out32.data_ptr(), _dtype_code(in16), _stream()))


def _i64(vals):
    return (c_i64 * len(vals))(*[int(v) for v in vals])


def _i32(vals):
    return (C.c_int32 * len(vals))(*[int(v) for v in vals])


def _ptrs(tensors):
    return (c_vp * len(tensors))(*[None if t is None else (t if isinstance(t, int) else t.data_ptr())
                                   for t in tensors])


class Plan:
    """Owner of one engine plan (handle + the device memory that holds its tables)."""

    def __init__(self, handle: int, dev_mem: Optional[torch.Tensor], keep):
        if handle <= 0:
            _check(int(handle))
        self.handle = handle
        self._dev_mem = dev_mem
        self._keep = keep          # tensors whose addresses are baked into the plan

    def __del__(self):
        try:
            if self.handle > 0 and _lib is not None:
                _lib.sso_plan_destroy(self.handle)
        except Exception:
            pass

    def status(self) -> int:
        """0, or the code of the first device-side wait of a tensor-core tile task that gave up in any
        run of this plan so far (synchronises; the tiles of such a task were written as NaN)."""
        return _check_status(lib().sso_plan_status(self.handle))

    # introspection (host side)
    def phases(self):
        L = lib()
        out = []
        for i in range(_check(L.sso_plan_num_phases(self.handle))):
            ph = Phase()
            _check(L.sso_plan_get_phase(self.handle, i, C.byref(ph)))
            out.append((ph.kind, ph.first, ph.count))
        return out

    def tasks(self):
        L = lib()
        n = _check(L.sso_plan_num_tasks(self.handle))
        arr = (TileTask * max(n, 1))()
        _check(L.sso_plan_copy_tasks(self.handle, arr, n))
        return arr, n

    def diag_recs(self):
        L = lib()
        n = _check(L.sso_plan_num_diag_recs(self.handle))
        arr = (DiagRec * max(n, 1))()
        _check(L.sso_plan_copy_diag_recs(self.handle, arr, n))
        return arr, n

    def copy_recs(self):
        L = lib()
        n = _check(L.sso_plan_num_copy_recs(self.handle))
        arr = (CopyRec * max(n, 1))()
        _check(L.sso_plan_copy_copy_recs(self.handle, arr, n))
        return arr, n


def _lds(*lists):
    """Leading dimensions (row strides) shared by the matrices at the same position of every list,
    or None when the entries are raw addresses (dense matrices assumed)."""
    first = lists[0]
    if not all(isinstance(m, torch.Tensor) for lst in lists if lst is not None for m in lst):
        return None
    out = []
    for i, m in enumerate(first):
        ld = m.stride(0) if m.dim() == 2 and m.shape[0] > 1 else m.shape[-1]
        for lst in lists[1:]:
            if lst is not None:
                o = lst[i]
                assert o.stride(-1) == 1 and (o.shape[0] == 1 or o.stride(0) == ld), 'matrices of one factor must share their leading dimension'
        out.append(ld)
    return _i64(out)


def kron_plan(dims, src, dst, work, std, partner, role, device, host_only=False, lds=None) -> Plan:
    L = lib()
    n = len(dims)
    d = _i64(dims)
    nbytes = L.sso_kron_plan_dev_bytes(n, d, int(std is not None))
    host_mem = None
    if host_only:
        # the plan's scratch matrices (the head of its memory block) must exist for a host-side
        # interpreter of the program; the tables behind them are not uploaded
        import numpy as np
        host_mem = np.full(nbytes // 4 + 64, np.nan, dtype=np.float32)
        mem = None
        mem_ptr = host_mem.ctypes.data
    else:
        mem = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=device)
        mem_ptr = mem.data_ptr()
    h = L.sso_kron_plan_create(n, d, _ptrs(src), _ptrs(dst), _ptrs(work),
                               None if std is None else _ptrs(std), _i32(partner), _i32(role),
                               mem_ptr, nbytes, int(host_only), _i64(lds) if lds is not None else _lds(src, dst, work, std))
    plan = Plan(h, mem, (src, dst, work, std, host_mem))
    plan.host_mem = host_mem
    return plan


def kron_plan_run(plan: Plan, damp_r: torch.Tensor, info: Optional[torch.Tensor], do_inverse: bool,
                  do_std: bool):
    _check(lib().sso_kron_plan_run(plan.handle, _ptr(damp_r), _ptr(info), int(do_inverse), int(do_std),
                                   _stream()))


def precond_plan(dA, dG, A_inv, G_inv, gw, gb, tmp, device, host_only=False) -> Plan:
    L = lib()
    n = len(dA)
    a, g = _i64(dA), _i64(dG)
    nbytes = L.sso_precond_plan_dev_bytes(n, a, g)
    mem = None if host_only else torch.empty(max(nbytes, 256), dtype=torch.uint8, device=device)
    h = L.sso_precond_plan_create(n, a, g, _ptrs(A_inv), _ptrs(G_inv), _ptrs(gw), _ptrs(gb), _ptrs(tmp),
                                  _ptr(mem), nbytes, int(host_only), _lds(A_inv), _lds(G_inv))
    return Plan(h, mem, (A_inv, G_inv, gw, gb, tmp))


def precond_plan_run(plan: Plan):
    _check(lib().sso_precond_plan_run(plan.handle, _stream()))


def sample_plan(dA, dG, U_A, U_G, noise, w, b, tmp, device, host_only=False) -> Plan:
    L = lib()
    n = len(dA)
    a, g = _i64(dA), _i64(dG)
    nbytes = L.sso_sample_plan_dev_bytes(n, a, g)
    mem = None if host_only else torch.empty(max(nbytes, 256), dtype=torch.uint8, device=device)
    h = L.sso_sample_plan_create(n, a, g, _ptrs(U_A), _ptrs(U_G), _ptrs(noise), _ptrs(w), _ptrs(b),
                                 _ptrs(tmp), _ptr(mem), nbytes, int(host_only), _lds(U_A), _lds(U_G))
    return Plan(h, mem, (U_A, U_G, noise, w, b, tmp))


def sample_plan_run(plan: Plan, std_scale: float):
    _check(lib().sso_sample_plan_run(plan.handle, std_scale, _stream()))
