"""Thin tensor-level wrappers over the C ABI: validate, allocate outputs, launch on the
current stream.  No arithmetic happens in Python.  Shapes follow the reference's pybind
entry points (src/convlogic/cuda/convlogic.cpp:29-44, src/difflogic/cuda/difflogic.cpp:15-34).
"""

import ctypes as C

import numpy as np
import torch

from . import _lib
from ._lib import check, check_input, dtype_code, lib, ptr, stream


def _geom(stride, padding, kernel):
    return (*stride, *padding, *kernel)


def _out_hw(h, w, sh, sw, ph, pw, kh, kw):
    return (h + 2 * ph - kh) // sh + 1, (w + 2 * pw - kw) // sw + 1


def _sel_ok(sel, c):
    if sel.dtype != torch.int32 or sel.shape != (c, 8):
        raise RuntimeError(f"convlogic_b200: selection must be int32 [{c}, 8], got {sel.dtype} {tuple(sel.shape)}")


def _sel_flag(sel, geom, ci):
    """SEL_UNBOUNDED when some tap lies outside the kh x kw window; raises when a tap names a channel the input
    does not have (the kernels index with it).  Checked once per selection tensor, in-place version and channel
    count; the result is cached on the tensor object."""
    key = (sel._version, geom[4], geom[5], ci)
    cache = getattr(sel, "_clb_window", None)
    if cache is None or cache[0] != key:
        inside, ch_ok = True, True
        if sel.numel():
            rows, cols, chans = (sel >> 8) & 0xFF, sel & 0xFF, (sel >> 16) & 0xFFFF
            flags = torch.stack([rows.max() < geom[4], cols.max() < geom[5], (chans.max() < ci) & (sel.min() >= 0)]).tolist()
            inside, ch_ok = flags[0] and flags[1], flags[2]
        cache = (key, 0 if inside else _lib.SEL_UNBOUNDED, ch_ok)
        sel._clb_window = cache
    if not cache[2]:
        raise RuntimeError("convlogic_b200: selection refers to a channel the input does not have")
    return cache[1]


# ------------------------------------------------------------------------------ fused block
def _is_feature_major(t):
    """A 4-D [N, C, h, w] tensor whose storage is the contiguous [C, h, w, N] one (what ``convtree_fwd`` returns with
    ``y_feature_major`` and what autograd hands back through the flat layers' transposed views)."""
    return t.dim() == 4 and not t.is_contiguous() and t.permute(1, 2, 3, 0).is_contiguous()


def convtree_fwd(x, w, sel, geom, wmode, want_amax=True, want_intermediate=False, want_indices=False, y_feature_major=False):
    """``y_feature_major``: ask for the output in the flat layers' layout -- storage [C, h, w, N], returned as the
    [N, C, h, w] view of it, so that ``flatten(1)`` and the flat layers' transposition are views.  Only the plane
    kernels write it; for other shapes the ordinary layout comes back."""
    check_input(x, w, sel)
    n, ci, h, wd = x.shape
    c = w.shape[0]
    if w.shape != (c, 7, 16) or w.dtype != x.dtype:
        raise RuntimeError(f"convlogic_b200: gate tensor must be [{c}, 7, 16] {x.dtype}")
    _sel_ok(sel, c)
    ho, wo = _out_hw(h, wd, *geom)
    if ho <= 0 or wo <= 0:
        raise RuntimeError(f"Invalid output shape: H_out={ho}, W_out={wo}")
    if ho % 2 or wo % 2:
        raise RuntimeError(
            "Output height and width after convolution must be divisible by 2 for 2x2 max pooling, "
            f"but got H_out={ho}, W_out={wo}")
    y = torch.empty((n, c, ho // 2, wo // 2), dtype=x.dtype, device=x.device)
    amax = torch.empty((n, c, ho // 2, wo // 2), dtype=torch.uint8, device=x.device) if want_amax else None
    x2 = x3 = idx = None
    if want_intermediate:
        x2 = torch.empty((n, c, ho, wo, 4), dtype=x.dtype, device=x.device)
        x3 = torch.empty((n, c, ho, wo, 2), dtype=x.dtype, device=x.device)
    if want_indices:
        idx = torch.empty((n, c, (ho // 2) * (wo // 2)), dtype=torch.int32, device=x.device)
    if n == 0 or c == 0:  # empty batch: nothing to launch
        return y, amax, x2, x3, idx
    if y_feature_major and x.dtype == torch.float32 and not want_intermediate and not want_indices and not _sel_flag(sel, geom, ci):
        y_fm = torch.empty((c, ho // 2, wo // 2, n), dtype=x.dtype, device=x.device)
        rc = lib().clb_convtree_fwd(ptr(x), ptr(w), ptr(sel), ptr(y_fm), ptr(amax), None, None, None, n, ci, h, wd, c, *geom,
                                    wmode | _lib.Y_FEATURE_MAJOR, dtype_code(x), stream())
        if rc != _lib.ERR_SHAPE:
            check(rc)
            return y_fm.permute(3, 0, 1, 2), amax, x2, x3, idx
    check(lib().clb_convtree_fwd(ptr(x), ptr(w), ptr(sel), ptr(y), ptr(amax), ptr(x2), ptr(x3), ptr(idx),
                                 n, ci, h, wd, c, *geom, wmode | _sel_flag(sel, geom, ci), dtype_code(x), stream()))
    return y, amax, x2, x3, idx


def conv_groups(sel, x_shape, geom, dtype):
    """Device tables for the input-gradient kernels.  They depend only on the selection tensor and
    the shapes, so they are cached ON the selection tensor object (keyed by its in-place version
    counter): no global state that could outlive the tensor and be matched by a recycled address."""
    n, ci, h, w = x_shape
    c = sel.shape[0]
    key = (sel._version, n, ci, h, w, c, geom, dtype)
    cache = getattr(sel, "_clb_groups", None)
    if cache is None:
        cache = {}
        sel._clb_groups = cache
    hit = cache.get(key)
    if hit is not None:
        return hit
    cg, nb = C.c_int(0), C.c_int(0)
    check(lib().clb_conv_group_plan(n, ci, h, w, c, *geom, _lib.F32 if dtype == torch.float32 else _lib.F64,
                                    C.byref(cg), C.byref(nb)))
    cg, nb = cg.value, nb.value
    g = -(-ci // cg)
    sel_host = np.ascontiguousarray(sel.detach().cpu().numpy(), dtype=np.int32)
    start = np.zeros(g + 1, dtype=np.int32)
    cap = max(1, c * min(g, 8))
    lst = np.zeros(cap, dtype=np.int32)
    cnt = lib().clb_conv_build_groups(sel_host.ctypes.data_as(C.c_void_p), c, ci, cg,
                                      start.ctypes.data_as(C.c_void_p), lst.ctypes.data_as(C.c_void_p), cap)
    if cnt < 0:
        if cnt == -1:
            raise RuntimeError("convlogic_b200: selection refers to a channel the input does not have")
        check(cnt)
    out = (torch.from_numpy(start).to(sel.device), torch.from_numpy(lst[:max(cnt, 1)].copy()).to(sel.device), cg, nb)
    if len(cache) > 16:
        cache.clear()
    cache[key] = out
    return out


def plane_lists(sel, ci, geom):
    """Per input channel, the (output channel, slot) gradient planes that belong to it -- the tables of
    ``clb_convtree_bwd_plane`` -- or None when the selection does not fit those kernels (an output channel with more
    than two input channels, or taps outside the window).  Cached on the selection tensor like ``conv_groups``."""
    key = (sel._version, ci, geom[4], geom[5])
    cache = getattr(sel, "_clb_planes", None)
    if cache is not None and cache[0] == key:
        return cache[1]
    c = sel.shape[0]
    sel_host = np.ascontiguousarray(sel.detach().cpu().numpy(), dtype=np.int32)
    start = np.zeros(ci + 1, dtype=np.int32)
    entry = np.zeros(max(2 * c, 1), dtype=np.int32)
    cnt = lib().clb_conv_channel_lists(sel_host.ctypes.data_as(C.c_void_p), c, ci, geom[4], geom[5],
                                       start.ctypes.data_as(C.c_void_p), entry.ctypes.data_as(C.c_void_p), entry.size)
    out = None
    if cnt >= 0:
        out = (torch.from_numpy(start).to(sel.device), torch.from_numpy(entry[:max(cnt, 1)].copy()).to(sel.device))
    elif cnt != _lib.ERR_SHAPE:
        check(cnt)
    sel._clb_planes = (key, out)
    return out


def _bwd_args_ok(gy, x, w, sel, amax, geom):
    """Shapes and dtypes of the fused block's backward inputs (the C ABI receives bare pointers)."""
    n, ci, h, wd = x.shape
    c = w.shape[0]
    _sel_ok(sel, c)
    ho, wo = _out_hw(h, wd, *geom)
    want = (n, c, ho // 2, wo // 2)
    if w.shape != (c, 7, 16) or w.dtype != x.dtype:
        raise RuntimeError(f"convlogic_b200: gate tensor must be [{c}, 7, 16] {x.dtype}")
    if tuple(gy.shape) != want or gy.dtype != x.dtype:
        raise RuntimeError(f"convlogic_b200: upstream gradient must be {want} {x.dtype}, got {tuple(gy.shape)} {gy.dtype}")
    if amax is not None and (tuple(amax.shape) != want or amax.dtype != torch.uint8):
        raise RuntimeError(f"convlogic_b200: arg-max tensor must be uint8 {want}, got {tuple(amax.shape)} {amax.dtype}")


def convtree_bwd_x(gy, x, w, sel, amax, geom, wmode, use_scratch=True):
    check_input(gy, x, w, sel)
    _bwd_args_ok(gy, x, w, sel, amax, geom)
    n, ci, h, wd = x.shape
    c = w.shape[0]
    gx = torch.empty_like(x)
    flag = _sel_flag(sel, geom, ci)
    nbytes = lib().clb_convtree_bwd_x_scratch_bytes(n, ci, h, wd, c, *geom, dtype_code(x)) if (use_scratch and not flag) else 0
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=x.device) if nbytes else None
    start, lst, cg, nb = conv_groups(sel, tuple(x.shape), geom, x.dtype)
    check(lib().clb_convtree_bwd_x(ptr(gy), ptr(x), ptr(w), ptr(sel), ptr(amax), ptr(gx), ptr(start), ptr(lst),
                                   cg, nb, ptr(scratch), nbytes, n, ci, h, wd, c, *geom, wmode | flag, dtype_code(x),
                                   stream()))
    return gx


def convtree_bwd(gy, x, w, sel, amax, geom, wmode, need_gx=True, need_gw=True, gw_out=None):
    """Both gradients of the fused block in one C-ABI call; returns (gx or None, gw or None).  ``gw_out``: a contiguous
    tensor of the gate tensor's shape to receive the gate gradient (e.g. a slice of a flat gradient bucket).  ``gy`` may
    be feature-major (see ``convtree_fwd``): the plane kernels read it as it is, other shapes get a contiguous copy."""
    gy_fm = gy.is_cuda and _is_feature_major(gy)
    check_input(x, w, sel) if gy_fm else check_input(gy, x, w, sel)
    _bwd_args_ok(gy, x, w, sel, amax, geom)
    n, ci, h, wd = x.shape
    c = w.shape[0]
    gx = torch.empty_like(x) if need_gx else None
    gw = None
    if need_gw:
        gw = torch.empty_like(w) if gw_out is None else gw_out
        if gw.shape != w.shape or gw.dtype != w.dtype or not gw.is_contiguous():
            raise RuntimeError("convlogic_b200: `gw_out` must be contiguous with the gate tensor's shape and dtype")
    if n == 0 or c == 0:  # empty batch: the gate gradient is an empty sum
        return gx, (gw.zero_() if gw is not None else None)
    flag = _sel_flag(sel, geom, ci)
    if not flag and x.dtype == torch.float32 and amax is not None:
        # The plane kernels (two channel planes per output channel streamed through shared memory): both gradients of the
        # many-channel layers (16x16 .. 4x4 images), the gate gradient alone of a 32x32 first block.
        nbytes = lib().clb_convtree_bwd_plane_scratch_bytes(n, ci, h, wd, c, *geom, dtype_code(x))
        lists = plane_lists(sel, ci, geom) if nbytes else None
        if lists is not None:
            scratch = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=x.device)
            rc = lib().clb_convtree_bwd_plane(ptr(gy), ptr(x), ptr(w), ptr(sel), ptr(amax), ptr(gx), ptr(gw), ptr(lists[0]), ptr(lists[1]),
                                              ptr(scratch), nbytes, n, ci, h, wd, c, *geom, wmode | (_lib.Y_FEATURE_MAJOR if gy_fm else 0),
                                              dtype_code(x), stream())
            if rc != _lib.ERR_SHAPE:
                check(rc)
                return gx, gw
    if gy_fm:
        gy = gy.contiguous()
    nbytes = lib().clb_convtree_bwd_scratch_bytes(n, ci, h, wd, c, *geom, int(need_gx), int(need_gw), dtype_code(x))
    scratch = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=x.device)
    if need_gx:
        start, lst, cg, nb = conv_groups(sel, tuple(x.shape), geom, x.dtype)
    else:
        start = lst = None
        cg = nb = 1
    check(lib().clb_convtree_bwd(ptr(gy), ptr(x), ptr(w), ptr(sel), ptr(amax), ptr(gx), ptr(gw), ptr(start), ptr(lst),
                                 cg, nb, ptr(scratch), nbytes, n, ci, h, wd, c, *geom, wmode | flag, dtype_code(x), stream()))
    return gx, gw


def convtree_bwd_w(gy, x, w, sel, amax, geom, wmode):
    check_input(gy, x, w, sel)
    _bwd_args_ok(gy, x, w, sel, amax, geom)
    n, ci, h, wd = x.shape
    _sel_flag(sel, geom, ci)
    c = w.shape[0]
    ho, wo = _out_hw(h, wd, *geom)
    gw = torch.empty_like(w)
    nbytes = lib().clb_convtree_bwd_w_scratch_bytes(n, c, ho, wo, dtype_code(x))
    scratch = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=x.device)
    check(lib().clb_convtree_bwd_w(ptr(gy), ptr(x), ptr(w), ptr(sel), ptr(amax), ptr(gw), ptr(scratch), nbytes,
                                   n, ci, h, wd, c, *geom, wmode, dtype_code(x), stream()))
    return gw


def convtree_bwd_w_noalloc(gy, x, w, sel, amax, geom, wmode, out):
    """Gate gradient of the fused block written into the caller's ``out`` ([C, 7, 16]) without
    any allocation on the way: the kernels' partial sums go to a fixed array inside the library
    instead of a scratch tensor.  For callers that may not allocate (inside a memory-planned or
    pre-allocated region).  Raises ValueError when the shape needs more than that array holds.
    All calls on a device share the array, so do not let two of them overlap on the GPU; make the
    first call on a device outside any stream capture (it looks the array's address up once)."""
    check_input(gy, x, w, sel, out)
    _bwd_args_ok(gy, x, w, sel, amax, geom)
    n, ci, h, wd = x.shape
    _sel_flag(sel, geom, ci)
    c = w.shape[0]
    if out.shape != w.shape or out.dtype != w.dtype:
        raise RuntimeError("convlogic_b200: `out` must have the gate tensor's shape and dtype")
    check(lib().clb_convtree_bwd_w_noalloc(ptr(gy), ptr(x), ptr(w), ptr(sel), ptr(amax), ptr(out),
                                           n, ci, h, wd, c, *geom, wmode, dtype_code(x), stream()))
    return out


# --------------------------------------------------------------------- stand-alone first level
def conv_fwd(x, w, sel, geom, wmode):
    check_input(x, w, sel)
    n, ci, h, wd = x.shape
    c = w.shape[0]
    if w.shape != (c, 4, 16) or w.dtype != x.dtype:
        raise RuntimeError(f"convlogic_b200: gate tensor must be [{c}, 4, 16] {x.dtype}")
    _sel_ok(sel, c)
    ho, wo = _out_hw(h, wd, *geom)
    if ho <= 0 or wo <= 0:
        raise RuntimeError(f"Invalid output shape: H_out={ho}, W_out={wo}")
    _sel_flag(sel, geom, ci)
    y = torch.empty((n, c, ho, wo, 4), dtype=x.dtype, device=x.device)
    check(lib().clb_conv_fwd(ptr(x), ptr(w), ptr(sel), ptr(y), n, ci, h, wd, c, *geom, wmode, dtype_code(x), stream()))
    return y


def conv_bwd_x(gy, x, w, sel, geom, wmode):
    check_input(gy, x, w, sel)
    n, ci, h, wd = x.shape
    c = w.shape[0]
    gx = torch.empty_like(x)
    start, lst, cg, nb = conv_groups(sel, tuple(x.shape), geom, x.dtype)
    check(lib().clb_conv_bwd_x(ptr(gy), ptr(x), ptr(w), ptr(sel), ptr(gx), ptr(start), ptr(lst), cg, nb,
                               n, ci, h, wd, c, *geom, wmode, dtype_code(x), stream()))
    return gx


def conv_bwd_w(gy, x, w, sel, geom, wmode):
    check_input(gy, x, w, sel)
    n, ci, h, wd = x.shape
    c = w.shape[0]
    ho, wo = _out_hw(h, wd, *geom)
    gw = torch.empty_like(w)
    nbytes = lib().clb_conv_bwd_w_scratch_bytes(n, c, ho, wo, dtype_code(x))
    scratch = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=x.device)
    check(lib().clb_conv_bwd_w(ptr(gy), ptr(x), ptr(w), ptr(sel), ptr(gw), ptr(scratch), nbytes,
                               n, ci, h, wd, c, *geom, wmode, dtype_code(x), stream()))
    return gw


# -------------------------------------------------------------------------------- tree level
def _tree_dims(x, w):
    if x.dim() != 5:
        raise RuntimeError(f"Expected input tensor x to be 5D (N, C, H, W, 2*Xout), but got {x.dim()}")
    n, c, h, wd, xin = x.shape
    xo = w.shape[1]
    if xin != 2 * xo:
        raise RuntimeError(f"Expected input x.size(4) (Xin) to equal 2*Xout ({2 * xo}), but got {xin}")
    if w.shape != (c, xo, 16) or w.dtype != x.dtype:
        raise RuntimeError(f"convlogic_b200: gate tensor must be [{c}, {xo}, 16] {x.dtype}")
    return n, c, h * wd, xo


def tree_fwd(x, w, wmode):
    check_input(x, w)
    n, c, hw, xo = _tree_dims(x, w)
    y = torch.empty((*x.shape[:4], xo), dtype=x.dtype, device=x.device)
    check(lib().clb_tree_fwd(ptr(x), ptr(w), ptr(y), n, c, hw, xo, wmode, dtype_code(x), stream()))
    return y


def tree_bwd_x(gy, x, w, wmode):
    check_input(gy, x, w)
    n, c, hw, xo = _tree_dims(x, w)
    gx = torch.empty_like(x)
    check(lib().clb_tree_bwd_x(ptr(gy), ptr(x), ptr(w), ptr(gx), n, c, hw, xo, wmode, dtype_code(x), stream()))
    return gx


def tree_bwd_w(gy, x, w, wmode):
    check_input(gy, x, w)
    n, c, hw, xo = _tree_dims(x, w)
    gw = torch.empty_like(w)
    nbytes = lib().clb_tree_bwd_w_scratch_bytes(n, c, hw, xo, dtype_code(x))
    scratch = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=x.device)
    check(lib().clb_tree_bwd_w(ptr(gy), ptr(x), ptr(w), ptr(gw), ptr(scratch), nbytes, n, c, hw, xo, wmode,
                               dtype_code(x), stream()))
    return gw


# -------------------------------------------------------------------------------- flat layer
def _logic_dims(x, a, b, w):
    if x.dim() != 2:
        raise RuntimeError(f"convlogic_b200: x must be [in_dim, batch], got {tuple(x.shape)}")
    out = w.shape[0]
    if w.shape != (out, 16) or w.dtype != x.dtype:
        raise RuntimeError(f"convlogic_b200: gate tensor must be [{out}, 16] {x.dtype}")
    if a.dtype != torch.int64 or b.dtype != torch.int64 or a.shape != (out,) or b.shape != (out,):
        raise RuntimeError("convlogic_b200: connection indices must be int64 [out_dim]")
    return x.shape[0], out, x.shape[1]


def logic_fwd(x, a, b, w, wmode):
    check_input(x, a, b, w)
    i, o, bsz = _logic_dims(x, a, b, w)
    y = torch.empty((o, bsz), dtype=x.dtype, device=x.device)
    if bsz == 0 or o == 0:
        return y
    check(lib().clb_logic_fwd(ptr(x), ptr(a), ptr(b), ptr(w), ptr(y), i, o, bsz, wmode, dtype_code(x), stream()))
    return y


def logic_bwd_w(x, a, b, w, gy, wmode, gw_out=None):
    check_input(x, a, b, w, gy)
    i, o, bsz = _logic_dims(x, a, b, w)
    gw = torch.empty_like(w) if gw_out is None else gw_out
    if bsz == 0 or o == 0:
        return gw.zero_()
    check(lib().clb_logic_bwd_w(ptr(x), ptr(a), ptr(b), ptr(w), ptr(gy), ptr(gw), i, o, bsz, wmode, dtype_code(x),
                                stream()))
    return gw


def logic_bwd_x(x, a, b, w, gy, start, consumers, wmode):
    check_input(x, a, b, w, gy, start, consumers)
    i, o, bsz = _logic_dims(x, a, b, w)
    if start.dtype != torch.int64 or consumers.dtype != torch.int64 or start.numel() != i + 1 or consumers.numel() != 2 * o:
        raise RuntimeError("convlogic_b200: consumer lists must be int64 [in_dim + 1] and [2 * out_dim]")
    gx = torch.empty_like(x)
    if bsz == 0:
        return gx
    check(lib().clb_logic_bwd_x(ptr(x), ptr(a), ptr(b), ptr(w), ptr(gy), ptr(gx), ptr(start), ptr(consumers),
                                i, o, bsz, wmode, dtype_code(x), stream()))
    return gx


# ------------------------------------------------------------------------------------ packed
_INT = {8: torch.int8, 16: torch.int16, 32: torch.int32, 64: torch.int64}


def _bits_of(t):
    return t.element_size() * 8


def pack_bits(t, bit_count, sample_major=False):
    """bool tensor -> (packed, pad_len).  ``sample_major=False``: t [F, B] (the reference's
    ``tensor_packbits_cuda`` layout); ``True``: t [B, F]."""
    if bit_count not in _INT:
        raise ValueError("`bit_count` has to be in { 8, 16, 32, 64 }")
    check_input(t)
    if t.dtype not in (torch.bool, torch.uint8):
        raise RuntimeError("convlogic_b200: pack_bits expects a bool or uint8 tensor")
    src = t.view(torch.uint8) if t.dtype == torch.bool else t
    if sample_major:
        b, f = src.shape
    else:
        f, b = src.shape
    words = -(-b // bit_count)
    packed = torch.empty((f, words), dtype=_INT[bit_count], device=t.device)
    fn = lib().clb_pack_bits_nmajor if sample_major else lib().clb_pack_bits
    check(fn(ptr(src), ptr(packed), b if sample_major else f, f if sample_major else b, bit_count, stream()))
    return packed, (bit_count - b % bit_count) % bit_count


def packed_logic(x, a, b, ops):
    check_input(x, a, b, ops)
    if ops.dtype != torch.uint8:
        raise RuntimeError("convlogic_b200: gate ids must be uint8")
    out = ops.shape[0]
    y = torch.empty((out, x.shape[1]), dtype=x.dtype, device=x.device)
    check(lib().clb_packed_logic(ptr(x), ptr(a), ptr(b), ptr(ops), ptr(y), x.shape[0], out, x.shape[1], _bits_of(x),
                                 stream()))
    return y


def group_popcount(x, pad_len, k):
    check_input(x)
    f, words = x.shape
    if f % k:
        raise ValueError(f"in_dim ({f}) has to be divisible by k ({k}) but it is not")
    bits = _bits_of(x)
    counts = torch.empty((words * bits - pad_len, k), dtype=torch.int32, device=x.device)
    check(lib().clb_group_popcount(ptr(x), ptr(counts), f, words, bits, pad_len, k, stream()))
    return counts


def packed_convtree(x, ops, sel, geom):
    check_input(x, ops, sel)
    ci, h, w, words = x.shape
    c = sel.shape[0]
    _sel_ok(sel, c)
    if ops.dtype != torch.uint8 or ops.shape != (c, 7):
        raise RuntimeError(f"convlogic_b200: gate ids must be uint8 [{c}, 7]")
    ho, wo = _out_hw(h, w, *geom)
    if ho <= 0 or wo <= 0 or ho % 2 or wo % 2:
        raise RuntimeError(
            "Output height and width after convolution must be divisible by 2 for 2x2 max pooling, "
            f"but got H_out={ho}, W_out={wo}")
    y = torch.empty((c, ho // 2, wo // 2, words), dtype=x.dtype, device=x.device)
    check(lib().clb_packed_convtree(ptr(x), ptr(ops), ptr(sel), ptr(y), ci, h, w, c, *geom, words, _bits_of(x),
                                    stream()))
    return y


# ---------------------------------------------------------------- packed conv block, slab layout
def packed_to_slab(t):
    """[C, H, W, words] -> [C, U, H, W, 16 // itemsize] (U 16-byte units per pixel row); None when a pixel row
    is not a multiple of 16 bytes."""
    check_input(t)
    c, h, w, words = t.shape
    rowbytes = words * t.element_size()
    if rowbytes % 16 or t.numel() == 0:
        return None
    u = rowbytes // 16
    out = torch.empty((c, u, h, w, 16 // t.element_size()), dtype=t.dtype, device=t.device)
    check(lib().clb_packed_layout(ptr(t), ptr(out), c, h * w, u, 1, stream()))
    return out


def packed_to_rows(slab):
    """[C, U, H, W, 16 // itemsize] -> [C, H, W, words]."""
    check_input(slab)
    c, u, h, w, per = slab.shape
    out = torch.empty((c, h, w, u * per), dtype=slab.dtype, device=slab.device)
    check(lib().clb_packed_layout(ptr(slab), ptr(out), c, h * w, u, 0, stream()))
    return out


def packed_convtree_slab(x, ops, sel, geom):
    """Packed fused block on the slab layout; raises ValueError for shapes it does not cover."""
    check_input(x, ops, sel)
    ci, u, h, w, per = x.shape
    c = sel.shape[0]
    _sel_ok(sel, c)
    if ops.dtype != torch.uint8 or ops.shape != (c, 7):
        raise RuntimeError(f"convlogic_b200: gate ids must be uint8 [{c}, 7]")
    ho, wo = _out_hw(h, w, *geom)
    if ho <= 0 or wo <= 0 or ho % 2 or wo % 2:
        raise RuntimeError(
            "Output height and width after convolution must be divisible by 2 for 2x2 max pooling, "
            f"but got H_out={ho}, W_out={wo}")
    y = torch.empty((c, u, ho // 2, wo // 2, per), dtype=x.dtype, device=x.device)
    scratch = torch.empty(max(lib().clb_packed_convtree_slab_scratch_bytes(c), 16), dtype=torch.uint8, device=x.device)
    check(lib().clb_packed_convtree_slab(ptr(x), ptr(ops), ptr(sel), ptr(y), ptr(scratch), ci, h, w, c, *geom, u, stream()))
    return y


def thermometer_pack(pixels, thresholds, slab=False):
    """pixels [N, Cp, H, W] float32 in [0, 1] (or uint8, compared as v / 255) -> the thermometer features
    ``pixels[:, c] > thresholds[i]`` (channel ``i * Cp + c``) packed 64 samples per int64 word:
    ``[L*Cp, H, W, words]``, or with ``slab=True`` ``[L*Cp, words // 2, H, W, 2]``.  Returns (packed, pad_len)."""
    check_input(pixels, thresholds)
    if pixels.dim() != 4 or pixels.dtype not in (torch.float32, torch.uint8):
        raise RuntimeError("convlogic_b200: thermometer_pack expects float32 or uint8 pixels [N, C, H, W]")
    if thresholds.dtype != torch.float32 or thresholds.dim() != 1:
        raise RuntimeError("convlogic_b200: thresholds must be a float32 vector")
    n, cp, h, w = pixels.shape
    levels = thresholds.numel()
    words = -(-n // 64)
    if slab and words % 2:
        raise RuntimeError("convlogic_b200: the slab layout needs the batch padded to a multiple of 128 samples")
    shape = (levels * cp, words // 2, h, w, 2) if slab else (levels * cp, h, w, words)
    out = torch.empty(shape, dtype=torch.int64, device=pixels.device)
    if out.numel():
        check(lib().clb_thermometer_pack(ptr(pixels), int(pixels.dtype == torch.uint8), ptr(thresholds), levels, ptr(out),
                                         n, cp, h * w, words, int(slab), stream()))
    return out, (64 - n % 64) % 64


def group_sum_fwd(y_fm, k, tau):
    """Feature-major activations [F, B] -> [B, k] class sums / tau."""
    check_input(y_fm)
    f, b = y_fm.shape
    out = torch.empty((b, k), dtype=y_fm.dtype, device=y_fm.device)
    nbytes = lib().clb_group_sum_scratch_bytes(f, b, k, dtype_code(y_fm))
    scratch = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=y_fm.device)
    check(lib().clb_group_sum_fwd(ptr(y_fm), ptr(out), ptr(scratch), nbytes, f, b, k, float(tau), dtype_code(y_fm), stream()))
    return out


def group_sum_bwd(gout, f, k, tau, scale=None):
    """Gradient of group_sum_fwd: [B, k] -> feature-major [F, B]; ``scale``: a one-element device tensor every value is
    multiplied by (the upstream gradient of a scalar loss), read by the kernel."""
    check_input(gout)
    b = gout.shape[0]
    gy = torch.empty((f, b), dtype=gout.dtype, device=gout.device)
    if scale is not None:
        check_input(scale)
        if scale.numel() != 1 or scale.dtype != gout.dtype:
            raise RuntimeError("convlogic_b200: `scale` must be a one-element tensor of the gradient's dtype")
    check(lib().clb_group_sum_bwd_scaled(ptr(gout), ptr(scale), ptr(gy), f, b, k, float(tau), dtype_code(gout), stream()))
    return gy


def logic_tree_fwd(x_fm, leaf, node, w0, w1, w2, wmode):
    """Three fused flat layers, forward: x [in, B] -> y [T, B] (see ``clb_logic_tree_fwd``)."""
    check_input(x_fm, leaf, node, w0, w1, w2)
    t, b = leaf.shape[0], x_fm.shape[1]
    y = torch.empty((t, b), dtype=torch.float32, device=x_fm.device)
    check(lib().clb_logic_tree_fwd(ptr(x_fm), ptr(leaf), ptr(node), ptr(w0), ptr(w1), ptr(w2), ptr(y), t, b, wmode, stream()))
    return y


def logic_tree_bwd(x_fm, leaf, node, w0, w1, w2, gy, start, slots, wmode, need_gx=True, gw_out=None, clear_gw=True, head=None):
    """Gradients of ``logic_tree_fwd``: (gx [in, B] or None, gw0, gw1, gw2).  ``gw_out``: three contiguous tensors to
    receive the gate gradients (cleared first: a neuron no tree reads keeps a zero gradient; ``clear_gw=False`` when the
    caller knows that every neuron sits in a tree).  ``head = (dscore [B, k], scale [1], k, tau)`` instead of ``gy``: the
    trees feed GroupSum + cross-entropy, and the upstream gradient is derived from that head's score gradient inside
    the kernel."""
    if head is None:
        check_input(x_fm, leaf, node, w0, w1, w2, gy, start, slots)
    else:
        check_input(x_fm, leaf, node, w0, w1, w2, head[0], head[1], start, slots)
        if head[0].dtype != torch.float32 or head[1].dtype != torch.float32 or tuple(head[0].shape) != (x_fm.shape[1], head[2]) \
                or head[1].numel() != 1 or leaf.shape[0] % head[2]:
            raise RuntimeError("convlogic_b200: the head of logic_tree_bwd is (dscore float32 [B, k], scale float32 [1], k, tau)")
    t, b, in_dim = leaf.shape[0], x_fm.shape[1], x_fm.shape[0]
    tapgrad = torch.empty((max(t * 8, 1), b), dtype=torch.float32, device=x_fm.device)
    if gw_out is None:
        gws = [torch.zeros_like(w) if clear_gw else torch.empty_like(w) for w in (w0, w1, w2)]
    else:
        gws = [g.zero_() if clear_gw else g for g in gw_out]
    gx = torch.empty_like(x_fm) if need_gx else None
    if head is None:
        check(lib().clb_logic_tree_bwd(ptr(x_fm), ptr(leaf), ptr(node), ptr(w0), ptr(w1), ptr(w2), ptr(gy), ptr(tapgrad), ptr(gws[0]),
                                       ptr(gws[1]), ptr(gws[2]), ptr(gx), ptr(start), ptr(slots), in_dim, t, b, wmode, stream()))
    else:
        check(lib().clb_logic_tree_bwd_scores(ptr(x_fm), ptr(leaf), ptr(node), ptr(w0), ptr(w1), ptr(w2), ptr(head[0]), ptr(head[1]),
                                              int(head[2]), float(head[3]), ptr(tapgrad), ptr(gws[0]), ptr(gws[1]), ptr(gws[2]), ptr(gx),
                                              ptr(start), ptr(slots), in_dim, t, b, wmode, stream()))
    return gx, gws[0], gws[1], gws[2]


def logic_tree_fwd_ce(x_fm, leaf, node, w0, w1, w2, labels, k, tau, wmode):
    """Fused flat layers + GroupSum + mean cross-entropy without the activation in between: (loss [1], dscore [B, k]),
    or None for a shape that path does not take (the caller then runs ``logic_tree_fwd`` and ``group_sum_ce``)."""
    check_input(x_fm, leaf, node, w0, w1, w2, labels)
    t, b = leaf.shape[0], x_fm.shape[1]
    if x_fm.dtype != torch.float32 or labels.dtype != torch.int64 or labels.shape != (b,):
        raise RuntimeError("convlogic_b200: logic_tree_fwd_ce expects float32 [in, B] activations and int64 [B] labels")
    nbytes = lib().clb_logic_tree_fwd_ce_scratch_bytes(t, b, k)
    if nbytes == 0 or b % 4 or b > 512 or k > 32:
        return None
    loss = torch.empty(1, dtype=torch.float32, device=x_fm.device)
    dscore = torch.empty((b, k), dtype=torch.float32, device=x_fm.device)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=x_fm.device)
    rc = lib().clb_logic_tree_fwd_ce(ptr(x_fm), ptr(leaf), ptr(node), ptr(w0), ptr(w1), ptr(w2), ptr(labels), ptr(dscore), ptr(loss),
                                     ptr(scratch), nbytes, t, b, k, float(tau), wmode, stream())
    if rc == _lib.ERR_SHAPE:
        return None
    check(rc)
    return loss, dscore


def group_sum_ce(y_fm, labels, k, tau, want_scores=False):
    """GroupSum + mean cross-entropy on feature-major activations [F, B]: (loss [1], dscore [B, k], scores or None)."""
    check_input(y_fm, labels)
    if y_fm.dtype != torch.float32 or labels.dtype != torch.int64 or labels.shape != (y_fm.shape[1],):
        raise RuntimeError("convlogic_b200: group_sum_ce expects float32 [F, B] activations and int64 [B] labels")
    f, b = y_fm.shape
    if f % k:
        raise ValueError(f"in_dim ({f}) has to be divisible by k ({k}) but it is not")
    loss = torch.empty(1, dtype=torch.float32, device=y_fm.device)
    dscore = torch.empty((b, k), dtype=torch.float32, device=y_fm.device)
    scores = torch.empty((b, k), dtype=torch.float32, device=y_fm.device) if want_scores else None
    nbytes = lib().clb_group_sum_scratch_bytes(f, b, k, dtype_code(y_fm))
    scratch = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=y_fm.device)
    check(lib().clb_group_sum_ce(ptr(y_fm), ptr(labels), ptr(scores), ptr(dscore), ptr(loss), ptr(scratch), nbytes, f, b, k, float(tau), stream()))
    return loss, dscore, scores


def transpose2d(x):
    """Contiguous [cols, rows] copy of a contiguous float32 [rows, cols] tensor (one tiled kernel)."""
    check_input(x)
    if x.dim() != 2 or x.dtype != torch.float32 or not x.is_contiguous():
        raise RuntimeError("convlogic_b200: transpose2d expects a contiguous 2-D float32 tensor")
    out = torch.empty((x.shape[1], x.shape[0]), dtype=x.dtype, device=x.device)
    check(lib().clb_transpose_f32(ptr(x), ptr(out), x.shape[0], x.shape[1], stream()))
    return out


def adam_step(p, g, m, v, lr, beta1, beta2, eps, weight_decay, step, decoupled):
    """One Adam / AdamW step over flat fp32 buffers, in place."""
    check_input(p, g, m, v)
    n = p.numel()
    if not (g.numel() == m.numel() == v.numel() == n) or any(t.dtype != torch.float32 for t in (p, g, m, v)):
        raise RuntimeError("convlogic_b200: adam_step expects four float32 buffers of equal size")
    check(lib().clb_adam_step(ptr(p), ptr(g), ptr(m), ptr(v), n, float(lr), float(beta1), float(beta2), float(eps), float(weight_decay),
                              int(step), int(bool(decoupled)), stream()))
