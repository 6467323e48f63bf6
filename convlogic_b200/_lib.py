"""ctypes binding of the C-ABI library ``csrc/libconvlogic_b200.so``.

The library is the product: there is no CPU or PyTorch fallback.  If it has not been built,
every operation raises (``python -m convlogic_b200.build`` builds it with nvcc).
"""

import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "csrc", "libconvlogic_b200.so")

F32, F64 = 0, 1
W_PROB, W_SOFTMAX, W_ARGMAX = 0, 1, 2
SEL_UNBOUNDED = 0x100
Y_FEATURE_MAJOR = 0x200   # wmode flag: the block's output / upstream gradient is [C][windows][N]
TUNE_TAPGRAD_SLICE_BYTES = 1
TUNE_PLANE_KERNELS = 2
TUNE_SLAB_MUX = 3
ERR_SHAPE, ERR_ODD_OUTPUT, ERR_TOO_LARGE = -2, -5, -6

_lib = None

_vp, _i, _i64, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_size_t
_conv = [_i] * 11  # N, Ci, H, W, C, sh, sw, ph, pw, kh, kw

_SIGNATURES = {
    "clb_version": ([], _i),
    "clb_status_string": ([_i], C.c_char_p),
    "clb_last_cuda_error": ([], _i),
    "clb_kernel_launches": ([], C.c_longlong),
    "clb_tune": ([_i, C.c_longlong], _i),
    "clb_tune_get": ([_i], C.c_longlong),
    "clb_trace": ([_i], _i),
    "clb_trace_report": ([C.c_char_p, _sz], C.c_longlong),
    "clb_convtree_fwd": ([_vp] * 8 + _conv + [_i, _i, _vp], _i),
    "clb_convtree_bwd_x_scratch_bytes": (_conv + [_i], _sz),
    "clb_convtree_bwd_x": ([_vp] * 8 + [_i, _i, _vp, _sz] + _conv + [_i, _i, _vp], _i),
    "clb_convtree_bwd_scratch_bytes": (_conv + [_i, _i, _i], _sz),
    "clb_convtree_bwd": ([_vp] * 9 + [_i, _i, _vp, _sz] + _conv + [_i, _i, _vp], _i),
    "clb_conv_channel_lists": ([_vp, _i, _i, _i, _i, _vp, _vp, _i], _i),
    "clb_convtree_bwd_plane_scratch_bytes": (_conv + [_i], _sz),
    "clb_convtree_bwd_plane": ([_vp] * 10 + [_sz] + _conv + [_i, _i, _vp], _i),
    "clb_plane_error": ([_vp], _i),
    "clb_conv_group_plan": (_conv + [_i, C.POINTER(_i), C.POINTER(_i)], _i),
    "clb_conv_build_groups": ([_vp, _i, _i, _i, _vp, _vp, _i], _i),
    "clb_convtree_bwd_w_scratch_bytes": ([_i, _i, _i, _i, _i], _sz),
    "clb_convtree_bwd_w": ([_vp] * 7 + [_sz] + _conv + [_i, _i, _vp], _i),
    "clb_convtree_bwd_w_noalloc_max_bytes": ([], _sz),
    "clb_convtree_bwd_w_noalloc": ([_vp] * 6 + _conv + [_i, _i, _vp], _i),
    "clb_conv_fwd": ([_vp] * 4 + _conv + [_i, _i, _vp], _i),
    "clb_conv_bwd_x": ([_vp] * 7 + [_i, _i] + _conv + [_i, _i, _vp], _i),
    "clb_conv_bwd_w_scratch_bytes": ([_i, _i, _i, _i, _i], _sz),
    "clb_conv_bwd_w": ([_vp] * 6 + [_sz] + _conv + [_i, _i, _vp], _i),
    "clb_tree_fwd": ([_vp] * 3 + [_i] * 6 + [_vp], _i),
    "clb_tree_bwd_x": ([_vp] * 4 + [_i] * 6 + [_vp], _i),
    "clb_tree_bwd_w_scratch_bytes": ([_i] * 5, _sz),
    "clb_tree_bwd_w": ([_vp] * 5 + [_sz] + [_i] * 6 + [_vp], _i),
    "clb_logic_fwd": ([_vp] * 5 + [_i64] * 3 + [_i, _i, _vp], _i),
    "clb_logic_bwd_w": ([_vp] * 6 + [_i64] * 3 + [_i, _i, _vp], _i),
    "clb_logic_bwd_x": ([_vp] * 8 + [_i64] * 3 + [_i, _i, _vp], _i),
    "clb_pack_bits": ([_vp, _vp, _i64, _i64, _i, _vp], _i),
    "clb_pack_bits_nmajor": ([_vp, _vp, _i64, _i64, _i, _vp], _i),
    "clb_packed_logic": ([_vp] * 5 + [_i64] * 3 + [_i, _vp], _i),
    "clb_group_popcount": ([_vp, _vp, _i64, _i64, _i, _i, _i, _vp], _i),
    "clb_packed_convtree": ([_vp] * 4 + [_i] * 10 + [_i64, _i, _vp], _i),
    "clb_packed_tree": ([_vp, _vp, _vp, _vp, _i64, _i64, _i, _i64, _i, _vp], _i),
    "clb_thermometer_pack": ([_vp, _i, _vp, _i, _vp, _i64, _i64, _i64, _i64, _i, _vp], _i),
    "clb_logic_tree_fwd": ([_vp] * 7 + [_i64, _i64, _i, _vp], _i),
    "clb_logic_tree_bwd": ([_vp] * 14 + [_i64, _i64, _i64, _i, _vp], _i),
    "clb_logic_tree_fwd_ce_scratch_bytes": ([_i64, _i64, _i], _sz),
    "clb_logic_tree_fwd_ce": ([_vp] * 10 + [_sz, _i64, _i64, _i, C.c_double, _i, _vp], _i),
    "clb_logic_tree_bwd_scores": ([_vp] * 8 + [_i, C.c_double] + [_vp] * 7 + [_i64, _i64, _i64, _i, _vp], _i),
    "clb_group_sum_scratch_bytes": ([_i64, _i64, _i, _i], _sz),
    "clb_group_sum_fwd": ([_vp, _vp, _vp, _sz, _i64, _i64, _i, C.c_double, _i, _vp], _i),
    "clb_group_sum_ce": ([_vp] * 6 + [_sz, _i64, _i64, _i, C.c_double, _vp], _i),
    "clb_transpose_f32": ([_vp, _vp, _i64, _i64, _vp], _i),
    "clb_adam_step": ([_vp] * 4 + [_i64] + [C.c_double] * 5 + [_i64, _i, _vp], _i),
    "clb_group_sum_bwd_scaled": ([_vp, _vp, _vp, _i64, _i64, _i, C.c_double, _i, _vp], _i),
    "clb_group_sum_bwd": ([_vp, _vp, _i64, _i64, _i, C.c_double, _i, _vp], _i),
    "clb_net_device_bytes": ([_vp, _sz, _vp], _i),
    "clb_net_create": ([_vp, _sz, _vp, _vp, _vp], _i),
    "clb_net_destroy": ([_vp], None),
    "clb_net_info": ([_vp, _vp, _vp, _vp], _i),
    "clb_net_workspace_bytes": ([_vp, _i64], _sz),
    "clb_net_forward": ([_vp, _i, _vp, _vp, _i, _i64, _vp, _vp, _sz, _vp], _i),
    "clb_packed_layout": ([_vp, _vp, _i64, _i64, _i64, _i, _vp], _i),
    "clb_packed_convtree_slab_scratch_bytes": ([_i], _i64),
    "clb_packed_convtree_slab": ([_vp] * 5 + [_i] * 10 + [_i64, _vp], _i),
}

EXPORTS = tuple(_SIGNATURES)


def lib():
    """The loaded library; raises RuntimeError when it is missing (no fallback exists)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"convlogic_b200: CUDA library not found at {LIB_PATH}. "
                "Build it with `python -m convlogic_b200.build` (needs nvcc); there is no CPU fallback.")
        handle = C.CDLL(LIB_PATH)
        for name, (args, res) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.argtypes, fn.restype = args, res
        _lib = handle
    return _lib


def trace(on):
    """Turn the library's launch tracing on (dropping earlier records) or off."""
    check(lib().clb_trace(int(bool(on))))


def trace_report():
    """{kernel name: (launches, total ms)} of the launches traced since ``trace(True)``; clears the records."""
    buf = C.create_string_buffer(1 << 16)
    lib().clb_trace_report(buf, len(buf))
    out = {}
    for line in buf.value.decode().splitlines():
        name, launches, ms = line.split("\t")
        out[name] = (int(launches), float(ms))
    return out


def check(status):
    """Map a C-ABI status to the exception the reference raises for the same condition."""
    if status == 0:
        return
    text = lib().clb_status_string(status).decode()
    if status == -3:
        err = lib().clb_last_cuda_error()
        raise RuntimeError(f"convlogic_b200: {text} (cudaError {err})")
    if status in (ERR_SHAPE, ERR_TOO_LARGE):
        raise ValueError(f"convlogic_b200: {text}")
    raise RuntimeError(f"convlogic_b200: {text}")


def dtype_code(t):
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.float64:
        return F64
    raise RuntimeError(f"convlogic_b200: expected a float32 or float64 tensor, got {t.dtype}")


def ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def check_input(*tensors):
    """The reference's CHECK_INPUT (src/common/cuda_utils.cuh:9-13): CUDA and contiguous."""
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("convlogic_b200: tensor must be a CUDA tensor")
        if not t.is_contiguous():
            raise RuntimeError("convlogic_b200: tensor must be contiguous")
