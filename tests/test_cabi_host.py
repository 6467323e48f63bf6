"""CPU-only checks of the C-ABI library: it loads, exports every symbol the header declares, and
its host-side helpers (no CUDA call) behave.  No kernel is launched here."""

import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from convlogic_b200.build import build
    from convlogic_b200 import _lib

    build()
    return _lib.lib()


def test_every_declared_symbol_is_exported(lib):
    from convlogic_b200 import _lib

    header = open(os.path.join(ROOT, "include", "convlogic_b200.h")).read()
    declared = set(re.findall(r"\b(clb_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in include/convlogic_b200.h but not exported"
    assert declared == set(_lib.EXPORTS), declared ^ set(_lib.EXPORTS)


def test_status_strings(lib):
    assert lib.clb_version() >= 100
    assert lib.clb_status_string(0) == b"ok"
    assert b"divisible by 2" in lib.clb_status_string(-5)
    assert lib.clb_status_string(-12345) == b"unknown status"


def test_null_arguments_are_rejected_before_any_launch(lib):
    # no device pointer is touched: argument validation comes first
    assert lib.clb_convtree_fwd(None, None, None, None, None, None, None, None, 1, 1, 4, 4, 1, 1, 1, 1, 1, 3, 3, 0, 0, None) == -1
    assert lib.clb_logic_fwd(None, None, None, None, None, 4, 4, 4, 0, 0, None) == -1
    assert lib.clb_group_popcount(None, None, 10, 1, 64, 0, 3, None) == -1
    assert lib.clb_pack_bits(None, None, 1, 1, 7, None) == -1


def test_group_plan_and_tables(lib):
    cg, nb = C.c_int(), C.c_int()
    # the microbenchmark block: one image per block, a 32 KiB tile of haloed 34x34 planes
    assert lib.clb_conv_group_plan(256, 9, 32, 32, 256, 1, 1, 1, 1, 3, 3, 0, C.byref(cg), C.byref(nb)) == 0
    assert (cg.value, nb.value) == (7, 1)
    # tiny images: several images per block, small channel groups (a tile of 4 KiB per warp keeps ~50 warps per SM)
    assert lib.clb_conv_group_plan(256, 4096, 4, 4, 8192, 1, 1, 1, 1, 3, 3, 0, C.byref(cg), C.byref(nb)) == 0
    assert nb.value == 64 and cg.value * nb.value * 36 * 4 <= 32 * 1024 and cg.value >= 1
    assert lib.clb_conv_group_plan(256, 256, 16, 16, 1024, 1, 1, 1, 1, 3, 3, 0, C.byref(cg), C.byref(nb)) == 0
    assert nb.value == 4 and cg.value * nb.value * 18 * 18 * 4 <= 16 * 1024 and cg.value >= 1
    # a channel plane that cannot fit shared memory is refused
    assert lib.clb_conv_group_plan(1, 1, 512, 512, 1, 1, 1, 1, 1, 3, 3, 0, C.byref(cg), C.byref(nb)) == -2

    sel = np.array([[(0 << 16) | 1, (0 << 16), (3 << 16), (3 << 16), 0, 0, 0, 0],
                    [(5 << 16)] * 8,
                    [(2 << 16)] * 4 + [(4 << 16)] * 4], dtype=np.int32)
    start = np.zeros(4, dtype=np.int32)
    lst = np.zeros(9, dtype=np.int32)
    n = lib.clb_conv_build_groups(sel.ctypes.data_as(C.c_void_p), 3, 6, 2, start.ctypes.data_as(C.c_void_p),
                                  lst.ctypes.data_as(C.c_void_p), 9)
    assert n == 5
    assert start.tolist() == [0, 1, 3, 5] and lst[:5].tolist() == [0, 0, 2, 1, 2]
    # a selection naming a channel beyond Ci is an argument error
    assert lib.clb_conv_build_groups(sel.ctypes.data_as(C.c_void_p), 3, 5, 2, start.ctypes.data_as(C.c_void_p),
                                     lst.ctypes.data_as(C.c_void_p), 9) == -1


def test_scratch_sizes(lib):
    assert lib.clb_convtree_bwd_w_scratch_bytes(256, 256, 32, 32, 0) % (256 * 28 * 4) == 0
    assert lib.clb_convtree_bwd_w_scratch_bytes(1, 1, 2, 2, 1) == 28 * 8
    assert lib.clb_tree_bwd_w_scratch_bytes(2, 3, 16, 2, 0) == 3 * 2 * 4 * 4


def test_modules_construct_on_cpu_and_refuse_to_run_there():
    import torch

    import convlogic_b200 as cb

    torch.manual_seed(0)
    layer = cb.ConvLogicLayer(3, 4, complete=True)
    assert layer.weights.shape == (4, 7, 16) and layer.selection.dtype == torch.int32
    ch, r, s = layer.unpack_selection(layer.selection)
    assert int(ch.max()) < 3 and int(r.max()) < 3 and int(s.max()) < 3
    for k in range(0, 8, 2):  # the two taps of a pair never coincide
        assert not bool(((layer.selection[:, k] == layer.selection[:, k + 1])).any())
    fl = cb.LogicLayer(16, 40)
    assert fl.given_x_indices_of_y_start.shape == (17,) and fl.given_x_indices_of_y.shape == (80,)
    assert set(fl.state_dict()) == {"weights", "indices_0", "indices_1", "given_x_indices_of_y_start", "given_x_indices_of_y"}
    with pytest.raises(RuntimeError):
        layer(torch.rand(1, 3, 4, 4))
    with pytest.raises(ValueError):
        cb.ConvLogicLayer(3, 4, implementation="python")
    with pytest.raises(NotImplementedError):
        cb.PackBitsTensor(torch.zeros(4, 4, dtype=torch.bool))
    m = cb.ConvLogicCifarModel(k_param=2, input_channels=3, tau=5)
    dims = [(l.in_dim, l.out_dim) for l in m.network if isinstance(l, cb.LogicLayer)]
    assert dims == [(256, 2560), (2560, 1280), (1280, 640)]


def test_network_blob_is_validated_on_the_host():
    """clb_net_device_bytes parses a blob without touching the GPU: a well-formed one is accepted, damaged ones
    (bad magic, truncated, inconsistent layer widths) come back as CLB_ERR_SHAPE."""
    import ctypes as C

    import torch

    import convlogic_b200 as cb
    from convlogic_b200 import _lib
    from convlogic_b200.compiled_model import serialise

    torch.manual_seed(0)
    model = torch.nn.Sequential(cb.ConvLogicLayer(3, 4, complete=True), torch.nn.Flatten(), cb.LogicLayer(4 * 4 * 4, 40), cb.GroupSum(10))
    blob = serialise(model, input_shape=(3, 8, 8))
    lib = _lib.lib()
    need = C.c_size_t()
    assert lib.clb_net_device_bytes(blob, len(blob), C.byref(need)) == 0 and need.value == len(blob)
    assert lib.clb_net_device_bytes(b"XXXXXXXX" + blob[8:], len(blob), C.byref(need)) == _lib.ERR_SHAPE
    assert lib.clb_net_device_bytes(blob[:-16], len(blob) - 16, C.byref(need)) == _lib.ERR_SHAPE
    wrong = serialise(model, input_shape=(3, 10, 10))  # the flat layer no longer matches the conv output
    assert lib.clb_net_device_bytes(wrong, len(wrong), C.byref(need)) == _lib.ERR_SHAPE
    with pytest.raises(AssertionError):
        serialise(torch.nn.Sequential(cb.LogicLayer(8, 10)))  # no GroupSum at the end


def test_network_blob_with_an_index_out_of_range_is_rejected():
    """A blob whose offsets and widths are fine but whose index VALUES are not (a flat connection beyond the input
    width, a conv tap naming a missing channel or a cell outside the window, a gate id above 15, a leaf of a fused
    gate tree beyond the input) must come back as CLB_ERR_SHAPE: the kernels index with these values unclamped."""
    import ctypes as C
    import struct

    import torch

    import convlogic_b200 as cb
    from convlogic_b200 import _lib
    from convlogic_b200.compiled_model import serialise

    torch.manual_seed(1)
    model = torch.nn.Sequential(cb.ConvLogicLayer(3, 4, complete=True), torch.nn.Flatten(), cb.LogicLayer(4 * 4 * 4, 40), cb.GroupSum(10))
    blob = serialise(model, input_shape=(3, 8, 8))
    lib = _lib.lib()
    need = C.c_size_t()

    def status(b):
        return lib.clb_net_device_bytes(bytes(b), len(b), C.byref(need))

    def layer_offsets(b, i):
        return struct.unpack_from("<3Q", b, 64 + 64 * i + 32)   # off_a, off_b, off_ops

    assert status(blob) == 0
    conv_sel, _, conv_ops = layer_offsets(blob, 0)
    flat_a, flat_b, flat_ops = layer_offsets(blob, 1)
    for off, fmt, bad in ((flat_a, "<q", 64), (flat_b, "<q", -1), (flat_a + 8 * 39, "<q", 1 << 40), (flat_ops, "<B", 16),
                          (conv_ops + 5, "<B", 200), (conv_sel, "<i", (3 << 16) | (1 << 8) | 1),      # channel 3 of 3
                          (conv_sel + 4, "<i", (0 << 16) | (3 << 8) | 0), (conv_sel + 8, "<i", (0 << 16) | (0 << 8) | 3)):
        damaged = bytearray(blob)
        struct.pack_into(fmt, damaged, off, bad)
        assert status(damaged) == _lib.ERR_SHAPE, (off, fmt, bad)
    # a fused gate tree (three flat layers halving their width)
    tree = torch.nn.Sequential(cb.LogicLayer(16, 80), cb.LogicLayer(80, 40), cb.LogicLayer(40, 20), cb.GroupSum(10))
    tb = serialise(tree)
    assert status(tb) == 0 and struct.unpack_from("<I", tb, 64)[0] == 3
    leaf, _, ops = layer_offsets(tb, 0)
    for off, fmt, bad in ((leaf + 4 * 7, "<i", 16), (leaf, "<i", -2), (ops + 3, "<B", 99)):
        damaged = bytearray(tb)
        struct.pack_into(fmt, damaged, off, bad)
        assert status(damaged) == _lib.ERR_SHAPE, (off, fmt, bad)
