"""CompiledLogicNet: the discretised network as a deployable artefact.

The reference's ``CompiledLogicNet`` (src/difflogic/compiled_model.py:41-361) takes a trained
``nn.Sequential`` of ``LogicLayer`` s ending in ``GroupSum``, writes every gate out as a line of C,
compiles that with gcc and calls the resulting ``apply_logic_gate_net(bool*, int*, size_t)`` on the CPU
through ctypes; fused conv blocks are not supported there.  Here the artefact is a *blob* -- the arg-max
gate of every neuron plus its connections, for fused ``ConvLogicLayer`` blocks as well as flat layers -- and
the code is the library's ``clb_net_*`` runtime, which runs the whole stack on the GPU with one C call
(any host language; no Python or torch needed at deployment).  The class keeps the reference's surface:
``CompiledLogicNet(model, num_bits=64)``, ``compile(save_lib_path=...)``, ``CompiledLogicNet.load(path, ...)``,
``forward(x)`` with ``x`` bool ``[B, F]`` (or ``[B, C, H, W]``) returning int32 counts ``[B, num_classes]``.
"""

import ctypes as C
import struct

import numpy as np
import torch

from . import _lib
from .convlogic_layer import ConvLogicLayer
from .difflogic import GroupSum, LogicLayer

_MAGIC = b"CLBNET01"


def _align16(n):
    return (n + 15) // 16 * 16


def fuse_flat_layers(run):
    """2 or 3 consecutive LogicLayers -> (leaf int32 [out, 2^m], ops uint8 [out, 2^m - 1]): every neuron of the last
    layer as a gate tree over rows of the first layer's input (``clb_packed_tree``'s tables)."""
    m = len(run)
    assert m in (2, 3)
    idx = [(l.indices_0.detach().cpu().numpy().astype(np.int64), l.indices_1.detach().cpu().numpy().astype(np.int64)) for l in run]
    gate = [l.weights.detach().argmax(-1).cpu().numpy().astype(np.uint8) for l in run]
    out = run[-1].out_dim
    # nodes[level] = neuron ids of layer `level` (0 = first layer) feeding the tree, in tree order, [out, 2^(m-1-level)]
    nodes = [None] * m
    nodes[m - 1] = np.arange(out, dtype=np.int64)[:, None]
    for lvl in range(m - 1, 0, -1):
        a, b = idx[lvl]
        cur = nodes[lvl]
        nodes[lvl - 1] = np.stack([a[cur], b[cur]], axis=-1).reshape(out, -1)  # children of node q at 2q, 2q+1
    a0, b0 = idx[0]
    leaf = np.stack([a0[nodes[0]], b0[nodes[0]]], axis=-1).reshape(out, -1).astype(np.int32)
    ops = np.concatenate([gate[lvl][nodes[lvl]] for lvl in range(m)], axis=1).astype(np.uint8)
    assert leaf.shape == (out, 1 << m) and ops.shape == (out, (1 << m) - 1)
    return leaf, ops


def serialise(model, input_shape=None, fuse=True):
    """``nn.Sequential`` (fused complete ConvLogicLayers, Flatten, LogicLayers, GroupSum last) -> blob bytes.

    ``input_shape`` = (C, H, W) is required when the stack starts with a conv block.  ``fuse``: emit runs of flat
    layers that halve their width as one gate-tree layer (no intermediate activations at run time)."""
    layers = list(model)
    if not isinstance(layers[-1], GroupSum):
        raise AssertionError(f"The last layer of the model must be GroupSum, but it is {type(layers[-1])} / {layers[-1]} instead.")
    num_classes = layers[-1].k
    recs, arrays = [], []
    offset = [0]

    def add(arr):
        data = np.ascontiguousarray(arr).tobytes()
        off = offset[0]
        arrays.append((off, data))
        offset[0] = _align16(off + len(data))
        return off

    in_features = None
    flat_run = []  # consecutive LogicLayers, emitted (fused where it pays) when the run ends

    def emit_flat(run):
        i = 0
        while i < len(run):
            # fuse up to three layers while every output of a layer is read at most about once by the next
            m = 1
            while fuse and m < 3 and i + m < len(run) and 2 * run[i + m].out_dim <= run[i + m - 1].out_dim:
                m += 1
            if m == 1:
                layer = run[i]
                a = layer.indices_0.detach().cpu().numpy().astype(np.int64)
                b = layer.indices_1.detach().cpu().numpy().astype(np.int64)
                ops = layer.weights.detach().argmax(-1).cpu().numpy().astype(np.uint8)
                recs.append((2, [layer.in_dim & 0xFFFFFFFF, layer.out_dim & 0xFFFFFFFF, layer.in_dim >> 32, layer.out_dim >> 32, 0, 0, 0],
                             add(a), add(b), add(ops)))
            else:
                leaf, ops = fuse_flat_layers(run[i:i + m])
                first, last = run[i], run[i + m - 1]
                recs.append((3, [first.in_dim & 0xFFFFFFFF, last.out_dim & 0xFFFFFFFF, first.in_dim >> 32, last.out_dim >> 32, m, 0, 0],
                             add(leaf), 0, add(ops)))
            i += m

    for layer in layers[:-1]:
        if flat_run and not isinstance(layer, LogicLayer):
            emit_flat(flat_run)
            flat_run = []
        if isinstance(layer, ConvLogicLayer):
            if not layer.complete:
                raise AssertionError("only complete (fused) ConvLogicLayer blocks can be compiled")
            if layer.stride[0] != layer.stride[1]:
                raise AssertionError("compiled conv blocks need equal strides")
            sel = layer.selection.detach().cpu().numpy().astype(np.int32)
            ops = layer.weights.detach().argmax(-1).cpu().numpy().astype(np.uint8)
            recs.append((1, [layer.in_channels, layer.out_channels, layer.kernel[0], layer.kernel[1], layer.stride[0],
                             layer.padding[0], layer.padding[1]], add(sel), 0, add(ops)))
        elif isinstance(layer, LogicLayer):
            if in_features is None and not recs:
                in_features = layer.in_dim
            flat_run.append(layer)
        elif isinstance(layer, torch.nn.Flatten):
            continue
        else:
            raise AssertionError(f"Error: layer {type(layer)} / {layer} unknown.")
    if flat_run:
        emit_flat(flat_run)
    if not recs:
        raise AssertionError("the model holds no logic layer")
    image = recs[0][0] == 1
    if image and input_shape is None:
        raise AssertionError("input_shape=(C, H, W) is needed for a stack that starts with a conv block")
    c, h, w = (int(v) for v in input_shape) if image else (0, 0, 0)
    base = 64 + 64 * len(recs)
    total = base + offset[0]
    out = bytearray(total)
    struct.pack_into("<8s6IQ", out, 0, _MAGIC, len(recs), num_classes, c, h, w, 0 if image else int(in_features), total)
    for i, (kind, p, oa, ob, oo) in enumerate(recs):
        struct.pack_into("<8I3Q", out, 64 + 64 * i, kind, *[int(v) for v in p], base + oa, base + ob, base + oo)
    for off, data in arrays:
        out[base + off: base + off + len(data)] = data
    return bytes(out)


class CompiledLogicNet(torch.nn.Module):
    def __init__(self, model=None, device="cuda", num_bits=64, input_shape=None, verbose=False, fuse=True):
        super().__init__()
        assert num_bits == 64, "the GPU runtime packs 64 samples per word"
        self.model, self.device, self.num_bits, self.input_shape = model, torch.device(device), num_bits, input_shape
        self.blob = None
        self._net = None
        self._params = None
        self._workspace = None
        if model is not None:
            self.num_classes = model[-1].k
            self.blob = serialise(model, input_shape, fuse)
            if verbose:
                print(f"blob of {len(self.blob)} bytes created.")

    # ---- the reference's compile / load pair
    def compile(self, opt_level=1, save_lib_path=None, verbose=False):
        """Uploads the blob and creates the runtime handle; ``save_lib_path`` also writes the blob to a file
        (the reference writes the compiled shared object there)."""
        del opt_level
        if save_lib_path is not None:
            with open(save_lib_path, "wb") as f:
                f.write(self.blob)
        self._create()
        if verbose:
            print(f"network of {len(self.blob)} parameter bytes is on {self.device}.")
        return self

    @staticmethod
    def load(save_lib_path, num_classes=None, num_bits=64, device="cuda"):
        self = CompiledLogicNet(None, device=device, num_bits=num_bits)
        with open(save_lib_path, "rb") as f:
            self.blob = f.read()
        self._create()
        if num_classes is not None and num_classes != self.num_classes:
            raise ValueError(f"the file holds a network with {self.num_classes} classes, not {num_classes}")
        return self

    def _create(self):
        lib = _lib.lib()
        need = C.c_size_t()
        _lib.check(lib.clb_net_device_bytes(self.blob, len(self.blob), C.byref(need)))
        self._params = torch.empty(max(need.value, 16), dtype=torch.uint8, device=self.device)
        handle = C.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(lib.clb_net_create(self.blob, len(self.blob), _lib.ptr(self._params), _lib.stream(), C.byref(handle)))
            torch.cuda.current_stream().synchronize()  # the blob is pageable host memory: wait for the copy
        self._net = handle
        feats, classes, n = C.c_int64(), C.c_int(), C.c_int()
        _lib.check(lib.clb_net_info(handle, C.byref(feats), C.byref(classes), C.byref(n)))
        self.num_inputs, self.num_classes, self.num_layers = feats.value, classes.value, n.value

    def __del__(self):
        if getattr(self, "_net", None) is not None:
            try:
                _lib.lib().clb_net_destroy(self._net)
            except Exception:
                pass
            self._net = None

    # ---- inference
    def _run(self, kind, x, batch, thresholds=None):
        if self._net is None:
            raise RuntimeError("convlogic_b200: call compile() or load() first")
        lib = _lib.lib()
        need = lib.clb_net_workspace_bytes(self._net, batch)
        if self._workspace is None or self._workspace.numel() < need:
            self._workspace = torch.empty(need, dtype=torch.uint8, device=self.device)
        counts = torch.empty((batch, self.num_classes), dtype=torch.int32, device=self.device)
        levels = 0 if thresholds is None else thresholds.numel()
        with torch.cuda.device(self.device):
            _lib.check(lib.clb_net_forward(self._net, kind, _lib.ptr(x), _lib.ptr(thresholds), levels, batch, _lib.ptr(counts),
                                           _lib.ptr(self._workspace), self._workspace.numel(), _lib.stream()))
        return counts

    # ---- CUDA graph replay for a fixed batch size (the runtime allocates nothing and never synchronises)
    def capture(self, example, thresholds=None):
        """Captures one forward call for ``example``'s shape and dtype (bool ``[B, F]`` / ``[B, C, H, W]``, or pixels
        with ``thresholds``) into a CUDA graph and returns ``replay(x) -> counts``: the input is copied into a
        static buffer, the graph is launched, and the static int32 ``[B, num_classes]`` result is returned (valid
        until the next replay).  Worth it for small networks, where a call is a dozen launches of a few
        microseconds each."""
        if self._net is None:
            raise RuntimeError("convlogic_b200: call compile() or load() first")
        pixels = thresholds is not None
        static_in = example.to(self.device).contiguous().clone()
        th = thresholds.to(self.device, torch.float32).contiguous() if pixels else None
        if not pixels:
            static_in = static_in.reshape(static_in.shape[0], -1).contiguous().view(torch.uint8)
        batch = static_in.shape[0]
        kind = (2 if static_in.dtype == torch.uint8 else 1) if pixels else 0
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):                      # warm-up outside the capture: shared-memory attributes, workspace
            for _ in range(2):
                self._run(kind, static_in, batch, th)
        torch.cuda.current_stream(self.device).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            static_out = self._run(kind, static_in, batch, th)

        def replay(x):
            x = x.to(self.device)
            static_in.copy_(x.reshape(static_in.shape) if pixels else x.reshape(batch, -1).view(torch.uint8))
            graph.replay()
            return static_out

        return replay

    def forward(self, x, verbose=False):
        """bool ``[B, F]`` or ``[B, C, H, W]`` (torch tensor or numpy array) -> int32 class counts ``[B, num_classes]``
        on the device."""
        del verbose
        if isinstance(x, np.ndarray):
            x = torch.from_numpy(x)
        x = x.to(self.device)
        if x.dtype not in (torch.bool, torch.uint8):
            raise RuntimeError("convlogic_b200: CompiledLogicNet.forward expects bool inputs")
        batch = x.shape[0]
        x = x.reshape(batch, -1).contiguous()
        if x.shape[1] != self.num_inputs:
            raise ValueError(f"expected {self.num_inputs} input bits per sample, got {x.shape[1]}")
        return self._run(0, x.view(torch.uint8), batch)

    def forward_packed(self, rows, batch):
        """Bit-packed input rows ``[in_features, 2 * ceil(batch / 128)]`` int64 (64 samples per word, the batch padded
        to whole 128-sample units with zero bits) -> counts for the first ``batch`` samples."""
        rows = rows.to(self.device).contiguous()
        words = 2 * (-(-batch // 128))
        if rows.dtype != torch.int64 or rows.dim() != 2 or rows.shape[0] != self.num_inputs or rows.shape[1] != words:
            raise ValueError(f"expected int64 rows [{self.num_inputs}, {words}], got {tuple(rows.shape)} {rows.dtype}")
        return self._run(3, rows, batch)

    def forward_pixels(self, pixels, thresholds):
        """float32 / uint8 pixels ``[B, C, H, W]`` + thermometer thresholds -> counts (input stage fused on the GPU)."""
        pixels = pixels.to(self.device).contiguous()
        thresholds = thresholds.to(self.device, torch.float32).contiguous()
        if pixels.dtype not in (torch.float32, torch.uint8):
            raise RuntimeError("convlogic_b200: pixels must be float32 or uint8")
        return self._run(2 if pixels.dtype == torch.uint8 else 1, pixels, pixels.shape[0], thresholds)
