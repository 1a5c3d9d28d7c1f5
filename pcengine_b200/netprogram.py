"""``NetProgram``: a network pass as ONE call into the library (``pce_net_run``).

The reference runs a network layer by layer from Python (script/spconv.py:86-98: ``conv3d.forward``
-> ``conv_func`` per layer).  At ~100 k voxels per pass the host work per layer (dispatch, output
allocation, argument marshalling: ~40 us) is longer than the layer's kernel, so the GPU waits for
the interpreter.  A program describes the layers once -- feature matrices ("buffers") at the
coordinate levels of a :class:`~pcengine_b200.planner.MapPlan`, and operations that read and write
column ranges of them through the plan's kernel maps -- and ``run`` hands the whole list to the
library, which fetches each map from the planner as the layer that needs it comes up and queues
the tensor-core kernels.  The launches are the ones the per-layer path issues, in the same order:
results are bit-identical.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import torch

from . import _lib
from . import functional as PF
from ._lib import lib

INPUT, OUTPUT = -1, -2


class NetProgram:
    def __init__(self, dtype=torch.float16):
        if dtype != torch.float16:
            raise NotImplementedError("NetProgram runs fp16 networks on the tensor-core kernel")
        self.dtype = dtype
        self.buffers: List[tuple] = []   # (level, width)
        self.ops: List[dict] = []
        self._keep: List[torch.Tensor] = []  # every tensor an operation points at
        self._c = None
        self.in_width = self.out_width = None
        self.max_level = 0

    # -- declaration ------------------------------------------------------------------------
    def buffer(self, level: int, width: int) -> int:
        """A [rows of coordinate level ``level``, ``width``] feature matrix; returns its id."""
        if width % 8:
            raise ValueError("buffer widths are multiples of 8 channels")
        self.buffers.append((int(level), int(width)))
        self.max_level = max(self.max_level, int(level))
        return len(self.buffers) - 1

    def _width_of(self, buf: int, role: str) -> Optional[int]:
        if buf >= 0:
            return self.buffers[buf][1]
        return None

    def _weights(self, kernel: torch.Tensor, as_linear: bool):
        packed = PF.packed_weights(kernel, as_linear=as_linear)
        if packed is None:
            raise NotImplementedError("NetProgram needs channel counts the tensor-core kernel covers "
                                      "(multiples of 16, at most 256 outputs)")
        self._keep += [kernel, packed]
        return packed

    def _const(self, t: Optional[torch.Tensor], c_out: int):
        if t is None:
            return None
        if t.dtype != torch.float32 or t.numel() != c_out or not t.is_cuda or not t.is_contiguous():
            raise ValueError(f"epilogue constants are contiguous fp32 CUDA tensors of {c_out} elements")
        self._keep.append(t)
        return t

    def conv(self, map_index: int, transposed: bool, kernel: torch.Tensor, src, dst, scale=None, shift=None, act=None,
             slope: float = 0.01, extra=None, extra_weight: Optional[torch.Tensor] = None) -> None:
        """Sparse convolution through plan map ``map_index``: ``kernel`` [kv,C_in,C_out] (fp16, CUDA,
        widths multiples of 16); ``src`` / ``dst`` = (buffer id, first column); ``extra`` = id of a whole
        buffer that joins the accumulator through ``extra_weight`` [C2, C_out]."""
        kv, c_in, c_out = kernel.shape
        op = dict(kind=0, map=int(map_index), transposed=1 if transposed else 0, kv=kv, c_in=c_in, c_out=c_out,
                  src=src, dst=dst, packed=self._weights(kernel, False), scale=self._const(scale, c_out),
                  shift=self._const(shift, c_out), act=PF._ACT[act], slope=float(slope), extra=-1, extra_c=0, extra_packed=None)
        if extra is not None:
            c2 = extra_weight.size(0)
            if extra < 0 or self.buffers[extra][1] != c2 or extra_weight.size(1) != c_out:
                raise ValueError("the second operand is a whole buffer whose width is extra_weight's first dimension")
            op.update(extra=int(extra), extra_c=int(c2), extra_packed=self._weights(extra_weight, True))
        self.ops.append(op)
        self._c = None

    def linear(self, weight: torch.Tensor, src, dst, scale=None, shift=None, act=None, slope: float = 0.01) -> None:
        """Dense rows x matrix product (a 1x1x1 layer): ``weight`` [C_in, C_out]."""
        c_in, c_out = weight.shape
        self.ops.append(dict(kind=1, map=-1, transposed=0, kv=1, c_in=c_in, c_out=c_out, src=src, dst=dst,
                             packed=self._weights(weight, True), scale=self._const(scale, c_out),
                             shift=self._const(shift, c_out), act=PF._ACT[act], slope=float(slope), extra=-1, extra_c=0,
                             extra_packed=None))
        self._c = None

    # -- execution ----------------------------------------------------------------------------
    def _compile(self):
        bufs = (_lib.NetBuffer * max(len(self.buffers), 1))()
        for b, (level, width) in zip(bufs, self.buffers):
            b.level, b.width = level, width
        ops = (_lib.NetOp * len(self.ops))()
        for c, o in zip(ops, self.ops):
            c.kind, c.map, c.transposed, c.kv, c.c_in, c.c_out = o["kind"], o["map"], o["transposed"], o["kv"], o["c_in"], o["c_out"]
            c.src_buf, c.src_col = o["src"]
            c.dst_buf, c.dst_col = o["dst"]
            c.packed_weights = o["packed"].data_ptr()
            c.scale = _lib.ptr(o["scale"])
            c.shift = _lib.ptr(o["shift"])
            c.act, c.slope = o["act"], o["slope"]
            c.extra_buf, c.extra_col, c.extra_c = o["extra"], 0, o["extra_c"]
            c.extra_packed_weights = _lib.ptr(o["extra_packed"])
        self._c = (bufs, ops)
        self.row_width = sum(w for _, w in self.buffers)  # arena bytes per input row (upper bound: rows never grow)
        return self._c

    def arena_bytes(self, n_rows: int) -> int:
        if self._c is None:
            self._compile()
        # + room for the fp32 partial sums of split layers (small maps): a part count P is chosen so that
        # P x tiles <= 1.5 x the GPU's CTA slots, i.e. at most ~90 MB per layer, placed afresh when it grows
        return 2 * n_rows * self.row_width + 256 * (len(self.buffers) + 1) + (400 << 20)

    def run(self, pass_handle: int, feats: torch.Tensor, out: torch.Tensor, arena: torch.Tensor) -> None:
        """Queue the whole pass on the current stream.  ``feats`` [N, C_in of the first layer] and ``out``
        [N, C_out of the last] are row-major fp16 (row pitch = width)."""
        bufs, ops = self._c or self._compile()
        _lib.check(lib.pce_net_run(pass_handle, bufs, len(self.buffers), ops, len(self.ops), feats.data_ptr(), feats.stride(0),
                                   out.data_ptr(), out.stride(0), arena.data_ptr(), arena.numel(), _lib.PCE_F16,
                                   _lib.stream_ptr(feats.device)), "pce_net_run")
