"""Thin tensor-level wrappers over the convolution entry points of the C ABI."""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib
from ._lib import lib
from .kmap import NeighbourCSR

_ACT = {None: _lib.ACT_NONE, "none": _lib.ACT_NONE, "relu": _lib.ACT_RELU, "leaky": _lib.ACT_LEAKY}
_KERNEL = {"auto": _lib.KERNEL_AUTO, "simt": _lib.KERNEL_SIMT, "umma": _lib.KERNEL_UMMA}
_KERNEL_NAME = {_lib.KERNEL_SIMT: "conv_simt", _lib.KERNEL_UMMA: "conv_umma"}

# When set to a list, every conv_forward call appends a record with CUDA events around its
# kernel launch (used by the benchmark to time the convolution kernels inside a model).
PROFILE = None
# Form the tensor-core kernel's tiles in bitmask-sorted row order (scheduling only; results are unchanged).
SORT_ROWS = True
# Rows per tile of the tensor-core kernel: 128, 256, or None for the automatic choice.
TILE_ROWS = None
# Take the offsets of layers with 16 / 32 input channels four / two per stage (scheduling only).
PACK_OFFSETS = True


class FusedEpilogue:
    """y = act(acc*scale + shift + residual); scale/shift are fp32 [C_out] CUDA tensors.

    ``extra_feats`` [N_out, C2] with ``extra_weight`` [C2, C_out] is a second operand that joins the
    accumulator itself, acc[row] += extra_feats[row] @ extra_weight (tensor-core kernel only, see
    :func:`supports_second_operand`): a block's residual (identity weight) or its 1x1x1 shortcut
    convolution, gathered by the kernel's pipeline instead of read in its epilogue.

    ``push_slots`` / ``push_bases``: the halo push of a slab-parallel scene (see
    ``multigpu.SlabScene.push_epilogue``): output row r is also stored to peer memory
    ``push_bases[s] + push_slots[s][r] * C_out`` for the slots that are >= 0."""

    __slots__ = ("scale", "shift", "residual", "act", "slope", "extra_feats", "extra_weight", "push_slots", "push_bases")

    def __init__(self, scale=None, shift=None, residual=None, act=None, slope=0.01, extra_feats=None,
                 extra_weight=None, push_slots=None, push_bases=None):
        self.scale, self.shift, self.residual, self.act, self.slope = scale, shift, residual, act, slope
        self.extra_feats, self.extra_weight = extra_feats, extra_weight
        self.push_slots, self.push_bases = push_slots, push_bases

    def replace(self, **fields) -> "FusedEpilogue":
        """A copy with ``fields`` replaced and every other field carried over."""
        kw = {name: getattr(self, name) for name in self.__slots__}
        kw.update(fields)
        return FusedEpilogue(**kw)

    def pack(self, c_out: int, n_out: int, dtype) -> _lib.Epilogue:
        e = _lib.Epilogue()
        for name in ("scale", "shift"):
            t = getattr(self, name)
            if t is not None:
                if t.dtype != torch.float32 or not t.is_cuda or t.numel() != c_out or not t.is_contiguous():
                    raise ValueError(f"epilogue {name} must be a contiguous fp32 CUDA tensor of {c_out} elements")
                setattr(e, name, t.data_ptr())
        if self.residual is not None:
            r = self.residual
            if r.dtype != dtype or tuple(r.shape) != (n_out, c_out) or not r.is_contiguous():
                raise ValueError("epilogue residual must match the output's shape and dtype")
            e.residual = r.data_ptr()
        e.act = _ACT[self.act]
        e.slope = float(self.slope)
        if self.extra_feats is not None:
            x2, w2 = self.extra_feats, self.extra_weight
            if w2 is None or w2.dim() != 2 or w2.size(1) != c_out or w2.size(0) != x2.size(1):
                raise ValueError("extra_weight must be [C2, C_out] for extra_feats [N_out, C2]")
            if x2.dtype != dtype or w2.dtype != dtype or tuple(x2.shape) != (n_out, w2.size(0)) or not x2.is_contiguous():
                raise ValueError("extra_feats must be contiguous [N_out, C2] in the features' dtype")
            packed = packed_weights(w2, as_linear=True) if w2.is_contiguous() else None
            if packed is None:
                raise NotImplementedError("the second operand needs fp16 and channel counts that are multiples of 16")
            e.extra_feats, e.extra_packed_weights, e.extra_c = x2.data_ptr(), packed.data_ptr(), w2.size(0)
        if self.push_slots is not None:
            for s, (slots, base) in enumerate(zip(self.push_slots, self.push_bases)):
                if slots is None or not base:
                    continue
                if slots.dtype != torch.int32 or slots.numel() != n_out or not slots.is_contiguous() or not slots.is_cuda:
                    raise ValueError("push_slots must be contiguous int32 CUDA tensors with one entry per output row")
                e.push_slot[s], e.push_base[s] = slots.data_ptr(), int(base)
        return e


def stage_slots(c_in: int) -> int:
    """Offsets per stage of the tile lists a layer with ``c_in`` (padded) input channels uses: a
    16- or 32-channel offset fills a quarter or half of the kernel's 64-channel K block."""
    if not PACK_OFFSETS:
        return 1
    return 4 if c_in == 16 else (2 if c_in == 32 else 1)


def supports_second_operand(dtype, c_in: int, c_out: int, c2: int) -> bool:
    """Whether a convolution with these widths can take ``FusedEpilogue.extra_feats``."""
    return (dtype == torch.float16 and c_in % 16 == 0 and c_out % 16 == 0 and c2 % 16 == 0 and 16 <= c_out <= 256
            and c2 >= 16)


def _pack(ep: Optional[FusedEpilogue], c_out, n_out, dtype, in_ld: int = 0, out_ld: int = 0, split=None):
    if ep is None and not in_ld and not out_ld and split is None:
        return None
    e = ep.pack(c_out, n_out, dtype) if ep is not None else _lib.Epilogue()
    e.in_ld, e.out_ld = in_ld, out_ld
    if split is not None:
        e.split_scratch, e.split_scratch_bytes = split.data_ptr(), split.numel() * split.element_size()
    return C.byref(e)


# Split the stage chains of maps with few tiles over several CTAs per tile (pce_conv_split_parts).
SPLIT_TILES = True


def _split_scratch(n_rows: int, n_src: int, c_in: int, c_out: int, kv: int, device):
    """fp32 scratch for the partial sums of a layer that the library will split, or None."""
    if not SPLIT_TILES:
        return None
    idx = device.index if device.index is not None else torch.cuda.current_device()
    sms = _SM_COUNT.get(idx)
    if sms is None:
        sms = _SM_COUNT[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    nbytes = int(lib.pce_conv_split_scratch_bytes(n_rows, n_src, c_in, c_out, kv, sms))
    if nbytes <= 0:
        return None
    return torch.empty((nbytes // 4,), dtype=torch.float32, device=device)


def _row_pitched(t: torch.Tensor) -> bool:
    """A [N, C] fp16 matrix the tensor-core kernel can address in place: rows contiguous, at a pitch
    that is a multiple of 8 elements, 16-byte aligned (a column range of a wider matrix qualifies)."""
    return (t.dim() == 2 and t.dtype == torch.float16 and t.stride(1) == 1 and t.stride(0) >= t.size(1)
            and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0)


def packed_weights(kernel: torch.Tensor, as_linear: bool = False) -> Optional[torch.Tensor]:
    """The tensor-core layout of ``kernel`` [kv,C_in,C_out], or None when the tensor-core kernel
    does not cover these channel counts.  The result is cached ON the tensor object (together
    with its version counter and address), so it lives and dies with the weights; a tensor
    that is rebuilt on every call is simply packed again."""
    tag = (kernel._version, kernel.data_ptr(), kernel.shape, as_linear)
    hit = getattr(kernel, "_pce_packed", None)
    if hit is not None and hit[0] == tag:
        return hit[1]
    kv, c_in, c_out = ((1,) + tuple(kernel.shape)) if as_linear else kernel.shape
    code = _lib.dtype_code(kernel.dtype)
    if lib.pce_conv_kernel_choice(c_in, c_out, code, _lib.KERNEL_UMMA) != _lib.KERNEL_UMMA or kv > 128:
        try:
            kernel._pce_packed = (tag, None)  # remembered like a packed layout: this tensor has none
        except AttributeError:
            pass
        return None
    out = torch.empty((lib.pce_packed_weights_bytes(kv, c_in, c_out),), dtype=torch.uint8, device=kernel.device)
    _lib.check(lib.pce_pack_weights(kernel.data_ptr(), kv, c_in, c_out, code, out.data_ptr(),
                                    _lib.stream_ptr(kernel.device)), "pce_pack_weights")
    try:
        kernel._pce_packed = (tag, out)
    except AttributeError:
        pass
    return out


def invalidate_packed(module_or_tensor) -> None:
    """Drop the cached tensor-core layouts (packed, padded) of a weight tensor or of every parameter
    of a module.  The caches are keyed by the tensor's version counter and address, which in-place
    writes through ``param.copy_`` or ``load_state_dict`` advance; writes through ``.data`` (``param.data.copy_``,
    ``param.data.uniform_``) do not, so call this after them."""
    tensors = [module_or_tensor] if isinstance(module_or_tensor, torch.Tensor) else list(module_or_tensor.parameters())
    if not isinstance(module_or_tensor, torch.Tensor):
        for m in module_or_tensor.modules():  # whole-pass programs and folded constants point at the old layouts
            m.__dict__.pop("_programs", None)
            if hasattr(m, "_folded"):
                m._folded = {}
    for t in tensors:
        for name in ("_pce_packed", "_pce_padded"):
            if hasattr(t, name):
                try:
                    delattr(t, name)
                except AttributeError:
                    pass


def _ceil16(c: int) -> int:
    return (int(c) + 15) // 16 * 16


def _padded_kernel(kernel: torch.Tensor, cin_p: int, cout_p: int) -> torch.Tensor:
    """``kernel`` [(kv,)C_in,C_out] zero-padded to [(kv,)cin_p,cout_p]; cached on the tensor like
    the packed layout, so static weights are padded once."""
    tag = (kernel._version, kernel.data_ptr(), tuple(kernel.shape), cin_p, cout_p)
    hit = getattr(kernel, "_pce_padded", None)
    if hit is not None and hit[0] == tag:
        return hit[1]
    c_in, c_out = kernel.shape[-2:]
    out = torch.nn.functional.pad(kernel.detach(), (0, cout_p - c_out, 0, cin_p - c_in)).contiguous()
    try:
        kernel._pce_padded = (tag, out)
    except AttributeError:
        pass
    return out


def _pad_for_tensor_cores(feats, kernel, epilogue, kernel_choice):
    """fp16 layers whose channel counts are not multiples of 16 (a 4-channel stem, a 19-class head)
    still run on the tensor-core kernel: input channels, weights and the per-channel epilogue
    constants are zero-padded to the next multiple of 16 and the caller drops the extra output
    columns.  The padded products are exact zeros, so the result is the unpadded one.  Returns
    (feats, kernel, epilogue, padded) with ``padded`` False when nothing changed."""
    kv, c_in, c_out = ((1,) + tuple(kernel.shape)) if kernel.dim() == 2 else kernel.shape
    cin_p, cout_p = _ceil16(c_in), _ceil16(c_out)
    if feats.dtype != torch.float16 or kernel_choice == "simt" or (cin_p == c_in and cout_p == c_out) \
            or cout_p > 256 or kv > 128:
        return feats, kernel, epilogue, False
    if cout_p != c_out and epilogue is not None and (epilogue.residual is not None or epilogue.extra_feats is not None
                                                     or epilogue.push_slots is not None):
        # operands shaped like the output (residual, second operand's weights, halo rows) are not
        # widened here: such a layer keeps its channel count and runs on the CUDA-core kernel
        return feats, kernel, epilogue, False
    kernel = _padded_kernel(kernel, cin_p, cout_p)
    if cin_p != c_in:  # (torch.nn.functional.pad costs 0.3 ms of host time here; cat does not)
        feats = torch.cat([feats, feats.new_zeros((feats.size(0), cin_p - c_in))], dim=1)
    if cout_p != c_out and epilogue is not None:
        def widen(t):
            return None if t is None else torch.cat([t, t.new_zeros((cout_p - c_out,))])
        epilogue = epilogue.replace(scale=widen(epilogue.scale), shift=widen(epilogue.shift))
    return feats, kernel, epilogue, True


_SM_COUNT = {}
_TILE_ROWS_MEMO = {}


def _auto_tile_rows(n_rows: int, c_in: int, c_out: int, device) -> int:
    """Rows per tile of the tensor-core kernel (pce_tile_rows_for): 128 rows times the sub-tiles that
    share every staged weight block (up to four, bounded by tensor memory and the map's size)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    key = (n_rows, c_in, c_out, idx)
    rows = _TILE_ROWS_MEMO.get(key)
    if rows is None:
        sms = _SM_COUNT.get(idx)
        if sms is None:
            sms = _SM_COUNT[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
        if len(_TILE_ROWS_MEMO) > 4096:
            _TILE_ROWS_MEMO.clear()
        rows = _TILE_ROWS_MEMO[key] = int(lib.pce_tile_rows_for(n_rows, c_in, c_out, sms))
    return rows


def device_status(reset: bool = True) -> int:
    """The library's device status word (0 = ok); synchronises the device."""
    v = C.c_int32(0)
    _lib.check(lib.pce_device_status(C.byref(v), 1 if reset else 0), "pce_device_status")
    return int(v.value)


def conv_forward(feats: torch.Tensor, kernel: torch.Tensor, csr: NeighbourCSR, epilogue: Optional[FusedEpilogue] = None,
                 kernel_choice: str = "auto", out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Fused gather-matmul-scatter over a neighbour CSR; returns [csr.n_rows, C_out] (written into
    ``out`` when given: a tensor of that shape and the features' dtype).  On the tensor-core path
    ``feats`` and ``out`` may be column ranges of wider row-major matrices (see :func:`_row_pitched`);
    they are then read and written in place."""
    _lib.require_cuda(feats, "feats")
    _lib.require_cuda(kernel, "kernel")
    if kernel.dim() == 2:
        kernel = kernel.unsqueeze(0)
    if not _row_pitched(feats):
        feats = feats.contiguous()
    if not kernel.is_contiguous() or kernel.dtype != feats.dtype:
        kernel = kernel.detach().contiguous().to(feats.dtype)
    if feats.size(1) != kernel.size(1):
        raise ValueError("Input feature size and kernel size mismatch")
    if feats.size(0) != csr.n_src:
        raise ValueError(f"feature rows ({feats.size(0)}) do not match the kernel map ({csr.n_src})")
    c_out_true = kernel.size(2)
    second = epilogue is not None and epilogue.extra_feats is not None
    if second and (kernel_choice == "simt" or kernel.size(0) > 128
                   or not supports_second_operand(feats.dtype, kernel.size(1), c_out_true, epilogue.extra_feats.size(1))):
        raise NotImplementedError("a second operand (FusedEpilogue.extra_feats) needs the tensor-core kernel")
    feats, kernel, epilogue, padded = _pad_for_tensor_cores(feats, kernel, epilogue, kernel_choice)
    kv, c_in, c_out = kernel.shape
    packed = packed_weights(kernel) if kernel_choice != "simt" else None
    if packed is None:
        feats = feats.contiguous()  # row pitches are the tensor-core kernel's
    given = None
    if out is not None and (tuple(out.shape) != (csr.n_rows, c_out_true) or out.dtype != feats.dtype):
        raise ValueError("`out` must be a [n_rows, C_out] tensor in the features' dtype")
    if out is not None and (padded or (not out.is_contiguous() and (packed is None or not _row_pitched(out)))):
        given, out = out, None  # computed into a tensor of this function's own, then copied
    if out is None:
        out = torch.empty((csr.n_rows, c_out), dtype=feats.dtype, device=feats.device)
    if csr.n_rows == 0:  # nothing to compute: an empty tensor stays empty
        return given if given is not None else (out[:, :c_out_true] if padded else out)
    in_ld = 0 if feats.is_contiguous() else feats.stride(0)
    out_ld = 0 if out.is_contiguous() else out.stride(0)
    rec = None
    if PROFILE is not None:
        which = _lib.KERNEL_UMMA if packed is not None else _lib.KERNEL_SIMT
        rec = dict(kernel=_KERNEL_NAME.get(which, "none"), n_in=feats.size(0), n_out=csr.n_rows, cin=c_in, cout=c_out,
                   kv=kv, esize=feats.element_size(),
                   extra_c=epilogue.extra_feats.size(1) if second else 0,
                   residual=epilogue is not None and epilogue.residual is not None,
                   start=torch.cuda.Event(enable_timing=True), end=torch.cuda.Event(enable_timing=True))
        rec["start"].record()
    tiles = split = None
    if packed is not None:
        # (the halo push lives in the one-accumulator kernel: 128-row tiles)
        pushes = epilogue is not None and epilogue.push_slots is not None
        rows = TILE_ROWS or (128 if pushes else _auto_tile_rows(csr.n_rows, c_in, c_out, feats.device))
        tiles = C.byref(csr.tiles(SORT_ROWS, rows, second, stage_slots(c_in)))
        if rows == 128 and not pushes:
            split = _split_scratch(csr.n_rows, feats.size(0), c_in, c_out, kv, feats.device)
    # the tensor-core kernel reads the tile lists only: a planned map's rowptr / nbr are not built for its sake
    rowptr, nbr = (csr._rowptr, csr._nbr) if tiles is not None else (csr.rowptr, csr.nbr)
    _lib.check(lib.pce_conv_fwd(feats.data_ptr(), feats.size(0), c_in, kernel.data_ptr(), _lib.ptr(packed), kv, c_out,
                                csr.mask.data_ptr(), _lib.ptr(rowptr), _lib.ptr(nbr), tiles, csr.n_rows,
                                out.data_ptr(), _lib.dtype_code(feats.dtype),
                                _pack(epilogue, c_out, csr.n_rows, feats.dtype, in_ld, out_ld, split),
                                _KERNEL[kernel_choice], _lib.stream_ptr(feats.device)), "pce_conv_fwd")
    if rec is not None:
        rec["end"].record()
        rec["pairs"] = csr.pair_count()  # (a new tensor: the record must not keep the map's storage alive)
        PROFILE.append(rec)
    if given is not None:
        given.copy_(out[:, :c_out_true])
        return given
    return out[:, :c_out_true].contiguous() if padded and c_out != c_out_true else out


def conv_forward_d1(feats: torch.Tensor, kernel: torch.Tensor, kmap, transposed: bool = False,
                    epilogue: Optional[FusedEpilogue] = None, buffer: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Explicit gather -> per-offset GEMM -> scatter over a buffer of qsum x (C_in + C_out) elements
    (the reference's D1 dataflow, script/spconv.py:146-161): ``kmap`` is a KernelMap, whose CSR-coded
    forms are used; a transposed layer swaps the two sides (script/spconv.py:142-151).  ``buffer`` may
    be a caller workspace (as ``spTensor.buffer``); it is allocated when missing or too small."""
    _lib.require_cuda(feats, "feats")
    if kernel.dim() == 2:
        kernel = kernel.unsqueeze(0)
    feats = feats.contiguous()
    if not kernel.is_contiguous() or kernel.dtype != feats.dtype:
        kernel = kernel.detach().contiguous().to(feats.dtype)
    if feats.size(1) != kernel.size(1):
        raise ValueError("Input feature size and kernel size mismatch")
    kv, c_in, c_out = kernel.shape
    imap_c, icsr, omap_c, ocsr = kmap.d1()
    _, qsum = kmap.sizes()
    n_in, n_out = kmap.n_in, kmap.n_out
    if transposed:
        imap_c, icsr, omap_c, ocsr = omap_c, ocsr, imap_c, icsr
        n_in, n_out = n_out, n_in
    if feats.size(0) != n_in:
        raise ValueError(f"feature rows ({feats.size(0)}) do not match the kernel map ({n_in})")
    esize = feats.element_size()
    need = qsum * (c_in + c_out) * esize + 1032 * (qsum // 128) + 1024
    if buffer is None or buffer.numel() * buffer.element_size() < need or not buffer.is_cuda:
        buffer = torch.empty((need,), dtype=torch.uint8, device=feats.device)
    out = torch.empty((n_out, c_out), dtype=feats.dtype, device=feats.device)
    packed = packed_weights(kernel)
    centre = kmap.mid if (kmap.subm and not transposed) else -1
    _lib.check(lib.pce_conv_fwd_d1(feats.data_ptr(), n_in, c_in, kernel.data_ptr(), _lib.ptr(packed), kv, c_out,
                                   kmap.qkpos.data_ptr(), qsum, imap_c.data_ptr(), icsr.data_ptr(), omap_c.data_ptr(),
                                   ocsr.data_ptr(), n_out, buffer.data_ptr(), buffer.numel() * buffer.element_size(),
                                   out.data_ptr(), _lib.dtype_code(feats.dtype), centre,
                                   _pack(epilogue, c_out, n_out, feats.dtype), _lib.stream_ptr(feats.device)),
               "pce_conv_fwd_d1")
    return out


def linear_forward(feats: torch.Tensor, weight: torch.Tensor, epilogue: Optional[FusedEpilogue] = None) -> torch.Tensor:
    """feats [N,C_in] @ weight [C_in,C_out] with the fused epilogue (the 1x1x1 shortcut)."""
    _lib.require_cuda(feats, "feats")
    feats = feats.contiguous()
    if not weight.is_contiguous() or weight.dtype != feats.dtype:
        weight = weight.detach().contiguous().to(feats.dtype)
    if feats.size(1) != weight.size(0):
        raise ValueError("Input feature size and kernel size mismatch")
    c_out_true = weight.size(1)
    feats, weight, epilogue, padded = _pad_for_tensor_cores(feats, weight, epilogue, "auto")
    n, c_in = feats.shape
    c_out = weight.size(1)
    out = torch.empty((n, c_out), dtype=feats.dtype, device=feats.device)
    packed = packed_weights(weight, as_linear=True)
    _lib.check(lib.pce_linear_fwd(feats.data_ptr(), n, c_in, weight.data_ptr(), _lib.ptr(packed), c_out, out.data_ptr(),
                                  _lib.dtype_code(feats.dtype), _pack(epilogue, c_out, n, feats.dtype),
                                  _lib.stream_ptr(feats.device)), "pce_linear_fwd")
    return out[:, :c_out_true].contiguous() if padded and c_out != c_out_true else out


def scale_shift_act(feats: torch.Tensor, epilogue: FusedEpilogue) -> torch.Tensor:
    """Stand-alone per-channel affine + activation over feature rows."""
    _lib.require_cuda(feats, "feats")
    feats = feats.contiguous()
    n, c = feats.shape
    out = torch.empty_like(feats)
    _lib.check(lib.pce_scale_shift_act(feats.data_ptr(), n, c, out.data_ptr(), _lib.dtype_code(feats.dtype),
                                       _pack(epilogue, c, n, feats.dtype), _lib.stream_ptr(feats.device)),
               "pce_scale_shift_act")
    return out
