"""The five entry points of the reference's ``PCEngine.backend`` extension
(backend/pybind_cuda.cpp:8-14) with the same positional signatures and the
same in-place contract, implemented on libpce_b200.so.  An unmodified
script/spconv.py that imports these names from here runs on the new kernels.

Differences a caller can observe:
  * work is enqueued on PyTorch's current stream, not legacy stream 0;
  * the ks == stride output-coordinate shortcut of backend/hash.cu:333-362 is not
    reproduced (it disagrees with the reference's own query kernel): the general
    rule is used for every kernel size and stride;
  * D1 buffer positions are canonical (index inside the offset's (kp, in)-ordered
    segment) instead of atomics-ordered;
  * features accumulate in fp32 and are written once, without atomics;
  * ``conv_bwd_d1_cuda`` raises: this is an inference engine.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._lib import lib
from .kmap import candidates_per_input, csr_from_pairs, make_geom


def _dec(code: int):
    x = code // 94273
    y = (code - x * 94273) // 311
    return (x, y, code - x * 94273 - y * 311)


def _mid(ks) -> int:
    return (ks[0] - 1) // 2 * ks[1] * ks[2] + (ks[1] - 1) // 2 * ks[2] + (ks[2] - 1) // 2


def _out_coords(in_coords, geom, ks, stride, separate_mid, st):
    if separate_mid:
        return in_coords, None  # the reference returns the very same tensor (backend/hash.cu:327-331)
    n_in = in_coords.size(0)
    dev = in_coords.device
    cap = max(1, n_in * candidates_per_input(ks, stride))
    ws = _lib.workspace(lib.pce_map_workspace_bytes(n_in, ks[0] * ks[1] * ks[2], cap), dev)
    oc = torch.empty((cap, 4), dtype=torch.int32, device=dev)
    n_out = C.c_int32(0)
    _lib.check(lib.pce_downsample_coords(in_coords.data_ptr(), n_in, C.byref(geom), ws.data_ptr(), ws.numel(),
                                         oc.data_ptr(), cap, C.byref(n_out), st), "pce_downsample_coords")
    return oc[: n_out.value].clone(), ws


def _build_d2(in_coords, k_size_code, k_vol, l_stride_code, padding_code, mins, maxs, map_, knnz, kpos, qkpos,
              separate_mid, want_map_out):
    _lib.require_cuda(in_coords, "in_coords")
    if in_coords.dtype != torch.int32:
        raise ValueError("in_coords must be int32")
    in_coords = in_coords if in_coords.is_contiguous() else in_coords.contiguous()
    ks, stride, pad = _dec(k_size_code), _dec(l_stride_code), _dec(padding_code)
    if ks[0] * ks[1] * ks[2] != k_vol:
        raise ValueError("kernel volume does not match the kernel size code")
    geom = make_geom(ks, stride, pad, mins, maxs, bool(separate_mid))
    dev = in_coords.device
    st = _lib.stream_ptr(dev)
    n_in = in_coords.size(0)
    out_coords, _ = _out_coords(in_coords, geom, ks, stride, separate_mid, st)
    n_out = out_coords.size(0)
    ws = _lib.workspace(lib.pce_map_workspace_bytes(n_in, k_vol, n_out), dev)
    map_out = None
    symmetric = bool(separate_mid) and all(k % 2 == 1 for k in ks)
    if want_map_out and not symmetric:
        map_out = torch.empty((k_vol * max(n_out, 1),), dtype=torch.int32, device=dev)
    kpos_full = kpos if kpos.numel() >= k_vol + 1 else torch.empty((k_vol + 1,), dtype=torch.int32, device=dev)
    _lib.check(lib.pce_map_build_d2(in_coords.data_ptr(), n_in, out_coords.data_ptr(), n_out, C.byref(geom),
                                    ws.data_ptr(), ws.numel(), _lib.ptr(map_), knnz.data_ptr(), kpos_full.data_ptr(),
                                    qkpos.data_ptr(), _lib.ptr(map_out), None, st), "pce_map_build_d2")
    if kpos_full is not kpos:  # the reference's D1 caller allocates kv entries only (script/spconv.py:396)
        kpos.copy_(kpos_full[: kpos.numel()])
    return out_coords, map_out, kpos_full, n_in, n_out, symmetric


def mapping_d2_cuda(in_coords, batch_size, k_size_code, k_vol, c_in, c_out, l_stride_code, t_stride_code,
                    padding_code, min_x, min_y, min_z, max_x, max_y, max_z, map, kernel_nnz, kernel_kpos,
                    kernel_qkpos, separate_mid):
    """HashMapD2 (backend/hash.h:37-58): fills ``map`` [kv*N_in], ``kernel_nnz`` [kv],
    ``kernel_kpos`` / ``kernel_qkpos`` [kv+1] in place and returns the output coordinates."""
    out_coords, _, _, _, _, _ = _build_d2(in_coords, k_size_code, k_vol, l_stride_code, padding_code,
                                       (min_x, min_y, min_z), (max_x, max_y, max_z), map, kernel_nnz, kernel_kpos,
                                       kernel_qkpos, separate_mid, False)
    return out_coords


def mapping_d1_cuda(in_coords, k_size_code, k_vol, c_in, c_out, l_stride_code, t_stride_code, padding_code,
                    min_x, min_y, min_z, max_x, max_y, max_z, imap, omap, icsr, ocsr, kernel_nnz, kernel_kpos,
                    kernel_qkpos, separate_mid):
    """HashMapD1 (backend/hash.h:11-34): fills the CSR-coded ``imap`` / ``omap`` (compacted
    at the front) and the row pointers ``icsr`` [N_in+1] / ``ocsr`` [N_out+1] in place."""
    dev = in_coords.device
    n_in = in_coords.size(0)
    dense = torch.empty((k_vol * max(n_in, 1),), dtype=torch.int32, device=dev)
    out_coords, map_out, kpos_full, n_in, n_out, symmetric = _build_d2(
        in_coords, k_size_code, k_vol, l_stride_code, padding_code, (min_x, min_y, min_z), (max_x, max_y, max_z),
        dense, kernel_nnz, kernel_kpos, kernel_qkpos, separate_mid, True)
    if imap.numel() < k_vol * n_in or omap.numel() < k_vol * n_out or icsr.numel() < n_in + 1 \
            or ocsr.numel() < n_out + 1:
        raise ValueError("mapping_d1_cuda: a map array is smaller than the reference's allocation")
    ws = _lib.workspace(8 * k_vol * max(n_in, 1) + 8 * (max(n_in, n_out) + 1) + (16 << 20), dev)
    _lib.check(lib.pce_map_build_d1(dense.data_ptr(), _lib.ptr(map_out), k_vol, n_in, n_out,
                                    1 if symmetric else 0, kpos_full.data_ptr(), ws.data_ptr(), ws.numel(),
                                    imap.data_ptr(), icsr.data_ptr(), omap.data_ptr(), ocsr.data_ptr(),
                                    _lib.stream_ptr(dev)), "pce_map_build_d1")
    return out_coords


def _flat_i32(t):
    t = t.reshape(-1)
    return t if t.dtype == torch.int32 else t.to(torch.int32)


def conv_fwd_d2_cuda(in_feats, kernel, ksize_code, sum_nnz, out_feats, kpos, qkpos, in_map, out_map, separate_mid,
                     tf32):
    """ConvolutionForwardD2 (backend/spconv.h:28-40): writes the convolution into
    ``out_feats`` in place.  ``in_map`` / ``out_map`` are the (kp, in)-ordered pair
    lists; the neighbour CSR derived from them is cached on ``out_map``."""
    _lib.require_cuda(in_feats, "in_feats")
    if in_feats.size(1) != kernel.size(1):
        raise ValueError("Input feature size and kernel size mismatch")
    kv, c_in, c_out = kernel.shape
    ks = _dec(ksize_code)
    n_in, n_out = in_feats.size(0), out_feats.size(0)
    ident = _mid(ks) if separate_mid else -1
    key = (in_map.data_ptr(), in_map._version, out_map._version, n_in, n_out, ident)
    cached = getattr(out_map, "_pce_csr", None)
    if cached is None or cached[0] != key:
        csr = csr_from_pairs(_flat_i32(out_map), _flat_i32(in_map), kpos, kv, n_out, n_in, ident)
        try:
            out_map._pce_csr = (key, csr)
        except AttributeError:
            pass
    else:
        csr = cached[1]
    if not out_feats.is_contiguous():
        raise ValueError("out_feats must be contiguous")
    feats = in_feats.contiguous()
    w = kernel.contiguous()
    if w.dtype != feats.dtype or out_feats.dtype != feats.dtype:
        raise ValueError("in_feats, kernel and out_feats must share one dtype")
    from .functional import packed_weights
    _lib.check(lib.pce_conv_fwd(feats.data_ptr(), n_in, c_in, w.data_ptr(), _lib.ptr(packed_weights(w)), kv, c_out,
                                csr.mask.data_ptr(), csr.rowptr.data_ptr(), csr.nbr.data_ptr(), C.byref(csr.tiles()),
                                n_out, out_feats.data_ptr(),
                                _lib.dtype_code(feats.dtype), None, _lib.KERNEL_AUTO, _lib.stream_ptr(feats.device)),
               "pce_conv_fwd")


def conv_fwd_d1_cuda(in_feats, kernel, ksize_code, qsum_nnz, out_feats, kernel_kpos, kernel_qkpos, in_map, out_map,
                     in_csr, out_csr, buffer, separate_mid, TensorCoreMode):
    """ConvolutionForwardD1 (backend/spconv.h:11-25): gather into ``buffer``, per-offset
    GEMM, CSR scatter into ``out_feats`` in place."""
    _lib.require_cuda(in_feats, "in_feats")
    if in_feats.size(1) != kernel.size(1):
        raise ValueError("Input feature size and kernel size mismatch")
    kv, c_in, c_out = kernel.shape
    ks = _dec(ksize_code)
    n_in, n_out = in_feats.size(0), out_feats.size(0)
    feats = in_feats.contiguous()
    w = kernel.contiguous()
    if w.dtype != feats.dtype or out_feats.dtype != feats.dtype:
        raise ValueError("in_feats, kernel and out_feats must share one dtype")
    qsum = int(qsum_nnz)
    if buffer.dtype != feats.dtype:
        buffer = buffer.view(torch.uint8).view(feats.dtype) if buffer.is_contiguous() else buffer.to(feats.dtype)
    from .functional import packed_weights
    _lib.check(lib.pce_conv_fwd_d1(feats.data_ptr(), n_in, c_in, w.data_ptr(), _lib.ptr(packed_weights(w)), kv, c_out,
                                   kernel_qkpos.data_ptr(),
                                   qsum, in_map.data_ptr(), in_csr.data_ptr(), out_map.data_ptr(),
                                   out_csr.data_ptr(), n_out, buffer.data_ptr(), buffer.numel() * buffer.element_size(),
                                   out_feats.data_ptr(), _lib.dtype_code(feats.dtype),
                                   _mid(ks) if separate_mid else -1, None, _lib.stream_ptr(feats.device)),
               "pce_conv_fwd_d1")


def conv_bwd_d1_cuda(*args, **kwargs):
    """ConvolutionBackwardD1 (backend/spconv.h:43-58) is not provided: inference only."""
    raise NotImplementedError("pcengine_b200 is an inference engine: conv_bwd_d1_cuda is not implemented")
