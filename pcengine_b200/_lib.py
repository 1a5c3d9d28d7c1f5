"""ctypes binding of libpce_b200.so (the C ABI declared in include/pce_b200.h).

There is no CPU fallback: importing this module without the built library, or
calling into it without a CUDA device, raises.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# PCE_B200_LIB: path of an alternative build of the library (an instrumented or debug build)
LIB_PATH = os.environ.get("PCE_B200_LIB") or os.path.join(_HERE, "libpce_b200.so")

PCE_OK = 0
PCE_ERR_INVALID = 1
PCE_ERR_CAPACITY = 8
PCE_F32, PCE_F16 = 0, 1
ACT_NONE, ACT_RELU, ACT_LEAKY = 0, 1, 2
KERNEL_AUTO, KERNEL_SIMT, KERNEL_UMMA = 0, 1, 2

EXPORTS = [
    "pce_strerror", "pce_version", "pce_last_cuda_error", "pce_kernel_launches", "pce_map_workspace_bytes", "pce_downsample_coords",
    "pce_map_build_d2", "pce_map_build_d2_noalloc", "pce_map_pairs", "pce_map_build_d1", "pce_csr_from_dense", "pce_csr_from_pairs",
    "pce_csr_from_pairs_workspace_bytes", "pce_csr_sort_rows", "pce_build_tile_lists", "pce_conv_kernel_choice", "pce_conv_split_parts", "pce_conv_split_scratch_bytes", "pce_conv_fwd", "pce_packed_weights_bytes",
    "pce_pack_weights", "pce_device_status", "pce_debug_timeout", "pce_tune", "pce_conv_fwd_d1", "pce_linear_fwd", "pce_scale_shift_act", "pce_push_rows",
    "pce_quantize_workspace_bytes", "pce_quantize_unique", "pce_tile_rows_for", "pce_plan_create", "pce_plan_destroy", "pce_plan_begin", "pce_pass_map", "pce_pass_release", "pce_net_run",
]


class Geom(C.Structure):
    _fields_ = [("ks", C.c_int32 * 3), ("stride", C.c_int32 * 3), ("pad", C.c_int32 * 3),
                ("cmin", C.c_int32 * 3), ("cmax", C.c_int32 * 3), ("submanifold", C.c_int32)]


class TileLists(C.Structure):
    _fields_ = [("order", C.c_void_p), ("tile_ptr", C.c_void_p), ("stage_kp", C.c_void_p), ("stage_nbr", C.c_void_p),
                ("tile_rows", C.c_int32), ("identity_stage", C.c_int32), ("slots", C.c_int32),
                ("settled", C.c_int32)]


PLAN_MAX_USES = 8


class PlanMapSpec(C.Structure):
    _fields_ = [("ks", C.c_int32 * 3), ("stride", C.c_int32 * 3), ("pad", C.c_int32 * 3), ("in_level", C.c_int32),
                ("submanifold", C.c_int32), ("want_fwd", C.c_int32), ("want_tr", C.c_int32),
                ("c_out_fwd", C.c_int32 * PLAN_MAX_USES), ("c_out_tr", C.c_int32 * PLAN_MAX_USES),
                ("c_in_fwd", C.c_int32 * PLAN_MAX_USES), ("c_in_tr", C.c_int32 * PLAN_MAX_USES)]


class PlannedCSR(C.Structure):
    _fields_ = [("mask", C.c_void_p), ("rowptr", C.c_void_p), ("nbr", C.c_void_p), ("n_rows", C.c_int32),
                ("n_src", C.c_int32), ("nbr_cap", C.c_int32), ("n_lists", C.c_int32),
                ("table", C.c_void_p), ("reverse_kp", C.c_int32), ("identity_kp", C.c_int32),
                ("lists", TileLists * PLAN_MAX_USES)]


class PlannedMap(C.Structure):
    _fields_ = [("n_in", C.c_int32), ("n_out", C.c_int32), ("kv", C.c_int32), ("symmetric", C.c_int32),
                ("cmax_out", C.c_int32 * 3), ("in_coords", C.c_void_p), ("out_coords", C.c_void_p), ("map", C.c_void_p),
                ("map_out", C.c_void_p), ("knnz", C.c_void_p), ("kpos", C.c_void_p), ("qkpos", C.c_void_p),
                ("status", C.c_void_p), ("has_fwd", C.c_int32), ("has_tr", C.c_int32), ("fwd", PlannedCSR),
                ("tr", PlannedCSR)]


class NetBuffer(C.Structure):
    _fields_ = [("level", C.c_int32), ("width", C.c_int32)]


class NetOp(C.Structure):
    _fields_ = [("kind", C.c_int32), ("map", C.c_int32), ("transposed", C.c_int32), ("kv", C.c_int32), ("c_in", C.c_int32),
                ("c_out", C.c_int32), ("src_buf", C.c_int32), ("src_col", C.c_int32), ("dst_buf", C.c_int32),
                ("dst_col", C.c_int32), ("packed_weights", C.c_void_p), ("scale", C.c_void_p), ("shift", C.c_void_p),
                ("act", C.c_int32), ("slope", C.c_float), ("extra_buf", C.c_int32), ("extra_col", C.c_int32),
                ("extra_c", C.c_int32), ("extra_packed_weights", C.c_void_p)]


class Epilogue(C.Structure):
    _fields_ = [("scale", C.c_void_p), ("shift", C.c_void_p), ("residual", C.c_void_p),
                ("act", C.c_int32), ("slope", C.c_float), ("extra_feats", C.c_void_p),
                ("extra_packed_weights", C.c_void_p), ("extra_c", C.c_int32),
                ("push_slot", C.c_void_p * 2), ("push_base", C.c_void_p * 2),
                ("in_ld", C.c_int32), ("out_ld", C.c_int32), ("split_scratch", C.c_void_p), ("split_scratch_bytes", C.c_size_t)]


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python pcengine_b200/csrc/build.py` "
            "(nvcc, sm_100a). pcengine_b200 has no CPU or PyTorch fallback.")
    lib = C.CDLL(LIB_PATH)
    vp, i32, i64, sz = C.c_void_p, C.c_int32, C.c_int64, C.c_size_t
    lib.pce_strerror.restype = C.c_char_p
    lib.pce_strerror.argtypes = [C.c_int]
    lib.pce_version.restype = C.c_int
    lib.pce_last_cuda_error.restype = C.c_int
    lib.pce_kernel_launches.restype = C.c_uint64
    lib.pce_map_workspace_bytes.restype = sz
    lib.pce_map_workspace_bytes.argtypes = [i32, i32, i32]
    lib.pce_downsample_coords.argtypes = [vp, i32, C.POINTER(Geom), vp, sz, vp, i32, C.POINTER(i32), vp]
    lib.pce_map_build_d2.argtypes = [vp, i32, vp, i32, C.POINTER(Geom), vp, sz, vp, vp, vp, vp, vp, vp, vp]
    lib.pce_map_build_d2_noalloc.argtypes = [vp, i32, vp, i32, C.POINTER(Geom), vp, vp, vp, vp, vp, vp, vp]
    lib.pce_map_pairs.argtypes = [vp, i32, i32, vp, sz, vp, vp, i32, vp]
    lib.pce_map_build_d1.argtypes = [vp, vp, i32, i32, i32, i32, vp, vp, sz, vp, vp, vp, vp, vp]
    lib.pce_csr_from_dense.argtypes = [vp, i32, i32, i32, i32, vp, sz, vp, vp, vp, i32, vp]
    lib.pce_csr_from_pairs.argtypes = [vp, vp, vp, i32, i32, i32, i32, vp, sz, vp, vp, vp, i32, vp]
    lib.pce_csr_from_pairs_workspace_bytes.restype = sz
    lib.pce_csr_from_pairs_workspace_bytes.argtypes = [i32, i32]
    lib.pce_conv_fwd.argtypes = [vp, i32, i32, vp, vp, i32, i32, vp, vp, vp, C.POINTER(TileLists), i32, vp, i32,
                                 C.POINTER(Epilogue), i32, vp]
    lib.pce_build_tile_lists.argtypes = [vp, vp, vp, vp, i32, i32, i32, i32, i32, vp, sz, vp, vp, vp, i32, vp]
    lib.pce_csr_sort_rows.argtypes = [vp, i32, i32, vp, sz, vp, vp]
    lib.pce_packed_weights_bytes.restype = sz
    lib.pce_packed_weights_bytes.argtypes = [i32, i32, i32]
    lib.pce_pack_weights.argtypes = [vp, i32, i32, i32, i32, vp, vp]
    lib.pce_device_status.argtypes = [C.POINTER(i32), i32]
    lib.pce_tune.argtypes = [i32, i32]
    lib.pce_debug_timeout.argtypes = [C.POINTER(i32)]
    lib.pce_conv_kernel_choice.argtypes = [i32, i32, i32, i32]
    lib.pce_conv_split_parts.restype = i32
    lib.pce_conv_split_parts.argtypes = [i32, i32, i32, i32, i32, i32]
    lib.pce_conv_split_scratch_bytes.restype = sz
    lib.pce_conv_split_scratch_bytes.argtypes = [i32, i32, i32, i32, i32, i32]
    lib.pce_conv_fwd_d1.argtypes = [vp, i32, i32, vp, vp, i32, i32, vp, i32, vp, vp, vp, vp, i32, vp, sz, vp, i32, i32,
                                    C.POINTER(Epilogue), vp]
    lib.pce_linear_fwd.argtypes = [vp, i32, i32, vp, vp, i32, vp, i32, C.POINTER(Epilogue), vp]
    lib.pce_scale_shift_act.argtypes = [vp, i64, i32, vp, i32, C.POINTER(Epilogue), vp]
    lib.pce_push_rows.argtypes = [vp, i64, vp, i32, i32, vp, i64, vp]
    lib.pce_quantize_workspace_bytes.restype = sz
    lib.pce_quantize_workspace_bytes.argtypes = [i32]
    lib.pce_quantize_unique.argtypes = [vp, i32, C.POINTER(C.c_float), i32, vp, sz, vp, vp, vp, C.POINTER(i32), vp]
    lib.pce_tile_rows_for.restype = i32
    lib.pce_tile_rows_for.argtypes = [i32, i32, i32, i32]
    lib.pce_plan_create.argtypes = [C.POINTER(PlanMapSpec), i32, C.POINTER(vp)]
    lib.pce_plan_destroy.restype = None
    lib.pce_plan_destroy.argtypes = [vp]
    lib.pce_plan_begin.argtypes = [vp, vp, i32, C.POINTER(i32), C.POINTER(i32), vp, C.POINTER(vp)]
    lib.pce_pass_map.argtypes = [vp, i32, vp, C.POINTER(PlannedMap)]
    lib.pce_pass_release.argtypes = [vp, vp]
    lib.pce_net_run.argtypes = [vp, C.POINTER(NetBuffer), i32, C.POINTER(NetOp), i32, vp, i32, vp, i32, vp, sz, i32, vp]
    for name in EXPORTS:
        fn = getattr(lib, name)
        if fn.restype is C.c_int and name not in ("pce_version", "pce_last_cuda_error"):
            fn.restype = C.c_int
    return lib


lib = _load()


def check(status: int, what: str = "") -> None:
    """Raise like the reference's pybind layer does: invalid arguments become
    ValueError (std::invalid_argument, backend/spconv.cu:39,234), the rest RuntimeError."""
    if status == PCE_OK:
        return
    msg = f"{what}: {lib.pce_strerror(status).decode()} (status {status}"
    if status == 2:
        msg += f", cudaError {lib.pce_last_cuda_error()}"
    msg += ")"
    if status == PCE_ERR_INVALID:
        raise ValueError(msg)
    raise RuntimeError(msg)


def require_cuda(t: torch.Tensor, name: str) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError(f"pcengine_b200: `{name}` must be a CUDA tensor; there is no CPU path")


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_ptr(device=None) -> int:
    """The current CUDA stream of ``device`` as an integer handle (called once or twice per launch:
    torch's raw-stream query, when present, costs a fraction of building a Stream object)."""
    if _raw_stream is not None:
        idx = device.index if isinstance(device, torch.device) else device
        return _raw_stream(torch.cuda.current_device() if idx is None else idx)
    return torch.cuda.current_stream(device).cuda_stream


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return PCE_F32
    if dt == torch.float16:
        return PCE_F16
    raise NotImplementedError(f"pcengine_b200 supports float32 and float16 features, got {dt}")


def workspace(nbytes: int, device) -> torch.Tensor:
    return torch.empty((max(int(nbytes), 256),), dtype=torch.uint8, device=device)
