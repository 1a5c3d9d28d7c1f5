// C-ABI entry points that dispatch between kernel families, plus the status
// helpers.  See include/pce_b200.h for the contract of every function.
#include "common.cuh"

namespace pce {
int conv_simt(const void* in, const void* w, const uint32_t* mask, const int* rowptr, const int* nbr, int n_out,
              int cin, int cout, int kv, void* out, int dtype, const pce_epilogue* ep, bool ident, cudaStream_t st);
bool conv_umma_supported(int cin, int cout, int dtype);
size_t umma_packed_bytes(int kv, int cin, int cout);
int umma_pack_weights(const void* w, int kv, int cin, int cout, void* packed, cudaStream_t st);
int umma_status_fetch(int* host_status, bool reset);
int umma_where_fetch(int* host4);
extern int umma_force_stages;
extern int umma_force_sub;
extern int umma_force_nacc;
extern int umma_overlap_launches;
extern int umma_multi_tile;
extern int kmap_query_lanes4;
extern int umma_split_enabled;
extern int umma_kb32_enabled;
extern int plan_short_route;
int conv_split_parts(int n_rows, int n_src, int cin, int cout, int kv, int sm_count);
size_t conv_split_scratch_bytes(int n_rows, int n_src, int cin, int cout, int kv, int sm_count);
extern int kmap_sort_top_bits;
int conv_umma(const void* in, int n_in, const void* wpacked, int kv, const pce_tile_lists* tiles, int n_out, int cin,
              int cout, void* out, const pce_epilogue* ep, cudaStream_t st);
}  // namespace pce

using namespace pce;

extern "C" {

const char* pce_strerror(int status) {
  switch (status) {
    case PCE_OK: return "ok";
    case PCE_ERR_INVALID: return "invalid argument";
    case PCE_ERR_CUDA: return "CUDA runtime error";
    case PCE_ERR_WORKSPACE: return "workspace too small";
    case PCE_ERR_RANGE: return "coordinate outside the packable range";
    case PCE_ERR_TABLE_FULL: return "hash table full";
    case PCE_ERR_UNSUPPORTED: return "unsupported shape or dtype";
    case PCE_ERR_TIMEOUT: return "bounded device wait expired";
    case PCE_ERR_CAPACITY: return "output capacity too small";
    default: return "unknown status";
  }
}

int pce_version(void) { return 102; }  // 102: pce_planned_csr.table / reverse_kp / identity_kp, rowptr may be NULL

int pce_last_cuda_error(void) { return g_last_cuda_error; }

uint64_t pce_kernel_launches(void) { return __atomic_load_n(&g_kernel_launches, __ATOMIC_RELAXED); }

int pce_conv_kernel_choice(int32_t c_in, int32_t c_out, int32_t dtype, int32_t kernel_choice) {
  bool umma_ok = conv_umma_supported(c_in, c_out, dtype);
  if (kernel_choice == PCE_KERNEL_UMMA) return umma_ok ? PCE_KERNEL_UMMA : -1;
  return (umma_ok && kernel_choice != PCE_KERNEL_SIMT) ? PCE_KERNEL_UMMA : PCE_KERNEL_SIMT;
}

size_t pce_packed_weights_bytes(int32_t kv, int32_t c_in, int32_t c_out) {
  if (kv < 1 || c_in < 1 || c_out < 1) return 0;
  return umma_packed_bytes(kv, c_in, c_out);
}

int pce_pack_weights(const void* weights, int32_t kv, int32_t c_in, int32_t c_out, int32_t dtype, void* packed,
                     void* stream) {
  if (!weights || !packed || kv < 1) return PCE_ERR_INVALID;
  if (!conv_umma_supported(c_in, c_out, dtype)) return PCE_ERR_UNSUPPORTED;
  return umma_pack_weights(weights, kv, c_in, c_out, packed, static_cast<cudaStream_t>(stream));
}

int pce_tune(int32_t what, int32_t value) {
  if (what == 0) {
    umma_force_stages = value;
    return PCE_OK;
  }
  if (what == 1) {
    umma_force_sub = value;
    return PCE_OK;
  }
  if (what == 2) {
    umma_force_nacc = value;
    return PCE_OK;
  }
  if (what == 3) {
    umma_overlap_launches = value < 0 || value > 2 ? 1 : value;
    return PCE_OK;
  }
  if (what == 4) {
    umma_multi_tile = value ? 1 : 0;
    return PCE_OK;
  }
  if (what == 5) {
    kmap_query_lanes4 = value ? 1 : 0;
    return PCE_OK;
  }
  if (what == 6) {
    kmap_sort_top_bits = value > 0 ? value : 0;
    return PCE_OK;
  }
  if (what == 7) {
    umma_split_enabled = value < 0 ? 0 : value;
    return PCE_OK;
  }
  if (what == 8) {
    umma_kb32_enabled = value ? 1 : 0;
    return PCE_OK;
  }
  if (what == 9) {
    plan_short_route = value ? 1 : 0;
    return PCE_OK;
  }
  return PCE_ERR_INVALID;
}

int pce_device_status(int32_t* status_host, int32_t reset) {
  if (!status_host) return PCE_ERR_INVALID;
  int v = 0;
  PCE_TRY(umma_status_fetch(&v, reset != 0));
  *status_host = v;
  return PCE_OK;
}

int32_t pce_conv_split_parts(int32_t n_rows, int32_t n_src, int32_t c_in, int32_t c_out, int32_t kv, int32_t sm_count) {
  if (!conv_umma_supported(c_in, c_out, PCE_F16) || kv > 128) return 1;
  return conv_split_parts(n_rows, n_src, c_in, c_out, kv, sm_count);
}

size_t pce_conv_split_scratch_bytes(int32_t n_rows, int32_t n_src, int32_t c_in, int32_t c_out, int32_t kv,
                                    int32_t sm_count) {
  if (!conv_umma_supported(c_in, c_out, PCE_F16) || kv > 128) return 0;
  return conv_split_scratch_bytes(n_rows, n_src, c_in, c_out, kv, sm_count);
}

int pce_debug_timeout(int32_t* where4) {
  if (!where4) return PCE_ERR_INVALID;
  return umma_where_fetch(where4);
}

int pce_conv_fwd(const void* in_feats, int32_t n_in, int32_t c_in, const void* weights, const void* packed_weights,
                 int32_t kv, int32_t c_out, const uint32_t* mask, const int32_t* rowptr, const int32_t* nbr,
                 const pce_tile_lists* tiles, int32_t n_out, void* out_feats, int32_t dtype, const pce_epilogue* ep,
                 int32_t kernel_choice, void* stream) {
  if (n_in < 0 || n_out < 0 || c_in < 1 || c_out < 1 || kv < 1) return PCE_ERR_INVALID;
  if (dtype != PCE_F32 && dtype != PCE_F16) return PCE_ERR_UNSUPPORTED;
  if (n_out == 0) return PCE_OK;
  if (!out_feats || (n_in > 0 && !in_feats)) return PCE_ERR_INVALID;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool umma_ok = conv_umma_supported(c_in, c_out, dtype) && kv <= 128;
  if (kernel_choice == PCE_KERNEL_UMMA && !umma_ok) return PCE_ERR_UNSUPPORTED;
  const bool have_tc = packed_weights && tiles && tiles->order && tiles->tile_ptr && tiles->stage_kp && tiles->stage_nbr;
  if (kernel_choice == PCE_KERNEL_UMMA && !have_tc) return PCE_ERR_INVALID;
  if (umma_ok && have_tc && kernel_choice != PCE_KERNEL_SIMT) {
    if ((reinterpret_cast<uintptr_t>(in_feats) | reinterpret_cast<uintptr_t>(out_feats) |
         reinterpret_cast<uintptr_t>(packed_weights)) & 15)
      return PCE_ERR_INVALID;
    return conv_umma(in_feats, n_in, packed_weights, kv, tiles, n_out, c_in, c_out, out_feats, ep, st);
  }
  if (ep && (ep->extra_feats || ep->push_slot[0] || ep->push_slot[1] || (ep->in_ld > 0 && ep->in_ld != c_in) ||
             (ep->out_ld > 0 && ep->out_ld != c_out)))
    return PCE_ERR_UNSUPPORTED;  // the second operand, the halo push and row pitches need the tensor-core kernel
  if (!weights || !mask || !rowptr || (n_in > 0 && !nbr)) return PCE_ERR_INVALID;
  return conv_simt(in_feats, weights, mask, rowptr, nbr, n_out, c_in, c_out, kv, out_feats, dtype, ep, false, st);
}

int pce_linear_fwd(const void* in_feats, int32_t n, int32_t c_in, const void* weights, const void* packed_weights,
                   int32_t c_out, void* out_feats, int32_t dtype, const pce_epilogue* ep, void* stream) {
  if (n < 0 || c_in < 1 || c_out < 1) return PCE_ERR_INVALID;
  if (n == 0) return PCE_OK;
  if (!in_feats || !out_feats || (!weights && !packed_weights)) return PCE_ERR_INVALID;
  if (ep && (ep->extra_feats || ep->push_slot[0] || ep->push_slot[1])) return PCE_ERR_UNSUPPORTED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool aligned = ((reinterpret_cast<uintptr_t>(in_feats) | reinterpret_cast<uintptr_t>(out_feats) |
                         reinterpret_cast<uintptr_t>(packed_weights)) & 15) == 0;
  if (packed_weights && aligned && conv_umma_supported(c_in, c_out, dtype))
    return conv_umma(in_feats, n, packed_weights, 1, nullptr, n, c_in, c_out, out_feats, ep, st);
  if (!weights) return PCE_ERR_INVALID;
  if (ep && ((ep->in_ld > 0 && ep->in_ld != c_in) || (ep->out_ld > 0 && ep->out_ld != c_out))) return PCE_ERR_UNSUPPORTED;
  return conv_simt(in_feats, weights, nullptr, nullptr, nullptr, n, c_in, c_out, 1, out_feats, dtype, ep, true, st);
}

}  // extern "C"
