// Explicit gather -> GEMM -> scatter dataflow over a caller-provided buffer
// (role of ConvolutionForwardD1, ref: backend/spconv.cu:24-222).  Buffer rows
// are addressed as qkpos[kp] + pos with (kp, pos) decoded from the CSR-coded
// maps (kp*1186111 + pos, ref: backend/hash.cuh:7-9); row/element offsets are
// 64-bit.  The scatter pass (one warp per output row, 16-byte pieces, fp32
// sums) adds each row's products in kp order and the centre offset product of a
// submanifold layer (a dense product on the tensor-core kernel beforehand where
// the widths allow), applies the fused epilogue and stores the row once.
#include "common.cuh"

namespace pce {

bool conv_umma_supported(int cin, int cout, int dtype);
int conv_umma(const void* in, int n_in, const void* wpacked, int kv, const pce_tile_lists* tiles, int n_out, int cin,
              int cout, void* out, const pce_epilogue* ep, cudaStream_t st);
int conv_umma_kb64(const void* in, int n_in, const void* wpacked, int kv, const pce_tile_lists* tiles, int n_out, int cin,
                   int cout, void* out, const pce_epilogue* ep, cudaStream_t st);

struct EpiDev {
  const float* scale;
  const float* shift;
  const void* residual;
  int act;
  float slope;
};
__device__ __forceinline__ float d1_to_f(float v) { return v; }
__device__ __forceinline__ float d1_to_f(__half v) { return __half2float(v); }
template <typename T>
__device__ __forceinline__ T d1_from_f(float v);
template <>
__device__ __forceinline__ float d1_from_f<float>(float v) {
  return v;
}
template <>
__device__ __forceinline__ __half d1_from_f<__half>(float v) {
  return __float2half_rn(v);
}

constexpr int kCode = 1186111;

// One warp per input row: copy the row to every buffer slot its CSR entries name
// (ref: backend/spconv.cuh:48-81 gather_all_input_major_csr_*); 16-byte pieces when the row
// length allows.
template <typename T>
__global__ void k_d1_gather(const T* __restrict__ in, int n_in, int cin, const int* __restrict__ qkpos,
                            const int* __restrict__ icsr, const int* __restrict__ imap, T* __restrict__ buf) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= n_in) return;
  const int a = __ldg(icsr + warp), b = __ldg(icsr + warp + 1);
  const T* src = in + static_cast<size_t>(warp) * cin;
  const int row_bytes = cin * static_cast<int>(sizeof(T));
  const bool vec = (row_bytes % 16 == 0) && ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(buf)) % 16 == 0);
  for (int e = a; e < b; ++e) {
    const int code = __ldg(imap + e);
    const size_t pos = static_cast<size_t>(__ldg(qkpos + code / kCode)) + code % kCode;
    T* dst = buf + pos * cin;
    if (vec) {
      const uint4* s4 = reinterpret_cast<const uint4*>(src);
      uint4* d4 = reinterpret_cast<uint4*>(dst);
      for (int c = lane; c < row_bytes / 16; c += 32) d4[c] = __ldg(s4 + c);
    } else {
      for (int c = lane; c < cin; c += 32) dst[c] = src[c];
    }
  }
}

// Tile lists for the per-offset GEMM over the gather buffer: rows are already dense and every
// 128-row tile lies inside one offset's padded segment (segments are padded to 128,
// ref: backend/hash.cuh:478-497), so tile t is one stage with offset = segment(t*128) and the
// rows fetch themselves.
__global__ void k_d1_tile_lists(const int* __restrict__ qkpos, int kv, int n_tiles, int* order, int* tile_ptr,
                                int* stage_kp, int* stage_nbr) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n_tiles * 128) {
    order[i] = i;
    stage_nbr[i] = i;
  }
  if (i <= n_tiles) tile_ptr[i] = i;
  if (i < n_tiles) {
    const int row = i * 128;
    int lo = 0, hi = kv;  // largest kp with qkpos[kp] <= row
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (__ldg(qkpos + mid) <= row)
        lo = mid;
      else
        hi = mid;
    }
    stage_kp[i] = lo;
  }
}

// buf_out[row] = buf_in[row] @ W[segment(row)] for every padded row; four
// output channels per thread, G threads per row.
template <typename T>
__global__ void __launch_bounds__(256)
    k_d1_gemm(const T* __restrict__ bin, const T* __restrict__ w, const int* __restrict__ qkpos, int kv, int qsum,
              int cin, int cout, T* __restrict__ bout, int g_threads) {
  const int rows_per_block = blockDim.x / g_threads;
  const int row = blockIdx.x * rows_per_block + threadIdx.x / g_threads;
  const int g = threadIdx.x % g_threads;
  if (row >= qsum) return;
  int lo = 0, hi = kv;  // largest kp with qkpos[kp] <= row
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (__ldg(qkpos + mid) <= row)
      lo = mid;
    else
      hi = mid;
  }
  const T* wk = w + static_cast<size_t>(lo) * cin * cout;
  const T* x = bin + static_cast<size_t>(row) * cin;
  for (int co0 = g * 4; co0 < cout; co0 += g_threads * 4) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int ci = 0; ci < cin; ++ci) {
      const float xv = d1_to_f(x[ci]);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (co0 + j < cout) acc[j] = fmaf(xv, d1_to_f(wk[static_cast<size_t>(ci) * cout + co0 + j]), acc[j]);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (co0 + j < cout) bout[static_cast<size_t>(row) * cout + co0 + j] = d1_from_f<T>(acc[j]);
  }
}

// One warp per output row, lanes over 16-byte pieces of the row: fp32 sums over the row's buffer rows
// (kp ascending, as the CSR lists them), plus the centre product -- read from `centre` when the
// tensor-core kernel computed it as a dense product beforehand, else formed here from W[centre] --
// then the epilogue and one 16-byte store per piece
// (ref: backend/spconv.cuh:337-422 scatter_all_output_major_csr_*).
template <typename T>
__global__ void __launch_bounds__(256)
    k_d1_scatter(const T* __restrict__ bout, const int* __restrict__ qkpos, const int* __restrict__ ocsr,
                 const int* __restrict__ omap, int n_out, int cout, const T* __restrict__ in, const T* __restrict__ wmid,
                 const T* centre, int cin, T* out, EpiDev ep) {
  constexpr int kVec = 16 / static_cast<int>(sizeof(T));  // elements per 16-byte piece
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= n_out) return;
  const int a = __ldg(ocsr + row), b = __ldg(ocsr + row + 1);
  const bool vec = (cout % kVec == 0) &&
                   ((reinterpret_cast<uintptr_t>(bout) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(centre) |
                     reinterpret_cast<uintptr_t>(ep.residual)) % 16 == 0);
  const int pieces = vec ? cout / kVec : (cout + kVec - 1) / kVec;
  for (int p0 = 0; p0 < pieces; p0 += 32) {
    const int p = p0 + lane;
    const int c0 = p * kVec;
    float acc[kVec];
#pragma unroll
    for (int q = 0; q < kVec; ++q) acc[q] = 0.f;
    if (p < pieces) {
      for (int e = a; e < b; ++e) {
        const int code = __ldg(omap + e);
        const size_t pos = static_cast<size_t>(__ldg(qkpos + code / kCode)) + code % kCode;
        const T* src = bout + pos * cout + c0;
        if (vec) {
          const uint4 v = *reinterpret_cast<const uint4*>(src);
          const T* t = reinterpret_cast<const T*>(&v);
#pragma unroll
          for (int q = 0; q < kVec; ++q) acc[q] += d1_to_f(t[q]);
        } else {
          for (int q = 0; q < kVec && c0 + q < cout; ++q) acc[q] += d1_to_f(src[q]);
        }
      }
      if (centre != nullptr) {
        const T* src = centre + static_cast<size_t>(row) * cout + c0;
        if (vec) {
          const uint4 v = *reinterpret_cast<const uint4*>(src);
          const T* t = reinterpret_cast<const T*>(&v);
#pragma unroll
          for (int q = 0; q < kVec; ++q) acc[q] += d1_to_f(t[q]);
        } else {
          for (int q = 0; q < kVec && c0 + q < cout; ++q) acc[q] += d1_to_f(src[q]);
        }
      } else if (wmid != nullptr) {
        const T* x = in + static_cast<size_t>(row) * cin;
        for (int ci = 0; ci < cin; ++ci) {
          const float xv = d1_to_f(x[ci]);
          const T* wr = wmid + static_cast<size_t>(ci) * cout + c0;
#pragma unroll
          for (int q = 0; q < kVec; ++q)
            if (c0 + q < cout) acc[q] = fmaf(xv, d1_to_f(wr[q]), acc[q]);
        }
      }
      alignas(16) T res[kVec];
#pragma unroll
      for (int q = 0; q < kVec; ++q) {
        const int c = c0 + q;
        float v = acc[q];
        if (c < cout) {
          if (ep.scale) v *= __ldg(ep.scale + c);
          if (ep.shift) v += __ldg(ep.shift + c);
          if (ep.residual) v += d1_to_f(static_cast<const T*>(ep.residual)[static_cast<size_t>(row) * cout + c]);
          if (ep.act == PCE_ACT_RELU) v = v > 0.f ? v : 0.f;
          if (ep.act == PCE_ACT_LEAKY) v = v > 0.f ? v : v * ep.slope;
        }
        res[q] = d1_from_f<T>(v);
      }
      T* dst = out + static_cast<size_t>(row) * cout + c0;
      if (vec) {
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(res);
      } else {
        for (int q = 0; q < kVec && c0 + q < cout; ++q) dst[q] = res[q];
      }
    }
  }
}

template <typename T>
static int run_d1(const void* in, int n_in, int cin, const void* w, const void* wpacked, int kv, int cout,
                  const int* qkpos, int qsum, const int* imap, const int* icsr, const int* omap, const int* ocsr,
                  int n_out, void* buffer, size_t buffer_bytes, void* out, int centre_kp, const EpiDev& ep, int dtype,
                  cudaStream_t st) {
  T* bin = static_cast<T*>(buffer);
  T* bout = bin + static_cast<size_t>(qsum) * cin;
  const T* in_t = static_cast<const T*>(in);
  const T* w_t = static_cast<const T*>(w);
  if (n_in > 0 && qsum > 0) {
    k_d1_gather<T><<<div_up(static_cast<long long>(n_in) * 32, 256), 256, 0, st>>>(in_t, n_in, cin, qkpos, icsr, imap,
                                                                                    bin);
    PCE_LAUNCH_CHECK();
    // The per-offset GEMM: tensor cores when packed weights are given and the scratch for the
    // tile lists fits behind the two halves of the buffer, else CUDA cores.
    const int n_tiles = qsum / 128;
    const size_t used = static_cast<size_t>(qsum) * (cin + cout) * sizeof(T);
    const size_t lists_at = (used + 255) & ~size_t(255);
    const size_t lists_bytes = sizeof(int) * (static_cast<size_t>(n_tiles) * 258 + 2);
    const bool tc = wpacked != nullptr && conv_umma_supported(cin, cout, dtype) && qsum % 128 == 0 &&
                    lists_at + lists_bytes <= buffer_bytes &&
                    ((reinterpret_cast<uintptr_t>(buffer) | reinterpret_cast<uintptr_t>(wpacked)) % 16 == 0) &&
                    (static_cast<size_t>(qsum) * cin * sizeof(T)) % 16 == 0;
    if (tc) {
      int* base = reinterpret_cast<int*>(static_cast<char*>(buffer) + lists_at);
      int* order = base;
      int* stage_nbr = order + static_cast<size_t>(n_tiles) * 128;
      int* tile_ptr = stage_nbr + static_cast<size_t>(n_tiles) * 128;
      int* stage_kp = tile_ptr + n_tiles + 1;
      k_d1_tile_lists<<<div_up(static_cast<long long>(n_tiles) * 128 + 1, 256), 256, 0, st>>>(qkpos, kv, n_tiles, order,
                                                                                               tile_ptr, stage_kp, stage_nbr);
      PCE_LAUNCH_CHECK();
      pce_tile_lists tl{order, tile_ptr, stage_kp, stage_nbr, 128, 0, 1, 0};
      PCE_TRY(conv_umma(bin, qsum, wpacked, kv, &tl, qsum, cin, cout, bout, nullptr, st));
    } else {
      if (w == nullptr) return PCE_ERR_INVALID;
      int need = (cout + 3) / 4, g = 1;
      while (g < need && g < 32) g <<= 1;
      k_d1_gemm<T><<<div_up(qsum, 256 / g), 256, 0, st>>>(bin, w_t, qkpos, kv, qsum, cin, cout, bout, g);
      PCE_LAUNCH_CHECK();
    }
  }
  if (n_out > 0) {
    const T* wmid = nullptr;
    const T* centre = nullptr;
    if (centre_kp >= 0) {
      // the centre offset is a dense rows x matrix product: on the tensor-core kernel when the packed
      // weights allow it (written into `out`, which the scatter then reads row by row and overwrites),
      // else formed inside the scatter from W[centre]
      const int kblocks = (cin + 63) / 64;
      const bool tc_centre = wpacked != nullptr && conv_umma_supported(cin, cout, dtype) &&
                             ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out) |
                               reinterpret_cast<uintptr_t>(wpacked)) % 16 == 0);
      if (tc_centre) {
        const __half* wp = static_cast<const __half*>(wpacked) + static_cast<size_t>(centre_kp) * kblocks * cout * 64;
        PCE_TRY(conv_umma_kb64(in, n_in, wp, 1, nullptr, n_out, cin, cout, out, nullptr, st));
        centre = static_cast<const T*>(out);
      } else {
        if (w == nullptr) return PCE_ERR_INVALID;
        wmid = w_t + static_cast<size_t>(centre_kp) * cin * cout;
      }
    }
    k_d1_scatter<T><<<div_up(static_cast<long long>(n_out) * 32, 256), 256, 0, st>>>(
        qsum > 0 ? bout : nullptr, qkpos, ocsr, omap, n_out, cout, in_t, wmid, centre, cin, static_cast<T*>(out), ep);
    PCE_LAUNCH_CHECK();
  }
  return PCE_OK;
}

}  // namespace pce

using namespace pce;

extern "C" int pce_conv_fwd_d1(const void* in_feats, int32_t n_in, int32_t c_in, const void* weights,
                               const void* packed_weights, int32_t kv, int32_t c_out, const int32_t* qkpos, int32_t qsum,
                               const int32_t* imap_coded, const int32_t* icsr, const int32_t* omap_coded,
                               const int32_t* ocsr, int32_t n_out, void* buffer, size_t buffer_bytes, void* out_feats,
                               int32_t dtype, int32_t centre_kp, const pce_epilogue* ep, void* stream) {
  if (n_in < 0 || n_out < 0 || c_in < 1 || c_out < 1 || kv < 1 || qsum < 0) return PCE_ERR_INVALID;
  if (dtype != PCE_F32 && dtype != PCE_F16) return PCE_ERR_UNSUPPORTED;
  if (n_out == 0) return PCE_OK;
  if ((!weights && !packed_weights) || !out_feats || !qkpos || !ocsr || !icsr) return PCE_ERR_INVALID;
  if (qsum > 0 && (!imap_coded || !omap_coded || !buffer || !in_feats)) return PCE_ERR_INVALID;
  if (centre_kp >= kv || (centre_kp >= 0 && n_in != n_out)) return PCE_ERR_INVALID;
  if (ep && (ep->extra_feats || ep->push_slot[0] || ep->push_slot[1] || (ep->in_ld > 0 && ep->in_ld != c_in) ||
             (ep->out_ld > 0 && ep->out_ld != c_out)))
    return PCE_ERR_UNSUPPORTED;
  const size_t esize = dtype == PCE_F32 ? 4 : 2;
  if (static_cast<size_t>(qsum) * (c_in + c_out) * esize > buffer_bytes) return PCE_ERR_WORKSPACE;
  EpiDev e{nullptr, nullptr, nullptr, PCE_ACT_NONE, 0.f};
  if (ep) e = EpiDev{ep->scale, ep->shift, ep->residual, ep->act, ep->slope};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == PCE_F32)
    return run_d1<float>(in_feats, n_in, c_in, weights, nullptr, kv, c_out, qkpos, qsum, imap_coded, icsr, omap_coded,
                         ocsr, n_out, buffer, buffer_bytes, out_feats, centre_kp, e, dtype, st);
  return run_d1<__half>(in_feats, n_in, c_in, weights, packed_weights, kv, c_out, qkpos, qsum, imap_coded, icsr,
                        omap_coded, ocsr, n_out, buffer, buffer_bytes, out_feats, centre_kp, e, dtype, st);
}
