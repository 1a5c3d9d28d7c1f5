// CUDA-core fused gather-matmul-scatter (output stationary) for narrow or odd
// channel counts, the dense rows x matrix product, and the stand-alone
// scale/shift/activation pass.  A group of G threads owns one output row; each
// thread keeps four fp32 accumulators (four consecutive output channels),
// walks the row's neighbour list once and stores the row once with the fused
// epilogue.  Weights are read through the read-only path and stay L1/L2
// resident.  Role of the reference's CUDA-core fetch-on-demand kernels
// (ref: backend/spconv.cuh:427-735,832-935,1162-1250) without their atomics.
#include "common.cuh"

namespace pce {

struct EpiDev {
  const float* scale;
  const float* shift;
  const void* residual;
  int act;
  float slope;
};

static EpiDev to_dev(const pce_epilogue* ep) {
  EpiDev e{nullptr, nullptr, nullptr, PCE_ACT_NONE, 0.f};
  if (ep) {
    e.scale = ep->scale;
    e.shift = ep->shift;
    e.residual = ep->residual;
    e.act = ep->act;
    e.slope = ep->slope;
  }
  return e;
}

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) {
  return v;
}
template <>
__device__ __forceinline__ __half from_f<__half>(float v) {
  return __float2half_rn(v);
}

__device__ __forceinline__ float apply_act(float v, int act, float slope) {
  if (act == PCE_ACT_RELU) return v > 0.f ? v : 0.f;
  if (act == PCE_ACT_LEAKY) return v > 0.f ? v : v * slope;
  return v;
}

template <typename T>
__device__ __forceinline__ void store_row4(T* out, const EpiDev& ep, size_t row, int cout, int co0,
                                           const float (&acc)[4]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    int c = co0 + j;
    if (c < cout) {
      float v = acc[j];
      if (ep.scale) v *= __ldg(ep.scale + c);
      if (ep.shift) v += __ldg(ep.shift + c);
      if (ep.residual) v += to_f(static_cast<const T*>(ep.residual)[row * cout + c]);
      out[row * cout + c] = from_f<T>(apply_act(v, ep.act, ep.slope));
    }
  }
}

// acc[0..3] += x_row[0..cin) . W[:, co0..co0+3]
template <typename T, bool VEC>
__device__ __forceinline__ void row_times_w(const T* __restrict__ xrow, const T* __restrict__ wk, int cin, int cout,
                                            int co0, float (&acc)[4]);

template <>
__device__ __forceinline__ void row_times_w<float, true>(const float* __restrict__ xrow, const float* __restrict__ wk,
                                                         int cin, int cout, int co0, float (&acc)[4]) {
  for (int ci = 0; ci < cin; ci += 4) {
    const float4 x = __ldg(reinterpret_cast<const float4*>(xrow + ci));
    const float xs[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float4 w = __ldg(reinterpret_cast<const float4*>(wk + static_cast<size_t>(ci + t) * cout + co0));
      acc[0] = fmaf(xs[t], w.x, acc[0]);
      acc[1] = fmaf(xs[t], w.y, acc[1]);
      acc[2] = fmaf(xs[t], w.z, acc[2]);
      acc[3] = fmaf(xs[t], w.w, acc[3]);
    }
  }
}

template <>
__device__ __forceinline__ void row_times_w<__half, true>(const __half* __restrict__ xrow,
                                                          const __half* __restrict__ wk, int cin, int cout, int co0,
                                                          float (&acc)[4]) {
  for (int ci = 0; ci < cin; ci += 8) {
    const uint4 xr = __ldg(reinterpret_cast<const uint4*>(xrow + ci));
    const __half2* xh = reinterpret_cast<const __half2*>(&xr);
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float2 xf = __half22float2(xh[t]);
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const float xv = u ? xf.y : xf.x;
        const uint2 wr = __ldg(reinterpret_cast<const uint2*>(wk + static_cast<size_t>(ci + 2 * t + u) * cout + co0));
        const float2 w01 = __half22float2(*reinterpret_cast<const __half2*>(&wr.x));
        const float2 w23 = __half22float2(*reinterpret_cast<const __half2*>(&wr.y));
        acc[0] = fmaf(xv, w01.x, acc[0]);
        acc[1] = fmaf(xv, w01.y, acc[1]);
        acc[2] = fmaf(xv, w23.x, acc[2]);
        acc[3] = fmaf(xv, w23.y, acc[3]);
      }
    }
  }
}

template <typename T>
__device__ __forceinline__ void row_times_w_scalar(const T* __restrict__ xrow, const T* __restrict__ wk, int cin,
                                                   int cout, int co0, float (&acc)[4]) {
  for (int ci = 0; ci < cin; ++ci) {
    const float xv = to_f(xrow[ci]);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (co0 + j < cout) acc[j] = fmaf(xv, to_f(wk[static_cast<size_t>(ci) * cout + co0 + j]), acc[j]);
    }
  }
}

template <>
__device__ __forceinline__ void row_times_w<float, false>(const float* __restrict__ xrow,
                                                          const float* __restrict__ wk, int cin, int cout, int co0,
                                                          float (&acc)[4]) {
  row_times_w_scalar<float>(xrow, wk, cin, cout, co0, acc);
}
template <>
__device__ __forceinline__ void row_times_w<__half, false>(const __half* __restrict__ xrow,
                                                           const __half* __restrict__ wk, int cin, int cout, int co0,
                                                           float (&acc)[4]) {
  row_times_w_scalar<__half>(xrow, wk, cin, cout, co0, acc);
}

// IDENT: every row has exactly the pair (row, kp 0, row) -- the dense product.
template <typename T, bool VEC, bool IDENT>
__global__ void __launch_bounds__(256)
    k_conv_simt(const T* __restrict__ in, const T* __restrict__ w, const uint32_t* __restrict__ mask,
                const int* __restrict__ rowptr, const int* __restrict__ nbr, int n_out, int cin, int cout, int kv,
                T* __restrict__ out, EpiDev ep, int g_threads) {
  const int rows_per_block = blockDim.x / g_threads;
  const int row = blockIdx.x * rows_per_block + threadIdx.x / g_threads;
  const int g = threadIdx.x % g_threads;
  if (row >= n_out) return;
  const int words = (kv + 31) / 32;
  const size_t wslab = static_cast<size_t>(cin) * cout;
  for (int co0 = g * 4; co0 < cout; co0 += g_threads * 4) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    if (IDENT) {
      row_times_w<T, VEC>(in + static_cast<size_t>(row) * cin, w, cin, cout, co0, acc);
    } else {
      int p = __ldg(rowptr + row);
      for (int wd = 0; wd < words; ++wd) {
        uint32_t m = __ldg(mask + static_cast<size_t>(row) * words + wd);
        while (m) {
          const int kp = wd * 32 + __ffs(m) - 1;
          m &= m - 1;
          const int nid = __ldg(nbr + p);
          ++p;
          row_times_w<T, VEC>(in + static_cast<size_t>(nid) * cin, w + kp * wslab, cin, cout, co0, acc);
        }
      }
    }
    store_row4<T>(out, ep, static_cast<size_t>(row), cout, co0, acc);
  }
}

template <typename T>
__global__ void k_scale_shift_act(const T* __restrict__ x, long long n, int c, T* __restrict__ y, EpiDev ep) {
  long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  long long total = n * c;
  for (; i < total; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    int ch = static_cast<int>(i % c);
    float v = to_f(x[i]);
    if (ep.scale) v *= __ldg(ep.scale + ch);
    if (ep.shift) v += __ldg(ep.shift + ch);
    if (ep.residual) v += to_f(static_cast<const T*>(ep.residual)[i]);
    y[i] = from_f<T>(apply_act(v, ep.act, ep.slope));
  }
}

template <typename T>
static int launch_simt(const void* in, const void* w, const uint32_t* mask, const int* rowptr, const int* nbr,
                       int n_out, int cin, int cout, int kv, void* out, const EpiDev& ep, bool ident,
                       cudaStream_t st) {
  if (n_out == 0) return PCE_OK;
  int need = (cout + 3) / 4;
  int g = 1;
  while (g < need && g < 32) g <<= 1;
  const int vec_in = sizeof(T) == 4 ? 4 : 8;
  const bool vec = (cin % vec_in == 0) && (cout % 4 == 0);
  const int rows_per_block = 256 / g;
  const int grid = div_up(n_out, rows_per_block);
  const T* in_t = static_cast<const T*>(in);
  const T* w_t = static_cast<const T*>(w);
  T* out_t = static_cast<T*>(out);
#define PCE_SIMT_LAUNCH(V, I) \
  k_conv_simt<T, V, I><<<grid, 256, 0, st>>>(in_t, w_t, mask, rowptr, nbr, n_out, cin, cout, kv, out_t, ep, g)
  if (vec) {
    if (ident)
      PCE_SIMT_LAUNCH(true, true);
    else
      PCE_SIMT_LAUNCH(true, false);
  } else {
    if (ident)
      PCE_SIMT_LAUNCH(false, true);
    else
      PCE_SIMT_LAUNCH(false, false);
  }
#undef PCE_SIMT_LAUNCH
  PCE_LAUNCH_CHECK();
  return PCE_OK;
}

int conv_simt(const void* in, const void* w, const uint32_t* mask, const int* rowptr, const int* nbr, int n_out,
              int cin, int cout, int kv, void* out, int dtype, const pce_epilogue* ep, bool ident,
              cudaStream_t st) {
  EpiDev e = to_dev(ep);
  if (dtype == PCE_F32)
    return launch_simt<float>(in, w, mask, rowptr, nbr, n_out, cin, cout, kv, out, e, ident, st);
  if (dtype == PCE_F16)
    return launch_simt<__half>(in, w, mask, rowptr, nbr, n_out, cin, cout, kv, out, e, ident, st);
  return PCE_ERR_UNSUPPORTED;
}

// Rows rows[i] (or i where rows == nullptr) of a row-major matrix, copied into consecutive rows of `dst` in
// 16-byte pieces.  `dst` may be another GPU's memory mapped into this process: plain stores, no loads from it.
__global__ void k_push_rows(const char* __restrict__ src, long long src_pitch, const int* __restrict__ rows, int n_rows,
                            int pieces, char* __restrict__ dst, long long dst_pitch) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= static_cast<long long>(n_rows) * pieces) return;
  const int r = static_cast<int>(i / pieces), p = static_cast<int>(i % pieces);
  const long long from = rows ? __ldg(rows + r) : r;
  const uint4 v = *reinterpret_cast<const uint4*>(src + from * src_pitch + 16ll * p);
  *reinterpret_cast<uint4*>(dst + r * dst_pitch + 16ll * p) = v;
}

}  // namespace pce

using namespace pce;

extern "C" {

int pce_push_rows(const void* src, int64_t src_pitch_bytes, const int32_t* rows, int32_t n_rows, int32_t row_bytes,
                  void* dst, int64_t dst_pitch_bytes, void* stream) {
  if (n_rows < 0 || row_bytes < 16 || (row_bytes & 15) || src_pitch_bytes < row_bytes || dst_pitch_bytes < row_bytes ||
      (src_pitch_bytes & 15) || (dst_pitch_bytes & 15))
    return PCE_ERR_INVALID;
  if (n_rows == 0) return PCE_OK;
  if (!src || !dst || ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15)) return PCE_ERR_INVALID;
  const int pieces = row_bytes / 16;
  const long long total = static_cast<long long>(n_rows) * pieces;
  k_push_rows<<<static_cast<unsigned>((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const char*>(src), src_pitch_bytes, rows, n_rows, pieces, static_cast<char*>(dst), dst_pitch_bytes);
  PCE_LAUNCH_CHECK();
  return PCE_OK;
}

int pce_scale_shift_act(const void* x, int64_t n, int32_t c, void* y, int32_t dtype, const pce_epilogue* ep,
                        void* stream) {
  if (n < 0 || c < 1) return PCE_ERR_INVALID;
  if (n == 0) return PCE_OK;
  if (!x || !y) return PCE_ERR_INVALID;
  if (ep && (ep->extra_feats || ep->push_slot[0] || ep->push_slot[1] || (ep->in_ld > 0 && ep->in_ld != c) ||
             (ep->out_ld > 0 && ep->out_ld != c)))
    return PCE_ERR_UNSUPPORTED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  EpiDev e = to_dev(ep);
  long long total = static_cast<long long>(n) * c;
  int grid = static_cast<int>(std::min<long long>((total + 255) / 256, 148ll * 16));
  if (dtype == PCE_F32)
    k_scale_shift_act<float><<<grid, 256, 0, st>>>(static_cast<const float*>(x), n, c, static_cast<float*>(y), e);
  else if (dtype == PCE_F16)
    k_scale_shift_act<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(x), n, c, static_cast<__half*>(y), e);
  else
    return PCE_ERR_UNSUPPORTED;
  PCE_LAUNCH_CHECK();
  return PCE_OK;
}

}  // extern "C"
