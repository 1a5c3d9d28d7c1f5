// Shared helpers of libpce_b200: status plumbing, a bump allocator over the
// caller's workspace, and the 64-bit packed coordinate key.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/pce_b200.h"

namespace pce {

extern thread_local int g_last_cuda_error;
extern unsigned long long g_kernel_launches;  // kernels of this library launched so far (all threads)

inline int cuda_fail(cudaError_t e) {
  g_last_cuda_error = static_cast<int>(e);
  return PCE_ERR_CUDA;
}

#define PCE_CUDA(expr)                                  \
  do {                                                  \
    cudaError_t e__ = (expr);                           \
    if (e__ != cudaSuccess) return ::pce::cuda_fail(e__); \
  } while (0)

#define PCE_LAUNCH_CHECK()                                  \
  do {                                                      \
    __atomic_fetch_add(&::pce::g_kernel_launches, 1ull, __ATOMIC_RELAXED); \
    PCE_CUDA(cudaPeekAtLastError());                        \
  } while (0)

#define PCE_TRY(expr)              \
  do {                             \
    int s__ = (expr);              \
    if (s__ != PCE_OK) return s__; \
  } while (0)

inline int div_up(long long a, long long b) { return static_cast<int>((a + b - 1) / b); }

// Carves 256-byte aligned pieces out of the caller's workspace.
struct Arena {
  char* base;
  size_t cap;
  size_t off = 0;
  bool ok = true;
  Arena(void* p, size_t n) : base(static_cast<char*>(p)), cap(n) {}
  template <typename T>
  T* take(size_t count) {
    size_t bytes = (count * sizeof(T) + 255) & ~size_t(255);
    if (base == nullptr || off + bytes > cap) {
      ok = false;
      return nullptr;
    }
    T* p = reinterpret_cast<T*>(base + off);
    off += bytes;
    return p;
  }
  size_t left() const { return cap - off; }
};

inline size_t pad256(size_t b) { return (b + 255) & ~size_t(255); }

// ---- packed coordinate key -------------------------------------------------
// key = b<<48 | (x+2^15)<<32 | (y+2^15)<<16 | (z+2^15); ascending key order is
// ascending (b,x,y,z) order.  All-ones is reserved for "empty slot".
constexpr unsigned long long kEmptyKey = ~0ull;

__host__ __device__ inline bool packable(int b, int x, int y, int z) {
  return (static_cast<unsigned>(b) < 65535u) && (static_cast<unsigned>(x + 32768) < 65536u) &&
         (static_cast<unsigned>(y + 32768) < 65536u) && (static_cast<unsigned>(z + 32768) < 65536u);
}

__host__ __device__ inline unsigned long long pack_key(int b, int x, int y, int z) {
  return (static_cast<unsigned long long>(static_cast<unsigned>(b)) << 48) |
         (static_cast<unsigned long long>(static_cast<unsigned>(x + 32768)) << 32) |
         (static_cast<unsigned long long>(static_cast<unsigned>(y + 32768)) << 16) |
         static_cast<unsigned long long>(static_cast<unsigned>(z + 32768));
}

__host__ __device__ inline void unpack_key(unsigned long long k, int& b, int& x, int& y, int& z) {
  b = static_cast<int>(k >> 48);
  x = static_cast<int>((k >> 32) & 0xFFFF) - 32768;
  y = static_cast<int>((k >> 16) & 0xFFFF) - 32768;
  z = static_cast<int>(k & 0xFFFF) - 32768;
}

// 64-bit finaliser used as the slot hash.
__host__ __device__ inline unsigned long long mix64(unsigned long long k) {
  k ^= k >> 33;
  k *= 0xff51afd7ed558ccdull;
  k ^= k >> 33;
  k *= 0xc4ceb9fe1a85ec53ull;
  k ^= k >> 33;
  return k;
}

}  // namespace pce
