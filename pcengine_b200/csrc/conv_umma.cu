// Fused gather-matmul-scatter on the 5th-generation tensor cores (tcgen05 + tensor
// memory), fp16 in / fp32 accumulate, output stationary.
//
// One CTA owns 128 consecutive output rows: the accumulator is a 128-lane x C_out-column
// fp32 tile in tensor memory.  For every kernel offset present in the tile (OR of the
// rows' indicator bitmasks; absent offsets are skipped) and every 64-channel K block:
//   * producer warps 0-3 (one thread per output row) gather the neighbour rows with
//     16-byte cp.async into a 128-byte-swizzled K-major shared-memory tile, zero-filling
//     rows that lack the offset (four rows per warp instruction, fully coalesced);
//   * producer thread 0 also pulls the matching pre-packed weight block with one bulk
//     async copy (cp.async.bulk, completion counted on an mbarrier);
//   * warp 4 (one elected thread) issues tcgen05.mma (M=128, N=C_out, K=16) over the
//     block and commits to the stage's "empty" mbarrier, which hands the stage back.
// After the last block the accumulator is committed, warps 0-3 read it back with
// tcgen05.ld, apply scale/shift/residual/activation, convert to fp16 and store each
// output row exactly once.  No atomics, no intermediate buffer in HBM.
//
// Every mbarrier wait is bounded: when a wait runs out the CTA raises an abort flag,
// records PCE_ERR_TIMEOUT in the library's device status word, drains its own copies,
// frees its tensor memory and returns.
//
// Replaces fetch_on_demand_gemm_fp16_tc4_async and the cuBLAS centre GEMM of the
// reference (ref: backend/spconv.cuh:1567-1730, backend/spconv.cu:273-298,338).
#include "common.cuh"

namespace pce {

__device__ int g_umma_status = 0;

namespace umma {

constexpr int kTileM = 128;
constexpr int kMaxStages = 6;
constexpr int kABytes = kTileM * 128;  // one A stage: 128 rows x 64 fp16
constexpr int kMaxWords = 4;       // kernel volume <= 128
constexpr long long kWaitCycles = 2000000000ll;  // ~1 s at 2 GHz

struct Epi {
  const float* scale;
  const float* shift;
  const __half* residual;
  int act;
  float slope;
};

struct SharedCtl {
  unsigned long long afull[kMaxStages];
  unsigned long long bfull[kMaxStages];
  unsigned long long empty[kMaxStages];
  unsigned long long tfull[2];
  unsigned long long tempty[2];
  unsigned long long accfull[2];
  unsigned long long accempty[2];
  uint32_t tmem_base;
  uint32_t warp_mask[2][4][kMaxWords];  // per tile-ring slot, per producer warp: OR of its rows' bitmasks
  int tile_stages[2];
  int acc_stages[2];
  volatile int abort_flag;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(bar),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait: false when the abort flag is up or the deadline passed.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, SharedCtl* ctl) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  int spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if (((++spins) & 255) == 0) {
      if (ctl->abort_flag) return false;
      if (clock64() - t0 > kWaitCycles) {
        ctl->abort_flag = 1;
        atomicMax(&g_umma_status, PCE_ERR_TIMEOUT);
        return false;
      }
    }
  }
  return true;
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc]; fp16 operands, fp32 accumulate.
__device__ __forceinline__ void tc_mma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// K-major, 128-byte swizzle: rows of 128 B, 8-row groups 1024 B apart, descriptor version 1.
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) {
  const uint32_t lo = ((smem_addr >> 4) & 0x3FFFu) | (1u << 16);
  const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
  return (static_cast<uint64_t>(hi) << 32) | lo;
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, "
      "[%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float act_apply(float v, int act, float slope) {
  if (act == PCE_ACT_RELU) return v > 0.f ? v : 0.f;
  if (act == PCE_ACT_LEAKY) return v > 0.f ? v : v * slope;
  return v;
}

// Weights [kv][cin][cout] fp16 -> per (kp, k-block) shared-memory images of cout rows x 128 B
// (64 K elements, zero padded), 16-byte chunks XOR-swizzled with the row index.
__global__ void k_pack_weights(const __half* __restrict__ w, int kv, int cin, int cout, int kblocks,
                               __half* __restrict__ packed) {
  const long long total = static_cast<long long>(kv) * kblocks * cout * 64;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int kk = static_cast<int>(i % 64);
    long long t = i / 64;
    const int co = static_cast<int>(t % cout);
    t /= cout;
    const int kb = static_cast<int>(t % kblocks);
    const int kp = static_cast<int>(t / kblocks);
    const int ci = kb * 64 + kk;
    __half v = __float2half(0.f);
    if (ci < cin) v = w[(static_cast<size_t>(kp) * cin + ci) * cout + co];
    const int chunk = kk >> 3, within = kk & 7;
    const size_t img = (static_cast<size_t>(kp) * kblocks + kb) * cout * 64;
    packed[img + static_cast<size_t>(co) * 64 + ((chunk ^ (co & 7)) << 3) + within] = v;
  }
}

// Persistent, warp-specialised kernel.  288 threads:
//   warps 0-3  producers: one thread per output row of the current tile (gather + weight copy)
//   warp  4    MMA issuer (one elected lane)
//   warps 5-8  epilogue: tensor memory -> registers -> scale/shift/residual/activation -> fp16 rows
// Each CTA walks tiles blockIdx.x, blockIdx.x + gridDim.x, ...  Three rings decouple the roles:
//   stage ring  (NS slots: afull/bfull/empty)  producers -> MMA, runs on across tile boundaries;
//   tile ring   (2 slots: tfull/tempty)        producers -> MMA: number of stages of a tile;
//   acc ring    (2 TMEM accumulators: accfull/accempty)  MMA -> epilogue.
// So the gather of tile i+1, the MMAs of tile i and the stores of tile i-1 overlap.
template <int NS>
__global__ void __launch_bounds__(288, 1)
    k_conv_umma(const __half* __restrict__ in, const __half* __restrict__ wpacked, const uint32_t* __restrict__ mask,
                const int* __restrict__ rowptr, const int* __restrict__ nbr, const int* __restrict__ order, int n_out,
                int cin, int cout, int kv, __half* __restrict__ out, Epi ep, int tmem_cols) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = ((raw_addr + 1023u) & ~1023u) - raw_addr;
  uint8_t* tiles = smem_raw + pad;  // 1024-byte aligned
  const uint32_t tiles_addr = raw_addr + pad;
  const int b_bytes = cout * 128;
  const int stage_bytes = kABytes + b_bytes;  // both multiples of 1024
  SharedCtl* ctl = reinterpret_cast<SharedCtl*>(tiles + NS * stage_bytes);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int words = (kv + 31) >> 5;
  const int kblocks = (cin + 63) >> 6;
  const int n_tiles = (n_out + kTileM - 1) / kTileM;

  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(smem_u32(&ctl->afull[s]), 128);
      mbar_init(smem_u32(&ctl->bfull[s]), 1);
      mbar_init(smem_u32(&ctl->empty[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&ctl->tfull[s]), 1);
      mbar_init(smem_u32(&ctl->tempty[s]), 1);
      mbar_init(smem_u32(&ctl->accfull[s]), 2);  // the MMA thread's own arrive + the tcgen05.commit
      mbar_init(smem_u32(&ctl->accempty[s]), 128);
      ctl->tile_stages[s] = 0;
      ctl->acc_stages[s] = 0;
    }
    ctl->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 4) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)),
                 "r"(static_cast<uint32_t>(tmem_cols))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;

  if (warp < 4) {
    // =========================== producers ===========================
    int j = 0;               // stages issued so far by this CTA (continuous over tiles)
    int pending_arrive = 0;  // next stage this thread still has to arrive on
    const int rsub = lane >> 3;  // row inside a 4-row group
    const int chunk = lane & 7;  // 16-byte chunk inside a 128-byte row
    // row bookkeeping of the NEXT tile is fetched while the current one is gathered
    int nxt_row = n_out;
    uint32_t nxt_mask[kMaxWords] = {0, 0, 0, 0};
    int nxt_cursor = 0;
    auto fetch_row = [&](int tile) {
      nxt_row = n_out;
      for (int w = 0; w < kMaxWords; ++w) nxt_mask[w] = 0;
      nxt_cursor = 0;
      const int slot = tile * kTileM + tid;
      if (tile < n_tiles && slot < n_out) {
        nxt_row = order ? __ldg(order + slot) : slot;
        if (mask != nullptr) {
          for (int w = 0; w < words; ++w) nxt_mask[w] = __ldg(mask + static_cast<size_t>(nxt_row) * words + w);
          nxt_cursor = __ldg(rowptr + nxt_row);
        } else {
          nxt_mask[0] = 1u;  // dense product: the row itself at offset 0
        }
      }
    };
    fetch_row(blockIdx.x);
    int it = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++it) {
      const int slot2 = it & 1;
      const int my_row = nxt_row;
      uint32_t my_mask[kMaxWords];
      for (int w = 0; w < kMaxWords; ++w) my_mask[w] = nxt_mask[w];
      int cursor = nxt_cursor;
      int next_nid = -1;
      if (my_row < n_out && (my_mask[0] | my_mask[1] | my_mask[2] | my_mask[3]))
        next_nid = mask != nullptr ? __ldg(nbr + cursor) : my_row;
      // Each producer warp publishes the OR of its rows' bitmasks in its own cell of the slot;
      // after the barrier everyone ORs the four cells.  A slot's cells are rewritten two tiles
      // later, after a barrier that all readers of this tile have passed: no clearing needed.
      for (int w = 0; w < words; ++w) {
        const uint32_t m = __reduce_or_sync(0xFFFFFFFFu, my_mask[w]);
        if (lane == 0) ctl->warp_mask[slot2][warp][w] = m;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (ctl->abort_flag) break;  // uniform: every producer reads it after the barrier
      uint32_t tile_mask[kMaxWords];
      int n_off = 0;
      for (int w = 0; w < kMaxWords; ++w) {
        tile_mask[w] = 0u;
        if (w < words)
          tile_mask[w] = ctl->warp_mask[slot2][0][w] | ctl->warp_mask[slot2][1][w] | ctl->warp_mask[slot2][2][w] |
                         ctl->warp_mask[slot2][3][w];
        n_off += __popc(tile_mask[w]);
      }
      bool ok = true;
      if (tid == 0) {
        // the tile-ring slot must have been consumed by the MMA warp (two tiles ago)
        if (it >= 2) ok = mbar_wait(smem_u32(&ctl->tempty[slot2]), ((it >> 1) - 1) & 1, ctl);
        if (ok) {
          ctl->tile_stages[slot2] = n_off * kblocks;
          mbar_arrive(smem_u32(&ctl->tfull[slot2]));
        }
      }
      fetch_row(tile + gridDim.x);  // loads for the next tile fly during this tile's gather
      ok = __all_sync(0xFFFFFFFFu, ok);
      for (int w = 0; w < words && ok; ++w) {
        uint32_t tm = tile_mask[w];
        while (tm && ok) {
          const int bit = __ffs(tm) - 1;
          tm &= tm - 1;
          const int kp = w * 32 + bit;
          int nid = -1;
          if ((my_mask[w] >> bit) & 1u) {
            nid = next_nid;
            ++cursor;
            uint32_t rest = my_mask[w] & ~((2u << bit) - 1u);
            bool more = rest != 0;
            for (int w2 = w + 1; w2 < words; ++w2) more |= my_mask[w2] != 0;
            next_nid = (more && mask != nullptr) ? __ldg(nbr + cursor) : -1;
          }
          for (int kb = 0; kb < kblocks && ok; ++kb, ++j) {
            const int s = j % NS;
            const int n = j / NS;
            if (n > 0) ok = mbar_wait(smem_u32(&ctl->empty[s]), (n - 1) & 1, ctl);
            ok = __all_sync(0xFFFFFFFFu, ok);  // keep the warp convergent for the shuffles below
            if (!ok) break;
            const uint32_t a_addr = tiles_addr + s * stage_bytes;
            if (tid == 0) {
              const uint32_t bbar = smem_u32(&ctl->bfull[s]);
              mbar_arrive_expect_tx(bbar, b_bytes);
              bulk_copy_g2s(a_addr + kABytes, wpacked + (static_cast<size_t>(kp) * kblocks + kb) * cout * 64, b_bytes,
                            bbar);
            }
            const int kchunks = min(8, (cin - kb * 64) >> 3);
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const int r = q * 4 + rsub;  // row inside this warp's 32
              const int src_row = __shfl_sync(0xFFFFFFFFu, nid, r);
              if (chunk < kchunks) {
                const uint32_t dst = a_addr + (warp * 32 + r) * 128 + ((chunk ^ (r & 7)) << 4);
                const __half* src = in + (src_row >= 0 ? static_cast<size_t>(src_row) * cin + kb * 64 + chunk * 8 : 0);
                cp_async16(dst, src, src_row >= 0 ? 16u : 0u);
              }
            }
            cp_async_commit();
            if (j >= NS - 1) {
              cp_async_wait<NS - 1>();
              fence_proxy_async();
              mbar_arrive(smem_u32(&ctl->afull[pending_arrive % NS]));
              ++pending_arrive;
            }
          }
        }
      }
    }
    cp_async_wait<0>();
    fence_proxy_async();
    if (!ctl->abort_flag) {
      for (; pending_arrive < j; ++pending_arrive) mbar_arrive(smem_u32(&ctl->afull[pending_arrive % NS]));
    } else if (tid == 0) {
      // aborting: give this thread's bulk copies a bounded chance to land before the CTA leaves
      for (int u = max(0, j - NS); u < j; ++u) {
        const uint32_t bar = smem_u32(&ctl->bfull[u % NS]);
        for (int spin = 0; spin < (1 << 20) && !mbar_try_wait(bar, (u / NS) & 1); ++spin) {
        }
      }
    }
  } else if (warp == 4) {
    // =========================== MMA issuer ===========================
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (static_cast<uint32_t>(cout >> 3) << 17) | (static_cast<uint32_t>(kTileM >> 4) << 24);
      int j = 0;
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++it) {
        const int slot2 = it & 1;
        const uint32_t par2 = (it >> 1) & 1;
        ok = mbar_wait(smem_u32(&ctl->tfull[slot2]), par2, ctl);
        if (!ok) break;
        const int nst = ctl->tile_stages[slot2];
        mbar_arrive(smem_u32(&ctl->tempty[slot2]));
        // the accumulator must have been drained by the epilogue (two tiles ago)
        if (it >= 2) ok = mbar_wait(smem_u32(&ctl->accempty[slot2]), (par2 ^ 1), ctl);
        if (!ok) break;
        tc_fence_after();
        ctl->acc_stages[slot2] = nst;
        const uint32_t tmem_acc = tmem_base + static_cast<uint32_t>(slot2 * cout);
        uint32_t accumulate = 0;
        for (int st = 0; st < nst && ok; ++st, ++j) {
          const int s = j % NS;
          const uint32_t par = (j / NS) & 1;
          ok = mbar_wait(smem_u32(&ctl->afull[s]), par, ctl) && mbar_wait(smem_u32(&ctl->bfull[s]), par, ctl);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_addr = tiles_addr + s * stage_bytes;
          const uint64_t da = make_desc(a_addr);
          const uint64_t db = make_desc(a_addr + kABytes);
          const int kb = st % kblocks;
          const int ksteps = min(4, (cin - kb * 64) >> 4);
          for (int k = 0; k < ksteps; ++k) {
            tc_mma_f16(tmem_acc, da + static_cast<uint64_t>(k * 2), db + static_cast<uint64_t>(k * 2), idesc, accumulate);
            accumulate = 1;
          }
          tc_commit(smem_u32(&ctl->empty[s]));
        }
        if (!ok) break;
        // two arrivals complete the phase: this thread's own (release: publishes acc_stages) and
        // the commit's, which lands when every MMA of the tile has finished
        mbar_arrive(smem_u32(&ctl->accfull[slot2]));
        if (nst > 0)
          tc_commit(smem_u32(&ctl->accfull[slot2]));
        else
          mbar_arrive(smem_u32(&ctl->accfull[slot2]));  // no MMA was issued: the epilogue writes zeros
      }
    }
    __syncwarp();
    tc_fence_before();
  } else {
    // =========================== epilogue ===========================
    const int et = tid - 160;            // 0..127: accumulator lane == row slot of the tile
    const int lane_quarter = warp & 3;   // the TMEM lanes this warp may read: 32*(warp%4)..+31
    const int slot_in_tile = lane_quarter * 32 + lane;
    (void)et;
    int it = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++it) {
      const int slot2 = it & 1;
      const uint32_t par2 = (it >> 1) & 1;
      const int slot = tile * kTileM + slot_in_tile;
      int my_row = n_out;
      if (slot < n_out) my_row = order ? __ldg(order + slot) : slot;
      bool ok = mbar_wait(smem_u32(&ctl->accfull[slot2]), par2, ctl);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      tc_fence_after();
      const bool any = ctl->acc_stages[slot2] > 0;
      const bool store_row = my_row < n_out;
      const uint32_t taddr = tmem_base + static_cast<uint32_t>(slot2 * cout) + (static_cast<uint32_t>(lane_quarter * 32) << 16);
      __half* orow = out + static_cast<size_t>(store_row ? my_row : 0) * cout;
      const __half* rrow = (ep.residual && store_row) ? ep.residual + static_cast<size_t>(my_row) * cout : nullptr;
      for (int c0 = 0; c0 < cout; c0 += 16) {
        uint32_t r[16];
        if (any) {
          tmem_ld16(taddr + c0, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int q = 0; q < 16; ++q) r[q] = 0u;
        }
        float v[16];
#pragma unroll
        for (int q = 0; q < 16; ++q) v[q] = __uint_as_float(r[q]);
        if (ep.scale) {
#pragma unroll
          for (int q = 0; q < 16; q += 4) {
            const float4 s4 = __ldg(reinterpret_cast<const float4*>(ep.scale + c0 + q));
            v[q] *= s4.x;
            v[q + 1] *= s4.y;
            v[q + 2] *= s4.z;
            v[q + 3] *= s4.w;
          }
        }
        if (ep.shift) {
#pragma unroll
          for (int q = 0; q < 16; q += 4) {
            const float4 s4 = __ldg(reinterpret_cast<const float4*>(ep.shift + c0 + q));
            v[q] += s4.x;
            v[q + 1] += s4.y;
            v[q + 2] += s4.z;
            v[q + 3] += s4.w;
          }
        }
        if (rrow) {
          const uint4 ra = *reinterpret_cast<const uint4*>(rrow + c0);
          const uint4 rb = *reinterpret_cast<const uint4*>(rrow + c0 + 8);
          const __half2* ha = reinterpret_cast<const __half2*>(&ra);
          const __half2* hb = reinterpret_cast<const __half2*>(&rb);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float2 fa = __half22float2(ha[q]);
            const float2 fb = __half22float2(hb[q]);
            v[2 * q] += fa.x;
            v[2 * q + 1] += fa.y;
            v[8 + 2 * q] += fb.x;
            v[8 + 2 * q + 1] += fb.y;
          }
        }
        uint4 oa, ob;
        __half2* pa = reinterpret_cast<__half2*>(&oa);
        __half2* pb = reinterpret_cast<__half2*>(&ob);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          pa[q] = __floats2half2_rn(act_apply(v[2 * q], ep.act, ep.slope), act_apply(v[2 * q + 1], ep.act, ep.slope));
          pb[q] = __floats2half2_rn(act_apply(v[8 + 2 * q], ep.act, ep.slope),
                                    act_apply(v[8 + 2 * q + 1], ep.act, ep.slope));
        }
        if (store_row) {
          *reinterpret_cast<uint4*>(orow + c0) = oa;
          *reinterpret_cast<uint4*>(orow + c0 + 8) = ob;
        }
      }
      tc_fence_before();
      mbar_arrive(smem_u32(&ctl->accempty[slot2]));  // 128 arrivals hand the accumulator back
    }
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 4) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(static_cast<uint32_t>(tmem_cols))
                 : "memory");
  }
}

}  // namespace umma

bool conv_umma_supported(int cin, int cout, int dtype) {
  return dtype == PCE_F16 && cin >= 16 && cin % 16 == 0 && cout >= 16 && cout % 16 == 0 && cout <= 256;
}

size_t umma_packed_bytes(int kv, int cin, int cout) {
  return static_cast<size_t>(kv) * ((cin + 63) / 64) * cout * 128;
}

int umma_pack_weights(const void* w, int kv, int cin, int cout, void* packed, cudaStream_t st) {
  const int kblocks = (cin + 63) / 64;
  const long long total = static_cast<long long>(kv) * kblocks * cout * 64;
  const int grid = static_cast<int>(std::min<long long>((total + 255) / 256, 148ll * 8));
  umma::k_pack_weights<<<grid, 256, 0, st>>>(static_cast<const __half*>(w), kv, cin, cout, kblocks,
                                             static_cast<__half*>(packed));
  PCE_LAUNCH_CHECK();
  return PCE_OK;
}

int conv_umma(const void* in, const void* wpacked, const uint32_t* mask, const int* rowptr, const int* nbr,
              const int* order, int n_out, int cin, int cout, int kv, void* out, const pce_epilogue* ep,
              cudaStream_t st) {
  if (kv > 32 * umma::kMaxWords) return PCE_ERR_UNSUPPORTED;
  umma::Epi e{nullptr, nullptr, nullptr, PCE_ACT_NONE, 0.f};
  if (ep) e = umma::Epi{ep->scale, ep->shift, static_cast<const __half*>(ep->residual), ep->act, ep->slope};
  int tmem_cols = 32;
  while (tmem_cols < 2 * cout) tmem_cols <<= 1;  // two accumulators
  const size_t stage = static_cast<size_t>(umma::kABytes + cout * 128);
  const size_t fixed = sizeof(umma::SharedCtl) + 1024 + 64;
  const int ns = 4;
  const size_t smem = ns * stage + fixed;
  static int sm_count[64] = {};
  int dev = 0;
  PCE_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return PCE_ERR_UNSUPPORTED;
  if (sm_count[dev] == 0) {
    const size_t max_smem = static_cast<size_t>(umma::kMaxStages) * (umma::kABytes + 256 * 128) + fixed;
    PCE_CUDA(cudaFuncSetAttribute(umma::k_conv_umma<4>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  static_cast<int>(max_smem > 232448 ? 232448 : max_smem)));
    int n = 0;
    PCE_CUDA(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
    sm_count[dev] = n > 0 ? n : 1;
  }
  // CTAs that fit one SM: shared memory (227 KB), tensor memory (512 columns), at most 3
  int per_sm = static_cast<int>((227 * 1024) / (smem + 1024));
  if (per_sm > 512 / tmem_cols) per_sm = 512 / tmem_cols;
  if (per_sm > 3) per_sm = 3;
  if (per_sm < 1) per_sm = 1;
  const int n_tiles = div_up(n_out, umma::kTileM);
  const int grid = n_tiles < sm_count[dev] * per_sm ? n_tiles : sm_count[dev] * per_sm;
  umma::k_conv_umma<4><<<grid, 288, smem, st>>>(static_cast<const __half*>(in), static_cast<const __half*>(wpacked),
                                                mask, rowptr, nbr, order, n_out, cin, cout, kv,
                                                static_cast<__half*>(out), e, tmem_cols);
  PCE_LAUNCH_CHECK();
  return PCE_OK;
}

int umma_status_fetch(int* host_status, bool reset) {
  int v = 0;
  PCE_CUDA(cudaMemcpyFromSymbol(&v, g_umma_status, sizeof(int)));
  if (reset && v != 0) {
    int z = 0;
    PCE_CUDA(cudaMemcpyToSymbol(g_umma_status, &z, sizeof(int)));
  }
  *host_status = v;
  return PCE_OK;
}

}  // namespace pce
