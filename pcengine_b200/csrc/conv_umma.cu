// Fused gather-matmul-scatter on the 5th-generation tensor cores (tcgen05 + tensor
// memory), fp16 in / fp32 accumulate, output stationary, persistent and warp-specialised.
//
// The kernel reads the map as TILE LISTS (built once per kernel map by pce_build_tile_lists):
// output rows are taken in sorted order (pce_csr_sort_rows) in tiles of 128 or 256; for every
// tile the offsets that at least one of its rows has are listed (`stage_kp`), each with the
// input row to fetch per tile row (`stage_nbr`, -1 = this row lacks the offset).  A stage is one
// (tile, offset); offsets nobody in the tile has cost nothing (the indicator).  Lists built with
// the identity stage end every tile with a stage in which each row names itself: there a second
// operand (a residual block's shortcut) joins the accumulation.
//
// One CTA owns a contiguous range of tiles holding about 1/gridDim of the work and
// streams through that range's stages.  Threads (SUB = 128-row sub-tiles per tile):
//   4*SUB producer warps, one thread per tile row: per stage and 64-channel K block they
//              gather the input rows with 16-byte cp.async (4 rows per warp instruction,
//              full 128-byte lines, zero-fill for -1) into a 128-byte-swizzled K-major tile and
//              attach the stage's barrier to the copies (cp.async.mbarrier.arrive.noinc): the
//              barrier fires when the data has landed, the thread does not wait for it.
//              Thread 0 also stages the pre-packed weight block with one bulk async copy
//              (cp.async.bulk, the TMA engine).  Stage indices are read four stages ahead
//              (coalesced reads) into registers that are never moved, so the loads stay in
//              flight until the stage that uses them.
//              Measured on B200 (random 128-byte rows, L2 resident): cp.async sustains more
//              than 100 GB/s per SM, while TMA tile::gather4 and per-row bulk copies cost
//              about 43 ns per operation per issuing warp (11 GB/s per SM per warp), so the
//              row gather stays on cp.async and only the dense weight block uses TMA.
//   one MMA warp: one lane issues tcgen05.mma (M=128, N=C_out, K=16; one per sub-tile on the
//              same weight descriptor) and commits to mbarriers.
//   4 epilogue warps: tcgen05.ld the finished accumulator, apply
//              act(acc*scale + shift + residual), convert to fp16, store each row once (and, in
//              the PUSH variant, boundary rows a second time into a neighbouring GPU's halo).
// Rings: kStages smem stages (afull / bfull / empty mbarriers) that run on across tile
// boundaries, and one or two accumulator sets in tensor memory (accfull / accempty); with two,
// the gather of tile i+1, the MMAs of tile i and the stores of tile i-1 overlap.
// No atomics, no intermediate buffer in HBM, bit-identical run to run.
//
// Every mbarrier wait is bounded (~1 s): when one expires the CTA raises an abort flag,
// records PCE_ERR_TIMEOUT in the library's device status word, drains its own copies,
// frees its tensor memory and returns.
//
// Replaces fetch_on_demand_gemm_fp16_tc4_async and the cuBLAS centre GEMM of the
// reference (ref: backend/spconv.cuh:1567-1730, backend/spconv.cu:273-298,338).
#include "common.cuh"

namespace pce {

__device__ int g_umma_status = 0;
// Where the first bounded wait of a launch gave up: {code, CTA, item, extra}; code = role | sub-tile << 4 |
// tile-in-CTA << 8 with role 1 producer/row slot free, 2 loader/weight slot free, 3 MMA/weights landed,
// 4 MMA/accumulator drained, 5 MMA/rows landed, 6 MMA/accumulator drained (nothing written), 7 epilogue/
// accumulator complete (k_conv_umma_mt), 9 any wait of k_conv_umma.
__device__ int g_umma_where[4] = {0, 0, 0, 0};

namespace umma {

constexpr int kTileM = 128;
constexpr int kMaxStages = 6;
constexpr int kABytes = kTileM * 128;  // one A stage: 128 rows x 64 fp16
constexpr long long kWaitCycles = 2000000000ll;  // ~1 s at 2 GHz

struct Epi {
  const float* scale;
  const float* shift;
  const __half* residual;
  int act;
  float slope;
  // halo push: output row r is also stored to push_base[s] + push_slot[s][r] * cout (slot >= 0), memory
  // of a neighbouring GPU mapped into this process (plain peer stores over NVLink)
  const int* push_slot[2];
  __half* push_base[2];
  // row pitch of the input and the output features in elements (the channel count when dense): a layer
  // may read and write a column range of a wider row-major matrix
  int ld_in;
  int ld_out;
  // parts > 1: `parts` CTAs share every tile (CTA b: tile b / parts, part b % parts of its stage list) and
  // store raw fp32 sums to partial[(part * n_out + row) * cout + c]; k_sum_parts finishes the layer
  float* partial;
  int parts;
  // streamk: every CTA takes an equal share of the layer's STAGES (CTA b: stages S*b/G .. S*(b+1)/G of the
  // concatenated tile lists), whatever tiles they fall in.  A tile that lies in one CTA's share is finished by
  // it; a tile cut between CTAs leaves raw fp32 sums in partial[((cta*2 + slot)*128 + row-in-tile)*cout + c]
  // (slot 0: the CTA's first tile, 1: its last) and k_sum_cut_tiles finishes it.
  int streamk;
};

struct Lists {
  const int* order;      // [n_out] processing order of the output rows, or nullptr (natural)
  const int* tile_ptr;   // [n_tiles+1] first stage of every tile, or nullptr (dense product)
  const int* stage_kp;   // [stages] offset of every stage
  const int* stage_nbr;  // [stages][tile rows] input row per tile row, -1 absent
  int identity;          // every tile's last stage is the identity stage (stage_kp = -1)
  const __half* wslots;  // SLOTS > 1: weights as [kv][cout][cin] (one 16-byte chunk row per output channel)
  int settled;           // the lists were complete before the previous kernel of the stream was launched
};

// Second operand: out[row] += in2[row] @ w2, joined to the accumulation at the identity stage.
// The residual of a block (w2 = identity matrix) and its 1x1x1 shortcut convolution take this path.
struct Second {
  const __half* in2;  // [n_out][cin2], nullptr: none
  const __half* w2;   // packed like the weights of one offset: kblocks2 images of cout x 128 B
  int cin2;
};

struct SharedCtl {
  unsigned long long afull[kMaxStages];
  unsigned long long bfull[kMaxStages];
  unsigned long long empty[kMaxStages];
  unsigned long long accfull[2];
  unsigned long long accempty[2];
  uint32_t tmem_base;
  int range[2];  // this CTA's tiles [range[0], range[1])
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
template <class Ctl>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, Ctl* ctl, int where = 9, int item = 0) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  int spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if (((++spins) & 255) == 0) {
      if (ctl->abort_flag) return false;
      if (clock64() - t0 > kWaitCycles) {
        ctl->abort_flag = 1;
        atomicMax(&g_umma_status, PCE_ERR_TIMEOUT);
        if (atomicCAS(&g_umma_where[0], 0, where) == 0) {
          g_umma_where[1] = static_cast<int>(blockIdx.x);
          g_umma_where[2] = item;
          g_umma_where[3] = static_cast<int>(parity);
        }
        return false;
      }
    }
  }
  return true;
}

__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
// Makes the mbarrier receive one (already counted) arrival once every cp.async this thread has
// issued so far has landed: the thread itself does not wait.
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

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
// The same for operand tiles of KB channels per row: KB = 64 as above; KB = 32 rows of 64 B, 64-byte swizzle
// (16-byte chunk c of row r at chunk c ^ ((r >> 1) & 3)), 8-row groups 512 B apart.
template <int KB>
__device__ __forceinline__ uint64_t make_desc_kb(uint32_t smem_addr) {
  if constexpr (KB == 64) return make_desc(smem_addr);
  const uint32_t lo = ((smem_addr >> 4) & 0x3FFFu) | (1u << 16);
  const uint32_t hi = (512u >> 4) | (1u << 14) | (4u << 29);
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

// 32 bytes of a row in ONE store (256-bit vector access): half the store instructions, and half the requests to
// the load/store unit, of two 16-byte stores; `p` must be 32-byte aligned.
__device__ __forceinline__ void store32(void* p, const uint4& a, const uint4& b) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w),
               "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w)
               : "memory");
}

__device__ __forceinline__ void load32(const void* p, uint4& a, uint4& b) {
  asm volatile("ld.global.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w), "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w)
               : "l"(p)
               : "memory");
}

__device__ __forceinline__ float act_apply(float v, int act, float slope) {
  if (act == PCE_ACT_RELU) return v > 0.f ? v : 0.f;
  if (act == PCE_ACT_LEAKY) return v > 0.f ? v : v * slope;
  return v;
}

// Weights [kv][cin][cout] fp16 -> per (kp, k-block) shared-memory images of cout rows x 128 B
// (64 K elements, zero padded), 16-byte chunks XOR-swizzled with the row index.
// kb_size = 32: images of cout rows x 64 B (32 K elements), 64-byte swizzle (chunk ^ ((row >> 1) & 3)).
__global__ void k_pack_weights(const __half* __restrict__ w, int kv, int cin, int cout, int kblocks,
                               __half* __restrict__ packed, int kb_size) {
  if (kb_size == 32) {
    const long long total32 = static_cast<long long>(kv) * kblocks * cout * 32;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total32;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
      const int kk = static_cast<int>(i % 32);
      long long t = i / 32;
      const int co = static_cast<int>(t % cout);
      t /= cout;
      const int kb = static_cast<int>(t % kblocks);
      const int kp = static_cast<int>(t / kblocks);
      const int ci = kb * 32 + kk;
      __half v = __float2half(0.f);
      if (ci < cin) v = w[(static_cast<size_t>(kp) * cin + ci) * cout + co];
      const int chunk = kk >> 3, within = kk & 7;
      const size_t img = (static_cast<size_t>(kp) * kblocks + kb) * cout * 32;
      packed[img + static_cast<size_t>(co) * 32 + ((chunk ^ ((co >> 1) & 3)) << 3) + within] = v;
    }
    return;
  }
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

// Weights [kv][cin][cout] -> [kv][cout][cin]: per offset and output channel the cin input-channel values in a row.
__global__ void k_pack_weight_slots(const __half* __restrict__ w, int kv, int cin, int cout, __half* __restrict__ out) {
  const long long total = static_cast<long long>(kv) * cout * cin;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int ci = static_cast<int>(i % cin);
    const long long t = i / cin;
    const int co = static_cast<int>(t % cout);
    const int kp = static_cast<int>(t / cout);
    out[i] = w[(static_cast<size_t>(kp) * cin + ci) * cout + co];
  }
}

// Work of tiles [0, t): their stages plus one unit per tile for its fixed cost (epilogue).
__device__ __forceinline__ long long cost_before(const int* tile_ptr, int t) {
  return (tile_ptr ? static_cast<long long>(__ldg(tile_ptr + t)) : static_cast<long long>(t)) + t;
}

// First tile whose preceding work reaches `target` (cost_before is strictly increasing), found by a
// whole warp: 32 probes per round, so a list of n tiles takes log32(n) dependent loads instead of the
// log2(n) of a binary search (about 20 L2 round trips per CTA for both ends of its range, a fixed
// 15 us that was a tenth of the large layers and a third of the small ones).
__device__ __forceinline__ int warp_tile_at_cost(const int* tile_ptr, int n_tiles, long long target, int lane) {
  int lo = 0, hi = n_tiles;  // the answer lies in [lo, hi]
  while (lo < hi) {
    const int step = (hi - lo + 31) / 32;
    const int p = min(lo + (lane + 1) * step - 1, hi - 1);
    const unsigned m = __ballot_sync(0xFFFFFFFFu, cost_before(tile_ptr, p) >= target);
    if (m == 0) return hi;  // no tile in [lo, hi) reaches the target
    const int f = __ffs(m) - 1;
    const int hit = min(lo + (f + 1) * step - 1, hi - 1);
    lo = f == 0 ? lo : min(lo + f * step - 1, hi - 1) + 1;
    hi = hit;
  }
  return lo;
}

__device__ __forceinline__ int first_stage(const int* tile_ptr, int t) { return tile_ptr ? __ldg(tile_ptr + t) : t; }

// First tile t in [0, n_tiles) with tile_ptr[t + 1] > s (the tile that holds stage s), by a whole warp;
// n_tiles when there is none.
__device__ __forceinline__ int warp_tile_of_stage(const int* tile_ptr, int n_tiles, int s, int lane) {
  int lo = 0, hi = n_tiles;
  while (lo < hi) {
    const int step = (hi - lo + 31) / 32;
    const int p = min(lo + (lane + 1) * step - 1, hi - 1);
    const unsigned m = __ballot_sync(0xFFFFFFFFu, __ldg(tile_ptr + p + 1) > s);
    if (m == 0) return hi;
    const int f = __ffs(m) - 1;
    const int hit = min(lo + (f + 1) * step - 1, hi - 1);
    lo = f == 0 ? lo : min(lo + f * step - 1, hi - 1) + 1;
    hi = hit;
  }
  return lo;
}

// Share of CTA b of G in S stages: [S*b/G, S*(b+1)/G).
__host__ __device__ __forceinline__ int share_begin(long long total, int b, int g) {
  return static_cast<int>(total * b / g);
}

// kStages = depth of the smem stage ring.  SUB = 128-row sub-tiles per tile (1 or 2): a tile of 128*SUB output rows
// has SUB accumulators and every staged weight block feeds SUB MMAs, which halves the weight
// traffic per row for SUB = 2.  Threads: 4*SUB producer warps, the MMA warp, 4 epilogue warps.
// SLOTS = offsets per stage (1, 2, 4): with 32 or 16 input channels an offset fills half or a quarter
// of the 64-channel K block, so SLOTS offsets of a tile share one ring stage: every row gathers one
// neighbour per slot into its part of the 128-byte row, and the producers assemble the stage's weight
// block from the per-offset images with cp.async (covered by the same barrier as the rows).
// KB = channels per K block (64, or 32 for layers whose width is an odd multiple of 32: every stage is then
// full, where 64-channel blocks would spend half of every second stage's rows and weights on padding).
template <int kStages, int SUB, bool PUSH, int SLOTS, int KB = 64>
__global__ void __launch_bounds__(32 * (4 * SUB + 5), SUB == 1 ? 3 : 2)
    k_conv_umma(const __half* __restrict__ in, const __half* __restrict__ wpacked, Lists ls, Second sec, int n_out, int cin,
                int cout, __half* __restrict__ out, Epi ep, int tmem_cols, int nacc) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = ((raw_addr + 1023u) & ~1023u) - raw_addr;
  uint8_t* tiles = smem_raw + pad;  // 1024-byte aligned
  const uint32_t tiles_addr = raw_addr + pad;
  static_assert(KB == 64 || (KB == 32 && SUB == 1 && SLOTS == 1), "32-channel K blocks: plain variant only");
  constexpr int kRowBytes = KB * 2;            // one operand row of a stage
  const int b_bytes = cout * kRowBytes;
  constexpr int kRows = kTileM * SUB;          // output rows per tile
  constexpr int kAStage = kTileM * kRowBytes * SUB;  // gathered rows of one stage
  constexpr int kMmaWarp = 4 * SUB;
  const int stage_bytes = kAStage + b_bytes;   // both multiples of 1024
  SharedCtl* ctl = reinterpret_cast<SharedCtl*>(tiles + kStages * stage_bytes);
  // per-channel scale [cout] and shift [cout] of the epilogue (1 and 0 where absent), staged once per CTA: every
  // epilogue thread needs all of them for every tile, and read through the global path they cost the epilogue
  // eight 16-byte loads per 16-channel piece (96->96 on 486 k rows: 104 us without scale/shift, 146 us with)
  float* affine = reinterpret_cast<float*>(ctl + 1);
  static_assert(sizeof(SharedCtl) % 16 == 0, "the staged scale/shift are read as float4");

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int kblocks = (cin + KB - 1) / KB;
  const int kblocks2 = sec.in2 ? (sec.cin2 + KB - 1) / KB : 0;  // ring stages of the identity stage
  const int n_tiles = (n_out + kRows - 1) / kRows;
  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&ctl->afull[s]), kRows);
      mbar_init(smem_u32(&ctl->bfull[s]), 1);
      mbar_init(smem_u32(&ctl->empty[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&ctl->accfull[s]), 1);
      mbar_init(smem_u32(&ctl->accempty[s]), 128);
    }
    ctl->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp > kMmaWarp && (ep.scale || ep.shift)) {  // (constants of the layer, not outputs of the previous kernel)
    for (int c = tid - 32 * (kMmaWarp + 1); c < cout; c += 128) {
      affine[c] = ep.scale ? __ldg(ep.scale + c) : 1.f;
      affine[cout + c] = ep.shift ? __ldg(ep.shift + c) : 0.f;
    }
  }
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)),
                 "r"(static_cast<uint32_t>(tmem_cols))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // Launched with programmatic stream serialisation: everything above ran while the kernel before
  // this one in the stream was still finishing; the features and the output buffer may not be touched
  // before that kernel has completed and its writes are visible.  The tile lists may, when they are
  // older than that kernel (ls.settled): the search for this CTA's tiles and the first index loads
  // then overlap its tail as well.
  if (!ls.settled) asm volatile("griddepcontrol.wait;" ::: "memory");
  const int parts = ep.parts > 1 ? ep.parts : 1;
  const bool streamk = ep.streamk != 0;
  int sk_begin = 0, sk_end = 0;  // this CTA's share of the stages (streamk)
  if (streamk) {
    const long long total = __ldg(ls.tile_ptr + n_tiles);
    sk_begin = share_begin(total, static_cast<int>(blockIdx.x), static_cast<int>(gridDim.x));
    sk_end = share_begin(total, static_cast<int>(blockIdx.x) + 1, static_cast<int>(gridDim.x));
    if (warp < 2) {
      int t = 0;
      if (sk_end > sk_begin) t = warp_tile_of_stage(ls.tile_ptr, n_tiles, warp == 0 ? sk_begin : sk_end - 1, lane) + warp;
      if (lane == 0) ctl->range[warp] = t;
    }
  } else if (parts > 1) {
    // split tiles: this CTA owns ONE tile and one part of its stage list
    if (tid == 0) {
      ctl->range[0] = static_cast<int>(blockIdx.x) / parts;
      ctl->range[1] = static_cast<int>(blockIdx.x) / parts + 1;
    }
  } else if (warp < 2) {
    // this CTA's contiguous share of the tiles, balanced by work: warp 0 finds its first tile,
    // warp 1 the next CTA's first tile
    const long long total = cost_before(ls.tile_ptr, n_tiles);
    const unsigned b = blockIdx.x + warp;
    const int t = b >= gridDim.x ? n_tiles : warp_tile_at_cost(ls.tile_ptr, n_tiles, total * b / gridDim.x, lane);
    if (lane == 0) ctl->range[warp] = t;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;

  const int t0 = ctl->range[0], t1 = ctl->range[1];
  // stage range of tile t that this CTA works on: the whole tile, or its part
  auto stage_range = [&](int t, int& sa, int& sb) {
    sa = first_stage(ls.tile_ptr, t);
    sb = first_stage(ls.tile_ptr, t + 1);
    if (streamk) {
      sa = max(sa, sk_begin);
      sb = min(sb, sk_end);
    } else if (parts > 1) {
      const int n = sb - sa, part = static_cast<int>(blockIdx.x) % parts;
      const int a = sa + static_cast<int>(static_cast<long long>(n) * part / parts);
      sb = sa + static_cast<int>(static_cast<long long>(n) * (part + 1) / parts);
      sa = a;
    }
  };
  // streamk: does this CTA hold only a piece of tile t?
  auto tile_cut = [&](int t) {
    return streamk && (sk_begin > first_stage(ls.tile_ptr, t) || sk_end < first_stage(ls.tile_ptr, t + 1));
  };
  // ring stages of tile t (this CTA's part of it): its listed offsets times the K blocks; the identity
  // stage, which is the tile's last, counts with the second operand's K blocks (none without one)
  auto tile_ident = [&](int t) {
    int sa, sb;
    stage_range(t, sa, sb);
    return (ls.identity && sb > sa && sb == first_stage(ls.tile_ptr, t + 1)) ? 1 : 0;
  };
  auto tile_main_stages = [&](int t) {
    int sa, sb;
    stage_range(t, sa, sb);
    return (sb - sa - tile_ident(t)) * kblocks;
  };

  if (warp < kMmaWarp) {
    // =========================== producers ===========================
    int g0 = first_stage(ls.tile_ptr, t0), g1 = first_stage(ls.tile_ptr, t1);
    if (parts > 1) stage_range(t0, g0, g1);
    if (streamk) {
      g0 = sk_begin;
      g1 = sk_end;
    }
    constexpr int kCpr = KB / 8;                // 16-byte chunks per operand row (8 or 4)
    constexpr int kRowsPerInstr = 32 / kCpr;    // rows one warp instruction covers (4 or 8)
    const int rsub = lane / kCpr;   // row inside the group of rows of one instruction
    const int chunk = lane % kCpr;  // 16-byte chunk inside the row
    int j = 0;  // smem stages issued so far (continuous over tiles)
    bool ok = true;
    // destination of this thread's copy q inside a stage: row q * kRowsPerInstr + rsub of the warp's 32, chunk
    // swizzled with the row; the swizzle term takes two values (q even / odd), everything else is q * constant
    const int sw_even = KB == 64 ? (chunk ^ rsub) : (chunk ^ ((rsub >> 1) & 3));
    const int sw_odd = KB == 64 ? (chunk ^ (rsub + 4)) : sw_even;
    const uint32_t dst_even = (warp * 32 + rsub) * kRowBytes + (sw_even << 4);
    const uint32_t dst_odd = (warp * 32 + rsub) * kRowBytes + (sw_odd << 4);
    if constexpr (SLOTS == 1) {
    auto load_stage = [&](int g, int& nid, int& kp) {
      nid = -1;
      kp = 0;
      if (g < g1) {
        if (ls.tile_ptr) {
          nid = __ldg(ls.stage_nbr + static_cast<size_t>(g) * kRows + tid);
          kp = __ldg(ls.stage_kp + g);
          if (kp >= 0) kp &= 255;  // bits 8.. hold the sub-tile presence mask (read by k_conv_umma_mt)
        } else {  // dense product: stage g is tile g, every row fetches itself at offset 0
          const int row = g * kRows + tid;
          nid = row < n_out ? row : -1;
        }
      }
    };
    auto run_stage = [&](int nid, int kp) {
      const bool second = kp < 0;  // the identity stage
      const char* src_base = reinterpret_cast<const char*>(second ? sec.in2 : in) + chunk * 16;
      const int width = second ? sec.cin2 : cin;
      const int pitch_bytes = (second ? sec.cin2 : ep.ld_in) * 2;
      const int nkb = second ? kblocks2 : kblocks;  // 0: listed, but this launch has no second operand
      // the rows this thread fetches in this stage (the same for every K block)
      int rows[kCpr];
#pragma unroll
      for (int q = 0; q < kCpr; ++q) rows[q] = __shfl_sync(0xFFFFFFFFu, nid, q * kRowsPerInstr + rsub);
      for (int kb = 0; kb < nkb; ++kb, ++j) {
        const int s = j % kStages;
        const int n = j / kStages;
        if (n > 0) ok = mbar_wait(smem_u32(&ctl->empty[s]), (n - 1) & 1, ctl);
        ok = __all_sync(0xFFFFFFFFu, ok);  // keep the warp convergent
        if (!ok) return;
        const uint32_t a_addr = tiles_addr + s * stage_bytes;
        if (tid == 0) {
          const uint32_t bbar = smem_u32(&ctl->bfull[s]);
          mbar_arrive_expect_tx(bbar, b_bytes);
          const __half* wsrc = second ? sec.w2 + static_cast<size_t>(kb) * cout * KB
                                      : wpacked + (static_cast<size_t>(kb) + static_cast<size_t>(kp) * kblocks) * cout * KB;
          bulk_copy_g2s(a_addr + kAStage, wsrc, b_bytes, bbar);
        }
        if (chunk < min(kCpr, (width - kb * KB) >> 3)) {
          const char* src_kb = src_base + kb * (KB * 2);
#pragma unroll
          for (int q = 0; q < kCpr; ++q) {
            const int row = rows[q];
            const uint32_t dst = a_addr + ((q & 1) ? dst_odd : dst_even) + q * (kRowsPerInstr * kRowBytes);
            const char* src = src_kb + static_cast<long long>(row > 0 ? row : 0) * pitch_bytes;
            cp_async16(dst, src, row >= 0 ? 16u : 0u);
          }
        }
        // the stage's "rows landed" barrier fires by itself when this thread's copies are done, so a
        // stage becomes usable as soon as its data is there, whatever this thread waits for next
        cp_async_arrive_noinc(smem_u32(&ctl->afull[s]));
      }
    };
    // Four index registers, each reloaded right after its stage has been issued and not
    // touched again until four stages later: the loads stay in flight across the stages between.
    int nid0, nid1, nid2, nid3, kp0, kp1, kp2, kp3;
    load_stage(g0, nid0, kp0);
    load_stage(g0 + 1, nid1, kp1);
    load_stage(g0 + 2, nid2, kp2);
    load_stage(g0 + 3, nid3, kp3);
    if (ls.settled) asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int g = g0; g < g1 && ok; g += 4) {
      run_stage(nid0, kp0);
      load_stage(g + 4, nid0, kp0);
      if (g + 1 < g1 && ok) run_stage(nid1, kp1);
      load_stage(g + 5, nid1, kp1);
      if (g + 2 < g1 && ok) run_stage(nid2, kp2);
      load_stage(g + 6, nid2, kp2);
      if (g + 3 < g1 && ok) run_stage(nid3, kp3);
      load_stage(g + 7, nid3, kp3);
    }
    } else {
    // ---- several offsets per stage (cin = 64 / SLOTS channels each) ----
    constexpr int kSlotChunks = 8 / SLOTS;  // 16-byte chunks of one slot inside the 128-byte row
    const int my_slot = chunk / kSlotChunks, my_cc = chunk % kSlotChunks;
    auto load_stage = [&](int g, int (&nid)[SLOTS], int (&kp)[SLOTS]) {
#pragma unroll
      for (int q = 0; q < SLOTS; ++q) {
        nid[q] = -1;
        kp[q] = -2;
        if (g < g1) {
          nid[q] = __ldg(ls.stage_nbr + (static_cast<size_t>(g) * SLOTS + q) * kRows + tid);
          kp[q] = __ldg(ls.stage_kp + static_cast<size_t>(g) * SLOTS + q);
        }
      }
    };
    auto run_stage = [&](const int (&nid)[SLOTS], const int (&kp)[SLOTS]) {
      const bool second = kp[0] == -1;  // the identity stage: slot 0 only, the second operand's width
      const int nkb = second ? kblocks2 : 1;
      for (int kb = 0; kb < nkb; ++kb, ++j) {
        const int s = j % kStages;
        const int n = j / kStages;
        if (n > 0) ok = mbar_wait(smem_u32(&ctl->empty[s]), (n - 1) & 1, ctl);
        ok = __all_sync(0xFFFFFFFFu, ok);
        if (!ok) return;
        const uint32_t a_addr = tiles_addr + s * stage_bytes;
        const uint32_t b_addr = a_addr + kAStage;
        if (second) {
          if (tid == 0) {
            const uint32_t bbar = smem_u32(&ctl->bfull[s]);
            mbar_arrive_expect_tx(bbar, b_bytes);
            bulk_copy_g2s(b_addr, sec.w2 + static_cast<size_t>(kb) * cout * 64, b_bytes, bbar);
          }
          const int kchunks = min(8, (sec.cin2 - kb * 64) >> 3);
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const int r = q * 4 + rsub;
            const int src_row = __shfl_sync(0xFFFFFFFFu, nid[0], r);
            if (chunk < kchunks) {
              const uint32_t dst = a_addr + (warp * 32 + r) * 128 + ((chunk ^ (r & 7)) << 4);
              const __half* src = sec.in2 + (src_row >= 0 ? static_cast<size_t>(src_row) * sec.cin2 + kb * 64 + chunk * 8 : 0);
              cp_async16(dst, src, src_row >= 0 ? 16u : 0u);
            }
          }
        } else {
          if (tid == 0) mbar_arrive(smem_u32(&ctl->bfull[s]));  // the weights below ride on afull; keep bfull's phase in step
          // weight block: per slot the offset's [cout][cin] image, chunk by chunk into the swizzled
          // K-major block; unused slots are zero-filled so that the MMA can always run all K steps
          // (chunk ch of output channel co's 128-byte row belongs to slot ch / kSlotChunks: no run-time division)
          for (int c = tid; c < cout * 8; c += kRows) {
            const int co = c >> 3, ch = c & 7;
            const int q = ch / kSlotChunks, cc = ch % kSlotChunks;
            int kq = kp[0];
#pragma unroll
            for (int u = 1; u < SLOTS; ++u) kq = q == u ? kp[u] : kq;
            const uint32_t dst = b_addr + co * 128 + ((ch ^ (co & 7)) << 4);
            const __half* src = ls.wslots + (kq >= 0 ? (static_cast<size_t>(kq) * cout + co) * cin + cc * 8 : 0);
            cp_async16(dst, src, kq >= 0 ? 16u : 0u);
          }
          const char* src_lane = reinterpret_cast<const char*>(in) + my_cc * 16;
          const int pitch_bytes = ep.ld_in * 2;
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const int r = q * 4 + rsub;
            int src_row = -1;
#pragma unroll
            for (int u = 0; u < SLOTS; ++u) {
              const int v = __shfl_sync(0xFFFFFFFFu, nid[u], r);
              if (u == my_slot) src_row = v;
            }
            const uint32_t dst = a_addr + ((q & 1) ? dst_odd : dst_even) + q * (4 * 128);
            const char* src = src_lane + static_cast<long long>(src_row > 0 ? src_row : 0) * pitch_bytes;
            cp_async16(dst, src, src_row >= 0 ? 16u : 0u);
          }
        }
        cp_async_arrive_noinc(smem_u32(&ctl->afull[s]));
      }
    };
    // two stages of indices in flight (SLOTS entries each)
    int nidA[SLOTS], kpA[SLOTS], nidB[SLOTS], kpB[SLOTS];
    load_stage(g0, nidA, kpA);
    load_stage(g0 + 1, nidB, kpB);
    if (ls.settled) asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int g = g0; g < g1 && ok; g += 2) {
      run_stage(nidA, kpA);
      load_stage(g + 2, nidA, kpA);
      if (g + 1 < g1 && ok) run_stage(nidB, kpB);
      load_stage(g + 3, nidB, kpB);
    }
    }
    cp_async_wait_all();
    if (!ok && tid == 0) {
      // aborting: give this thread's bulk copies a bounded chance to land before the CTA leaves
      for (int u = max(0, j - kStages); u < j; ++u) {
        const uint32_t bar = smem_u32(&ctl->bfull[u % kStages]);
        for (int spin = 0; spin < (1 << 20) && !mbar_try_wait(bar, (u / kStages) & 1); ++spin) {
        }
      }
    }
  } else if (warp == kMmaWarp) {
    // =========================== MMA issuer ===========================
    if (ls.settled) asm volatile("griddepcontrol.wait;" ::: "memory");
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (static_cast<uint32_t>(cout >> 3) << 17) | (static_cast<uint32_t>(kTileM >> 4) << 24);
      int j = 0;
      bool ok = true;
      for (int t = t0; t < t1 && ok; ++t) {
        const int it = t - t0;
        const int buf = it % nacc;
        const int nst_main = tile_main_stages(t);
        const int nst = nst_main + (tile_ident(t) ? kblocks2 : 0);
        // the accumulator must have been drained by the epilogue (two tiles ago)
        if (it >= nacc) ok = mbar_wait(smem_u32(&ctl->accempty[buf]), ((it / nacc) - 1) & 1, ctl);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_acc = tmem_base + static_cast<uint32_t>(buf * SUB * cout);
        uint32_t accumulate = 0;
        for (int st = 0; st < nst && ok; ++st, ++j) {
          const int s = j % kStages;
          const uint32_t par = (j / kStages) & 1;
          ok = mbar_wait(smem_u32(&ctl->afull[s]), par, ctl) && mbar_wait(smem_u32(&ctl->bfull[s]), par, ctl);
          if (!ok) break;
          fence_proxy_async();  // the gathered rows were written through the generic proxy
          tc_fence_after();
          const uint32_t a_addr = tiles_addr + s * stage_bytes;
          const uint64_t db = make_desc_kb<KB>(a_addr + kAStage);
          const bool second = st >= nst_main;
          const int kb = second ? st - nst_main : st % kblocks;
          // with several offsets per stage the whole 64-channel block is always filled (unused slots with zeros)
          const int ksteps = (SLOTS > 1 && !second) ? 4 : min(KB / 16, ((second ? sec.cin2 : cin) - kb * KB) >> 4);
          for (int k = 0; k < ksteps; ++k) {
#pragma unroll
            for (int sub = 0; sub < SUB; ++sub) {  // the same weight block feeds every sub-tile
              const uint64_t da = make_desc_kb<KB>(a_addr + sub * (kTileM * kRowBytes));
              tc_mma_f16(tmem_acc + static_cast<uint32_t>(sub * cout), da + static_cast<uint64_t>(k * 2),
                         db + static_cast<uint64_t>(k * 2), idesc, accumulate);
            }
            accumulate = 1;
          }
          tc_commit(smem_u32(&ctl->empty[s]));
        }
        if (!ok) break;
        if (nst > 0)
          tc_commit(smem_u32(&ctl->accfull[buf]));  // arrives when every MMA of the tile has finished
        else
          mbar_arrive(smem_u32(&ctl->accfull[buf]));  // no MMA was issued: the epilogue writes zeros
      }
    }
    __syncwarp();
    tc_fence_before();
  } else {
    // =========================== epilogue ===========================
    const int lane_quarter = warp & 3;  // the TMEM lanes this warp may read: 32*(warp%4)..+31
    const int slot_in_tile = lane_quarter * 32 + lane;
    // every 16-channel piece of an output row is 32-byte aligned: one 256-bit store per piece
    const bool wide_out = (ep.ld_out & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 31) == 0;
    const bool wide_res = (reinterpret_cast<uintptr_t>(ep.residual) & 31) == 0;  // (rows of C_out = 16k channels)
    if (ls.settled) asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int t = t0; t < t1; ++t) {
      const int it = t - t0;
      const int buf = it % nacc;
      int rows_of[SUB];
#pragma unroll
      for (int sub = 0; sub < SUB; ++sub) {
        const int slot = t * kRows + sub * kTileM + slot_in_tile;
        rows_of[sub] = n_out;
        if (slot < n_out) rows_of[sub] = ls.order ? __ldg(ls.order + slot) : slot;
      }
      const bool any = tile_main_stages(t) + (tile_ident(t) ? kblocks2 : 0) > 0;
      const bool cut = tile_cut(t);
      if (ep.residual) {
        // the rows are known before the accumulator is: pull the residual rows into L2 while waiting
#pragma unroll
        for (int sub = 0; sub < SUB; ++sub) {
          if (rows_of[sub] < n_out) {
            const char* rp = reinterpret_cast<const char*>(ep.residual + static_cast<size_t>(rows_of[sub]) * cout);
            for (int off = 0; off < cout * 2; off += 64) asm volatile("prefetch.global.L2 [%0];" ::"l"(rp + off));
          }
        }
      }
      bool ok = mbar_wait(smem_u32(&ctl->accfull[buf]), (it / nacc) & 1, ctl);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      tc_fence_after();
      // last tile of this CTA: once every CTA is here (or gone), the next kernel of the stream may be
      // set up on the SMs; it waits for this grid's completion before it touches memory
      if (t == t1 - 1) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#pragma unroll
      for (int sub = 0; sub < SUB; ++sub) {
      const int my_row = rows_of[sub];
      const bool store_row = my_row < n_out;
      const uint32_t taddr = tmem_base + static_cast<uint32_t>((buf * SUB + sub) * cout) +
                             (static_cast<uint32_t>(lane_quarter * 32) << 16);
      __half* orow = out + static_cast<size_t>(store_row ? my_row : 0) * ep.ld_out;
      __half* prow[2] = {nullptr, nullptr};
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        if (PUSH && ep.push_slot[s] && store_row) {
          const int slot = __ldg(ep.push_slot[s] + my_row);
          if (slot >= 0) prow[s] = ep.push_base[s] + static_cast<size_t>(slot) * cout;
        }
      }
      const __half* rrow = (ep.residual && store_row) ? ep.residual + static_cast<size_t>(my_row) * cout : nullptr;
      for (int c0 = 0; c0 < cout; c0 += 16) {
        uint4 ra = make_uint4(0u, 0u, 0u, 0u), rb = ra;
        if (rrow) {  // issued ahead of the tensor-memory load, consumed after it
          if (wide_res) {
            load32(rrow + c0, ra, rb);
          } else {
            ra = *reinterpret_cast<const uint4*>(rrow + c0);
            rb = *reinterpret_cast<const uint4*>(rrow + c0 + 8);
          }
        }
        uint32_t r[16];
        if (any) {  // warp-uniform: the tensor-memory load is warp-collective
          tmem_ld16(taddr + c0, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int q = 0; q < 16; ++q) r[q] = 0u;
        }
        float v[16];
#pragma unroll
        for (int q = 0; q < 16; ++q) v[q] = __uint_as_float(r[q]);
        if (parts > 1) {  // a part of a split tile: the raw sums go to the scratch, k_sum_parts finishes the row
          if (store_row) {
            float4* dst = reinterpret_cast<float4*>(
                ep.partial + (static_cast<size_t>(blockIdx.x % parts) * n_out + my_row) * cout + c0);
#pragma unroll
            for (int q = 0; q < 4; ++q) dst[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
          }
          continue;
        }
        if (cut) {  // a piece of a tile cut between CTAs: k_sum_cut_tiles adds the pieces
          float4* dst = reinterpret_cast<float4*>(
              ep.partial + ((static_cast<size_t>(blockIdx.x) * 2 + (t == t0 ? 0 : 1)) * kTileM + slot_in_tile) * cout + c0);
#pragma unroll
          for (int q = 0; q < 4; ++q) dst[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
          continue;
        }
        if (ep.scale || ep.shift) {
#pragma unroll
          for (int q = 0; q < 16; q += 4) {
            const float4 s4 = *reinterpret_cast<const float4*>(affine + c0 + q);
            const float4 t4 = *reinterpret_cast<const float4*>(affine + cout + c0 + q);
            v[q] = fmaf(v[q], s4.x, t4.x);
            v[q + 1] = fmaf(v[q + 1], s4.y, t4.y);
            v[q + 2] = fmaf(v[q + 2], s4.z, t4.z);
            v[q + 3] = fmaf(v[q + 3], s4.w, t4.w);
          }
        }
        if (rrow) {
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
          if (wide_out) {
            store32(orow + c0, oa, ob);
          } else {
            *reinterpret_cast<uint4*>(orow + c0) = oa;
            *reinterpret_cast<uint4*>(orow + c0 + 8) = ob;
          }
        }
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          if (PUSH && prow[s]) {
            *reinterpret_cast<uint4*>(prow[s] + c0) = oa;
            *reinterpret_cast<uint4*>(prow[s] + c0 + 8) = ob;
          }
        }
      }
      }  // sub-tiles
      tc_fence_before();
      mbar_arrive(smem_u32(&ctl->accempty[buf]));  // 128 arrivals hand the accumulator back
    }
    tc_fence_before();
  }
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(static_cast<uint32_t>(tmem_cols))
                 : "memory");
  }
}


// =====================================================================================================
// k_conv_umma_mt: several accumulators per CTA, offsets taken in offset-major order, row ring and weight
// ring decoupled.
//
// A super-tile is SUB (1, 2 or 4) consecutive 128-row sub-tiles of the processing order, each with its own
// accumulator in tensor memory.  The tile lists of a super-tile name every offset that any of its rows has,
// with a presence bit per sub-tile (stage_kp bits 8..).  Per listed offset and 64-channel K block the weight
// block is staged ONCE (weight ring, nb slots of C_out x 128 B, one bulk async copy each) and multiplied
// with the gathered rows of every sub-tile that has the offset (row ring, na slots of 128 rows x 128 B).
// Against one ring stage = rows + weights per (128-row tile, offset) this
//   * divides the weight traffic from L2 by the number of sub-tiles that share an offset (rows are sorted
//     by indicator bitmask, so neighbouring sub-tiles share most of theirs), and
//   * frees the shared memory that every stage spent on its own weight copy for row slots: what limits
//     the fused kernel is the number of row gathers in flight per SM (a ring slot is occupied for about
//     3 us from the first copy instruction to the release by the tensor core).
// Warps: 4*SUB producers (one thread per row of the super-tile; the four warps of a sub-tile fill that
// sub-tile's row slots), one MMA warp (one lane issues), one weight-loader warp (one lane), 4*EPIW
// epilogue warps (EPIW teams; team e drains the accumulators of sub-tiles e, e+EPIW, ..).  All follow the
// same sequence: stage g of the super-tile, K block kb, present sub-tiles in ascending order.  Every
// sub-tile has its OWN ring of na row slots: a slot is then filled and released by the same warps in
// strict alternation, which the parity waits of mbarriers need (a ring shared between sub-tiles lets a
// sub-tile that skipped a use of a slot run two phases ahead of its barrier, where the parity test
// passes wrongly).  With nsets = 2 the accumulators alternate between super-tiles, so the epilogue
// of super-tile i overlaps the products of i+1.  Same bounded waits, abort protocol, programmatic dependent
// launch and epilogue as k_conv_umma; results are bit-identical to it (same products, same order per row).
constexpr int kMaxA = 16;
constexpr int kMaxB = 4;
constexpr int kMaxAcc = 8;

struct SharedCtlMt {
  unsigned long long afull[kMaxA];
  unsigned long long aempty[kMaxA];
  unsigned long long bfull[kMaxB];
  unsigned long long bempty[kMaxB];
  unsigned long long accfull[kMaxAcc];
  unsigned long long accempty[kMaxAcc];
  uint32_t tmem_base;
  int range[2];
  volatile int abort_flag;
};

// stage_kp entry -> (offset or -1 for the identity stage, presence mask over the sub-tiles)
template <int SUB>
__device__ __forceinline__ void decode_stage(int code, int& kp, uint32_t& present) {
  constexpr uint32_t kAll = (1u << SUB) - 1u;
  if (code < 0) {
    kp = code;
    present = code == -1 ? kAll : 0u;
    return;
  }
  kp = code & 255;
  present = (static_cast<uint32_t>(code) >> 8) & kAll;
  if (present == 0u) present = kAll;  // lists without presence bits: every sub-tile takes part
}

template <int SUB, int EPIW>
__global__ void __launch_bounds__(32 * (4 * SUB + 2 + 4 * EPIW), SUB == 1 ? 2 : 1)
    k_conv_umma_mt(const __half* __restrict__ in, const __half* __restrict__ wpacked, Lists ls, Second sec, int n_out, int cin,
                   int cout, __half* __restrict__ out, Epi ep, int tmem_cols, int na, int nb, int nsets) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = ((raw_addr + 1023u) & ~1023u) - raw_addr;
  uint8_t* tiles = smem_raw + pad;  // 1024-byte aligned
  const uint32_t a_base = raw_addr + pad;
  const int b_bytes = cout * 128;
  const uint32_t b_base = a_base + static_cast<uint32_t>(SUB * na) * kABytes;  // na row slots per sub-tile
  constexpr int kRows = kTileM * SUB;
  constexpr int kProd = 4 * SUB;  // producer warps
  constexpr int kMmaWarp = kProd;
  constexpr int kLoadWarp = kProd + 1;
  SharedCtlMt* ctl =
      reinterpret_cast<SharedCtlMt*>(tiles + static_cast<size_t>(SUB * na) * kABytes + static_cast<size_t>(nb) * b_bytes);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int kblocks = (cin + 63) >> 6;
  const int kblocks2 = sec.in2 ? (sec.cin2 + 63) >> 6 : 0;
  const int n_tiles = (n_out + kRows - 1) / kRows;

  if (tid == 0) {
    for (int s = 0; s < SUB * na; ++s) {
      mbar_init(smem_u32(&ctl->afull[s]), kTileM);
      mbar_init(smem_u32(&ctl->aempty[s]), 1);
    }
    for (int s = 0; s < nb; ++s) {
      mbar_init(smem_u32(&ctl->bfull[s]), 1);
      mbar_init(smem_u32(&ctl->bempty[s]), 1);
    }
    for (int s = 0; s < kMaxAcc; ++s) {
      mbar_init(smem_u32(&ctl->accfull[s]), 1);
      mbar_init(smem_u32(&ctl->accempty[s]), 128);
    }
    ctl->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)),
                 "r"(static_cast<uint32_t>(tmem_cols))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (!ls.settled) asm volatile("griddepcontrol.wait;" ::: "memory");
  if (warp < 2) {
    const long long total = cost_before(ls.tile_ptr, n_tiles);
    const unsigned b = blockIdx.x + warp;
    const int t = b >= gridDim.x ? n_tiles : warp_tile_at_cost(ls.tile_ptr, n_tiles, total * b / gridDim.x, lane);
    if (lane == 0) ctl->range[warp] = t;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  const int t0 = ctl->range[0], t1 = ctl->range[1];
  const int g0 = __ldg(ls.tile_ptr + t0), g1 = __ldg(ls.tile_ptr + t1);

  if (warp < kProd) {
    // =========================== row producers ===========================
    const int sub = warp >> 2;          // this warp's sub-tile
    const int row_in_sub = tid & 127;   // this thread's row inside it
    const int wq = warp & 3;            // warp inside the sub-tile
    const int rsub = lane >> 3;         // row inside a 4-row group
    const int chunk = lane & 7;         // 16-byte chunk inside a 128-byte row
    const int ring0 = sub * na;  // this sub-tile's own row slots: ring0 .. ring0 + na - 1
    int js = 0;                  // row items this sub-tile has produced so far
    bool ok = true;
    auto load_stage = [&](int g, int& nid, int& code) {
      nid = -1;
      code = -2;
      if (g < g1) {
        code = __ldg(ls.stage_kp + g);
        int kp;
        uint32_t present;
        decode_stage<SUB>(code, kp, present);
        if ((present >> sub) & 1u) nid = __ldg(ls.stage_nbr + static_cast<size_t>(g) * kRows + sub * kTileM + row_in_sub);
      }
    };
    auto run_stage = [&](int nid, int code) {
      int kp;
      uint32_t present;
      decode_stage<SUB>(code, kp, present);
      if (!((present >> sub) & 1u)) return;
      const bool second = kp == -1;
      const int nkb = second ? kblocks2 : kblocks;
      const __half* src_base = second ? sec.in2 : in;
      const int width = second ? sec.cin2 : cin;
      const int pitch = second ? sec.cin2 : ep.ld_in;
      for (int kb = 0; kb < nkb; ++kb, ++js) {
        const int s = ring0 + js % na;
        const int n = js / na;
        if (n > 0) ok = mbar_wait(smem_u32(&ctl->aempty[s]), (n - 1) & 1, ctl, 1 | (sub << 4), js);
        ok = __all_sync(0xFFFFFFFFu, ok);  // keep the warp convergent for the shuffles below
        if (!ok) return;
        const uint32_t a_addr = a_base + static_cast<uint32_t>(s) * kABytes;
        const int kchunks = min(8, (width - kb * 64) >> 3);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const int r = q * 4 + rsub;  // row inside this warp's 32
          const int src_row = __shfl_sync(0xFFFFFFFFu, nid, r);
          if (chunk < kchunks) {
            const uint32_t dst = a_addr + (wq * 32 + r) * 128 + ((chunk ^ (r & 7)) << 4);
            const __half* src = src_base + (src_row >= 0 ? static_cast<size_t>(src_row) * pitch + kb * 64 + chunk * 8 : 0);
            cp_async16(dst, src, src_row >= 0 ? 16u : 0u);
          }
        }
        cp_async_arrive_noinc(smem_u32(&ctl->afull[s]));
      }
    };
    int nid0, nid1, nid2, nid3, c0, c1, c2, c3;
    load_stage(g0, nid0, c0);
    load_stage(g0 + 1, nid1, c1);
    load_stage(g0 + 2, nid2, c2);
    load_stage(g0 + 3, nid3, c3);
    if (ls.settled) asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int g = g0; g < g1 && ok; g += 4) {
      run_stage(nid0, c0);
      load_stage(g + 4, nid0, c0);
      if (g + 1 < g1 && ok) run_stage(nid1, c1);
      load_stage(g + 5, nid1, c1);
      if (g + 2 < g1 && ok) run_stage(nid2, c2);
      load_stage(g + 6, nid2, c2);
      if (g + 3 < g1 && ok) run_stage(nid3, c3);
      load_stage(g + 7, nid3, c3);
    }
    cp_async_wait_all();
  } else if (warp == kLoadWarp) {
    // =========================== weight loader ===========================
    if (ls.settled) asm volatile("griddepcontrol.wait;" ::: "memory");
    if (lane == 0) {
      int jb = 0;
      bool ok = true;
      for (int g = g0; g < g1 && ok; ++g) {
        int kp;
        uint32_t present;
        decode_stage<SUB>(__ldg(ls.stage_kp + g), kp, present);
        const bool second = kp == -1;
        const int nkb = second ? kblocks2 : kblocks;
        if (present == 0u) continue;
        for (int kb = 0; kb < nkb; ++kb, ++jb) {
          const int s = jb % nb;
          const int n = jb / nb;
          if (n > 0) ok = mbar_wait(smem_u32(&ctl->bempty[s]), (n - 1) & 1, ctl, 2, jb);
          if (!ok) break;
          const uint32_t bbar = smem_u32(&ctl->bfull[s]);
          mbar_arrive_expect_tx(bbar, b_bytes);
          const __half* wsrc = second ? sec.w2 + static_cast<size_t>(kb) * cout * 64
                                      : wpacked + (static_cast<size_t>(kp) * kblocks + kb) * cout * 64;
          bulk_copy_g2s(b_base + static_cast<uint32_t>(s) * b_bytes, wsrc, b_bytes, bbar);
        }
      }
      if (!ok) {
        // aborting: give the bulk copies in flight a bounded chance to land before the CTA leaves
        for (int u = max(0, jb - nb); u < jb; ++u) {
          const uint32_t bar = smem_u32(&ctl->bfull[u % nb]);
          for (int spin = 0; spin < (1 << 20) && !mbar_try_wait(bar, (u / nb) & 1); ++spin) {
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == kMmaWarp) {
    // =========================== MMA issuer ===========================
    if (ls.settled) asm volatile("griddepcontrol.wait;" ::: "memory");
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (static_cast<uint32_t>(cout >> 3) << 17) | (static_cast<uint32_t>(kTileM >> 4) << 24);
      int jb = 0;
      int js[SUB];  // row items consumed so far, per sub-tile
#pragma unroll
      for (int sub = 0; sub < SUB; ++sub) js[sub] = 0;
      bool ok = true;
      for (int t = t0; t < t1 && ok; ++t) {
        const int it = t - t0;
        const int set = it % nsets;
        const uint32_t acc_par = static_cast<uint32_t>((it / nsets) - 1) & 1u;  // phase of the previous use's release
        uint32_t touched = 0u;
        const int ga = __ldg(ls.tile_ptr + t), gb = __ldg(ls.tile_ptr + t + 1);
        for (int g = ga; g < gb && ok; ++g) {
          int kp;
          uint32_t present;
          decode_stage<SUB>(__ldg(ls.stage_kp + g), kp, present);
          const bool second = kp == -1;
          const int nkb = second ? kblocks2 : kblocks;
          if (present == 0u) continue;
          for (int kb = 0; kb < nkb && ok; ++kb, ++jb) {
            const int bs = jb % nb;
            ok = mbar_wait(smem_u32(&ctl->bfull[bs]), (jb / nb) & 1, ctl, 3 | (it << 8), jb);
            if (!ok) break;
            const uint64_t db = make_desc(b_base + static_cast<uint32_t>(bs) * b_bytes);
            const int ksteps = min(4, ((second ? sec.cin2 : cin) - kb * 64) >> 4);
#pragma unroll
            for (int sub = 0; sub < SUB; ++sub) {
              if (!((present >> sub) & 1u)) continue;
              const int acc = set * SUB + sub;
              if (!((touched >> sub) & 1u) && it >= nsets) {
                // first product into this accumulator: its previous contents must have been drained
                ok = mbar_wait(smem_u32(&ctl->accempty[acc]), acc_par, ctl, 4 | (sub << 4) | (it << 8), js[sub]);
                if (!ok) break;
              }
              const int as = sub * na + js[sub] % na;
              ok = mbar_wait(smem_u32(&ctl->afull[as]), (js[sub] / na) & 1, ctl, 5 | (sub << 4) | (it << 8), js[sub]);
              if (!ok) break;
              fence_proxy_async();  // the gathered rows were written through the generic proxy
              tc_fence_after();
              const uint64_t da = make_desc(a_base + static_cast<uint32_t>(as) * kABytes);
              const uint32_t tmem_acc = tmem_base + static_cast<uint32_t>(acc * cout);
              for (int k = 0; k < ksteps; ++k)
                tc_mma_f16(tmem_acc, da + static_cast<uint64_t>(k * 2), db + static_cast<uint64_t>(k * 2), idesc,
                           (((touched >> sub) & 1u) || k > 0) ? 1u : 0u);
              touched |= 1u << sub;
              tc_commit(smem_u32(&ctl->aempty[as]));
              ++js[sub];
            }
            if (!ok) break;
            tc_commit(smem_u32(&ctl->bempty[bs]));
          }
        }
        if (!ok) break;
#pragma unroll
        for (int sub = 0; sub < SUB; ++sub) {
          const int acc = set * SUB + sub;
          if ((touched >> sub) & 1u) {
            tc_commit(smem_u32(&ctl->accfull[acc]));  // arrives when every product issued so far has finished
          } else {
            // nothing went into this accumulator: the epilogue writes zeros.  The signal may still not
            // run two phases ahead of the epilogue, so the previous use's release is waited for here too.
            if (it >= nsets) ok = mbar_wait(smem_u32(&ctl->accempty[acc]), acc_par, ctl, 6 | (sub << 4) | (it << 8), jb);
            if (!ok) break;
            mbar_arrive(smem_u32(&ctl->accfull[acc]));
          }
        }
      }
    }
    __syncwarp();
    tc_fence_before();
  } else {
    // =========================== epilogue ===========================
    const int e = warp - (kProd + 2);
    const int team = e >> 2;
    const int lane_quarter = warp & 3;  // the TMEM lanes this warp may read: 32*(warp%4)..+31
    const int slot_in_sub = lane_quarter * 32 + lane;
    if (ls.settled) asm volatile("griddepcontrol.wait;" ::: "memory");
    bool ok = true;
    for (int t = t0; t < t1 && ok; ++t) {
      const int it = t - t0;
      const int set = it % nsets;
      // which accumulators of this super-tile received products: OR of the stages' presence masks
      uint32_t any_mask = 0u;
      {
        const int ga = __ldg(ls.tile_ptr + t), gb = __ldg(ls.tile_ptr + t + 1);
        for (int g = ga + lane; g < gb; g += 32) {
          int kp;
          uint32_t present;
          decode_stage<SUB>(__ldg(ls.stage_kp + g), kp, present);
          if (kp == -1 && kblocks2 == 0) present = 0u;  // identity stage listed, but no second operand in this launch
          any_mask |= present;
        }
        any_mask = __reduce_or_sync(0xFFFFFFFFu, any_mask);
      }
      if (t == t1 - 1) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
      for (int sub = team; sub < SUB && ok; sub += EPIW) {
        const int acc = set * SUB + sub;
        const int slot = t * kRows + sub * kTileM + slot_in_sub;
        int my_row = n_out;
        if (slot < n_out) my_row = ls.order ? __ldg(ls.order + slot) : slot;
        const bool store_row = my_row < n_out;
        const bool any = (any_mask >> sub) & 1u;
        if (ep.residual && store_row) {
          const char* rp = reinterpret_cast<const char*>(ep.residual + static_cast<size_t>(my_row) * cout);
          for (int off = 0; off < cout * 2; off += 64) asm volatile("prefetch.global.L2 [%0];" ::"l"(rp + off));
        }
        ok = mbar_wait(smem_u32(&ctl->accfull[acc]), (it / nsets) & 1, ctl, 7 | (sub << 4) | (it << 8), t);
        ok = __all_sync(0xFFFFFFFFu, ok);
        if (!ok) break;
        tc_fence_after();
        const uint32_t taddr = tmem_base + static_cast<uint32_t>(acc * cout) + (static_cast<uint32_t>(lane_quarter * 32) << 16);
        __half* orow = out + static_cast<size_t>(store_row ? my_row : 0) * ep.ld_out;
        const __half* rrow = (ep.residual && store_row) ? ep.residual + static_cast<size_t>(my_row) * cout : nullptr;
        for (int c0 = 0; c0 < cout; c0 += 16) {
          uint4 ra = make_uint4(0u, 0u, 0u, 0u), rb = ra;
          if (rrow) {  // issued ahead of the tensor-memory load, consumed after it
            ra = *reinterpret_cast<const uint4*>(rrow + c0);
            rb = *reinterpret_cast<const uint4*>(rrow + c0 + 8);
          }
          uint32_t r[16];
          if (any) {  // warp-uniform: the tensor-memory load is warp-collective
            tmem_ld16(taddr + c0, r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int q = 0; q < 16; ++q) r[q] = 0u;
          }
          float v[16];
#pragma unroll
          for (int q = 0; q < 16; ++q) v[q] = __uint_as_float(r[q]);
          if (ep.scale || ep.shift) {  // one fused multiply-add per value, as in k_conv_umma (bit-identical results)
#pragma unroll
            for (int q = 0; q < 16; q += 4) {
              const float4 s4 = ep.scale ? __ldg(reinterpret_cast<const float4*>(ep.scale + c0 + q)) : make_float4(1.f, 1.f, 1.f, 1.f);
              const float4 t4 = ep.shift ? __ldg(reinterpret_cast<const float4*>(ep.shift + c0 + q)) : make_float4(0.f, 0.f, 0.f, 0.f);
              v[q] = fmaf(v[q], s4.x, t4.x);
              v[q + 1] = fmaf(v[q + 1], s4.y, t4.y);
              v[q + 2] = fmaf(v[q + 2], s4.z, t4.z);
              v[q + 3] = fmaf(v[q + 3], s4.w, t4.w);
            }
          }
          if (rrow) {
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
        mbar_arrive(smem_u32(&ctl->accempty[acc]));  // 128 arrivals hand the accumulator back
      }
    }
    tc_fence_before();
  }
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(static_cast<uint32_t>(tmem_cols))
                 : "memory");
  }
}

// Second kernel of a split layer: out[row] = act((sum over parts of partial[part][row]) * scale + shift +
// residual), parts added in ascending order in fp32; one thread per 8 output channels.
__global__ void __launch_bounds__(256)
    k_sum_parts(const float* __restrict__ partial, int parts, int n_out, int cout, __half* __restrict__ out, Epi ep) {
  asm volatile("griddepcontrol.wait;" ::: "memory");  // launched while the convolution kernel drains
  const int chunks = cout >> 3;
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<long long>(n_out) * chunks) return;
  const int row = static_cast<int>(i / chunks), c0 = static_cast<int>(i % chunks) * 8;
  float v[8];
#pragma unroll
  for (int q = 0; q < 8; ++q) v[q] = 0.f;
  for (int p = 0; p < parts; ++p) {
    const float4* src = reinterpret_cast<const float4*>(partial + (static_cast<size_t>(p) * n_out + row) * cout + c0);
    const float4 a = __ldg(src), b = __ldg(src + 1);
    v[0] += a.x; v[1] += a.y; v[2] += a.z; v[3] += a.w;
    v[4] += b.x; v[5] += b.y; v[6] += b.z; v[7] += b.w;
  }
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    if (ep.scale || ep.shift)
      v[q] = fmaf(v[q], ep.scale ? __ldg(ep.scale + c0 + q) : 1.f, ep.shift ? __ldg(ep.shift + c0 + q) : 0.f);
  }
  if (ep.residual) {
    const uint4 r = *reinterpret_cast<const uint4*>(ep.residual + static_cast<size_t>(row) * cout + c0);
    const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 f = __half22float2(h[q]);
      v[2 * q] += f.x;
      v[2 * q + 1] += f.y;
    }
  }
  uint4 o;
  __half2* po = reinterpret_cast<__half2*>(&o);
#pragma unroll
  for (int q = 0; q < 4; ++q)
    po[q] = __floats2half2_rn(act_apply(v[2 * q], ep.act, ep.slope), act_apply(v[2 * q + 1], ep.act, ep.slope));
  *reinterpret_cast<uint4*>(out + static_cast<size_t>(row) * ep.ld_out + c0) = o;
}

// Second kernel of a stream-K layer: for every tile that was cut between CTAs, adds the pieces in CTA order
// (fp32) and applies the epilogue; tiles that one CTA finished are left alone.  Block (x, t) handles 256 of the
// tile's (row, 8 output channels) items: its first warp works out which CTAs hold pieces of tile t (consecutive
// CTAs, one per lane, 32 per round; the divisions are done once per block, not per item), then every thread sums
// its item over them.  `ctas` = the grid of the convolution launch.
__global__ void __launch_bounds__(256)
    k_sum_cut_tiles(const float* __restrict__ partial, const int* __restrict__ tile_ptr, const int* __restrict__ order,
                    int n_tiles, int ctas, int n_out, int cout, __half* __restrict__ out, Epi ep) {
  __shared__ int s_slot[32];  // per CTA of the round: 2*b + which, or -1 (its share misses the tile)
  __shared__ int s_whole;     // some CTA held the whole tile: nothing to do
  asm volatile("griddepcontrol.wait;" ::: "memory");  // launched while the convolution kernel drains
  const int t = blockIdx.y;
  const int a = __ldg(tile_ptr + t), e = __ldg(tile_ptr + t + 1);
  const long long total = __ldg(tile_ptr + n_tiles);
  const int chunks = cout >> 3;
  const int item = static_cast<int>(blockIdx.x) * 256 + static_cast<int>(threadIdx.x);
  const bool live = item < kTileM * chunks;
  const int r = live ? item / chunks : 0, c0 = live ? (item % chunks) * 8 : 0;
  // CTAs that can hold stages of [a, e): b with share_begin(b) < e and share_begin(b + 1) > a
  int b0 = 0, b1 = -1;
  if (e > a && total > 0) {
    b0 = static_cast<int>(static_cast<long long>(a) * ctas / total) - 1;
    b1 = static_cast<int>(static_cast<long long>(e) * ctas / total) + 1;
    b0 = b0 < 0 ? 0 : b0;
    b1 = b1 > ctas - 1 ? ctas - 1 : b1;
  }
  if (threadIdx.x == 0) s_whole = 0;
  float v[8];
#pragma unroll
  for (int q = 0; q < 8; ++q) v[q] = 0.f;
  for (int base = b0; base <= b1; base += 32) {
    __syncthreads();
    if (threadIdx.x < 32) {
      const int b = base + static_cast<int>(threadIdx.x);
      int slot = -1;
      if (b <= b1) {
        const int sb = share_begin(total, b, ctas), se = share_begin(total, b + 1, ctas);
        if ((sb > a ? sb : a) < (se < e ? se : e)) {
          if (sb <= a && se >= e) s_whole = 1;
          slot = 2 * b + (sb >= a ? 0 : 1);  // the tile is the CTA's first tile when its share starts inside it
        }
      }
      s_slot[threadIdx.x] = slot;
    }
    __syncthreads();
    if (s_whole) return;
    if (live) {
      for (int k = 0; k < 32; ++k) {
        const int slot = s_slot[k];
        if (slot < 0) continue;
        const float4* src = reinterpret_cast<const float4*>(partial + (static_cast<size_t>(slot) * kTileM + r) * cout + c0);
        const float4 x = __ldg(src), y = __ldg(src + 1);
        v[0] += x.x; v[1] += x.y; v[2] += x.z; v[3] += x.w;
        v[4] += y.x; v[5] += y.y; v[6] += y.z; v[7] += y.w;
      }
    }
  }
  // (a tile without stages belongs to no share: its rows get the epilogue of zero here)
  const int slot_row = t * kTileM + r;
  if (!live || slot_row >= n_out) return;
  const int row = order ? __ldg(order + slot_row) : slot_row;
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    if (ep.scale || ep.shift)
      v[q] = fmaf(v[q], ep.scale ? __ldg(ep.scale + c0 + q) : 1.f, ep.shift ? __ldg(ep.shift + c0 + q) : 0.f);
  }
  if (ep.residual) {
    const uint4 rr = *reinterpret_cast<const uint4*>(ep.residual + static_cast<size_t>(row) * cout + c0);
    const __half2* h = reinterpret_cast<const __half2*>(&rr);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 f = __half22float2(h[q]);
      v[2 * q] += f.x;
      v[2 * q + 1] += f.y;
    }
  }
  uint4 o;
  __half2* po = reinterpret_cast<__half2*>(&o);
#pragma unroll
  for (int q = 0; q < 4; ++q)
    po[q] = __floats2half2_rn(act_apply(v[2 * q], ep.act, ep.slope), act_apply(v[2 * q + 1], ep.act, ep.slope));
  *reinterpret_cast<uint4*>(out + static_cast<size_t>(row) * ep.ld_out + c0) = o;
}

}  // namespace umma

bool conv_umma_supported(int cin, int cout, int dtype) {
  return dtype == PCE_F16 && cin >= 16 && cin % 16 == 0 && cout >= 16 && cout % 16 == 0 && cout <= 256;
}

// Per-offset blocks, and for 16 or 32 input channels also the per-offset [cout][cin] images from which
// stages that hold several offsets assemble their weight block.
// Behind them, a second copy as 32-channel blocks (cout rows x 64 B, 64-byte swizzle) for widths that are an odd
// multiple of 32 (the kernel variant with 32-channel K blocks) and for every single-offset weight (a second
// operand is read in the K-block size of the layer it joins).
static bool has_kb32_image(int kv, int cin) { return kv == 1 || (cin > 32 && cin % 64 == 32); }
static size_t kb64_image_bytes(int kv, int cin, int cout) {
  const size_t blocks = static_cast<size_t>(kv) * ((cin + 63) / 64) * cout * 128;
  return blocks + ((cin == 16 || cin == 32) ? static_cast<size_t>(kv) * cout * cin * 2 : 0);
}
size_t umma_packed_bytes(int kv, int cin, int cout) {
  const size_t kb32 = has_kb32_image(kv, cin) ? static_cast<size_t>(kv) * ((cin + 31) / 32) * cout * 64 : 0;
  return kb64_image_bytes(kv, cin, cout) + kb32;
}

int umma_pack_weights(const void* w, int kv, int cin, int cout, void* packed, cudaStream_t st) {
  const int kblocks = (cin + 63) / 64;
  const long long total = static_cast<long long>(kv) * kblocks * cout * 64;
  const int grid = static_cast<int>(std::min<long long>((total + 255) / 256, 148ll * 8));
  umma::k_pack_weights<<<grid, 256, 0, st>>>(static_cast<const __half*>(w), kv, cin, cout, kblocks,
                                             static_cast<__half*>(packed), 64);
  PCE_LAUNCH_CHECK();
  if (has_kb32_image(kv, cin)) {
    const int kblocks32 = (cin + 31) / 32;
    const long long total32 = static_cast<long long>(kv) * kblocks32 * cout * 32;
    umma::k_pack_weights<<<static_cast<int>(std::min<long long>((total32 + 255) / 256, 148ll * 8)), 256, 0, st>>>(
        static_cast<const __half*>(w), kv, cin, cout, kblocks32,
        reinterpret_cast<__half*>(static_cast<char*>(packed) + kb64_image_bytes(kv, cin, cout)), 32);
    PCE_LAUNCH_CHECK();
  }
  if (cin == 16 || cin == 32) {
    const long long n = static_cast<long long>(kv) * cout * cin;
    umma::k_pack_weight_slots<<<static_cast<int>(std::min<long long>((n + 255) / 256, 148ll * 8)), 256, 0, st>>>(
        static_cast<const __half*>(w), kv, cin, cout, static_cast<__half*>(packed) + total);
    PCE_LAUNCH_CHECK();
  }
  return PCE_OK;
}

// Tuning hooks (tests / experiments): 0 = choose; stages 2..4; sub-tiles 1 or 2; accumulator sets 1 or 2.
int umma_force_stages = 0;
int umma_force_sub = 0;
int umma_force_nacc = 0;
// Programmatic dependent launch: the kernel's set-up (barriers, tensor-memory allocation; with settled
// tile lists also the tile search and the first index loads) overlaps the tail of the kernel before it
// in the stream.  0 = off, 1 = on, 2 = on but every list is treated as not settled.
int umma_overlap_launches = 1;
// 1: layers with one offset per stage and no halo push run k_conv_umma_mt (several accumulators per CTA,
// decoupled row and weight rings); 0 (default): k_conv_umma, which measured faster at every tile height
// both kernels share (512-row tiles exist for k_conv_umma_mt only and always run on it).
int umma_multi_tile = 0;

template <int SUB, int EPIW>
static void launch_umma_mt(int grid, size_t smem, cudaStream_t st, const __half* in, const __half* w, const umma::Lists& ls,
                           const umma::Second& sec, int n_out, int cin, int cout, __half* out, const umma::Epi& e,
                           int tmem_cols, int na, int nb, int nsets) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(32 * (4 * SUB + 2 + 4 * EPIW));
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = umma_overlap_launches ? 1 : 0;
  cudaLaunchKernelEx(&cfg, umma::k_conv_umma_mt<SUB, EPIW>, in, w, ls, sec, n_out, cin, cout, out, e, tmem_cols, na, nb, nsets);
}

// Configuration of k_conv_umma_mt for a layer: sub-tiles per super-tile come with the lists; accumulator
// sets, CTAs per SM and the two ring depths follow from tensor memory (512 columns per SM) and shared memory.
static int conv_umma_mt(const __half* in, const __half* w, const umma::Lists& ls, const umma::Second& sec, int n_out, int cin,
                        int cout, __half* out, const umma::Epi& e, int sub, int sm_count, cudaStream_t st) {
  if (sub != 1 && sub != 2 && sub != 4) return PCE_ERR_INVALID;
  if (sub * cout > 512) return PCE_ERR_UNSUPPORTED;
  static bool attr_set[64] = {};
  int dev = 0;
  PCE_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return PCE_ERR_UNSUPPORTED;
  if (!attr_set[dev]) {
    const int cap = 227 * 1024;
    PCE_CUDA(cudaFuncSetAttribute(umma::k_conv_umma_mt<1, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, cap));
    PCE_CUDA(cudaFuncSetAttribute(umma::k_conv_umma_mt<2, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, cap));
    PCE_CUDA(cudaFuncSetAttribute(umma::k_conv_umma_mt<4, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, cap));
    attr_set[dev] = true;
  }
  // two CTAs per SM only for single sub-tiles with narrow accumulators (two sets of <= 128 columns each)
  const int ctas = (sub == 1 && 2 * cout <= 256) ? 2 : 1;
  int nsets = (2 * sub * cout * ctas <= 512) ? 2 : 1;
  if ((umma_force_nacc == 1 || umma_force_nacc == 2) && umma_force_nacc * sub * cout * ctas <= 512) nsets = umma_force_nacc;
  int tmem_cols = 32;
  while (tmem_cols < nsets * sub * cout) tmem_cols <<= 1;
  const size_t fixed = sizeof(umma::SharedCtlMt) + 1024 + 64;
  const size_t budget = static_cast<size_t>(227 * 1024) / ctas - fixed - (ctas > 1 ? 1024 : 0);
  const size_t b_bytes = static_cast<size_t>(cout) * 128;
  int nb = 3 * b_bytes * 3 <= budget ? 3 : 2;
  if (2 * b_bytes + 2 * umma::kABytes > budget) return PCE_ERR_UNSUPPORTED;
  // row slots per sub-tile; a third weight slot only where it does not cost a row slot per sub-tile
  int na = static_cast<int>((budget - nb * b_bytes) / umma::kABytes) / sub;
  if (nb == 3 && static_cast<int>((budget - 2 * b_bytes) / umma::kABytes) / sub > na) {
    nb = 2;
    na = static_cast<int>((budget - nb * b_bytes) / umma::kABytes) / sub;
  }
  if (na * sub > umma::kMaxA) na = umma::kMaxA / sub;
  if (umma_force_stages >= 2 && umma_force_stages <= na) na = umma_force_stages;
  if (na < 2) return PCE_ERR_UNSUPPORTED;
  const size_t smem = static_cast<size_t>(na) * sub * umma::kABytes + nb * b_bytes + fixed;
  const int n_tiles = div_up(n_out, umma::kTileM * sub);
  const int grid = n_tiles < sm_count * ctas ? n_tiles : sm_count * ctas;
  if (sub == 1)
    launch_umma_mt<1, 1>(grid, smem, st, in, w, ls, sec, n_out, cin, cout, out, e, tmem_cols, na, nb, nsets);
  else if (sub == 2)
    launch_umma_mt<2, 1>(grid, smem, st, in, w, ls, sec, n_out, cin, cout, out, e, tmem_cols, na, nb, nsets);
  else
    launch_umma_mt<4, 2>(grid, smem, st, in, w, ls, sec, n_out, cin, cout, out, e, tmem_cols, na, nb, nsets);
  PCE_LAUNCH_CHECK();
  return PCE_OK;
}

template <int NS, int SUB, bool PUSH, int SLOTS, int KB = 64>
static void launch_umma(int grid, size_t smem, cudaStream_t st, const __half* in, const __half* w, const umma::Lists& ls,
                        const umma::Second& sec, int n_out, int cin, int cout, __half* out, const umma::Epi& e, int tmem_cols,
                        int nacc) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(32 * (4 * SUB + 5));
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = umma_overlap_launches ? 1 : 0;
  cudaLaunchKernelEx(&cfg, umma::k_conv_umma<NS, SUB, PUSH, SLOTS, KB>, in, w, ls, sec, n_out, cin, cout, out, e, tmem_cols,
                     nacc);
}

// 1: layers whose width is an odd multiple of 32 channels (96, 160, 224) run with 32-channel K blocks, where every
// ring stage is full (64-channel blocks pad half of every second stage); 0: 64-channel blocks everywhere.
int umma_kb32_enabled = 1;

// 1: maps with few tiles are split over several CTAs per tile, mid-size maps into equal shares of stages,
// when the caller gives scratch (see conv_split_parts, conv_streamk_grid); 2: only the former; 0: never.
int umma_split_enabled = 1;

// Parts per tile for a layer of n_rows outputs: 8, 4 or 2 CTAs per tile where all of them are resident at
// once (tiles x parts <= the SMs' CTA slots) and every part keeps a chain of at least 8 stages.  The chain of
// a tile is estimated as min(kv, 16) offsets x K blocks: deep levels of a network, where maps are small, are
// also where tiles have many offsets.  Measured on B200 (LiDAR scans, kernel-only): 256 -> 256 on 27 tiles
// 104 -> 42 us with 8 parts, on 68 tiles 100 -> 54 us with 4, on 132 tiles 102 -> 77 us with 2; 384 -> 256 on
// 132 tiles 144 -> 99 us; more parts than slots do not pay for the second kernel and the fp32 round trip
// (189 tiles, 128 -> 256, two parts on 296 slots: 63 -> 74 us), so such maps stay unsplit.  Layers with 16 or
// 32 input channels (shallow levels) are never split.
// Estimated ring stages per tile: min(kv, 16) offsets x K blocks, fewer where the map has fewer source rows than
// output rows (a transposed 2x2x2 layer has ONE pair per output row: its tiles list up to 8 offsets, each nearly
// empty, and splitting them only adds the partial sums; measured 16 -> 30 us on 159 tiles of 128 -> 128).
static int chain_estimate(int n_rows, int n_src, int cin, int kv) {
  long long offsets = kv < 16 ? kv : 16;
  if (n_src < n_rows) {
    const long long per_row = static_cast<long long>(kv) * n_src / n_rows;
    offsets = per_row < offsets ? (per_row > 1 ? per_row : 1) : offsets;
  }
  return static_cast<int>(offsets) * ((cin + 63) / 64);
}

int conv_split_parts(int n_rows, int n_src, int cin, int cout, int kv, int sm_count) {
  if (!umma_split_enabled || n_rows < 1) return 1;
  const int cin_p = (cin + 15) / 16 * 16;
  if (cin_p == 16 || cin_p == 32) return 1;
  const int chain = chain_estimate(n_rows, n_src, cin, kv);
  const long long n_tiles = (static_cast<long long>(n_rows) + umma::kTileM - 1) / umma::kTileM;
  const long long slots = static_cast<long long>(sm_count > 0 ? sm_count : 148) * (cout <= 128 ? 3 : 2);
  int p = 8;
  while (p > 1 && (n_tiles * p > slots || chain < 8 * p)) p >>= 1;
  return p;
}

// Maps of half a wave to one wave of tiles (tiles / CTA slots in (0.5, 1]) that conv_split_parts leaves
// whole: CTAs take equal shares of the STAGES instead of whole tiles (stream-K), wherever the cuts fall, so
// every CTA slot works for the same time instead of some running a whole chain while others idle.  A tile
// that two or more CTAs worked on costs fp32 partial sums (written, then read by k_sum_cut_tiles), which is
// why it pays only for long chains on less than one wave.  Measured on B200 (LiDAR scans, kernel-only, us,
// whole -> shares): 256->256 on 189 tiles 111 -> 82, on 273 tiles 111 -> 97, 384->256 on 273 tiles 156 -> 114;
// but 256->256 on 489 tiles (1.65 waves) 119 -> 136, 128->128 on 273 tiles 59 -> 58, and the 2x2x2
// strided / transposed layers (chains of 8 offsets at most) 35-49 -> 56-65: those run whole.
// Returns the grid (= the CTA slots) or 0.
int conv_streamk_grid(int n_rows, int n_src, int cin, int cout, int kv, int sm_count) {
  if (!umma_split_enabled || umma_split_enabled == 2 || n_rows < 1) return 0;
  const int cin_p = (cin + 15) / 16 * 16;
  if (cin_p == 16 || cin_p == 32) return 0;
  if (conv_split_parts(n_rows, n_src, cin, cout, kv, sm_count) > 1) return 0;
  const int chain = chain_estimate(n_rows, n_src, cin, kv);
  const long long n_tiles = (static_cast<long long>(n_rows) + umma::kTileM - 1) / umma::kTileM;
  const long long slots = static_cast<long long>(sm_count > 0 ? sm_count : 148) * (cout <= 128 ? 3 : 2);
  if (umma_split_enabled == 3) return (chain >= 8 && 2 * n_tiles > slots && n_tiles <= 4 * slots) ? static_cast<int>(slots) : 0;
  if (kv <= 8 || chain < 16 || 2 * n_tiles <= slots || n_tiles > slots) return 0;
  return static_cast<int>(slots);
}

// Scratch (bytes of fp32 partial sums) that lets a layer be split, 0 when it runs whole.
size_t conv_split_scratch_bytes(int n_rows, int n_src, int cin, int cout, int kv, int sm_count) {
  const int parts = conv_split_parts(n_rows, n_src, cin, cout, kv, sm_count);
  if (parts > 1) return static_cast<size_t>(parts) * n_rows * cout * sizeof(float);
  const int grid = conv_streamk_grid(n_rows, n_src, cin, cout, kv, sm_count);
  return grid > 0 ? static_cast<size_t>(grid) * 2 * umma::kTileM * cout * sizeof(float) : 0;
}

// tiles == nullptr: the dense rows x matrix product (every row fetches itself, one offset).
static int conv_umma_impl(const void* in, int n_in, const void* wpacked, int kv, const pce_tile_lists* tiles, int n_out,
                          int cin, int cout, void* out, const pce_epilogue* ep, cudaStream_t st, bool kb64_slice);

int conv_umma(const void* in, int n_in, const void* wpacked, int kv, const pce_tile_lists* tiles, int n_out, int cin,
              int cout, void* out, const pce_epilogue* ep, cudaStream_t st) {
  return conv_umma_impl(in, n_in, wpacked, kv, tiles, n_out, cin, cout, out, ep, st, false);
}

// The same for weights that are a SLICE of a larger packed buffer (one offset's 64-channel blocks): there is no
// second image behind them, so the layer runs with 64-channel K blocks whatever its width.
int conv_umma_kb64(const void* in, int n_in, const void* wpacked, int kv, const pce_tile_lists* tiles, int n_out, int cin,
                   int cout, void* out, const pce_epilogue* ep, cudaStream_t st) {
  return conv_umma_impl(in, n_in, wpacked, kv, tiles, n_out, cin, cout, out, ep, st, true);
}

static int conv_umma_impl(const void* in, int n_in, const void* wpacked, int kv, const pce_tile_lists* tiles, int n_out,
                          int cin, int cout, void* out, const pce_epilogue* ep, cudaStream_t st, bool kb64_slice) {
  umma::Epi e{nullptr, nullptr, nullptr, PCE_ACT_NONE, 0.f, {nullptr, nullptr}, {nullptr, nullptr}, cin, cout};
  if (ep) {
    e = umma::Epi{ep->scale, ep->shift, static_cast<const __half*>(ep->residual), ep->act, ep->slope,
                  {ep->push_slot[0], ep->push_slot[1]},
                  {static_cast<__half*>(ep->push_base[0]), static_cast<__half*>(ep->push_base[1])},
                  ep->in_ld > 0 ? ep->in_ld : cin, ep->out_ld > 0 ? ep->out_ld : cout};
    // rows stay 16-byte aligned: the pitch is a multiple of 8 halves and covers the channels
    if (e.ld_in < cin || e.ld_out < cout || (e.ld_in & 7) || (e.ld_out & 7)) return PCE_ERR_INVALID;
    for (int s = 0; s < 2; ++s) {
      if (e.push_slot[s] && (!e.push_base[s] || (reinterpret_cast<uintptr_t>(e.push_base[s]) & 15))) return PCE_ERR_INVALID;
      if (!e.push_slot[s]) e.push_base[s] = nullptr;
    }
  }
  umma::Lists ls{nullptr, nullptr, nullptr, nullptr, 0, nullptr, 0};
  int slots = 1;
  umma::Second sec{nullptr, nullptr, 0};
  int sub = umma_force_sub == 1 || umma_force_sub == 2 ? umma_force_sub : 1;
  if (tiles) {
    ls = umma::Lists{tiles->order, tiles->tile_ptr, tiles->stage_kp, tiles->stage_nbr, tiles->identity_stage ? 1 : 0, nullptr,
                     (tiles->settled && umma_overlap_launches == 1) ? 1 : 0};
    slots = tiles->slots > 1 ? tiles->slots : 1;
    if (slots != 1) {
      // several offsets per stage: the lists must match the layer's width, and the packed weights carry
      // the per-offset [cout][cin] images behind the per-offset blocks
      if ((slots != 2 && slots != 4) || cin * slots != 64) return PCE_ERR_INVALID;
      ls.wslots = static_cast<const __half*>(wpacked) + static_cast<size_t>(kv) * cout * 64;
    }
    if (tiles->tile_rows != 128 && tiles->tile_rows != 256 && tiles->tile_rows != 512) return PCE_ERR_INVALID;
    sub = tiles->tile_rows / 128;  // the lists fix the tile height
  }
  if (sub * cout > 512) return PCE_ERR_UNSUPPORTED;
  if (sub > 2 && (slots != 1 || !tiles)) return PCE_ERR_UNSUPPORTED;
  if (ep && ep->extra_feats) {
    // the second operand rides on the identity stage of the tile lists
    if (!ls.identity || !ep->extra_packed_weights || ep->extra_c < 16 || ep->extra_c % 16) return PCE_ERR_UNSUPPORTED;
    sec = umma::Second{static_cast<const __half*>(ep->extra_feats), static_cast<const __half*>(ep->extra_packed_weights),
                       ep->extra_c};
  }
  const size_t fixed = sizeof(umma::SharedCtl) + 1024 + 64 + 2 * sizeof(float) * cout;  // (+ staged scale / shift)
  // 32-channel K blocks for widths that are an odd multiple of 32 (plain variant: one sub-tile, one offset per
  // stage, no halo push); operands then come from the second image of the packed weights
  const bool kb32 = umma_kb32_enabled && !kb64_slice && sub == 1 && slots == 1 && !(e.push_slot[0] || e.push_slot[1]) && cin > 32 &&
                    cin % 64 == 32 && !(tiles && umma_multi_tile);
  const size_t stage = kb32 ? static_cast<size_t>(umma::kTileM) * 64 + static_cast<size_t>(cout) * 64
                            : static_cast<size_t>(umma::kABytes) * sub + static_cast<size_t>(cout) * 128;
  static int sm_count[64] = {};
  // registers per thread by kernel variant (plain, push, 2 slots, 4 slots) and sub-tile count, in
  // allocation units of 8; read back from the compiled kernels at set-up
  static int regs_per_thread[4][2] = {{72, 72}, {80, 80}, {80, 80}, {96, 88}};
  static int regs_kb32 = 72;
  int dev = 0;
  PCE_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return PCE_ERR_UNSUPPORTED;
  if (sm_count[dev] == 0) {
    const int cap = 227 * 1024;
#define PCE_SET_SMEM(NS, SB) \
  PCE_CUDA(cudaFuncSetAttribute(umma::k_conv_umma<NS, SB, false, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, cap)); \
  PCE_CUDA(cudaFuncSetAttribute(umma::k_conv_umma<NS, SB, true, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, cap));  \
  PCE_CUDA(cudaFuncSetAttribute(umma::k_conv_umma<NS, SB, false, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, cap)); \
  PCE_CUDA(cudaFuncSetAttribute(umma::k_conv_umma<NS, SB, false, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, cap))
    PCE_CUDA(cudaFuncSetAttribute(umma::k_conv_umma<4, 1, false, 1, 32>, cudaFuncAttributeMaxDynamicSharedMemorySize, cap));
    PCE_CUDA(cudaFuncSetAttribute(umma::k_conv_umma<5, 1, false, 1, 32>, cudaFuncAttributeMaxDynamicSharedMemorySize, cap));
    PCE_CUDA(cudaFuncSetAttribute(umma::k_conv_umma<6, 1, false, 1, 32>, cudaFuncAttributeMaxDynamicSharedMemorySize, cap));
    PCE_SET_SMEM(4, 1);
    PCE_SET_SMEM(3, 1);
    PCE_SET_SMEM(2, 1);
    PCE_SET_SMEM(4, 2);
    PCE_SET_SMEM(3, 2);
    PCE_SET_SMEM(2, 2);
#undef PCE_SET_SMEM
    cudaFuncAttributes fa;
#define PCE_REGS(V, SB, KERNEL) \
  if (cudaFuncGetAttributes(&fa, KERNEL) == cudaSuccess && fa.numRegs > 0) regs_per_thread[V][SB - 1] = (fa.numRegs + 7) / 8 * 8
    PCE_REGS(0, 1, (umma::k_conv_umma<2, 1, false, 1>));
    PCE_REGS(0, 2, (umma::k_conv_umma<2, 2, false, 1>));
    PCE_REGS(1, 1, (umma::k_conv_umma<2, 1, true, 1>));
    PCE_REGS(1, 2, (umma::k_conv_umma<2, 2, true, 1>));
    PCE_REGS(2, 1, (umma::k_conv_umma<2, 1, false, 2>));
    PCE_REGS(2, 2, (umma::k_conv_umma<2, 2, false, 2>));
    PCE_REGS(3, 1, (umma::k_conv_umma<2, 1, false, 4>));
    PCE_REGS(3, 2, (umma::k_conv_umma<2, 2, false, 4>));
#undef PCE_REGS
    if (cudaFuncGetAttributes(&fa, umma::k_conv_umma<4, 1, false, 1, 32>) == cudaSuccess && fa.numRegs > 0)
      regs_kb32 = (fa.numRegs + 7) / 8 * 8;
    int n = 0;
    PCE_CUDA(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
    sm_count[dev] = n > 0 ? n : 1;
  }
  {
    const bool push_any = e.push_slot[0] || e.push_slot[1];
    if (tiles && slots == 1 && !push_any && (umma_multi_tile || sub == 4))
      return conv_umma_mt(static_cast<const __half*>(in), static_cast<const __half*>(wpacked), ls, sec, n_out, cin, cout,
                          static_cast<__half*>(out), e, sub, sm_count[dev], st);
    if (sub > 2) return PCE_ERR_UNSUPPORTED;  // 512-row super-tiles exist for k_conv_umma_mt only
  }
  // Configuration = (ring depth, accumulator sets).  What the kernel needs most is row gathers in
  // flight, i.e. stages resident per SM = resident CTAs x ring depth; the CTAs per SM are bounded by
  // shared memory, by the 512 tensor-memory columns and by the register file.  Measured on LiDAR
  // layers (486k / 297k / 149k rows): at an equal stage count more CTAs win (C=96: 3 CTAs x 2 stages
  // with one accumulator set 146 us, 2 x 3 with two sets 159 us; C=128: 115 vs 122 us), and at equal
  // CTAs two accumulator sets win (the epilogue of a tile then overlaps the next tile's MMAs).
  const int threads = 32 * (4 * sub + 5);
  const bool push = e.push_slot[0] || e.push_slot[1];
  if (push && slots != 1) return PCE_ERR_UNSUPPORTED;  // the halo push has no several-offsets-per-stage variant
  const int variant = push ? 1 : (slots == 2 ? 2 : (slots == 4 ? 3 : 0));
  const int by_regs = 65536 / (threads * (kb32 ? regs_kb32 : regs_per_thread[variant][sub - 1]));
  auto tmem_for = [&](int sets) {
    int cols = 32;
    while (cols < sets * sub * cout) cols <<= 1;
    return cols;
  };
  auto ctas_for = [&](int n, int sets) {
    if (sets * sub * cout > 512) return 0;
    int c = static_cast<int>((227 * 1024) / (n * stage + fixed + 1024));
    if (c > 512 / tmem_for(sets)) c = 512 / tmem_for(sets);
    if (c > by_regs) c = by_regs;
    return c > 4 ? 4 : c;
  };
  int ns = 2, nacc = 1, per_sm = 0;
  for (int n = (kb32 ? 6 : 4); n >= (kb32 ? 4 : 2); --n) {  // (32-channel blocks: half-size stages, rings of 4 to 6)
    for (int sets = 2; sets >= 1; --sets) {
      const int c = ctas_for(n, sets);
      const bool better = c * n > per_sm * ns || (c * n == per_sm * ns && c > per_sm);
      if (c > 0 && (per_sm == 0 || better)) {
        ns = n;
        nacc = sets;
        per_sm = c;
      }
    }
  }
  if (umma_force_stages >= (kb32 ? 4 : 2) && umma_force_stages <= (kb32 ? 6 : 4)) ns = umma_force_stages;
  if ((umma_force_nacc == 1 || umma_force_nacc == 2) && umma_force_nacc * sub * cout <= 512) nacc = umma_force_nacc;
  per_sm = ctas_for(ns, nacc);
  const int tmem_cols = tmem_for(nacc);
  if (per_sm < 1) per_sm = 1;
  const size_t smem = ns * stage + fixed;
  if (smem > 227 * 1024) return PCE_ERR_UNSUPPORTED;
  const int n_tiles = div_up(n_out, umma::kTileM * sub);
  int grid = n_tiles < sm_count[dev] * per_sm ? n_tiles : sm_count[dev] * per_sm;
  // few tiles, long stage chains: several CTAs per tile, partial sums through the caller's scratch
  int parts = 1;
  bool streamk = false;
  if (tiles && sub == 1 && slots == 1 && !push && ep && ep->split_scratch &&
      (reinterpret_cast<uintptr_t>(ep->split_scratch) & 15) == 0) {
    parts = conv_split_parts(n_out, n_in, cin, cout, kv, sm_count[dev]);
    while (parts > 1 && static_cast<size_t>(parts) * n_out * cout * sizeof(float) > ep->split_scratch_bytes) parts >>= 1;
    if (parts > 1) {
      grid = n_tiles * parts;
      e.partial = static_cast<float*>(ep->split_scratch);
      e.parts = parts;
    } else {
      const int g = conv_streamk_grid(n_out, n_in, cin, cout, kv, sm_count[dev]);
      if (g > 0 && g <= sm_count[dev] * per_sm &&
          static_cast<size_t>(g) * 2 * umma::kTileM * cout * sizeof(float) <= ep->split_scratch_bytes) {
        grid = g;
        streamk = true;
        e.partial = static_cast<float*>(ep->split_scratch);
        e.streamk = 1;
      }
    }
  }
  const __half* in_h = static_cast<const __half*>(in);
  const __half* w_h = static_cast<const __half*>(wpacked);
  __half* out_h = static_cast<__half*>(out);
  if (kb32) {
    w_h = reinterpret_cast<const __half*>(static_cast<const char*>(wpacked) + kb64_image_bytes(kv, cin, cout));
    if (sec.in2)
      sec.w2 = reinterpret_cast<const __half*>(reinterpret_cast<const char*>(sec.w2) + kb64_image_bytes(1, sec.cin2, cout));
    if (ns == 6)
      launch_umma<6, 1, false, 1, 32>(grid, smem, st, in_h, w_h, ls, sec, n_out, cin, cout, out_h, e, tmem_cols, nacc);
    else if (ns == 5)
      launch_umma<5, 1, false, 1, 32>(grid, smem, st, in_h, w_h, ls, sec, n_out, cin, cout, out_h, e, tmem_cols, nacc);
    else
      launch_umma<4, 1, false, 1, 32>(grid, smem, st, in_h, w_h, ls, sec, n_out, cin, cout, out_h, e, tmem_cols, nacc);
  } else {
#define PCE_GO(NS, SB)                                                                                              \
  do {                                                                                                              \
    if (push)                                                                                                         \
      launch_umma<NS, SB, true, 1>(grid, smem, st, in_h, w_h, ls, sec, n_out, cin, cout, out_h, e, tmem_cols, nacc);  \
    else if (slots == 2)                                                                                              \
      launch_umma<NS, SB, false, 2>(grid, smem, st, in_h, w_h, ls, sec, n_out, cin, cout, out_h, e, tmem_cols, nacc); \
    else if (slots == 4)                                                                                              \
      launch_umma<NS, SB, false, 4>(grid, smem, st, in_h, w_h, ls, sec, n_out, cin, cout, out_h, e, tmem_cols, nacc); \
    else                                                                                                              \
      launch_umma<NS, SB, false, 1>(grid, smem, st, in_h, w_h, ls, sec, n_out, cin, cout, out_h, e, tmem_cols, nacc); \
  } while (0)
  if (sub == 1) {
    if (ns == 4) PCE_GO(4, 1); else if (ns == 3) PCE_GO(3, 1); else PCE_GO(2, 1);
  } else {
    if (ns == 4) PCE_GO(4, 2); else if (ns == 3) PCE_GO(3, 2); else PCE_GO(2, 2);
  }
#undef PCE_GO
  }
  PCE_LAUNCH_CHECK();
  if (parts > 1 || streamk) {
    // the second kernel of a split layer is set up on the SMs while the convolution's last CTAs drain
    // (programmatic dependent launch; it waits for that grid before it reads a partial sum)
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = umma_overlap_launches ? 1 : 0;
    const float* partial = e.partial;
    if (parts > 1) {
      cfg.gridDim = dim3(div_up(static_cast<long long>(n_out) * (cout >> 3), 256));
      cudaLaunchKernelEx(&cfg, umma::k_sum_parts, partial, parts, n_out, cout, out_h, e);
    } else {
      cfg.gridDim = dim3(div_up(umma::kTileM * (cout >> 3), 256), n_tiles);
      const int* tile_ptr = ls.tile_ptr;
      const int* order = ls.order;
      cudaLaunchKernelEx(&cfg, umma::k_sum_cut_tiles, partial, tile_ptr, order, n_tiles, grid, n_out, cout, out_h, e);
    }
    PCE_LAUNCH_CHECK();
  }
  return PCE_OK;
}

int umma_where_fetch(int* host4) {
  PCE_CUDA(cudaMemcpyFromSymbol(host4, g_umma_where, 4 * sizeof(int)));
  int z[4] = {0, 0, 0, 0};
  PCE_CUDA(cudaMemcpyToSymbol(g_umma_where, z, 4 * sizeof(int)));
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
