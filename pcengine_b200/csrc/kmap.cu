// Kernel-map construction for sm_100a: coordinate hash table on 64-bit packed
// (b,x,y,z) keys, input-major neighbour query, per-offset scans, and the
// derived forms (pair lists, CSR-coded gather/scatter maps, neighbour CSR with
// indicator bitmask).  Replaces backend/hash.cu + backend/hash.cuh of the
// reference and the tensor post-pass of script/spconv.py:370-376.
//
// Table layout: 16-byte slots {u64 key, i32 value, i32 pad}; a probe is one
// 16-byte load, so a lookup that hits on its first slot costs one L2 access
// (the tables are 1-70 MB and live in the 126 MB L2).  Linear probing on a
// power-of-two table at load <= 0.5; every probe loop is bounded by the table
// size and reports PCE_ERR_TABLE_FULL through the status word instead of
// spinning.
#include <sched.h>

#include <chrono>
#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_scan.cuh>

#include "common.cuh"

namespace pce {

thread_local int g_last_cuda_error = 0;
unsigned long long g_kernel_launches = 0;

struct __align__(16) Slot {
  unsigned long long key;
  int val;
  int pad;
};

struct GeomDev {
  int ks[3], st[3], pd[3], lo[3], hi[3];
  int subm, kv, mid;
};

static GeomDev to_dev(const pce_geom* g) {
  GeomDev d;
  for (int i = 0; i < 3; ++i) {
    d.ks[i] = g->ks[i];
    d.st[i] = g->stride[i];
    d.pd[i] = g->pad[i];
    d.lo[i] = g->cmin[i];
    d.hi[i] = g->cmax[i];
  }
  d.subm = g->submanifold;
  d.kv = g->ks[0] * g->ks[1] * g->ks[2];
  d.mid = (g->ks[0] - 1) / 2 * g->ks[1] * g->ks[2] + (g->ks[1] - 1) / 2 * g->ks[2] + (g->ks[2] - 1) / 2;
  return d;
}

static unsigned table_size_for(long long n) {
  unsigned t = 1024;
  while (static_cast<long long>(t) < 2 * n) t <<= 1;
  return t;
}

// Offset of weight index kp (x slowest).  Submanifold: centred
// (ref: backend/hash.cuh:313-315); strided: +1 for odd sizes above one
// (ref: backend/hash.cuh:396-401).
__device__ __forceinline__ void offset_of(const GeomDev& g, int kp, int& kx, int& ky, int& kz) {
  kx = kp / (g.ks[2] * g.ks[1]) - (g.ks[0] - 1) / 2;
  ky = (kp / g.ks[2]) % g.ks[1] - (g.ks[1] - 1) / 2;
  kz = kp % g.ks[2] - (g.ks[2] - 1) / 2;
  if (!g.subm) {
    kx += (g.ks[0] % 2 == 0 || g.ks[0] == 1) ? 0 : 1;
    ky += (g.ks[1] % 2 == 0 || g.ks[1] == 1) ? 0 : 1;
    kz += (g.ks[2] % 2 == 0 || g.ks[2] == 1) ? 0 : 1;
  }
}

// The output voxel that input (x,y,z) feeds through offset kp, if any:
// (in + pad - k) / stride, exact, inside [lo, hi]
// (ref: backend/hash.cuh:591-604; for a submanifold map stride = 1, pad = 0 and
// the bounds do not apply, ref: backend/hash.cuh:313-319 read from the input side).
__device__ __forceinline__ bool candidate(const GeomDev& g, int kp, int x, int y, int z, int& qx, int& qy,
                                          int& qz) {
  int kx, ky, kz;
  offset_of(g, kp, kx, ky, kz);
  if (g.subm) {
    qx = x - kx;
    qy = y - ky;
    qz = z - kz;
    return true;
  }
  int cx = x - kx + g.pd[0], cy = y - ky + g.pd[1], cz = z - kz + g.pd[2];
  qx = cx / g.st[0];
  qy = cy / g.st[1];
  qz = cz / g.st[2];
  if (qx < g.lo[0] || qx > g.hi[0] || cx % g.st[0] != 0) return false;
  if (qy < g.lo[1] || qy > g.hi[1] || cy % g.st[1] != 0) return false;
  if (qz < g.lo[2] || qz > g.hi[2] || cz % g.st[2] != 0) return false;
  return true;
}

__device__ __forceinline__ Slot load_slot(const Slot* t, unsigned s) {
  const int4 v = __ldg(reinterpret_cast<const int4*>(t) + s);
  Slot r;
  r.key = (static_cast<unsigned long long>(static_cast<unsigned>(v.y)) << 32) | static_cast<unsigned>(v.x);
  r.val = v.z;
  r.pad = v.w;
  return r;
}

// Returns the value stored for `key`, or -1.
__device__ __forceinline__ int table_find(const Slot* t, unsigned tmask, unsigned long long key) {
  unsigned s = static_cast<unsigned>(mix64(key)) & tmask;
  for (unsigned n = 0; n <= tmask; ++n) {
    Slot sl = load_slot(t, s);
    if (sl.key == key) return sl.val;
    if (sl.key == kEmptyKey) return -1;
    s = (s + 1) & tmask;
  }
  return -1;
}

// Claims a slot for `key`.  Returns the slot index, sets `fresh` when this
// call inserted the key; returns 0xFFFFFFFF when the table is full.
__device__ __forceinline__ unsigned table_claim(Slot* t, unsigned tmask, unsigned long long key, bool& fresh) {
  unsigned s = static_cast<unsigned>(mix64(key)) & tmask;
  fresh = false;
  for (unsigned n = 0; n <= tmask; ++n) {
    unsigned long long prev = atomicCAS(&t[s].key, kEmptyKey, key);
    if (prev == kEmptyKey) {
      fresh = true;
      return s;
    }
    if (prev == key) return s;
    s = (s + 1) & tmask;
  }
  return 0xFFFFFFFFu;
}

// ---- kernels ---------------------------------------------------------------

// value = row index (duplicate coordinates are outside the contract; the largest row wins).
__global__ void k_insert_rows(const int4* __restrict__ coords, int n, Slot* table, unsigned tmask, int* status) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int4 c = __ldg(coords + i);
  if (!packable(c.x, c.y, c.z, c.w)) {
    atomicMax(status, PCE_ERR_RANGE);
    return;
  }
  bool fresh;
  unsigned s = table_claim(table, tmask, pack_key(c.x, c.y, c.z, c.w), fresh);
  if (s == 0xFFFFFFFFu) {
    atomicMax(status, PCE_ERR_TABLE_FULL);
    return;
  }
  (void)fresh;
  atomicMax(&table[s].val, i);  // slots start at -1; duplicate rows keep the largest index
}

// Sort key of an output coordinate: (b, x - lo, y - lo, z - lo) in as few bits as the output bounds
// need (z lowest), so that the radix sort of the unique keys runs over ~30 bits instead of 64.
struct KeyBits {
  int sh_y, sh_x, sh_b;  // shifts of the y, x and batch fields
};

static KeyBits key_bits_for(const GeomDev& g) {
  auto bits = [](long long extent) {
    int b = 1;
    while (b < 16 && (1ll << b) < extent) ++b;
    return b;
  };
  KeyBits k;
  k.sh_y = bits(static_cast<long long>(g.hi[2]) - g.lo[2] + 1);
  k.sh_x = k.sh_y + bits(static_cast<long long>(g.hi[1]) - g.lo[1] + 1);
  k.sh_b = k.sh_x + bits(static_cast<long long>(g.hi[0]) - g.lo[0] + 1);
  return k;
}

// Strided output coordinates, step 1: every valid candidate is inserted into a
// set; the sort keys of first-time members are appended to ukeys (unordered).
// One thread per input coordinate walks the kernel offsets and keeps the new keys it finds in a small
// register buffer; a warp appends its buffers with ONE atomic on the shared counter (when a lane's buffer
// is full, and at the end): the counter is a single address, and an atomic per key, or per warp and
// offset, serialises the kernel on it.
__global__ void k_candidates(const int4* __restrict__ coords, int n_in, GeomDev g, KeyBits kb, Slot* table,
                             unsigned tmask, unsigned long long* ukeys, int ucap, int* counter, int* status,
                             int* max_batch) {
  constexpr int kHold = 4;
  constexpr unsigned kFull = 0xFFFFFFFFu;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const unsigned lane = threadIdx.x & 31;
  const bool live = i < n_in;
  const int4 c = live ? __ldg(coords + i) : make_int4(0, 0, 0, 0);
  unsigned long long held[kHold];
  int n_held = 0;
  bool any_fresh = false;
  auto flush = [&]() {
    int incl = n_held;  // inclusive prefix of the lanes' counts
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int v = __shfl_up_sync(kFull, incl, d);
      if (lane >= static_cast<unsigned>(d)) incl += v;
    }
    const int total = __shfl_sync(kFull, incl, 31);
    if (total == 0) return;
    int base = 0;
    if (lane == 31) base = atomicAdd(counter, total);
    base = __shfl_sync(kFull, base, 31) + incl - n_held;
#pragma unroll
    for (int u = 0; u < kHold; ++u) {
      if (u < n_held) {
        if (base + u < ucap)
          ukeys[base + u] = held[u];
        else
          atomicMax(status, PCE_ERR_CAPACITY);
      }
    }
    n_held = 0;
  };
  // Per axis the kernel offsets are o = omin + i, i in [0, ks) (offset_of), and an offset reaches an output
  // from this input when x + pad - o is a multiple of the stride: i = r, r + stride, ... < ks with
  // r = (x + pad - omin) mod stride; the output is then q0 - j for the j-th of them.  Walking those directly
  // costs three divisions per input instead of six per (input, offset).  The loop bounds are the same for
  // every lane (the warp-wide flush sits inside).
  int r[3], q0[3];
  {
    const int xyz[3] = {c.y, c.z, c.w};
    int a[3];
#pragma unroll
    for (int d = 0; d < 3; ++d) {
      const int omin = -((g.ks[d] - 1) / 2) + ((g.ks[d] % 2 == 0 || g.ks[d] == 1) ? 0 : 1);
      a[d] = xyz[d] + g.pd[d] - omin;
    }
#pragma unroll
    for (int d = 0; d < 3; ++d) {
      int m = a[d] % g.st[d];
      if (m < 0) m += g.st[d];
      r[d] = m;
      q0[d] = (a[d] - m) / g.st[d];
    }
  }
  const int nx = (g.ks[0] + g.st[0] - 1) / g.st[0], ny = (g.ks[1] + g.st[1] - 1) / g.st[1],
            nz = (g.ks[2] + g.st[2] - 1) / g.st[2];
  for (int jx = 0; jx < nx; ++jx) {
    for (int jy = 0; jy < ny; ++jy) {
      for (int jz = 0; jz < nz; ++jz) {
        const int qx = q0[0] - jx, qy = q0[1] - jy, qz = q0[2] - jz;
        const bool reach = live && r[0] + jx * g.st[0] < g.ks[0] && r[1] + jy * g.st[1] < g.ks[1] &&
                           r[2] + jz * g.st[2] < g.ks[2] && qx >= g.lo[0] && qx <= g.hi[0] && qy >= g.lo[1] &&
                           qy <= g.hi[1] && qz >= g.lo[2] && qz <= g.hi[2];
        if (reach) {
          if (!packable(c.x, qx, qy, qz)) {
            atomicMax(status, PCE_ERR_RANGE);
          } else {
            bool fresh = false;
            const unsigned s = table_claim(table, tmask, pack_key(c.x, qx, qy, qz), fresh);
            if (s == 0xFFFFFFFFu) {
              atomicMax(status, PCE_ERR_TABLE_FULL);
            } else if (fresh) {
              // q lies inside [lo, hi], so every field fits its bits
              const unsigned long long key = (static_cast<unsigned long long>(c.x) << kb.sh_b) |
                                             (static_cast<unsigned long long>(qx - g.lo[0]) << kb.sh_x) |
                                             (static_cast<unsigned long long>(qy - g.lo[1]) << kb.sh_y) |
                                             static_cast<unsigned long long>(qz - g.lo[2]);
#pragma unroll
              for (int u = 0; u < kHold; ++u)
                if (u == n_held) held[u] = key;
              ++n_held;
              any_fresh = true;
            }
          }
        }
        if (__any_sync(kFull, n_held == kHold)) flush();
      }
    }
  }
  flush();
  // the largest batch index among the new keys (it sizes the sort key): one atomic per warp at most
  const int wmax = __reduce_max_sync(kFull, any_fresh ? c.x : 0);
  if (lane == 0 && wmax > *reinterpret_cast<volatile int*>(max_batch)) atomicMax(max_batch, wmax);
}

__global__ void k_decode_keys(const unsigned long long* __restrict__ keys, int n, GeomDev g, KeyBits kb, int4* coords) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const unsigned long long k = keys[i];
  const int z = static_cast<int>(k & ((1ull << kb.sh_y) - 1)) + g.lo[2];
  const int y = static_cast<int>((k >> kb.sh_y) & ((1ull << (kb.sh_x - kb.sh_y)) - 1)) + g.lo[1];
  const int x = static_cast<int>((k >> kb.sh_x) & ((1ull << (kb.sh_b - kb.sh_x)) - 1)) + g.lo[0];
  coords[i] = make_int4(static_cast<int>(k >> kb.sh_b), x, y, z);
}

// Input-major query: one thread per (input row, offset).  Writes the dense
// indicator table map[kp][in] (= the reference's D2 `map`), optionally the
// transposed table map_out[kp][out], and per-offset hit counts.
// MIRROR (submanifold maps with odd kernel sizes): only the offsets below the centre are
// probed (gridDim.y = mid); a hit "input i feeds output j through kp" is also the hit
// "input j feeds output i through kv-1-kp", so each probe fills two entries and the rows
// kp >= mid, preset to -1 by the caller, receive only their hits.
template <bool MIRROR>
__global__ void k_query(const int4* __restrict__ in_coords, int n_in, GeomDev g, const Slot* __restrict__ table,
                        unsigned tmask, int* __restrict__ map, int* __restrict__ map_out, int n_out,
                        int* knnz, int* status) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int kp = blockIdx.y;
  int res = -1;
  if (i < n_in && !(g.subm && kp == g.mid)) {
    int4 c = __ldg(in_coords + i);
    int qx, qy, qz;
    if (candidate(g, kp, c.y, c.z, c.w, qx, qy, qz) && packable(c.x, qx, qy, qz)) {
      res = table_find(table, tmask, pack_key(c.x, qx, qy, qz));
    }
  }
  if (i < n_in) map[static_cast<size_t>(kp) * n_in + i] = res;
  if (MIRROR) {
    if (res >= 0) map[static_cast<size_t>(g.kv - 1 - kp) * n_in + res] = i;
  } else {
    if (res >= 0 && map_out != nullptr) map_out[static_cast<size_t>(kp) * n_out + res] = i;
  }
  int cnt = __syncthreads_count(res >= 0);
  if (threadIdx.x == 0 && cnt) {
    atomicAdd(&knnz[kp], cnt);
    if (MIRROR) atomicAdd(&knnz[g.kv - 1 - kp], cnt);
  }
}

// Warp-cooperative form of k_query: FOUR lanes share one (input row, offset) query and read four
// consecutive slots of its probe sequence per round (one aligned-or-not 64-byte request instead of
// dependent 16-byte loads); ballots over the four lanes find the key or the first empty slot.  Same
// results as k_query (linear probing visits the slots in the same order); 64 queries per block.
template <bool MIRROR>
__global__ void __launch_bounds__(256)
    k_query_coop(const int4* __restrict__ in_coords, int n_in, GeomDev g, const Slot* __restrict__ table, unsigned tmask,
                 int* __restrict__ map, int* __restrict__ map_out, int n_out, int* knnz, int* status) {
  const int sub = threadIdx.x & 3;
  const int i = blockIdx.x * 64 + (threadIdx.x >> 2);
  const int kp = blockIdx.y;
  const unsigned group = 0xFu << (threadIdx.x & 28);  // the four lanes of this query inside the warp
  int res = -1;
  if (i < n_in && !(g.subm && kp == g.mid)) {
    const int4 c = __ldg(in_coords + i);
    int qx, qy, qz;
    if (candidate(g, kp, c.y, c.z, c.w, qx, qy, qz) && packable(c.x, qx, qy, qz)) {
      const unsigned long long key = pack_key(c.x, qx, qy, qz);
      unsigned s = static_cast<unsigned>(mix64(key)) & tmask;
      for (unsigned n = 0; n <= tmask; n += 4) {  // bounded: at most one pass over the table
        const Slot sl = load_slot(table, (s + sub) & tmask);
        const unsigned hit = __ballot_sync(group, sl.key == key) & group;
        const unsigned empty = __ballot_sync(group, sl.key == kEmptyKey) & group;
        if (hit) {  // keys are unique and never behind an empty slot of their own probe sequence
          res = __shfl_sync(group, sl.val, __ffs(hit) - 1);
          break;
        }
        if (empty) break;
        s = (s + 4) & tmask;
      }
    }
  }
  const bool writer = sub == 0 && i < n_in;
  if (writer) map[static_cast<size_t>(kp) * n_in + i] = res;
  if (writer && res >= 0) {
    if (MIRROR)
      map[static_cast<size_t>(g.kv - 1 - kp) * n_in + res] = i;
    else if (map_out != nullptr)
      map_out[static_cast<size_t>(kp) * n_out + res] = i;
  }
  const int cnt = __syncthreads_count(writer && res >= 0);
  if (threadIdx.x == 0 && cnt) {
    atomicAdd(&knnz[kp], cnt);
    if (MIRROR) atomicAdd(&knnz[g.kv - 1 - kp], cnt);
  }
}

// 0: one thread per query (k_query, the default: measured faster); 1: four lanes per query (k_query_coop).
int kmap_query_lanes4 = 0;
// Row-order sort on the most significant N bits of the rarity-permuted bitmask key only (0 = all bits).
int kmap_sort_top_bits = 0;

// Launches the query for all offsets; n_in, n_out > 0.
static int run_query(const int32_t* in_coords, int n_in, const GeomDev& gd, const Slot* table, unsigned tsize, int* map,
                     int* map_out, int n_out, int* knnz, int* st_word, cudaStream_t st) {
  const bool odd = (gd.ks[0] & 1) && (gd.ks[1] & 1) && (gd.ks[2] & 1);
  const bool coop = kmap_query_lanes4 != 0;
  const int per_block = coop ? 64 : 256;
  if (gd.subm && odd && gd.kv > 1 && map_out == nullptr && n_in == n_out) {
    PCE_CUDA(cudaMemsetAsync(map + static_cast<size_t>(gd.mid) * n_in, 0xFF,
                             sizeof(int) * static_cast<size_t>(gd.kv - gd.mid) * n_in, st));
    dim3 grid(div_up(n_in, per_block), gd.mid);
    if (coop)
      k_query_coop<true><<<grid, 256, 0, st>>>(reinterpret_cast<const int4*>(in_coords), n_in, gd, table, tsize - 1, map,
                                               nullptr, n_out, knnz, st_word);
    else
      k_query<true><<<grid, 256, 0, st>>>(reinterpret_cast<const int4*>(in_coords), n_in, gd, table, tsize - 1, map,
                                          nullptr, n_out, knnz, st_word);
  } else {
    dim3 grid(div_up(n_in, per_block), gd.kv);
    if (coop)
      k_query_coop<false><<<grid, 256, 0, st>>>(reinterpret_cast<const int4*>(in_coords), n_in, gd, table, tsize - 1, map,
                                                map_out, n_out, knnz, st_word);
    else
      k_query<false><<<grid, 256, 0, st>>>(reinterpret_cast<const int4*>(in_coords), n_in, gd, table, tsize - 1, map,
                                           map_out, n_out, knnz, st_word);
  }
  PCE_LAUNCH_CHECK();
  return PCE_OK;
}

// kpos / qkpos (segments padded to 128), kv+1 entries each
// (ref: backend/hash.cuh:478-497).
__global__ void k_offset_scans(const int* __restrict__ knnz, int kv, int* kpos, int* qkpos) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    int a = 0, q = 0;
    kpos[0] = 0;
    qkpos[0] = 0;
    for (int k = 0; k < kv; ++k) {
      a += knnz[k];
      q += (knnz[k] + 127) / 128 * 128;
      kpos[k + 1] = a;
      qkpos[k + 1] = q;
    }
  }
}

struct FlagOf {
  const int* map;
  __host__ __device__ int operator()(const int& idx) const { return map[idx] != -1 ? 1 : 0; }
};

__global__ void k_flags(const int* __restrict__ map, long long n, int* flags) {
  long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) flags[i] = map[i] != -1 ? 1 : 0;
}

__global__ void k_emit_pairs(const int* __restrict__ map, const int* __restrict__ rank, int kv, int n_in,
                             int* imap, int* omap, int cap) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  int kp = blockIdx.y;
  if (i >= n_in) return;
  size_t idx = static_cast<size_t>(kp) * n_in + i;
  int o = map[idx];
  if (o < 0) return;
  int p = rank[idx];
  if (p < cap) {
    imap[p] = i;
    omap[p] = o;
  }
}

// Row-wise passes over a dense [kv][n_rows] table.
//   MODE 0: neighbour CSR     value = the table entry (or the row itself for identity_kp)
//   MODE 1: coded input rows  value = kp*1186111 + rank[kp][row] - kpos[kp]
//   MODE 2: coded output rows value = kp*1186111 + rank[kp][entry] - kpos[kp]
struct RowArgs {
  const int* table;
  int kv, n_rows, reverse, identity_kp;
  const int* rank;  // [kv][n_in] global pair index (modes 1, 2)
  const int* kpos;
  int n_in;
};

__device__ __forceinline__ int row_entry(const RowArgs& a, int kp, int r) {
  if (kp == a.identity_kp) return r;
  int src = a.reverse ? (a.kv - 1 - kp) : kp;
  return a.table[static_cast<size_t>(src) * a.n_rows + r];
}

__global__ void k_row_count(RowArgs a, uint32_t* mask, int* counts) {
  int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r > a.n_rows) return;
  if (r == a.n_rows) {
    counts[r] = 0;
    return;
  }
  const int words = (a.kv + 31) / 32;
  int cnt = 0;
  for (int w = 0; w < words; ++w) {
    uint32_t m = 0;
    int kend = min(32, a.kv - w * 32);
    for (int b = 0; b < kend; ++b) {
      if (row_entry(a, w * 32 + b, r) >= 0) m |= (1u << b);
    }
    cnt += __popc(m);
    if (mask) mask[static_cast<size_t>(r) * words + w] = m;
  }
  counts[r] = cnt;
}

template <int MODE>
__global__ void k_row_fill(RowArgs a, const int* __restrict__ rowptr, int* out, int cap) {
  int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= a.n_rows) return;
  int p = rowptr[r];
  for (int kp = 0; kp < a.kv; ++kp) {
    int v = row_entry(a, kp, r);
    if (v < 0) continue;
    int val;
    if (MODE == 0) {
      val = v;
    } else {
      int in_row = (MODE == 1) ? r : v;
      val = kp * 1186111 + a.rank[static_cast<size_t>(kp) * a.n_in + in_row] - a.kpos[kp];
    }
    if (p < cap) out[p] = val;
    ++p;
  }
}

// Pair lists -> sortable (row, index) arrays with the identity pairs spliced in
// at the centre offset so that a stable sort by row keeps kp ascending.
__global__ void k_pairs_keys(const int* __restrict__ rows, const int* __restrict__ kpos, int n_pairs, int n_rows,
                             int identity_kp, int* keys, int* vals) {
  int e = blockIdx.x * blockDim.x + threadIdx.x;
  int total = n_pairs + (identity_kp >= 0 ? n_rows : 0);
  if (e >= total) return;
  int row;
  if (identity_kp >= 0) {
    int km = kpos[identity_kp];
    if (e < km)
      row = rows[e];
    else if (e < km + n_rows)
      row = e - km;
    else
      row = rows[e - n_rows];
  } else {
    row = rows[e];
  }
  keys[e] = row;
  vals[e] = e;
}

__global__ void k_pairs_rows(const int* __restrict__ skeys, const int* __restrict__ svals,
                             const int* __restrict__ nbrs, const int* __restrict__ kpos, int kv, int n_pairs,
                             int n_rows, int identity_kp, uint32_t* mask, int* counts, int* nbr, int cap) {
  int j = blockIdx.x * blockDim.x + threadIdx.x;
  int total = n_pairs + (identity_kp >= 0 ? n_rows : 0);
  if (j >= total) return;
  int row = skeys[j];
  int e = svals[j];
  int kp, v;
  int km = identity_kp >= 0 ? kpos[identity_kp] : 0;
  int p = e;
  bool ident = false;
  if (identity_kp >= 0) {
    if (e >= km && e < km + n_rows) {
      ident = true;
    } else if (e >= km + n_rows) {
      p = e - n_rows;
    }
  }
  if (ident) {
    kp = identity_kp;
    v = row;
  } else {
    // largest kp with kpos[kp] <= p
    int lo = 0, hi = kv;
    while (hi - lo > 1) {
      int mid = (lo + hi) >> 1;
      if (kpos[mid] <= p)
        lo = mid;
      else
        hi = mid;
    }
    kp = lo;
    v = nbrs[p];
  }
  const int words = (kv + 31) / 32;
  atomicOr(&mask[static_cast<size_t>(row) * words + (kp >> 5)], 1u << (kp & 31));
  atomicAdd(&counts[row], 1);
  if (j < cap) nbr[j] = v;
}

// Row order for the tile lists.  Rows that share offsets should share tiles, and a tile pays one
// stage for every offset ANY of its rows has, so the expensive offsets are the rare ones: a tile
// that contains a single row with a rare offset pays a stage that is 1/128 full.  The sort key is
// therefore the indicator bitmask with its bits permuted by rarity, the rarest offset in the most
// significant position: rows with a rare offset end up next to each other and the tiles in between
// do not pay for it.  Measured stages per 128-row tile against the plain bitmask as key: 3x3x3
// LiDAR levels 3-7 % fewer, 5x5x5 indoor 16.0 instead of 23.5 (19.0 for the unpermuted full mask).
// Only used to group similar rows, never for correctness.

// counts[k] = rows that have offset k.
__global__ void k_offset_counts(const uint32_t* __restrict__ mask, int n_rows, int words, int* counts) {
  __shared__ int local[128];
  if (threadIdx.x < 128) local[threadIdx.x] = 0;
  __syncthreads();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  const int lane = threadIdx.x & 31;
  for (int w = 0; w < words; ++w) {
    const uint32_t m = r < n_rows ? __ldg(mask + static_cast<size_t>(r) * words + w) : 0u;
    const uint32_t any = __reduce_or_sync(0xFFFFFFFFu, m);
    for (uint32_t rest = any; rest; rest &= rest - 1) {
      const int bit = __ffs(rest) - 1;
      const int c = __popc(__ballot_sync(0xFFFFFFFFu, (m >> bit) & 1u));
      if (lane == 0) atomicAdd(&local[w * 32 + bit], c);
    }
  }
  __syncthreads();
  if (threadIdx.x < 128 && local[threadIdx.x]) atomicAdd(&counts[threadIdx.x], local[threadIdx.x]);
}

// keys = the bitmask with offset k moved to bit kv-1-rank(k), rank 0 = rarest (ties by index);
// lo holds positions 0..63, hi positions 64..127 (kv > 64 only).
__global__ void k_mask_keys(const uint32_t* __restrict__ mask, int n_rows, int words, int kv,
                            const int* __restrict__ counts, unsigned long long* lo, unsigned long long* hi,
                            int* vals) {
  __shared__ int pos[128];
  if (threadIdx.x < 128) {
    const int k = threadIdx.x;
    int rank = 0;
    if (k < kv) {
      const int ck = counts[k];
      for (int j = 0; j < kv; ++j) {
        const int cj = counts[j];
        rank += (cj < ck || (cj == ck && j < k)) ? 1 : 0;
      }
    }
    pos[k] = kv - 1 - rank;
  }
  __syncthreads();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= n_rows) return;
  unsigned long long klo = 0, khi = 0;
  for (int w = 0; w < words; ++w) {
    for (uint32_t m = mask[static_cast<size_t>(r) * words + w]; m; m &= m - 1) {
      const int p = pos[w * 32 + __ffs(m) - 1];
      if (p < 64)
        klo |= 1ull << p;
      else
        khi |= 1ull << (p - 64);
    }
  }
  lo[r] = klo;
  if (hi) hi[r] = khi;
  vals[r] = r;
}

// pos[k] = bit position of offset k in the sort key: kv-1-rank(k), rank 0 = the rarest offset (ties by
// index).  count_of(k) = rows that have offset k.
template <typename CountOf>
__device__ __forceinline__ int key_position(int k, int kv, CountOf count_of) {
  int rank = 0;
  const int ck = count_of(k);
  for (int j = 0; j < kv; ++j) {
    const int cj = count_of(j);
    rank += (cj < ck || (cj == ck && j < k)) ? 1 : 0;
  }
  return kv - 1 - rank;
}

// The same key in 32 bits (kv <= 32): half the key bytes through the radix sort's passes.
__global__ void k_mask_keys32(const uint32_t* __restrict__ mask, int n_rows, int kv, const int* __restrict__ counts,
                              uint32_t* keys, int* vals) {
  __shared__ int pos[32];
  if (threadIdx.x < 32) {
    const int k = threadIdx.x;
    int rank = 0;
    if (k < kv) {
      const int ck = counts[k];
      for (int j = 0; j < kv; ++j) {
        const int cj = counts[j];
        rank += (cj < ck || (cj == ck && j < k)) ? 1 : 0;
      }
    }
    pos[k] = kv - 1 - rank;
  }
  __syncthreads();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= n_rows) return;
  uint32_t key = 0;
  for (uint32_t m = mask[r]; m; m &= m - 1) key |= 1u << pos[__ffs(m) - 1];
  keys[r] = key;
  vals[r] = r;
}

// One pass over the dense table for maps of at most 32 offsets: the row's bitmask and its sort key (what
// k_row_count, k_offset_counts and k_mask_keys32 produce in three passes).  The number of rows that have
// offset k is known without counting: it is the map's knnz at the table column the offset reads (every row
// holds at most one pair per offset), and n_rows for the identity offset.
__global__ void k_row_mask_key32(RowArgs a, const int* __restrict__ knnz, uint32_t* mask, int* counts, uint32_t* keys,
                                 int* vals) {
  __shared__ int pos[32];
  if (threadIdx.x < 32) {
    const int k = threadIdx.x;
    auto count_of = [&](int j) { return j == a.identity_kp ? a.n_rows : __ldg(knnz + (a.reverse ? a.kv - 1 - j : j)); };
    pos[k] = k < a.kv ? key_position(k, a.kv, count_of) : 0;
  }
  __syncthreads();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r > a.n_rows) return;
  if (r == a.n_rows) {
    if (counts) counts[r] = 0;
    return;
  }
  uint32_t m = 0, key = 0;
  for (int b = 0; b < a.kv; ++b) {
    if (row_entry(a, b, r) >= 0) {
      m |= 1u << b;
      key |= 1u << pos[b];
    }
  }
  mask[r] = m;
  if (counts) counts[r] = __popc(m);
  keys[r] = key;
  vals[r] = r;
}

__global__ void k_gather_u64(const unsigned long long* __restrict__ src, const int* __restrict__ idx, int n,
                             unsigned long long* dst) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = src[idx[i]];
}

// Tile lists: the map re-laid for output tiles of blockDim.x (128, 256 or 512) rows taken in
// processing order.  One CTA per tile; thread r owns the tile's r-th row.  With one offset per stage
// (slots == 1) stage_kp carries, above the offset's 8 bits, one presence bit per 128-row sub-tile of
// the tile: bit 8+s is set when a row of sub-tile s has the offset.
//   FILL = false: tile_cnt[t] = number of offsets any row of the tile has (+1 with `identity`).
//   FILL = true : for the tile's s-th present offset (ascending kp) write stage_kp[base+s] and
//                 stage_nbr[(base+s)*rows + r] = the row's input at that offset, or -1.
//   identity: every tile ends with one more stage, stage_kp = -1, whose entry for a row is the row
//   itself: the place where a second operand indexed like the output joins the accumulation.
//   slots (1, 2 or 4): offsets per stage.  A layer with 32 (16) input channels fills only half (a
//   quarter) of the kernel's 64-channel K block, so 2 (4) of a tile's offsets share one stage:
//   stage_kp[g*slots + q] and stage_nbr[(g*slots + q)*rows + r]; unused slots hold kp = -2, nbr = -1.
//   DENSE: the row's input at an offset is read from the dense table (`dense`, as k_row_count reads it)
//   instead of from the neighbour CSR, which then need not exist.
template <bool FILL, bool DENSE = false>
__global__ void __launch_bounds__(512)
    k_tile_lists(const uint32_t* __restrict__ mask, const int* __restrict__ rowptr, const int* __restrict__ nbr,
                 const int* __restrict__ order, int n_rows, int words, int identity, int slots, int* tile_cnt,
                 const int* __restrict__ tile_ptr, int* stage_kp, int* stage_nbr, int stage_cap, RowArgs dense = RowArgs{}) {
  __shared__ uint32_t wmask[16][4];
  const int t = blockIdx.x, r = threadIdx.x, warp = r >> 5, lane = r & 31;
  const int rows = blockDim.x, nwarps = blockDim.x >> 5;
  const int slot = t * rows + r;
  int row = -1;
  if (slot < n_rows) row = order ? __ldg(order + slot) : slot;
  uint32_t my[4] = {0, 0, 0, 0};
  if (row >= 0)
    for (int w = 0; w < words; ++w) my[w] = __ldg(mask + static_cast<size_t>(row) * words + w);
  for (int w = 0; w < 4; ++w) {
    const uint32_t m = __reduce_or_sync(0xFFFFFFFFu, my[w]);
    if (lane == 0) wmask[warp][w] = m;
  }
  __syncthreads();
  uint32_t tm[4];
  int cnt = 0;
  for (int w = 0; w < 4; ++w) {
    tm[w] = 0;
    for (int q = 0; q < nwarps; ++q) tm[w] |= wmask[q][w];
    cnt += __popc(tm[w]);
  }
  if (!FILL) {
    if (r == 0) tile_cnt[t] = (cnt + slots - 1) / slots + (identity ? 1 : 0);
    return;
  }
  const int base = __ldg(tile_ptr + t);
  int cursor = (!DENSE && row >= 0) ? __ldg(rowptr + row) : 0;
  int s = 0;
  for (int w = 0; w < words; ++w) {
    uint32_t m = tm[w];
    while (m) {
      const int bit = __ffs(m) - 1;
      m &= m - 1;
      int v = -1;
      if ((my[w] >> bit) & 1u) v = DENSE ? row_entry(dense, w * 32 + bit, row) : __ldg(nbr + cursor++);
      const int g = base + s / slots;
      if (g < stage_cap) {
        const size_t e = static_cast<size_t>(g) * slots + s % slots;
        stage_nbr[e * rows + r] = v;
        if (r == 0) {
          int code = w * 32 + bit;
          if (slots == 1) {
            for (int sub = 0; sub < (nwarps >> 2); ++sub) {
              const uint32_t m4 = wmask[4 * sub][w] | wmask[4 * sub + 1][w] | wmask[4 * sub + 2][w] | wmask[4 * sub + 3][w];
              if ((m4 >> bit) & 1u) code |= 1 << (8 + sub);
            }
          }
          stage_kp[e] = code;
        }
      }
      ++s;
    }
  }
  for (; s % slots; ++s) {  // unused slots of the last stage
    const int g = base + s / slots;
    if (g < stage_cap) {
      const size_t e = static_cast<size_t>(g) * slots + s % slots;
      stage_nbr[e * rows + r] = -1;
      if (r == 0) stage_kp[e] = -2;
    }
  }
  if (identity) {
    const int g = base + s / slots;
    if (g < stage_cap) {
      for (int q = 0; q < slots; ++q) {
        const size_t e = static_cast<size_t>(g) * slots + q;
        stage_nbr[e * rows + r] = q == 0 ? row : -1;
        if (r == 0) stage_kp[e] = q == 0 ? -1 : -2;
      }
    }
  }
}

// ---- host helpers ------------------------------------------------------------

// Waits for everything queued on `st` without burning a core: polls an event, yielding the
// processor between polls, for a short while (the usual case: a few microseconds of work ahead),
// then sleeps on it.  cudaStreamSynchronize spins, and the size read-back of a strided layer can
// wait for milliseconds behind other work; with one process per GPU and several planner threads
// per process, spinning starves the threads that queue the kernels being waited for.
static int wait_for_stream(cudaStream_t st) {
  static thread_local cudaEvent_t ev[64] = {};
  int dev = 0;
  PCE_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) {
    PCE_CUDA(cudaStreamSynchronize(st));
    return PCE_OK;
  }
  if (!ev[dev]) PCE_CUDA(cudaEventCreateWithFlags(&ev[dev], cudaEventBlockingSync | cudaEventDisableTiming));
  PCE_CUDA(cudaEventRecord(ev[dev], st));
  const auto t0 = std::chrono::steady_clock::now();
  for (;;) {
    const cudaError_t q = cudaEventQuery(ev[dev]);
    if (q == cudaSuccess) return PCE_OK;
    if (q != cudaErrorNotReady) return cuda_fail(q);
    (void)cudaGetLastError();  // "not ready" is an answer, not a failure
    if (std::chrono::steady_clock::now() - t0 > std::chrono::microseconds(200)) break;
    sched_yield();
  }
  PCE_CUDA(cudaEventSynchronize(ev[dev]));
  return PCE_OK;
}

// Exclusive sum of a SHORT array by one block (tile counts: a few thousand entries): out[i] = in[0] + .. + in[i-1] for
// i < n, out[n] = the total; one launch where the library scan takes two (tile-state set-up + scan) and a memset for
// the extra element, for every tile list of every map of a pass.
__global__ void __launch_bounds__(1024) k_scan_small(const int* __restrict__ in, int* __restrict__ out, int n) {
  __shared__ int warp_sum[32];
  __shared__ int carry_s;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) carry_s = 0;
  __syncthreads();
  for (int base = 0; base <= n; base += 1024) {
    const int i = base + tid;
    const int v = i < n ? in[i] : 0;
    int incl = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int u = __shfl_up_sync(0xFFFFFFFFu, incl, d);
      if (lane >= d) incl += u;
    }
    if (lane == 31) warp_sum[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      int w = warp_sum[lane];
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int u = __shfl_up_sync(0xFFFFFFFFu, w, d);
        if (lane >= d) w += u;
      }
      warp_sum[lane] = w;  // inclusive over the warps
    }
    __syncthreads();
    const int carry = carry_s;
    const int before = carry + (warp > 0 ? warp_sum[warp - 1] : 0) + incl - v;
    if (i <= n) out[i] = before;
    __syncthreads();
    if (tid == 0) carry_s = carry + warp_sum[31];
    __syncthreads();
  }
}

static int exclusive_scan_i32(Arena& ar, const int* in, int* out, long long n, cudaStream_t st) {
  size_t need = 0;
  PCE_CUDA(cub::DeviceScan::ExclusiveSum(nullptr, need, in, out, static_cast<int>(n), st));
  char* tmp = ar.take<char>(need);
  if (!ar.ok) return PCE_ERR_WORKSPACE;
  PCE_CUDA(cub::DeviceScan::ExclusiveSum(tmp, need, in, out, static_cast<int>(n), st));
  return PCE_OK;
}


// Tile lists from the neighbour CSR (dense == nullptr) or straight from the dense table the CSR would be
// built from (rowptr / nbr unused).  Same lists either way.
static int tile_lists_impl(const uint32_t* mask, const int32_t* rowptr, const int32_t* nbr, const RowArgs* dense,
                           const int32_t* order, int32_t n_rows, int32_t kv, int32_t tile_rows, int32_t identity_stage,
                           int32_t slots, void* workspace, size_t workspace_bytes, int32_t* tile_ptr, int32_t* stage_kp,
                           int32_t* stage_nbr, int32_t stage_cap, cudaStream_t st) {
  if (n_rows < 0 || kv < 1 || kv > 128 || stage_cap < 0 || !tile_ptr) return PCE_ERR_INVALID;
  if (tile_rows != 128 && tile_rows != 256 && tile_rows != 512) return PCE_ERR_INVALID;
  if (slots != 1 && slots != 2 && slots != 4) return PCE_ERR_INVALID;
  if (tile_rows == 512 && slots != 1) return PCE_ERR_INVALID;
  const int n_tiles = div_up(n_rows, tile_rows);
  if (n_tiles == 0) {
    PCE_CUDA(cudaMemsetAsync(tile_ptr, 0, sizeof(int), st));
    return PCE_OK;
  }
  if (!mask || !stage_kp || !stage_nbr) return PCE_ERR_INVALID;
  if (!dense && (!rowptr || !nbr)) return PCE_ERR_INVALID;
  const int words = (kv + 31) / 32;
  Arena ar(workspace, workspace_bytes);
  int* cnt = ar.take<int>(static_cast<size_t>(n_tiles) + 1);
  if (!ar.ok) return PCE_ERR_WORKSPACE;
  k_tile_lists<false><<<n_tiles, tile_rows, 0, st>>>(mask, rowptr, nbr, order, n_rows, words, identity_stage ? 1 : 0, slots,
                                                     cnt, nullptr, nullptr, nullptr, 0);
  PCE_LAUNCH_CHECK();
  if (n_tiles <= (1 << 16)) {
    k_scan_small<<<1, 1024, 0, st>>>(cnt, tile_ptr, n_tiles);
    PCE_LAUNCH_CHECK();
  } else {
    PCE_CUDA(cudaMemsetAsync(cnt + n_tiles, 0, sizeof(int), st));
    PCE_TRY(exclusive_scan_i32(ar, cnt, tile_ptr, n_tiles + 1, st));
  }
  if (dense)
    k_tile_lists<true, true><<<n_tiles, tile_rows, 0, st>>>(mask, nullptr, nullptr, order, n_rows, words, identity_stage ? 1 : 0,
                                                            slots, nullptr, tile_ptr, stage_kp, stage_nbr, stage_cap, *dense);
  else
    k_tile_lists<true><<<n_tiles, tile_rows, 0, st>>>(mask, rowptr, nbr, order, n_rows, words, identity_stage ? 1 : 0, slots,
                                                      nullptr, tile_ptr, stage_kp, stage_nbr, stage_cap);
  PCE_LAUNCH_CHECK();
  return PCE_OK;
}

// The planner's route for one direction of a map with at most 32 offsets: bitmask and row order in one pass over
// the dense table plus the radix sort (no neighbour CSR: the tile lists are filled from the table).
int map_mask_and_order32(const int32_t* table, int kv, int n_rows, int reverse, int identity_kp, const int32_t* knnz,
                         void* workspace, size_t workspace_bytes, uint32_t* mask, int32_t* order, cudaStream_t st) {
  if (kv < 1 || kv > 32 || n_rows < 1 || !table || !knnz || !mask || !order) return PCE_ERR_INVALID;
  Arena ar(workspace, workspace_bytes);
  uint32_t* k32 = ar.take<uint32_t>(n_rows);
  uint32_t* s32 = ar.take<uint32_t>(n_rows);
  int* vals = ar.take<int>(n_rows);
  if (!ar.ok) return PCE_ERR_WORKSPACE;
  RowArgs a{table, kv, n_rows, reverse, identity_kp, nullptr, nullptr, n_rows};
  k_row_mask_key32<<<div_up(n_rows + 1, 256), 256, 0, st>>>(a, knnz, mask, nullptr, k32, vals);
  PCE_LAUNCH_CHECK();
  size_t need = 0;
  PCE_CUDA(cub::DeviceRadixSort::SortPairs(nullptr, need, k32, s32, vals, order, n_rows, 0, kv, st));
  char* tmp = ar.take<char>(need);
  if (!ar.ok) return PCE_ERR_WORKSPACE;
  PCE_CUDA(cub::DeviceRadixSort::SortPairs(tmp, need, k32, s32, vals, order, n_rows, 0, kv, st));
  return PCE_OK;
}

int tile_lists_from_dense(const uint32_t* mask, const int32_t* table, int reverse, int identity_kp, const int32_t* order,
                          int32_t n_rows, int32_t kv, int32_t tile_rows, int32_t identity_stage, int32_t slots,
                          void* workspace, size_t workspace_bytes, int32_t* tile_ptr, int32_t* stage_kp,
                          int32_t* stage_nbr, int32_t stage_cap, cudaStream_t st) {
  if (!table) return PCE_ERR_INVALID;
  const RowArgs a{table, kv, n_rows, reverse, identity_kp, nullptr, nullptr, n_rows};
  return tile_lists_impl(mask, nullptr, nullptr, &a, order, n_rows, kv, tile_rows, identity_stage, slots, workspace,
                         workspace_bytes, tile_ptr, stage_kp, stage_nbr, stage_cap, st);
}

}  // namespace pce

using namespace pce;

extern "C" {

size_t pce_map_workspace_bytes(int32_t n_in, int32_t kv, int32_t n_out_cap) {
  long long n = n_in > n_out_cap ? n_in : n_out_cap;
  if (n < 1) n = 1;
  size_t table = sizeof(Slot) * static_cast<size_t>(table_size_for(n));
  size_t keys = 2 * pad256(sizeof(unsigned long long) * static_cast<size_t>(n));
  size_t dense = 2 * pad256(sizeof(int) * static_cast<size_t>(kv) * static_cast<size_t>(n_in > 0 ? n_in : 1));
  size_t counts = 2 * pad256(sizeof(int) * (static_cast<size_t>(n) + 1));
  size_t cub_tmp = 16ull * static_cast<size_t>(n) + (static_cast<size_t>(kv) * n_in) / 64 + (8u << 20);
  return table + keys + dense + counts + cub_tmp + 4096;
}

int pce_downsample_coords(const int32_t* in_coords, int32_t n_in, const pce_geom* g, void* workspace,
                          size_t workspace_bytes, int32_t* out_coords, int32_t out_cap, int32_t* n_out_host,
                          void* stream) {
  if (!g || !n_out_host || n_in < 0 || out_cap < 0) return PCE_ERR_INVALID;
  if (n_in > 0 && (!in_coords || !out_coords)) return PCE_ERR_INVALID;
  for (int i = 0; i < 3; ++i)
    if (g->ks[i] < 1 || g->stride[i] < 1) return PCE_ERR_INVALID;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  *n_out_host = 0;
  if (n_in == 0) return PCE_OK;
  GeomDev gd = to_dev(g);
  gd.subm = 0;
  Arena ar(workspace, workspace_bytes);
  unsigned tsize = table_size_for(out_cap);
  Slot* table = ar.take<Slot>(tsize);
  unsigned long long* ukeys = ar.take<unsigned long long>(out_cap);
  unsigned long long* skeys = ar.take<unsigned long long>(out_cap);
  int* ctr = ar.take<int>(64);
  if (!ar.ok) return PCE_ERR_WORKSPACE;
  PCE_CUDA(cudaMemsetAsync(table, 0xFF, sizeof(Slot) * tsize, st));
  PCE_CUDA(cudaMemsetAsync(ctr, 0, 3 * sizeof(int), st));
  const KeyBits kb = key_bits_for(gd);
  const int grid = div_up(n_in, 256);
  k_candidates<<<grid, 256, 0, st>>>(reinterpret_cast<const int4*>(in_coords), n_in, gd, kb, table, tsize - 1, ukeys,
                                     out_cap, ctr, ctr + 1, ctr + 2);
  PCE_LAUNCH_CHECK();
  // read back through pinned memory: a copy to pageable memory would make the copy call itself wait
  // (spinning) for the stream, a pinned one returns at once and the wait below sleeps
  static thread_local int* pinned = nullptr;
  if (!pinned) PCE_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&pinned), 64, cudaHostAllocDefault));
  int* host = pinned;
  host[0] = host[1] = host[2] = 0;
  PCE_CUDA(cudaMemcpyAsync(host, ctr, 3 * sizeof(int), cudaMemcpyDeviceToHost, st));
  PCE_TRY(wait_for_stream(st));
  if (host[1] != 0) return host[1];
  int n_out = host[0];
  if (n_out > out_cap) return PCE_ERR_CAPACITY;
  *n_out_host = n_out;
  if (n_out == 0) return PCE_OK;
  int end_bit = kb.sh_b + 1;  // the batch field ends at its highest index seen
  while (end_bit < 64 && (host[2] >> (end_bit - kb.sh_b)) != 0) ++end_bit;
  size_t need = 0;
  PCE_CUDA(cub::DeviceRadixSort::SortKeys(nullptr, need, ukeys, skeys, n_out, 0, end_bit, st));
  char* tmp = ar.take<char>(need);
  if (!ar.ok) return PCE_ERR_WORKSPACE;
  PCE_CUDA(cub::DeviceRadixSort::SortKeys(tmp, need, ukeys, skeys, n_out, 0, end_bit, st));
  k_decode_keys<<<div_up(n_out, 256), 256, 0, st>>>(skeys, n_out, gd, kb, reinterpret_cast<int4*>(out_coords));
  PCE_LAUNCH_CHECK();
  return PCE_OK;
}

int pce_map_build_d2(const int32_t* in_coords, int32_t n_in, const int32_t* out_coords, int32_t n_out,
                     const pce_geom* g, void* workspace, size_t workspace_bytes, int32_t* map, int32_t* knnz,
                     int32_t* kpos, int32_t* qkpos, int32_t* map_out, int32_t* status, void* stream) {
  if (!g || !knnz || !kpos || !qkpos || n_in < 0 || n_out < 0) return PCE_ERR_INVALID;
  if ((n_in > 0 && (!in_coords || !map)) || (n_out > 0 && !out_coords)) return PCE_ERR_INVALID;
  for (int i = 0; i < 3; ++i)
    if (g->ks[i] < 1 || g->stride[i] < 1) return PCE_ERR_INVALID;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  GeomDev gd = to_dev(g);
  if (static_cast<long long>(gd.kv) * n_in >= (1ll << 31)) return PCE_ERR_UNSUPPORTED;
  Arena ar(workspace, workspace_bytes);
  unsigned tsize = table_size_for(n_out);
  Slot* table = ar.take<Slot>(tsize);
  int* st_word = status ? status : ar.take<int>(64);
  if (!ar.ok) return PCE_ERR_WORKSPACE;
  PCE_CUDA(cudaMemsetAsync(knnz, 0, sizeof(int) * gd.kv, st));
  if (!status) PCE_CUDA(cudaMemsetAsync(st_word, 0, sizeof(int), st));
  if (n_in > 0 && n_out > 0) {
    PCE_CUDA(cudaMemsetAsync(table, 0xFF, sizeof(Slot) * tsize, st));
    if (map_out) PCE_CUDA(cudaMemsetAsync(map_out, 0xFF, sizeof(int) * static_cast<size_t>(gd.kv) * n_out, st));
    k_insert_rows<<<div_up(n_out, 256), 256, 0, st>>>(reinterpret_cast<const int4*>(out_coords), n_out, table,
                                                      tsize - 1, st_word);
    PCE_LAUNCH_CHECK();
    PCE_TRY(run_query(in_coords, n_in, gd, table, tsize, map, map_out, n_out, knnz, st_word, st));
  } else if (n_in > 0) {
    PCE_CUDA(cudaMemsetAsync(map, 0xFF, sizeof(int) * static_cast<size_t>(gd.kv) * n_in, st));
  }
  k_offset_scans<<<1, 32, 0, st>>>(knnz, gd.kv, kpos, qkpos);
  PCE_LAUNCH_CHECK();
  return PCE_OK;
}

// ---- allocation-free variant of pce_map_build_d2 -----------------------------------------
// Scratch (hash table + status word) lives in one file-scope device array instead of a
// caller workspace.  2^18 slots of 16 bytes cover 131072 output rows at load <= 0.5; the
// array (4 MiB + 256 B) is part of the module image, so every GPU that loads the library
// holds it until the process exits.
constexpr int kNoAllocMaxRows = 131072;
constexpr unsigned kNoAllocSlots = 262144;
constexpr size_t kNoAllocBytes = sizeof(Slot) * kNoAllocSlots + 256;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

// In host code `g_noalloc_scratch` is only a handle for the symbol, not a device address:
// the address is looked up once per device (with that device current) and kept.
static void* g_noalloc_addr[64] = {};

static int noalloc_scratch_address(void** out) {
  int dev = -1;
  PCE_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return PCE_ERR_UNSUPPORTED;
  void* p = __atomic_load_n(&g_noalloc_addr[dev], __ATOMIC_ACQUIRE);
  if (p == nullptr) {
    PCE_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
    if (p == nullptr) return PCE_ERR_CUDA;
    __atomic_store_n(&g_noalloc_addr[dev], p, __ATOMIC_RELEASE);  // every thread finds the same address
  }
  *out = p;
  return PCE_OK;
}

int pce_map_build_d2_noalloc(const int32_t* in_coords, int32_t n_in, const int32_t* out_coords, int32_t n_out,
                             const pce_geom* g, int32_t* map, int32_t* knnz, int32_t* kpos, int32_t* qkpos,
                             int32_t* map_out, int32_t* status, void* stream) {
  if (!g || !knnz || !kpos || !qkpos || n_in < 0 || n_out < 0) return PCE_ERR_INVALID;
  if ((n_in > 0 && (!in_coords || !map)) || (n_out > 0 && !out_coords)) return PCE_ERR_INVALID;
  for (int i = 0; i < 3; ++i)
    if (g->ks[i] < 1 || g->stride[i] < 1) return PCE_ERR_INVALID;
  if (n_out > kNoAllocMaxRows) return PCE_ERR_CAPACITY;  // the built-in table holds 131072 output rows
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  GeomDev gd = to_dev(g);
  if (static_cast<long long>(gd.kv) * n_in >= (1ll << 31)) return PCE_ERR_UNSUPPORTED;
  void* base = nullptr;
  PCE_TRY(noalloc_scratch_address(&base));
  Slot* table = static_cast<Slot*>(base);
  int* st_word = status ? status : reinterpret_cast<int*>(static_cast<unsigned char*>(base) + sizeof(Slot) * kNoAllocSlots);
  const unsigned tsize = table_size_for(n_out);  // <= kNoAllocSlots by the row limit above
  PCE_CUDA(cudaMemsetAsync(knnz, 0, sizeof(int) * gd.kv, st));
  if (!status) PCE_CUDA(cudaMemsetAsync(st_word, 0, sizeof(int), st));
  if (n_in > 0 && n_out > 0) {
    // the array keeps the previous call's table: every slot this call can probe is emptied first
    PCE_CUDA(cudaMemsetAsync(table, 0xFF, sizeof(Slot) * tsize, st));
    if (map_out) PCE_CUDA(cudaMemsetAsync(map_out, 0xFF, sizeof(int) * static_cast<size_t>(gd.kv) * n_out, st));
    k_insert_rows<<<div_up(n_out, 256), 256, 0, st>>>(reinterpret_cast<const int4*>(out_coords), n_out, table,
                                                      tsize - 1, st_word);
    PCE_LAUNCH_CHECK();
    PCE_TRY(run_query(in_coords, n_in, gd, table, tsize, map, map_out, n_out, knnz, st_word, st));
  } else if (n_in > 0) {
    PCE_CUDA(cudaMemsetAsync(map, 0xFF, sizeof(int) * static_cast<size_t>(gd.kv) * n_in, st));
  }
  k_offset_scans<<<1, 32, 0, st>>>(knnz, gd.kv, kpos, qkpos);
  PCE_LAUNCH_CHECK();
  return PCE_OK;
}

int pce_map_pairs(const int32_t* map, int32_t kv, int32_t n_in, void* workspace, size_t workspace_bytes,
                  int32_t* imap, int32_t* omap, int32_t pair_cap, void* stream) {
  if (kv < 1 || n_in < 0 || pair_cap < 0) return PCE_ERR_INVALID;
  if (n_in == 0 || pair_cap == 0) return PCE_OK;
  if (!map || !imap || !omap) return PCE_ERR_INVALID;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  long long total = static_cast<long long>(kv) * n_in;
  if (total >= (1ll << 31)) return PCE_ERR_UNSUPPORTED;
  Arena ar(workspace, workspace_bytes);
  int* flags = ar.take<int>(total);
  int* rank = ar.take<int>(total);
  if (!ar.ok) return PCE_ERR_WORKSPACE;
  k_flags<<<div_up(total, 256), 256, 0, st>>>(map, total, flags);
  PCE_LAUNCH_CHECK();
  PCE_TRY(exclusive_scan_i32(ar, flags, rank, total, st));
  dim3 grid(div_up(n_in, 256), kv);
  k_emit_pairs<<<grid, 256, 0, st>>>(map, rank, kv, n_in, imap, omap, pair_cap);
  PCE_LAUNCH_CHECK();
  return PCE_OK;
}

int pce_map_build_d1(const int32_t* map, const int32_t* map_out, int32_t kv, int32_t n_in, int32_t n_out,
                     int32_t submanifold, const int32_t* kpos, void* workspace, size_t workspace_bytes,
                     int32_t* imap_coded, int32_t* icsr, int32_t* omap_coded, int32_t* ocsr, void* stream) {
  if (kv < 1 || n_in < 0 || n_out < 0 || !kpos || !icsr || !ocsr) return PCE_ERR_INVALID;
  if (!submanifold && !map_out && n_out > 0) return PCE_ERR_INVALID;
  if (submanifold && n_in != n_out) return PCE_ERR_INVALID;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (n_in == 0 || n_out == 0) {
    PCE_CUDA(cudaMemsetAsync(icsr, 0, sizeof(int) * (n_in + 1), st));
    PCE_CUDA(cudaMemsetAsync(ocsr, 0, sizeof(int) * (n_out + 1), st));
    return PCE_OK;
  }
  if (!map || !imap_coded || !omap_coded) return PCE_ERR_INVALID;
  long long total = static_cast<long long>(kv) * n_in;
  if (total >= (1ll << 31)) return PCE_ERR_UNSUPPORTED;
  Arena ar(workspace, workspace_bytes);
  int* flags = ar.take<int>(total);
  int* rank = ar.take<int>(total);
  int* counts = ar.take<int>(static_cast<size_t>(n_in > n_out ? n_in : n_out) + 1);
  if (!ar.ok) return PCE_ERR_WORKSPACE;
  k_flags<<<div_up(total, 256), 256, 0, st>>>(map, total, flags);
  PCE_LAUNCH_CHECK();
  PCE_TRY(exclusive_scan_i32(ar, flags, rank, total, st));
  const int cap = 0x7FFFFFFF;
  // input-major rows
  RowArgs a{map, kv, n_in, 0, -1, rank, kpos, n_in};
  k_row_count<<<div_up(n_in + 1, 256), 256, 0, st>>>(a, nullptr, counts);
  PCE_LAUNCH_CHECK();
  PCE_TRY(exclusive_scan_i32(ar, counts, icsr, n_in + 1, st));
  k_row_fill<1><<<div_up(n_in, 256), 256, 0, st>>>(a, icsr, imap_coded, cap);
  PCE_LAUNCH_CHECK();
  // output-major rows
  RowArgs b{submanifold ? map : map_out, kv, n_out, submanifold ? 1 : 0, -1, rank, kpos, n_in};
  k_row_count<<<div_up(n_out + 1, 256), 256, 0, st>>>(b, nullptr, counts);
  PCE_LAUNCH_CHECK();
  PCE_TRY(exclusive_scan_i32(ar, counts, ocsr, n_out + 1, st));
  k_row_fill<2><<<div_up(n_out, 256), 256, 0, st>>>(b, ocsr, omap_coded, cap);
  PCE_LAUNCH_CHECK();
  return PCE_OK;
}

int pce_csr_from_dense(const int32_t* table, int32_t kv, int32_t n_rows, int32_t reverse_kp, int32_t identity_kp,
                       void* workspace, size_t workspace_bytes, uint32_t* mask, int32_t* rowptr, int32_t* nbr,
                       int32_t nbr_cap, void* stream) {
  if (kv < 1 || n_rows < 0 || !rowptr || nbr_cap < 0) return PCE_ERR_INVALID;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (n_rows == 0) {
    PCE_CUDA(cudaMemsetAsync(rowptr, 0, sizeof(int), st));
    return PCE_OK;
  }
  if (!table || !mask || !nbr) return PCE_ERR_INVALID;
  Arena ar(workspace, workspace_bytes);
  int* counts = ar.take<int>(static_cast<size_t>(n_rows) + 1);
  if (!ar.ok) return PCE_ERR_WORKSPACE;
  RowArgs a{table, kv, n_rows, reverse_kp, identity_kp, nullptr, nullptr, n_rows};
  k_row_count<<<div_up(n_rows + 1, 256), 256, 0, st>>>(a, mask, counts);
  PCE_LAUNCH_CHECK();
  PCE_TRY(exclusive_scan_i32(ar, counts, rowptr, n_rows + 1, st));
  k_row_fill<0><<<div_up(n_rows, 256), 256, 0, st>>>(a, rowptr, nbr, nbr_cap);
  PCE_LAUNCH_CHECK();
  return PCE_OK;
}

int pce_csr_sort_rows(const uint32_t* mask, int32_t n_rows, int32_t kv, void* workspace, size_t workspace_bytes,
                      int32_t* order, void* stream) {
  if (n_rows < 0 || kv < 1 || kv > 128) return PCE_ERR_INVALID;
  if (n_rows == 0) return PCE_OK;
  if (!mask || !order) return PCE_ERR_INVALID;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int words = (kv + 31) / 32;
  const bool two = kv > 64;  // the key needs a second 64-bit word
  Arena ar(workspace, workspace_bytes);
  unsigned long long* lo = ar.take<unsigned long long>(n_rows);
  unsigned long long* sorted = ar.take<unsigned long long>(n_rows);
  unsigned long long* hi = two ? ar.take<unsigned long long>(n_rows) : nullptr;
  unsigned long long* hi_by_lo = two ? ar.take<unsigned long long>(n_rows) : nullptr;
  int* vals = ar.take<int>(n_rows);
  int* by_lo = two ? ar.take<int>(n_rows) : order;
  int* counts = ar.take<int>(128);
  if (!ar.ok) return PCE_ERR_WORKSPACE;
  PCE_CUDA(cudaMemsetAsync(counts, 0, 128 * sizeof(int), st));
  k_offset_counts<<<div_up(n_rows, 256), 256, 0, st>>>(mask, n_rows, words, counts);
  PCE_LAUNCH_CHECK();
  if (kv <= 32) {
    // the key fits 32 bits (3x3x3 and 2x2x2 kernels): same order, half the bytes per radix pass
    uint32_t* k32 = reinterpret_cast<uint32_t*>(lo);
    uint32_t* s32 = reinterpret_cast<uint32_t*>(sorted);
    k_mask_keys32<<<div_up(n_rows, 256), 256, 0, st>>>(mask, n_rows, kv, counts, k32, vals);
    PCE_LAUNCH_CHECK();
    int begin = 0;
    if (kmap_sort_top_bits > 0 && kmap_sort_top_bits < kv) begin = kv - kmap_sort_top_bits;
    size_t need32 = 0;
    PCE_CUDA(cub::DeviceRadixSort::SortPairs(nullptr, need32, k32, s32, vals, order, n_rows, begin, kv, st));
    char* tmp32 = ar.take<char>(need32);
    if (!ar.ok) return PCE_ERR_WORKSPACE;
    PCE_CUDA(cub::DeviceRadixSort::SortPairs(tmp32, need32, k32, s32, vals, order, n_rows, begin, kv, st));
    return PCE_OK;
  }
  k_mask_keys<<<div_up(n_rows, 256), 256, 0, st>>>(mask, n_rows, words, kv, counts, lo, hi, vals);
  PCE_LAUNCH_CHECK();
  // least significant word first; the radix sort is stable, so the second pass keeps its order
  const int lo_bits = kv < 64 ? kv : 64;
  // The key's low bits are the COMMON offsets (bit kv-1-rank, rank 0 = rarest): most rows of a tile
  // have them whatever the order, so the sort may leave them out (kmap_sort_top_bits > 0: only that
  // many of the most significant bits are sorted on; one radix pass per 8 bits).
  int lo_begin = 0;
  if (!two && kmap_sort_top_bits > 0 && kmap_sort_top_bits < lo_bits) lo_begin = lo_bits - kmap_sort_top_bits;
  size_t need = 0, need_hi = 0;
  PCE_CUDA(cub::DeviceRadixSort::SortPairs(nullptr, need, lo, sorted, vals, by_lo, n_rows, lo_begin, lo_bits, st));
  if (two) {
    PCE_CUDA(cub::DeviceRadixSort::SortPairs(nullptr, need_hi, hi_by_lo, sorted, by_lo, order, n_rows, 0, kv - 64, st));
    if (need_hi > need) need = need_hi;
  }
  char* tmp = ar.take<char>(need);
  if (!ar.ok) return PCE_ERR_WORKSPACE;
  PCE_CUDA(cub::DeviceRadixSort::SortPairs(tmp, need, lo, sorted, vals, by_lo, n_rows, lo_begin, lo_bits, st));
  if (two) {
    k_gather_u64<<<div_up(n_rows, 256), 256, 0, st>>>(hi, by_lo, n_rows, hi_by_lo);
    PCE_LAUNCH_CHECK();
    PCE_CUDA(cub::DeviceRadixSort::SortPairs(tmp, need, hi_by_lo, sorted, by_lo, order, n_rows, 0, kv - 64, st));
  }
  return PCE_OK;
}

int pce_build_tile_lists(const uint32_t* mask, const int32_t* rowptr, const int32_t* nbr, const int32_t* order,
                         int32_t n_rows, int32_t kv, int32_t tile_rows, int32_t identity_stage, int32_t slots,
                         void* workspace, size_t workspace_bytes, int32_t* tile_ptr, int32_t* stage_kp,
                         int32_t* stage_nbr, int32_t stage_cap, void* stream) {
  return tile_lists_impl(mask, rowptr, nbr, nullptr, order, n_rows, kv, tile_rows, identity_stage, slots, workspace,
                         workspace_bytes, tile_ptr, stage_kp, stage_nbr, stage_cap, static_cast<cudaStream_t>(stream));
}

size_t pce_csr_from_pairs_workspace_bytes(int32_t n_pairs, int32_t n_rows) {
  size_t total = static_cast<size_t>(n_pairs > 0 ? n_pairs : 0) + static_cast<size_t>(n_rows > 0 ? n_rows : 0) + 1;
  return 4 * pad256(sizeof(int) * total) + pad256(sizeof(int) * (static_cast<size_t>(n_rows) + 1)) +
         16 * total + (8u << 20);
}

int pce_csr_from_pairs(const int32_t* rows, const int32_t* nbrs, const int32_t* kpos, int32_t kv, int32_t n_pairs,
                       int32_t n_rows, int32_t identity_kp, void* workspace, size_t workspace_bytes,
                       uint32_t* mask, int32_t* rowptr, int32_t* nbr, int32_t nbr_cap, void* stream) {
  if (kv < 1 || n_pairs < 0 || n_rows < 0 || !rowptr || !kpos) return PCE_ERR_INVALID;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (n_rows == 0) {
    PCE_CUDA(cudaMemsetAsync(rowptr, 0, sizeof(int), st));
    return PCE_OK;
  }
  if (!mask || !nbr || (n_pairs > 0 && (!rows || !nbrs))) return PCE_ERR_INVALID;
  const int total = n_pairs + (identity_kp >= 0 ? n_rows : 0);
  if (nbr_cap < total) return PCE_ERR_CAPACITY;
  const int words = (kv + 31) / 32;
  Arena ar(workspace, workspace_bytes);
  int* keys = ar.take<int>(total + 1);
  int* vals = ar.take<int>(total + 1);
  int* skeys = ar.take<int>(total + 1);
  int* svals = ar.take<int>(total + 1);
  int* counts = ar.take<int>(static_cast<size_t>(n_rows) + 1);
  if (!ar.ok) return PCE_ERR_WORKSPACE;
  PCE_CUDA(cudaMemsetAsync(mask, 0, sizeof(uint32_t) * static_cast<size_t>(n_rows) * words, st));
  PCE_CUDA(cudaMemsetAsync(counts, 0, sizeof(int) * (static_cast<size_t>(n_rows) + 1), st));
  if (total > 0) {
    k_pairs_keys<<<div_up(total, 256), 256, 0, st>>>(rows, kpos, n_pairs, n_rows, identity_kp, keys, vals);
    PCE_LAUNCH_CHECK();
    int bits = 1;
    while ((1ll << bits) < n_rows) ++bits;
    size_t need = 0;
    PCE_CUDA(cub::DeviceRadixSort::SortPairs(nullptr, need, keys, skeys, vals, svals, total, 0, bits, st));
    char* tmp = ar.take<char>(need);
    if (!ar.ok) return PCE_ERR_WORKSPACE;
    PCE_CUDA(cub::DeviceRadixSort::SortPairs(tmp, need, keys, skeys, vals, svals, total, 0, bits, st));
    k_pairs_rows<<<div_up(total, 256), 256, 0, st>>>(skeys, svals, nbrs, kpos, kv, n_pairs, n_rows, identity_kp,
                                                     mask, counts, nbr, nbr_cap);
    PCE_LAUNCH_CHECK();
  }
  PCE_TRY(exclusive_scan_i32(ar, counts, rowptr, n_rows + 1, st));
  return PCE_OK;
}

}  // extern "C"
