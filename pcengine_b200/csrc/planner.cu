// Kernel-map planner: builds every kernel map of a network pass on host threads of its own,
// which feed CUDA streams of their own, while the calling thread queues the feature kernels.
//
// Why: a kernel map is ~30 short launches (hash insert, query, scans, radix passes, tile lists)
// and, for a strided layer, one size read back to the host.  Queued lazily by the layer that
// first needs the map, they leave the GPU waiting for the host: on the LiDAR benchmark the host
// needed 7.7 ms to queue a pass of which 6 ms were map construction, against 5.4 ms of feature
// kernels.  Maps depend on coordinates only, so nothing forces them onto the feature stream.
//
// The reference builds each map inside the first convolution that uses it
// (script/spconv.py:338-427) and keeps it in the tensor's `kmaps` dictionary; the planner
// produces the same maps (same entry points as the lazy path, so bit-identical) ahead of time.
//
// Lanes: a map needs the coordinates of its level(s) and nothing else, so only the chain of
// down-sampled coordinates is sequential.  Lane 0 runs that chain (each step reads one size back
// and therefore synchronises lane 0's stream only); the map lanes take the maps in first-use
// order, wait on the host until the levels they read exist, make their stream wait for the
// level's event and queue hash / query / CSR / row order / tile lists.  One lane alone was
// measured launch-bound: 400 launches in 3.3 ms for a 5-level network whose convolutions wait
// for them.
//
// Memory: a pass owns a device arena (bump allocation over cudaMalloc'ed chunks, recycled with
// the pass object); transient workspaces come from one grow-only scratch buffer per lane, which
// is safe because a lane's kernels all run on its one stream.  Ordering against the caller:
// pce_plan_begin records an event on the stream that produced the coordinates and every lane
// waits for it; pce_pass_release records an event on the stream that read the maps and the
// lanes of the pass that recycles the arena wait for that one.  Nothing else ties the planner
// to the feature stream, so the maps of pass i+1 are built while pass i still computes.
#include <condition_variable>
#include <chrono>
#include <deque>
#include <mutex>
#include <thread>
#include <vector>

#include "common.cuh"

namespace pce {

bool conv_umma_supported(int cin, int cout, int dtype);
size_t conv_split_scratch_bytes(int n_rows, int n_src, int cin, int cout, int kv, int sm_count);
int conv_umma(const void* in, int n_in, const void* wpacked, int kv, const pce_tile_lists* tiles, int n_out, int cin,
              int cout, void* out, const pce_epilogue* ep, cudaStream_t st);
int map_mask_and_order32(const int32_t* table, int kv, int n_rows, int reverse, int identity_kp, const int32_t* knnz,
                         void* workspace, size_t workspace_bytes, uint32_t* mask, int32_t* order, cudaStream_t st);
int tile_lists_from_dense(const uint32_t* mask, const int32_t* table, int reverse, int identity_kp, const int32_t* order,
                          int32_t n_rows, int32_t kv, int32_t tile_rows, int32_t identity_stage, int32_t slots,
                          void* workspace, size_t workspace_bytes, int32_t* tile_ptr, int32_t* stage_kp,
                          int32_t* stage_nbr, int32_t stage_cap, cudaStream_t st);

struct DeviceArena {
  struct Chunk {
    char* base;
    size_t cap, used;
  };
  std::vector<Chunk> chunks;
  size_t cur = 0;
  int error = PCE_OK;

  void reset() {
    for (auto& c : chunks) c.used = 0;
    cur = 0;
    error = PCE_OK;
  }
  void* take(size_t bytes) {
    bytes = pad256(bytes ? bytes : 1);
    while (cur < chunks.size()) {
      Chunk& c = chunks[cur];
      if (c.cap - c.used >= bytes) {
        void* p = c.base + c.used;
        c.used += bytes;
        return p;
      }
      ++cur;
    }
    const size_t cap = bytes > (size_t(256) << 20) ? bytes : (size_t(256) << 20);
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, cap);
    if (e != cudaSuccess) {
      error = cuda_fail(e);
      return nullptr;
    }
    chunks.push_back(Chunk{static_cast<char*>(p), cap, bytes});
    cur = chunks.size() - 1;
    return p;
  }
  template <typename T>
  T* take_n(size_t count) {
    return static_cast<T*>(take(count * sizeof(T)));
  }
  void release() {
    for (auto& c : chunks) cudaFree(c.base);
    chunks.clear();
  }
};

struct LevelState {
  const int32_t* coords = nullptr;
  int32_t n = 0;
  int32_t cmax[3] = {0, 0, 0};
  cudaEvent_t ev = nullptr;  // recorded once the coordinates are written (levels >= 1)
  int ready = 0;             // host side: n is known, ev is recorded (guarded by plan->m)
};

constexpr int kMapLanes = 2;
constexpr int kLanes = 1 + kMapLanes;

}  // namespace pce

using namespace pce;

struct pce_pass {
  pce_plan* plan = nullptr;
  std::mutex arena_m;
  DeviceArena arena;
  int32_t cmin[3] = {0, 0, 0};
  cudaEvent_t start = nullptr;
  cudaEvent_t released = nullptr;          // recorded at release on the stream that read the maps
  bool has_released = false;
  std::vector<LevelState> levels;          // [0] = the input
  std::vector<cudaEvent_t> ready;          // one per map
  std::vector<pce_planned_map> maps;
  // guarded by plan->m
  std::vector<int> queued;
  int next_map = 0;
  int lanes_done = 0;
  int error = PCE_OK;
  bool finished = false;

  void* take(size_t bytes) {
    std::lock_guard<std::mutex> lk(arena_m);
    return arena.take(bytes);
  }
  template <typename T>
  T* take_n(size_t count) {
    return static_cast<T*>(take(count * sizeof(T)));
  }
};

struct PlanLane {
  cudaStream_t stream = nullptr;
  void* scratch = nullptr;
  size_t scratch_cap = 0;
  std::deque<pce_pass*> queue;  // guarded by plan->m
  std::thread thread;
};

struct pce_plan {
  std::vector<pce_plan_map_spec> specs;
  std::vector<int> out_level;  // per spec: the level its outputs live on
  int n_levels = 1;
  int device = 0;
  int sm_count = 148;
  PlanLane lanes[kLanes];
  std::mutex m;
  std::condition_variable cv;
  std::deque<pce_pass*> idle;  // released passes (arena + events), oldest first
  int n_passes = 0;            // pass objects created so far
  bool stop = false;
};

namespace pce {

// 1: maps of at most 32 offsets whose uses all run on tile lists are planned without their neighbour CSR (build_csr);
// 0: every map gets its CSR first and the lists from it (same lists).
int plan_short_route = 1;

static int scratch_for(PlanLane* l, size_t bytes, void** out) {
  if (bytes > l->scratch_cap) {
    PCE_CUDA(cudaStreamSynchronize(l->stream));  // nothing queued may still use the old buffer
    if (l->scratch) PCE_CUDA(cudaFree(l->scratch));
    l->scratch = nullptr;
    l->scratch_cap = 0;
    const size_t cap = pad256(bytes + bytes / 4);
    PCE_CUDA(cudaMalloc(&l->scratch, cap));
    l->scratch_cap = cap;
  }
  *out = l->scratch;
  return PCE_OK;
}

// Rows per tile of the tile lists = 128 x the sub-tiles that share every staged weight block.
// Measured on B200 (LiDAR layers, kernel-only): taller tiles lose from 64 input channels up, on both
// kernels.  One-accumulator kernel, 486k rows: C=96 146 -> 168 us, C=256 169 -> 205 us with 256 rows.
// Several accumulators per CTA with decoupled row / weight rings (k_conv_umma_mt), 128 / 256 / 512 rows:
// C=96 486k rows 121 / 184 / 201 us, C=128 149k rows 92 / 150 / 143 us, C=256 63k rows 115 / 156 us: what
// the fused kernel needs is many independent gather -> multiply chains per SM (CTAs), and a CTA that owns
// all of an SM's tensor memory is one chain whose sub-tiles advance in lock step.  So 128 rows, except
// for layers with 16 or 32 input channels and narrow outputs on large maps (C=32: 72 -> 67 us with 256).
static int tile_rows_policy(int n_rows, int c_in, int c_out, int sm_count) {
  const int cin_p = (c_in + 15) / 16 * 16, cout_p = (c_out + 15) / 16 * 16;
  if ((cin_p == 16 || cin_p == 32) && cout_p <= 32 && static_cast<long long>(n_rows) >= 6ll * 256 * sm_count) return 256;
  return 128;
}

static void fill_geom(const pce_plan_map_spec& sp, const int32_t* cmin, const int32_t* cmax_out, pce_geom* g) {
  for (int d = 0; d < 3; ++d) {
    g->ks[d] = sp.ks[d];
    g->stride[d] = sp.stride[d];
    g->pad[d] = sp.pad[d];
    g->cmin[d] = cmin[d];
    g->cmax[d] = cmax_out[d];
  }
  g->submanifold = sp.submanifold ? 1 : 0;
}

// One direction of a map: bitmask, row order and the requested tile lists.  Maps of at most 32 offsets whose
// uses all run on tile lists take the short route: one pass over the dense table gives bitmask and sort key (the
// rarity of an offset is its knnz), the lists are filled from the table, and the neighbour CSR (rowptr / nbr) is
// left to whoever asks for it (pce_csr_from_dense on the fields kept in the record).  Every other map gets the
// CSR first and the lists from it.  The lists are the same either way.
static int build_csr(pce_plan* p, PlanLane* l, pce_pass* ps, const int32_t* table, int kv, int n_rows, int n_src, int reverse,
                     int ident, size_t nbr_cap, const int32_t* c_outs, const int32_t* c_ins, int identity_stage,
                     const int32_t* knnz, pce_planned_csr* out) {
  cudaStream_t st = l->stream;
  const int words = (kv + 31) / 32;
  // the distinct (tile height, offsets per stage) among the uses
  int want_rows[PCE_PLAN_MAX_USES], want_slots[PCE_PLAN_MAX_USES], n_want = 0;
  for (int u = 0; u < PCE_PLAN_MAX_USES && c_outs[u] > 0; ++u) {
    const int rows = tile_rows_policy(n_rows, c_ins[u], c_outs[u], p->sm_count);
    const int slots = c_ins[u] == 32 ? 2 : (c_ins[u] == 16 ? 4 : 1);
    bool seen = false;
    for (int v = 0; v < n_want; ++v) seen = seen || (want_rows[v] == rows && want_slots[v] == slots);
    if (!seen) {
      want_rows[n_want] = rows;
      want_slots[n_want] = slots;
      ++n_want;
    }
  }
  const bool lists_wanted = n_want > 0 && kv <= 128 && n_rows > 0;
  const bool short_route = lists_wanted && kv <= 32 && plan_short_route;
  uint32_t* mask = ps->take_n<uint32_t>(static_cast<size_t>(n_rows > 0 ? n_rows : 1) * words);
  if (!mask) return ps->arena.error ? ps->arena.error : PCE_ERR_CUDA;
  out->mask = mask;
  out->rowptr = nullptr;
  out->nbr = nullptr;
  out->n_rows = n_rows;
  out->n_src = n_src;
  out->nbr_cap = static_cast<int32_t>(nbr_cap);
  out->n_lists = 0;
  out->table = table;
  out->reverse_kp = reverse;
  out->identity_kp = ident;
  void* ws = nullptr;
  int32_t* rowptr = nullptr;
  int32_t* nbr = nullptr;
  if (!short_route) {
    rowptr = ps->take_n<int32_t>(static_cast<size_t>(n_rows) + 1);
    nbr = ps->take_n<int32_t>(nbr_cap);
    if (!rowptr || !nbr) return ps->arena.error ? ps->arena.error : PCE_ERR_CUDA;
    PCE_TRY(scratch_for(l, 8 * (static_cast<size_t>(n_rows) + 1) + (8u << 20), &ws));
    PCE_TRY(pce_csr_from_dense(table, kv, n_rows, reverse, ident, ws, l->scratch_cap, mask, rowptr, nbr,
                               static_cast<int32_t>(nbr_cap), st));
    out->rowptr = rowptr;
    out->nbr = nbr;
  }
  if (!lists_wanted) return PCE_OK;
  int32_t* order = ps->take_n<int32_t>(n_rows);
  if (!order) return ps->arena.error ? ps->arena.error : PCE_ERR_CUDA;
  PCE_TRY(scratch_for(l, 64 * static_cast<size_t>(n_rows) + (16u << 20), &ws));
  if (short_route)
    PCE_TRY(map_mask_and_order32(table, kv, n_rows, reverse, ident, knnz, ws, l->scratch_cap, mask, order, st));
  else
    PCE_TRY(pce_csr_sort_rows(mask, n_rows, kv, ws, l->scratch_cap, order, st));
  for (int h = 0; h < n_want; ++h) {
    const int rows = want_rows[h], slots = want_slots[h];
    const int n_tiles = div_up(n_rows, rows);
    const size_t cap = static_cast<size_t>(n_tiles) * ((kv + slots - 1) / slots + (identity_stage ? 1 : 0));
    int32_t* tile_ptr = ps->take_n<int32_t>(static_cast<size_t>(n_tiles) + 1);
    int32_t* stage_kp = ps->take_n<int32_t>(cap * slots);
    int32_t* stage_nbr = ps->take_n<int32_t>(cap * slots * rows);
    if (!tile_ptr || !stage_kp || !stage_nbr) return ps->arena.error ? ps->arena.error : PCE_ERR_CUDA;
    PCE_TRY(scratch_for(l, 8 * (static_cast<size_t>(n_tiles) + 1) + (1u << 20), &ws));
    if (short_route)
      PCE_TRY(tile_lists_from_dense(mask, table, reverse, ident, order, n_rows, kv, rows, identity_stage, slots, ws,
                                    l->scratch_cap, tile_ptr, stage_kp, stage_nbr, static_cast<int32_t>(cap), st));
    else
      PCE_TRY(pce_build_tile_lists(mask, rowptr, nbr, order, n_rows, kv, rows, identity_stage, slots, ws, l->scratch_cap,
                                   tile_ptr, stage_kp, stage_nbr, static_cast<int32_t>(cap), st));
    out->lists[out->n_lists++] = pce_tile_lists{order, tile_ptr, stage_kp, stage_nbr, rows, identity_stage, slots, 1};
  }
  return PCE_OK;
}

// Lane 0: the output coordinates of every strided spec, in order.
static int run_coords_lane(pce_plan* p, PlanLane* l, pce_pass* ps) {
  PCE_CUDA(cudaStreamWaitEvent(l->stream, ps->start, 0));
  if (ps->has_released) PCE_CUDA(cudaStreamWaitEvent(l->stream, ps->released, 0));
  for (size_t i = 0; i < p->specs.size(); ++i) {
    const pce_plan_map_spec& sp = p->specs[i];
    if (sp.submanifold) continue;
    const LevelState in = ps->levels[sp.in_level];  // produced by this lane (or the input): no wait needed
    LevelState& lv = ps->levels[p->out_level[i]];
    int32_t cmax_out[3];
    for (int d = 0; d < 3; ++d) cmax_out[d] = (in.cmax[d] + 2 * sp.pad[d] - (sp.ks[d] - 1)) / sp.stride[d];
    pce_geom g;
    fill_geom(sp, ps->cmin, cmax_out, &g);
    const int kv = sp.ks[0] * sp.ks[1] * sp.ks[2];
    long long per_input = 1;
    for (int d = 0; d < 3; ++d) per_input *= (sp.ks[d] + sp.stride[d] - 1) / sp.stride[d];
    const long long cap = in.n * per_input > 1 ? in.n * per_input : 1;
    if (cap >= (1ll << 31)) return PCE_ERR_UNSUPPORTED;
    int32_t* oc = ps->take_n<int32_t>(static_cast<size_t>(cap) * 4);
    if (!oc) return ps->arena.error ? ps->arena.error : PCE_ERR_CUDA;
    void* ws = nullptr;
    PCE_TRY(scratch_for(l, pce_map_workspace_bytes(in.n, kv, static_cast<int32_t>(cap)), &ws));
    int32_t n_out = 0;
    PCE_TRY(pce_downsample_coords(in.coords, in.n, &g, ws, l->scratch_cap, oc, static_cast<int32_t>(cap), &n_out, l->stream));
    PCE_CUDA(cudaEventRecord(lv.ev, l->stream));
    {
      std::lock_guard<std::mutex> lk(p->m);
      lv.coords = oc;
      lv.n = n_out;
      for (int d = 0; d < 3; ++d) lv.cmax[d] = cmax_out[d];
      lv.ready = 1;
    }
    p->cv.notify_all();
  }
  return PCE_OK;
}

// Copies a level once it exists on the host side; false when the pass failed meanwhile.
static bool wait_level(pce_plan* p, pce_pass* ps, int level, LevelState* out) {
  std::unique_lock<std::mutex> lk(p->m);
  p->cv.wait(lk, [&] { return ps->levels[level].ready != 0 || ps->error != PCE_OK; });
  if (ps->error != PCE_OK) return false;
  *out = ps->levels[level];
  return true;
}

static int build_map(pce_plan* p, PlanLane* l, pce_pass* ps, int i) {
  const pce_plan_map_spec& sp = p->specs[i];
  cudaStream_t st = l->stream;
  LevelState in, outl;
  if (!wait_level(p, ps, sp.in_level, &in)) return PCE_OK;  // the failing lane reports the error
  if (!wait_level(p, ps, p->out_level[i], &outl)) return PCE_OK;
  if (in.ev) PCE_CUDA(cudaStreamWaitEvent(st, in.ev, 0));
  if (outl.ev && outl.ev != in.ev) PCE_CUDA(cudaStreamWaitEvent(st, outl.ev, 0));
  pce_planned_map& out = ps->maps[i];
  pce_geom g;
  fill_geom(sp, ps->cmin, outl.cmax, &g);
  const int kv = sp.ks[0] * sp.ks[1] * sp.ks[2];
  const bool odd = (sp.ks[0] % 2 == 1) && (sp.ks[1] % 2 == 1) && (sp.ks[2] % 2 == 1);
  for (int d = 0; d < 3; ++d) out.cmax_out[d] = outl.cmax[d];
  const int n_in = in.n, n_out = outl.n;
  const bool symmetric = sp.submanifold && odd;
  int32_t* map = ps->take_n<int32_t>(static_cast<size_t>(kv) * (n_in > 0 ? n_in : 1));
  int32_t* map_out = symmetric ? nullptr : ps->take_n<int32_t>(static_cast<size_t>(kv) * (n_out > 0 ? n_out : 1));
  int32_t* small = ps->take_n<int32_t>(3 * static_cast<size_t>(kv) + 3 + 64);
  if (!map || !small || (!symmetric && !map_out)) return ps->arena.error ? ps->arena.error : PCE_ERR_CUDA;
  int32_t* knnz = small;
  int32_t* kpos = small + kv;
  int32_t* qkpos = kpos + kv + 1;
  int32_t* status = qkpos + kv + 1;
  PCE_CUDA(cudaMemsetAsync(status, 0, sizeof(int32_t), st));
  void* ws = nullptr;
  PCE_TRY(scratch_for(l, pce_map_workspace_bytes(n_in, kv, n_out), &ws));
  PCE_TRY(pce_map_build_d2(in.coords, n_in, outl.coords, n_out, &g, ws, l->scratch_cap, map, knnz, kpos, qkpos, map_out,
                           status, st));
  out.n_in = n_in;
  out.n_out = n_out;
  out.kv = kv;
  out.symmetric = symmetric ? 1 : 0;
  out.in_coords = in.coords;
  out.out_coords = outl.coords;
  out.map = map;
  out.map_out = map_out;
  out.knnz = knnz;
  out.kpos = kpos;
  out.qkpos = qkpos;
  out.status = status;
  out.has_fwd = 0;
  out.has_tr = 0;
  const int ident = sp.submanifold ? ((sp.ks[0] - 1) / 2 * sp.ks[1] * sp.ks[2] + (sp.ks[1] - 1) / 2 * sp.ks[2] + (sp.ks[2] - 1) / 2)
                                   : -1;
  const int n_min = n_in < n_out ? n_in : n_out;
  const size_t cap_nbr = static_cast<size_t>(kv) * (sp.submanifold ? (n_in > 0 ? n_in : 1) : (n_min > 0 ? n_min : 1));
  if (cap_nbr >= (size_t(1) << 31)) return PCE_ERR_UNSUPPORTED;
  if (sp.want_fwd) {
    // output-major table: the map itself read with kp reversed when symmetric, else map_out
    // residual blocks live on submanifold maps: their lists carry the identity stage
    PCE_TRY(build_csr(p, l, ps, symmetric ? map : map_out, kv, n_out, n_in, symmetric ? 1 : 0, ident, cap_nbr,
                      sp.c_out_fwd, sp.c_in_fwd, sp.submanifold ? 1 : 0, knnz, &out.fwd));
    out.has_fwd = 1;
  }
  if (sp.want_tr) {
    // roles swapped: the input-major table is the output-major one of the transposed layer
    PCE_TRY(build_csr(p, l, ps, map, kv, n_in, n_out, 0, ident, cap_nbr, sp.c_out_tr, sp.c_in_tr, 0, knnz, &out.tr));
    out.has_tr = 1;
  }
  PCE_CUDA(cudaEventRecord(ps->ready[i], st));
  {
    std::lock_guard<std::mutex> lk(p->m);
    ps->queued[i] = 1;
  }
  p->cv.notify_all();
  return PCE_OK;
}

// Map lanes: take the next map in first-use order until none is left.
static int run_map_lane(pce_plan* p, PlanLane* l, pce_pass* ps) {
  PCE_CUDA(cudaStreamWaitEvent(l->stream, ps->start, 0));
  if (ps->has_released) PCE_CUDA(cudaStreamWaitEvent(l->stream, ps->released, 0));
  for (;;) {
    int i;
    {
      std::lock_guard<std::mutex> lk(p->m);
      if (ps->error != PCE_OK) return PCE_OK;
      i = ps->next_map++;
    }
    if (i >= static_cast<int>(p->specs.size())) return PCE_OK;
    PCE_TRY(build_map(p, l, ps, i));
  }
}

static void lane_main(pce_plan* p, int lane) {
  cudaSetDevice(p->device);
  PlanLane* l = &p->lanes[lane];
  for (;;) {
    pce_pass* ps = nullptr;
    {
      std::unique_lock<std::mutex> lk(p->m);
      p->cv.wait(lk, [&] { return p->stop || !l->queue.empty(); });
      if (l->queue.empty()) return;  // stop requested and nothing left
      ps = l->queue.front();
      l->queue.pop_front();
    }
    const int status = lane == 0 ? run_coords_lane(p, l, ps) : run_map_lane(p, l, ps);
    {
      std::lock_guard<std::mutex> lk(p->m);
      if (status != PCE_OK && ps->error == PCE_OK) ps->error = status;
      if (++ps->lanes_done == kLanes) ps->finished = true;
    }
    p->cv.notify_all();
  }
}

}  // namespace pce

extern "C" {

int32_t pce_tile_rows_for(int32_t n_rows, int32_t c_in, int32_t c_out, int32_t sm_count) {
  return tile_rows_policy(n_rows, c_in, c_out, sm_count > 0 ? sm_count : 148);
}

static void free_pass(pce_pass* ps) {
  ps->arena.release();
  if (ps->start) cudaEventDestroy(ps->start);
  if (ps->released) cudaEventDestroy(ps->released);
  for (cudaEvent_t ev : ps->ready)
    if (ev) cudaEventDestroy(ev);
  for (LevelState& lv : ps->levels)
    if (lv.ev) cudaEventDestroy(lv.ev);
  delete ps;
}

int pce_plan_create(const pce_plan_map_spec* specs, int32_t n_specs, pce_plan** out) {
  if (!specs || n_specs < 1 || !out) return PCE_ERR_INVALID;
  int levels = 1;
  std::vector<int> out_level;
  for (int i = 0; i < n_specs; ++i) {
    const pce_plan_map_spec& s = specs[i];
    for (int d = 0; d < 3; ++d)
      if (s.ks[d] < 1 || s.stride[d] < 1 || s.pad[d] < 0) return PCE_ERR_INVALID;
    if (s.in_level < 0 || s.in_level >= levels) return PCE_ERR_INVALID;
    out_level.push_back(s.submanifold ? s.in_level : levels);
    if (!s.submanifold) ++levels;
  }
  pce_plan* p = new pce_plan();
  p->specs.assign(specs, specs + n_specs);
  p->out_level = out_level;
  p->n_levels = levels;
  cudaError_t e = cudaGetDevice(&p->device);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&p->sm_count, cudaDevAttrMultiProcessorCount, p->device);
  for (int l = 0; l < kLanes && e == cudaSuccess; ++l)
    e = cudaStreamCreateWithFlags(&p->lanes[l].stream, cudaStreamNonBlocking);
  if (e != cudaSuccess) {
    for (int l = 0; l < kLanes; ++l)
      if (p->lanes[l].stream) cudaStreamDestroy(p->lanes[l].stream);
    delete p;
    return cuda_fail(e);
  }
  for (int l = 0; l < kLanes; ++l) p->lanes[l].thread = std::thread(lane_main, p, l);
  *out = p;
  return PCE_OK;
}

void pce_plan_destroy(pce_plan* p) {
  if (!p) return;
  {
    std::lock_guard<std::mutex> lk(p->m);
    p->stop = true;
  }
  p->cv.notify_all();
  for (int l = 0; l < kLanes; ++l)
    if (p->lanes[l].thread.joinable()) p->lanes[l].thread.join();
  int prev = -1;
  cudaGetDevice(&prev);
  cudaSetDevice(p->device);
  for (int l = 0; l < kLanes; ++l) cudaStreamSynchronize(p->lanes[l].stream);
  for (pce_pass* ps : p->idle) free_pass(ps);
  for (int l = 0; l < kLanes; ++l) {
    if (p->lanes[l].scratch) cudaFree(p->lanes[l].scratch);
    cudaStreamDestroy(p->lanes[l].stream);
  }
  if (prev >= 0) cudaSetDevice(prev);
  delete p;
}

int pce_plan_begin(pce_plan* p, const int32_t* coords, int32_t n, const int32_t* cmin, const int32_t* cmax, void* stream,
                   pce_pass** out) {
  if (!p || !coords || n < 1 || !cmin || !cmax || !out) return PCE_ERR_INVALID;
  int dev = -1;
  PCE_CUDA(cudaGetDevice(&dev));
  if (dev != p->device) return PCE_ERR_INVALID;
  // Storage to build into: the oldest released pass whose readers have finished; if they have not,
  // a new pass (up to kMaxPasses), so that the maps of this pass are built while the previous
  // pass still computes; beyond that the oldest one, whose readers the lanes then wait for.
  // A caller that keeps the maps of many passes alive gets at most kHardPasses arenas; the next
  // begin then fails with PCE_ERR_CAPACITY (the caller builds that pass's maps lazily instead).
  constexpr int kMaxPasses = 3;
  constexpr int kHardPasses = 8;
  pce_pass* ps = nullptr;
  {
    std::lock_guard<std::mutex> lk(p->m);
    if (p->stop) return PCE_ERR_INVALID;
    if (!p->idle.empty()) {
      pce_pass* oldest = p->idle.front();
      bool drained = true;
      if (oldest->has_released) {
        const cudaError_t q = cudaEventQuery(oldest->released);
        drained = q == cudaSuccess;
        if (q == cudaErrorNotReady) (void)cudaGetLastError();  // "not ready" is an answer, not a failure
      }
      if (drained || p->n_passes >= kMaxPasses) {
        ps = oldest;
        p->idle.pop_front();
      }
    }
    if (!ps) {
      if (p->n_passes >= kHardPasses) return PCE_ERR_CAPACITY;
      ++p->n_passes;
    }
  }
  if (!ps) {
    ps = new pce_pass();
    ps->plan = p;
    cudaError_t e = cudaEventCreateWithFlags(&ps->start, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ps->released, cudaEventDisableTiming);
    ps->ready.assign(p->specs.size(), nullptr);
    ps->levels.assign(p->n_levels, LevelState{});
    for (size_t i = 0; i < p->specs.size() && e == cudaSuccess; ++i)
      e = cudaEventCreateWithFlags(&ps->ready[i], cudaEventDisableTiming);
    for (int k = 1; k < p->n_levels && e == cudaSuccess; ++k)
      e = cudaEventCreateWithFlags(&ps->levels[k].ev, cudaEventDisableTiming);
    if (e != cudaSuccess) {
      free_pass(ps);
      return cuda_fail(e);
    }
  }
  ps->arena.reset();
  for (int k = 0; k < p->n_levels; ++k) {
    ps->levels[k].coords = nullptr;
    ps->levels[k].n = 0;
    ps->levels[k].ready = 0;
  }
  ps->levels[0].coords = coords;
  ps->levels[0].n = n;
  ps->levels[0].ready = 1;  // its producer precedes `start`, which every lane's stream waits for
  for (int d = 0; d < 3; ++d) {
    ps->cmin[d] = cmin[d];
    ps->levels[0].cmax[d] = cmax[d];
  }
  ps->queued.assign(p->specs.size(), 0);
  ps->maps.assign(p->specs.size(), pce_planned_map{});
  ps->next_map = 0;
  ps->lanes_done = 0;
  ps->error = PCE_OK;
  ps->finished = false;
  // everything queued on `stream` so far (the coordinates' producer) precedes the planner's
  // first kernel
  cudaError_t e = cudaEventRecord(ps->start, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) {
    std::lock_guard<std::mutex> lk(p->m);
    p->idle.push_back(ps);
    return cuda_fail(e);
  }
  {
    std::lock_guard<std::mutex> lk(p->m);
    for (int l = 0; l < kLanes; ++l) p->lanes[l].queue.push_back(ps);
  }
  p->cv.notify_all();
  *out = ps;
  return PCE_OK;
}

int pce_pass_map(pce_pass* ps, int32_t index, void* stream, pce_planned_map* out) {
  if (!ps || !out || index < 0 || index >= static_cast<int32_t>(ps->maps.size())) return PCE_ERR_INVALID;
  pce_plan* p = ps->plan;
  {
    std::unique_lock<std::mutex> lk(p->m);
    const bool done = p->cv.wait_for(lk, std::chrono::seconds(30),
                                     [&] { return ps->queued[index] != 0 || ps->error != PCE_OK || ps->finished; });
    if (!done) return PCE_ERR_TIMEOUT;
    if (ps->error != PCE_OK) return ps->error;
    if (!ps->queued[index]) return PCE_ERR_INVALID;
  }
  PCE_CUDA(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), ps->ready[index], 0));
  *out = ps->maps[index];
  return PCE_OK;
}

int pce_pass_release(pce_pass* ps, void* stream) {
  if (!ps) return PCE_ERR_INVALID;
  pce_plan* p = ps->plan;
  // the readers of the maps were queued on `stream`: whoever recycles the storage waits for them
  const cudaError_t e = cudaEventRecord(ps->released, static_cast<cudaStream_t>(stream));
  std::unique_lock<std::mutex> lk(p->m);
  const bool done = p->cv.wait_for(lk, std::chrono::seconds(30), [&] { return ps->finished; });
  if (!done) return PCE_ERR_TIMEOUT;  // the pass stays with the planner; its storage is not recycled
  if (e != cudaSuccess) return cuda_fail(e);  // not recycled either: its readers are unknown
  ps->has_released = true;
  p->idle.push_back(ps);
  return PCE_OK;
}


// ---- whole-pass execution -------------------------------------------------------------------
// One call queues every feature kernel of a network pass whose maps the planner builds: the host
// walks a flat list of operations (sparse convolution through planned map i, or dense rows x matrix
// product), fetches each map when an operation first needs it (pce_pass_map: waits on the host until
// the map's kernels are queued, makes the stream wait for them), places the intermediate feature
// matrices in the caller's arena as their row counts become known, and launches the tensor-core
// kernel.  The same launches, in the same order, as calling pce_conv_fwd / pce_linear_fwd per layer.
static int net_run_on(pce_pass* ps, const pce_net_buffer* buffers, int32_t n_buffers, const pce_net_op* ops, int32_t n_ops,
                      const void* input, int32_t in_ld, void* output, int32_t out_ld, void* arena, size_t arena_bytes,
                      int32_t dtype, cudaStream_t st) {
  pce_plan* p = ps->plan;
  const int n_specs = static_cast<int>(p->specs.size());
  void* stream = st;
  std::vector<pce_planned_map> maps(n_specs);
  std::vector<char> have(n_specs, 0);
  std::vector<int32_t> level_rows(p->n_levels, -1);
  level_rows[0] = ps->levels[0].n;
  std::vector<char*> base(n_buffers, nullptr);
  size_t used = 0;
  char* arena_c = static_cast<char*>(arena);
  char* split = nullptr;  // scratch of split layers (fp32 partial sums)
  size_t split_bytes = 0;
  auto fetch = [&](int i) -> int {
    if (i < 0 || i >= n_specs) return PCE_ERR_INVALID;
    if (!have[i]) {
      PCE_TRY(pce_pass_map(ps, i, stream, &maps[i]));
      have[i] = 1;
      level_rows[p->specs[i].in_level] = maps[i].n_in;
      level_rows[p->out_level[i]] = maps[i].n_out;
    }
    return PCE_OK;
  };
  // address, row pitch (elements) and row count of a view; places the buffer on first use
  auto view = [&](int buf, int col, int width, const void* ext, int ext_ld, const __half** ptr, int* ld, int* rows) -> int {
    if (buf < 0) {  // the network's input (-1) or output (-2)
      *ptr = static_cast<const __half*>(ext) + col;
      *ld = ext_ld;
      *rows = level_rows[0];
      return PCE_OK;
    }
    if (buf >= n_buffers) return PCE_ERR_INVALID;
    const pce_net_buffer& b = buffers[buf];
    if (b.level < 0 || b.level >= p->n_levels || b.width < 8 || (b.width & 7) || col < 0 || (col & 7) || col + width > b.width)
      return PCE_ERR_INVALID;
    const int32_t n = level_rows[b.level];
    if (n < 0) return PCE_ERR_INVALID;  // used before the layer that creates its level
    if (!base[buf]) {
      const size_t bytes = pad256(static_cast<size_t>(n > 0 ? n : 1) * b.width * sizeof(__half));
      if (!arena_c || used + bytes > arena_bytes) return PCE_ERR_WORKSPACE;
      base[buf] = arena_c + used;
      used += bytes;
    }
    *ptr = reinterpret_cast<const __half*>(base[buf]) + col;
    *ld = b.width;
    *rows = n;
    return PCE_OK;
  };
  for (int i = 0; i < n_ops; ++i) {
    const pce_net_op& op = ops[i];
    if (op.c_in < 16 || op.c_out < 16 || !conv_umma_supported(op.c_in, op.c_out, dtype) || !op.packed_weights)
      return PCE_ERR_UNSUPPORTED;
    const pce_planned_csr* csr = nullptr;
    if (op.kind == 0) {
      PCE_TRY(fetch(op.map));
      const pce_planned_map& m = maps[op.map];
      if (op.transposed ? !m.has_tr : !m.has_fwd) return PCE_ERR_INVALID;
      csr = op.transposed ? &m.tr : &m.fwd;
      if (op.kv != m.kv) return PCE_ERR_INVALID;
    } else if (op.kind != 1) {
      return PCE_ERR_INVALID;
    }
    const __half *src = nullptr, *extra = nullptr;
    const __half* dst = nullptr;
    int src_ld = 0, dst_ld = 0, extra_ld = 0, src_rows = 0, dst_rows = 0, extra_rows = 0;
    PCE_TRY(view(op.src_buf, op.src_col, op.c_in, input, in_ld, &src, &src_ld, &src_rows));
    if (csr) {  // the destination's level exists once the map is known
      if (src_rows != csr->n_src) return PCE_ERR_INVALID;
    }
    PCE_TRY(view(op.dst_buf, op.dst_col, op.c_out, output, out_ld, &dst, &dst_ld, &dst_rows));
    if (csr ? dst_rows != csr->n_rows : dst_rows != src_rows) return PCE_ERR_INVALID;
    pce_epilogue ep = {};
    ep.scale = op.scale;
    ep.shift = op.shift;
    ep.act = op.act;
    ep.slope = op.slope;
    ep.in_ld = src_ld;
    ep.out_ld = dst_ld;
    if (op.extra_c > 0) {
      if (!op.extra_packed_weights || !csr) return PCE_ERR_INVALID;
      PCE_TRY(view(op.extra_buf, op.extra_col, op.extra_c, input, in_ld, &extra, &extra_ld, &extra_rows));
      if (extra_rows != dst_rows || extra_ld != op.extra_c) return PCE_ERR_UNSUPPORTED;  // the second operand is read densely
      ep.extra_feats = extra;
      ep.extra_packed_weights = op.extra_packed_weights;
      ep.extra_c = op.extra_c;
    }
    if (dst_rows == 0) continue;
    if (!csr) {
      PCE_TRY(conv_umma(src, src_rows, op.packed_weights, 1, nullptr, dst_rows, op.c_in, op.c_out, const_cast<__half*>(dst), &ep, st));
      continue;
    }
    const int rows = tile_rows_policy(csr->n_rows, op.c_in, op.c_out, p->sm_count);
    const int slots = op.c_in == 32 ? 2 : (op.c_in == 16 ? 4 : 1);
    const pce_tile_lists* tl = nullptr;
    for (int u = 0; u < csr->n_lists; ++u) {
      const pce_tile_lists& c = csr->lists[u];
      if (c.tile_rows == rows && (c.slots > 1 ? c.slots : 1) == slots && (c.identity_stage || op.extra_c == 0)) tl = &c;
    }
    if (!tl) return PCE_ERR_INVALID;  // the plan was declared without this layer's widths
    // small and mid-size maps: tiles split between CTAs; the fp32 partial sums live behind the buffers
    // (one region, reused by every split layer: the layers run in stream order)
    const size_t want = conv_split_scratch_bytes(dst_rows, src_rows, op.c_in, op.c_out, op.kv, p->sm_count);
    if (want > 0) {
      const size_t need = pad256(want);
      if (need > split_bytes) {  // a larger region behind what is placed so far (the old one stays unused)
        if (!arena_c || used + need > arena_bytes) return PCE_ERR_WORKSPACE;
        split = arena_c + used;
        split_bytes = need;
        used += need;
      }
      ep.split_scratch = split;
      ep.split_scratch_bytes = split_bytes;
    }
    PCE_TRY(conv_umma(src, src_rows, op.packed_weights, op.kv, tl, dst_rows, op.c_in, op.c_out, const_cast<__half*>(dst), &ep, st));
  }
  return PCE_OK;
}

int pce_net_run(pce_pass* ps, const pce_net_buffer* buffers, int32_t n_buffers, const pce_net_op* ops, int32_t n_ops,
                const void* input, int32_t in_ld, void* output, int32_t out_ld, void* arena, size_t arena_bytes,
                int32_t dtype, void* stream) {
  if (!ps || !ops || n_ops < 1 || n_buffers < 0 || (n_buffers > 0 && !buffers) || !input || !output) return PCE_ERR_INVALID;
  if (dtype != PCE_F16) return PCE_ERR_UNSUPPORTED;
  // (A stream of the highest priority for the pass, forked from and joined to the caller's, was measured:
  // 3.93 -> 3.98 ms per 8-scan step beside the next pass's map construction, no change on 1 or 2 scans.)
  return net_run_on(ps, buffers, n_buffers, ops, n_ops, input, in_ld, output, out_ld, arena, arena_bytes, dtype,
                    static_cast<cudaStream_t>(stream));
}

}  // extern "C"
