// Kernel-map planner: builds every kernel map of a network pass on a host thread of its own,
// which feeds a second CUDA stream, while the calling thread queues the feature kernels.
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
// Memory: a pass owns a device arena (bump allocation over cudaMalloc'ed chunks, recycled with
// the pass object); transient workspaces share one grow-only scratch buffer, which is safe
// because every planner kernel runs on the one planning stream.  pce_plan_begin records an
// event on the caller's stream and the planning stream waits for it, so a recycled arena is
// never written before the previous pass's readers have finished.
#include <condition_variable>
#include <chrono>
#include <deque>
#include <mutex>
#include <thread>
#include <vector>

#include "common.cuh"

namespace pce {


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

struct Level {
  const int32_t* coords;
  int32_t n;
  int32_t cmax[3];
};

}  // namespace pce

using namespace pce;

struct pce_pass {
  pce_plan* plan = nullptr;
  DeviceArena arena;
  const int32_t* coords = nullptr;
  int32_t n = 0;
  int32_t cmin[3] = {0, 0, 0}, cmax[3] = {0, 0, 0};
  cudaEvent_t start = nullptr;
  std::vector<cudaEvent_t> ready;          // one per map
  std::vector<int> queued;                 // guarded by plan->m
  std::vector<pce_planned_map> maps;
  int error = PCE_OK;                      // guarded by plan->m
  bool finished = false;                   // guarded by plan->m
};

struct pce_plan {
  std::vector<pce_plan_map_spec> specs;
  int device = 0;
  int sm_count = 148;
  cudaStream_t stream = nullptr;
  void* scratch = nullptr;
  size_t scratch_cap = 0;
  std::mutex m;
  std::condition_variable cv;
  std::deque<pce_pass*> queue;
  std::vector<pce_pass*> idle;  // recycled passes (arena + events)
  bool stop = false;
  std::thread worker;
};

namespace pce {

static int scratch_for(pce_plan* p, size_t bytes, void** out) {
  if (bytes > p->scratch_cap) {
    PCE_CUDA(cudaStreamSynchronize(p->stream));  // nothing queued may still use the old buffer
    if (p->scratch) PCE_CUDA(cudaFree(p->scratch));
    p->scratch = nullptr;
    p->scratch_cap = 0;
    const size_t cap = pad256(bytes + bytes / 4);
    PCE_CUDA(cudaMalloc(&p->scratch, cap));
    p->scratch_cap = cap;
  }
  *out = p->scratch;
  return PCE_OK;
}

static int tile_rows_policy(int n_rows, int c_out, int sm_count) {
  return (c_out <= 128 && static_cast<long long>(n_rows) >= 6ll * 256 * sm_count) ? 256 : 128;
}

// One direction of a map: neighbour CSR, row order and the requested tile lists.
static int build_csr(pce_plan* p, pce_pass* ps, const int32_t* table, int kv, int n_rows, int n_src, int reverse, int ident,
                     size_t nbr_cap, const int32_t* c_outs, pce_planned_csr* out) {
  cudaStream_t st = p->stream;
  DeviceArena& ar = ps->arena;
  const int words = (kv + 31) / 32;
  uint32_t* mask = ar.take_n<uint32_t>(static_cast<size_t>(n_rows > 0 ? n_rows : 1) * words);
  int32_t* rowptr = ar.take_n<int32_t>(static_cast<size_t>(n_rows) + 1);
  int32_t* nbr = ar.take_n<int32_t>(nbr_cap);
  if (ar.error) return ar.error;
  void* ws = nullptr;
  const size_t ws_csr = 8 * (static_cast<size_t>(n_rows) + 1) + (8u << 20);
  PCE_TRY(scratch_for(p, ws_csr, &ws));
  PCE_TRY(pce_csr_from_dense(table, kv, n_rows, reverse, ident, ws, p->scratch_cap, mask, rowptr, nbr,
                             static_cast<int32_t>(nbr_cap), st));
  out->mask = mask;
  out->rowptr = rowptr;
  out->nbr = nbr;
  out->n_rows = n_rows;
  out->n_src = n_src;
  out->nbr_cap = static_cast<int32_t>(nbr_cap);
  out->tiles128 = pce_tile_lists{nullptr, nullptr, nullptr, nullptr, 0};
  out->tiles256 = pce_tile_lists{nullptr, nullptr, nullptr, nullptr, 0};
  bool want[2] = {false, false};
  for (int u = 0; u < PCE_PLAN_MAX_USES && c_outs[u] > 0; ++u)
    want[tile_rows_policy(n_rows, c_outs[u], p->sm_count) == 256 ? 1 : 0] = true;
  if ((!want[0] && !want[1]) || kv > 128 || n_rows == 0) return PCE_OK;
  int32_t* order = ar.take_n<int32_t>(n_rows);
  if (ar.error) return ar.error;
  PCE_TRY(scratch_for(p, 64 * static_cast<size_t>(n_rows) + (16u << 20), &ws));
  PCE_TRY(pce_csr_sort_rows(mask, n_rows, kv, ws, p->scratch_cap, order, st));
  for (int h = 0; h < 2; ++h) {
    if (!want[h]) continue;
    const int rows = h ? 256 : 128;
    const int n_tiles = div_up(n_rows, rows);
    const size_t cap = static_cast<size_t>(n_tiles) * kv;
    int32_t* tile_ptr = ar.take_n<int32_t>(static_cast<size_t>(n_tiles) + 1);
    int32_t* stage_kp = ar.take_n<int32_t>(cap);
    int32_t* stage_nbr = ar.take_n<int32_t>(cap * rows);
    if (ar.error) return ar.error;
    PCE_TRY(scratch_for(p, 8 * (static_cast<size_t>(n_tiles) + 1) + (1u << 20), &ws));
    PCE_TRY(pce_build_tile_lists(mask, rowptr, nbr, order, n_rows, kv, rows, ws, p->scratch_cap, tile_ptr, stage_kp,
                                 stage_nbr, static_cast<int32_t>(cap), st));
    (h ? out->tiles256 : out->tiles128) = pce_tile_lists{order, tile_ptr, stage_kp, stage_nbr, rows};
  }
  return PCE_OK;
}

static int build_map(pce_plan* p, pce_pass* ps, std::vector<Level>& levels, int i) {
  const pce_plan_map_spec& sp = p->specs[i];
  cudaStream_t st = p->stream;
  DeviceArena& ar = ps->arena;
  if (sp.in_level < 0 || sp.in_level >= static_cast<int>(levels.size())) return PCE_ERR_INVALID;
  const Level in = levels[sp.in_level];
  pce_planned_map& out = ps->maps[i];
  pce_geom g;
  const int kv = sp.ks[0] * sp.ks[1] * sp.ks[2];
  bool odd = true;
  for (int d = 0; d < 3; ++d) {
    g.ks[d] = sp.ks[d];
    g.stride[d] = sp.stride[d];
    g.pad[d] = sp.pad[d];
    g.cmin[d] = ps->cmin[d];
    g.cmax[d] = sp.submanifold ? in.cmax[d] : (in.cmax[d] + 2 * sp.pad[d] - (sp.ks[d] - 1)) / sp.stride[d];
    out.cmax_out[d] = g.cmax[d];
    odd = odd && (sp.ks[d] % 2 == 1);
  }
  g.submanifold = sp.submanifold ? 1 : 0;
  const int n_in = in.n;
  int n_out = n_in;
  const int32_t* out_coords = in.coords;
  void* ws = nullptr;
  if (!sp.submanifold) {
    long long per_input = 1;
    for (int d = 0; d < 3; ++d) per_input *= (sp.ks[d] + sp.stride[d] - 1) / sp.stride[d];
    const long long cap = n_in * per_input > 1 ? n_in * per_input : 1;
    if (cap >= (1ll << 31)) return PCE_ERR_UNSUPPORTED;
    int32_t* oc = ar.take_n<int32_t>(static_cast<size_t>(cap) * 4);
    if (ar.error) return ar.error;
    PCE_TRY(scratch_for(p, pce_map_workspace_bytes(n_in, kv, static_cast<int32_t>(cap)), &ws));
    PCE_TRY(pce_downsample_coords(in.coords, n_in, &g, ws, p->scratch_cap, oc, static_cast<int32_t>(cap), &n_out, st));
    out_coords = oc;
    Level lv;
    lv.coords = oc;
    lv.n = n_out;
    for (int d = 0; d < 3; ++d) lv.cmax[d] = g.cmax[d];
    levels.push_back(lv);
  }
  const bool symmetric = sp.submanifold && odd;
  int32_t* map = ar.take_n<int32_t>(static_cast<size_t>(kv) * (n_in > 0 ? n_in : 1));
  int32_t* map_out = symmetric ? nullptr : ar.take_n<int32_t>(static_cast<size_t>(kv) * (n_out > 0 ? n_out : 1));
  int32_t* small = ar.take_n<int32_t>(3 * static_cast<size_t>(kv) + 3 + 64);
  if (ar.error) return ar.error;
  int32_t* knnz = small;
  int32_t* kpos = small + kv;
  int32_t* qkpos = kpos + kv + 1;
  int32_t* status = qkpos + kv + 1;
  PCE_CUDA(cudaMemsetAsync(status, 0, sizeof(int32_t), st));
  PCE_TRY(scratch_for(p, pce_map_workspace_bytes(n_in, kv, n_out), &ws));
  PCE_TRY(pce_map_build_d2(in.coords, n_in, out_coords, n_out, &g, ws, p->scratch_cap, map, knnz, kpos, qkpos, map_out,
                           status, st));
  out.n_in = n_in;
  out.n_out = n_out;
  out.kv = kv;
  out.symmetric = symmetric ? 1 : 0;
  out.in_coords = in.coords;
  out.out_coords = out_coords;
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
  const size_t cap_nbr = sp.submanifold ? static_cast<size_t>(kv) * (n_in > 0 ? n_in : 1)
                                        : static_cast<size_t>(kv) * ((n_in < n_out ? n_in : n_out) > 0 ? (n_in < n_out ? n_in : n_out) : 1);
  if (cap_nbr >= (size_t(1) << 31)) return PCE_ERR_UNSUPPORTED;
  if (sp.want_fwd) {
    // output-major table: the map itself read with kp reversed when symmetric, else map_out
    PCE_TRY(build_csr(p, ps, symmetric ? map : map_out, kv, n_out, n_in, symmetric ? 1 : 0, ident, cap_nbr, sp.c_out_fwd,
                      &out.fwd));
    out.has_fwd = 1;
  }
  if (sp.want_tr) {
    // roles swapped: the input-major table is the output-major one of the transposed layer
    PCE_TRY(build_csr(p, ps, map, kv, n_in, n_out, 0, ident, cap_nbr, sp.c_out_tr, &out.tr));
    out.has_tr = 1;
  }
  return PCE_OK;
}

static void run_pass(pce_plan* p, pce_pass* ps) {
  int status = PCE_OK;
  std::vector<Level> levels;
  Level l0;
  l0.coords = ps->coords;
  l0.n = ps->n;
  for (int d = 0; d < 3; ++d) l0.cmax[d] = ps->cmax[d];
  levels.push_back(l0);
  cudaError_t e = cudaStreamWaitEvent(p->stream, ps->start, 0);
  if (e != cudaSuccess) status = cuda_fail(e);
  for (size_t i = 0; i < p->specs.size() && status == PCE_OK; ++i) {
    status = build_map(p, ps, levels, static_cast<int>(i));
    if (status == PCE_OK) {
      e = cudaEventRecord(ps->ready[i], p->stream);
      if (e != cudaSuccess) status = cuda_fail(e);
    }
    if (status == PCE_OK) {
      std::lock_guard<std::mutex> lk(p->m);
      ps->queued[i] = 1;
    }
    p->cv.notify_all();
  }
  {
    std::lock_guard<std::mutex> lk(p->m);
    if (status != PCE_OK) ps->error = status;
    ps->finished = true;
  }
  p->cv.notify_all();
}

static void worker_main(pce_plan* p) {
  cudaSetDevice(p->device);
  for (;;) {
    pce_pass* ps = nullptr;
    {
      std::unique_lock<std::mutex> lk(p->m);
      p->cv.wait(lk, [&] { return p->stop || !p->queue.empty(); });
      if (p->queue.empty()) return;  // stop requested and nothing left
      ps = p->queue.front();
      p->queue.pop_front();
    }
    run_pass(p, ps);
  }
}

}  // namespace pce

extern "C" {

int32_t pce_tile_rows_for(int32_t n_rows, int32_t c_out, int32_t sm_count) {
  return tile_rows_policy(n_rows, c_out, sm_count > 0 ? sm_count : 148);
}

int pce_plan_create(const pce_plan_map_spec* specs, int32_t n_specs, pce_plan** out) {
  if (!specs || n_specs < 1 || !out) return PCE_ERR_INVALID;
  int levels = 1;
  for (int i = 0; i < n_specs; ++i) {
    const pce_plan_map_spec& s = specs[i];
    for (int d = 0; d < 3; ++d)
      if (s.ks[d] < 1 || s.stride[d] < 1 || s.pad[d] < 0) return PCE_ERR_INVALID;
    if (s.in_level < 0 || s.in_level >= levels) return PCE_ERR_INVALID;
    if (!s.submanifold) ++levels;
  }
  pce_plan* p = new pce_plan();
  p->specs.assign(specs, specs + n_specs);
  cudaError_t e = cudaGetDevice(&p->device);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&p->sm_count, cudaDevAttrMultiProcessorCount, p->device);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&p->stream, cudaStreamNonBlocking);
  if (e != cudaSuccess) {
    delete p;
    return cuda_fail(e);
  }
  p->worker = std::thread(worker_main, p);
  *out = p;
  return PCE_OK;
}

static void free_pass(pce_pass* ps) {
  ps->arena.release();
  if (ps->start) cudaEventDestroy(ps->start);
  for (cudaEvent_t ev : ps->ready) cudaEventDestroy(ev);
  delete ps;
}

void pce_plan_destroy(pce_plan* p) {
  if (!p) return;
  {
    std::lock_guard<std::mutex> lk(p->m);
    p->stop = true;
  }
  p->cv.notify_all();
  if (p->worker.joinable()) p->worker.join();
  int prev = -1;
  cudaGetDevice(&prev);
  cudaSetDevice(p->device);
  cudaStreamSynchronize(p->stream);
  for (pce_pass* ps : p->idle) free_pass(ps);
  if (p->scratch) cudaFree(p->scratch);
  cudaStreamDestroy(p->stream);
  if (prev >= 0) cudaSetDevice(prev);
  delete p;
}

int pce_plan_begin(pce_plan* p, const int32_t* coords, int32_t n, const int32_t* cmin, const int32_t* cmax, void* stream,
                   pce_pass** out) {
  if (!p || !coords || n < 1 || !cmin || !cmax || !out) return PCE_ERR_INVALID;
  int dev = -1;
  PCE_CUDA(cudaGetDevice(&dev));
  if (dev != p->device) return PCE_ERR_INVALID;
  pce_pass* ps = nullptr;
  {
    std::lock_guard<std::mutex> lk(p->m);
    if (p->stop) return PCE_ERR_INVALID;
    if (!p->idle.empty()) {
      ps = p->idle.back();
      p->idle.pop_back();
    }
  }
  if (!ps) {
    ps = new pce_pass();
    ps->plan = p;
    cudaError_t e = cudaEventCreateWithFlags(&ps->start, cudaEventDisableTiming);
    ps->ready.resize(p->specs.size(), nullptr);
    for (size_t i = 0; i < p->specs.size() && e == cudaSuccess; ++i)
      e = cudaEventCreateWithFlags(&ps->ready[i], cudaEventDisableTiming);
    if (e != cudaSuccess) {
      free_pass(ps);
      return cuda_fail(e);
    }
  }
  ps->arena.reset();
  ps->coords = coords;
  ps->n = n;
  for (int d = 0; d < 3; ++d) {
    ps->cmin[d] = cmin[d];
    ps->cmax[d] = cmax[d];
  }
  ps->queued.assign(p->specs.size(), 0);
  ps->maps.assign(p->specs.size(), pce_planned_map{});
  ps->error = PCE_OK;
  ps->finished = false;
  // everything queued on the caller's stream so far (the coordinates' producer, the previous
  // pass's readers of a recycled arena) precedes the planner's first kernel
  cudaError_t e = cudaEventRecord(ps->start, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) {
    std::lock_guard<std::mutex> lk(p->m);
    p->idle.push_back(ps);
    return cuda_fail(e);
  }
  {
    std::lock_guard<std::mutex> lk(p->m);
    p->queue.push_back(ps);
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

int pce_pass_release(pce_pass* ps) {
  if (!ps) return PCE_ERR_INVALID;
  pce_plan* p = ps->plan;
  std::unique_lock<std::mutex> lk(p->m);
  const bool done = p->cv.wait_for(lk, std::chrono::seconds(30), [&] { return ps->finished; });
  if (!done) return PCE_ERR_TIMEOUT;  // the pass stays with the worker; its storage is not recycled
  p->idle.push_back(ps);
  return PCE_OK;
}

}  // extern "C"
