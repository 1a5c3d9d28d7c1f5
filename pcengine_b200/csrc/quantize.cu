// Voxelisation on the device: floor(points / voxel) and one row per occupied voxel, the step in
// front of the kernel maps (ref: script/utils.py:34-55 sparse_quantize, which does it with NumPy on
// the host: floor-divide, ravel hash, np.unique with return_index / return_inverse).
//
// Same results as that host code: the division is done in double precision (NumPy promotes the
// float32 points against the Python-float voxel size), the voxels come out in ascending (x,y,z)
// order (the order of the ravel hash), `index` names the FIRST point of every voxel (stable sort)
// and `inverse` maps every point to its voxel.
#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_scan.cuh>

#include "common.cuh"

namespace pce {

__global__ void k_voxel_keys(const float* __restrict__ pts, int n, double vx, double vy, double vz, int batch,
                             unsigned long long* keys, int* vals, int* status) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int x = static_cast<int>(floor(static_cast<double>(pts[3 * i]) / vx));
  const int y = static_cast<int>(floor(static_cast<double>(pts[3 * i + 1]) / vy));
  const int z = static_cast<int>(floor(static_cast<double>(pts[3 * i + 2]) / vz));
  if (!packable(batch, x, y, z)) atomicMax(status, PCE_ERR_RANGE);
  keys[i] = pack_key(batch, x, y, z);
  vals[i] = i;
}

__global__ void k_voxel_heads(const unsigned long long* __restrict__ keys, int n, int* heads) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) heads[i] = (i == 0 || keys[i] != keys[i - 1]) ? 1 : 0;
}

// rank[i] = inclusive count of heads up to i; voxel id of sorted position i = rank[i] - 1.
__global__ void k_voxel_emit(const unsigned long long* __restrict__ keys, const int* __restrict__ src,
                             const int* __restrict__ heads, const int* __restrict__ rank, int n, int4* coords,
                             int* index, int* inverse, int* n_unique) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int u = rank[i] - 1;
  if (heads[i]) {
    int b, x, y, z;
    unpack_key(keys[i], b, x, y, z);
    coords[u] = make_int4(b, x, y, z);
    if (index) index[u] = src[i];
  }
  if (inverse) inverse[src[i]] = u;
  if (i == n - 1) *n_unique = u + 1;
}

}  // namespace pce

using namespace pce;

extern "C" {

size_t pce_quantize_workspace_bytes(int32_t n) {
  const size_t m = n > 0 ? static_cast<size_t>(n) : 1;
  return 2 * pad256(8 * m) + 4 * pad256(4 * m) + 16 * m + (8u << 20) + 4096;
}

int pce_quantize_unique(const float* points, int32_t n, const float* voxel_host, int32_t batch, void* workspace,
                        size_t workspace_bytes, int32_t* out_coords, int32_t* out_index, int32_t* out_inverse,
                        int32_t* n_unique_host, void* stream) {
  if (!n_unique_host || n < 0 || !voxel_host || batch < 0) return PCE_ERR_INVALID;
  *n_unique_host = 0;
  if (n == 0) return PCE_OK;
  if (!points || !out_coords) return PCE_ERR_INVALID;
  for (int d = 0; d < 3; ++d)
    if (!(voxel_host[d] > 0.f)) return PCE_ERR_INVALID;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Arena ar(workspace, workspace_bytes);
  unsigned long long* keys = ar.take<unsigned long long>(n);
  unsigned long long* skeys = ar.take<unsigned long long>(n);
  int* vals = ar.take<int>(n);
  int* src = ar.take<int>(n);
  int* heads = ar.take<int>(n);
  int* rank = ar.take<int>(n);
  int* small = ar.take<int>(64);  // [0] status, [1] n_unique
  if (!ar.ok) return PCE_ERR_WORKSPACE;
  PCE_CUDA(cudaMemsetAsync(small, 0, 2 * sizeof(int), st));
  k_voxel_keys<<<div_up(n, 256), 256, 0, st>>>(points, n, static_cast<double>(voxel_host[0]),
                                                static_cast<double>(voxel_host[1]), static_cast<double>(voxel_host[2]),
                                                batch, keys, vals, small);
  PCE_LAUNCH_CHECK();
  size_t need = 0, need_scan = 0;
  PCE_CUDA(cub::DeviceRadixSort::SortPairs(nullptr, need, keys, skeys, vals, src, n, 0, 64, st));
  PCE_CUDA(cub::DeviceScan::InclusiveSum(nullptr, need_scan, heads, rank, n, st));
  if (need_scan > need) need = need_scan;
  char* tmp = ar.take<char>(need);
  if (!ar.ok) return PCE_ERR_WORKSPACE;
  PCE_CUDA(cub::DeviceRadixSort::SortPairs(tmp, need, keys, skeys, vals, src, n, 0, 64, st));  // stable
  k_voxel_heads<<<div_up(n, 256), 256, 0, st>>>(skeys, n, heads);
  PCE_LAUNCH_CHECK();
  PCE_CUDA(cub::DeviceScan::InclusiveSum(tmp, need, heads, rank, n, st));
  k_voxel_emit<<<div_up(n, 256), 256, 0, st>>>(skeys, src, heads, rank, n, reinterpret_cast<int4*>(out_coords), out_index,
                                               out_inverse, small + 1);
  PCE_LAUNCH_CHECK();
  int host[2] = {0, 0};
  PCE_CUDA(cudaMemcpyAsync(host, small, sizeof(host), cudaMemcpyDeviceToHost, st));
  PCE_CUDA(cudaStreamSynchronize(st));
  if (host[0] != 0) return host[0];
  *n_unique_host = host[1];
  return PCE_OK;
}

}  // extern "C"
