/*
 * pce_b200.h — C ABI of libpce_b200.so, a Blackwell (sm_100a) sparse-convolution
 * inference core that replaces the CUDA backend of hkeee21/PCEngine.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless its name ends in _host;
 *   - the caller owns every buffer (as the reference's Python layer does: it
 *     allocates all map arrays and passes them in, script/spconv.py:345-352,390-403);
 *   - nothing here allocates device memory unless stated; scratch is the caller's
 *     `workspace` (size from the matching *_workspace_bytes query);
 *   - all work is enqueued on `stream` (a cudaStream_t passed as void*); calls do
 *     not synchronise unless stated;
 *   - every function returns a pce status code and never throws.
 *
 * Coordinates are int32 rows (b, x, y, z), b in [0, 65534], x/y/z in
 * [-32768, 32767]; rows must be unique.  Geometry triples use the reference's
 * x, y, z order (script/utils.py:233-242).
 *
 * Paths cited as "ref:" are relative to the reference project's root.
 */
#ifndef PCE_B200_H_
#define PCE_B200_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define PCE_API __attribute__((visibility("default")))
#else
#define PCE_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

enum {
  PCE_OK = 0,
  PCE_ERR_INVALID = 1,     /* bad argument (null pointer, negative size, channel mismatch) */
  PCE_ERR_CUDA = 2,        /* a CUDA runtime call or launch failed; see pce_last_cuda_error */
  PCE_ERR_WORKSPACE = 3,   /* workspace smaller than the *_workspace_bytes answer */
  PCE_ERR_RANGE = 4,       /* a coordinate lies outside the packable range */
  PCE_ERR_TABLE_FULL = 5,  /* hash insert ran out of probes (duplicate-free input never does) */
  PCE_ERR_UNSUPPORTED = 6, /* shape/dtype combination that no kernel covers */
  PCE_ERR_TIMEOUT = 7,     /* a bounded device-side wait expired */
  PCE_ERR_CAPACITY = 8     /* an output buffer's stated capacity is too small */
};

enum { PCE_F32 = 0, PCE_F16 = 1 };
enum { PCE_ACT_NONE = 0, PCE_ACT_RELU = 1, PCE_ACT_LEAKY = 2 };
/* which convolution kernel family pce_conv_fwd may use */
enum { PCE_KERNEL_AUTO = 0, PCE_KERNEL_SIMT = 1, PCE_KERNEL_UMMA = 2 };

/* Layer geometry; replaces the integer codes 94273*x + 311*y + z that the
 * reference decodes again in C++ (ref: backend/hash.cu:57-76). */
typedef struct pce_geom {
  int32_t ks[3];
  int32_t stride[3];
  int32_t pad[3];
  int32_t cmin[3];     /* output-coordinate lower bound (ref: script/spconv.py:339) */
  int32_t cmax[3];     /* output-coordinate upper bound (ref: script/spconv.py:355-360) */
  int32_t submanifold; /* 1: outputs are the inputs, centre offset kept apart */
} pce_geom;

/* Fused epilogue applied to the fp32 accumulator before the single store of an
 * output row: y = act(acc * scale[c] + shift[c] + residual[row][c]).
 * Replaces the separate passes of ref: script/batchnorm.py:7-11,
 * script/activation.py:6-15, the bias add at script/spconv.py:325,453 and the
 * residual add of script/sptensor.py:80-91.  Any pointer may be NULL.
 *
 * extra_*: a second operand that joins the accumulation itself,
 *   acc[row] += extra_feats[row] @ W2,   W2 [extra_c, c_out] given in the packed layout
 * (pce_pack_weights with kv = 1).  It is multiplied by `scale` like the rest of the
 * accumulator, so a block that wants y = act(bn2(conv2(x)) + bn_s(shortcut(x0))) folds both
 * BatchNorm scales into the two weight tensors and passes only the summed shifts; the
 * plain residual of a block is the case W2 = identity.  Compared with `residual`, the rows
 * travel through the kernel's gather pipeline instead of being read in its epilogue, and a
 * 1x1x1 shortcut convolution costs no launch and no round trip of its output through
 * memory.  Tensor-core kernel only (fp16, extra_c a multiple of 16, tile lists built with
 * identity_stage = 1); other calls return PCE_ERR_UNSUPPORTED when it is set. */
typedef struct pce_epilogue {
  const float* scale;   /* [c_out] */
  const float* shift;   /* [c_out] */
  const void* residual; /* [n_out, c_out], same dtype as the features */
  int32_t act;
  float slope;
  const void* extra_feats;          /* [n_out, extra_c] fp16 */
  const void* extra_packed_weights; /* pce_packed_weights_bytes(1, extra_c, c_out) bytes */
  int32_t extra_c;
  /* Halo push (slab-parallel scenes): output row r is stored a second time to
   * push_base[s] + push_slot[s][r] * c_out elements for s = 0, 1 where push_slot[s][r] >= 0.
   * push_base[s] is the feature buffer of a neighbouring GPU mapped into this process
   * (peer memory); the stores are plain 16-byte peer stores from the convolution's
   * epilogue, so the boundary rows cross NVLink while the interior is still computed and
   * no separate exchange step reads them back.  The caller orders the neighbour's reads
   * after this launch (a barrier between the GPUs).  Tensor-core kernel only. */
  const int32_t* push_slot[2]; /* [n_out] each, or NULL */
  void* push_base[2];
  /* Row pitches in elements, 0 = dense (c_in / c_out).  A layer may read its input from, and write
   * its output into, a column range of a wider row-major matrix (in_feats / out_feats then point at
   * the first column of the range): the output of an up-sampling layer and the skip features land
   * side by side in one buffer without a concatenation pass.  Tensor-core kernel only; a pitch must
   * be a multiple of 8 elements and the pointers 16-byte aligned. */
  int32_t in_ld;
  int32_t out_ld;
  /* Scratch for maps with few tiles (optional).  A 128-row tile is one sequential chain of
   * (offset, K block) stages on one CTA; a map with fewer tiles than the GPU has CTA slots leaves
   * SMs idle while those chains run, and one with a few times as many ends in a half-empty wave.
   * With split_scratch of at least pce_conv_split_scratch_bytes(...) bytes (16-byte aligned) the
   * tiles are split between CTAs -- 2, 4 or 8 CTAs per tile on small maps, equal shares of the
   * stages whatever tiles they fall in on mid-size ones --, the CTAs leave fp32 partial sums here
   * and a second kernel adds them in a fixed order and applies the epilogue (deterministic; the
   * fp32 sum is associated differently than in the one-CTA chain).  Without scratch the layer runs
   * whole. */
  void* split_scratch;
  size_t split_scratch_bytes;
} pce_epilogue;

/* The kernel map re-laid for the tensor-core kernel (pce_build_tile_lists): output
 * rows in bitmask-sorted `order`, cut into tiles of tile_rows (128, 256 or 512); tile t
 * owns the stages tile_ptr[t] .. tile_ptr[t+1]-1, one per offset that any of its rows
 * has; stage g applies offset stage_kp[g] & 255 and fetches input row
 * stage_nbr[g*tile_rows + r] for the tile's r-th row (-1: that row lacks the offset).
 * A tile of 256 or 512 rows is two or four 128-row sub-tiles, each with its own
 * tensor-memory accumulator, fed by one staged weight block; with slots = 1, bit 8+s of
 * stage_kp[g] says whether sub-tile s has a row with the offset (a sub-tile without one
 * neither gathers nor multiplies for that stage).  With identity_stage = 1 every tile ends with one more stage, stage_kp = -1, whose
 * entry for a row is the row itself: where pce_epilogue.extra_feats joins the accumulation
 * (a launch without a second operand skips it).  With slots = 2 or 4 a stage holds that
 * many of the tile's offsets (stage_kp[g*slots + q], stage_nbr[(g*slots + q)*tile_rows + r],
 * unused slots kp = -2): a layer with 32 or 16 input channels fills only half or a quarter
 * of the kernel's 64-channel K block, so its offsets are taken two or four at a time and the
 * tile needs half or a quarter of the stages.  pce_conv_fwd takes slots = 64 / c_in for
 * c_in = 32 or 16, else 1.  No reference counterpart: it is the CSR-coded map + indicator in the layout
 * the tensor-core kernel consumes with coalesced reads. */
typedef struct pce_tile_lists {
  const int32_t* order;     /* [n_rows] */
  const int32_t* tile_ptr;  /* [ceil(n_rows/tile_rows) + 1] */
  const int32_t* stage_kp;  /* [stages] */
  const int32_t* stage_nbr; /* [stages * tile_rows] */
  int32_t tile_rows;        /* 128, 256 or 512 (512: slots = 1 only) */
  int32_t identity_stage;   /* 0 or 1 */
  int32_t slots;            /* offsets per stage: 1, 2 or 4 */
  int32_t settled;          /* non-zero: the lists were complete before the kernel that precedes this
                             * launch in its stream was launched (planner lists, lists kept from an
                             * earlier call).  The tensor-core kernel is launched so that its set-up
                             * overlaps that kernel's tail, and may then read the lists that early
                             * too; 0 is always safe. */
} pce_tile_lists;

PCE_API const char* pce_strerror(int status);
/* 100 * major + minor of this header's struct layouts (101: pce_epilogue.in_ld / out_ld,
 * pce_tile_lists.settled); a binding checks it before it passes structs. */
PCE_API int pce_version(void);
/* cudaError_t of the most recent failing CUDA call made by this library on the
 * calling thread (0 if none). */
PCE_API int pce_last_cuda_error(void);
/* Number of this library's own kernels launched by the process so far (library
 * primitives such as radix sort / scan passes and memsets are not counted). */
PCE_API uint64_t pce_kernel_launches(void);

/* ---------------------------------------------------------- voxelisation -- */

/* floor(points / voxel) and one row per occupied voxel: the device form of
 * sparse_quantize (ref: script/utils.py:34-55, NumPy on the host), the step before the
 * kernel maps.  points float32 [n,3] (device), voxel_host 3 floats (host).  The division
 * is done in double precision as NumPy does it; out_coords [<= n, 4] = (batch, x, y, z)
 * in ascending (x,y,z) order (the order of the reference's ravel hash); out_index[u]
 * (optional) = the first point of voxel u, out_inverse[i] (optional) = the voxel of point
 * i.  SYNCHRONISES `stream` once to return *n_unique_host.  A voxel coordinate outside
 * the packable range gives PCE_ERR_RANGE. */
PCE_API size_t pce_quantize_workspace_bytes(int32_t n);
PCE_API int pce_quantize_unique(const float* points, int32_t n, const float* voxel_host, int32_t batch,
                                void* workspace, size_t workspace_bytes, int32_t* out_coords,
                                int32_t* out_index, int32_t* out_inverse, int32_t* n_unique_host,
                                void* stream);

/* ------------------------------------------------------------------ maps -- */

/* Scratch bytes needed by the map-building calls below for n_in inputs. */
PCE_API size_t pce_map_workspace_bytes(int32_t n_in, int32_t kv, int32_t n_out_cap);

/* Output coordinates of a strided convolution: the unique, ascending-(b,x,y,z)
 * set of (in + pad - k) / stride that divide exactly and lie in [cmin, cmax].
 * Replaces coordsDownsampleExpand + thrust remove/sort/unique + coordsGenerator
 * (ref: backend/hash.cuh:535-641, backend/hash.cu:141-175,364-398); the same rule
 * is used when ks == stride, where the reference's shortcut (hash.cu:333-362)
 * disagrees with its own query kernel.  out_coords has room for out_cap rows.
 * SYNCHRONISES `stream` once to return *n_out_host (the reference does the same
 * through thrust's end pointer). */
PCE_API int pce_downsample_coords(const int32_t* in_coords, int32_t n_in, const pce_geom* g,
                          void* workspace, size_t workspace_bytes,
                          int32_t* out_coords, int32_t out_cap, int32_t* n_out_host, void* stream);

/* The fetch-on-demand map (ref: HashMapD2, backend/hash.cu:258-435, declared at
 * backend/hash.h:37-58): map[kp*n_in + in] = out or -1, knnz[kv], kpos[kv+1],
 * qkpos[kv+1] (segments padded to 128, ref: backend/hash.cuh:478-497).  Buffers need
 * no initialisation.  For a submanifold map pass out_coords = in_coords; the centre
 * offset row of `map` is left at -1 as in the reference.  map_out (optional, may
 * be NULL) receives the transposed table map_out[kp*n_out + out] = in or -1.
 * `status` (optional) is a device int that receives PCE_ERR_RANGE / TABLE_FULL. */
PCE_API int pce_map_build_d2(const int32_t* in_coords, int32_t n_in, const int32_t* out_coords, int32_t n_out,
                     const pce_geom* g, void* workspace, size_t workspace_bytes,
                     int32_t* map, int32_t* knnz, int32_t* kpos, int32_t* qkpos,
                     int32_t* map_out, int32_t* status, void* stream);

/* pce_map_build_d2 for callers that cannot hand over a workspace and must not trigger a
 * device allocation: a vehicle or robot perception loop whose memory is fixed at start-up
 * and whose safety rules forbid allocating once the loop runs, or a host runtime that owns
 * all device memory and gives a plug-in nothing but its input and output buffers.  It has
 * no counterpart in the reference (whose map builders allocate their hash tables through
 * ATen on every call).  Same inputs, outputs and results as pce_map_build_d2; the hash table
 * and the fallback status word live in a 4 MiB device array inside the library image, which
 * every GPU that loads the library holds until the process exits.
 *   - Limit: n_out <= 131072 output rows; more returns PCE_ERR_CAPACITY and launches nothing.
 *   - The first call on each device looks the array's address up; make that call during
 *     set-up, before any stream capture begins.  No call allocates or frees device memory
 *     itself; the CUDA runtime, however, may load a kernel's code the first time that kernel
 *     is launched (lazy module loading) and take memory for it.  The kernels differ by map
 *     kind, so the set-up calls should build one submanifold map with odd kernel sizes and
 *     one strided map with map_out: after those two, later calls leave device memory as it is.
 *   - All calls on a device share the array and it keeps the previous call's contents (the
 *     part a call uses is cleared first), so two calls whose GPU work can overlap - different
 *     streams, or threads - race on it: serialise them on one stream. */
PCE_API int pce_map_build_d2_noalloc(const int32_t* in_coords, int32_t n_in, const int32_t* out_coords,
                                     int32_t n_out, const pce_geom* g, int32_t* map, int32_t* knnz, int32_t* kpos,
                                     int32_t* qkpos, int32_t* map_out, int32_t* status, void* stream);

/* Indicator -> pair lists ordered by (kp, in): the device form of
 * `nonzero(map != -1)`, `omap = map[idx]`, `imap = idx % n_in`
 * (ref: script/spconv.py:370-372).  Lists have room for pair_cap entries; the
 * pair count is kpos[kv]. */
PCE_API int pce_map_pairs(const int32_t* map, int32_t kv, int32_t n_in, void* workspace, size_t workspace_bytes,
                  int32_t* imap, int32_t* omap, int32_t pair_cap, void* stream);

/* The CSR-coded gather/scatter map (ref: HashMapD1, backend/hash.cu:20-255,
 * declared at backend/hash.h:11-34) derived from the two dense tables:
 * icsr[n_in+1] / ocsr[n_out+1] row pointers and row entries kp*1186111 + pos,
 * kp-ascending, where pos is the pair's index inside its offset's segment of
 * the (kp, in)-ordered pair list (the reference takes pos from an atomic
 * counter, ref: backend/hash.cuh:161-165, so only this canonical numbering is
 * reproducible).  map_out may be NULL for a submanifold map. */
PCE_API int pce_map_build_d1(const int32_t* map, const int32_t* map_out, int32_t kv, int32_t n_in, int32_t n_out,
                     int32_t submanifold, const int32_t* kpos, void* workspace, size_t workspace_bytes,
                     int32_t* imap_coded, int32_t* icsr, int32_t* omap_coded, int32_t* ocsr, void* stream);

/* Row-major neighbour lists + indicator bitmask from a dense table
 * table[kp*n_rows + row] (-1 absent): mask[n_rows * ceil(kv/32)], rowptr[n_rows+1],
 * nbr[<= nbr_cap] (kp-ascending per row).  reverse_kp reads table[(kv-1-kp)*n_rows+row]
 * (a submanifold map is its own transpose under kp -> kv-1-kp); identity_kp >= 0
 * adds the pair (row, identity_kp, row), which is how the centre offset that
 * the reference applies as a separate dense GEMM (ref: backend/spconv.cu:273-298)
 * is folded in.  This is the form pce_conv_fwd consumes; the reference has no
 * literal bitmask, its indicator is the -1 sentinel of `map`. */
PCE_API int pce_csr_from_dense(const int32_t* table, int32_t kv, int32_t n_rows, int32_t reverse_kp,
                       int32_t identity_kp, void* workspace, size_t workspace_bytes,
                       uint32_t* mask, int32_t* rowptr, int32_t* nbr, int32_t nbr_cap, void* stream);

/* Same output as pce_csr_from_dense, built from (kp, in)-ordered pair lists as
 * the reference's forward takes them (ref: backend/spconv.h:28-40); used by the
 * drop-in conv_fwd_d2_cuda, which receives nothing else.  rows = the side that
 * becomes the output, nbrs = the other side; n_pairs is a host value. */
PCE_API int pce_csr_from_pairs(const int32_t* rows, const int32_t* nbrs, const int32_t* kpos, int32_t kv,
                       int32_t n_pairs, int32_t n_rows, int32_t identity_kp,
                       void* workspace, size_t workspace_bytes,
                       uint32_t* mask, int32_t* rowptr, int32_t* nbr, int32_t nbr_cap, void* stream);
PCE_API size_t pce_csr_from_pairs_workspace_bytes(int32_t n_pairs, int32_t n_rows);

/* ----------------------------------------------------------- convolution -- */

/* Fused gather-matmul-scatter, output stationary: every output row is
 * accumulated in registers / tensor memory over its neighbour list and stored
 * once, with the epilogue applied; no atomics and no intermediate buffer.
 * Replaces ConvolutionForwardD2 and its kernel family
 * (ref: backend/spconv.cu:224-398, backend/spconv.cuh:427-735,832-935,1162-1413,
 * 1567-1730) including the centre-offset cuBLAS call and the zero fill of
 * script/spconv.py:247.  weights [kv, c_in, c_out] as the reference's `kernel`
 * parameter (ref: script/spconv.py:61-65).  fp16 features accumulate in fp32.
 * packed_weights (may be NULL) is the same tensor re-laid by pce_pack_weights for
 * the tensor-core kernel; without it only the CUDA-core kernel can run.  Either
 * `weights` or `packed_weights` may be NULL when the kernel that needs it is not
 * the one chosen.  The CUDA-core kernel walks mask/rowptr/nbr; the tensor-core
 * kernel needs `tiles` (from pce_build_tile_lists) and runs only when both
 * `tiles` and `packed_weights` are given.  Results do not depend on the kernel's
 * processing order. */
PCE_API int pce_conv_fwd(const void* in_feats, int32_t n_in, int32_t c_in, const void* weights,
                         const void* packed_weights, int32_t kv, int32_t c_out, const uint32_t* mask,
                         const int32_t* rowptr, const int32_t* nbr, const pce_tile_lists* tiles, int32_t n_out,
                         void* out_feats, int32_t dtype, const pce_epilogue* ep, int32_t kernel_choice,
                         void* stream);

/* Processing order for the tensor-core kernel: output rows sorted (stable radix sort) by
 * their indicator bitmask with the bits permuted by rarity, the rarest offset most
 * significant, so rows with the same neighbourhood pattern land in the same tile, rows
 * with a rare offset land next to each other, and a tile skips every offset none of its
 * rows has.  Purely a scheduling aid with no reference counterpart.  order[n_rows]
 * receives the permutation; kv <= 128; workspace >= 64*n_rows + 16 MiB bytes. */
PCE_API int pce_csr_sort_rows(const uint32_t* mask, int32_t n_rows, int32_t kv, void* workspace,
                              size_t workspace_bytes, int32_t* order, void* stream);

/* Fills the arrays of a pce_tile_lists from the neighbour CSR and a row order (NULL =
 * natural order) for tiles of tile_rows = 128, 256 or 512 rows.  tile_ptr needs
 * ceil(n_rows/tile_rows)+1 entries; stage_kp / stage_nbr have room for stage_cap stages of
 * `slots` entries each (tiles*(ceil(kv/slots) + identity_stage) always suffices; the stage
 * count ends up in tile_ptr[last]).  kv <= 128.
 * workspace >= 8*(tiles+1) + 1 MiB bytes. */
PCE_API int pce_build_tile_lists(const uint32_t* mask, const int32_t* rowptr, const int32_t* nbr,
                                 const int32_t* order, int32_t n_rows, int32_t kv, int32_t tile_rows,
                                 int32_t identity_stage, int32_t slots, void* workspace,
                                 size_t workspace_bytes, int32_t* tile_ptr, int32_t* stage_kp,
                                 int32_t* stage_nbr, int32_t stage_cap, void* stream);

/* Weight re-layout for the tensor-core kernel: per (offset, 64-channel K block) a
 * c_out x 128-byte K-major image with 16-byte chunks XOR-swizzled by the row index
 * (the shared-memory layout tcgen05.mma reads), zero padded in K.  Weights are
 * static at inference, so this runs once per layer. */
PCE_API size_t pce_packed_weights_bytes(int32_t kv, int32_t c_in, int32_t c_out);
PCE_API int pce_pack_weights(const void* weights, int32_t kv, int32_t c_in, int32_t c_out, int32_t dtype,
                             void* packed, void* stream);

/* Tuning hook for experiments and tests; what = 0: force the tensor-core kernel's stage-ring
 * depth (value 2, 3 or 4; 0 restores the automatic choice); what = 1: sub-tiles per tile (1 or
 * 2) of the dense product, which has no tile lists to fix it; what = 2: accumulator sets in
 * tensor memory (1 or 2); what = 3: programmatic dependent launch of the tensor-core kernel (its
 * set-up overlaps the tail of the kernel before it in the stream; 1 = on, the default, 0 = off,
 * 2 = on, but tile lists are never read before that kernel has finished); what = 4: 1 runs
 * layers with one offset per stage on the kernel with several accumulators per CTA and decoupled
 * row / weight rings (k_conv_umma_mt), 0 (default) on the one-accumulator kernel, which measured
 * faster; tile lists of 512 rows always run on the former; what = 5: hash-table queries of the
 * map builder with four cooperating lanes per query (1) or one thread per query (0, default);
 * what = 6: sort the rows on the most significant `value` bits of their key only (0 = all, default);
 * what = 7: 0 never splits tiles between CTAs; 1 (default) as pce_conv_split_scratch_bytes says;
 *           2 only the split of small maps into parts, no shares of stages on mid-size maps.
 * what = 8: 0 runs layers whose width is an odd multiple of 32 channels with 64-channel K blocks
 *           like every other layer (1, default: with 32-channel blocks, every ring stage full).
 * what = 9: 0 makes the planner build the neighbour CSR of every map and the tile lists from it; 1 (default)
 *           lets it skip the CSR where only tile lists are used (pce_planned_csr.rowptr == NULL). */
PCE_API int pce_tune(int32_t what, int32_t value);

/* Reads (and optionally clears) the library's device status word, where a kernel whose
 * bounded wait expired records PCE_ERR_TIMEOUT.  SYNCHRONISES the device. */
PCE_API int pce_device_status(int32_t* status_host, int32_t reset);

/* Diagnostics for PCE_ERR_TIMEOUT: where the first bounded wait since the last call gave up, as
 * {code, CTA, item, phase parity} (code = role | sub-tile << 4 | tile-in-CTA << 8; roles are listed
 * beside g_umma_where in csrc/conv_umma.cu); all zero when no wait expired.  Reads and clears. */
PCE_API int pce_debug_timeout(int32_t* where4);

/* Parts per tile (1, 2, 4 or 8) that pce_conv_fwd uses for a tensor-core layer of n_rows outputs
 * gathered from n_src input rows when pce_epilogue.split_scratch is given; 1 = the layer is not split
 * into parts (large maps, layers with 16 or 32 input channels, short stage chains, up-sampling
 * layers: few pairs per output row). */
PCE_API int32_t pce_conv_split_parts(int32_t n_rows, int32_t n_src, int32_t c_in, int32_t c_out, int32_t kv,
                                     int32_t sm_count);

/* Bytes of pce_epilogue.split_scratch with which pce_conv_fwd splits a tensor-core layer of n_rows
 * outputs gathered from n_src input rows; 0 = the layer runs whole. */
PCE_API size_t pce_conv_split_scratch_bytes(int32_t n_rows, int32_t n_src, int32_t c_in, int32_t c_out,
                                            int32_t kv, int32_t sm_count);

/* Which kernel family pce_conv_fwd runs for these channel counts: PCE_KERNEL_SIMT,
 * PCE_KERNEL_UMMA, or -1 when the forced choice is unsupported. */
PCE_API int pce_conv_kernel_choice(int32_t c_in, int32_t c_out, int32_t dtype, int32_t kernel_choice);

/* Explicit gather -> GEMM -> scatter over a caller-provided buffer of at least
 * qsum*(c_in+c_out) elements (ref: ConvolutionForwardD1, backend/spconv.cu:24-222,
 * declared at backend/spconv.h:11-25; buffer sizing script/spconv.py:426-429).
 * Takes the CSR-coded maps of pce_map_build_d1; centre_kp >= 0 adds in @ W[centre_kp]
 * (the reference's cuBLAS beta=1 call, backend/spconv.cu:163-221) inside the
 * scatter pass.  Products are stored in the feature dtype in the buffer and
 * summed in fp32.  With packed_weights (pce_pack_weights; may be NULL) and
 * 1032*(qsum/128)+8 spare bytes behind the two buffer halves the per-offset GEMM
 * runs on the tensor-core kernel (every 128-row tile of the padded buffer lies
 * in one offset's segment), otherwise on CUDA cores. */
PCE_API int pce_conv_fwd_d1(const void* in_feats, int32_t n_in, int32_t c_in, const void* weights,
                            const void* packed_weights, int32_t kv, int32_t c_out, const int32_t* qkpos,
                            int32_t qsum, const int32_t* imap_coded, const int32_t* icsr,
                            const int32_t* omap_coded, const int32_t* ocsr, int32_t n_out, void* buffer,
                            size_t buffer_bytes, void* out_feats, int32_t dtype, int32_t centre_kp,
                            const pce_epilogue* ep, void* stream);

/* Dense rows x matrix with the same epilogue: the 1x1x1 stride-1 shortcut
 * (ref: script/spconv.py:297-304). */
PCE_API int pce_linear_fwd(const void* in_feats, int32_t n, int32_t c_in, const void* weights,
                           const void* packed_weights, int32_t c_out, void* out_feats, int32_t dtype,
                           const pce_epilogue* ep, void* stream);

/* Stand-alone y = act(x*scale + shift) over feature rows for BatchNorm / ReLU
 * modules that were not fused into a convolution (ref: script/utils.py:141-149). */
PCE_API int pce_scale_shift_act(const void* x, int64_t n, int32_t c, void* y, int32_t dtype,
                        const pce_epilogue* ep, void* stream);

/* Copies rows rows[i] (rows == NULL: row i) of a row-major matrix into consecutive rows of dst, 16 bytes per
 * store.  dst may be a neighbouring GPU's memory mapped into this process (a peer pointer): the halo exchange
 * of a slab-parallel scene outside a convolution's epilogue (pce_epilogue.push_*): a rank stores its boundary
 * rows straight into the neighbour's mailbox, no message.  Only stores go to dst, nothing is loaded from it.
 * No reference counterpart (the reference is single-GPU).  row_bytes and both pitches are multiples of 16. */
PCE_API int pce_push_rows(const void* src, int64_t src_pitch_bytes, const int32_t* rows, int32_t n_rows,
                          int32_t row_bytes, void* dst, int64_t dst_pitch_bytes, void* stream);

/* ------------------------------------------------------ kernel-map planner -- */

/* The reference builds a kernel map inside the first convolution that needs it and keeps
 * it in the tensor's `kmaps` dictionary (ref: script/spconv.py:338-427).  A map depends on
 * coordinates only, and building one is ~30 short launches plus, for a strided layer, a
 * size read back to the host, so built lazily the maps leave the GPU waiting for the
 * host.  A plan lists the maps of a network in first-use order; pce_plan_begin hands the
 * input coordinates to a host thread of the library, which queues all maps (with the
 * same entry points as above, so bit-identical) on a CUDA stream of its own while the
 * caller queues feature kernels; pce_pass_map gives the caller map i once its kernels are
 * queued and makes the caller's stream wait for them.  Unlike the calls above, the planner
 * owns its device memory: cudaMalloc'ed arenas that grow to the largest pass seen and are
 * recycled from pass to pass, freed by pce_plan_destroy. */

#define PCE_PLAN_MAX_USES 8

typedef struct pce_plan_map_spec {
  int32_t ks[3], stride[3], pad[3];
  int32_t in_level;    /* coordinate level the map reads: 0 = the input, k = created by the
                        * k-th non-submanifold spec before this one */
  int32_t submanifold; /* 1: outputs = inputs; 0: the output coordinates form a new level */
  int32_t want_fwd;    /* neighbour CSR of the layer itself (rows = the map's outputs) */
  int32_t want_tr;     /* neighbour CSR of the matching transposed layer (rows = the map's inputs) */
  /* widths of the layers that use each CSR on the tensor-core kernel, c_out 0-terminated;
   * c_out selects the tile height (pce_tile_rows_for) and c_in the offsets per stage (64/c_in
   * for 16 or 32 input channels, else 1) of the tile lists that are prepared */
  int32_t c_out_fwd[PCE_PLAN_MAX_USES];
  int32_t c_out_tr[PCE_PLAN_MAX_USES];
  int32_t c_in_fwd[PCE_PLAN_MAX_USES];
  int32_t c_in_tr[PCE_PLAN_MAX_USES];
} pce_plan_map_spec;

typedef struct pce_planned_csr {
  const uint32_t* mask;
  const int32_t* rowptr; /* NULL (with nbr) where the planner took the short route: a map of at most 32 offsets */
  const int32_t* nbr;    /* whose uses all run on tile lists; pce_csr_from_dense(table, kv, n_rows, reverse_kp,
                          * identity_kp, ...) with nbr_cap entries builds both on demand */
  int32_t n_rows, n_src, nbr_cap;
  int32_t n_lists;
  const int32_t* table;  /* the dense table this direction reads (the map's `map` or `map_out`) */
  int32_t reverse_kp, identity_kp;
  pce_tile_lists lists[PCE_PLAN_MAX_USES]; /* distinct (tile_rows, slots) among the uses; the
                                            * forward lists of a submanifold map carry the
                                            * identity stage */
} pce_planned_csr;

typedef struct pce_planned_map {
  int32_t n_in, n_out, kv, symmetric;
  int32_t cmax_out[3];
  const int32_t* in_coords;  /* [n_in,4] */
  const int32_t* out_coords; /* [n_out,4]; == in_coords for a submanifold map */
  const int32_t* map;        /* [kv*n_in] as pce_map_build_d2 */
  const int32_t* map_out;    /* [kv*n_out] or NULL when symmetric */
  const int32_t *knnz, *kpos, *qkpos, *status;
  int32_t has_fwd, has_tr;
  pce_planned_csr fwd, tr;
} pce_planned_map;

typedef struct pce_plan pce_plan; /* specs + planning thread + stream + recycled storage */
typedef struct pce_pass pce_pass; /* the maps of one network pass; device memory owned by it */

/* Rows per tile the engine uses for a layer of n_rows outputs with c_in / c_out channels on a
 * GPU with sm_count SMs: 128, or 256 for layers with 16 or 32 input channels and at most 32
 * output channels on maps large enough to give every CTA several tiles (taller tiles stage every
 * weight block once for two or four accumulators but leave fewer independent tiles in flight per
 * SM, which measured slower from 64 input channels up). */
PCE_API int32_t pce_tile_rows_for(int32_t n_rows, int32_t c_in, int32_t c_out, int32_t sm_count);

/* Binds to the current device; starts the planning thread. */
PCE_API int pce_plan_create(const pce_plan_map_spec* specs, int32_t n_specs, pce_plan** plan);
/* Joins the thread and frees recycled storage; passes not yet released are leaked. */
PCE_API void pce_plan_destroy(pce_plan* plan);
/* Starts building the maps for coords [n,4] (device memory that stays valid for the pass);
 * cmin / cmax are the coordinate bounds of the input level.  Work queued on `stream` before
 * this call (the producer of the coordinates) precedes the planner's kernels; nothing else
 * orders the planner against the caller, so with the coordinates produced on a stream of
 * their own the maps of the next pass are built while the current one computes.  Returns
 * at once.  Up to three passes are created freely and at most eight exist; with eight
 * passes unreleased the call returns PCE_ERR_CAPACITY. */
PCE_API int pce_plan_begin(pce_plan* plan, const int32_t* coords, int32_t n, const int32_t* cmin,
                           const int32_t* cmax, void* stream, pce_pass** pass);
/* Blocks the host until map `index` is queued (30 s limit: PCE_ERR_TIMEOUT), makes `stream`
 * wait for its kernels and returns its arrays, valid until the pass is released. */
PCE_API int pce_pass_map(pce_pass* pass, int32_t index, void* stream, pce_planned_map* out);
/* Gives the pass's storage back to the plan for reuse (waits for the planning threads to be
 * done with it).  `stream` is the stream the kernels that read the maps were queued on: the
 * pass that recycles the storage waits for everything queued there up to this call. */
PCE_API int pce_pass_release(pce_pass* pass, void* stream);

/* ------------------------------------------------------ whole-pass execution -- */

/* The reference runs a network layer by layer from Python (ref: script/spconv.py:86-98 conv3d.forward
 * -> conv_func per layer); at ~100 k voxels the per-layer host work is longer than the kernels.
 * pce_net_run queues EVERY feature kernel of a planned pass in one call: the caller describes the
 * network once as a flat list of operations over feature matrices ("buffers"), each a sparse
 * convolution through planned map `map` (kind 0) or a dense rows x matrix product (kind 1, the 1x1x1
 * layer of ref: script/spconv.py:297-304), with the fused epilogue of pce_epilogue.  Buffers are
 * [rows of coordinate level `level`] x width fp16 matrices placed in `arena` in order of first use
 * (256-byte aligned; PCE_ERR_WORKSPACE when it is too small; sum over buffers of rows x width x 2
 * bytes with rows <= the input's rows, plus 400 MB for the fp32 partial sums of layers on small maps
 * that are split over several CTAs per tile (pce_conv_split_parts), always fits); an operation reads / writes a column range of one
 * (col, c_in / c_out wide, multiples of 8), so skip concatenations cost nothing.  Buffer -1 is the
 * network input (`input`, row pitch in_ld), -2 its output (`output`, out_ld).  Maps are fetched as
 * operations first need them (pce_pass_map), so the pass's map construction overlaps the kernels.
 * fp16, channel counts multiples of 16 (c_out <= 256), packed weights (pce_pack_weights).  Issues the
 * same launches as one pce_conv_fwd / pce_linear_fwd call per layer: bit-identical results. */
typedef struct pce_net_buffer {
  int32_t level; /* coordinate level whose row count the buffer has (0 = the input's) */
  int32_t width; /* channels per row (multiple of 8) */
} pce_net_buffer;

typedef struct pce_net_op {
  int32_t kind;       /* 0 sparse convolution, 1 dense product */
  int32_t map;        /* kind 0: index of the plan's map spec */
  int32_t transposed; /* kind 0: run the map transposed (rows = the map's inputs) */
  int32_t kv, c_in, c_out;
  int32_t src_buf, src_col;
  int32_t dst_buf, dst_col;
  const void* packed_weights;
  const float* scale; /* [c_out] or NULL */
  const float* shift; /* [c_out] or NULL */
  int32_t act;
  float slope;
  int32_t extra_buf, extra_col, extra_c; /* second operand (pce_epilogue.extra_*): a whole buffer, extra_c = its width; 0: none */
  const void* extra_packed_weights;
} pce_net_op;

PCE_API int pce_net_run(pce_pass* pass, const pce_net_buffer* buffers, int32_t n_buffers, const pce_net_op* ops,
                        int32_t n_ops, const void* input, int32_t in_ld, void* output, int32_t out_ld, void* arena,
                        size_t arena_bytes, int32_t dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PCE_B200_H_ */
