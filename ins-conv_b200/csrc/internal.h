// Internal declarations shared by the translation units of libinsconv_b200.so.
// Nothing in this file is part of the C ABI (see include/insconv_b200.h).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <string>
#include <atomic>
#include "insconv_b200.h"

namespace scn {

// ---- error plumbing ---------------------------------------------------------
void set_error(const std::string &msg);
int fail(int code, const std::string &msg);
#define SCN_CUDA(expr)                                                                              \
  do {                                                                                              \
    cudaError_t e_ = (expr);                                                                        \
    if (e_ != cudaSuccess)                                                                          \
      return ::scn::fail(SCN_E_CUDA, std::string(#expr) + ": " + cudaGetErrorString(e_));           \
  } while (0)
#define SCN_TRY(expr)                                                                               \
  do {                                                                                              \
    int r_ = (expr);                                                                                \
    if (r_ != SCN_OK) return r_;                                                                    \
  } while (0)

extern std::atomic<uint64_t> g_launches;
// Counts a launch and checks for a launch-configuration error.
#define SCN_LAUNCHED()                                                                              \
  do {                                                                                              \
    ::scn::g_launches.fetch_add(1, std::memory_order_relaxed);                                      \
    SCN_CUDA(cudaGetLastError());                                                                   \
  } while (0)

// ---- device memory: stream-ordered pool --------------------------------------
int dev_alloc(void **p, size_t bytes, cudaStream_t s);
void dev_free(void *p, cudaStream_t s);
template <typename T> int dev_alloc_t(T **p, size_t count, cudaStream_t s) {
  return dev_alloc(reinterpret_cast<void **>(p), count * sizeof(T), s);
}

// ---- key / table layout -----------------------------------------------------
// key = batch<<48 | z<<32 | y<<16 | x : ascending key order is batch-major, then z, y, x,
// the order the reference's packed key (z<<21 | y<<10 | x per batch grid) induces.
struct Slot {
  unsigned long long key;  // ~0 = empty
  int row;                 // site row
  int count;               // number of source points that fell in the site
};
static_assert(sizeof(Slot) == 16, "slot must be one 16-byte vector");
static const unsigned long long kEmptyKey = ~0ull;

// Written by the build kernels, read back by the host once per build.
struct BuildInfo {
  int mn[4];  // bounding box minimum  x,y,z,batch
  int mx[4];  // bounding box maximum
  unsigned int err;         // bit0: coordinate out of key range; bit1: a point outside the box the bitmap was laid out for
  unsigned int n_unique;    // sites found
  unsigned int max_active;  // most source points in one site
  unsigned int reserved;
};

// Bounding box in key order used to rank keys: pos = ((b*ez + z)*ey + y)*ex + x (box-relative).
struct Box {
  int o[4];            // origin x,y,z,b
  unsigned int e[4];   // extents
};

// One scale of a scene.
struct Grid {
  int64_t n = 0;           // active sites
  Box box = {{0, 0, 0, 0}, {0, 0, 0, 0}};  // the box the ranking structure is laid out for: contains every site (valid when n > 0)
  Box tight = {{0, 0, 0, 0}, {0, 0, 0, 0}};  // measured bounding box of the source points (input scale only)
  int32_t *coords = nullptr;  // SoA [4][n]: x, y, z, batch
  // open-addressing table key -> row: a second index beside the ranking structure below, filled on first use
  // (grid_ensure_table) because only the public coordinate query and the table dump read it
  mutable Slot *table = nullptr;
  mutable uint32_t mask = 0;  // capacity - 1
  // relation to the source rows this grid was built from (input points, or the sites of the
  // next finer scale):
  int64_t n_src = 0;
  int32_t *src_row = nullptr;   // [n_src] source -> site row
  int32_t *csr_off = nullptr;   // [n+1]  (nullptr when every site has exactly one source: off[i] = i)
  mutable int32_t *csr_item = nullptr;  // [n_src] sources of each site, ascending; when every site has one source it is
                                        // only made on request (grid_ensure_source_lists): row -> its source
  int32_t max_active = 0;
  // optional: how many points each site stands for, when that is not the length of its source list (a scene kept as
  // per-voxel sums hands in one entry per voxel that stands for all the points merged into it); owned by the grid
  int32_t *site_count = nullptr;
  // occupancy bitmap of the box in key order and the exclusive prefix sums of its word popcounts: the ranking
  // structure of the build, kept because "row of the site at (x,y,z)" = prefix[word] + popcount(bits below) answers
  // the neighbour queries of the 3x3x3 map with coherent reads instead of hash probes
  unsigned long long *bitmap = nullptr;
  uint32_t *prefix = nullptr;
  // submanifold 3x3x3 neighbour map: nbr[k*n + o] = input row of offset k for output o, or -1
  int32_t *nbr = nullptr;
  int64_t nbr_count[27] = {0};
  int64_t nbr_total = 0;
  // size-2/stride-2 relation to the next finer grid (valid on grids built by downsampling):
  int32_t *child = nullptr;      // [8][n]: fine row of offset k, or -1
  int32_t *fine_up = nullptr;    // [8][n_src]: up[k*n_src+f] = coarse row if offset(f)==k else -1
  int64_t child_count[8] = {0};
  // one allocation that holds several of the arrays above (coarse scales are built with all their buffers sized
  // up front): grid_free releases it once and skips the pointers that lie inside
  unsigned char *arena = nullptr;
  size_t arena_bytes = 0;
};

int grid_free(Grid &g, cudaStream_t s);
// Fills g.table from the site coordinates when it does not exist yet (capacity: the smallest power of two >= 2n, at
// least 16; linear probing cannot fail at that load).  No host round trip.
int grid_ensure_table(const Grid &g, cudaStream_t s);
int grid_ensure_source_lists(const Grid &g, cudaStream_t s);
// true when the next coarser scale of `fine_box` (every axis halved) is small enough for a ranking bitmap
bool coarse_box_fits_bitmap(const Box &fine_box, Box *coarse_box);

// Builds g from source points.  Exactly one of coords64 / coords_soa is given:
//   coords64  : int64 [n_src, ncols] rows (x,y,z[,b]) on the device
//   coords_soa: int32 SoA [4][n_src] on the device, shifted right by `shift` bits (downsampling)
// box_hint (optional): a box known to contain every source point; saves the host round trip that otherwise
// fetches the measured bounding box.
// with_ssc: also fill the 3x3x3 neighbour map before the build's last host round trip (saves the one
// grid_build_ssc would make).
int grid_build(Grid &g, const int64_t *coords64, int ncols, const int32_t *coords_soa, int shift,
               int64_t n_src, bool want_csr, const Box *box_hint, bool with_ssc, cudaStream_t s);
// a box that holds `tight` with a margin on the three spatial axes (clipped to the key range): what the next build of
// a similar scene is laid out for, so that it needs no round trip to measure its own
Box box_with_margin(const Box &tight, int margin);
// largest number of cells a ranking bitmap is laid out for; scenes whose bounding box is larger are ranked by sorting
// their keys and looked up through the open-addressing table
extern const unsigned long long kMaxDenseBits;
// The next coarser scale of `fine` (sites at coordinates >> 1) with its size-2/stride-2 maps and, on request,
// its neighbour map, in one pass with a single host round trip at the end: the site count stays
// on the device while the kernels run, buffers are sized by the bound n_coarse <= n_fine.
int grid_build_coarse(Grid &coarse, const Grid &fine, bool with_ssc, cudaStream_t s);
// `count` successive coarser scales of fine0 (levels[0] from fine0, levels[1] from levels[0], ...) chained on the
// device, one host round trip for all of them; buffers are sized by the bound n_level <= min(n_fine0, cells of the box)
int grid_build_coarse_chain(Grid *const *levels, int count, const Grid &fine0, bool with_ssc, cudaStream_t s);
int grid_build_ssc(Grid &g, cudaStream_t s);               // fills nbr / nbr_count
int grid_build_conv(Grid &coarse, const Grid &fine, cudaStream_t s);  // fills child / fine_up
// by_rank: answer from the grid's ranking structure (bitmap + prefix sums) instead of probing its hash table
int grid_query(const Grid &g, const int32_t *coords_soa, int64_t n, int64_t soa_stride, int32_t *rows, bool by_rank,
               cudaStream_t s);
// ordered compaction of a [K][n] map (entries >= 0) into `expected_pairs` pairs, k-major and ascending
// in the column inside each k.  swap = 0: pair (value, column); swap = 1: pair (column, value).
int map_to_pairs(const int32_t *map, int K, int64_t n, int swap, int64_t expected_pairs, int32_t *pairs_host,
                 cudaStream_t s);
int grid_locations(const Grid &g, int64_t *out_host, cudaStream_t s);
// incremental helpers
int build_incre_nbr(const Grid &g, const Grid &pre, const int32_t *pre_exist, int32_t *nbr2,
                    int64_t *counts_host, cudaStream_t s);
struct IncreNbrJob {
  const Grid *g, *pre;
  const int32_t *pre_exist;
  int32_t *nbr2;
  int64_t *counts_host;  // [27]
};
int build_incre_nbr_batch(const IncreNbrJob *jobs, int count, cudaStream_t s);
int build_incre_up(const Grid &coarse, const int32_t *pe_coarse, const int32_t *pe_fine, int32_t *up2,
                   cudaStream_t s);

// ---- feature kernels --------------------------------------------------------
// Optional second output of a gather-GEMM, formed in its epilogue from the finished row (after the init/bias term):
// leaky(v * scale[c] + shift[c]) as fp16 rows -- the BatchNorm + ReLU that follows the convolution in the network,
// handed to the next convolution without a pass of its own.  skip_raw: the fp32 result itself is not written.
struct EpiBn {
  const float *scale = nullptr;  // [n_planes_out]  gamma / sqrt(var + eps)
  const float *shift = nullptr;  // [n_planes_out]  beta - mean * scale
  float leak = 0.f;
  void *dst = nullptr;           // __half rows [n_out, stride]
  long long stride = 0;
  int skip_raw = 0;
  // incremental form (pre_exist given): for an output row that existed in the saved frame (pre_exist[row] >= 0) the
  // fp16 result is the residual act((v + x_saved) * scale + shift) - y_saved, with x_saved the saved frame's fp32 row
  // and y_saved its BatchNorm's fp16 row (CUDA/BatchNormalization.cu:112-150)
  const int32_t *pre_exist = nullptr;
  const float *pre_in = nullptr;
  long long pre_in_stride = 0;
  const void *pre_out = nullptr;  // __half rows
  long long pre_out_stride = 0;
};

// out[o] = (init ? init[o] : bias) + sum_k in[map[k*n_out + o]] * W[k]   (map == nullptr: identity, K = 1)
// init: rows [n_out, n_planes_out] with stride init_stride, or nullptr; it may be `out` itself (accumulate in place).
// in has in_rows rows; map entries are -1 or in [0, in_rows).
int gather_gemm(const float *in, int64_t in_stride, int64_t in_rows, const int32_t *map, int K, int64_t n_out, const float *W,
                const float *bias, float *out, int64_t out_stride, int64_t n_in, int64_t n_planes_out,
                const float *init, int64_t init_stride, int precision, cudaStream_t s);
// reads and clears the error word of the tensor-core kernels; synchronises s
int tc_check_errors(cudaStream_t s);
// narrow layers (n_in, n_out in {16, 32, 64}) run a warp-level mma.sync kernel with its own packed weight layout;
// which kernel a shape uses, and therefore which layout tc_pack_weights produces, depends on the shape alone
bool warp_mma_shape(int64_t K, int64_t Cin, int64_t Cout);
int warp_mma_pack(const float *W, int64_t K, int64_t Cin, int64_t Cout, float *packed, cudaStream_t s);
int gather_mma_warp(const float *in, int64_t in_stride, const int32_t *map, int K, int64_t n_out, const float *W,
                    const float *bias, float *out, int64_t out_stride, int64_t Cin, int64_t Cout, const float *init,
                    int64_t init_stride, bool packed,
                    cudaStream_t s, bool *handled);
bool tc_packable(int64_t K, int64_t Cin, int64_t Cout);
int tc_pack_weights(const float *W, int64_t K, int64_t Cin, int64_t Cout, float *packed, cudaStream_t s);
int nin_forward_noalloc(const float *in, int64_t in_stride, float *out, int64_t out_stride, int64_t rows,
                        const float *W, const float *bias, int64_t Cin, int64_t Cout, cudaStream_t s);
int bn_forward(const float *in, int64_t in_stride, float *out, int64_t out_stride, int64_t rows, int64_t planes,
               const float *mean, const float *var, const float *gamma, const float *beta, float eps,
               float leak, const int32_t *pre_exist, const float *pre_out, const float *pre_in,
               cudaStream_t s);
// BatchNorm + leaky ReLU (running statistics) with the result stored as fp16 rows (out: __half [rows, planes],
// out_stride in fp16 elements)
// pre_exist (optional, [rows]): incremental form, the residual against the saved frame's rows pre_out (fp16) / pre_in (fp32)
// affine_given: `mean` holds the per-plane scale and `var` the shift (gamma, beta, eps unused)
int bn_forward_f16out(const float *in, int64_t in_stride, void *out, int64_t out_stride, int64_t rows, int64_t planes,
                      const float *mean, const float *var, const float *gamma, const float *beta, float eps, float leak,
                      cudaStream_t s, const int32_t *pre_exist = nullptr, const void *pre_out = nullptr, int64_t pre_out_stride = 0,
                      const float *pre_in = nullptr, int64_t pre_in_stride = 0, bool affine_given = false);
// A second set of gathered rows for the same weights and the same output rows: out = init + sum_k in[map[k]] W[k] +
// sum_k in2[map2[k]] W[k] in one launch (the incremental submanifold convolution: residual rows of the changed
// neighbours and saved rows of the old neighbours of new sites).  Carried by the warp-level and slab fp16 kernels.
struct SecondRows {
  const void *in = nullptr;  // __half rows
  long long stride = 0;      // in fp16 elements
  const int32_t *map = nullptr;  // [K][n_out]
};
// true when an fp16 layer of this shape on this many rows runs on a kernel that takes SecondRows
bool f16_second_rows_ok(int64_t K, int64_t Cin, int64_t Cout, int64_t n_out);
// JoinTable + BatchNorm + leaky ReLU in one pass: joined = [a | b] (fp32 rows), rows16 = activation(joined * scale + shift) (fp16 rows)
int join_bn_forward_f16(const float *a, int64_t a_stride, int64_t a_planes, const float *b, int64_t b_stride, int64_t b_planes,
                        int64_t rows, float *joined, int64_t joined_stride, const float *scale, const float *shift, float leak,
                        void *rows16, int64_t rows16_stride, cudaStream_t s);
// fp16 form of the warp-level gather-GEMM: in = __half rows, weights packed by warp_mma_pack_f16 (fp16 fragments)
bool warp_mma_f16_shape(int64_t K, int64_t Cin, int64_t Cout);
// fp16 rows through the persistent tcgen05 kernel: planes multiples of 32, weights [vol][n_out][n_in padded to 64] fp16
bool tc_f16_shape(int64_t K, int64_t Cin, int64_t Cout);
int64_t tc_f16_packed_size(int64_t K, int64_t Cin, int64_t Cout);
int tc_pack_weights_f16(const float *W, int64_t K, int64_t Cin, int64_t Cout, void *packed, cudaStream_t s);
int gather_gemm_tc_f16(const void *in, int64_t in_stride, const int32_t *map, int K, int64_t n_out, const void *Wp,
                       const float *bias, float *out, int64_t out_stride, int64_t Cin, int64_t Cout, const float *init,
                       int64_t init_stride, cudaStream_t s, const EpiBn *epi = nullptr, const SecondRows *second = nullptr);
int warp_mma_pack_f16(const float *W, int64_t K, int64_t Cin, int64_t Cout, void *packed, cudaStream_t s);
// wide layers on small grids: 16 rows x 32 output planes per warp, whole reduction in one launch
// ascending row lists [4][cap] (int64) of the planes x == lo, hi - 1, lo - 1, hi (a side without a neighbour: empty) and their lengths
int halo_plane_lists(const int32_t *x, int64_t n, int lo, int hi, bool left, bool right, int64_t cap, int64_t *lists,
                     int64_t *counts, cudaStream_t s);
bool warp_slab_f16_shape(int64_t K, int64_t Cin, int64_t Cout);
extern int g_slab_share;
extern long long g_slab_max_rows;
int warp_mma_pack_f16_any(const float *W, int64_t K, int64_t Cin, int64_t Cout, void *packed, cudaStream_t s);
int gather_mma_slab_f16(const void *in, int64_t in_stride, const int32_t *map, int K, int64_t n_out, const void *Wp,
                        const float *bias, float *out, int64_t out_stride, int64_t Cin, int64_t Cout, const float *init,
                        int64_t init_stride, cudaStream_t s, const EpiBn *epi = nullptr, const SecondRows *second = nullptr);
int gather_mma_warp_f16(const void *in, int64_t in_stride, const int32_t *map, int K, int64_t n_out, const void *Wp,
                        const float *bias, float *out, int64_t out_stride, int64_t Cin, int64_t Cout, const float *init,
                        int64_t init_stride, cudaStream_t s, const EpiBn *epi = nullptr, const SecondRows *second = nullptr);
int bn_forward_train(const float *in, int64_t in_stride, float *out, int64_t out_stride, int64_t rows, int64_t planes,
                     float *running_mean, float *running_var, float *save_mean, float *save_invstd, const float *gamma,
                     const float *beta, float eps, float momentum, float leak, cudaStream_t s);
int input_forward(const Grid &g, const float *in, float *out, int64_t planes, int average,
                  const int32_t *pre_exist, const Grid *pre, const float *pre_out, cudaStream_t s);
int output_forward(const Grid &g, const float *in, float *out, int64_t planes, const int32_t *pre_exist,
                   const float *pre_in, cudaStream_t s);

}  // namespace scn
