// C ABI (include/insconv_b200.h) and the Metadata object behind it: per-scale grids, cached
// rulebook maps and pre-exist maps.  Host orchestration only; kernels live in grid_build.cu,
// feature_ops.cu and gather_gemm_tc.cu.
//
// Mirrors the roles of the reference's Metadata<3> (sparseconvnet/SCN/Metadata/Metadata.h:218-386,
// Metadata.cpp:442-463, 521-626, 669-697, 793-821) and of the cuda_* host functions in
// sparseconvnet/SCN/CUDA/{Convolution,Deconvolution,BatchNormalization,IOLayers,NetworkInNetwork}.cpp.
#include "internal.h"
#include <array>
#include <map>
#include <memory>
#include <mutex>
#include <vector>
#include <string.h>

namespace scn {

// ---- errors -----------------------------------------------------------------------------------
static thread_local std::string t_error;
void set_error(const std::string &msg) { t_error = msg; }
int fail(int code, const std::string &msg) {
  t_error = msg;
  return code;
}
std::atomic<uint64_t> g_launches{0};

// ---- device memory ----------------------------------------------------------------------------
// cudaMallocAsync on the device's default pool; the pool keeps freed blocks (release threshold
// raised once per device) so steady-state frames do not reach the driver allocator.
static std::mutex g_pool_mutex;
static bool g_pool_ready[64] = {false};
int dev_alloc(void **p, size_t bytes, cudaStream_t s) {
  *p = nullptr;
  if (bytes == 0) bytes = 16;
  int dev = 0;
  SCN_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !g_pool_ready[dev]) {
    std::lock_guard<std::mutex> lock(g_pool_mutex);
    if (!g_pool_ready[dev]) {
      cudaMemPool_t pool;
      SCN_CUDA(cudaDeviceGetDefaultMemPool(&pool, dev));
      uint64_t keep = ~0ull;
      SCN_CUDA(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep));
      g_pool_ready[dev] = true;
    }
  }
  SCN_CUDA(cudaMallocAsync(p, bytes, s));
  return SCN_OK;
}
void dev_free(void *p, cudaStream_t s) {
  if (p) cudaFreeAsync(p, s);
}

// ---- metadata ---------------------------------------------------------------------------------
typedef std::array<int64_t, 3> Size3;
static Size3 to_size(const int64_t *p) { return Size3{p[0], p[1], p[2]}; }

struct IncreMaps {  // per scale, relative to one saved metadata
  const void *pre = nullptr;
  int32_t *pre_exist = nullptr;  // [n]
  int32_t *nbr2 = nullptr;       // [27][n] rows of pre feeding new sites
  int64_t nbr2_count[27] = {0};
  int64_t nbr2_total = 0;
  int32_t *up2 = nullptr;        // [8][n_fine], stored on the coarse scale
};

}  // namespace scn

struct scn_metadata {
  std::map<scn::Size3, std::unique_ptr<scn::Grid>> grids;
  std::map<scn::Size3, scn::IncreMaps> incre;
  scn::Size3 input_size{{0, 0, 0}};
  bool has_input = false;
  int mode = 0;
  int64_t batch_size = 0;
  // the stream of the latest call that read this object's grids: what clear() releases them on, so that the release is
  // ordered behind every kernel that reads them (a build may have run on another stream than the layers)
  cudaStream_t last_stream = nullptr;
  // what the next scn_input_layer_build on this object builds beyond the input scale (-1: the process default), and
  // what the network that ran on it went on to ask for (the caller's record for its next frame)
  int ahead_ssc = -1, ahead_levels = -1;
  bool used_ssc = false;
  int used_levels = 0;
  // the box the next input-layer build lays its ranking bitmap out for without measuring first (the last build's
  // bounding box with a margin), and the point count it was measured on; both survive clear()
  scn::Box hint_box = {{0, 0, 0, 0}, {0, 0, 0, 0}};
  int64_t hint_points = 0;

  scn::Grid *find(const int64_t *size) {
    auto it = grids.find(scn::to_size(size));
    return it == grids.end() ? nullptr : it->second.get();
  }
  void clear(cudaStream_t s) {
    for (auto &kv : grids) scn::grid_free(*kv.second, s);
    grids.clear();
    for (auto &kv : incre) {
      scn::dev_free(kv.second.pre_exist, s);
      scn::dev_free(kv.second.nbr2, s);
      scn::dev_free(kv.second.up2, s);
    }
    incre.clear();
    has_input = false;
    used_ssc = false;
    used_levels = 0;
  }
};

namespace scn {

static int need_grid(scn_metadata *m, const int64_t *size, Grid **g) {
  if (!m || !size) return fail(SCN_E_INVALID, "null metadata or size");
  *g = m->find(size);
  if (!*g) {
    char buf[128];
    snprintf(buf, sizeof buf, "metadata has no grid at spatial size (%lld,%lld,%lld)", (long long)size[0],
             (long long)size[1], (long long)size[2]);
    return fail(SCN_E_STATE, buf);
  }
  return SCN_OK;
}

// What an input-layer build does beyond the input scale: the metadata's own setting (scn_metadata_set_build_ahead),
// else the process default (scn_set_build_ahead), else nothing.  A build ends with a host round trip, which in the
// middle of a network drains the queue of feature kernels first: a caller that knows what its network will ask for
// (the Python InputLayer reads it off the previous frame's metadata) has it built while the stream is still empty.
static std::atomic<int> g_force_ssc{-1}, g_force_levels{-1};
static bool want_ssc(const scn_metadata *m) {
  if (m->ahead_ssc >= 0) return m->ahead_ssc != 0;
  const int f = g_force_ssc.load(std::memory_order_relaxed);
  return f > 0;
}
static int want_levels(const scn_metadata *m) {
  if (m->ahead_levels >= 0) return m->ahead_levels;
  const int f = g_force_levels.load(std::memory_order_relaxed);
  return f > 0 ? f : 0;
}
static int ensure_ssc(scn_metadata *m, Grid &g, cudaStream_t s) {
  m->used_ssc = true;
  return grid_build_ssc(g, s);
}

// coarse grid of in_size -> out_size (filter 2, stride 2), built on first use
static int need_coarse(scn_metadata *m, const int64_t *in_size, const int64_t *out_size, Grid **fine, Grid **coarse,
                       cudaStream_t s) {
  SCN_TRY(need_grid(m, in_size, fine));
  for (int d = 0; d < 3; ++d)
    if (out_size[d] * 2 != in_size[d])
      return fail(SCN_E_UNSUPPORTED, "only filter size 2 / stride 2 convolutions are supported (input = 2 * output)");
  *coarse = m->find(out_size);
  if (!*coarse) {
    std::unique_ptr<Grid> g(new Grid());
    SCN_TRY(grid_build_coarse(*g, **fine, want_ssc(m), s));
    *coarse = g.get();
    m->grids[to_size(out_size)] = std::move(g);
  }
  if (m->has_input && out_size[0] > 0) {  // how deep below the input scale the network has gone
    int level = 0;
    for (int64_t sz = m->input_size[0]; sz > out_size[0] && sz % 2 == 0; sz /= 2) ++level;
    if (level > m->used_levels) m->used_levels = level;
  }
  if ((*coarse)->n_src != (*fine)->n) return fail(SCN_E_STATE, "coarse grid was not built from this fine grid");
  SCN_TRY(grid_build_conv(**coarse, **fine, s));
  return SCN_OK;
}

static int need_incre(scn_metadata *m, scn_metadata *pre, const int64_t *size, Grid **g, Grid **pg, IncreMaps **im,
                      cudaStream_t s) {
  if (!pre) return fail(SCN_E_INVALID, "null saved metadata");
  SCN_TRY(need_grid(m, size, g));
  SCN_TRY(need_grid(pre, size, pg));
  IncreMaps &x = m->incre[to_size(size)];
  if (x.pre != pre || !x.pre_exist) {
    dev_free(x.pre_exist, s);
    dev_free(x.nbr2, s);
    dev_free(x.up2, s);
    x = IncreMaps();
    x.pre = pre;
    int r = dev_alloc_t(&x.pre_exist, (size_t)(*g)->n, s);
    if (r == SCN_OK) r = grid_query(**pg, (*g)->coords, (*g)->n, (*g)->n, x.pre_exist, true, s);
    if (r != SCN_OK) {  // no half-made entry: the next call starts over
      dev_free(x.pre_exist, s);
      x = IncreMaps();
      return r;
    }
  }
  *im = &x;
  return SCN_OK;
}

// the C ABI's epilogue description -> the kernels' (init rows, second output); checks what can be checked here
static int take_epilogue(const scn_epilogue *epi, const float *bias, int64_t n_out, const float **init, int64_t *init_stride,
                         const float **bias_out, EpiBn *e, bool *has) {
  *init = nullptr;
  *init_stride = 0;
  *bias_out = bias;
  *has = false;
  if (!epi) return SCN_OK;
  if (epi->addend) {
    *init = epi->addend;
    *init_stride = epi->addend_stride;
    *bias_out = nullptr;
  }
  if (epi->bn_out) {
    if (!epi->bn_scale || !epi->bn_shift) return fail(SCN_E_INVALID, "fused BatchNorm output without scale / shift");
    if (epi->bn_out_stride < n_out) return fail(SCN_E_INVALID, "fused BatchNorm output stride smaller than the plane count");
    e->scale = epi->bn_scale;
    e->shift = epi->bn_shift;
    e->leak = (float)epi->bn_leakiness;
    e->dst = epi->bn_out;
    e->stride = epi->bn_out_stride;
    e->skip_raw = epi->skip_raw ? 1 : 0;
    if (epi->bn_pre_in || epi->bn_pre_out) {  // incremental form: the caller of this function adds pre_exist
      if (!epi->bn_pre_in || !epi->bn_pre_out || epi->skip_raw)
        return fail(SCN_E_INVALID, "incremental fused BatchNorm needs both saved row sets and a stored fp32 result");
      e->pre_in = epi->bn_pre_in;
      e->pre_in_stride = epi->bn_pre_in_stride;
      e->pre_out = epi->bn_pre_out;
      e->pre_out_stride = epi->bn_pre_out_stride;
    }
    *has = true;
  } else if (epi->skip_raw) {
    return fail(SCN_E_INVALID, "skip_raw without a fused BatchNorm output leaves nothing to compute");
  }
  return SCN_OK;
}

static int no_saved_rows(const scn_epilogue *epi) {
  if (epi && (epi->bn_pre_in || epi->bn_pre_out)) return fail(SCN_E_INVALID, "bn_pre_in / bn_pre_out belong to the incremental operators");
  return SCN_OK;
}

static int check_feat(const void *in, const void *out, const void *w, int64_t n_in, int64_t n_out) {
  if (!in || !out || !w) return fail(SCN_E_INVALID, "null feature or weight pointer");
  if (n_in <= 0 || n_out <= 0) return fail(SCN_E_INVALID, "plane counts must be positive");
  return SCN_OK;
}

// One convolution through the gather-GEMM; SCN_PREC_F16: `in` holds fp16 rows and `weight` fp16 fragments
static int run_conv(const float *in, int64_t in_stride, int64_t in_rows, const int32_t *map, int K, int64_t n_out,
                    const float *weight, const float *bias, float *out, int64_t out_stride, int64_t n_in, int64_t n_planes_out,
                    const float *init, int64_t init_stride, int precision, cudaStream_t s, const EpiBn *epi = nullptr,
                    const SecondRows *second = nullptr) {
  if (precision == SCN_PREC_F16) {  // narrow layers: warp-level kernel; wide layers: tcgen05 kernel
    if (warp_mma_f16_shape(K, n_in, n_planes_out))
      return gather_mma_warp_f16(in, in_stride, map, K, n_out, weight, bias, out, out_stride, n_in, n_planes_out, init,
                                 init_stride, s, epi, second);
    return gather_gemm_tc_f16(in, in_stride, map, K, n_out, weight, bias, out, out_stride, n_in, n_planes_out, init,
                              init_stride, s, epi, second);
  }
  if (second) return fail(SCN_E_UNSUPPORTED, "a second set of gathered rows needs fp16 rows (SCN_PREC_F16)");
  if (epi && epi->dst) return fail(SCN_E_UNSUPPORTED, "a fused BatchNorm output needs a convolution that reads fp16 rows (SCN_PREC_F16)");
  return gather_gemm(in, in_stride, in_rows, map, K, n_out, weight, bias, out, out_stride, n_in, n_planes_out, init,
                     init_stride, precision, s);
}

}  // namespace scn

using namespace scn;

extern "C" {

const char *scn_last_error(void) { return t_error.c_str(); }
const char *scn_version(void) { return "insconv_b200 0.1 (sm_100a)"; }
uint64_t scn_launch_count(void) { return g_launches.load(); }
int scn_set_slab_share(int warps) {
  if (warps != 0 && warps != 1 && warps != 2 && warps != 4 && warps != 8) return fail(SCN_E_INVALID, "0 (automatic), 1, 2, 4 or 8");
  g_slab_share = warps;
  return SCN_OK;
}
int scn_set_slab_max_rows(int64_t rows) {
  if (rows < 0) return fail(SCN_E_INVALID, "rows must not be negative");
  g_slab_max_rows = rows;
  return SCN_OK;
}
int scn_n_rulebook_bits(void) { return 32; }
int scn_check_errors(void *stream) {
  SCN_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  return tc_check_errors((cudaStream_t)stream);
}

int scn_metadata_create(scn_metadata **out) {
  if (!out) return fail(SCN_E_INVALID, "null output pointer");
  *out = new scn_metadata();
  return SCN_OK;
}
void scn_metadata_destroy(scn_metadata *m) {
  if (!m) return;
  m->clear(m->last_stream);
  delete m;
}
int scn_metadata_clear(scn_metadata *m, void *stream) {
  if (!m) return fail(SCN_E_INVALID, "null metadata");
  m->clear((cudaStream_t)stream);
  return SCN_OK;
}
int64_t scn_metadata_n_active(scn_metadata *m, const int64_t size[3]) {
  if (!m || !size) return -1;
  Grid *g = m->find(size);
  return g ? g->n : -1;
}
int scn_metadata_spatial_locations(scn_metadata *m, const int64_t size[3], int64_t *out_host, void *stream) {
  Grid *g;
  SCN_TRY(need_grid(m, size, &g));
  if (!out_host && g->n) return fail(SCN_E_INVALID, "null output");
  return grid_locations(*g, out_host, (cudaStream_t)stream);
}
int scn_metadata_site_coords(scn_metadata *m, const int64_t size[3], const int32_t **coords, int64_t *n) {
  Grid *g;
  SCN_TRY(need_grid(m, size, &g));
  if (coords) *coords = g->coords;
  if (n) *n = g->n;
  return SCN_OK;
}
int scn_metadata_hash_dump(scn_metadata *m, const int64_t size[3], uint64_t *keys_host, int32_t *rows_host,
                           int64_t *capacity, void *stream) {
  Grid *g;
  SCN_TRY(need_grid(m, size, &g));
  SCN_TRY(grid_ensure_table(*g, (cudaStream_t)stream));
  const int64_t cap = g->table ? (int64_t)g->mask + 1 : 0;
  if (capacity) *capacity = cap;
  if (!keys_host || !rows_host || cap == 0) return SCN_OK;
  std::vector<Slot> h((size_t)cap);
  cudaStream_t s = (cudaStream_t)stream;
  SCN_CUDA(cudaMemcpyAsync(h.data(), g->table, (size_t)cap * sizeof(Slot), cudaMemcpyDeviceToHost, s));
  SCN_CUDA(cudaStreamSynchronize(s));
  for (int64_t i = 0; i < cap; ++i) {
    keys_host[i] = h[i].key;
    rows_host[i] = h[i].key == kEmptyKey ? -1 : h[i].row;
  }
  return SCN_OK;
}
int scn_metadata_query(scn_metadata *m, const int64_t size[3], const int32_t *coords_soa, int64_t n, int32_t *rows,
                       void *stream) {
  Grid *g;
  SCN_TRY(need_grid(m, size, &g));
  if (n < 0 || (n && (!coords_soa || !rows))) return fail(SCN_E_INVALID, "bad query arguments");
  return grid_query(*g, coords_soa, n, n, rows, false, (cudaStream_t)stream);  // the hash table's query path
}

// ---- input / output layer ----------------------------------------------------------------------
int scn_set_build_ahead(int neighbour_maps, int coarse_levels) {
  if (neighbour_maps < -1 || neighbour_maps > 1 || coarse_levels < -1 || coarse_levels > 16)
    return fail(SCN_E_INVALID, "build-ahead settings out of range");
  g_force_ssc.store(neighbour_maps, std::memory_order_relaxed);
  g_force_levels.store(coarse_levels, std::memory_order_relaxed);
  return SCN_OK;
}

int scn_metadata_set_build_ahead(scn_metadata *m, int neighbour_maps, int coarse_levels) {
  if (!m) return fail(SCN_E_INVALID, "null metadata");
  if (neighbour_maps < -1 || neighbour_maps > 1 || coarse_levels < -1 || coarse_levels > 16)
    return fail(SCN_E_INVALID, "build-ahead settings out of range");
  m->ahead_ssc = neighbour_maps;
  m->ahead_levels = coarse_levels;
  return SCN_OK;
}
int scn_metadata_inherit(scn_metadata *m, const scn_metadata *previous) {
  if (!m || !previous) return fail(SCN_E_INVALID, "null metadata");
  m->ahead_ssc = (previous->used_ssc || previous->ahead_ssc > 0) ? 1 : previous->ahead_ssc;
  m->ahead_levels = previous->used_levels > previous->ahead_levels ? previous->used_levels : previous->ahead_levels;
  m->hint_box = previous->hint_box;
  m->hint_points = previous->hint_points;
  return SCN_OK;
}
int scn_metadata_build_used(scn_metadata *m, int *neighbour_maps, int *coarse_levels) {
  if (!m) return fail(SCN_E_INVALID, "null metadata");
  if (neighbour_maps) *neighbour_maps = m->used_ssc ? 1 : 0;
  if (coarse_levels) *coarse_levels = m->used_levels;
  return SCN_OK;
}

int scn_input_layer_build(scn_metadata *m, const int64_t size[3], const int64_t *coords, int coords_on_host,
                          int64_t n_in, int ncols, int64_t batch_size, int mode, void *stream, int64_t *n_active) {
  if (!m || !size) return fail(SCN_E_INVALID, "null metadata or size");
  if (mode != 3 && mode != 4) return fail(SCN_E_UNSUPPORTED, "InputLayer mode must be 3 (sum) or 4 (mean)");
  if (ncols != 3 && ncols != 4) return fail(SCN_E_INVALID, "coords must have 3 or 4 columns");
  if (n_in < 0 || (n_in && !coords)) return fail(SCN_E_INVALID, "bad coords");
  cudaStream_t s = (cudaStream_t)stream;
  m->last_stream = s;
  m->clear(s);
  std::unique_ptr<Grid> g(new Grid());
  const int64_t *dev_coords = coords;
  int64_t *staged = nullptr;
  if (coords_on_host && n_in) {
    SCN_TRY(dev_alloc_t(&staged, (size_t)n_in * ncols, s));
    SCN_CUDA(cudaMemcpyAsync(staged, coords, (size_t)n_in * ncols * 8, cudaMemcpyHostToDevice, s));
    dev_coords = staged;
  }
  // the last build's box serves when this frame is of a similar size (a much smaller or larger point set is
  // another kind of frame -- the changed sites of an incremental update, say -- and would only miss it)
  const bool use_hint = m->hint_points > 0 && n_in * 2 >= m->hint_points && n_in <= m->hint_points * 2;
  int r = grid_build(*g, dev_coords, ncols, nullptr, 0, n_in, true, use_hint ? &m->hint_box : nullptr, want_ssc(m), s);
  dev_free(staged, s);
  if (r != SCN_OK) {
    grid_free(*g, s);
    return r;
  }
  if (n_active) *n_active = g->n;
  if (g->n > 0) {
    m->hint_box = box_with_margin(g->tight, 16);
    m->hint_points = n_in;
  }
  m->grids[to_size(size)] = std::move(g);
  m->input_size = to_size(size);
  m->has_input = true;
  m->mode = mode;
  m->batch_size = batch_size;
  // the coarse scales earlier networks went down to, now rather than in the middle of the network, chained on the
  // device with one host round trip for all of them
  std::vector<Size3> sizes;
  Size3 cur = m->input_size;
  for (int level = 0, levels = want_levels(m); level < levels; ++level) {
    if (cur[0] % 2 || cur[1] % 2 || cur[2] % 2 || cur[0] < 2 || cur[1] < 2 || cur[2] < 2) break;
    cur = Size3{{cur[0] / 2, cur[1] / 2, cur[2] / 2}};
    sizes.push_back(cur);
  }
  if (!sizes.empty()) {
    std::vector<std::unique_ptr<Grid>> owned;
    std::vector<Grid *> ptrs;
    for (size_t i = 0; i < sizes.size(); ++i) {
      owned.emplace_back(new Grid());
      ptrs.push_back(owned.back().get());
    }
    const Grid *src = m->find(m->input_size.data());
    size_t first = 0;
    // scales too spread out for a ranking bitmap (or built from one that has none) one at a time, the rest chained
    while (first < sizes.size() && (!src->bitmap || !coarse_box_fits_bitmap(src->box, nullptr))) {
      SCN_TRY(grid_build_coarse(*ptrs[first], *src, want_ssc(m), s));
      src = ptrs[first];
      ++first;
    }
    if (first < sizes.size())
      SCN_TRY(grid_build_coarse_chain(ptrs.data() + first, (int)(ptrs.size() - first), *src, want_ssc(m), s));
    for (size_t i = 0; i < sizes.size(); ++i) m->grids[sizes[i]] = std::move(owned[i]);
  }
  return SCN_OK;
}

static int input_grid(scn_metadata *m, Grid **g) {
  if (!m || !m->has_input) return fail(SCN_E_STATE, "metadata has no input layer");
  *g = m->find(m->input_size.data());
  return *g ? SCN_OK : fail(SCN_E_STATE, "metadata has no input layer");
}

int scn_input_layer_forward(scn_metadata *m, const float *in, float *out, int64_t planes, void *stream) {
  Grid *g;
  SCN_TRY(input_grid(m, &g));
  m->last_stream = (cudaStream_t)stream;
  if (g->n && (!in || !out)) return fail(SCN_E_INVALID, "null features");
  return input_forward(*g, in, out, planes, m->mode == 4, nullptr, nullptr, nullptr, (cudaStream_t)stream);
}
int scn_output_layer_forward(scn_metadata *m, const float *in, float *out, int64_t planes, void *stream) {
  Grid *g;
  SCN_TRY(input_grid(m, &g));
  m->last_stream = (cudaStream_t)stream;
  if (g->n && (!in || !out)) return fail(SCN_E_INVALID, "null features");
  return output_forward(*g, in, out, planes, nullptr, nullptr, (cudaStream_t)stream);
}
int64_t scn_input_layer_n_points(scn_metadata *m) {
  Grid *g;
  if (input_grid(m, &g) != SCN_OK) return -1;
  return g->n_src;
}
int64_t scn_metadata_input_n_active(scn_metadata *m) {
  Grid *g;
  if (input_grid(m, &g) != SCN_OK) return -1;
  return g->n;
}
int scn_halo_plane_lists(scn_metadata *m, const int64_t size[3], int lo, int hi, int left, int right, int64_t cap,
                         int64_t *lists, int64_t *counts, void *stream) {
  Grid *g;
  SCN_TRY(need_grid(m, size, &g));
  if (cap < 0 || !counts || (cap && !lists)) return fail(SCN_E_INVALID, "scn_halo_plane_lists: bad argument");
  cudaStream_t s = (cudaStream_t)stream;
  if (g->n == 0) {
    SCN_CUDA(cudaMemsetAsync(counts, 0, 4 * sizeof(int64_t), s));
    return SCN_OK;
  }
  return halo_plane_lists(g->coords, g->n, lo, hi, left != 0, right != 0, cap, lists, counts, s);
}
int scn_input_layer_set_site_counts(scn_metadata *m, const int32_t *counts, int64_t n, void *stream) {
  Grid *g;
  SCN_TRY(input_grid(m, &g));
  if (n != g->n || (n && !counts)) return fail(SCN_E_INVALID, "one count per site of the input scale is expected");
  cudaStream_t s = (cudaStream_t)stream;
  if (n == 0) return SCN_OK;
  if (!g->site_count) SCN_TRY(dev_alloc_t(&g->site_count, (size_t)n, s));
  SCN_CUDA(cudaMemcpyAsync(g->site_count, counts, (size_t)n * 4, cudaMemcpyDeviceToDevice, s));
  return SCN_OK;
}
int scn_input_layer_rules(scn_metadata *m, int32_t header_host[4], int32_t *rows_host, void *stream) {
  Grid *g;
  SCN_TRY(input_grid(m, &g));
  cudaStream_t s = (cudaStream_t)stream;
  const int32_t max_active = g->n ? g->max_active : 0;
  if (header_host) {
    header_host[0] = m->mode;
    header_host[1] = max_active;
    header_host[2] = (int32_t)g->n_src;
    header_host[3] = (int32_t)g->n;
  }
  if (!rows_host || g->n == 0) return SCN_OK;
  SCN_TRY(grid_ensure_source_lists(*g, s));
  std::vector<int32_t> off((size_t)g->n + 1), item((size_t)g->n_src);
  if (g->csr_off) {
    SCN_CUDA(cudaMemcpyAsync(off.data(), g->csr_off, off.size() * 4, cudaMemcpyDeviceToHost, s));
  } else {
    for (size_t i = 0; i < off.size(); ++i) off[i] = (int32_t)i;
  }
  SCN_CUDA(cudaMemcpyAsync(item.data(), g->csr_item, item.size() * 4, cudaMemcpyDeviceToHost, s));
  SCN_CUDA(cudaStreamSynchronize(s));
  const int64_t w = 1 + max_active;
  memset(rows_host, 0, (size_t)(g->n * w) * 4);
  for (int64_t r = 0; r < g->n; ++r) {
    int32_t *row = rows_host + r * w;
    row[0] = off[r + 1] - off[r];
    for (int32_t j = off[r]; j < off[r + 1]; ++j) row[1 + j - off[r]] = item[j];
  }
  return SCN_OK;
}

// ---- rulebooks ---------------------------------------------------------------------------------
int scn_ssc_rulebook(scn_metadata *m, const int64_t size[3], int64_t counts_host[27], int32_t *pairs_host,
                     void *stream) {
  Grid *g;
  SCN_TRY(need_grid(m, size, &g));
  cudaStream_t s = (cudaStream_t)stream;
  SCN_TRY(ensure_ssc(m, *g, s));
  if (counts_host)
    for (int k = 0; k < 27; ++k) counts_host[k] = g->nbr_count[k];
  if (pairs_host) SCN_TRY(map_to_pairs(g->nbr, 27, g->n, 0, g->nbr_total, pairs_host, s));
  return SCN_OK;
}
int scn_conv_rulebook(scn_metadata *m, const int64_t in_size[3], const int64_t out_size[3], int64_t counts_host[8],
                      int32_t *pairs_host, void *stream) {
  Grid *fine, *coarse;
  cudaStream_t s = (cudaStream_t)stream;
  SCN_TRY(need_coarse(m, in_size, out_size, &fine, &coarse, s));
  if (counts_host)
    for (int k = 0; k < 8; ++k) counts_host[k] = coarse->child_count[k];
  // fine_up[k][f] = coarse row: pair (fine, coarse), ascending fine inside an offset
  if (pairs_host) SCN_TRY(map_to_pairs(coarse->fine_up, 8, fine->n, 1, fine->n, pairs_host, s));
  return SCN_OK;
}

// ---- feature ops -------------------------------------------------------------------------------
int scn_weights_packable(int64_t volume, int64_t n_in, int64_t n_out) { return tc_packable(volume, n_in, n_out) ? 1 : 0; }
int scn_pack_weights(const float *weight, int64_t volume, int64_t n_in, int64_t n_out, float *packed, void *stream) {
  return tc_pack_weights(weight, volume, n_in, n_out, packed, (cudaStream_t)stream);
}
int64_t scn_packed_size_f16(int64_t volume, int64_t n_in, int64_t n_out) {
  if (warp_mma_f16_shape(volume, n_in, n_out)) return volume * n_in * n_out;
  if (tc_f16_shape(volume, n_in, n_out)) return tc_f16_packed_size(volume, n_in, n_out);
  return 0;
}
int scn_weights_packable_f16(int64_t volume, int64_t n_in, int64_t n_out) {
  return scn_packed_size_f16(volume, n_in, n_out) > 0 ? 1 : 0;
}
int scn_pack_weights_f16(const float *weight, int64_t volume, int64_t n_in, int64_t n_out, void *packed, void *stream) {
  if (warp_mma_f16_shape(volume, n_in, n_out))
    return warp_mma_pack_f16(weight, volume, n_in, n_out, packed, (cudaStream_t)stream);
  return tc_pack_weights_f16(weight, volume, n_in, n_out, packed, (cudaStream_t)stream);
}
int scn_ssc_forward_ex(scn_metadata *m, const int64_t size[3], const float *in, int64_t in_stride, float *out,
                       int64_t out_stride, const float *weight, const float *bias, int64_t n_in, int64_t n_out, int precision,
                       const scn_epilogue *epi, void *stream, double *flops) {
  Grid *g;
  SCN_TRY(need_grid(m, size, &g));
  m->last_stream = (cudaStream_t)stream;
  if (flops) *flops = 0;
  if (g->n == 0) return SCN_OK;
  const float *init, *b;
  int64_t init_stride;
  EpiBn e;
  bool fused;
  SCN_TRY(take_epilogue(epi, bias, n_out, &init, &init_stride, &b, &e, &fused));
  SCN_TRY(check_feat(in, (fused && e.skip_raw) ? (const void *)weight : (const void *)out, weight, n_in, n_out));
  cudaStream_t s = (cudaStream_t)stream;
  SCN_TRY(no_saved_rows(epi));
  SCN_TRY(ensure_ssc(m, *g, s));
  SCN_TRY(run_conv(in, in_stride, g->n, g->nbr, 27, g->n, weight, b, out, out_stride, n_in, n_out, init, init_stride, precision, s,
                   fused ? &e : nullptr));
  if (flops) *flops = (double)g->nbr_total * (double)n_in * (double)n_out;
  return SCN_OK;
}
int scn_ssc_forward(scn_metadata *m, const int64_t size[3], const float *in, int64_t in_stride, float *out,
                    int64_t out_stride, const float *weight, const float *bias, int64_t n_in, int64_t n_out,
                    int precision, void *stream, double *flops) {
  return scn_ssc_forward_ex(m, size, in, in_stride, out, out_stride, weight, bias, n_in, n_out, precision, nullptr, stream, flops);
}
int scn_ssc_forward_add(scn_metadata *m, const int64_t size[3], const float *in, int64_t in_stride, float *out,
                        int64_t out_stride, const float *weight, const float *addend, int64_t addend_stride, int64_t n_in,
                        int64_t n_out, int precision, void *stream, double *flops) {
  if (!addend) return fail(SCN_E_INVALID, "null addend");
  scn_epilogue epi;
  memset(&epi, 0, sizeof epi);
  epi.addend = addend;
  epi.addend_stride = addend_stride;
  return scn_ssc_forward_ex(m, size, in, in_stride, out, out_stride, weight, nullptr, n_in, n_out, precision, &epi, stream, flops);
}
int scn_conv_prepare(scn_metadata *m, const int64_t in_size[3], const int64_t out_size[3], void *stream,
                     int64_t *n_active_out) {
  Grid *fine, *coarse;
  SCN_TRY(need_coarse(m, in_size, out_size, &fine, &coarse, (cudaStream_t)stream));
  if (n_active_out) *n_active_out = coarse->n;
  return SCN_OK;
}
static int conv_forward_impl(scn_metadata *m, scn_metadata *pre, const int64_t in_size[3], const int64_t out_size[3],
                             const float *in, int64_t in_stride, float *out, int64_t out_stride, const float *weight,
                             const float *bias, int64_t n_in, int64_t n_out, int precision, const scn_epilogue *epi,
                             cudaStream_t s, double *flops) {
  Grid *fine, *coarse;
  SCN_TRY(need_coarse(m, in_size, out_size, &fine, &coarse, s));
  m->last_stream = s;
  if (flops) *flops = 0;
  if (coarse->n == 0) return SCN_OK;
  const float *init, *b;
  int64_t init_stride;
  EpiBn e;
  bool fused;
  SCN_TRY(take_epilogue(epi, bias, n_out, &init, &init_stride, &b, &e, &fused));
  if (fused && e.pre_in) {  // incremental form: which coarse sites existed in the saved frame
    Grid *g2, *pg2;
    IncreMaps *im;
    SCN_TRY(need_incre(m, pre, out_size, &g2, &pg2, &im, s));
    e.pre_exist = im->pre_exist;
  }
  SCN_TRY(check_feat(in, (fused && e.skip_raw) ? (const void *)weight : (const void *)out, weight, n_in, n_out));
  SCN_TRY(run_conv(in, in_stride, fine->n, coarse->child, 8, coarse->n, weight, b, out, out_stride, n_in, n_out, init, init_stride,
                   precision, s, fused ? &e : nullptr));
  if (flops) *flops = (double)fine->n * (double)n_in * (double)n_out;
  return SCN_OK;
}
int scn_conv_forward_ex(scn_metadata *m, const int64_t in_size[3], const int64_t out_size[3], const float *in,
                        int64_t in_stride, float *out, int64_t out_stride, const float *weight, const float *bias, int64_t n_in,
                        int64_t n_out, int precision, const scn_epilogue *epi, void *stream, double *flops) {
  SCN_TRY(no_saved_rows(epi));
  return conv_forward_impl(m, nullptr, in_size, out_size, in, in_stride, out, out_stride, weight, bias, n_in, n_out, precision, epi,
                           (cudaStream_t)stream, flops);
}
int scn_incre_conv_forward_ex(scn_metadata *m, scn_metadata *pre, const int64_t in_size[3], const int64_t out_size[3],
                              const float *in, int64_t in_stride, float *out, int64_t out_stride, const float *weight,
                              const float *bias, int64_t n_in, int64_t n_out, int precision, const scn_epilogue *epi,
                              void *stream, double *flops) {
  if (epi && (epi->bn_pre_in || epi->bn_pre_out) && !pre) return fail(SCN_E_INVALID, "null saved metadata");
  return conv_forward_impl(m, pre, in_size, out_size, in, in_stride, out, out_stride, weight, bias, n_in, n_out, precision, epi,
                           (cudaStream_t)stream, flops);
}
int scn_conv_forward(scn_metadata *m, const int64_t in_size[3], const int64_t out_size[3], const float *in,
                     int64_t in_stride, float *out, int64_t out_stride, const float *weight, const float *bias,
                     int64_t n_in, int64_t n_out, int precision, void *stream, double *flops) {
  return scn_conv_forward_ex(m, in_size, out_size, in, in_stride, out, out_stride, weight, bias, n_in, n_out, precision, nullptr,
                             stream, flops);
}
int scn_deconv_forward_ex(scn_metadata *m, const int64_t in_size[3], const int64_t out_size[3], const float *in,
                          int64_t in_stride, float *out, int64_t out_stride, const float *weight, const float *bias,
                          int64_t n_in, int64_t n_out, int precision, const scn_epilogue *epi, void *stream, double *flops) {
  Grid *fine, *coarse;
  cudaStream_t s = (cudaStream_t)stream;
  SCN_TRY(no_saved_rows(epi));
  SCN_TRY(need_coarse(m, out_size, in_size, &fine, &coarse, s));
  m->last_stream = s;
  if (flops) *flops = 0;
  if (fine->n == 0) return SCN_OK;
  const float *init, *b;
  int64_t init_stride;
  EpiBn e;
  bool fused;
  SCN_TRY(take_epilogue(epi, bias, n_out, &init, &init_stride, &b, &e, &fused));
  SCN_TRY(check_feat(in, (fused && e.skip_raw) ? (const void *)weight : (const void *)out, weight, n_in, n_out));
  SCN_TRY(run_conv(in, in_stride, coarse->n, coarse->fine_up, 8, fine->n, weight, b, out, out_stride, n_in, n_out, init, init_stride,
                   precision, s, fused ? &e : nullptr));
  if (flops) *flops = (double)fine->n * (double)n_in * (double)n_out;
  return SCN_OK;
}
int scn_deconv_forward(scn_metadata *m, const int64_t in_size[3], const int64_t out_size[3], const float *in,
                       int64_t in_stride, float *out, int64_t out_stride, const float *weight, const float *bias,
                       int64_t n_in, int64_t n_out, int precision, void *stream, double *flops) {
  return scn_deconv_forward_ex(m, in_size, out_size, in, in_stride, out, out_stride, weight, bias, n_in, n_out, precision, nullptr,
                               stream, flops);
}
int scn_join_bn_forward_f16(const float *a, int64_t a_stride, int64_t a_planes, const float *b, int64_t b_stride, int64_t b_planes,
                            int64_t rows, float *joined, int64_t joined_stride, const float *scale, const float *shift,
                            double leakiness, void *rows_f16, int64_t rows_f16_stride, void *stream) {
  if (rows < 0) return fail(SCN_E_INVALID, "negative size");
  if (rows && (!a || !b || !joined || !scale || !shift || !rows_f16)) return fail(SCN_E_INVALID, "null pointer");
  return join_bn_forward_f16(a, a_stride, a_planes, b, b_stride, b_planes, rows, joined, joined_stride, scale, shift, (float)leakiness,
                             rows_f16, rows_f16_stride, (cudaStream_t)stream);
}

int scn_bn_forward_f16(const float *in, int64_t in_stride, void *out, int64_t out_stride, int64_t rows, int64_t planes,
                       const float *running_mean, const float *running_var, const float *gamma, const float *beta,
                       double eps, double leakiness, void *stream) {
  if (rows < 0 || planes < 0) return fail(SCN_E_INVALID, "negative size");
  if (rows && planes && (!in || !out || !running_mean || !running_var)) return fail(SCN_E_INVALID, "null pointer");
  return bn_forward_f16out(in, in_stride, out, out_stride, rows, planes, running_mean, running_var, gamma, beta, (float)eps,
                           (float)leakiness, (cudaStream_t)stream);
}
int scn_bn_forward(const float *in, int64_t in_stride, float *out, int64_t out_stride, int64_t rows, int64_t planes,
                   const float *running_mean, const float *running_var, const float *gamma, const float *beta,
                   double eps, double leakiness, void *stream) {
  if (rows < 0 || planes < 0) return fail(SCN_E_INVALID, "negative size");
  if (rows && planes && (!in || !out || !running_mean || !running_var)) return fail(SCN_E_INVALID, "null pointer");
  return bn_forward(in, in_stride, out, out_stride, rows, planes, running_mean, running_var, gamma, beta, (float)eps,
                    (float)leakiness, nullptr, nullptr, nullptr, (cudaStream_t)stream);
}
int scn_bn_forward_train(const float *in, int64_t in_stride, float *out, int64_t out_stride, int64_t rows,
                         int64_t planes, float *running_mean, float *running_var, float *save_mean,
                         float *save_invstd, const float *gamma, const float *beta, double eps, double momentum,
                         double leakiness, void *stream) {
  if (rows < 0 || planes < 0) return fail(SCN_E_INVALID, "negative size");
  if (rows && planes && (!in || !out || !running_mean || !running_var)) return fail(SCN_E_INVALID, "null pointer");
  if (rows == 1) return fail(SCN_E_INVALID, "batch statistics need at least two rows");
  return bn_forward_train(in, in_stride, out, out_stride, rows, planes, running_mean, running_var, save_mean,
                          save_invstd, gamma, beta, (float)eps, (float)momentum, (float)leakiness, (cudaStream_t)stream);
}
int scn_nin_forward(const float *in, int64_t in_stride, float *out, int64_t out_stride, int64_t rows,
                    const float *weight, const float *bias, int64_t n_in, int64_t n_out, int precision, void *stream,
                    double *flops) {
  if (flops) *flops = (double)rows * (double)n_in * (double)n_out;
  if (rows == 0) return SCN_OK;
  SCN_TRY(check_feat(in, out, weight, n_in, n_out));
  return gather_gemm(in, in_stride, rows, nullptr, 1, rows, weight, bias, out, out_stride, n_in, n_out, nullptr, 0, precision,
                     (cudaStream_t)stream);
}

int scn_nin_forward_noalloc(const float *in, int64_t in_stride, float *out, int64_t out_stride, int64_t rows,
                            const float *weight, const float *bias, int64_t n_in, int64_t n_out, void *stream) {
  return nin_forward_noalloc(in, in_stride, out, out_stride, rows, weight, bias, n_in, n_out, (cudaStream_t)stream);
}

// ---- incremental path --------------------------------------------------------------------------
int scn_incre_pre_exist(scn_metadata *m, scn_metadata *pre, const int64_t size[3], const int32_t **map, int64_t *n,
                        void *stream) {
  Grid *g, *pg;
  IncreMaps *im;
  SCN_TRY(need_incre(m, pre, size, &g, &pg, &im, (cudaStream_t)stream));
  if (map) *map = im->pre_exist;
  if (n) *n = g->n;
  return SCN_OK;
}
int scn_incre_input_layer_forward(scn_metadata *m, scn_metadata *pre, const float *in, float *out,
                                  const float *pre_out, int64_t planes, void *stream) {
  Grid *g0;
  SCN_TRY(input_grid(m, &g0));
  Grid *g, *pg;
  IncreMaps *im;
  cudaStream_t s = (cudaStream_t)stream;
  SCN_TRY(need_incre(m, pre, m->input_size.data(), &g, &pg, &im, s));
  if (g->n && (!in || !out || !pre_out)) return fail(SCN_E_INVALID, "null features");
  // The incremental neighbour maps of every scale both frames have, now and with one host round trip, instead of
  // one round trip per scale in the middle of the network (once a network has used neighbour maps at all).
  if (want_ssc(m)) {
    std::vector<IncreNbrJob> jobs;
    std::vector<IncreMaps *> ims;
    for (auto &kv : m->grids) {
      Grid *gl = kv.second.get(), *pl = pre->find(kv.first.data());
      if (!pl || gl->n == 0) continue;
      Grid *g2, *p2;
      IncreMaps *im2;
      SCN_TRY(need_incre(m, pre, kv.first.data(), &g2, &p2, &im2, s));
      if (im2->nbr2) continue;
      SCN_TRY(dev_alloc_t(&im2->nbr2, (size_t)gl->n * 27, s));
      jobs.push_back(IncreNbrJob{gl, pl, im2->pre_exist, im2->nbr2, im2->nbr2_count});
      ims.push_back(im2);
    }
    SCN_TRY(build_incre_nbr_batch(jobs.data(), (int)jobs.size(), s));
    for (IncreMaps *x : ims) {
      x->nbr2_total = 0;
      for (int k = 0; k < 27; ++k) x->nbr2_total += x->nbr2_count[k];
    }
  }
  return input_forward(*g, in, out, planes, m->mode == 4, im->pre_exist, pg, pre_out, s);
}
int scn_incre_output_layer_forward(scn_metadata *m, scn_metadata *pre, const float *in, float *out,
                                   const float *pre_in, int64_t planes, void *stream) {
  Grid *g0;
  SCN_TRY(input_grid(m, &g0));
  Grid *g, *pg;
  IncreMaps *im;
  cudaStream_t s = (cudaStream_t)stream;
  SCN_TRY(need_incre(m, pre, m->input_size.data(), &g, &pg, &im, s));
  if (g->n && (!in || !out || !pre_in)) return fail(SCN_E_INVALID, "null features");
  return output_forward(*g, in, out, planes, im->pre_exist, pre_in, s);
}

static int need_nbr2(Grid *g, Grid *pg, IncreMaps *im, cudaStream_t s) {
  if (im->nbr2 || g->n == 0) return SCN_OK;
  SCN_TRY(dev_alloc_t(&im->nbr2, (size_t)g->n * 27, s));
  SCN_TRY(build_incre_nbr(*g, *pg, im->pre_exist, im->nbr2, im->nbr2_count, s));
  im->nbr2_total = 0;
  for (int k = 0; k < 27; ++k) im->nbr2_total += im->nbr2_count[k];
  return SCN_OK;
}

int scn_incre_ssc_forward_ex(scn_metadata *m, scn_metadata *pre, const int64_t size[3], const float *in,
                             int64_t in_stride, float *out, int64_t out_stride, const float *weight, const float *bias,
                             const float *pre_in, int64_t pre_in_stride, int64_t n_in, int64_t n_out, int precision,
                             const scn_epilogue *epi, void *stream, double *flops) {
  Grid *g, *pg;
  IncreMaps *im;
  cudaStream_t s = (cudaStream_t)stream;
  SCN_TRY(need_incre(m, pre, size, &g, &pg, &im, s));
  if (flops) *flops = 0;
  if (g->n == 0) return SCN_OK;
  SCN_TRY(check_feat(in, out, weight, n_in, n_out));
  if (!pre_in) return fail(SCN_E_INVALID, "null saved features");
  const float *init = nullptr, *bias1 = bias;
  int64_t init_stride = 0;
  EpiBn e;
  bool has = false;
  SCN_TRY(take_epilogue(epi, bias, n_out, &init, &init_stride, &bias1, &e, &has));
  if (has && e.pre_in) e.pre_exist = im->pre_exist;
  SCN_TRY(ensure_ssc(m, *g, s));
  SCN_TRY(need_nbr2(g, pg, im, s));
  // the epilogue rides on the last pass: the second one (saved neighbours of new sites) when there is one
  const bool two = im->nbr2_total != 0;
  if (two && precision == SCN_PREC_F16 && f16_second_rows_ok(27, n_in, n_out, g->n)) {
    // both gathers in one launch: the kernel walks the second map through the same accumulators
    SecondRows second;
    second.in = pre_in;
    second.stride = pre_in_stride;
    second.map = im->nbr2;
    SCN_TRY(run_conv(in, in_stride, g->n, g->nbr, 27, g->n, weight, bias1, out, out_stride, n_in, n_out, init, init_stride, precision,
                     s, has ? &e : nullptr, &second));
    if (flops) *flops = (double)(g->nbr_total + im->nbr2_total) * (double)n_in * (double)n_out;
    return SCN_OK;
  }
  SCN_TRY(run_conv(in, in_stride, g->n, g->nbr, 27, g->n, weight, bias1, out, out_stride, n_in, n_out, init, init_stride, precision, s,
                   has && !two ? &e : nullptr));
  if (two)
    SCN_TRY(run_conv(pre_in, pre_in_stride, pg->n, im->nbr2, 27, g->n, weight, nullptr, out, out_stride, n_in, n_out, out, out_stride,
                     precision, s, has ? &e : nullptr));
  if (flops) *flops = (double)(g->nbr_total + im->nbr2_total) * (double)n_in * (double)n_out;
  return SCN_OK;
}
int scn_incre_ssc_forward(scn_metadata *m, scn_metadata *pre, const int64_t size[3], const float *in,
                          int64_t in_stride, float *out, int64_t out_stride, const float *weight, const float *bias,
                          const float *pre_in, int64_t pre_in_stride, int64_t n_in, int64_t n_out, int precision,
                          void *stream, double *flops) {
  return scn_incre_ssc_forward_ex(m, pre, size, in, in_stride, out, out_stride, weight, bias, pre_in, pre_in_stride, n_in, n_out,
                                  precision, nullptr, stream, flops);
}
int scn_incre_ssc_rulebook(scn_metadata *m, scn_metadata *pre, const int64_t size[3], int64_t counts_host[27],
                           int32_t *pairs_host, void *stream) {
  Grid *g, *pg;
  IncreMaps *im;
  cudaStream_t s = (cudaStream_t)stream;
  SCN_TRY(need_incre(m, pre, size, &g, &pg, &im, s));
  SCN_TRY(need_nbr2(g, pg, im, s));
  if (counts_host)
    for (int k = 0; k < 27; ++k) counts_host[k] = im->nbr2_count[k];
  if (pairs_host && g->n) SCN_TRY(map_to_pairs(im->nbr2, 27, g->n, 0, im->nbr2_total, pairs_host, s));
  return SCN_OK;
}
int scn_incre_deconv_forward(scn_metadata *m, scn_metadata *pre, const int64_t in_size[3], const int64_t out_size[3],
                             const float *in, int64_t in_stride, float *out, int64_t out_stride, const float *weight,
                             const float *bias, const float *pre_in, int64_t pre_in_stride, int64_t n_in,
                             int64_t n_out, int precision, void *stream, double *flops) {
  Grid *fine, *coarse;
  cudaStream_t s = (cudaStream_t)stream;
  SCN_TRY(need_coarse(m, out_size, in_size, &fine, &coarse, s));
  if (flops) *flops = 0;
  if (fine->n == 0) return SCN_OK;
  SCN_TRY(check_feat(in, out, weight, n_in, n_out));
  if (!pre_in) return fail(SCN_E_INVALID, "null saved features");
  Grid *g1, *pg1, *g2, *pg2;
  IncreMaps *im_c, *im_f;
  SCN_TRY(need_incre(m, pre, in_size, &g1, &pg1, &im_c, s));
  SCN_TRY(need_incre(m, pre, out_size, &g2, &pg2, &im_f, s));
  if (!im_c->up2) {
    SCN_TRY(dev_alloc_t(&im_c->up2, (size_t)fine->n * 8, s));
    SCN_TRY(build_incre_up(*coarse, im_c->pre_exist, im_f->pre_exist, im_c->up2, s));
  }
  if (precision == SCN_PREC_F16 && f16_second_rows_ok(8, n_in, n_out, fine->n)) {  // both gathers in one launch
    SecondRows second;
    second.in = pre_in;
    second.stride = pre_in_stride;
    second.map = im_c->up2;
    SCN_TRY(run_conv(in, in_stride, coarse->n, coarse->fine_up, 8, fine->n, weight, bias, out, out_stride, n_in, n_out, nullptr, 0,
                     precision, s, nullptr, &second));
  } else {
    SCN_TRY(run_conv(in, in_stride, coarse->n, coarse->fine_up, 8, fine->n, weight, bias, out, out_stride, n_in, n_out, nullptr, 0,
                     precision, s));
    SCN_TRY(run_conv(pre_in, pre_in_stride, pg1->n, im_c->up2, 8, fine->n, weight, nullptr, out, out_stride, n_in, n_out, out,
                     out_stride, precision, s));
  }
  if (flops) *flops = (double)fine->n * (double)n_in * (double)n_out;
  return SCN_OK;
}
int scn_incre_bn_forward(scn_metadata *m, scn_metadata *pre, const int64_t size[3], const float *in, int64_t in_stride,
                         float *out, int64_t out_stride, int64_t planes, const float *running_mean,
                         const float *running_var, const float *gamma, const float *beta, double eps,
                         double leakiness, const float *pre_out, const float *pre_in, void *stream) {
  Grid *g, *pg;
  IncreMaps *im;
  cudaStream_t s = (cudaStream_t)stream;
  SCN_TRY(need_incre(m, pre, size, &g, &pg, &im, s));
  if (g->n == 0) return SCN_OK;
  if (!in || !out || !running_mean || !running_var || !pre_out || !pre_in) return fail(SCN_E_INVALID, "null pointer");
  return bn_forward(in, in_stride, out, out_stride, g->n, planes, running_mean, running_var, gamma, beta, (float)eps,
                    (float)leakiness, im->pre_exist, pre_out, pre_in, s);
}
int scn_incre_bn_forward_f16(scn_metadata *m, scn_metadata *pre, const int64_t size[3], const float *in, int64_t in_stride,
                             void *out, int64_t out_stride, int64_t planes, const float *running_mean,
                             const float *running_var, const float *gamma, const float *beta, double eps, double leakiness,
                             const void *pre_out, int64_t pre_out_stride, const float *pre_in, int64_t pre_in_stride,
                             void *stream) {
  Grid *g, *pg;
  IncreMaps *im;
  cudaStream_t s = (cudaStream_t)stream;
  SCN_TRY(need_incre(m, pre, size, &g, &pg, &im, s));
  if (g->n == 0) return SCN_OK;
  if (!in || !out || !running_mean || !running_var || !pre_out || !pre_in) return fail(SCN_E_INVALID, "null pointer");
  return bn_forward_f16out(in, in_stride, out, out_stride, g->n, planes, running_mean, running_var, gamma, beta, (float)eps,
                           (float)leakiness, s, im->pre_exist, pre_out, pre_out_stride, pre_in, pre_in_stride);
}

}  // extern "C"
