// Grid (voxel hash) and rulebook construction kernels.
//
// A grid is built from source rows (input points, or the sites of the next finer scale) in four
// device passes, none of which sorts:
//   1. pack      coordinates -> 64-bit keys, bounding box of the scene          (reads coords once)
//   2. mark      one bit per occupied cell in a bitmap laid out in key order    (atomicOr, L2 resident)
//   3. rank      exclusive prefix sum of the bitmap word popcounts
//   4. assign    row of a source = prefix[word] + popcount(bits below): the rank of its key among the unique
//                keys, which is the reference's site numbering; every source writes its site's coordinates
//                (sources of one site write the same values, so no arbitration is needed).
// Bitmap and prefixes stay with the grid and answer every later lookup (neighbour queries of the 3x3x3
// rulebook, pre-exist maps, incremental rulebooks) with one or two coherent reads.  The open-addressing table
// key -> row (linear probing, 16-byte slots, load factor <= 0.5) serves the public coordinate query and is
// filled from the site coordinates the first time it is asked for.
//
// Reference behaviour restated here (paths relative to sparseconvnet/SCN/):
//   key order / site numbering   CUDA/CUDPPWrapper.cu:72-119, extra/cudpp/src/cudpp_hash/hash_multivalue.cpp:45-110
//   site coords, point -> site   CUDA/CUDPPWrapper.cu:212-231
//   input rules                  CUDA/CUDPPWrapper.cu:53-64, Metadata/IOLayersRules.h:135-203
//   3x3x3 offsets and pairs      CUDA/SubmanifoldRules_cuda.cu:45-114
//   2x2x2 stride-2 pairs         CUDA/SubmanifoldRules_cuda.cu:744-780, Metadata/ConvolutionRules.h:344-380
#include "internal.h"
#include <vector>
#include <limits.h>

namespace scn {

// ---------------------------------------------------------------------------------------------
// device helpers
// ---------------------------------------------------------------------------------------------
__host__ __device__ __forceinline__ unsigned long long pack_key(int x, int y, int z, int b) {
  return ((unsigned long long)(unsigned)b << 48) | ((unsigned long long)(unsigned)z << 32) |
         ((unsigned long long)(unsigned)y << 16) | (unsigned long long)(unsigned)x;
}
__device__ __forceinline__ void unpack_key(unsigned long long k, int &x, int &y, int &z, int &b) {
  x = (int)(k & 0xFFFF);
  y = (int)((k >> 16) & 0xFFFF);
  z = (int)((k >> 32) & 0xFFFF);
  b = (int)(k >> 48);
}
// murmur3 finaliser: spreads the low-entropy packed coordinates over the table.
__device__ __forceinline__ uint32_t hash_key(unsigned long long k) {
  k ^= k >> 33;
  k *= 0xff51afd7ed558ccdULL;
  k ^= k >> 33;
  k *= 0xc4ceb9fe1a85ec53ULL;
  k ^= k >> 33;
  return (uint32_t)k;
}
__device__ __forceinline__ bool coord_ok(long long x, long long y, long long z, long long b) {
  return x >= 0 && y >= 0 && z >= 0 && b >= 0 && x <= SCN_MAX_COORD && y <= SCN_MAX_COORD &&
         z <= SCN_MAX_COORD && b <= SCN_MAX_BATCH;
}
// Open-addressing table, linear probing, probed by TEAMS of four lanes: the four lanes read four consecutive 16-byte
// slots -- one aligned 64-byte line -- per step and vote, so a probe sequence costs one memory round trip per four
// slots instead of one per slot, and every load of a warp is a whole line.  The window that holds the key's home slot
// is aligned down to a multiple of four; slots in front of the home slot are not on the key's probe path and are
// ignored in that first window.  All four lanes of a team call with the same key.  Capacity is a power of two >= 16.
constexpr int kTeam = 4;

__device__ __forceinline__ int table_find_team(const Slot *__restrict__ t, uint32_t mask, unsigned long long key,
                                               unsigned team_mask, int lane) {
  const uint32_t h = hash_key(key) & mask;
  uint32_t base = h & ~(uint32_t)(kTeam - 1);
  const uint32_t windows = (mask + 1) / kTeam;
  const int j = lane & (kTeam - 1);
  for (uint32_t w = 0; w <= windows; ++w) {  // bounded: at most one sweep of the table
    const uint32_t idx = base + (uint32_t)j;
    const ulonglong2 s = __ldg(reinterpret_cast<const ulonglong2 *>(t + idx));
    const bool on_path = w > 0 || idx >= h;
    const unsigned hit = __ballot_sync(team_mask, on_path && s.x == key);
    if (hit) return __shfl_sync(team_mask, (int)(uint32_t)(s.y & 0xFFFFFFFFull), __ffs(hit) - 1);
    if (__ballot_sync(team_mask, on_path && s.x == kEmptyKey)) return -1;
    base = (base + kTeam) & mask;
  }
  return -1;
}

__device__ __forceinline__ unsigned long long box_pos(const Box &bx, int x, int y, int z, int b) {
  return (((unsigned long long)(unsigned)(b - bx.o[3]) * bx.e[2] + (unsigned)(z - bx.o[2])) * bx.e[1] +
          (unsigned)(y - bx.o[1])) * bx.e[0] + (unsigned)(x - bx.o[0]);
}

// Sets bit p of the bitmap.  Most cells hold one point, but duplicates and neighbours share words: the atomic is
// skipped when the bit already shows.  (Combining the bits of a warp's lanes that hit the same word first, with
// match.any and shuffles, measured slower: 101 us against 64 us for 4 M points.)
__device__ __forceinline__ void mark_bit(unsigned long long *bitmap, unsigned long long p, bool active) {
  if (!active) return;
  const unsigned long long bit = 1ull << (p & 63);
  unsigned long long *w = bitmap + (p >> 6);
  if ((*(volatile unsigned long long *)w & bit) == 0) atomicOr(w, bit);
}

// ---------------------------------------------------------------------------------------------
// pass 1: keys + bounding box
// ---------------------------------------------------------------------------------------------
__global__ void k_init_info(BuildInfo *info) {
  if (threadIdx.x < 4) {
    info->mn[threadIdx.x] = INT_MAX;
    info->mx[threadIdx.x] = INT_MIN;
  }
  if (threadIdx.x == 0) {
    info->err = 0;
    info->n_unique = 0;
    info->max_active = 0;
    info->reserved = 0;
  }
}

// Bounding box: warp shuffle, then one shared-memory round per block, then at most eight global
// atomics per block -- and none when the block cannot widen the box it already sees.
__device__ __forceinline__ void reduce_box(int x, int y, int z, int b, bool valid, BuildInfo *info) {
  __shared__ int s_mn[8][4], s_mx[8][4];  // blocks have at most 8 warps
  int mn[4] = {valid ? x : INT_MAX, valid ? y : INT_MAX, valid ? z : INT_MAX, valid ? b : INT_MAX};
  int mx[4] = {valid ? x : INT_MIN, valid ? y : INT_MIN, valid ? z : INT_MIN, valid ? b : INT_MIN};
#pragma unroll
  for (int d = 0; d < 4; ++d) {
    mn[d] = __reduce_min_sync(0xffffffffu, mn[d]);
    mx[d] = __reduce_max_sync(0xffffffffu, mx[d]);
  }
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  if (lane == 0) {
#pragma unroll
    for (int d = 0; d < 4; ++d) {
      s_mn[wid][d] = mn[d];
      s_mx[wid][d] = mx[d];
    }
  }
  __syncthreads();
  if (threadIdx.x < 8) {
    const int d = threadIdx.x & 3;
    const bool is_max = threadIdx.x >= 4;
    const int nw = (blockDim.x + 31) >> 5;
    int v = is_max ? INT_MIN : INT_MAX;
    for (int w = 0; w < nw; ++w) v = is_max ? max(v, s_mx[w][d]) : min(v, s_mn[w][d]);
    if (is_max) {
      if (v != INT_MIN && v > *(volatile int *)&info->mx[d]) atomicMax(&info->mx[d], v);
    } else {
      if (v != INT_MAX && v < *(volatile int *)&info->mn[d]) atomicMin(&info->mn[d], v);
    }
  }
}

// int64 AoS rows (x,y,z[,b]) -> keys.  One thread per point; blocks are multiples of 32 threads and
// every lane of a warp reaches reduce_box (the tail is padded with invalid lanes).
__global__ void k_pack_keys_i64(const long long *__restrict__ coords, int ncols, int vec, long long n,
                                unsigned long long *__restrict__ keys, BuildInfo *info) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  bool valid = i < n;
  long long x = 0, y = 0, z = 0, b = 0;
  if (valid) {
    if (vec) {  // ncols == 4 and 16-byte aligned base: two 16-byte loads per point
      const longlong2 *p = reinterpret_cast<const longlong2 *>(coords + 4 * i);
      longlong2 a = __ldg(p), c = __ldg(p + 1);
      x = a.x; y = a.y; z = c.x; b = c.y;
    } else {
      const long long *p = coords + (long long)ncols * i;
      x = p[0]; y = p[1]; z = p[2];
      b = ncols > 3 ? p[3] : 0;
    }
    if (!coord_ok(x, y, z, b)) {
      atomicOr(&info->err, 1u);
      valid = false;
      keys[i] = 0;
    } else {
      keys[i] = pack_key((int)x, (int)y, (int)z, (int)b);
    }
  }
  reduce_box((int)x, (int)y, (int)z, (int)b, valid, info);
}


// int64 AoS rows -> keys, bounding box AND the occupancy bits in one pass over the coordinates, for a build that
// already knows a box (from the previous build of a similar scene) that should hold every point.  A point outside
// that box sets bit 1 of info->err and marks nothing: the host then repeats the build with the measured box.
__global__ void k_pack_mark_i64(const long long *__restrict__ coords, int ncols, int vec, long long n, Box bx,
                                unsigned long long *__restrict__ keys, unsigned long long *bitmap, BuildInfo *info) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  bool valid = i < n, inside = false;
  unsigned long long p = 0;
  long long x = 0, y = 0, z = 0, b = 0;
  if (valid) {
    if (vec) {
      const longlong2 *q = reinterpret_cast<const longlong2 *>(coords + 4 * i);
      longlong2 a = __ldg(q), c = __ldg(q + 1);
      x = a.x; y = a.y; z = c.x; b = c.y;
    } else {
      const long long *q = coords + (long long)ncols * i;
      x = q[0]; y = q[1]; z = q[2];
      b = ncols > 3 ? q[3] : 0;
    }
    if (!coord_ok(x, y, z, b)) {
      atomicOr(&info->err, 1u);
      valid = false;
      keys[i] = kEmptyKey;
    } else {
      keys[i] = pack_key((int)x, (int)y, (int)z, (int)b);
      const unsigned ux = (unsigned)((int)x - bx.o[0]), uy = (unsigned)((int)y - bx.o[1]), uz = (unsigned)((int)z - bx.o[2]),
                     ub = (unsigned)((int)b - bx.o[3]);
      if (ux < bx.e[0] && uy < bx.e[1] && uz < bx.e[2] && ub < bx.e[3]) {
        p = (((unsigned long long)ub * bx.e[2] + uz) * bx.e[1] + uy) * bx.e[0] + ux;
        inside = true;
      } else {
        atomicOr(&info->err, 2u);
      }
    }
  }
  mark_bit(bitmap, p, inside);
  reduce_box((int)x, (int)y, (int)z, (int)b, valid, info);
}

// int32 SoA coordinates of a finer grid, shifted right (downsampling by 2^shift).
// src (optional): the build record of the grid c belongs to, when its site count is not known on the host yet
__global__ void k_pack_keys_soa(const int32_t *__restrict__ c, long long n, int shift,
                                unsigned long long *__restrict__ keys, BuildInfo *info, int measure_box,
                                const BuildInfo *src) {
  if (src) n = src->n_unique;
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  bool valid = i < n;
  int x = 0, y = 0, z = 0, b = 0;
  if (valid) {
    x = c[i] >> shift;
    y = c[n + i] >> shift;
    z = c[2 * n + i] >> shift;
    b = c[3 * n + i];
    keys[i] = pack_key(x, y, z, b);
  }
  if (measure_box) reduce_box(x, y, z, b, valid, info);
}

// ---------------------------------------------------------------------------------------------
// pass 2: occupancy bitmap in key order
// ---------------------------------------------------------------------------------------------
__global__ void k_mark(const unsigned long long *__restrict__ keys, long long n, Box bx,
                       unsigned long long *bitmap, const BuildInfo *src) {
  if (src) n = src->n_unique;
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // blocks are multiples of 32 threads
  unsigned long long p = 0;
  if (i < n) {
    int x, y, z, b;
    unpack_key(keys[i], x, y, z, b);
    p = box_pos(bx, x, y, z, b);
  }
  mark_bit(bitmap, p, i < n);
}

// The same from the SoA coordinates of the next finer grid, shifted right: a coarse level's box is the fine box
// halved, so no key array and no box measurement are needed.  src (optional): the build record of the grid c
// belongs to, when its site count is not known on the host yet.
__global__ void k_mark_soa(const int32_t *__restrict__ c, long long n, int shift, Box bx, unsigned long long *bitmap,
                           const BuildInfo *src) {
  if (src) n = src->n_unique;
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  unsigned long long p = 0;
  if (i < n) p = box_pos(bx, c[i] >> shift, c[n + i] >> shift, c[2 * n + i] >> shift, c[3 * n + i]);
  mark_bit(bitmap, p, i < n);
}

// ---------------------------------------------------------------------------------------------
// generic two-level exclusive scan: 256 threads x 8 consecutive items per block
// ---------------------------------------------------------------------------------------------
constexpr int kScanThreads = 256;
constexpr int kScanItems = 8;
constexpr int kScanChunk = kScanThreads * kScanItems;

// exclusive scan of one value per thread over the block; *total = block sum (same in all threads)
__device__ __forceinline__ uint32_t block_exclusive_scan(uint32_t v, uint32_t *total) {
  __shared__ uint32_t warp_sum[kScanThreads / 32 + 1];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  uint32_t incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  __syncthreads();  // protects warp_sum against the previous use
  if (lane == 31) warp_sum[wid] = incl;
  __syncthreads();
  if (wid == 0) {
    uint32_t w = lane < kScanThreads / 32 ? warp_sum[lane] : 0;
    uint32_t wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      uint32_t t = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += t;
    }
    if (lane < kScanThreads / 32) warp_sum[lane] = wi - w;  // exclusive warp offsets
    if (lane == kScanThreads / 32 - 1) warp_sum[kScanThreads / 32] = wi;
  }
  __syncthreads();
  *total = warp_sum[kScanThreads / 32];
  return warp_sum[wid] + incl - v;
}

template <class F>
__global__ void k_scan_sums(F f, long long n, uint32_t *__restrict__ block_sums) {
  long long base = (long long)blockIdx.x * kScanChunk + (long long)threadIdx.x * kScanItems;
  uint32_t s = 0;
#pragma unroll
  for (int j = 0; j < kScanItems; ++j)
    if (base + j < n) s += f(base + j);
  uint32_t total;
  block_exclusive_scan(s, &total);
  if (threadIdx.x == 0) block_sums[blockIdx.x] = total;
}

// single block: in-place exclusive scan of the block sums, total to *total
__global__ void k_scan_top(uint32_t *block_sums, long long nb, uint32_t *total_out) {
  uint32_t carry = 0;
  for (long long base = 0; base < nb; base += kScanThreads) {
    long long i = base + threadIdx.x;
    uint32_t v = i < nb ? block_sums[i] : 0;
    uint32_t total;
    uint32_t ex = block_exclusive_scan(v, &total);
    if (i < nb) block_sums[i] = carry + ex;
    carry += total;
  }
  if (threadIdx.x == 0 && total_out) *total_out = carry;
}

// second sweep: each thread knows the exclusive prefix of its first item and hands every item to g
template <class F, class G>
__global__ void k_scan_emit(F f, G g, long long n, const uint32_t *__restrict__ block_offsets) {
  long long base = (long long)blockIdx.x * kScanChunk + (long long)threadIdx.x * kScanItems;
  uint32_t v[kScanItems];
  uint32_t s = 0;
#pragma unroll
  for (int j = 0; j < kScanItems; ++j) {
    v[j] = (base + j < n) ? f(base + j) : 0;
    s += v[j];
  }
  uint32_t total;
  uint32_t ex = block_exclusive_scan(s, &total) + block_offsets[blockIdx.x];
#pragma unroll
  for (int j = 0; j < kScanItems; ++j) {
    if (base + j < n) g(base + j, ex, v[j]);
    ex += v[j];
  }
}

// The whole scan in one block, for inputs of a few chunks (the bitmaps of the coarse scales): one launch instead of
// three.  Launched with kScanThreads threads.
template <class F, class G>
__global__ void k_scan_one_block(F f, G g, long long n, uint32_t *total_out) {
  uint32_t carry = 0;
  for (long long chunk = 0; chunk < n; chunk += kScanChunk) {
    const long long base = chunk + (long long)threadIdx.x * kScanItems;
    uint32_t v[kScanItems];
    uint32_t sum = 0;
#pragma unroll
    for (int j = 0; j < kScanItems; ++j) {
      v[j] = (base + j < n) ? f(base + j) : 0;
      sum += v[j];
    }
    uint32_t total;
    uint32_t ex = block_exclusive_scan(sum, &total) + carry;
#pragma unroll
    for (int j = 0; j < kScanItems; ++j) {
      if (base + j < n) g(base + j, ex, v[j]);
      ex += v[j];
    }
    carry += total;
  }
  if (threadIdx.x == 0 && total_out) *total_out = carry;
}
constexpr long long kScanOneBlockMax = 4 * kScanChunk;  // 8192 items: four rounds of one block

template <class F, class G>
static int scan_emit(F f, G g, long long n, uint32_t *total_dev, cudaStream_t s) {
  if (n <= 0) {
    if (total_dev) SCN_CUDA(cudaMemsetAsync(total_dev, 0, sizeof(uint32_t), s));
    return SCN_OK;
  }
  if (n <= kScanOneBlockMax) {
    k_scan_one_block<<<1, kScanThreads, 0, s>>>(f, g, n, total_dev);
    SCN_LAUNCHED();
    return SCN_OK;
  }
  long long nb = (n + kScanChunk - 1) / kScanChunk;
  uint32_t *sums = nullptr;
  SCN_TRY(dev_alloc_t(&sums, (size_t)nb, s));
  k_scan_sums<<<(unsigned)nb, kScanThreads, 0, s>>>(f, n, sums);
  SCN_LAUNCHED();
  k_scan_top<<<1, kScanThreads, 0, s>>>(sums, nb, total_dev);
  SCN_LAUNCHED();
  k_scan_emit<<<(unsigned)nb, kScanThreads, 0, s>>>(f, g, n, sums);
  SCN_LAUNCHED();
  dev_free(sums, s);
  return SCN_OK;
}

struct PopcWords {
  const unsigned long long *w;
  __device__ uint32_t operator()(long long i) const { return (uint32_t)__popcll(w[i]); }
};
struct U32Values {
  const uint32_t *v;
  __device__ uint32_t operator()(long long i) const { return v[i]; }
};
struct NonNegFlags {
  const int32_t *v;
  __device__ uint32_t operator()(long long i) const { return v[i] >= 0 ? 1u : 0u; }
};
struct StorePrefix {
  uint32_t *out;
  __device__ void operator()(long long i, uint32_t ex, uint32_t) const { out[i] = ex; }
};
// writes off[i] and, for the last element, off[n] = total
struct StoreOffsets {
  int32_t *off;
  long long n;
  __device__ void operator()(long long i, uint32_t ex, uint32_t v) const {
    off[i] = (int32_t)ex;
    if (i == n - 1) off[n] = (int32_t)(ex + v);
  }
};
// ordered compaction of a [K][n] map into pairs
struct EmitPairs {
  const int32_t *map;
  int32_t *pairs;
  long long n;
  int swap;
  __device__ void operator()(long long i, uint32_t ex, uint32_t v) const {
    if (!v) return;
    int32_t a = map[i], b = (int32_t)(i % n);
    pairs[2ll * ex] = swap ? b : a;
    pairs[2ll * ex + 1] = swap ? a : b;
  }
};

// ---------------------------------------------------------------------------------------------
// pass 4: source -> row
// ---------------------------------------------------------------------------------------------
// position (0-based) of the k-th set bit of a 64-bit word, k < popcount: five halvings inside one 32-bit half
__device__ __forceinline__ uint32_t select_bit(unsigned long long bits, uint32_t k) {
  uint32_t w = (uint32_t)bits, pos = 0;
  const uint32_t c = (uint32_t)__popc(w);
  if (k >= c) {
    k -= c;
    w = (uint32_t)(bits >> 32);
    pos = 32;
  }
#pragma unroll
  for (int shift = 16; shift >= 1; shift >>= 1) {
    const uint32_t low = w & ((1u << shift) - 1u);
    const uint32_t cl = (uint32_t)__popc(low);
    if (k >= cl) {
      k -= cl;
      w >>= shift;
      pos += (uint32_t)shift;
    } else {
      w = low;
    }
  }
  return pos;
}

// Second sweep of the popcount scan: the exclusive prefix of every bitmap word.  A block of 1024 threads takes
// kScanChunk = 2048 words (two per thread).
// block_sums: the per-chunk popcount totals of the first sweep (offsets_given = 0: every block adds up the totals in
// front of it -- a few thousand values out of L2) or their exclusive prefix sums made by k_scan_top (offsets_given = 1,
// for very large bitmaps; the site count is then already in info->n_unique).
constexpr int kEmitThreads = 1024;
__global__ void __launch_bounds__(kEmitThreads)
k_rank_emit(const unsigned long long *__restrict__ bitmap, long long nwords, const uint32_t *__restrict__ block_sums, long long nb,
            int offsets_given, uint32_t *__restrict__ prefix, BuildInfo *info) {
  __shared__ uint32_t s_red[2][kEmitThreads / 32];
  __shared__ uint32_t s_before, s_total;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (offsets_given) {
    if (tid == 0) {
      s_before = block_sums[blockIdx.x];
      s_total = info->n_unique;
    }
  } else {
    uint32_t before = 0, total = 0;
    for (long long i = tid; i < nb; i += kEmitThreads) {
      const uint32_t v = block_sums[i];
      total += v;
      if (i < (long long)blockIdx.x) before += v;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      before += __shfl_xor_sync(0xffffffffu, before, o);
      total += __shfl_xor_sync(0xffffffffu, total, o);
    }
    if (lane == 0) {
      s_red[0][warp] = before;
      s_red[1][warp] = total;
    }
    __syncthreads();
    if (warp == 0) {
      uint32_t b = s_red[0][lane], t = s_red[1][lane];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        b += __shfl_xor_sync(0xffffffffu, b, o);
        t += __shfl_xor_sync(0xffffffffu, t, o);
      }
      if (lane == 0) {
        s_before = b;
        s_total = t;
        if (blockIdx.x == 0) info->n_unique = t;
      }
    }
  }
  // two consecutive words per thread, exclusive scan of their popcounts over the block
  const long long base = (long long)blockIdx.x * kScanChunk + 2 * tid;
  const unsigned long long w0 = base < nwords ? bitmap[base] : 0ull, w1 = base + 1 < nwords ? bitmap[base + 1] : 0ull;
  const uint32_t c0 = (uint32_t)__popcll(w0), c1 = (uint32_t)__popcll(w1);
  uint32_t incl = c0 + c1;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t up = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += up;
  }
  __syncthreads();  // s_red is free again, s_before / s_total are visible
  if (lane == 31) s_red[0][warp] = incl;
  __syncthreads();
  if (warp == 0) {
    const uint32_t v = s_red[0][lane];
    uint32_t wi = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t up = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += up;
    }
    s_red[1][lane] = wi - v;  // exclusive offset of every warp
  }
  __syncthreads();
  const uint32_t ex = s_red[1][warp] + incl - (c0 + c1);
  const uint32_t before = s_before;
  if (base < nwords) prefix[base] = ex + before;
  if (base + 1 < nwords) prefix[base + 1] = ex + c0 + before;
}

// Site coordinates from the finished ranking structure.  The position of a set bit in the key-ordered bitmap is the
// site's coordinate and its rank is the site's row, so row r is decoded by finding the word that holds the r-th set
// bit (the last word whose exclusive prefix is <= r; empty words share their successor's prefix and lose) and the bit
// inside it.  Work is dealt out by SITES, one thread per row: a floor plane fills whole words while most of the box is
// empty, and whoever dealt out words would hand some threads a thousand times the average load.  A block of
// consecutive rows first finds the words of its first and last row (two warps, a 32-way search each), stages
// the prefixes of the words in between in shared memory (a few thousand words) and lets every thread bisect there:
// twelve steps in shared memory instead of twenty-odd dependent reads of global memory per row (one bisection per row
// over the whole array measured 113 us for 4M sites; walking the words with one thread per word, 214 us: a full word
// is 64 rows of serial divisions).
constexpr int kDecodeThreads = 256;  // a block decodes 256 rows (below a million sites: more blocks in flight) or 1024
constexpr int kDecodeStage = 4096;  // prefixes staged per block (16 KB); wider spans are bisected in global memory

__device__ __forceinline__ long long word_of_row(const uint32_t *__restrict__ prefix, long long nwords, uint32_t r, int lane) {
  long long lo = 0, hi = nwords;  // prefix[lo] <= r always (prefix[0] = 0); the answer lies in [lo, hi)
  while (hi - lo > 1) {
    const long long step = (hi - lo + 31) >> 5;
    const long long probe = lo + (long long)(lane + 1) * step;
    const bool ok = probe < hi && prefix[probe] <= r;
    const int cnt = __popc(__ballot_sync(0xffffffffu, ok));  // the prefixes ascend: the lanes that pass are the first cnt
    const long long nlo = lo + (long long)cnt * step;
    hi = nlo + step < hi ? nlo + step : hi;
    lo = nlo;
  }
  return lo;
}

__global__ void __launch_bounds__(kDecodeThreads)
k_decode_sites(const unsigned long long *__restrict__ bitmap, const uint32_t *__restrict__ prefix, long long nwords, Box bx,
               int32_t *__restrict__ coords, const BuildInfo *info, int sites_per_block) {
  const long long n = info->n_unique;
  const long long s0 = (long long)blockIdx.x * sites_per_block;
  if (s0 >= n) return;
  const long long s1 = (s0 + sites_per_block < n ? s0 + sites_per_block : n) - 1;  // last row of this block
  __shared__ long long s_w[2];
  __shared__ uint32_t s_pre[kDecodeStage];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (warp < 2) {
    const long long w = word_of_row(prefix, nwords, (uint32_t)(warp == 0 ? s0 : s1), lane);
    if (lane == 0) s_w[warp] = w;
  }
  __syncthreads();
  const long long w0 = s_w[0], span = s_w[1] - w0 + 1;
  const bool staged = span <= kDecodeStage;
  if (staged) {
    for (long long i = threadIdx.x; i < span; i += kDecodeThreads) s_pre[i] = prefix[w0 + i];
    __syncthreads();
  }
  for (long long r = s0 + threadIdx.x; r <= s1; r += kDecodeThreads) {
    long long lo = 0, hi = span;  // words w0 + [lo, hi): the prefix of w0 + lo is <= r
    while (hi - lo > 1) {
      const long long mid = (lo + hi) >> 1;
      const uint32_t p = staged ? s_pre[mid] : prefix[w0 + mid];
      if (p <= (uint32_t)r) lo = mid;
      else hi = mid;
    }
    const long long w = w0 + lo;
    const uint32_t before = staged ? s_pre[lo] : prefix[w];
    uint32_t pos = (uint32_t)(w << 6) + select_bit(bitmap[w], (uint32_t)r - before);  // below 2^32 by the limit on the box
    const uint32_t cx = pos % bx.e[0];
    pos /= bx.e[0];
    const uint32_t cy = pos % bx.e[1];
    pos /= bx.e[1];
    const uint32_t cz = pos % bx.e[2];
    const uint32_t cb = pos / bx.e[2];
    coords[r] = (int)cx + bx.o[0];
    coords[n + r] = (int)cy + bx.o[1];
    coords[2 * n + r] = (int)cz + bx.o[2];
    coords[3 * n + r] = (int)cb + bx.o[3];
  }
}

// source -> row from the finished ranking structure (keys made by the pack kernels; ~0 marks a rejected point)
__global__ void k_rank_src(const unsigned long long *__restrict__ keys, long long n_src, Box bx,
                           const unsigned long long *__restrict__ bitmap, const uint32_t *__restrict__ prefix,
                           int32_t *__restrict__ src_row) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_src) return;
  const unsigned long long key = keys[i];
  int row = -1;
  if (key != kEmptyKey) {
    int x, y, z, b;
    unpack_key(key, x, y, z, b);
    // a point outside the box the bitmap was laid out for (a hinted build that has to be repeated) has no row
    const unsigned ux = (unsigned)(x - bx.o[0]), uy = (unsigned)(y - bx.o[1]), uz = (unsigned)(z - bx.o[2]), ub = (unsigned)(b - bx.o[3]);
    if (ux < bx.e[0] && uy < bx.e[1] && uz < bx.e[2] && ub < bx.e[3]) {
      const unsigned long long p = (((unsigned long long)ub * bx.e[2] + uz) * bx.e[1] + uy) * bx.e[0] + ux;
      const unsigned long long w = __ldg(bitmap + (p >> 6));
      row = (int)(__ldg(prefix + (p >> 6)) + (uint32_t)__popcll(w & ((1ull << (p & 63)) - 1ull)));
    }
  }
  src_row[i] = row;
}

// per-site source counts (only built when some site has more than one source)
__global__ void k_count_rows(const int32_t *__restrict__ src_row, long long n_src, uint32_t *cnt) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_src) return;
  const int r = src_row[i];
  if (r >= 0) atomicAdd(&cnt[r], 1u);
}

// inverse of a one-to-one source -> row map: item[row] = source (the source list of a grid without duplicates)
__global__ void k_invert_rows(const int32_t *__restrict__ src_row, long long n_src, int32_t *__restrict__ item) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_src) return;
  const int r = src_row[i];
  if (r >= 0) item[r] = (int32_t)i;
}

// key -> row of every site into the (empty) open-addressing table; with capacity >= 2n an insert always finds a slot
__global__ void k_table_fill(const int32_t *__restrict__ c, long long n, Slot *table, uint32_t mask) {
  // one thread per site: at load <= 0.5 an insert ends in its home slot or the next one nearly always, and the
  // four-lane teams that pay off for lookups (whole 64-byte lines per step) only serialise four inserts here
  // (measured: 4 M sites in 3.0 ms by teams against 0.14 ms by single threads)
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const unsigned long long key = pack_key(c[i], c[n + i], c[2 * n + i], c[3 * n + i]);
  uint32_t h = hash_key(key) & mask;
  for (uint32_t probe = 0; probe <= mask; ++probe) {  // bounded: at most one sweep of the table
    const unsigned long long old = atomicCAS(&table[h].key, kEmptyKey, key);
    if (old == kEmptyKey || old == key) {
      table[h].row = (int)i;
      return;
    }
    h = (h + 1) & mask;
  }
}

// sources of each site (CSR), ascending source index inside a site
__global__ void k_csr_fill(const int32_t *__restrict__ src_row, long long n_src, const int32_t *__restrict__ off,
                           uint32_t *cursor, int32_t *item) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_src) return;
  int r = src_row[i];
  uint32_t p = atomicAdd(&cursor[r], 1u);
  item[off[r] + (int)p] = (int32_t)i;
}
__global__ void k_csr_sort(const int32_t *__restrict__ off, long long n, int32_t *item, BuildInfo *info) {
  long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  unsigned int c = 0;
  if (r < n) {
    const int b = off[r], e = off[r + 1];
    c = (unsigned)(e - b);
    for (int i = b + 1; i < e; ++i) {  // insertion sort: segments are a handful of points
      int v = item[i], j = i - 1;
      while (j >= b && item[j] > v) {
        item[j + 1] = item[j];
        --j;
      }
      item[j + 1] = v;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) c = max(c, __shfl_xor_sync(0xffffffffu, c, o));
  if ((threadIdx.x & 31) == 0 && c) atomicMax(&info->max_active, c);
}

// ---------------------------------------------------------------------------------------------
// lookups and rulebook maps
// ---------------------------------------------------------------------------------------------
__global__ void k_query(const int32_t *__restrict__ c, long long stride, long long n, const Slot *__restrict__ table,
                        uint32_t mask, int32_t *__restrict__ rows) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int lane = threadIdx.x & 31, first = lane & ~(kTeam - 1);
  const unsigned team_mask = ((1u << kTeam) - 1u) << first;
  bool valid = i < n;
  unsigned long long key = 0;
  if (valid) {
    const int x = c[i], y = c[stride + i], z = c[2 * stride + i], b = c[3 * stride + i];
    valid = coord_ok(x, y, z, b);
    key = pack_key(x, y, z, b);
  }
  int mine = -1;
#pragma unroll
  for (int r = 0; r < kTeam; ++r) {
    const unsigned long long k = __shfl_sync(team_mask, key, first + r);
    const int v = __shfl_sync(team_mask, (int)valid, first + r);
    const int found = v ? table_find_team(table, mask, k, team_mask, lane) : -1;
    if (lane == first + r) mine = found;
  }
  if (i < n) rows[i] = mine;
}

// 3x3x3 neighbour map.  blockIdx.y = offset k = (dx+1)*9 + (dy+1)*3 + (dz+1); the input site of
// offset k for output o is o + (dx,dy,dz).  When `absent` is given only sites with absent[o] < 0 are
// looked up (incremental rulebook against the saved grid), the others get -1.
__global__ void k_ssc_nbr(const int32_t *__restrict__ c, long long n, const Slot *__restrict__ table, uint32_t mask,
                          const int32_t *__restrict__ absent, int self_ok, int32_t *__restrict__ nbr,
                          unsigned long long *counts, const BuildInfo *dyn) {
  if (dyn) n = dyn->n_unique;  // launched with a grid sized for an upper bound of n
  const int k = blockIdx.y;
  const int dx = k / 9 - 1, dy = (k / 3) % 3 - 1, dz = k % 3 - 1;
  const long long o = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int lane = threadIdx.x & 31, first = lane & ~(kTeam - 1);
  const unsigned team_mask = ((1u << kTeam) - 1u) << first;
  int r = -1;
  bool probe = false;
  unsigned long long key = 0;
  if (o < n && (absent == nullptr || absent[o] < 0)) {
    if (k == 13 && self_ok) {
      r = (int)o;
    } else {
      const int x = c[o] + dx, y = c[n + o] + dy, z = c[2 * n + o] + dz, b = c[3 * n + o];
      probe = coord_ok(x, y, z, b);
      key = pack_key(x, y, z, b);
    }
  }
#pragma unroll
  for (int q = 0; q < kTeam; ++q) {  // the team answers its four queries one after the other
    const unsigned long long kq = __shfl_sync(team_mask, key, first + q);
    const int v = __shfl_sync(team_mask, (int)probe, first + q);
    const int found = v ? table_find_team(table, mask, kq, team_mask, lane) : -1;
    if (v && lane == first + q) r = found;
  }
  if (o < n) nbr[(long long)k * n + o] = r;
  const int cnt = __syncthreads_count(r >= 0);
  if (threadIdx.x == 0 && cnt) atomicAdd(&counts[k], (unsigned long long)cnt);
}

// The same map from the ranking structure of the looked-up grid (its box, bitmap and prefix sums) instead of its
// hash table.  blockIdx.y = line (dy, dz); a thread handles site o and the three offsets dx = -1, 0, +1 of that
// line: the cells (x-1, x, x+1) of a line are adjacent bits of the bitmap (x runs fastest in key order), so one
// word read (two when the three bits straddle a word) and one prefix read answer three queries, and neighbouring
// sites read neighbouring words.  self_ok: the grid is looked up in itself and the centre is the site's own row.
__device__ __forceinline__ int rank_lookup(const unsigned long long *__restrict__ bitmap, const uint32_t *__restrict__ prefix,
                                           unsigned long long p) {
  const unsigned long long w = __ldg(bitmap + (p >> 6));
  if (!((w >> (p & 63)) & 1ull)) return -1;
  return (int)(__ldg(prefix + (p >> 6)) + (uint32_t)__popcll(w & ((1ull << (p & 63)) - 1ull)));
}

__global__ void k_ssc_nbr_rank(const int32_t *__restrict__ c, long long n, Box bx,
                               const unsigned long long *__restrict__ bitmap, const uint32_t *__restrict__ prefix,
                               const int32_t *__restrict__ absent, int self_ok, int32_t *__restrict__ nbr,
                               unsigned long long *counts, const BuildInfo *dyn) {
  if (dyn) n = dyn->n_unique;
  const int line = blockIdx.y, dy = line / 3 - 1, dz = line % 3 - 1;
  const long long o = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  int r[3] = {-1, -1, -1};
  if (o < n) {
    if (absent == nullptr || absent[o] < 0) {
      const int x = c[o], y = c[n + o] + dy, z = c[2 * n + o] + dz, b = c[3 * n + o];
      const unsigned uy = (unsigned)(y - bx.o[1]), uz = (unsigned)(z - bx.o[2]), ub = (unsigned)(b - bx.o[3]);
      if (uy < bx.e[1] && uz < bx.e[2] && ub < bx.e[3]) {
        const long long ux = (long long)x - bx.o[0];  // may lie outside the box of another grid
        const unsigned long long row_base =
            (((unsigned long long)ub * bx.e[2] + uz) * bx.e[1] + uy) * bx.e[0];  // cell (box x origin, y, z, b)
#pragma unroll
        for (int j = 0; j < 3; ++j) {
          const long long cx = ux + j - 1;
          if (cx < 0 || cx >= (long long)bx.e[0]) continue;
          if (j == 1 && line == 4 && self_ok) r[1] = (int)o;
          else r[j] = rank_lookup(bitmap, prefix, row_base + (unsigned long long)cx);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 3; ++j) nbr[(long long)(j * 9 + line) * n + o] = r[j];
  }
#pragma unroll
  for (int j = 0; j < 3; ++j) {
    const int cnt = __syncthreads_count(r[j] >= 0);
    if (threadIdx.x == 0 && cnt) atomicAdd(&counts[j * 9 + line], (unsigned long long)cnt);
  }
}

// sites of another grid (SoA coordinates, stride `stride`) -> row in this grid or -1, from the ranking structure
__global__ void k_query_rank(const int32_t *__restrict__ c, long long stride, long long n, Box bx,
                             const unsigned long long *__restrict__ bitmap, const uint32_t *__restrict__ prefix,
                             int32_t *__restrict__ rows) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const unsigned ux = (unsigned)(c[i] - bx.o[0]), uy = (unsigned)(c[stride + i] - bx.o[1]),
                 uz = (unsigned)(c[2 * stride + i] - bx.o[2]), ub = (unsigned)(c[3 * stride + i] - bx.o[3]);
  int r = -1;
  if (ux < bx.e[0] && uy < bx.e[1] && uz < bx.e[2] && ub < bx.e[3])
    r = rank_lookup(bitmap, prefix, (((unsigned long long)ub * bx.e[2] + uz) * bx.e[1] + uy) * bx.e[0] + ux);
  rows[i] = r;
}

// 2x2x2 / stride 2: offset of a fine site inside its coarse cell k = (x&1)*4 + (y&1)*2 + (z&1).  The coarse row of
// a fine site is read from `parent`, or -- when parent is null -- ranked here in the coarse grid's bitmap and
// written to parent_out together with the coarse site's coordinates (the coarse build then needs no pass of its
// own for either).
__global__ void k_conv_maps(const int32_t *__restrict__ fc, long long nf, const int32_t *__restrict__ parent,
                            long long nc, int32_t *child, int32_t *up, unsigned long long *counts, const BuildInfo *dyn,
                            const BuildInfo *src, Box bx, const unsigned long long *__restrict__ bitmap,
                            const uint32_t *__restrict__ prefix, int32_t *__restrict__ parent_out, int32_t *coarse_coords) {
  if (dyn) nc = dyn->n_unique;
  if (src) nf = src->n_unique;
  long long f = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  __shared__ unsigned int hist[8];
  if (threadIdx.x < 8) hist[threadIdx.x] = 0;
  __syncthreads();
  if (f < nf) {
    const int x = fc[f], y = fc[nf + f], z = fc[2 * nf + f];
    int k = ((x & 1) << 2) | ((y & 1) << 1) | (z & 1);
    int p;
    if (parent) {
      p = parent[f];
    } else {
      const int b = fc[3 * nf + f];
      p = rank_lookup(bitmap, prefix, box_pos(bx, x >> 1, y >> 1, z >> 1, b));
      parent_out[f] = p;
      coarse_coords[p] = x >> 1;  // the (up to eight) fine sites of a coarse site write the same four values
      coarse_coords[nc + p] = y >> 1;
      coarse_coords[2 * nc + p] = z >> 1;
      coarse_coords[3 * nc + p] = b;
    }
    child[(long long)k * nc + p] = (int32_t)f;
#pragma unroll
    for (int j = 0; j < 8; ++j) up[(long long)j * nf + f] = (j == k) ? p : -1;
    atomicAdd(&hist[k], 1u);
  }
  __syncthreads();
  if (threadIdx.x < 8 && hist[threadIdx.x]) atomicAdd(&counts[threadIdx.x], (unsigned long long)hist[threadIdx.x]);
}

// incremental deconvolution: the saved coarse row feeds a fine output only when the coarse site
// existed in the saved frame and the fine site did not.
__global__ void k_incre_up(const int32_t *__restrict__ up, long long nf, const int32_t *__restrict__ pe_coarse,
                           const int32_t *__restrict__ pe_fine, int32_t *__restrict__ up2) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= 8 * nf) return;
  long long f = i % nf;
  int p = up[i];
  int v = -1;
  if (p >= 0 && pe_fine[f] < 0) v = pe_coarse[p];
  up2[i] = v;
}

__global__ void k_locations(const int32_t *__restrict__ c, long long n, long long *__restrict__ out) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  out[4 * i] = c[i];
  out[4 * i + 1] = c[n + i];
  out[4 * i + 2] = c[2 * n + i];
  out[4 * i + 3] = c[3 * n + i];
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
static inline unsigned blocks_for(long long n, int t) { return (unsigned)((n + t - 1) / t); }

int grid_free(Grid &g, cudaStream_t s) {
  auto release = [&](const void *p) {  // members carved out of the arena go with it
    const unsigned char *q = static_cast<const unsigned char *>(p);
    if (q && !(g.arena && q >= g.arena && q < g.arena + g.arena_bytes)) dev_free(const_cast<void *>(p), s);
  };
  release(g.coords);
  release(g.table);
  release(g.src_row);
  release(g.csr_off);
  release(g.csr_item);
  release(g.site_count);
  release(g.nbr);
  release(g.bitmap);
  release(g.prefix);
  release(g.child);
  release(g.fine_up);
  dev_free(g.arena, s);
  g = Grid();
  return SCN_OK;
}

// A ranking bitmap is laid out for at most this many cells (512 MiB of words plus 256 MiB of prefixes).  Scenes whose
// bounding box is larger -- two clusters at opposite corners of a 4096^3 volume, say -- are ranked by sorting their keys
// and answer lookups through the open-addressing table; nothing limits their extent but the key range.
const unsigned long long kMaxDenseBits = 1ull << 32;

// The few words a build reads back land in pinned host memory: a copy into pageable memory goes through a driver
// staging buffer and costs several microseconds more per round trip.  One 8 KB block per host thread; when it
// cannot be had the reads go to the caller's stack as before.
constexpr size_t kPinnedBytes = 8192;
static unsigned char *pinned_scratch() {
  thread_local unsigned char *p = nullptr;
  thread_local bool tried = false;
  if (!tried) {
    tried = true;
    void *q = nullptr;
    if (cudaHostAlloc(&q, kPinnedBytes, cudaHostAllocDefault) == cudaSuccess) p = static_cast<unsigned char *>(q);
    else (void)cudaGetLastError();
  }
  return p;
}
// reads `bytes` from the device into dst through the pinned block (at `slot`, 512-byte slots) and waits for the stream
static int read_back(void *dst, const void *src, size_t bytes, int slot, cudaStream_t s, bool sync) {
  unsigned char *pin = pinned_scratch();
  void *land = (pin && bytes <= 512) ? pin + 512 * slot : dst;
  SCN_CUDA(cudaMemcpyAsync(land, src, bytes, cudaMemcpyDeviceToHost, s));
  if (sync) SCN_CUDA(cudaStreamSynchronize(s));
  return SCN_OK;
}
static void take(void *dst, size_t bytes, int slot) {  // after the synchronisation that followed read_back(..., false)
  unsigned char *pin = pinned_scratch();
  if (pin && bytes <= 512) memcpy(dst, pin + 512 * slot, bytes);
}


// Releases a stream-ordered temporary when it goes out of scope, on every path out of a build.
struct Tmp {
  void *p = nullptr;
  cudaStream_t s;
  explicit Tmp(cudaStream_t s_) : s(s_) {}
  ~Tmp() { dev_free(p, s); }
  Tmp(const Tmp &) = delete;
  Tmp &operator=(const Tmp &) = delete;
  template <typename T> int alloc(T **out, size_t count) {
    dev_free(p, s);
    int r = dev_alloc(&p, count * sizeof(T), s);
    *out = static_cast<T *>(p);
    return r;
  }
};

Box box_with_margin(const Box &tight, int margin) {
  Box b = tight;
  for (int d = 0; d < 3; ++d) {
    int lo = tight.o[d] - margin, hi = tight.o[d] + (int)tight.e[d] - 1 + margin;
    if (lo < 0) lo = 0;
    if (hi > SCN_MAX_COORD) hi = SCN_MAX_COORD;
    b.o[d] = lo;
    b.e[d] = (unsigned)(hi - lo + 1);
  }
  return b;
}

static unsigned long long box_cells(const Box &b, bool *fits) {
  unsigned long long bits = 1;
  *fits = true;
  for (int d = 0; d < 4; ++d) {
    bits *= b.e[d];
    if (bits > kMaxDenseBits) {
      *fits = false;
      return bits;
    }
  }
  return bits;
}

// ---------------------------------------------------------------------------------------------
// LSD radix sort of (key, source index) pairs, 4 bits per pass, stable: the ranking of scenes too spread out
// for a bitmap.  A block sorts nothing itself: it counts its digits, the counts of all blocks are scanned
// digit-major, and every item is written straight to its final place of the pass (position of its digit's bucket
// for this block + number of equal digits in front of it inside the block, counted in thread order, then item order,
// which is the input order -- hence stable).
// ---------------------------------------------------------------------------------------------
constexpr int kSortThreads = 256;
constexpr int kSortItems = 8;
constexpr int kSortChunk = kSortThreads * kSortItems;

__global__ void k_sort_hist(const unsigned long long *__restrict__ keys, long long n, int shift, uint32_t *__restrict__ hist,
                            long long nb) {
  __shared__ uint32_t h[16];
  if (threadIdx.x < 16) h[threadIdx.x] = 0;
  __syncthreads();
  const long long base = (long long)blockIdx.x * kSortChunk + (long long)threadIdx.x * kSortItems;
#pragma unroll
  for (int j = 0; j < kSortItems; ++j)
    if (base + j < n) atomicAdd(&h[(unsigned)(keys[base + j] >> shift) & 15u], 1u);
  __syncthreads();
  if (threadIdx.x < 16) hist[(long long)threadIdx.x * nb + blockIdx.x] = h[threadIdx.x];
}

__global__ void k_sort_scatter(const unsigned long long *__restrict__ keys, const int32_t *__restrict__ idx, long long n, int shift,
                               const uint32_t *__restrict__ offs, long long nb, unsigned long long *__restrict__ keys_out,
                               int32_t *__restrict__ idx_out) {
  __shared__ unsigned short cnt[16][kSortThreads];
  __shared__ uint32_t dig_base[16];
  const int t = threadIdx.x;
#pragma unroll
  for (int d = 0; d < 16; ++d) cnt[d][t] = 0;
  const long long base = (long long)blockIdx.x * kSortChunk + (long long)t * kSortItems;
  unsigned long long k[kSortItems];
  unsigned short r[kSortItems];
#pragma unroll
  for (int j = 0; j < kSortItems; ++j) {
    k[j] = 0;
    r[j] = 0;
    if (base + j < n) {
      k[j] = keys[base + j];
      r[j] = cnt[(unsigned)(k[j] >> shift) & 15u][t]++;  // own column: no other thread touches it
    }
  }
  __syncthreads();
  // exclusive scan of every digit's row across the threads: warp w takes digits 2w and 2w+1, a lane 8 entries
  const int warp = t >> 5, lane = t & 31;
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    const int d = 2 * warp + q;
    uint32_t v[8], sum = 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      v[e] = cnt[d][lane * 8 + e];
      sum += v[e];
    }
    uint32_t incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    uint32_t ex = incl - sum;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      cnt[d][lane * 8 + e] = (unsigned short)ex;
      ex += v[e];
    }
  }
  if (t < 16) dig_base[t] = offs[(long long)t * nb + blockIdx.x];
  __syncthreads();
#pragma unroll
  for (int j = 0; j < kSortItems; ++j) {
    if (base + j < n) {
      const unsigned d = (unsigned)(k[j] >> shift) & 15u;
      const uint32_t pos = dig_base[d] + cnt[d][t] + r[j];
      keys_out[pos] = k[j];
      idx_out[pos] = idx ? idx[base + j] : (int32_t)(base + j);
    }
  }
}

// Sorts n (key, index) pairs by key; `vary` has a bit set wherever keys may differ (passes over digits that are the
// same in every key are skipped).  On return *keys_sorted / *idx_sorted point into the buffers a/b.
static int radix_sort_pairs(const unsigned long long *keys, long long n, unsigned long long vary, unsigned long long *ka,
                            unsigned long long *kb, int32_t *ia, int32_t *ib, const unsigned long long **keys_sorted,
                            const int32_t **idx_sorted, cudaStream_t s) {
  const long long nb = (n + kSortChunk - 1) / kSortChunk;
  Tmp t_hist(s), t_offs(s);
  uint32_t *hist = nullptr, *offs = nullptr;
  SCN_TRY(t_hist.alloc(&hist, (size_t)nb * 16));
  SCN_TRY(t_offs.alloc(&offs, (size_t)nb * 16));
  const unsigned long long *src_k = keys;
  const int32_t *src_i = nullptr;
  unsigned long long *dst_k = ka;
  int32_t *dst_i = ia;
  bool any = false;
  for (int shift = 0; shift < 64; shift += 4) {
    if (((vary >> shift) & 15ull) == 0 && !(shift == 60 && !any)) continue;  // at least one pass: the output buffers must be filled
    k_sort_hist<<<(unsigned)nb, kSortThreads, 0, s>>>(src_k, n, shift, hist, nb);
    SCN_LAUNCHED();
    SCN_TRY(scan_emit(U32Values{hist}, StorePrefix{offs}, nb * 16, nullptr, s));
    k_sort_scatter<<<(unsigned)nb, kSortThreads, 0, s>>>(src_k, src_i, n, shift, offs, nb, dst_k, dst_i);
    SCN_LAUNCHED();
    any = true;
    src_k = dst_k;
    src_i = dst_i;
    dst_k = (dst_k == ka) ? kb : ka;
    dst_i = (dst_i == ia) ? ib : ia;
  }
  *keys_sorted = src_k;
  *idx_sorted = src_i;
  return SCN_OK;
}

struct RunStarts {
  const unsigned long long *k;
  __device__ uint32_t operator()(long long i) const { return (i == 0 || k[i] != k[i - 1]) ? 1u : 0u; }
};
// row of every sorted element: the number of run starts up to and including it, minus one
struct StoreRunRow {
  int32_t *row;
  __device__ void operator()(long long i, uint32_t ex, uint32_t v) const { row[i] = (int32_t)(ex + v) - 1; }
};
__global__ void k_sorted_emit(const unsigned long long *__restrict__ keys, const int32_t *__restrict__ idx,
                              const int32_t *__restrict__ row_of, long long n_src, long long n, int32_t *__restrict__ src_row,
                              int32_t *__restrict__ coords, int32_t *__restrict__ csr_off, int32_t *__restrict__ csr_item) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_src) return;
  const int r = row_of[i];
  const int src = idx[i];
  src_row[src] = r;
  if (csr_item) csr_item[i] = src;  // sources of a site in ascending index: the sort is stable
  if (i == 0 || keys[i] != keys[i - 1]) {
    int x, y, z, b;
    unpack_key(keys[i], x, y, z, b);
    coords[r] = x;
    coords[n + r] = y;
    coords[2 * n + r] = z;
    coords[3 * n + r] = b;
    if (csr_off) csr_off[r] = (int32_t)i;
  }
  if (i == n_src - 1 && csr_off) csr_off[n] = (int32_t)n_src;
}
__global__ void k_max_run(const int32_t *__restrict__ off, long long n, BuildInfo *info) {
  const long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  unsigned int c = r < n ? (unsigned)(off[r + 1] - off[r]) : 0u;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) c = max(c, __shfl_xor_sync(0xffffffffu, c, o));
  if ((threadIdx.x & 31) == 0 && c) atomicMax(&info->max_active, c);
}

// Ranking by sorting: site row = rank of the key among the distinct keys, sources of a site in ascending index.
// Leaves the grid without a bitmap; lookups go through its open-addressing table.
static int grid_build_sorted(Grid &g, const unsigned long long *keys, const BuildInfo &measured, BuildInfo *info_d,
                             int64_t n_src, bool want_csr, cudaStream_t s) {
  unsigned long long vary = 0;
  const int field_shift[4] = {0, 16, 32, 48};
  for (int d = 0; d < 4; ++d) {
    unsigned diff = (unsigned)measured.mn[d] ^ (unsigned)measured.mx[d];
    unsigned long long m = 0;
    while (diff) {
      m = (m << 1) | 1ull;
      diff >>= 1;
    }
    vary |= m << field_shift[d];
  }
  Tmp t_ka(s), t_kb(s), t_ia(s), t_ib(s), t_row(s);
  unsigned long long *ka, *kb;
  int32_t *ia, *ib, *row_of;
  SCN_TRY(t_ka.alloc(&ka, (size_t)n_src));
  SCN_TRY(t_kb.alloc(&kb, (size_t)n_src));
  SCN_TRY(t_ia.alloc(&ia, (size_t)n_src));
  SCN_TRY(t_ib.alloc(&ib, (size_t)n_src));
  SCN_TRY(t_row.alloc(&row_of, (size_t)n_src));
  const unsigned long long *ks = nullptr;
  const int32_t *is = nullptr;
  SCN_TRY(radix_sort_pairs(keys, n_src, vary, ka, kb, ia, ib, &ks, &is, s));
  SCN_TRY(scan_emit(RunStarts{ks}, StoreRunRow{row_of}, n_src, &info_d->n_unique, s));
  uint32_t n_u = 0;
  SCN_TRY(read_back(&n_u, &info_d->n_unique, sizeof(uint32_t), 0, s, true));
  take(&n_u, sizeof(uint32_t), 0);
  const int64_t n = n_u;
  g.n = n;
  SCN_TRY(dev_alloc_t(&g.coords, (size_t)n * 4, s));
  SCN_TRY(dev_alloc_t(&g.src_row, (size_t)n_src, s));
  const bool dup = n != n_src;
  if (want_csr) {
    SCN_TRY(dev_alloc_t(&g.csr_item, (size_t)n_src, s));
    if (dup) SCN_TRY(dev_alloc_t(&g.csr_off, (size_t)n + 1, s));
  }
  k_sorted_emit<<<blocks_for(n_src, 256), 256, 0, s>>>(ks, is, row_of, n_src, n, g.src_row, g.coords, g.csr_off, g.csr_item);
  SCN_LAUNCHED();
  g.max_active = 1;
  if (want_csr && dup) {
    k_max_run<<<blocks_for(n, 256), 256, 0, s>>>(g.csr_off, n, info_d);
    SCN_LAUNCHED();
    BuildInfo info;
    SCN_TRY(read_back(&info, info_d, sizeof(info), 0, s, true));
    take(&info, sizeof(info), 0);
    g.max_active = (int32_t)info.max_active;
  }
  return SCN_OK;
}

// the source lists of a grid whose sites have several sources: counts, offsets, items in ascending source index
static int build_source_lists(Grid &g, BuildInfo *info_d, cudaStream_t s) {
  const int T = 256;
  Tmp t_cnt(s);
  uint32_t *cnt = nullptr;
  SCN_TRY(t_cnt.alloc(&cnt, (size_t)g.n));
  SCN_CUDA(cudaMemsetAsync(cnt, 0, (size_t)g.n * 4, s));
  k_count_rows<<<blocks_for(g.n_src, T), T, 0, s>>>(g.src_row, g.n_src, cnt);
  SCN_LAUNCHED();
  SCN_TRY(dev_alloc_t(&g.csr_off, (size_t)g.n + 1, s));
  SCN_TRY(dev_alloc_t(&g.csr_item, (size_t)g.n_src, s));
  SCN_TRY(scan_emit(U32Values{cnt}, StoreOffsets{g.csr_off, (long long)g.n}, g.n, nullptr, s));
  SCN_CUDA(cudaMemsetAsync(cnt, 0, (size_t)g.n * 4, s));
  k_csr_fill<<<blocks_for(g.n_src, T), T, 0, s>>>(g.src_row, g.n_src, g.csr_off, cnt, g.csr_item);
  SCN_LAUNCHED();
  k_csr_sort<<<blocks_for(g.n, T), T, 0, s>>>(g.csr_off, g.n, g.csr_item, info_d);
  SCN_LAUNCHED();
  return SCN_OK;
}

int grid_ensure_source_lists(const Grid &g, cudaStream_t s) {
  if (g.csr_item || g.n == 0) return SCN_OK;
  int32_t *item = nullptr;
  SCN_TRY(dev_alloc_t(&item, (size_t)g.n_src, s));
  k_invert_rows<<<blocks_for(g.n_src, 256), 256, 0, s>>>(g.src_row, g.n_src, item);
  SCN_LAUNCHED();
  g.csr_item = item;
  return SCN_OK;
}

static int grid_build_impl(Grid &g, const int64_t *coords64, int ncols, const int32_t *coords_soa, int shift, int64_t n_src,
                           bool want_csr, const Box *box_hint, bool with_ssc, cudaStream_t s) {
  g.n_src = n_src;
  if (n_src == 0) return SCN_OK;
  if (n_src > 0x7FFFFFF0ll) return fail(SCN_E_CAPACITY, "more than 2^31 source rows");
  const int T = 256;
  // the build's temporaries in one allocation: record, neighbour counters, scan totals (bounded by the largest
  // bitmap's chunk count), keys
  Tmp t_tmp(s);
  unsigned long long *counters = nullptr;  // [0..7]: BuildInfo; [8..34]: neighbour counts; [40...]: scan totals; [head...]: keys
  const size_t sums_words = (size_t)(((kMaxDenseBits >> 6) + kScanChunk - 1) / kScanChunk);
  const size_t head = 64 + (sums_words + 1) / 2;  // in 8-byte units
  SCN_TRY(t_tmp.alloc(&counters, head + (size_t)n_src));
  BuildInfo *info_d = reinterpret_cast<BuildInfo *>(counters);
  unsigned long long *keys = counters + head;
  k_init_info<<<1, 32, 0, s>>>(info_d);
  SCN_LAUNCHED();
  BuildInfo info;
  Box bx;
  bool fits = false;
  unsigned long long bits = 0;
  // With a box that should hold the scene (the previous build's, widened), keys, bounding box and occupancy bits come
  // out of one pass over the coordinates and the build has a single host round trip, at its end.
  const bool hinted = box_hint != nullptr && coords64 != nullptr && (bits = box_cells(*box_hint, &fits), fits);
  if (hinted) {
    bx = *box_hint;
  } else {
    if (coords64) {
      const int vec = (ncols == 4 && (reinterpret_cast<uintptr_t>(coords64) & 15) == 0) ? 1 : 0;
      k_pack_keys_i64<<<blocks_for(n_src, T), T, 0, s>>>(reinterpret_cast<const long long *>(coords64), ncols, vec, n_src, keys, info_d);
    } else {
      k_pack_keys_soa<<<blocks_for(n_src, T), T, 0, s>>>(coords_soa, n_src, shift, keys, info_d, 1, nullptr);
    }
    SCN_LAUNCHED();
    SCN_TRY(read_back(&info, info_d, sizeof(info), 0, s, true));
    take(&info, sizeof(info), 0);
    if (info.err & 1u) return fail(SCN_E_RANGE, "coordinate outside [0, 65534] or batch index outside [0, 32766]");
    for (int d = 0; d < 4; ++d) {
      bx.o[d] = info.mn[d];
      bx.e[d] = (unsigned)(info.mx[d] - info.mn[d] + 1);
    }
    g.tight = bx;
    bits = box_cells(bx, &fits);
    if (!fits) {  // too spread out for a bitmap: rank by sorting
      g.box = bx;
      return grid_build_sorted(g, keys, info, info_d, n_src, want_csr, s);
    }
  }
  const long long nwords = (long long)((bits + 63) >> 6);
  const long long nb = (nwords + kScanChunk - 1) / kScanChunk;
  // everything the grid keeps in one allocation (one pool call instead of four, and one release when the grid goes);
  // the site count stays on the device until the end: buffers are sized by the bound n <= n_src
  {
    size_t off = 0;
    auto carve = [&off](size_t bytes) {
      const size_t at = off;
      off += (bytes + 255) & ~(size_t)255;
      return at;
    };
    const size_t o_bitmap = carve((size_t)nwords * 8), o_prefix = carve((size_t)nwords * 4);
    const size_t o_coords = carve((size_t)n_src * 16), o_src_row = carve((size_t)n_src * 4);
    const size_t o_nbr = with_ssc ? carve((size_t)n_src * 108) : 0;
    void *arena = nullptr;
    SCN_TRY(dev_alloc(&arena, off, s));
    g.arena = static_cast<unsigned char *>(arena);
    g.arena_bytes = off;
    g.bitmap = reinterpret_cast<unsigned long long *>(g.arena + o_bitmap);
    g.prefix = reinterpret_cast<uint32_t *>(g.arena + o_prefix);
    g.coords = reinterpret_cast<int32_t *>(g.arena + o_coords);
    g.src_row = reinterpret_cast<int32_t *>(g.arena + o_src_row);
    if (with_ssc) g.nbr = reinterpret_cast<int32_t *>(g.arena + o_nbr);
  }
  SCN_CUDA(cudaMemsetAsync(g.bitmap, 0, (size_t)nwords * 8, s));
  if (hinted) {
    const int vec = (ncols == 4 && (reinterpret_cast<uintptr_t>(coords64) & 15) == 0) ? 1 : 0;
    k_pack_mark_i64<<<blocks_for(n_src, T), T, 0, s>>>(reinterpret_cast<const long long *>(coords64), ncols, vec, n_src, bx, keys,
                                                      g.bitmap, info_d);
  } else {
    k_mark<<<blocks_for(n_src, T), T, 0, s>>>(keys, n_src, bx, g.bitmap, nullptr);
  }
  SCN_LAUNCHED();
  // popcount scan; its second sweep also writes the site coordinates
  uint32_t *sums = reinterpret_cast<uint32_t *>(counters + 40);
  k_scan_sums<<<(unsigned)nb, kScanThreads, 0, s>>>(PopcWords{g.bitmap}, nwords, sums);
  SCN_LAUNCHED();
  const int offsets_given = nb > 8192 ? 1 : 0;
  if (offsets_given) {
    k_scan_top<<<1, kScanThreads, 0, s>>>(sums, nb, &info_d->n_unique);
    SCN_LAUNCHED();
  }
  k_rank_emit<<<(unsigned)nb, kEmitThreads, 0, s>>>(g.bitmap, nwords, sums, nb, offsets_given, g.prefix, info_d);
  SCN_LAUNCHED();
  const int decode_rows = n_src >= (1 << 20) ? 1024 : 256;
  k_decode_sites<<<blocks_for(n_src, decode_rows), kDecodeThreads, 0, s>>>(g.bitmap, g.prefix, nwords, bx, g.coords, info_d, decode_rows);
  SCN_LAUNCHED();
  k_rank_src<<<blocks_for(n_src, T), T, 0, s>>>(keys, n_src, bx, g.bitmap, g.prefix, g.src_row);
  SCN_LAUNCHED();
  // the neighbour map rides along when asked for: its counts come back with the build record
  unsigned long long *nbr_counts_d = nullptr, nbr_counts[27];
  if (with_ssc) {
    nbr_counts_d = counters + 8;
    SCN_CUDA(cudaMemsetAsync(nbr_counts_d, 0, 27 * 8, s));
    k_ssc_nbr_rank<<<dim3(blocks_for(n_src, 256), 9), 256, 0, s>>>(g.coords, 0, bx, g.bitmap, g.prefix, nullptr, 1, g.nbr, nbr_counts_d,
                                                                  info_d);
    SCN_LAUNCHED();
    SCN_TRY(read_back(nbr_counts, nbr_counts_d, sizeof(nbr_counts), 1, s, false));
  }
  SCN_TRY(read_back(&info, info_d, sizeof(info), 0, s, true));  // the one round trip of a hinted build
  take(&info, sizeof(info), 0);
  if (info.err & 1u) return fail(SCN_E_RANGE, "coordinate outside [0, 65534] or batch index outside [0, 32766]");
  if (hinted) {
    Box tight;
    for (int d = 0; d < 4; ++d) {
      tight.o[d] = info.mn[d];
      tight.e[d] = (unsigned)(info.mx[d] - info.mn[d] + 1);
    }
    g.tight = tight;
    if (info.err & 2u) return SCN_E_STATE + 100;  // a point outside the hinted box: the caller repeats with the measured one
  }
  if (with_ssc) take(nbr_counts, sizeof(nbr_counts), 1);
  g.n = info.n_unique;
  g.box = bx;
  g.max_active = 1;
  if (with_ssc) {
    g.nbr_total = 0;
    for (int k = 0; k < 27; ++k) {
      g.nbr_count[k] = (int64_t)nbr_counts[k];
      g.nbr_total += g.nbr_count[k];
    }
  }
  if (want_csr && g.n != n_src) {  // some site has several sources: their lists, and the longest one
    SCN_TRY(build_source_lists(g, info_d, s));
    SCN_TRY(read_back(&info, info_d, sizeof(info), 0, s, true));
    take(&info, sizeof(info), 0);
    g.max_active = (int32_t)info.max_active;
  }
  return SCN_OK;
}

int grid_build(Grid &g, const int64_t *coords64, int ncols, const int32_t *coords_soa, int shift, int64_t n_src,
               bool want_csr, const Box *box_hint, bool with_ssc, cudaStream_t s) {
  grid_free(g, s);
  int r = grid_build_impl(g, coords64, ncols, coords_soa, shift, n_src, want_csr, box_hint, with_ssc, s);
  if (r == SCN_E_STATE + 100) {  // the hinted box did not hold the scene; the pass measured the box that does
    const Box measured = g.tight;
    grid_free(g, s);
    r = grid_build_impl(g, coords64, ncols, coords_soa, shift, n_src, want_csr, &measured, with_ssc, s);
    if (r == SCN_E_STATE + 100) r = fail(SCN_E_STATE, "grid build: the measured bounding box does not hold the scene");
  }
  if (r != SCN_OK) {  // never leave a half-built grid behind
    const int64_t n_src_keep = 0;
    grid_free(g, s);
    g.n_src = n_src_keep;
  }
  return r;
}

// What one level of a chained coarse build leaves on the device for the host to read at the end.
struct LevelRecord {
  BuildInfo info;
  unsigned long long counts[8 + 27];  // stride-2 offsets, then the 27 neighbour offsets
};

int grid_build_coarse_chain(Grid *const *levels, int count, const Grid &fine0, bool with_ssc, cudaStream_t s) {
  for (int l = 0; l < count; ++l) grid_free(*levels[l], s);
  if (count <= 0) return SCN_OK;
  if (fine0.n == 0) {
    for (int l = 0; l < count; ++l) levels[l]->n_src = 0;
    return SCN_OK;
  }
  const int T = 256;
  LevelRecord *rec_d = nullptr;
  SCN_TRY(dev_alloc_t(&rec_d, (size_t)count, s));
  Tmp rec_guard(s);  // released on every way out
  rec_guard.p = rec_d;
  SCN_CUDA(cudaMemsetAsync(rec_d, 0, (size_t)count * sizeof(LevelRecord), s));
  Box box = fine0.box;
  int64_t bound = fine0.n;  // upper bound of the site count of the source level (exact for the first level)
  const int32_t *src_coords = fine0.coords;
  std::vector<Box> boxes((size_t)count);
  int rc = SCN_OK;
  for (int l = 0; l < count && rc == SCN_OK; ++l) {
    Grid &g = *levels[l];
    const BuildInfo *src = l == 0 ? nullptr : &rec_d[l - 1].info;  // level 0 knows its source count on the host
    BuildInfo *info_d = &rec_d[l].info;
    unsigned long long *counts_d = rec_d[l].counts;
    // the coarse box is the fine box halved: nothing to measure
    Box bx;
    unsigned long long bits = 1;
    for (int d = 0; d < 4; ++d) {
      const int sh = d < 3 ? 1 : 0;
      const int lo = box.o[d] >> sh, hi = (box.o[d] + (int)box.e[d] - 1) >> sh;
      bx.o[d] = lo;
      bx.e[d] = (unsigned)(hi - lo + 1);
      bits *= bx.e[d];
    }
    if (bits > kMaxDenseBits) {
      rc = fail(SCN_E_CAPACITY, "coarse scale: bounding box too large for a ranking bitmap");
      break;
    }
    boxes[(size_t)l] = bx;
    const long long nwords = (long long)((bits + 63) >> 6);
    const int64_t n_src = bound;                                         // rows the source level may have
    const int64_t n_max = (int64_t)bits < bound ? (int64_t)bits : bound;  // rows this level may have
    // every buffer of the level in one allocation (one pool call instead of seven, and one release per frame)
    size_t off = 0;
    auto carve = [&off](size_t bytes) {
      const size_t at = off;
      off += (bytes + 255) & ~(size_t)255;
      return at;
    };
    const size_t o_bitmap = carve((size_t)nwords * 8), o_prefix = carve((size_t)nwords * 4);
    const size_t o_coords = carve((size_t)n_max * 16), o_src_row = carve((size_t)n_src * 4);
    const size_t o_child = carve((size_t)n_max * 32), o_up = carve((size_t)n_src * 32);
    const size_t o_nbr = with_ssc ? carve((size_t)n_max * 108) : 0;
    void *arena = nullptr;
    if ((rc = dev_alloc(&arena, off, s)) != SCN_OK) break;
    g.arena = static_cast<unsigned char *>(arena);
    g.arena_bytes = off;
    g.bitmap = reinterpret_cast<unsigned long long *>(g.arena + o_bitmap);  // kept with the grid
    g.prefix = reinterpret_cast<uint32_t *>(g.arena + o_prefix);
    g.coords = reinterpret_cast<int32_t *>(g.arena + o_coords);
    g.src_row = reinterpret_cast<int32_t *>(g.arena + o_src_row);
    g.child = reinterpret_cast<int32_t *>(g.arena + o_child);
    g.fine_up = reinterpret_cast<int32_t *>(g.arena + o_up);
    if (with_ssc) g.nbr = reinterpret_cast<int32_t *>(g.arena + o_nbr);
    // the record was zeroed with the others: no error, and the scan leaves the site count in it
    if (cudaMemsetAsync(g.bitmap, 0, (size_t)nwords * 8, s) != cudaSuccess ||
        cudaMemsetAsync(g.child, 0xFF, (size_t)n_max * 8 * 4, s) != cudaSuccess) {
      rc = fail(SCN_E_CUDA, "coarse grid build: memset failed");
      break;
    }
    k_mark_soa<<<blocks_for(n_src, T), T, 0, s>>>(src_coords, n_src, 1, bx, g.bitmap, src);
    if ((rc = scan_emit(PopcWords{g.bitmap}, StorePrefix{g.prefix}, nwords, &info_d->n_unique, s)) != SCN_OK) break;
    k_conv_maps<<<blocks_for(n_src, 256), 256, 0, s>>>(src_coords, n_src, nullptr, 0, g.child, g.fine_up, counts_d, info_d, src,
                                                       bx, g.bitmap, g.prefix, g.src_row, g.coords);
    if (with_ssc) {
      k_ssc_nbr_rank<<<dim3(blocks_for(n_max, 256), 9), 256, 0, s>>>(g.coords, 0, bx, g.bitmap, g.prefix, nullptr, 1, g.nbr, counts_d + 8, info_d);
    }
    for (int i = 0; i < 2 + (with_ssc ? 1 : 0); ++i) g_launches.fetch_add(1, std::memory_order_relaxed);  // the scan counts its own
    if (cudaGetLastError() != cudaSuccess) {
      rc = fail(SCN_E_CUDA, "a kernel of the coarse grid build could not be launched");
      break;
    }
    box = bx;
    bound = n_max;
    src_coords = g.coords;
  }
  // one host round trip for all levels
  std::vector<LevelRecord> rec((size_t)count);
  if (rc == SCN_OK) {
    unsigned char *pin = pinned_scratch();
    const size_t bytes = (size_t)count * sizeof(LevelRecord);
    void *land = (pin && bytes <= kPinnedBytes) ? (void *)pin : (void *)rec.data();
    if (cudaMemcpyAsync(land, rec_d, bytes, cudaMemcpyDeviceToHost, s) != cudaSuccess || cudaStreamSynchronize(s) != cudaSuccess)
      rc = fail(SCN_E_CUDA, std::string("coarse grid build: ") + cudaGetErrorString(cudaGetLastError()));
    else if (land != rec.data()) memcpy(rec.data(), land, bytes);
  }
  if (rc != SCN_OK) {
    for (int l = 0; l < count; ++l) grid_free(*levels[l], s);
    return rc;
  }
  int64_t n_prev = fine0.n;
  for (int l = 0; l < count; ++l) {
    Grid &g = *levels[l];
    const LevelRecord &r = rec[(size_t)l];
    g.n_src = n_prev;
    g.n = r.info.n_unique;
    g.box = boxes[(size_t)l];
    g.max_active = 1;
    for (int k = 0; k < 8; ++k) g.child_count[k] = (int64_t)r.counts[k];
    if (with_ssc) {
      g.nbr_total = 0;
      for (int k = 0; k < 27; ++k) {
        g.nbr_count[k] = (int64_t)r.counts[8 + k];
        g.nbr_total += g.nbr_count[k];
      }
    }
    n_prev = g.n;
  }
  return rc;
}

bool coarse_box_fits_bitmap(const Box &fine_box, Box *coarse_box) {
  Box bx;
  for (int d = 0; d < 4; ++d) {
    const int sh = d < 3 ? 1 : 0;
    const int lo = fine_box.o[d] >> sh, hi = (fine_box.o[d] + (int)fine_box.e[d] - 1) >> sh;
    bx.o[d] = lo;
    bx.e[d] = (unsigned)(hi - lo + 1);
  }
  if (coarse_box) *coarse_box = bx;
  bool fits;
  (void)box_cells(bx, &fits);
  return fits;
}

int grid_build_coarse(Grid &g, const Grid &fine, bool with_ssc, cudaStream_t s) {
  if (!fine.bitmap || !coarse_box_fits_bitmap(fine.box, nullptr)) {
    // a scene too spread out for a bitmap at this scale: rank the halved coordinates by sorting, then the stride-2
    // maps from the source rows; the neighbour map (when asked for) through the table
    SCN_TRY(grid_build(g, nullptr, 0, fine.coords, 1, fine.n, false, nullptr, false, s));
    SCN_TRY(grid_build_conv(g, fine, s));
    if (with_ssc) SCN_TRY(grid_build_ssc(g, s));
    return SCN_OK;
  }
  Grid *one = &g;
  return grid_build_coarse_chain(&one, 1, fine, with_ssc, s);
}

int grid_ensure_table(const Grid &g, cudaStream_t s) {
  if (g.table || g.n == 0) return SCN_OK;
  uint64_t cap = 16;
  while (cap < (uint64_t)g.n * 2) cap <<= 1;
  Slot *t = nullptr;
  SCN_TRY(dev_alloc_t(&t, (size_t)cap, s));
  SCN_CUDA(cudaMemsetAsync(t, 0xFF, (size_t)cap * sizeof(Slot), s));
  k_table_fill<<<blocks_for(g.n, 256), 256, 0, s>>>(g.coords, g.n, t, (uint32_t)(cap - 1));
  SCN_LAUNCHED();
  g.table = t;
  g.mask = (uint32_t)(cap - 1);
  return SCN_OK;
}

int grid_query(const Grid &g, const int32_t *coords_soa, int64_t n, int64_t soa_stride, int32_t *rows, bool by_rank,
               cudaStream_t s) {
  if (n == 0) return SCN_OK;
  if (g.n == 0) {
    SCN_CUDA(cudaMemsetAsync(rows, 0xFF, (size_t)n * 4, s));
    return SCN_OK;
  }
  if (by_rank && g.bitmap && g.prefix) {
    k_query_rank<<<blocks_for(n, 256), 256, 0, s>>>(coords_soa, soa_stride, n, g.box, g.bitmap, g.prefix, rows);
  } else {
    SCN_TRY(grid_ensure_table(g, s));
    k_query<<<blocks_for(n, 256), 256, 0, s>>>(coords_soa, soa_stride, n, g.table, g.mask, rows);
  }
  SCN_LAUNCHED();
  return SCN_OK;
}

// launches the neighbour-map kernel of g looked up in `lookup`; counts_d: 27 zeroed device counters
static int nbr_launch(const Grid &g, const Grid &lookup, const int32_t *absent, int self_ok, int32_t *nbr,
                      unsigned long long *counts_d, cudaStream_t s) {
  if (lookup.bitmap && lookup.prefix) {
    k_ssc_nbr_rank<<<dim3(blocks_for(g.n, 256), 9), 256, 0, s>>>(g.coords, g.n, lookup.box, lookup.bitmap, lookup.prefix, absent,
                                                                self_ok, nbr, counts_d, nullptr);
  } else {
    SCN_TRY(grid_ensure_table(lookup, s));
    dim3 grid(blocks_for(g.n, 256), 27);
    k_ssc_nbr<<<grid, 256, 0, s>>>(g.coords, g.n, lookup.table, lookup.mask, absent, self_ok, nbr, counts_d, nullptr);
  }
  SCN_LAUNCHED();
  return SCN_OK;
}

static int nbr_common(const Grid &g, const Grid &lookup, const int32_t *absent, int self_ok, int32_t *nbr,
                      int64_t *counts_host, cudaStream_t s) {
  unsigned long long *counts_d = nullptr;
  SCN_TRY(dev_alloc_t(&counts_d, 27, s));
  SCN_CUDA(cudaMemsetAsync(counts_d, 0, 27 * 8, s));
  SCN_TRY(nbr_launch(g, lookup, absent, self_ok, nbr, counts_d, s));
  unsigned long long h[27];
  SCN_TRY(read_back(h, counts_d, sizeof(h), 1, s, true));
  take(h, sizeof(h), 1);
  dev_free(counts_d, s);
  for (int k = 0; k < 27; ++k) counts_host[k] = (int64_t)h[k];
  return SCN_OK;
}

// The incremental neighbour maps of several scales with one host round trip: jobs[i] = (grid, saved grid, pre_exist,
// nbr2 out, counts out [27]).
int build_incre_nbr_batch(const IncreNbrJob *jobs, int count, cudaStream_t s) {
  if (count <= 0) return SCN_OK;
  unsigned long long *counts_d = nullptr;
  SCN_TRY(dev_alloc_t(&counts_d, (size_t)count * 27, s));
  SCN_CUDA(cudaMemsetAsync(counts_d, 0, (size_t)count * 27 * 8, s));
  for (int i = 0; i < count; ++i) {
    const IncreNbrJob &j = jobs[i];
    if (j.g->n == 0) continue;
    if (j.pre->n == 0) SCN_CUDA(cudaMemsetAsync(j.nbr2, 0xFF, (size_t)j.g->n * 27 * 4, s));
    else SCN_TRY(nbr_launch(*j.g, *j.pre, j.pre_exist, 0, j.nbr2, counts_d + 27 * i, s));
  }
  std::vector<unsigned long long> h((size_t)count * 27);
  SCN_CUDA(cudaMemcpyAsync(h.data(), counts_d, h.size() * 8, cudaMemcpyDeviceToHost, s));
  SCN_CUDA(cudaStreamSynchronize(s));
  dev_free(counts_d, s);
  for (int i = 0; i < count; ++i)
    for (int k = 0; k < 27; ++k) jobs[i].counts_host[k] = (int64_t)h[(size_t)i * 27 + k];
  return SCN_OK;
}

int grid_build_ssc(Grid &g, cudaStream_t s) {
  if (g.nbr || g.n == 0) return SCN_OK;
  SCN_TRY(dev_alloc_t(&g.nbr, (size_t)g.n * 27, s));
  if (g.bitmap && g.prefix) {
    unsigned long long *counts_d = nullptr, h[27];
    SCN_TRY(dev_alloc_t(&counts_d, 27, s));
    SCN_CUDA(cudaMemsetAsync(counts_d, 0, 27 * 8, s));
    k_ssc_nbr_rank<<<dim3(blocks_for(g.n, 256), 9), 256, 0, s>>>(g.coords, g.n, g.box, g.bitmap, g.prefix, nullptr, 1, g.nbr, counts_d, nullptr);
    SCN_LAUNCHED();
    SCN_TRY(read_back(h, counts_d, sizeof(h), 1, s, true));
    take(h, sizeof(h), 1);
    dev_free(counts_d, s);
    for (int k = 0; k < 27; ++k) g.nbr_count[k] = (int64_t)h[k];
  } else {
    SCN_TRY(nbr_common(g, g, nullptr, 1, g.nbr, g.nbr_count, s));
  }
  g.nbr_total = 0;
  for (int k = 0; k < 27; ++k) g.nbr_total += g.nbr_count[k];
  return SCN_OK;
}

int build_incre_nbr(const Grid &g, const Grid &pre, const int32_t *pre_exist, int32_t *nbr2, int64_t *counts_host,
                    cudaStream_t s) {
  if (g.n == 0) return SCN_OK;
  if (pre.n == 0) {
    SCN_CUDA(cudaMemsetAsync(nbr2, 0xFF, (size_t)g.n * 27 * 4, s));
    for (int k = 0; k < 27; ++k) counts_host[k] = 0;
    return SCN_OK;
  }
  return nbr_common(g, pre, pre_exist, 0, nbr2, counts_host, s);
}

int grid_build_conv(Grid &coarse, const Grid &fine, cudaStream_t s) {
  if (coarse.child || coarse.n == 0) return SCN_OK;
  unsigned long long *counts_d = nullptr;
  SCN_TRY(dev_alloc_t(&counts_d, 8, s));
  SCN_CUDA(cudaMemsetAsync(counts_d, 0, 8 * 8, s));
  SCN_TRY(dev_alloc_t(&coarse.child, (size_t)coarse.n * 8, s));
  SCN_TRY(dev_alloc_t(&coarse.fine_up, (size_t)fine.n * 8, s));
  SCN_CUDA(cudaMemsetAsync(coarse.child, 0xFF, (size_t)coarse.n * 8 * 4, s));
  k_conv_maps<<<blocks_for(fine.n, 256), 256, 0, s>>>(fine.coords, fine.n, coarse.src_row, coarse.n, coarse.child,
                                                     coarse.fine_up, counts_d, nullptr, nullptr, coarse.box, nullptr, nullptr,
                                                     nullptr, nullptr);
  SCN_LAUNCHED();
  unsigned long long h[8];
  SCN_CUDA(cudaMemcpyAsync(h, counts_d, sizeof(h), cudaMemcpyDeviceToHost, s));
  SCN_CUDA(cudaStreamSynchronize(s));
  dev_free(counts_d, s);
  for (int k = 0; k < 8; ++k) coarse.child_count[k] = (int64_t)h[k];
  return SCN_OK;
}

int build_incre_up(const Grid &coarse, const int32_t *pe_coarse, const int32_t *pe_fine, int32_t *up2,
                   cudaStream_t s) {
  const long long nf = coarse.n_src;
  if (nf == 0) return SCN_OK;
  k_incre_up<<<blocks_for(8 * nf, 256), 256, 0, s>>>(coarse.fine_up, nf, pe_coarse, pe_fine, up2);
  SCN_LAUNCHED();
  return SCN_OK;
}

int map_to_pairs(const int32_t *map, int K, int64_t n, int swap, int64_t expected_pairs, int32_t *pairs_host,
                 cudaStream_t s) {
  if (n == 0 || expected_pairs == 0) return SCN_OK;
  const long long total_items = (long long)K * n;
  int32_t *pairs_d = nullptr;
  uint32_t *total_d = nullptr;
  SCN_TRY(dev_alloc_t(&pairs_d, (size_t)expected_pairs * 2, s));
  SCN_TRY(dev_alloc_t(&total_d, 1, s));
  SCN_TRY(scan_emit(NonNegFlags{map}, EmitPairs{map, pairs_d, (long long)n, swap}, total_items, total_d, s));
  uint32_t total = 0;
  SCN_CUDA(cudaMemcpyAsync(&total, total_d, 4, cudaMemcpyDeviceToHost, s));
  SCN_CUDA(cudaMemcpyAsync(pairs_host, pairs_d, (size_t)expected_pairs * 8, cudaMemcpyDeviceToHost, s));
  SCN_CUDA(cudaStreamSynchronize(s));
  dev_free(pairs_d, s);
  dev_free(total_d, s);
  if ((int64_t)total != expected_pairs) return fail(SCN_E_STATE, "rulebook pair count changed under the caller");
  return SCN_OK;
}

int grid_locations(const Grid &g, int64_t *out_host, cudaStream_t s) {
  if (g.n == 0) return SCN_OK;
  long long *tmp = nullptr;
  SCN_TRY(dev_alloc_t(&tmp, (size_t)g.n * 4, s));
  k_locations<<<blocks_for(g.n, 256), 256, 0, s>>>(g.coords, g.n, tmp);
  SCN_LAUNCHED();
  SCN_CUDA(cudaMemcpyAsync(out_host, tmp, (size_t)g.n * 32, cudaMemcpyDeviceToHost, s));
  SCN_CUDA(cudaStreamSynchronize(s));
  dev_free(tmp, s);
  return SCN_OK;
}

}  // namespace scn
