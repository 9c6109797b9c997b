// Label fusion: the per-voxel vote table that follows the network in online segmentation.
//
// Replaces Result<3> (Metadata/resultHash.h:22-138: a google::dense_hash_map from a voxel to (label, confidence),
// updated point by point on the host) and ResultOfWeight<3> (resultHash.h:141-218: a map from a voxel to a probability
// vector, blended 0.5 * old + new) by a device-resident open-addressing table that a frame's predictions are merged
// into by a few kernels, with the prediction tensor never leaving the GPU.
//
//   keys   [capacity]  batch << 48 | z << 32 | y << 16 | x, ~0 = empty; linear probing, load factor <= 1/2
//   label  [capacity], conf [capacity]            vote mode
//   probs  [capacity * classes]                   weight mode
//
// update(points, scores), per point (resultHash.h:62-98): a voxel seen for the first time takes (argmax, max score);
// a known voxel with the same label adds the score, capped at `maximum`; with another label the score is subtracted
// and, when the confidence falls below zero, the label flips and the confidence changes sign.  Points are applied as
// if one after the other in row order: the reference's loop is sequential in its first pass and races in its second
// when one call names a voxel twice; here the first row of a voxel in a call is applied by a parallel kernel and any
// further rows of the same voxel by a serial pass in row order, so the result is that of the sequential loop.
//
// Steps of an update: (1) find-or-insert every point's key (64-bit CAS), remember its slot, take the smallest row
// index per slot; (2) first rows vote in parallel; (3) the other rows, collected in ascending order by one block,
// vote one after the other; (4) the per-call marks are cleared.  The table doubles (rehash kernel) before it would
// pass half full, counting every row of the call as a possible new voxel.
#include "internal.h"
#include <limits.h>

namespace scn {
namespace {

constexpr unsigned long long kNoKey = ~0ull;
constexpr int kFirstNone = INT_MAX;

__device__ __forceinline__ uint32_t mix_key(unsigned long long k) {
  k ^= k >> 33;
  k *= 0xff51afd7ed558ccdULL;
  k ^= k >> 33;
  k *= 0xc4ceb9fe1a85ec53ULL;
  k ^= k >> 33;
  return (uint32_t)k;
}

// key of row i of an int64 [n, ncols] array (ncols 3: batch 0); false when a coordinate is outside the key range
__device__ __forceinline__ bool row_key(const long long *__restrict__ pts, int ncols, long long i, unsigned long long *key) {
  const long long x = pts[i * ncols], y = pts[i * ncols + 1], z = pts[i * ncols + 2], b = ncols > 3 ? pts[i * ncols + 3] : 0;
  if (x < 0 || y < 0 || z < 0 || b < 0 || x > SCN_MAX_COORD || y > SCN_MAX_COORD || z > SCN_MAX_COORD || b > SCN_MAX_BATCH)
    return false;
  *key = ((unsigned long long)b << 48) | ((unsigned long long)z << 32) | ((unsigned long long)y << 16) | (unsigned long long)x;
  return true;
}

__device__ __forceinline__ int find_slot(const unsigned long long *__restrict__ keys, uint32_t mask, unsigned long long key) {
  uint32_t s = mix_key(key) & mask;
  for (uint32_t probes = 0; probes <= mask; ++probes) {
    const unsigned long long cur = keys[s];
    if (cur == key) return (int)s;
    if (cur == kNoKey) return -1;
    s = (s + 1) & mask;
  }
  return -1;
}

// returns the slot, *created = this call put the key there; -1 when the table is full (never below half load)
__device__ __forceinline__ int find_or_insert(unsigned long long *keys, uint32_t mask, unsigned long long key, bool *created) {
  uint32_t s = mix_key(key) & mask;
  *created = false;
  for (uint32_t probes = 0; probes <= mask; ++probes) {
    unsigned long long cur = keys[s];
    if (cur == kNoKey) {
      cur = atomicCAS(&keys[s], kNoKey, key);
      if (cur == kNoKey) {
        *created = true;
        return (int)s;
      }
    }
    if (cur == key) return (int)s;
    s = (s + 1) & mask;
  }
  return -1;
}

struct Table {
  unsigned long long *keys;
  int *label;
  float *conf;
  float *probs;
  int *first;            // per slot: smallest row index of the running call that names it (kFirstNone otherwise)
  unsigned char *fresh;  // per slot: the running call created it
  uint32_t mask;
  int classes;  // 0: vote mode
};

// status word: bit0 coordinate outside the key range, bit1 table full
__global__ void k_lab_insert(Table t, const long long *__restrict__ pts, int ncols, long long n, int *__restrict__ slot_of,
                             unsigned int *size, unsigned int *status) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  unsigned long long key;
  int slot = -1;
  if (!row_key(pts, ncols, i, &key)) {
    atomicOr(status, 1u);
  } else {
    bool created;
    slot = find_or_insert(t.keys, t.mask, key, &created);
    if (slot < 0) {
      atomicOr(status, 2u);
    } else {
      if (created) {
        t.fresh[slot] = 1;
        atomicAdd(size, 1u);
      }
      atomicMin(&t.first[slot], (int)i);
    }
  }
  slot_of[i] = slot;
}

__device__ __forceinline__ void arg_max(const float *__restrict__ row, int classes, int *val, float *best) {
  int v = 0;
  float b = row[0];
  for (int c = 1; c < classes; ++c) {
    const float x = row[c];
    if (x > b) {  // first maximum, as torch's max does
      b = x;
      v = c;
    }
  }
  *val = v;
  *best = b;
}

// resultHash.h:86-96
__device__ __forceinline__ void vote(Table &t, int slot, bool is_new, int val, float p, float maximum) {
  if (is_new) {
    t.label[slot] = val;
    t.conf[slot] = p;
    return;
  }
  int l = t.label[slot];
  float c = t.conf[slot];
  if (l == val) c = fminf(maximum, c + p);
  else c -= p;
  if (c < 0.f) {
    l = val;
    c = -c;
  }
  t.label[slot] = l;
  t.conf[slot] = c;
}

// mode 0: update; mode 1: set (resultHash.h:37-50: label = argmax, confidence 0, whatever was there)
__global__ void k_lab_vote_first(Table t, const int *__restrict__ slot_of, long long n, const float *__restrict__ scores,
                                 long long stride, int classes, float maximum, int mode, int *__restrict__ list,
                                 unsigned int *n_later) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int slot = slot_of[i];
  if (slot < 0) return;
  if (t.first[slot] != (int)i) {  // not the first row of its voxel in this call: left to the serial pass
    list[atomicAdd(n_later, 1u)] = (int)i;
    return;
  }
  int val;
  float p;
  arg_max(scores + i * stride, classes, &val, &p);
  if (mode == 1) {
    t.label[slot] = val;
    t.conf[slot] = 0.f;
  } else {
    vote(t, slot, t.fresh[slot] != 0, val, p, maximum);
  }
}

// ResultOfWeight::update (resultHash.h:146-158): one thread per (row, class)
__global__ void k_lab_blend_first(Table t, const int *__restrict__ slot_of, long long n, const float *__restrict__ scores,
                                  long long stride, int *__restrict__ list, unsigned int *n_later) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long i = idx / t.classes;
  const int c = (int)(idx - i * t.classes);
  if (i >= n) return;
  const int slot = slot_of[i];
  if (slot < 0) return;
  if (t.first[slot] != (int)i) {
    if (c == 0) list[atomicAdd(n_later, 1u)] = (int)i;
    return;
  }
  float *dst = t.probs + (long long)slot * t.classes + c;
  const float x = scores[i * stride + c];
  *dst = t.fresh[slot] ? x : *dst * 0.5f + x;
}

// Rows that are not the first of their voxel in this call (collected in no particular order by the kernel above),
// applied one after the other in row order by one block: the list is sorted (in shared memory when it has at most 8192
// entries, else rebuilt in order by scanning the rows), then the votes are applied serially (vote table: thread 0;
// weight table: thread c for class c).  Nothing to do in the common case of a call that names every voxel once.
constexpr int kSortMax = 8192;
__global__ void __launch_bounds__(1024) k_lab_later_rows(Table t, const int *__restrict__ slot_of, long long n,
                                                         const float *__restrict__ scores, long long stride, int classes,
                                                         float maximum, int mode, int *__restrict__ list,
                                                         const unsigned int *__restrict__ n_later) {
  const unsigned int total = *n_later;
  if (total == 0) return;
  __shared__ int sorted[kSortMax];
  __shared__ unsigned int offs[1024];
  const int T = blockDim.x, tid = threadIdx.x;
  const int *order = sorted;
  if (total <= (unsigned)kSortMax) {
    unsigned int m = 1;
    while (m < total) m <<= 1;
    for (unsigned int j = tid; j < m; j += T) sorted[j] = j < total ? list[j] : INT_MAX;
    __syncthreads();
    for (unsigned int k = 2; k <= m; k <<= 1)
      for (unsigned int j = k >> 1; j > 0; j >>= 1) {
        for (unsigned int x = tid; x < m; x += T) {
          const unsigned int y = x ^ j;
          if (y > x) {
            const int a = sorted[x], b = sorted[y];
            const bool up = (x & k) == 0;
            if ((a > b) == up) {
              sorted[x] = b;
              sorted[y] = a;
            }
          }
        }
        __syncthreads();
      }
  } else {
    const long long per = (n + T - 1) / T, lo = per * tid, hi = lo + per < n ? lo + per : n;
    unsigned int mine = 0;
    for (long long i = lo; i < hi; ++i) {
      const int s = slot_of[i];
      mine += (s >= 0 && t.first[s] != (int)i) ? 1u : 0u;
    }
    offs[tid] = mine;
    __syncthreads();
    if (tid == 0) {
      unsigned int run = 0;
      for (int k = 0; k < T; ++k) {
        const unsigned int v = offs[k];
        offs[k] = run;
        run += v;
      }
    }
    __syncthreads();
    unsigned int at = offs[tid];
    for (long long i = lo; i < hi; ++i) {
      const int s = slot_of[i];
      if (s >= 0 && t.first[s] != (int)i) list[at++] = (int)i;
    }
    __syncthreads();
    order = list;
  }
  for (unsigned int j = 0; j < total; ++j) {
    const int i = order[j], slot = slot_of[i];
    if (t.classes == 0) {
      if (tid == 0) {
        int val;
        float p;
        arg_max(scores + (long long)i * stride, classes, &val, &p);
        if (mode == 1) {
          t.label[slot] = val;
          t.conf[slot] = 0.f;
        } else {
          vote(t, slot, false, val, p, maximum);
        }
      }
    } else {
      for (int c = tid; c < t.classes; c += T) {
        float *dst = t.probs + (long long)slot * t.classes + c;
        *dst = *dst * 0.5f + scores[(long long)i * stride + c];
      }
    }
    __syncthreads();
  }
}

__global__ void k_lab_unmark(Table t, const int *__restrict__ slot_of, long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int s = slot_of[i];
  if (s >= 0) {
    t.first[s] = kFirstNone;
    t.fresh[s] = 0;
  }
}

__global__ void k_lab_query(Table t, const long long *__restrict__ pts, int ncols, long long n, long long *__restrict__ out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  unsigned long long key;
  long long r = -1;
  if (row_key(pts, ncols, i, &key)) {
    const int s = find_slot(t.keys, t.mask, key);
    if (s >= 0) {
      if (t.classes == 0) {
        r = t.label[s];
      } else {
        int val;
        float p;
        arg_max(t.probs + (long long)s * t.classes, t.classes, &val, &p);
        r = val;
      }
    }
  }
  out[i] = r;
}

// every entry as (x, y, z, label), in no particular order (the reference iterates its hash map)
__global__ void k_lab_dump(Table t, long long *__restrict__ out, long long capacity_rows, unsigned int *count) {
  const uint32_t s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s > t.mask) return;
  const unsigned long long k = t.keys[s];
  if (k == kNoKey) return;
  const unsigned int at = atomicAdd(count, 1u);
  if ((long long)at >= capacity_rows) return;
  int lab;
  if (t.classes == 0) {
    lab = t.label[s];
  } else {
    float p;
    arg_max(t.probs + (long long)s * t.classes, t.classes, &lab, &p);
  }
  out[4ll * at] = (long long)(k & 0xFFFF);
  out[4ll * at + 1] = (long long)((k >> 16) & 0xFFFF);
  out[4ll * at + 2] = (long long)((k >> 32) & 0xFFFF);
  out[4ll * at + 3] = lab;
}

// finalize (resultHash.h:128-138): marks the entries named by the points
__global__ void k_lab_mark_kept(Table t, const long long *__restrict__ pts, int ncols, long long n, unsigned char *keep) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  unsigned long long key;
  if (!row_key(pts, ncols, i, &key)) return;
  const int s = find_slot(t.keys, t.mask, key);
  if (s >= 0) keep[s] = 1;
}

// moves the entries of `from` (all of them, or those with keep[slot] set) into the empty table `to`
__global__ void k_lab_rehash(Table from, Table to, const unsigned char *__restrict__ keep, unsigned int *size, unsigned int *status) {
  const uint32_t s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s > from.mask) return;
  const unsigned long long k = from.keys[s];
  if (k == kNoKey || (keep && !keep[s])) return;
  bool created;
  const int d = find_or_insert(to.keys, to.mask, k, &created);
  if (d < 0) {
    atomicOr(status, 2u);
    return;
  }
  atomicAdd(size, 1u);
  if (from.classes == 0) {
    to.label[d] = from.label[s];
    to.conf[d] = from.conf[s];
  } else {
    for (int c = 0; c < from.classes; ++c) to.probs[(long long)d * from.classes + c] = from.probs[(long long)s * from.classes + c];
  }
}

__global__ void k_lab_fill(unsigned long long *keys, int *first, unsigned char *fresh, uint32_t cap) {
  const uint32_t s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= cap) return;
  keys[s] = kNoKey;
  first[s] = kFirstNone;
  fresh[s] = 0;
}

inline unsigned blocks(long long n, int t) { return (unsigned)((n + t - 1) / t); }

}  // namespace
}  // namespace scn

using namespace scn;

struct scn_labels {
  Table t = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, 0, 0};
  unsigned char *arena = nullptr;
  uint32_t cap = 0;
  int classes = 0;
  float maximum = 0.f;
  int64_t size_bound = 0;        // entries the table may hold by now (every row of every update counted as new)
  unsigned int *counters = nullptr;  // device: [0] entries, [1] status, [2] rows applied serially by the last update, [3] dump count
};

namespace {

int table_alloc(Table *t, unsigned char **arena, uint32_t cap, int classes, cudaStream_t s) {
  size_t off = 0;
  auto carve = [&off](size_t bytes) {
    const size_t at = off;
    off += (bytes + 255) & ~(size_t)255;
    return at;
  };
  const size_t o_keys = carve((size_t)cap * 8), o_first = carve((size_t)cap * 4), o_fresh = carve((size_t)cap);
  const size_t o_label = classes ? 0 : carve((size_t)cap * 4), o_conf = classes ? 0 : carve((size_t)cap * 4);
  const size_t o_probs = classes ? carve((size_t)cap * classes * 4) : 0;
  void *p = nullptr;
  SCN_TRY(dev_alloc(&p, off, s));
  *arena = static_cast<unsigned char *>(p);
  t->keys = reinterpret_cast<unsigned long long *>(*arena + o_keys);
  t->first = reinterpret_cast<int *>(*arena + o_first);
  t->fresh = *arena + o_fresh;
  t->label = classes ? nullptr : reinterpret_cast<int *>(*arena + o_label);
  t->conf = classes ? nullptr : reinterpret_cast<float *>(*arena + o_conf);
  t->probs = classes ? reinterpret_cast<float *>(*arena + o_probs) : nullptr;
  t->mask = cap - 1;
  t->classes = classes;
  k_lab_fill<<<blocks(cap, 256), 256, 0, s>>>(t->keys, t->first, t->fresh, cap);
  SCN_LAUNCHED();
  return SCN_OK;
}

// reads the status word; a set bit fails the call that found it
int check_status(scn_labels *h, cudaStream_t s, const char *what) {
  unsigned int st = 0;
  SCN_CUDA(cudaMemcpyAsync(&st, h->counters + 1, sizeof(st), cudaMemcpyDeviceToHost, s));
  SCN_CUDA(cudaStreamSynchronize(s));
  if (!st) return SCN_OK;
  SCN_CUDA(cudaMemsetAsync(h->counters + 1, 0, sizeof(unsigned int), s));
  if (st & 1u) return fail(SCN_E_RANGE, std::string(what) + ": a coordinate or batch index is outside the key range");
  return fail(SCN_E_CAPACITY, std::string(what) + ": the label table is full");
}

// moves the table into a fresh one of `cap` slots (all entries, or those with keep[slot] set)
int rebuild(scn_labels *h, uint64_t cap, const unsigned char *keep, cudaStream_t s) {
  if (cap > (1ull << 31)) return fail(SCN_E_CAPACITY, "label table beyond 2^31 slots");
  Table nt;
  unsigned char *na = nullptr;
  SCN_TRY(table_alloc(&nt, &na, (uint32_t)cap, h->classes, s));
  if (h->cap) {
    int rc = SCN_OK;
    if (cudaMemsetAsync(h->counters, 0, sizeof(unsigned int), s) != cudaSuccess) rc = fail(SCN_E_CUDA, "label table: memset failed");
    if (rc == SCN_OK) {
      k_lab_rehash<<<blocks(h->cap, 256), 256, 0, s>>>(h->t, nt, keep, h->counters, h->counters + 1);
      g_launches.fetch_add(1, std::memory_order_relaxed);
      if (cudaGetLastError() != cudaSuccess) rc = fail(SCN_E_CUDA, "label table: launch failed");
    }
    if (rc != SCN_OK) {
      dev_free(na, s);
      return rc;
    }
    dev_free(h->arena, s);
  }
  h->t = nt;
  h->arena = na;
  h->cap = (uint32_t)cap;
  return SCN_OK;
}

// makes room for `more` new entries: the table stays at most half full
int reserve(scn_labels *h, int64_t more, cudaStream_t s) {
  int64_t want = h->size_bound + more;
  if (h->cap && want * 2 > (int64_t)h->cap) {  // the bound counts every row as new: look at the true size before growing
    unsigned int size = 0;
    SCN_CUDA(cudaMemcpyAsync(&size, h->counters, sizeof(size), cudaMemcpyDeviceToHost, s));
    SCN_CUDA(cudaStreamSynchronize(s));
    want = (int64_t)size + more;
  }
  if (!h->cap || want * 2 > (int64_t)h->cap) {
    uint64_t cap = 1024;
    while ((int64_t)cap < want * 2) cap <<= 1;
    SCN_TRY(rebuild(h, cap, nullptr, s));
  }
  h->size_bound = want;
  return SCN_OK;
}

int apply(scn_labels *h, const int64_t *points, int ncols, int64_t n, const float *scores, int64_t stride, int64_t classes, int mode,
          cudaStream_t s) {
  if (!h || n < 0 || (n && (!points || !scores)) || (ncols != 3 && ncols != 4) || classes < 1 || stride < classes)
    return fail(SCN_E_INVALID, "label table: bad argument");
  if (h->classes && classes != h->classes) return fail(SCN_E_INVALID, "label table: the number of classes differs from the table's");
  if (mode == 1 && h->classes) return fail(SCN_E_UNSUPPORTED, "set() belongs to the vote table");
  if (n > INT_MAX) return fail(SCN_E_CAPACITY, "more than 2^31 rows in one call");
  if (n == 0) return SCN_OK;
  SCN_TRY(reserve(h, n, s));
  int *slot_of = nullptr, *list = nullptr;
  SCN_TRY(dev_alloc_t(&slot_of, (size_t)n * 2, s));
  list = slot_of + n;
  const long long *pts = reinterpret_cast<const long long *>(points);
  if (cudaMemsetAsync(h->counters + 2, 0, sizeof(unsigned int), s) != cudaSuccess) {
    dev_free(slot_of, s);
    return fail(SCN_E_CUDA, "label table: memset failed");
  }
  k_lab_insert<<<blocks(n, 256), 256, 0, s>>>(h->t, pts, ncols, n, slot_of, h->counters, h->counters + 1);
  SCN_LAUNCHED();
  if (h->classes == 0)
    k_lab_vote_first<<<blocks(n, 256), 256, 0, s>>>(h->t, slot_of, n, scores, stride, (int)classes, h->maximum, mode, list,
                                                    h->counters + 2);
  else
    k_lab_blend_first<<<blocks(n * classes, 256), 256, 0, s>>>(h->t, slot_of, n, scores, stride, list, h->counters + 2);
  SCN_LAUNCHED();
  k_lab_later_rows<<<1, 1024, 0, s>>>(h->t, slot_of, n, scores, stride, (int)classes, h->maximum, mode, list, h->counters + 2);
  SCN_LAUNCHED();
  k_lab_unmark<<<blocks(n, 256), 256, 0, s>>>(h->t, slot_of, n);
  SCN_LAUNCHED();
  dev_free(slot_of, s);
  return SCN_OK;
}

}  // namespace

extern "C" {

int scn_labels_create(scn_labels **out, int weight_classes, double maximum) {
  if (!out || weight_classes < 0) return fail(SCN_E_INVALID, "scn_labels_create: bad argument");
  scn_labels *h = new scn_labels();
  h->classes = weight_classes;
  h->maximum = (float)maximum;
  cudaError_t e = cudaMalloc(reinterpret_cast<void **>(&h->counters), 4 * sizeof(unsigned int));
  if (e == cudaSuccess) e = cudaMemset(h->counters, 0, 4 * sizeof(unsigned int));
  if (e != cudaSuccess) {
    if (h->counters) cudaFree(h->counters);
    delete h;
    return fail(SCN_E_CUDA, std::string("label table: ") + cudaGetErrorString(e));
  }
  *out = h;
  return SCN_OK;
}

void scn_labels_destroy(scn_labels *h) {
  if (!h) return;
  cudaDeviceSynchronize();
  if (h->arena) cudaFree(h->arena);
  cudaFree(h->counters);
  delete h;
}

int scn_labels_clear(scn_labels *h, void *stream) {
  if (!h) return fail(SCN_E_INVALID, "null handle");
  cudaStream_t s = (cudaStream_t)stream;
  if (h->cap) {
    k_lab_fill<<<blocks(h->cap, 256), 256, 0, s>>>(h->t.keys, h->t.first, h->t.fresh, h->cap);
    SCN_LAUNCHED();
  }
  SCN_CUDA(cudaMemsetAsync(h->counters, 0, 4 * sizeof(unsigned int), s));
  h->size_bound = 0;
  return SCN_OK;
}

int scn_labels_update(scn_labels *h, const int64_t *points, int ncols, int64_t n, const float *scores, int64_t scores_stride,
                      int64_t classes, void *stream) {
  return apply(h, points, ncols, n, scores, scores_stride, classes, 0, (cudaStream_t)stream);
}

int scn_labels_set(scn_labels *h, const int64_t *points, int ncols, int64_t n, const float *scores, int64_t scores_stride,
                   int64_t classes, void *stream) {
  return apply(h, points, ncols, n, scores, scores_stride, classes, 1, (cudaStream_t)stream);
}

int scn_labels_query(scn_labels *h, const int64_t *points, int ncols, int64_t n, int64_t *labels, void *stream) {
  if (!h || n < 0 || (n && (!points || !labels)) || (ncols != 3 && ncols != 4)) return fail(SCN_E_INVALID, "scn_labels_query: bad argument");
  cudaStream_t s = (cudaStream_t)stream;
  if (n == 0) return SCN_OK;
  if (!h->cap) {
    SCN_CUDA(cudaMemsetAsync(labels, 0xFF, (size_t)n * 8, s));  // all -1
    return SCN_OK;
  }
  k_lab_query<<<blocks(n, 256), 256, 0, s>>>(h->t, reinterpret_cast<const long long *>(points), ncols, n,
                                             reinterpret_cast<long long *>(labels));
  SCN_LAUNCHED();
  return SCN_OK;
}

int scn_labels_size(scn_labels *h, int64_t *size, int64_t *rows_applied_serially, void *stream) {
  if (!h || !size) return fail(SCN_E_INVALID, "scn_labels_size: bad argument");
  cudaStream_t s = (cudaStream_t)stream;
  SCN_TRY(check_status(h, s, "label table"));
  unsigned int c[3] = {0, 0, 0};
  SCN_CUDA(cudaMemcpyAsync(c, h->counters, sizeof(c), cudaMemcpyDeviceToHost, s));
  SCN_CUDA(cudaStreamSynchronize(s));
  *size = c[0];
  if (rows_applied_serially) *rows_applied_serially = c[2];
  h->size_bound = c[0];
  return SCN_OK;
}

int scn_labels_dump(scn_labels *h, int64_t *out, int64_t capacity_rows, int64_t *n_written, void *stream) {
  if (!h || capacity_rows < 0 || (capacity_rows && !out) || !n_written) return fail(SCN_E_INVALID, "scn_labels_dump: bad argument");
  cudaStream_t s = (cudaStream_t)stream;
  *n_written = 0;
  if (!h->cap) return SCN_OK;
  SCN_CUDA(cudaMemsetAsync(h->counters + 3, 0, sizeof(unsigned int), s));
  k_lab_dump<<<blocks(h->cap, 256), 256, 0, s>>>(h->t, reinterpret_cast<long long *>(out), capacity_rows, h->counters + 3);
  SCN_LAUNCHED();
  unsigned int c = 0;
  SCN_CUDA(cudaMemcpyAsync(&c, h->counters + 3, sizeof(c), cudaMemcpyDeviceToHost, s));
  SCN_CUDA(cudaStreamSynchronize(s));
  if ((int64_t)c > capacity_rows) return fail(SCN_E_CAPACITY, "scn_labels_dump: the output holds fewer rows than the table has entries");
  *n_written = c;
  return SCN_OK;
}

int scn_labels_finalize(scn_labels *h, const int64_t *points, int ncols, int64_t n, void *stream) {
  if (!h || n < 0 || (n && !points) || (ncols != 3 && ncols != 4)) return fail(SCN_E_INVALID, "scn_labels_finalize: bad argument");
  cudaStream_t s = (cudaStream_t)stream;
  if (!h->cap) return SCN_OK;
  unsigned char *keep = nullptr;
  SCN_TRY(dev_alloc_t(&keep, (size_t)h->cap, s));
  int rc = SCN_OK;
  if (cudaMemsetAsync(keep, 0, (size_t)h->cap, s) != cudaSuccess) rc = fail(SCN_E_CUDA, "scn_labels_finalize: memset failed");
  if (rc == SCN_OK && n) {
    k_lab_mark_kept<<<blocks(n, 256), 256, 0, s>>>(h->t, reinterpret_cast<const long long *>(points), ncols, n, keep);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    if (cudaGetLastError() != cudaSuccess) rc = fail(SCN_E_CUDA, "scn_labels_finalize: launch failed");
  }
  if (rc == SCN_OK) rc = rebuild(h, h->cap, keep, s);  // same capacity: entries only go away
  dev_free(keep, s);
  return rc;
}

}  // extern "C"
