// Halo rows of a scene split into slabs over several GPUs, pushed straight into the neighbour's memory.
//
// Every rank owns an INBOX: per side (0 = from the left neighbour, 1 = from the right neighbour) two message slots
// and one 64-bit sequence number.  Exchange number e (counted by every rank alike: all ranks run the same network)
// is two launches per rank on the rank's own stream:
//
//   k_halo_push    gathers the rows of the plane next to each cut and stores them, over NVLink, into slot e % 2 of
//                  the neighbour's inbox; the last block to finish publishes e in the neighbour's sequence number
//                  (data stores, system-wide fence, then the number);
//   k_halo_unpack  waits until its own inbox shows e on the sides that have a neighbour -- a bounded wait: after
//                  `spin_limit` polls it records a time-out in the status word and returns, the rows stay as they
//                  were -- and scatters the slot's rows onto the first ghost layer.
//
// Nothing on the host takes part: row lists and counts are device arrays, so a frame queues without a round trip.
// Slot reuse is safe with two slots: a rank pushes exchange e after it has unpacked e-1 (stream order), which it
// could only do after the neighbour pushed e-1, which the neighbour did after unpacking e-2 from the same slot.
// The waits are between kernels on DIFFERENT GPUs; a rank that is its own neighbour (the single-GPU self-test:
// periodic boundary) pushes before it unpacks in stream order and never waits.
//
// Inboxes are plain cudaMalloc allocations shared through CUDA IPC handles (the ranks are processes of one box).
// The reference has no multi-GPU path; there is nothing this replaces.
#include "internal.h"
#include <limits.h>
#include <string.h>

namespace scn {
namespace {

constexpr int kFlagStride = 16;  // in 64-bit words: one 128-byte line per sequence number

struct HaloSide {
  char *out;                     // neighbour's inbox slot to write (null: no neighbour on this side)
  unsigned long long *out_seq;   // neighbour's sequence number for messages from me
  const char *in;                // my inbox slot written by that neighbour
  const unsigned long long *in_seq;
};

struct HaloArgs {
  HaloSide side[2];
  const int64_t *rows;    // [4][cap]: send-left, send-right, receive-left, receive-right; ascending
  const int64_t *counts;  // [4]
  int64_t cap;
  char *a, *b;            // one or two row-major arrays patched in place (b may be null)
  int a_row_bytes, b_row_bytes;
  int64_t slot_bytes;
  unsigned long long seq;
  unsigned int *done;     // blocks of the running push kernel that have finished
  unsigned int *status;   // bit0: a wait ran out; bit1: a plane did not fit a slot
  unsigned int spin_limit;
};

template <typename W> __device__ __forceinline__ int64_t rows_that_fit(const HaloArgs &p, int list) {
  int64_t n = p.counts[list];
  bool cut = false;
  if (n > p.cap) {  // the caller's list is shorter than the plane
    n = p.cap;
    cut = true;
  }
  const int64_t row_bytes = p.a_row_bytes + p.b_row_bytes;
  if (n * row_bytes > p.slot_bytes) {
    n = p.slot_bytes / row_bytes;
    cut = true;
  }
  if (cut && threadIdx.x == 0 && blockIdx.x == 0) atomicOr(p.status, 2u);
  return n;
}

template <typename W> __global__ void __launch_bounds__(256) k_halo_push(const HaloArgs p) {
  const int wa = p.a_row_bytes / (int)sizeof(W), wb = p.b_row_bytes / (int)sizeof(W), w = wa + wb;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int s = 0; s < 2; ++s) {
    if (!p.side[s].out) continue;
    const int64_t n = rows_that_fit<W>(p, s);
    const int64_t *rows = p.rows + s * p.cap;
    W *out = reinterpret_cast<W *>(p.side[s].out);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n * w; i += stride) {
      const int64_t r = i / w;
      const int k = (int)(i - r * w);
      const int64_t row = rows[r];
      const W *src = k < wa ? reinterpret_cast<const W *>(p.a + row * p.a_row_bytes) + k
                            : reinterpret_cast<const W *>(p.b + row * p.b_row_bytes) + (k - wa);
      out[i] = *src;
    }
  }
  // publish: every block fences its own stores system-wide before it is counted; the last one writes the numbers
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int ticket = atomicAdd(p.done, 1u);
    if (ticket == gridDim.x - 1) {
      *p.done = 0;
      __threadfence_system();
      for (int s = 0; s < 2; ++s)
        if (p.side[s].out_seq) *reinterpret_cast<volatile unsigned long long *>(p.side[s].out_seq) = p.seq;
      __threadfence_system();
    }
  }
}

template <typename W> __global__ void __launch_bounds__(256) k_halo_unpack(const HaloArgs p) {
  __shared__ int arrived[2];
  if (threadIdx.x < 2) {
    const int s = threadIdx.x;
    int ok = 1;
    if (p.side[s].in_seq) {
      const volatile unsigned long long *flag = p.side[s].in_seq;
      // after one time-out the ranks are out of step for good: later exchanges give up at once instead of waiting again
      unsigned int polls = (*reinterpret_cast<volatile unsigned int *>(p.status) & 1u) ? p.spin_limit : 0;
      while (*flag < p.seq) {
        if (++polls > p.spin_limit) {
          ok = 0;
          atomicOr(p.status, 1u);
          break;
        }
        __nanosleep(200);
      }
      __threadfence_system();
    }
    arrived[s] = ok;
  }
  __syncthreads();
  const int wa = p.a_row_bytes / (int)sizeof(W), wb = p.b_row_bytes / (int)sizeof(W), w = wa + wb;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int s = 0; s < 2; ++s) {
    if (!p.side[s].in || !arrived[s]) continue;
    const int64_t n = rows_that_fit<W>(p, 2 + s);
    const int64_t *rows = p.rows + (2 + s) * p.cap;
    const W *in = reinterpret_cast<const W *>(p.side[s].in);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n * w; i += stride) {
      const int64_t r = i / w;
      const int k = (int)(i - r * w);
      const int64_t row = rows[r];
      W *dst = k < wa ? reinterpret_cast<W *>(p.a + row * p.a_row_bytes) + k
                      : reinterpret_cast<W *>(p.b + row * p.b_row_bytes) + (k - wa);
      *dst = __ldcg(in + i);  // written by the neighbour while this kernel may already be running: not through L1
    }
  }
}

// Row lists of the four planes next to a rank's cuts (x == lo: sent left, x == hi - 1: sent right, x == lo - 1:
// received from the left, x == hi: received from the right), each ascending, from a scale's x coordinates.  Two
// launches of the same grid: every block counts the hits of its contiguous piece of the rows, then (second launch)
// adds up the counts of the pieces in front of it and writes its hits in order.  plane[i] = INT_MIN switches list i off.
constexpr int kListBlocks = 128;
constexpr int kListThreads = 256;

__global__ void __launch_bounds__(kListThreads) k_plane_lists(const int32_t *__restrict__ x, long long n, int4 plane,
                                                              unsigned int *__restrict__ piece_counts, int64_t *__restrict__ lists,
                                                              int64_t *__restrict__ counts, long long cap, int pass) {
  __shared__ unsigned int s_warp[4][kListThreads / 32];
  __shared__ unsigned int s_base[4];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const long long per = (n + gridDim.x - 1) / gridDim.x;
  const long long lo = per * blockIdx.x, hi = lo + per < n ? lo + per : n;
  const int want[4] = {plane.x, plane.y, plane.z, plane.w};
  unsigned int run[4] = {0, 0, 0, 0};  // hits of this block so far (second pass: in front of the current chunk)
  if (pass == 1) {
    if (tid < 4) {
      unsigned int before = 0;
      for (int b = 0; b < (int)blockIdx.x; ++b) before += piece_counts[4 * b + tid];
      s_base[tid] = before;
      if (blockIdx.x == gridDim.x - 1) counts[tid] = (int64_t)before + piece_counts[4 * blockIdx.x + tid];
    }
    __syncthreads();
  }
  for (long long c0 = lo; c0 < hi; c0 += kListThreads) {
    const long long i = c0 + tid;
    const int v = i < hi ? x[i] : INT_MIN + 1;
    unsigned int below[4];
#pragma unroll
    for (int l = 0; l < 4; ++l) {
      const unsigned int b = __ballot_sync(0xffffffffu, v == want[l]);
      below[l] = __popc(b & ((1u << lane) - 1u));
      if (lane == 0) s_warp[l][warp] = __popc(b);
    }
    __syncthreads();
#pragma unroll
    for (int l = 0; l < 4; ++l) {
      unsigned int before = 0, total = 0;
#pragma unroll
      for (int w = 0; w < kListThreads / 32; ++w) {
        const unsigned int c = s_warp[l][w];
        before += w < warp ? c : 0u;
        total += c;
      }
      if (pass == 1 && v == want[l]) {
        const long long at = (long long)s_base[l] + run[l] + before + below[l];
        if (at < cap) lists[(long long)l * cap + at] = i;
      }
      run[l] += total;
    }
    __syncthreads();
  }
  if (pass == 0 && tid < 4) piece_counts[4 * blockIdx.x + tid] = run[tid];
}

}  // namespace

int halo_plane_lists(const int32_t *x, int64_t n, int lo, int hi, bool left, bool right, int64_t cap, int64_t *lists,
                     int64_t *counts, cudaStream_t s) {
  unsigned int *pieces = nullptr;
  SCN_TRY(dev_alloc_t(&pieces, (size_t)4 * kListBlocks, s));
  const int off = INT_MIN;
  const int4 plane = make_int4(left ? lo : off, right ? hi - 1 : off, left ? lo - 1 : off, right ? hi : off);
  for (int pass = 0; pass < 2; ++pass) {
    k_plane_lists<<<kListBlocks, kListThreads, 0, s>>>(x, n, plane, pieces, lists, counts, cap, pass);
    g_launches.fetch_add(1, std::memory_order_relaxed);
  }
  const cudaError_t e = cudaGetLastError();
  dev_free(pieces, s);
  if (e != cudaSuccess) return fail(SCN_E_CUDA, std::string("plane lists: ") + cudaGetErrorString(e));
  return SCN_OK;
}

}  // namespace scn

using namespace scn;

struct scn_halo {
  char *inbox = nullptr;         // [flags: 2 lines][side][slot][slot_bytes]
  int64_t slot_bytes = 0;
  char *peer[2] = {nullptr, nullptr};  // neighbours' inboxes as mapped here (left, right); may be my own
  bool peer_is_ipc[2] = {false, false};
  unsigned int *done = nullptr;  // [0] block counter, [1] status
  unsigned long long seq = 0;
  unsigned int spin_limit = 4u << 20;  // ~1 s of 200 ns sleeps
};

namespace {
constexpr size_t kHeader = 2 * scn::kFlagStride * sizeof(unsigned long long);
inline char *slot_of(char *inbox, int64_t slot_bytes, int side, int slot) {
  return inbox + kHeader + (size_t)(side * 2 + slot) * (size_t)slot_bytes;
}
inline unsigned long long *seq_of(char *inbox, int side) {
  return reinterpret_cast<unsigned long long *>(inbox) + side * scn::kFlagStride;
}
}  // namespace

extern "C" {

int scn_halo_create(scn_halo **out, int64_t slot_bytes) {
  if (!out || slot_bytes < 16 || slot_bytes % 16) return fail(SCN_E_INVALID, "slot_bytes must be a positive multiple of 16");
  scn_halo *h = new scn_halo();
  h->slot_bytes = slot_bytes;
  const size_t bytes = kHeader + 4 * (size_t)slot_bytes;
  cudaError_t e = cudaMalloc(reinterpret_cast<void **>(&h->inbox), bytes);
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&h->done), 2 * sizeof(unsigned int));
  if (e == cudaSuccess) e = cudaMemset(h->inbox, 0, kHeader);
  if (e == cudaSuccess) e = cudaMemset(h->done, 0, 2 * sizeof(unsigned int));
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    if (h->inbox) cudaFree(h->inbox);
    if (h->done) cudaFree(h->done);
    delete h;
    return fail(SCN_E_CUDA, std::string("halo inbox: ") + cudaGetErrorString(e));
  }
  *out = h;
  return SCN_OK;
}

void scn_halo_destroy(scn_halo *h) {
  if (!h) return;
  cudaDeviceSynchronize();
  for (int s = 0; s < 2; ++s)
    if (h->peer[s] && h->peer_is_ipc[s]) cudaIpcCloseMemHandle(h->peer[s]);
  cudaFree(h->inbox);
  cudaFree(h->done);
  delete h;
}

int scn_halo_ipc_handle(scn_halo *h, void *handle64) {
  if (!h || !handle64) return fail(SCN_E_INVALID, "null argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  cudaIpcMemHandle_t mh;
  SCN_CUDA(cudaIpcGetMemHandle(&mh, h->inbox));
  memcpy(handle64, &mh, 64);
  return SCN_OK;
}

int scn_halo_connect(scn_halo *h, int side, const void *handle64) {
  if (!h || side < 0 || side > 1) return fail(SCN_E_INVALID, "side must be 0 (left) or 1 (right)");
  if (h->peer[side]) return fail(SCN_E_STATE, "this side is connected already");
  if (!handle64) {  // my own inbox: a rank that is its own neighbour
    h->peer[side] = h->inbox;
    h->peer_is_ipc[side] = false;
    return SCN_OK;
  }
  cudaIpcMemHandle_t mh;
  memcpy(&mh, handle64, 64);
  void *p = nullptr;
  SCN_CUDA(cudaIpcOpenMemHandle(&p, mh, cudaIpcMemLazyEnablePeerAccess));
  h->peer[side] = static_cast<char *>(p);
  h->peer_is_ipc[side] = true;
  return SCN_OK;
}

int scn_halo_set_spin_limit(scn_halo *h, int64_t polls) {
  if (!h || polls < 1 || polls > (1ll << 31)) return fail(SCN_E_INVALID, "polls out of range");
  h->spin_limit = (unsigned int)polls;
  return SCN_OK;
}

int scn_halo_exchange(scn_halo *h, const int64_t *rows, const int64_t *counts, int64_t cap, void *a,
                      int64_t a_row_bytes, void *b, int64_t b_row_bytes, void *stream) {
  if (!h || !rows || !counts || cap < 0 || !a || a_row_bytes <= 0 || (b && b_row_bytes <= 0))
    return fail(SCN_E_INVALID, "scn_halo_exchange: bad argument");
  if (!b) b_row_bytes = 0;
  if (a_row_bytes % 4 || b_row_bytes % 4) return fail(SCN_E_INVALID, "rows must be multiples of 4 bytes");
  if (a_row_bytes + b_row_bytes > h->slot_bytes) return fail(SCN_E_CAPACITY, "one row does not fit a message slot");
  cudaStream_t s = (cudaStream_t)stream;
  h->seq += 1;
  const int slot = (int)(h->seq & 1);
  HaloArgs p;
  for (int sd = 0; sd < 2; ++sd) {
    // what I send to my left neighbour arrives from ITS right, and the other way round
    p.side[sd].out = h->peer[sd] ? slot_of(h->peer[sd], h->slot_bytes, 1 - sd, slot) : nullptr;
    p.side[sd].out_seq = h->peer[sd] ? seq_of(h->peer[sd], 1 - sd) : nullptr;
    p.side[sd].in = h->peer[sd] ? slot_of(h->inbox, h->slot_bytes, sd, slot) : nullptr;
    p.side[sd].in_seq = h->peer[sd] ? seq_of(h->inbox, sd) : nullptr;
  }
  p.rows = rows;
  p.counts = counts;
  p.cap = cap;
  p.a = static_cast<char *>(a);
  p.b = static_cast<char *>(b);
  p.a_row_bytes = (int)a_row_bytes;
  p.b_row_bytes = (int)b_row_bytes;
  p.slot_bytes = h->slot_bytes;
  p.seq = h->seq;
  p.done = h->done;
  p.status = h->done + 1;
  p.spin_limit = h->spin_limit;
  const bool wide = a_row_bytes % 16 == 0 && b_row_bytes % 16 == 0 && (uintptr_t)a % 16 == 0 && (uintptr_t)b % 16 == 0;
  const int grid = 148 * 2;
  if (wide) {
    k_halo_push<uint4><<<grid, 256, 0, s>>>(p);
    SCN_LAUNCHED();
    k_halo_unpack<uint4><<<grid, 256, 0, s>>>(p);
    SCN_LAUNCHED();
  } else {
    k_halo_push<uint32_t><<<grid, 256, 0, s>>>(p);
    SCN_LAUNCHED();
    k_halo_unpack<uint32_t><<<grid, 256, 0, s>>>(p);
    SCN_LAUNCHED();
  }
  return SCN_OK;
}

int scn_halo_status(scn_halo *h, int *timed_out, int *overflow, void *stream) {
  if (!h) return fail(SCN_E_INVALID, "null handle");
  unsigned int st = 0;
  cudaStream_t s = (cudaStream_t)stream;
  SCN_CUDA(cudaMemcpyAsync(&st, h->done + 1, sizeof(st), cudaMemcpyDeviceToHost, s));
  SCN_CUDA(cudaStreamSynchronize(s));
  if (timed_out) *timed_out = (int)(st & 1u);
  if (overflow) *overflow = (int)((st >> 1) & 1u);
  if (st) SCN_CUDA(cudaMemsetAsync(h->done + 1, 0, sizeof(unsigned int), s));
  return SCN_OK;
}

}  // extern "C"
