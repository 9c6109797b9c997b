// Tensor-core gather-GEMM for sm_100a: tcgen05.mma kind::tf32 with the accumulator in TMEM.
//
//     out[o] = init(o) + sum_k in[ map[k][o] ] * W[k]           (same contract as the fp32 kernel)
//
// A work item is a tile of 128 consecutive output rows and all n_out <= 256 output planes; its accumulator
// [128 x n_out] fp32 lives in tensor memory.  The reduction runs over (offset k, 32-plane block kb); every
// step stages
//     A = the 128 gathered input rows x 32 planes (16 KB)  -> K-major, 128-byte swizzle
//     B = W[k]^T, n_out rows x 32 planes                    -> K-major, 128-byte swizzle
// and issues four tcgen05.mma (K = 8 each).  Offsets for which no row of the tile has a neighbour are skipped.
// The weights are used transposed, [volume][n_out][n_in], so that both operands are K-major (the layout in
// which 32-bit operands take the plain 128-byte swizzle); the copy is made per call, or once by the caller
// (scn_pack_weights).  fp32 inputs are consumed as tf32 (the low 13 mantissa bits are ignored), accumulation
// is fp32.
//
// Two kernels:
//   k_gather_gemm_tc_persist    the production kernel: persistent CTAs, warp-specialised (cp.async producers for
//                               the gathered rows, one bulk-tensor (TMA) copy per step for the weight block, one
//                               lane driving the tensor core, epilogue warps), two accumulators, split-K items
//   k_gather_gemm_tf32          one CTA per tile, all threads copy and one issues the MMAs, a CTA barrier per
//                               step; kept for the entry point that must not allocate and as a fallback
// Staging the gathered rows with bulk-tensor copies in tile::gather4 mode (four rows per request) was built
// and measured too: correct, but 1.3x slower than cp.async on the 250k-voxel layer, because the copy engine keeps
// few such small requests in flight; it is not part of the code any more.
//
// Every wait on an mbarrier is bounded; a wait that runs out sets an error word that the host reads
// at its next scn_check_errors, and the kernel still releases its tensor memory before returning.
#include "internal.h"
#include <cuda.h>
#include <cuda_fp16.h>
#include <stddef.h>
#include <stdlib.h>

namespace scn {

namespace {

constexpr int kTileM = 128;
constexpr int kThreads = 128;
constexpr int kABytes = kTileM * 128;  // 128 rows x 32 fp32
constexpr uint32_t kSpinLimit = 1u << 20;

__device__ unsigned int g_tc_error = 0;  // 1: an mbarrier wait ran out

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}
__device__ __forceinline__ void fence_async_proxy() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false (and records the failure) when the phase never completes.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *failed) {
  if (mbar_try_wait(bar, parity)) return true;
  if (*failed) return false;
  for (uint32_t i = 0; i < kSpinLimit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  *failed = 1;
  atomicOr(&g_tc_error, 1u);
  return false;
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }

// shared-memory matrix descriptor, 128-byte swizzle, descriptor version 1 (sm_100)
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;  // version
  d |= (uint64_t)2 << 61;  // SWIZZLE_128B
  return d;
}
// instruction descriptor: D fp32, A/B tf32, both K-major, M = 128, N = n
__host__ __device__ constexpr uint32_t instr_desc(int n) {
  return (1u << 4) | (2u << 7) | (2u << 10) | (0u << 15) | (0u << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(kTileM >> 4) << 24);
}
// the same for fp16 operands (kind::f16): A and B format fields 0 (F16)
__host__ __device__ constexpr uint32_t instr_desc_f16(int n) {
  return (1u << 4) | (0u << 7) | (0u << 10) | (0u << 15) | (0u << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(kTileM >> 4) << 24);
}
__device__ __forceinline__ void mma_tf32(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(tmem_d),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float *v) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

struct alignas(16) Ctl {     // control block behind the stages in dynamic shared memory
  unsigned long long done[8];  // per stage: MMAs that read the stage have retired
  unsigned long long acc;      // all MMAs of the tile have retired
  uint32_t tmem_base;
  int failed;
  int nk;                      // offsets with at least one valid row
  unsigned int kmask;          // bit k: offset k has a valid row
  int klist[32];
};

// STAGES ring slots; copies run AHEAD steps in front of the tensor core, which leaves the MMAs of a
// step STAGES - AHEAD iterations to retire before their slot is refilled.
// gridDim.y > 1 splits the reduction steps of a tile over several CTAs (few tiles, long reductions):
// each CTA then writes its partial tile to `partial` [gridDim.y][tiles * 128][Cout] and a second kernel
// adds the partials in a fixed order.
template <int STAGES, int AHEAD>
__global__ void __launch_bounds__(kThreads)
k_gather_gemm_tf32(const float *__restrict__ in, long long in_stride, const int32_t *__restrict__ map, int K,
                   long long n_out, const float *__restrict__ W, const float *__restrict__ bias,
                   float *out, long long out_stride, int Cin, int Cout, const float *init, long long init_stride,
                   uint32_t tmem_cols, float *__restrict__ partial) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // layout: [stages: A (16 KB) + B (Cout*128 B)] [Ctl] [s_map: K*128 ints]
  const uint32_t stage_bytes = kABytes + (uint32_t)Cout * 128u;
  unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  Ctl *ctl = reinterpret_cast<Ctl *>(smem + (size_t)STAGES * stage_bytes);
  int *s_map = reinterpret_cast<int *>(ctl + 1);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const long long row0 = (long long)blockIdx.x * kTileM;
  const int KB = Cin >> 5;

  // ---- neighbour rows of the tile, and the list of offsets that have any -------------------------
  // thread t owns row t: all K loads are issued back to back (independent), then one block-wide OR
  if (tid == 0) {
    ctl->failed = 0;
    ctl->kmask = 0;
  }
  __syncthreads();
  {
    const long long row = row0 + tid;
    unsigned int mine = 0;
#pragma unroll
    for (int k = 0; k < 27; ++k) {
      if (k < K) {
        int v = -1;
        if (row < n_out) v = map ? __ldg(map + (long long)k * n_out + row) : (int)row;
        s_map[k * kTileM + tid] = v;
        mine |= (v >= 0 ? 1u : 0u) << k;
      }
    }
    mine = __reduce_or_sync(0xffffffffu, mine);
    if (lane == 0 && mine) atomicOr(&ctl->kmask, mine);
  }
  __syncthreads();
  if (tid == 0) {
    int n = 0;
    const unsigned int km = ctl->kmask;
    for (int k = 0; k < K; ++k)
      if (km >> k & 1u) ctl->klist[n++] = k;
    ctl->nk = n;
  }
  __syncthreads();
  const int nk = ctl->nk;
  const int Tall = nk * KB;
  const int t0 = (int)(((long long)Tall * blockIdx.y) / gridDim.y);
  const int T = (int)(((long long)Tall * (blockIdx.y + 1)) / gridDim.y) - t0;
  float *pdst = partial ? partial + ((long long)blockIdx.y * gridDim.x * kTileM + (long long)blockIdx.x * kTileM) * Cout : nullptr;
  if (T == 0) {  // nothing to reduce here: the tile (or this share of it) contributes zero
    if (pdst) {
      for (int i = tid; i < kTileM * Cout; i += kThreads) pdst[i] = 0.f;
    } else if (init != out) {
      for (long long i = tid; i < (long long)kTileM * Cout; i += kThreads) {
        const long long row = row0 + i / Cout;
        const int c = (int)(i % Cout);
        if (row < n_out) out[row * out_stride + c] = init ? init[row * init_stride + c] : (bias ? __ldg(bias + c) : 0.f);
      }
    }
    return;
  }

  // ---- barriers and tensor memory ----------------------------------------------------------------
  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) mbar_init(smem_u32(&ctl->done[s]), 1);
    mbar_init(smem_u32(&ctl->acc), 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&ctl->tmem_base)),
                 "r"(tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_d = ctl->tmem_base;
  const uint32_t idesc = instr_desc(Cout);
  const uint32_t smem_base = smem_u32(smem);
  volatile int *failed = &ctl->failed;

  // stage the operands of reduction step `it` into ring slot `slot`
  // the step to be staged next: offset index into klist and plane block, advanced without divisions;
  // tiles start at different offsets so that concurrently running CTAs do not all fetch the same weight
  // block from the same L2 lines at the same time
  int ld_ki = (t0 / KB + (int)(blockIdx.x % 27u)) % nk, ld_kb = t0 % KB;
  const int lc = tid & 7, lr0 = tid >> 3;
  const uint32_t ldst0 = (uint32_t)((lr0 >> 3) << 10) + (uint32_t)((lr0 & 7) << 7) + (uint32_t)((lc ^ (lr0 & 7)) << 4);
  const float *in_c = in + (lc << 2);
  auto load_step = [&](int /*it*/, int slot) {
    const int k = ctl->klist[ld_ki];
    const int kb = ld_kb;
    if (++ld_kb == KB) {
      ld_kb = 0;
      if (++ld_ki == nk) ld_ki = 0;
    }
    const uint32_t a_base = smem_base + (uint32_t)slot * stage_bytes;
    const uint32_t b_base = a_base + kABytes;
    const int *mr = s_map + k * kTileM + lr0;
    int src[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) src[j] = mr[16 * j];
    const float *in_kb = in_c + (kb << 5);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float *p = src[j] >= 0 ? in_kb + (long long)src[j] * in_stride : in;
      cp_async16(a_base + ldst0 + (uint32_t)(j << 11), p, src[j] >= 0 ? 16u : 0u);
    }
    // transposed weights Wt[k][n][Cin]: row n of the tile is 32 consecutive planes of Wt[k][n]
    const float *wk = W + (long long)k * Cout * Cin + (kb << 5) + (lc << 2);
    for (int n = lr0; n < Cout; n += 16) {
      const uint32_t dst = b_base + (uint32_t)((n >> 3) << 10) + (uint32_t)((n & 7) << 7) + (uint32_t)((lc ^ (n & 7)) << 4);
      cp_async16(dst, wk + (long long)n * Cin, 16u);
    }
  };

  // ---- software pipeline --------------------------------------------------------------------------
  for (int st = 0; st < AHEAD; ++st) {
    if (st < T) load_step(st, st % STAGES);
    cp_async_commit();
  }
  for (int it = 0; it < T; ++it) {
    cp_async_wait<AHEAD - 1>();  // this thread's copies of step `it` have landed
    fence_async_proxy();         // make them visible to the tensor core (async proxy)
    __syncthreads();
    const int slot = it % STAGES;
    if (tid == 0 && !*failed) {
      tc_fence_after();
      const uint32_t a_base = smem_base + (uint32_t)slot * stage_bytes;
      const uint32_t b_base = a_base + kABytes;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint64_t a_desc = smem_desc(a_base + j * 32, 16, 1024);
        const uint64_t b_desc = smem_desc(b_base + j * 32, 16, 1024);
        mma_tf32(tmem_d, a_desc, b_desc, idesc, (it > 0 || j > 0) ? 1u : 0u);
      }
      mma_commit(smem_u32(&ctl->done[slot]));
      if (it == T - 1) mma_commit(smem_u32(&ctl->acc));
    }
    // refill: step it+AHEAD goes into the slot last read by step it+AHEAD-STAGES
    const int nxt = it + AHEAD;
    if (nxt < T) {
      const int prev = nxt - STAGES;
      if (prev >= 0) mbar_wait(smem_u32(&ctl->done[prev % STAGES]), (uint32_t)((prev / STAGES) & 1), failed);
      if (!*failed) load_step(nxt, nxt % STAGES);
    }
    cp_async_commit();
  }
  cp_async_wait<0>();

  // ---- epilogue: TMEM -> registers -> global ------------------------------------------------------
  mbar_wait(smem_u32(&ctl->acc), 0, failed);
  __syncthreads();
  const bool ok = !*failed;  // block-uniform: tcgen05.ld below is warp-collective
  tc_fence_after();
  if (ok) {
    const long long row = row0 + warp * 32 + lane;
    for (int c0 = 0; c0 < Cout; c0 += 32) {
      float v[32];
      tmem_ld32(tmem_d + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, v);  // warp-collective: all lanes take part
      if (pdst) {
        float *o = pdst + (long long)(warp * 32 + lane) * Cout + c0;
#pragma unroll
        for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4 *>(o + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
      } else if (row < n_out) {
        float *o = out + row * out_stride + c0;
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          float4 r = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
          if (init) {
            const float4 old = *reinterpret_cast<const float4 *>(init + row * init_stride + c0 + j);
            r.x += old.x; r.y += old.y; r.z += old.z; r.w += old.w;
          } else if (bias) {
            r.x += __ldg(bias + c0 + j); r.y += __ldg(bias + c0 + j + 1);
            r.z += __ldg(bias + c0 + j + 2); r.w += __ldg(bias + c0 + j + 3);
          }
          *reinterpret_cast<float4 *>(o + j) = r;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_d), "r"(tmem_cols) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------
// bulk-tensor (TMA) helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_tile2d(uint32_t dst, const CUtensorMap *tm, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(tm)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

// ---------------------------------------------------------------------------------------------
// persistent, warp-specialised kernel
// ---------------------------------------------------------------------------------------------
// One CTA per SM walks over work items (item = blockIdx.x + i * gridDim.x).  Thirteen warps, three roles:
//   warps 0-3   epilogue   wait for a finished accumulator, TMEM -> registers -> global, hand the
//                          accumulator back (two accumulators alternate, so the tensor core starts the
//                          next tile while this one is written out)
//   warps 4-11  producers  every reduction step (offset k, 32-plane block kb) belongs to ONE producer warp
//                          (the one that owns the step's ring slot): the warp waits for the slot, copies all 128
//                          gathered rows with 16-byte cp.async (zero-fill for missing neighbours; 32 copies per
//                          lane, all in flight together), has one lane fetch the step's weight block with a
//                          single bulk-tensor copy, waits for its own copies, makes them visible to the tensor
//                          core's proxy and arrives on the slot's `full` barrier.  As many steps as there are
//                          slots (up to eight) are therefore in flight and the fixed cost of a step (barrier waits, fences, arrivals) is
//                          paid by one warp instead of all eight.  The producers together stage each tile's map
//                          entries in shared memory one tile ahead (three buffers) and agree on the offsets
//                          that have any neighbour; all of them walk the same list of steps.
//   warp 12     tensor core waits `full`; one elected lane issues the four tcgen05.mma of the step (descriptors
//                          are advanced by adding to their low words) and lets tcgen05.commit release the slot
//                          (`empty`) and, at the end of a tile, publish the accumulator (`accfull`).  The whole
//                          warp runs the loop so that the ring position stays a warp-uniform value.
// Every blocking primitive is a bounded mbarrier wait.  A tile with no neighbour at all still runs one step
// of zero rows so that all roles see the same sequence of tiles.
constexpr int kPThreads = 448;  // 4 epilogue warps, 8 producer warps, 1 tensor-core warp, 1 weight-loading warp
constexpr int kProdWarps = 8;
constexpr int kMaxStages = 8;
constexpr int kMapBufs = 3;
constexpr uint32_t kInfoDone = 1;  // info word of a step: (steps of the item << 8 | its first plane block << 1) on an item's first step, or this flag

struct alignas(16) CtlP {
  unsigned long long full[kMaxStages];
  unsigned long long empty[kMaxStages];
  unsigned long long accfull[2];
  unsigned long long accempty[2];
  unsigned long long mapfull[kMapBufs];
  unsigned long long pad_;  // keeps kmask_part on a 16-byte boundary (it is read as two uint4): 8 + 8 + 2 + 2 + 3 + 1 words
  uint32_t info[kMaxStages];
  uint32_t kmask_part[kMapBufs][kProdWarps];
  uint32_t tmem_base;
  int failed;
};
static_assert(offsetof(CtlP, kmask_part) % 16 == 0, "kmask_part is read with 16-byte loads");

// tcgen05.mma with the descriptors given as (low word, shared high word)
template <bool HALF>
__device__ __forceinline__ void mma_lohi(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t idesc,
                                         uint32_t accumulate) {
  if (HALF)
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}\n" ::"r"(tmem_d),
        "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "r"(accumulate)
        : "memory");
  else
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], da, db, %4, p;\n\t}\n" ::"r"(tmem_d),
        "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "r"(accumulate)
        : "memory");
}

// HALF: the feature rows are fp16 (in_stride in fp16 elements) and so are the weights; a reduction step then covers
// 64 planes (a 128-byte operand row holds 64 fp16) with four K = 16 MMAs, planes beyond n_in are zero-filled.
template <bool HALF>
__global__ void __launch_bounds__(kPThreads, 1)
k_gather_gemm_tc_persist(const void *__restrict__ in_v, long long in_stride, const __grid_constant__ CUtensorMap tmB,
                           const int32_t *__restrict__ map, int K, long long n_out, const float *__restrict__ bias,
                           float *out, long long out_stride, int Cin, int Cout, const float *init, long long init_stride,
                           uint32_t acc_cols, int stages, int stages_b, long long tiles, int Z, float *__restrict__ partial,
                           const EpiBn epi) {
  // shared memory: `stages` operand tiles (the gathered rows of a step, 16 KB each), `stages_b` weight boxes
  // (n_out x 128 bytes each), the control block, the map buffers.  The two rings are separate because what bounds the
  // kernel is the number of gathered bytes in flight: a weight box per operand slot would take half of the room.
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t b_bytes = (uint32_t)Cout * 128u;
  unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t b_ring = (uint32_t)stages * kABytes;  // offset of the weight ring
  CtlP *ctl = reinterpret_cast<CtlP *>(smem + (size_t)b_ring + (size_t)stages_b * b_bytes);
  int *s_map = reinterpret_cast<int *>(ctl + 1);  // [kMapBufs][K][128]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr int kStepPlanes = HALF ? 64 : 32;  // planes per reduction step (128 bytes of a row)
  constexpr int kChunkPlanes = HALF ? 8 : 4;   // planes per 16-byte copy
  constexpr int kElem = HALF ? 2 : 4;
  const int KB = (Cin + kStepPlanes - 1) / kStepPlanes;
  const unsigned char *in = static_cast<const unsigned char *>(in_v);
  // work items: (tile, share z of its reduction steps); Z == 1 means whole tiles
  const long long items = tiles * Z;
  const long long my_tiles = (items - (long long)blockIdx.x + gridDim.x - 1) / gridDim.x;

  if (tid == 0) {
    ctl->failed = 0;
    for (int s = 0; s < stages; ++s) {
      // a step is ready when its gathered rows AND its weight box have landed: the owning producer warp's arrival and
      // the weight warp's expect_tx arrival complete the same barrier, so the issuing warp waits once per step
      mbar_init(smem_u32(&ctl->full[s]), 2);
      mbar_init(smem_u32(&ctl->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&ctl->accfull[b]), 1);
      mbar_init(smem_u32(&ctl->accempty[b]), 4);  // one arrival per epilogue warp
    }
    // one arrival per producer warp, one of the weight-loading warp (which thereby keeps the producers from reusing a
    // map buffer whose offset mask it has not read yet)
    for (int b = 0; b < kMapBufs; ++b) mbar_init(smem_u32(&ctl->mapfull[b]), kProdWarps + 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&ctl->tmem_base)),
                 "r"(acc_cols * 2)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  const uint32_t smem_base = smem_u32(smem);
  volatile int *failed = &ctl->failed;

  if (warp >= 4 && warp < 4 + kProdWarps) {
    // =========================== producers ========================================================
    const int tp = tid - 128, pw = warp - 4;
    // map staging: thread tp and thread tp + 128 share row (tp & 127) of a tile: one takes the even offsets, the other the odd
    const int prow = tp & 127, par = tp >> 7;
    // where row prow's entry sits among an offset's 128: the copying lanes take rows q, q + 4, q + 8, ... and read their
    // 32 entries as eight 16-byte words, so the entries of rows with the same (row & 3) are stored next to each other
    const int pslot = ((prow & 3) << 5) | (prow >> 2);
    int nxt[14];  // map entries of this thread's row, offsets par, par + 2, ..., of the tile after the current one
    auto load_map = [&](long long item) {
      const long long tile = item / Z;
      const long long row = tile * kTileM + prow;
#pragma unroll
      for (int j = 0; j < 14; ++j) {
        const int k = 2 * j + par;
        int v = -1;
        if (k < K && item < items && row < n_out) v = map ? __ldg(map + (long long)k * n_out + row) : (int)row;
        nxt[j] = v;
      }
    };
    auto publish_map = [&](int buf) {  // registers -> shared memory; which offsets have any row
      int *mrows = s_map + buf * K * kTileM;
      unsigned int mine = 0;
#pragma unroll
      for (int j = 0; j < 14; ++j) {
        const int k = 2 * j + par;
        if (k < K) {
          mrows[k * kTileM + pslot] = nxt[j];
          mine |= (nxt[j] >= 0 ? 1u : 0u) << k;
        }
      }
      mine = __reduce_or_sync(0xffffffffu, mine);
      __syncwarp();
      if (lane == 0) {
        ctl->kmask_part[buf][pw] = mine;
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(&ctl->mapfull[buf])) : "memory");
      }
    };
    load_map(blockIdx.x);
    publish_map(0);
    load_map((long long)blockIdx.x + gridDim.x);
    // ring position of the step being enumerated, kept without divisions
    int slot = 0;
    uint32_t wrapped = 0;  // completed passes over the ring
    // A ring slot belongs to one producer warp (slot s to warp s): the warp then waits for consecutive phases of
    // the slot's `empty` barrier, which a parity wait can tell apart; with fewer slots than producer warps the
    // surplus warps only help staging the maps.
    // copies of a step: lane covers 16-byte chunk c of rows q + 4j, j = 0..31; the swizzle term depends on row & 7
    const int c = lane & 7, q = lane >> 3;
    const uint32_t dst_even = (uint32_t)(q << 7) + (uint32_t)((c ^ q) << 4);
    const uint32_t dst_odd = (uint32_t)((q + 4) << 7) + (uint32_t)((c ^ (q + 4)) << 4);
    const unsigned char *in_c = in + (size_t)c * 16;  // this lane's 16-byte chunk of a row block
    const uint32_t row_bytes = (uint32_t)(in_stride * kElem);  // the launcher keeps rows below 4 GB
    int mbuf = 0;
    uint32_t mphase = 0;
    for (long long i = 0; i < my_tiles && !*failed; ++i) {
      const long long item = (long long)blockIdx.x + i * gridDim.x;
      // This tile's map entries were published while the previous tile ran, so the wait is normally free.  Once it
      // has passed, every producer warp is done with the tile before the previous one, whose buffer (the third)
      // takes the next tile's entries; the loads for the tile after that start right away.
      if (!mbar_wait(smem_u32(&ctl->mapfull[mbuf]), mphase, failed)) break;
      publish_map(mbuf + 1 == kMapBufs ? 0 : mbuf + 1);
      load_map(item + 2ll * gridDim.x);
      const int *mrows = s_map + mbuf * K * kTileM;
      const uint4 km0 = *reinterpret_cast<const uint4 *>(&ctl->kmask_part[mbuf][0]);
      const uint4 km1 = *reinterpret_cast<const uint4 *>(&ctl->kmask_part[mbuf][4]);
      const unsigned int kmask = km0.x | km0.y | km0.z | km0.w | km1.x | km1.y | km1.z | km1.w;
      if (++mbuf == kMapBufs) {
        mbuf = 0;
        mphase ^= 1u;
      }
      // this item's share [t0, t1) of the tile's reduction steps; an empty share still runs one step of zero rows
      const int z = (int)(item % Z);
      const int nk_all = __popc(kmask);
      const int Tall = nk_all * KB;
      const int t0 = (int)(((long long)Tall * z) / Z);
      const int Tz = (int)(((long long)Tall * (z + 1)) / Z) - t0;
      const int nk = Tz > 0 ? nk_all : 0;  // 0: stage zero rows only
      const int T = Tz > 0 ? Tz : 1;
      unsigned int rest = kmask;
      int kb = 0;
      if (Tz > 0) {
        for (int r = t0 / KB; r > 0; --r) rest &= rest - 1;
        kb = t0 % KB;
      }
      int k = (Tz > 0 && rest) ? __ffs(rest) - 1 : 0;
      bool stop = false;
      for (int it = 0; it < T; ++it) {
        if (slot == pw) {
          if (wrapped > 0 && !mbar_wait(smem_u32(&ctl->empty[slot]), (wrapped - 1) & 1u, failed)) {
            stop = true;
            break;
          }
          const uint32_t a_base = smem_base + (uint32_t)slot * kABytes;
          const uint32_t bar = smem_u32(&ctl->full[slot]);
          if (lane == 0 && it == 0) ctl->info[slot] = ((uint32_t)T << 8) | ((uint32_t)kb << 1);  // the item's step count and first plane block ride on its first step
          const int4 *mr = reinterpret_cast<const int4 *>(mrows + k * kTileM + (q << 5));
          const unsigned char *in_kb = in_c + (size_t)kb * 128;
          // fp16 rows: the last block of a row may be half empty (n_in = 32, 96, 160, 224).  The tensor-core warp then
          // issues only the two K = 16 MMAs that cover the first 32 planes, so the other chunks of the slot are never
          // read and their lanes copy nothing.
          const bool chunk_ok = !HALF || kb * kStepPlanes + c * kChunkPlanes < Cin;
          if (chunk_ok) {
#pragma unroll
            for (int j0 = 0; j0 < 32; j0 += 8) {
              int src[8];
              {
                const int4 lo = mr[j0 >> 2], hi = mr[(j0 >> 2) + 1];
                src[0] = lo.x; src[1] = lo.y; src[2] = lo.z; src[3] = lo.w;
                src[4] = hi.x; src[5] = hi.y; src[6] = hi.z; src[7] = hi.w;
              }
              if (!nk) {
#pragma unroll
                for (int j = 0; j < 8; ++j) src[j] = -1;
              }
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                // an absent neighbour copies zero bytes (the chunk is zero-filled) from row 0, so that the address is
                // one 32 x 32 -> 64-bit multiply-add for every lane
                const unsigned char *p = in_kb + (unsigned long long)(uint32_t)max(src[j], 0) * row_bytes;
                const uint32_t dst = a_base + (uint32_t)(((j0 + j) >> 1) << 10) + (((j0 + j) & 1) ? dst_odd : dst_even);
                cp_async16(dst, p, src[j] >= 0 ? 16u : 0u);
              }
            }
          }
          cp_async_commit();
          cp_async_wait<0>();
          fence_async_proxy();
          __syncwarp();
          if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
        }
        if (++slot == stages) {
          slot = 0;
          ++wrapped;
        }
        if (++kb == KB) {
          kb = 0;
          rest &= rest - 1;
          k = rest ? __ffs(rest) - 1 : 0;
        }
      }
      if (stop) break;
    }
    // sentinel step: tells the tensor-core warp that no more work follows
    if (slot == pw && !*failed) {
      bool okw = true;
      if (wrapped > 0) okw = mbar_wait(smem_u32(&ctl->empty[slot]), (wrapped - 1) & 1u, failed);
      if (okw && lane == 0) {
        const uint32_t bar = smem_u32(&ctl->full[slot]);
        ctl->info[slot] = kInfoDone;
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
      }
    }
    __syncwarp();
  } else if (warp == 4 + kProdWarps) {
    // =========================== tensor core ======================================================
    // The whole warp runs the loop, so that ring position and descriptors are warp-uniform values; one elected
    // lane issues.  The first step of an item carries the item's step count, the steps after it are counted.
    const uint32_t idesc = HALF ? instr_desc_f16(Cout) : instr_desc(Cout);
    // descriptor words: low = start address / 16 | leading offset 16 B; high = stride offset 1024 B, version, 128-byte swizzle
    const uint32_t desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);
    const uint32_t a_lo0 = ((smem_base >> 4) & 0x3FFFu) | (1u << 16);
    const uint32_t stage16 = kABytes >> 4, bstage16 = b_bytes >> 4;
    const uint32_t b_lo0 = (((smem_base + b_ring) >> 4) & 0x3FFFu) | (1u << 16);
    const uint32_t full0 = smem_u32(&ctl->full[0]), empty0 = smem_u32(&ctl->empty[0]);
    long long tile_i = 0;
    int slot = 0, bslot = 0;
    uint32_t phase = 0, a_lo = a_lo0, b_lo = b_lo0;
    const bool half_block = HALF && Cin - (KB - 1) * kStepPlanes <= 32;  // the last plane block of a row holds 32 planes
    bool alive = true;
    while (alive) {
      if (!mbar_wait(full0 + 8u * (uint32_t)slot, phase, failed)) break;
      const uint32_t info = __shfl_sync(0xffffffffu, ctl->info[slot], 0);
      if (info & kInfoDone) break;
      const int T = (int)(info >> 8);
      int kb = (int)((info >> 1) & 7u);
      const int buf = (int)(tile_i & 1);
      const uint32_t tmem_d = tmem_base + (uint32_t)buf * acc_cols;
      // the epilogue must have drained this accumulator (used by tile tile_i - 2)
      if (tile_i >= 2 && !mbar_wait(smem_u32(&ctl->accempty[buf]), (uint32_t)(((tile_i >> 1) - 1) & 1), failed)) break;
      tc_fence_after();  // the epilogue's TMEM reads of this accumulator are ordered before the new MMAs
      for (int t = 0; t < T; ++t) {
        if (t > 0 && !mbar_wait(full0 + 8u * (uint32_t)slot, phase, failed)) {
          alive = false;
          break;
        }
        if (elect_one()) {
          mma_lohi<HALF>(tmem_d, a_lo, b_lo, desc_hi, idesc, t > 0 ? 1u : 0u);
          mma_lohi<HALF>(tmem_d, a_lo + 2, b_lo + 2, desc_hi, idesc, 1u);
          if (kb != KB - 1 || !half_block) {
            mma_lohi<HALF>(tmem_d, a_lo + 4, b_lo + 4, desc_hi, idesc, 1u);
            mma_lohi<HALF>(tmem_d, a_lo + 6, b_lo + 6, desc_hi, idesc, 1u);
          }
          mma_commit(empty0 + 8u * (uint32_t)slot);  // releases the operand slot and, for the weight warp, the weight slot
          if (t == T - 1) mma_commit(smem_u32(&ctl->accfull[buf]));
        }
        if (++kb == KB) kb = 0;
        a_lo += stage16;
        if (++slot == stages) {
          slot = 0;
          phase ^= 1u;
          a_lo = a_lo0;
        }
        b_lo += bstage16;
        if (++bslot == stages_b) {
          bslot = 0;
          b_lo = b_lo0;
        }
      }
      ++tile_i;
    }
    __syncwarp();
  } else if (warp == 4 + kProdWarps + 1) {
    // =========================== weights ==========================================================
    // One warp walks all steps in order and fetches each step's weight block with one TMA box into the weight ring.
    // The copy completes the step's `full` barrier (its second arrival, with the box's byte count), so the issuing
    // warp has one wait per step.  The ring has no barriers of its own: the weight slot of step g was last used by step
    // g - stages_b, whose tcgen05.commit arrived on that step's operand-slot `empty` barrier; the warp waits for that
    // phase.  There are more operand slots than weight slots, so that barrier cannot be a phase further (step
    // g - stages_b + stages has no weights yet), and when the wait has passed, step g - stages has been consumed too:
    // the arrival on `full` lands in the phase that belongs to step g.  The warp takes part in the map barriers like a
    // producer warp: its arrival for tile i + 1 comes after it has read tile i's offset mask, which keeps the
    // producers from reusing that buffer early.
    const uint32_t full0 = smem_u32(&ctl->full[0]), empty0 = smem_u32(&ctl->empty[0]);
    int bslot = 0, mbuf = 0, aslot = 0, eslot = 0;
    uint32_t mphase = 0, ephase = 0;
    long long g = 0;  // steps walked so far
    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(&ctl->mapfull[0])) : "memory");
    bool stop = false;
    for (long long i = 0; i < my_tiles && !*failed && !stop; ++i) {
      const long long item = (long long)blockIdx.x + i * gridDim.x;
      if (!mbar_wait(smem_u32(&ctl->mapfull[mbuf]), mphase, failed)) break;
      const uint4 km0 = *reinterpret_cast<const uint4 *>(&ctl->kmask_part[mbuf][0]);
      const uint4 km1 = *reinterpret_cast<const uint4 *>(&ctl->kmask_part[mbuf][4]);
      const unsigned int kmask = km0.x | km0.y | km0.z | km0.w | km1.x | km1.y | km1.z | km1.w;
      if (++mbuf == kMapBufs) {
        mbuf = 0;
        mphase ^= 1u;
      }
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(&ctl->mapfull[mbuf])) : "memory");
      // the same enumeration of the item's steps as the producers'
      const int z = (int)(item % Z);
      const int nk_all = __popc(kmask);
      const int Tall = nk_all * KB;
      const int t0 = (int)(((long long)Tall * z) / Z);
      const int Tz = (int)(((long long)Tall * (z + 1)) / Z) - t0;
      const int T = Tz > 0 ? Tz : 1;
      unsigned int rest = kmask;
      int kb = 0;
      if (Tz > 0) {
        for (int r = t0 / KB; r > 0; --r) rest &= rest - 1;
        kb = t0 % KB;
      }
      int k = (Tz > 0 && rest) ? __ffs(rest) - 1 : 0;
      for (int it = 0; it < T; ++it) {
        if (g >= stages_b) {
          if (!mbar_wait(empty0 + 8u * (uint32_t)eslot, ephase, failed)) {
            stop = true;
            break;
          }
          if (++eslot == stages) {
            eslot = 0;
            ephase ^= 1u;
          }
        }
        if (lane == 0) {
          const uint32_t bar = full0 + 8u * (uint32_t)aslot;
          mbar_expect_tx(bar, b_bytes);
          tma_tile2d(smem_base + b_ring + (uint32_t)bslot * b_bytes, &tmB, bar, kb * kStepPlanes, k * Cout);
        }
        ++g;
        if (++aslot == stages) aslot = 0;
        if (++bslot == stages_b) bslot = 0;
        if (++kb == KB) {
          kb = 0;
          rest &= rest - 1;
          k = rest ? __ffs(rest) - 1 : 0;
        }
      }
    }
    // the sentinel step carries no weights: the second arrival its `full` barrier waits for
    if (!stop && !*failed && lane == 0)
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(full0 + 8u * (uint32_t)aslot) : "memory");
    __syncwarp();
  } else {
    // =========================== epilogue =========================================================
    for (long long i = 0; i < my_tiles; ++i) {
      const long long item = (long long)blockIdx.x + i * gridDim.x;
      const long long tile = item / Z;
      float *pdst = partial ? partial + (((item % Z) * tiles + tile) * kTileM + warp * 32 + lane) * Cout : nullptr;
      const int buf = (int)(i & 1);
      if (!mbar_wait(smem_u32(&ctl->accfull[buf]), (uint32_t)((i >> 1) & 1), failed)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + (uint32_t)buf * acc_cols + ((uint32_t)(warp * 32) << 16);
      const long long row = tile * kTileM + warp * 32 + lane;
      for (int c0 = 0; c0 < Cout; c0 += 32) {
        float v[32];
        tmem_ld32(taddr + (uint32_t)c0, v);
        if (c0 + 32 >= Cout) {  // last read of this accumulator: hand it back before the stores
          tc_fence_before();
          __syncwarp();
          if (lane == 0)
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(&ctl->accempty[buf])) : "memory");
        }
        if (pdst) {
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<float4 *>(pdst + c0 + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        } else if (row < n_out) {
          float *o = out + row * out_stride + c0;
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            float4 r = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            if (init) {
              const float4 old = *reinterpret_cast<const float4 *>(init + row * init_stride + c0 + j);
              r.x += old.x; r.y += old.y; r.z += old.z; r.w += old.w;
            } else if (bias) {
              r.x += __ldg(bias + c0 + j); r.y += __ldg(bias + c0 + j + 1);
              r.z += __ldg(bias + c0 + j + 2); r.w += __ldg(bias + c0 + j + 3);
            }
            if (!epi.skip_raw) *reinterpret_cast<float4 *>(o + j) = r;
            v[j] = r.x; v[j + 1] = r.y; v[j + 2] = r.z; v[j + 3] = r.w;
          }
          if (epi.dst) {  // the BatchNorm + ReLU behind this convolution, as fp16 rows for the next one
            __half *hd = static_cast<__half *>(epi.dst) + row * epi.stride + c0;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              __align__(16) __half h8[8];
#pragma unroll
              for (int u = 0; u < 8; ++u) {
                float y = fmaf(v[j + u], __ldg(epi.scale + c0 + j + u), __ldg(epi.shift + c0 + j + u));
                y = y > 0.f ? y : y * epi.leak;
                h8[u] = __float2half_rn(fminf(fmaxf(y, -65504.f), 65504.f));
              }
              *reinterpret_cast<uint4 *>(hd + j) = *reinterpret_cast<const uint4 *>(h8);
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(acc_cols * 2) : "memory");
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime's driver entry point lookup (no link-time libcuda dependency)
static int encode_2d(CUtensorMap *tm, const void *base, bool half, uint64_t cols, uint64_t rows, uint64_t row_stride_bytes,
                     uint32_t box_cols, uint32_t box_rows) {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    SCN_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
    if (!p || q != cudaDriverEntryPointSuccess) return fail(SCN_E_CUDA, "cuTensorMapEncodeTiled is not available");
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {row_stride_bytes};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(tm, half ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void *>(base), dims,
                  strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(SCN_E_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
  return SCN_OK;
}

// The persistent kernel's launches sit in the host-bound part of a frame (deep levels: kernels of 10-20 us), so the
// host side of a launch is kept short: tensor maps are encoded once per (weights, shape) and kept, and the split-K
// scratch is one grow-only block per host thread that consecutive launches on the same stream reuse (stream order
// makes that safe); a launch on another stream falls back to the stream-ordered pool.
struct TensorMapKey {
  const void *base;
  uint64_t cols, rows;
  uint32_t box_cols, box_rows;
  bool half;
  bool operator==(const TensorMapKey &o) const {
    return base == o.base && cols == o.cols && rows == o.rows && box_cols == o.box_cols && box_rows == o.box_rows && half == o.half;
  }
};
static int cached_tensor_map(CUtensorMap *tm, const void *base, bool half, uint64_t cols, uint64_t rows, uint32_t box_cols,
                             uint32_t box_rows) {
  constexpr int kSlots = 256;  // direct-mapped on the weight address; a network has tens of weight tensors
  thread_local TensorMapKey keys[kSlots] = {};
  thread_local CUtensorMap maps[kSlots];
  const TensorMapKey k{base, cols, rows, box_cols, box_rows, half};
  const size_t slot = (reinterpret_cast<uintptr_t>(base) >> 8) % kSlots;
  if (keys[slot].base && keys[slot] == k) {
    *tm = maps[slot];
    return SCN_OK;
  }
  SCN_TRY(encode_2d(tm, base, half, cols, rows, cols * (half ? 2 : 4), box_cols, box_rows));
  keys[slot] = k;
  maps[slot] = *tm;
  return SCN_OK;
}

struct SplitKScratch {
  float *p = nullptr;
  size_t floats = 0;
  cudaStream_t stream = nullptr;
  int device = -1;
};
// returns scratch for `floats` floats; *pooled tells the caller to hand it back with dev_free
static int splitk_scratch(float **out, size_t floats, cudaStream_t s, bool *pooled) {
  thread_local SplitKScratch sc;
  int dev = 0;
  SCN_CUDA(cudaGetDevice(&dev));
  *pooled = false;
  if (sc.p && (sc.stream != s || sc.device != dev)) {  // another stream or device: leave the cached block alone
    *pooled = true;
    return dev_alloc_t(out, floats, s);
  }
  if (sc.floats < floats) {
    if (sc.p) dev_free(sc.p, s);
    sc.p = nullptr;
    sc.floats = 0;
    const size_t want = floats + floats / 2;
    SCN_TRY(dev_alloc_t(&sc.p, want, s));
    sc.floats = want;
    sc.stream = s;
    sc.device = dev;
  }
  *out = sc.p;
  return SCN_OK;
}

// W [vol][Cin][Cout] -> Wt [vol][Cout][Cin]; 32x32 tiles through shared memory
__global__ void k_transpose_weights(const float *__restrict__ W, float *__restrict__ Wt, int Cin, int Cout) {
  __shared__ float tile[32][33];
  const float *w = W + (long long)blockIdx.z * Cin * Cout;
  float *wt = Wt + (long long)blockIdx.z * Cin * Cout;
  const int ci0 = blockIdx.y * 32, co0 = blockIdx.x * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) tile[r][threadIdx.x] = w[(long long)(ci0 + r) * Cout + co0 + threadIdx.x];
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) wt[(long long)(co0 + r) * Cin + ci0 + threadIdx.x] = tile[threadIdx.x][r];
}

// out[r][c] = (init ? init : bias) + sum_z partial[z][r][c], z ascending
__global__ void k_splitk_reduce(const float *__restrict__ partial, int Z, long long rows_padded, long long n_out, int Cout,
                                const float *__restrict__ bias, float *out, long long out_stride, const float *init,
                                long long init_stride, const EpiBn epi) {
  const int cv = Cout >> 2;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_out * cv) return;
  const long long r = i / cv;
  const int c = (int)(i % cv) << 2;
  float4 acc;
  float *o = out + r * out_stride + c;
  if (init) acc = *reinterpret_cast<const float4 *>(init + r * init_stride + c);
  else if (bias) acc = __ldg(reinterpret_cast<const float4 *>(bias + c));
  else acc = make_float4(0.f, 0.f, 0.f, 0.f);
  const float *p0 = partial + r * Cout + c;
  const long long zstride = rows_padded * Cout;
  for (int z0 = 0; z0 < Z; z0 += 8) {  // eight independent loads in flight, added in ascending z
    float4 p[8];
#pragma unroll
    for (int u = 0; u < 8; ++u)
      p[u] = (z0 + u < Z) ? __ldg(reinterpret_cast<const float4 *>(p0 + (long long)(z0 + u) * zstride))
                          : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      acc.x += p[u].x; acc.y += p[u].y; acc.z += p[u].z; acc.w += p[u].w;
    }
  }
  if (!epi.skip_raw) *reinterpret_cast<float4 *>(o) = acc;
  if (epi.dst) {
    const float4 sc = __ldg(reinterpret_cast<const float4 *>(epi.scale + c)), sh = __ldg(reinterpret_cast<const float4 *>(epi.shift + c));
    float y[4] = {fmaf(acc.x, sc.x, sh.x), fmaf(acc.y, sc.y, sh.y), fmaf(acc.z, sc.z, sh.z), fmaf(acc.w, sc.w, sh.w)};
    __align__(8) __half h4[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float t = y[u] > 0.f ? y[u] : y[u] * epi.leak;
      h4[u] = __float2half_rn(fminf(fmaxf(t, -65504.f), 65504.f));
    }
    *reinterpret_cast<uint2 *>(static_cast<__half *>(epi.dst) + r * epi.stride + c) = *reinterpret_cast<const uint2 *>(h4);
  }
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

bool tc_packable(int64_t K, int64_t Cin, int64_t Cout) {
  if (warp_mma_shape(K, Cin, Cout)) return true;
  return K >= 1 && K <= 27 && Cin > 0 && Cout > 0 && Cin % 32 == 0 && Cout % 32 == 0 && Cout <= 256;
}
int tc_pack_weights(const float *W, int64_t K, int64_t Cin, int64_t Cout, float *packed, cudaStream_t s) {
  if (!tc_packable(K, Cin, Cout)) return fail(SCN_E_INVALID, "shape cannot be packed for the tensor-core kernels");
  if (!W || !packed) return fail(SCN_E_INVALID, "null pointer");
  if (warp_mma_shape(K, Cin, Cout)) return warp_mma_pack(W, K, Cin, Cout, packed, s);
  k_transpose_weights<<<dim3((unsigned)(Cout / 32), (unsigned)(Cin / 32), (unsigned)K), dim3(32, 8), 0, s>>>(W, packed, (int)Cin,
                                                                                                          (int)Cout);
  SCN_LAUNCHED();
  return SCN_OK;
}

// Reads and clears the error word of the tensor-core kernels (synchronises the stream).
int tc_check_errors(cudaStream_t s) {
  unsigned int e = 0, zero = 0;
  SCN_CUDA(cudaMemcpyFromSymbolAsync(&e, g_tc_error, sizeof(e), 0, cudaMemcpyDeviceToHost, s));
  SCN_CUDA(cudaStreamSynchronize(s));
  if (e) {
    SCN_CUDA(cudaMemcpyToSymbolAsync(g_tc_error, &zero, sizeof(zero), 0, cudaMemcpyHostToDevice, s));
    return fail(SCN_E_CUDA, "a tensor-core kernel gave up waiting on an mbarrier; its output is invalid");
  }
  return SCN_OK;
}

// Shared-memory plan of the persistent kernel: operand slots (16 KB each, at most one per producer warp) and weight
// slots (n_out x 128 bytes each).  Three weight slots when that leaves six operand slots or more, else two.
struct PersistPlan {
  int stages, stages_b;
  size_t smem;
};
static PersistPlan persist_plan(int64_t K, int64_t Cout) {
  const size_t b_bytes = (size_t)Cout * 128;
  const size_t fixed_p = sizeof(CtlP) + (size_t)kMapBufs * K * kTileM * sizeof(int) + 1024;
  const long long room = 220ll * 1024 - (long long)fixed_p;
  PersistPlan p;
  p.stages_b = 3;
  p.stages = (int)((room - 3ll * (long long)b_bytes) / kABytes);
  if (p.stages < 6) {
    p.stages_b = 2;
    p.stages = (int)((room - 2ll * (long long)b_bytes) / kABytes);
  }
  if (p.stages > kMaxStages) p.stages = kMaxStages;
  if (p.stages_b >= p.stages) p.stages_b = p.stages > 1 ? p.stages - 1 : 1;  // the kernel relies on fewer weight slots than operand slots
  p.smem = (size_t)p.stages * kABytes + (size_t)p.stages_b * b_bytes + fixed_p;
  return p;
}

int gather_gemm_tf32(const float *in, int64_t in_stride, int64_t in_rows, const int32_t *map, int K, int64_t n_out, const float *W,
                     const float *bias, float *out, int64_t out_stride, int64_t Cin, int64_t Cout, const float *init,
                     int64_t init_stride, bool packed, cudaStream_t s, bool *handled) {
  *handled = false;
  if (Cin % 32 != 0 || Cout % 32 != 0 || Cout > 256 || K > 27) return SCN_OK;
  if (in_stride % 4 != 0 || out_stride % 4 != 0 || !aligned16(in) || !aligned16(W) || !aligned16(out)) return SCN_OK;
  if (in_stride > (1ll << 29)) return SCN_OK;  // the kernel multiplies row numbers by a 32-bit row size
  if (bias && !aligned16(bias)) return SCN_OK;
  if (init && (!aligned16(init) || init_stride % 4 != 0)) return SCN_OK;
  const size_t stage_bytes = (size_t)kABytes + (size_t)Cout * 128;
  const size_t fixed = sizeof(Ctl) + (size_t)K * kTileM * sizeof(int) + 1024;  // + alignment slack
  // two CTAs per SM when four stages fit in half an SM's shared memory, else as many stages as fit
  int stages = 4;
  if (4 * stage_bytes + fixed > 112 * 1024) {
    stages = (int)((200 * 1024 - fixed) / stage_bytes);
    if (stages > 6) stages = 6;
  }
  if (stages < 3) return SCN_OK;
  const size_t smem = (size_t)stages * stage_bytes + fixed;
  uint32_t cols = 32;
  while (cols < (uint32_t)Cout) cols <<= 1;
  const long long tiles = (n_out + kTileM - 1) / kTileM;
  int sm_count = 148;
  {
    int dev = 0;
    SCN_CUDA(cudaGetDevice(&dev));
    static int cached[64] = {0};
    if (dev >= 0 && dev < 64) {
      if (!cached[dev]) SCN_CUDA(cudaDeviceGetAttribute(&cached[dev], cudaDevAttrMultiProcessorCount, dev));
      sm_count = cached[dev];
    }
  }
  // Few tiles and a long reduction: share the steps of a tile among Z work items.  The longest chain of
  // steps any CTA runs is (items per CTA) x (steps per item + a fixed cost per item); a step takes about half a
  // microsecond.  The smallest Z whose chain is short anyway (<= 40 steps, ~20 us) is taken, because every Z > 1
  // costs a scratch allocation and a reduction launch; otherwise the Z with the shortest chain.
  const int steps_max = K * (int)(Cin / 32);
  int Z = 1;
  if (tiles < 2 * sm_count && steps_max >= 4) {
    long long best = -1;
    const int zmax = steps_max / 2 < 32 ? steps_max / 2 : 32;
    for (int z = 1; z <= zmax; ++z) {
      const long long per_cta = (tiles * z + sm_count - 1) / sm_count;
      const long long cost = per_cta * ((steps_max + z - 1) / z + 3) + (z > 1 ? 2 + z / 4 : 0);
      if (best < 0 || cost < best) {
        best = cost;
        Z = z;
      }
      if (cost <= 40) break;
    }
  }
  float *Wt = nullptr, *Wt_own = nullptr, *partial = nullptr;
  if (packed) {
    Wt = const_cast<float *>(W);  // the caller made the transposed copy once (scn_pack_weights)
  } else {
    SCN_TRY(dev_alloc_t(&Wt_own, (size_t)K * Cin * Cout, s));
    Wt = Wt_own;
    k_transpose_weights<<<dim3((unsigned)(Cout / 32), (unsigned)(Cin / 32), (unsigned)K), dim3(32, 8), 0, s>>>(
        W, Wt, (int)Cin, (int)Cout);
    SCN_LAUNCHED();
  }
  bool partial_pooled = false;
  if (Z > 1) SCN_TRY(splitk_scratch(&partial, (size_t)Z * tiles * kTileM * Cout, s, &partial_pooled));
  const dim3 grid((unsigned)tiles, (unsigned)Z);
  const size_t fixed_p = sizeof(CtlP) + (size_t)kMapBufs * K * kTileM * sizeof(int) + 1024;
  int st_p = (int)((220 * 1024 - fixed_p) / stage_bytes);
  if (st_p > kMaxStages) st_p = kMaxStages;
  if (cols * 2 <= 512 && st_p >= 4) {
    CUtensorMap tmB;
    if (packed) SCN_TRY(cached_tensor_map(&tmB, Wt, false, (uint64_t)Cin, (uint64_t)K * Cout, 32, (uint32_t)Cout));
    else SCN_TRY(encode_2d(&tmB, Wt, false, (uint64_t)Cin, (uint64_t)K * Cout, (uint64_t)Cin * 4, 32, (uint32_t)Cout));
    const PersistPlan plan = persist_plan(K, Cout);
    const size_t smem_p = plan.smem;
    {
      // the opt-in shared memory limit is raised once per device, to the most this kernel ever asks for
      static bool raised[64] = {false};
      int dev = 0;
      SCN_CUDA(cudaGetDevice(&dev));
      if (dev < 0 || dev >= 64 || !raised[dev]) {
        SCN_CUDA(cudaFuncSetAttribute(k_gather_gemm_tc_persist<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024));
        SCN_CUDA(cudaFuncSetAttribute(k_gather_gemm_tc_persist<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024));
        if (dev >= 0 && dev < 64) raised[dev] = true;
      }
    }
    const long long n_items = tiles * Z;
    k_gather_gemm_tc_persist<false><<<(unsigned)(n_items < sm_count ? n_items : sm_count), kPThreads, smem_p, s>>>(
        in, in_stride, tmB, map, K, n_out, bias, out, out_stride, (int)Cin, (int)Cout, init, init_stride, cols, plan.stages,
        plan.stages_b, tiles, Z, partial, EpiBn());
  } else {
#define SCN_TC_LAUNCH(S, A)                                                                                          \
  do {                                                                                                               \
    SCN_CUDA(cudaFuncSetAttribute(k_gather_gemm_tf32<S, A>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    k_gather_gemm_tf32<S, A><<<grid, kThreads, smem, s>>>(in, in_stride, map, K, n_out, Wt, bias, out, out_stride,    \
                                                           (int)Cin, (int)Cout, init, init_stride, cols, partial); \
  } while (0)
  if (stages >= 6) SCN_TC_LAUNCH(6, 3);
  else if (stages == 5) SCN_TC_LAUNCH(5, 3);
  else if (stages == 4) SCN_TC_LAUNCH(4, 2);
  else SCN_TC_LAUNCH(3, 2);
#undef SCN_TC_LAUNCH
  }
  SCN_LAUNCHED();
  if (Z > 1) {
    const long long work = n_out * (Cout / 4);
    k_splitk_reduce<<<(unsigned)((work + 255) / 256), 256, 0, s>>>(partial, Z, tiles * kTileM, n_out, (int)Cout, bias, out,
                                                                  out_stride, init, init_stride, EpiBn());
    SCN_LAUNCHED();
  }
  if (partial_pooled) dev_free(partial, s);
  dev_free(Wt_own, s);
  *handled = true;
  return SCN_OK;
}

// ---------------------------------------------------------------------------------------------
// fp16 rows through the persistent tcgen05 kernel (wide layers of the 'fp16' precision)
// ---------------------------------------------------------------------------------------------
namespace {
inline int64_t padded_planes(int64_t Cin) { return (Cin + 63) / 64 * 64; }
// which shapes the fp16 path takes (kept as it was when a ring slot held operand tile and weight box together, so that
// packed weights and the shapes the interface announces stay what they were)
inline int persist_stages(int64_t K, int64_t Cout) {
  const size_t stage_bytes = (size_t)kABytes + (size_t)Cout * 128;
  const size_t fixed_p = sizeof(CtlP) + (size_t)kMapBufs * K * kTileM * sizeof(int) + 1024;
  const int st = (int)((220 * 1024 - fixed_p) / stage_bytes);
  return st > kMaxStages ? kMaxStages : st;
}

// W [vol][n_in][n_out] fp32 -> [vol][n_out][n_in padded to a multiple of 64] fp16, zero in the padding
__global__ void k_pack_weights_tc_f16(const float *__restrict__ W, __half *__restrict__ Wp, int Cin, int Cout, int Cin_pad,
                                      long long total) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int ci = (int)(i % Cin_pad);
  const long long rest = i / Cin_pad;
  const int co = (int)(rest % Cout);
  const long long k = rest / Cout;
  Wp[i] = __float2half_rn(ci < Cin ? W[(k * Cin + ci) * Cout + co] : 0.f);
}
}  // namespace

bool tc_f16_shape(int64_t K, int64_t Cin, int64_t Cout) {
  return K >= 1 && K <= 27 && Cin >= 32 && Cin % 32 == 0 && Cout >= 32 && Cout % 32 == 0 && Cout <= 256 &&
         persist_stages(K, Cout) >= 4;
}
// the pack of a wide layer: the tcgen05 layout, followed (where the slab kernel covers the shape) by the warp-fragment
// layout that kernel reads on small grids
int64_t tc_f16_packed_size(int64_t K, int64_t Cin, int64_t Cout) {
  return K * Cout * padded_planes(Cin) + (warp_slab_f16_shape(K, Cin, Cout) ? K * Cin * Cout : 0);
}

int tc_pack_weights_f16(const float *W, int64_t K, int64_t Cin, int64_t Cout, void *packed, cudaStream_t s) {
  if (!tc_f16_shape(K, Cin, Cout)) return fail(SCN_E_INVALID, "shape cannot be packed for the fp16 tcgen05 kernel");
  if (!W || !packed) return fail(SCN_E_INVALID, "null pointer");
  const long long total = K * Cout * padded_planes(Cin);
  k_pack_weights_tc_f16<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(W, static_cast<__half *>(packed), (int)Cin, (int)Cout,
                                                                       (int)padded_planes(Cin), total);
  SCN_LAUNCHED();
  if (warp_slab_f16_shape(K, Cin, Cout)) SCN_TRY(warp_mma_pack_f16_any(W, K, Cin, Cout, static_cast<__half *>(packed) + total, s));
  return SCN_OK;
}

// rows up to which a wide fp16 layer goes to the slab kernel instead of the tcgen05 kernel (scn_set_slab_max_rows)
long long g_slab_max_rows = 8192;

int gather_gemm_tc_f16(const void *in, int64_t in_stride, const int32_t *map, int K, int64_t n_out, const void *Wp,
                       const float *bias, float *out, int64_t out_stride, int64_t Cin, int64_t Cout, const float *init,
                       int64_t init_stride, cudaStream_t s, const EpiBn *epi, const SecondRows *second) {
  EpiBn e = epi ? *epi : EpiBn();
  // The incremental form of the fused BatchNorm (residual against the saved frame's rows) lives in the epilogues of the
  // warp-level and slab kernels; where the tcgen05 kernel takes the layer, the convolution stores its fp32 result and
  // the BatchNorm kernel follows as a launch of its own.
  EpiBn later;
  const bool slab = n_out <= g_slab_max_rows && warp_slab_f16_shape(K, Cin, Cout);
  if (e.dst && e.pre_exist && !slab) {
    later = e;
    e = EpiBn();
  }
  if (e.dst && (e.stride % 8 != 0 || !aligned16(e.dst) || !aligned16(e.scale) || !aligned16(e.shift)))
    return fail(SCN_E_INVALID, "the fp16 rows of a fused BatchNorm must be 16-byte aligned with a stride that is a multiple of 8");
  if (!tc_f16_shape(K, Cin, Cout)) return fail(SCN_E_INVALID, "the fp16 tcgen05 gather-GEMM takes planes that are multiples of 32, n_out <= 224");
  if (!map && K != 1) return fail(SCN_E_INVALID, "no map given for a filter volume above 1");
  {
    // small grids: too few 128-row tiles for the persistent kernel to fill the GPU without splitting reductions; the
    // slab kernel covers them with rows/16 x n_out/32 tiles whose reductions several warps share.  Measured on the
    // levels of a 255k-voxel room (slab kernel against this kernel): 14.6k rows 96->96 37 against 29 us, 192->96 62
    // against 49; 3.5k rows 128->128 24 against 24; 2k rows 160->160 21.5 against 27; 502 rows 192->192 16 against 27;
    // 116 rows 224->224 12.5 against 31.  The line is drawn at 8192 rows.
    if (slab)
      return gather_mma_slab_f16(in, in_stride, map, K, n_out, static_cast<const __half *>(Wp) + K * Cout * padded_planes(Cin), bias,
                                 out, out_stride, Cin, Cout, init, init_stride, s, epi, second);
  }
  if (second) return fail(SCN_E_UNSUPPORTED, "the tcgen05 kernel gathers one set of rows (f16_second_rows_ok says which layers take two)");
  if (in_stride % 8 != 0 || out_stride % 4 != 0 || !aligned16(in) || !aligned16(Wp) || !aligned16(out) ||
      (bias && !aligned16(bias)) || (init && (!aligned16(init) || init_stride % 4 != 0)))
    return fail(SCN_E_INVALID, "rows must be 16-byte aligned (fp16 stride a multiple of 8, fp32 strides multiples of 4)");
  if (in_stride > (1ll << 30)) return fail(SCN_E_INVALID, "input row stride above 2^30 elements");
  const PersistPlan plan = persist_plan(K, Cout);
  uint32_t cols = 32;
  while (cols < (uint32_t)Cout) cols <<= 1;
  const long long tiles = (n_out + kTileM - 1) / kTileM;
  int sm_count = 148;
  {
    int dev = 0;
    SCN_CUDA(cudaGetDevice(&dev));
    static int cached[64] = {0};
    static bool raised[64] = {false};
    if (dev >= 0 && dev < 64) {
      if (!cached[dev]) SCN_CUDA(cudaDeviceGetAttribute(&cached[dev], cudaDevAttrMultiProcessorCount, dev));
      sm_count = cached[dev];
    }
    if (dev < 0 || dev >= 64 || !raised[dev]) {
      SCN_CUDA(cudaFuncSetAttribute(k_gather_gemm_tc_persist<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024));
      if (dev >= 0 && dev < 64) raised[dev] = true;
    }
  }
  // split-K choice as for tf32, with 64 planes per step
  const int64_t Cin_pad = padded_planes(Cin);
  const int steps_max = K * (int)(Cin_pad / 64);
  int Z = 1;
  if (tiles < 2 * sm_count && steps_max >= 4) {
    long long best = -1;
    const int zmax = steps_max / 2 < 32 ? steps_max / 2 : 32;
    for (int z = 1; z <= zmax; ++z) {
      const long long per_cta = (tiles * z + sm_count - 1) / sm_count;
      const long long cost = per_cta * ((steps_max + z - 1) / z + 3) + (z > 1 ? 2 + z / 4 : 0);
      if (best < 0 || cost < best) {
        best = cost;
        Z = z;
      }
      if (cost <= 40) break;
    }
  }
  float *partial = nullptr;
  bool partial_pooled = false;
  if (Z > 1) SCN_TRY(splitk_scratch(&partial, (size_t)Z * tiles * kTileM * Cout, s, &partial_pooled));
  CUtensorMap tmB;
  int rc = cached_tensor_map(&tmB, Wp, true, (uint64_t)Cin_pad, (uint64_t)K * Cout, 64, (uint32_t)Cout);
  if (rc != SCN_OK) {
    if (partial_pooled) dev_free(partial, s);
    return rc;
  }
  const long long n_items = tiles * Z;
  k_gather_gemm_tc_persist<true><<<(unsigned)(n_items < sm_count ? n_items : sm_count), kPThreads, plan.smem, s>>>(
      in, in_stride, tmB, map, K, n_out, bias, out, out_stride, (int)Cin, (int)Cout, init, init_stride, cols, plan.stages,
      plan.stages_b, tiles, Z, partial, Z > 1 ? EpiBn() : e);
  SCN_LAUNCHED();
  if (Z > 1) {
    const long long work = n_out * (Cout / 4);
    k_splitk_reduce<<<(unsigned)((work + 255) / 256), 256, 0, s>>>(partial, Z, tiles * kTileM, n_out, (int)Cout, bias, out,
                                                                  out_stride, init, init_stride, e);
    SCN_LAUNCHED();
  }
  if (partial_pooled) dev_free(partial, s);
  if (later.dst)
    SCN_TRY(bn_forward_f16out(out, out_stride, later.dst, later.stride, n_out, Cout, later.scale, later.shift, nullptr, nullptr, 0.f,
                              later.leak, s, later.pre_exist, later.pre_out, later.pre_out_stride, later.pre_in, later.pre_in_stride,
                              true));
  return SCN_OK;
}

// ---------------------------------------------------------------------------------------------
// 1x1 convolution that allocates nothing
// ---------------------------------------------------------------------------------------------
// The tensor-core kernels above want the weights transposed, and normally park the transposed copy in
// memory taken from the device pool for the duration of the call.  This variant parks it in a fixed
// buffer that is part of the library image instead, so the call never reaches a device allocator.
// Every GPU that loads the library carries the buffer (512 KiB) until the process exits.
constexpr size_t kNoAllocMaxWeights = 512 * 256;  // floats: n_in * n_out may not exceed this
static __device__ __align__(256) float g_noalloc_weights[kNoAllocMaxWeights];

// In host code `g_noalloc_weights` is only a handle for the runtime, not an address a kernel can use:
// the device address is looked up once per device with cudaGetSymbolAddress and cached here.
static float *g_noalloc_ptr[64] = {nullptr};
static int noalloc_scratch(float **p) {
  int dev = 0;
  SCN_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(SCN_E_INVALID, "device index out of range");
  if (!g_noalloc_ptr[dev]) {
    void *addr = nullptr;
    SCN_CUDA(cudaGetSymbolAddress(&addr, g_noalloc_weights));
    g_noalloc_ptr[dev] = static_cast<float *>(addr);
  }
  *p = g_noalloc_ptr[dev];
  return SCN_OK;
}

int nin_forward_noalloc(const float *in, int64_t in_stride, float *out, int64_t out_stride, int64_t rows,
                        const float *W, const float *bias, int64_t Cin, int64_t Cout, cudaStream_t s) {
  if (rows < 0) return fail(SCN_E_INVALID, "negative row count");
  if (rows == 0) return SCN_OK;
  if (!in || !out || !W) return fail(SCN_E_INVALID, "null feature or weight pointer");
  if (Cin <= 0 || Cout <= 0 || Cin % 32 != 0 || Cout % 32 != 0 || Cout > 256)
    return fail(SCN_E_INVALID, "the no-allocation 1x1 convolution needs n_in and n_out to be multiples of 32 and n_out <= 256");
  if ((size_t)Cin * (size_t)Cout > kNoAllocMaxWeights)
    return fail(SCN_E_CAPACITY, "n_in * n_out exceeds the fixed scratch buffer of the no-allocation 1x1 convolution (131072 weights)");
  if (in_stride % 4 != 0 || out_stride % 4 != 0 || !aligned16(in) || !aligned16(W) || !aligned16(out) ||
      (bias && !aligned16(bias)))
    return fail(SCN_E_INVALID, "pointers must be 16-byte aligned and row strides multiples of 4 elements");
  float *Wt = nullptr;
  SCN_TRY(noalloc_scratch(&Wt));
  const size_t stage_bytes = (size_t)kABytes + (size_t)Cout * 128;
  const size_t fixed = sizeof(Ctl) + (size_t)kTileM * sizeof(int) + 1024;
  int stages = 4;
  if (4 * stage_bytes + fixed > 112 * 1024) {
    stages = (int)((200 * 1024 - fixed) / stage_bytes);
    if (stages > 6) stages = 6;
  }
  const size_t smem = (size_t)stages * stage_bytes + fixed;
  uint32_t cols = 32;
  while (cols < (uint32_t)Cout) cols <<= 1;
  const long long tiles = (rows + kTileM - 1) / kTileM;
  k_transpose_weights<<<dim3((unsigned)(Cout / 32), (unsigned)(Cin / 32), 1), dim3(32, 8), 0, s>>>(W, Wt, (int)Cin, (int)Cout);
  SCN_LAUNCHED();
  const dim3 grid((unsigned)tiles, 1);
#define SCN_NA_LAUNCH(S, A)                                                                                          \
  do {                                                                                                               \
    SCN_CUDA(cudaFuncSetAttribute(k_gather_gemm_tf32<S, A>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    k_gather_gemm_tf32<S, A><<<grid, kThreads, smem, s>>>(in, in_stride, nullptr, 1, rows, Wt, bias, out, out_stride, \
                                                           (int)Cin, (int)Cout, nullptr, 0, cols, nullptr);          \
  } while (0)
  if (stages >= 6) SCN_NA_LAUNCH(6, 3);
  else if (stages == 5) SCN_NA_LAUNCH(5, 3);
  else if (stages == 4) SCN_NA_LAUNCH(4, 2);
  else SCN_NA_LAUNCH(3, 2);
#undef SCN_NA_LAUNCH
  SCN_LAUNCHED();
  return SCN_OK;
}

}  // namespace scn
