// Warp-level gather-GEMM for narrow layers (n_in, n_out in {16, 32, 64}): rows gathered straight into registers.
//
//     out[o] = init(o) + sum_k in[ map[k][o] ] * W[k]           (same contract as the other gather-GEMM kernels)
//
// With 32 or 64 planes a reduction step carries too little arithmetic to pay for staging 128-row operand tiles
// in shared memory and driving them through tcgen05 from a single thread: that pipeline spends its time on
// barriers, copies and issue overhead (measured: 850-1300 cycles per 128-row step of 4 MMAs).  Here a warp owns 16 or 32
// consecutive output rows and all output planes, keeps the accumulator in registers and works through the
// offsets that have at least one neighbour among its rows:
//   * the rows' map entries [K][rows] are staged once in a warp-private slice of shared memory (all loads of
//     the slice in flight together),
//   * for an offset, lane (g, t) (g = lane / 4, t = lane % 4) loads 16 bytes of rows g, g + 8, ... for every
//     16-plane chunk, straight from global memory through L1 (neighbouring rows of a tile share most of their
//     neighbours, so L1 catches the reuse); absent neighbours load nothing and contribute zeros,
//   * the product is formed transposed, out^T = W^T * in^T, with mma.sync.m16n8k8 (tf32): the gathered rows are
//     the 8-column operand, whose two registers per lane are (k-slot t, k-slot t + 4) of ONE row.  The reduction
//     index is permuted so that these are two adjacent floats of a 16-byte load: a load feeds two MMAs with no
//     shuffle, no shared-memory transpose and no register moves (an MMA operand must sit in consecutive
//     registers; with the rows as the 16-row operand every MMA needed four moves).  The weights are the 16-row
//     operand, packed once in fragment order, [K][n_in / 16][n_out / 16][2][lane] float4, rounded to tf32,
//   * the loads of the next offset are issued before the MMAs of the current one (two register buffers).
// No barrier inside the reduction, no scratch memory; skipping works at 16/32-row granularity instead of 128.
// fp32 inputs are consumed as tf32 (low 13 mantissa bits ignored), accumulation is fp32.
// One tile per warp; the weight fragments are read through L1 (a variant that kept them in shared memory, one
// persistent CTA per SM, measured the same: both go through the same L1 data pipe, which is the busiest unit).
#include "internal.h"
#include <cuda_fp16.h>
#include <stdlib.h>

namespace scn {

namespace {

constexpr int kWarps = 4;  // warps per block; every warp works alone
constexpr int kMaxK = 27;

// D[16 x 8] += A[16 x 8] * B[8 x 8]; here A holds weights (rows = output planes) and B gathered rows
// (columns = output rows), so that both register groups of an instruction are what one 16-byte load delivers.
__device__ __forceinline__ void mma_m16n8k8_tf32(float (&d)[4], const float4 &a, float b0, float b1) {
  asm("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(__float_as_uint(a.x)), "r"(__float_as_uint(a.y)), "r"(__float_as_uint(a.z)), "r"(__float_as_uint(a.w)),
        "r"(__float_as_uint(b0)), "r"(__float_as_uint(b1)));
}

// gathered rows of one offset: [group of 8 rows][16-plane chunk]; lane (g, t) holds planes 4t..4t+3 of row g
template <int CIN, int NTR> struct Frag {
  float4 v[NTR][CIN / 16];
};

template <int CIN, int NTR>
__device__ __forceinline__ void load_rows(Frag<CIN, NTR> &f, const int *mp_k, const float *__restrict__ in_t, long long in_stride,
                                          int g) {
#pragma unroll
  for (int n = 0; n < NTR; ++n) {
    const int s = mp_k[n * 8 + g];
    const float4 *p = reinterpret_cast<const float4 *>(in_t + (long long)s * in_stride);
#pragma unroll
    for (int c = 0; c < CIN / 16; ++c) {
      f.v[n][c] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (s >= 0) f.v[n][c] = __ldg(p + 4 * c);  // an absent neighbour costs no load
    }
  }
}

// wk: this lane's float4 of the first weight fragment of offset k
template <int CIN, int COUT, int NTR>
__device__ __forceinline__ void mma_rows(float (&acc)[COUT / 16][NTR][4], const Frag<CIN, NTR> &f, const float4 *__restrict__ wk) {
  constexpr int MTC = COUT / 16;
#pragma unroll
  for (int c = 0; c < CIN / 16; ++c) {
    float4 a[MTC][2];
#pragma unroll
    for (int m = 0; m < MTC; ++m) {
      a[m][0] = __ldg(wk + ((c * MTC + m) * 2) * 32);
      a[m][1] = __ldg(wk + ((c * MTC + m) * 2 + 1) * 32);
    }
    // consecutive MMAs go to different accumulators: the same one comes up again MTC * NTR instructions later
#pragma unroll
    for (int m = 0; m < MTC; ++m)
#pragma unroll
      for (int n = 0; n < NTR; ++n) mma_m16n8k8_tf32(acc[m][n], a[m][0], f.v[n][c].x, f.v[n][c].y);
#pragma unroll
    for (int m = 0; m < MTC; ++m)
#pragma unroll
      for (int n = 0; n < NTR; ++n) mma_m16n8k8_tf32(acc[m][n], a[m][1], f.v[n][c].z, f.v[n][c].w);
  }
}

// Map entries [K][ROWS] of a tile's rows: loaded into registers with all loads in flight together, then published
// in the warp's slice of shared memory together with the set of offsets that have any entry.
// map == nullptr: identity, K = 1.
template <int ROWS> struct MapRegs {
  static constexpr int PER = 32 / ROWS;               // offsets covered by one warp-wide load
  static constexpr int NL = (kMaxK + PER - 1) / PER;  // warp-wide loads for the largest K
  int v[NL];
};

template <int ROWS>
__device__ __forceinline__ void load_map(MapRegs<ROWS> &m, long long row0, const int32_t *__restrict__ map, int K, long long n_out,
                                         int lane) {
  constexpr int PER = MapRegs<ROWS>::PER, NL = MapRegs<ROWS>::NL;
  const int r = lane % ROWS, ksub = lane / ROWS;
  const bool row_ok = row0 + r < n_out;
  if (map) {
    const int32_t *mrow = map + row0 + r;
#pragma unroll
    for (int j = 0; j < NL; ++j) {
      const int k = j * PER + ksub;
      m.v[j] = (k < K && row_ok) ? __ldg(mrow + (long long)k * n_out) : -1;
    }
  } else {
#pragma unroll
    for (int j = 0; j < NL; ++j) m.v[j] = (j == 0 && ksub == 0 && row_ok) ? (int)(row0 + r) : -1;
  }
}

template <int ROWS>
__device__ __forceinline__ unsigned int publish_map(const MapRegs<ROWS> &m, int *mp, int K, int lane) {
  constexpr int PER = MapRegs<ROWS>::PER, NL = MapRegs<ROWS>::NL;
  const int r = lane % ROWS, ksub = lane / ROWS;
  unsigned int mask = 0;
#pragma unroll
  for (int j = 0; j < NL; ++j) {
    const int k = j * PER + ksub;
    if (k < K) mp[k * ROWS + r] = m.v[j];
    const unsigned int b = __ballot_sync(0xffffffffu, m.v[j] >= 0);
    if (PER == 2) {
      mask |= ((b & 0xffffu) ? 1u : 0u) << (j * PER);
      mask |= ((b >> 16) ? 1u : 0u) << (j * PER + 1);
    } else {
      mask |= (b ? 1u : 0u) << j;
    }
  }
  __syncwarp();
  return mask;
}

// accumulator fragment: c0,c1 -> plane 16m + g, rows 8n + 2t, +1; c2,c3 -> plane 16m + g + 8
// e (optional second output): leaky(v * scale + shift) of the finished value as fp16; plane0 = first plane of this
// call's slab inside the full row (scale, shift and the fp16 rows are indexed by full-row planes).
template <int COUT, int NTR>
__device__ __forceinline__ void store_acc(const float (&acc)[COUT / 16][NTR][4], long long row0, long long n_out,
                                          const float *__restrict__ bias, float *out, long long out_stride,
                                          const float *init, long long init_stride, int g, int t, const EpiBn &e = EpiBn(),
                                          int plane0 = 0) {
  float sc[COUT / 16][2], sh[COUT / 16][2];
  if (e.dst) {
#pragma unroll
    for (int m = 0; m < COUT / 16; ++m)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        sc[m][h] = __ldg(e.scale + plane0 + 16 * m + 8 * h + g);
        sh[m][h] = __ldg(e.shift + plane0 + 16 * m + 8 * h + g);
      }
  }
#pragma unroll
  for (int n = 0; n < NTR; ++n)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const long long row = row0 + n * 8 + 2 * t + j;
      if (row < n_out) {
        float *o = out + row * out_stride + g;
        const float *ini = init ? init + row * init_stride + g : nullptr;
        __half *hd = e.dst ? static_cast<__half *>(e.dst) + row * e.stride + plane0 + g : nullptr;
        const int pe = (hd && e.pre_exist) ? e.pre_exist[row] : -1;
        const float *xs = pe >= 0 ? e.pre_in + (long long)pe * e.pre_in_stride + plane0 + g : nullptr;
        const __half *ys = pe >= 0 ? static_cast<const __half *>(e.pre_out) + (long long)pe * e.pre_out_stride + plane0 + g : nullptr;
#pragma unroll
        for (int m = 0; m < COUT / 16; ++m)
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            float v = acc[m][n][2 * h + j];
            const int c = 16 * m + 8 * h;
            if (ini) v += ini[c];
            else if (bias) v += __ldg(bias + c + g);
            if (!e.skip_raw) o[c] = v;
            if (hd) {
              float y = fmaf(xs ? v + xs[c] : v, sc[m][h], sh[m][h]);
              y = y > 0.f ? y : y * e.leak;
              if (ys) y -= __half2float(ys[c]);
              hd[c] = __float2half_rn(fminf(fmaxf(y, -65504.f), 65504.f));
            }
          }
      }
    }
}

// One tile of 8 * NTR output rows, done by one warp.  mp: the warp's [K][ROWS] slice of shared memory, holding the
// tile's map entries; mask: the offsets that have any.
template <int CIN, int COUT, int NTR>
__device__ __forceinline__ void warp_tile(long long row0, const int *mp, unsigned int mask, const float *__restrict__ in,
                                          long long in_stride, long long n_out, const float4 *wl,
                                          const float *__restrict__ bias, float *out, long long out_stride,
                                          const float *init, long long init_stride, int lane) {
  constexpr int ROWS = 8 * NTR, MTC = COUT / 16, C16 = CIN / 16;
  const int g = lane >> 2, t = lane & 3;

  float acc[MTC][NTR][4];
#pragma unroll
  for (int m = 0; m < MTC; ++m)
#pragma unroll
    for (int n = 0; n < NTR; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[m][n][i] = 0.f;

  constexpr int WK = C16 * MTC * 2 * 32;  // float4 per offset
  const float *in_t = in + 4 * t;
  if (mask) {
    Frag<CIN, NTR> f0, f1;
    int k0 = __ffs(mask) - 1;
    mask &= mask - 1;
    load_rows<CIN, NTR>(f0, mp + k0 * ROWS, in_t, in_stride, g);
    while (true) {
      int k1 = -1;
      if (mask) {
        k1 = __ffs(mask) - 1;
        mask &= mask - 1;
        load_rows<CIN, NTR>(f1, mp + k1 * ROWS, in_t, in_stride, g);
      }
      mma_rows<CIN, COUT, NTR>(acc, f0, wl + k0 * WK);
      if (k1 < 0) break;
      k0 = -1;
      if (mask) {
        k0 = __ffs(mask) - 1;
        mask &= mask - 1;
        load_rows<CIN, NTR>(f0, mp + k0 * ROWS, in_t, in_stride, g);
      }
      mma_rows<CIN, COUT, NTR>(acc, f1, wl + k1 * WK);
      if (k0 < 0) break;
    }
  }
  store_acc<COUT, NTR>(acc, row0, n_out, bias, out, out_stride, init, init_stride, g, t);
}

// One tile per warp.  (A persistent form, warps walking over tiles and fetching the next tile's map entries
// while working on the current one, measured 10-15 % slower: the hardware's block scheduler balances the uneven
// tiles better than a fixed stride does.)
template <int CIN, int COUT, int NTR, int MINB>
__global__ void __launch_bounds__(kWarps * 32, MINB)
k_gather_mma_tf32(const float *__restrict__ in, long long in_stride, const int32_t *__restrict__ map, int K, long long n_out,
                  const float4 *__restrict__ Wp, const float *__restrict__ bias, float *out, long long out_stride,
                  const float *init, long long init_stride) {
  constexpr int ROWS = 8 * NTR;
  __shared__ int s_map[kWarps][kMaxK * ROWS];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long row0 = ((long long)blockIdx.x * kWarps + warp) * ROWS;
  if (row0 >= n_out) return;  // warps never synchronise with each other
  int *mp = s_map[warp];
  MapRegs<ROWS> regs;
  load_map<ROWS>(regs, row0, map, K, n_out, lane);
  const unsigned int mask = publish_map<ROWS>(regs, mp, K, lane);
  warp_tile<CIN, COUT, NTR>(row0, mp, mask, in, in_stride, n_out, Wp + lane, bias, out, out_stride, init, init_stride, lane);
}

// ---------------------------------------------------------------------------------------------
// fp16 form: the gathered rows are fp16 (written by the BatchNorm in front of the convolution), the weights are
// packed as fp16 fragments, mma.sync.m16n8k16, fp32 accumulation.  Same structure as above with half of
// everything per unit: a 32-plane row is 64 bytes = ONE 16-byte load per lane of the quad, which feeds two K = 16
// MMAs; lane (g, t) holds planes 8t..8t+7 of row g, the k-slots (2t, 2t+1) and (2t+8, 2t+9) of the two MMAs are
// planes 8t+4j+{0,1} and 8t+4j+{2,3} (j = 0, 1).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_m16n8k16_f16(float (&d)[4], const uint4 &a, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b0), "r"(b1));
}

template <int CIN, int NTR> struct FragH {
  uint4 v[NTR][CIN / 32];
};

template <int CIN, int NTR>
__device__ __forceinline__ void load_rows_h(FragH<CIN, NTR> &f, const int *mp_k, const __half *__restrict__ in_t, long long in_stride,
                                            int g) {
#pragma unroll
  for (int n = 0; n < NTR; ++n) {
    const int s = mp_k[n * 8 + g];
    const uint4 *p = reinterpret_cast<const uint4 *>(in_t + (long long)s * in_stride);
#pragma unroll
    for (int c = 0; c < CIN / 32; ++c) {
      f.v[n][c] = make_uint4(0u, 0u, 0u, 0u);
      if (s >= 0) f.v[n][c] = __ldg(p + 4 * c);
    }
  }
}

template <int CIN, int COUT, int NTR>
__device__ __forceinline__ void mma_rows_h(float (&acc)[COUT / 16][NTR][4], const FragH<CIN, NTR> &f, const uint4 *__restrict__ wk) {
  constexpr int MTC = COUT / 16;
#pragma unroll
  for (int c = 0; c < CIN / 32; ++c) {
    uint4 a[MTC][2];
#pragma unroll
    for (int m = 0; m < MTC; ++m) {
      a[m][0] = __ldg(wk + ((c * MTC + m) * 2) * 32);
      a[m][1] = __ldg(wk + ((c * MTC + m) * 2 + 1) * 32);
    }
#pragma unroll
    for (int m = 0; m < MTC; ++m)
#pragma unroll
      for (int n = 0; n < NTR; ++n) mma_m16n8k16_f16(acc[m][n], a[m][0], f.v[n][c].x, f.v[n][c].y);
#pragma unroll
    for (int m = 0; m < MTC; ++m)
#pragma unroll
      for (int n = 0; n < NTR; ++n) mma_m16n8k16_f16(acc[m][n], a[m][1], f.v[n][c].z, f.v[n][c].w);
  }
}

// Row ADDRESSES instead of row numbers in the warp's slice of shared memory: the address of a gathered row is formed once
// per (offset, row) when the map entries are published, not by every lane of the quad at every use, and an absent
// neighbour points at a row of zeros, so the loads of the reduction loop are unconditional (no predicate, no zeroing
// of the destination registers).  In the loop a row costs one 8-byte shared-memory read, one 64-bit add (the lane's
// 16 bytes inside the row) and the load itself.
//
// Order of the offsets: a 3x3x3 filter's offsets are visited with dx innermost (k = 9 (dx+1) + 3 (dy+1) + (dz+1) is
// visited as ..., k, k + 9, k + 18, ...).  Rows are numbered along x, so the three dx variants of a (dy, dz) pair read
// the same rows shifted by one: visited back to back the second and third find the lines the first just fetched in L1.
__device__ __align__(256) unsigned char g_zero_row[512];  // never written: zero-initialised with the module

__device__ __forceinline__ constexpr int visit_pos(int k) { return (k % 9) * 3 + k / 9; }  // position of offset k
__device__ __forceinline__ int visit_offset(int p, bool permuted) { return permuted ? (p % 3) * 9 + p / 3 : p; }

// Publishes the addresses and returns the set of occupied offsets as a mask over VISIT positions (permuted: K == 27).
template <int ROWS>
__device__ __forceinline__ unsigned int publish_addr(const MapRegs<ROWS> &m, unsigned long long *mp, int K, int lane,
                                                     const char *in_bytes, long long stride_bytes, bool permuted) {
  constexpr int PER = MapRegs<ROWS>::PER, NL = MapRegs<ROWS>::NL;
  const int r = lane % ROWS, ksub = lane / ROWS;
  const unsigned long long zero = reinterpret_cast<unsigned long long>(g_zero_row);
  const unsigned long long base = reinterpret_cast<unsigned long long>(in_bytes);
  unsigned int mask = 0;
#pragma unroll
  for (int j = 0; j < NL; ++j) {
    const int k = j * PER + ksub;
    if (k < K) mp[k * ROWS + r] = m.v[j] >= 0 ? base + (unsigned long long)((long long)m.v[j] * stride_bytes) : zero;
    const unsigned int b = __ballot_sync(0xffffffffu, m.v[j] >= 0);
    if (PER == 2) {
      const int ka = j * PER, kb = j * PER + 1;
      mask |= ((b & 0xffffu) ? 1u : 0u) << (permuted ? visit_pos(ka) : ka);
      if (kb < kMaxK) mask |= ((b >> 16) ? 1u : 0u) << (permuted ? visit_pos(kb) : kb);
    } else {
      mask |= (b ? 1u : 0u) << (permuted ? visit_pos(j) : j);
    }
  }
  __syncwarp();
  return mask;
}

template <int CIN, int NTR>
__device__ __forceinline__ void load_rows_a(FragH<CIN, NTR> &f, const unsigned long long *mp_k, int g, int lane_bytes) {
#pragma unroll
  for (int n = 0; n < NTR; ++n) {
    const uint4 *p = reinterpret_cast<const uint4 *>(mp_k[n * 8 + g] + (unsigned long long)lane_bytes);
#pragma unroll
    for (int c = 0; c < CIN / 32; ++c) f.v[n][c] = __ldg(p + 4 * c);
  }
}

// Epilogue of a 32-plane pass through the warp's slice of shared memory: the accumulator fragments hold single floats
// of rows 2t, 2t + 1 (a lane would store 4 bytes at a time, 16 * NTR stores and as many again for the fp16 rows); staged
// with a pitch of 36 floats (conflict-free both ways) a lane reads 4 consecutive planes of a row and every store is
// 16 bytes (8 for the fp16 rows).  Needs 16-byte aligned rows (vec); otherwise the element-wise form is used.
template <int NTR>
__device__ __forceinline__ void store_pass(const float (&a0)[NTR][4], const float (&a1)[NTR][4], float *st, long long row0,
                                           long long n_out, const float *__restrict__ bias, float *out, long long out_stride,
                                           const float *init, long long init_stride, int lane, const EpiBn &e, int plane0) {
  constexpr int ROWS = 8 * NTR, PITCH = 36;
  const int g = lane >> 2, t = lane & 3;
  __syncwarp();
#pragma unroll
  for (int n = 0; n < NTR; ++n)
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        st[(8 * n + 2 * t + j) * PITCH + 8 * h + g] = a0[n][2 * h + j];
        st[(8 * n + 2 * t + j) * PITCH + 16 + 8 * h + g] = a1[n][2 * h + j];
      }
  __syncwarp();
  const int q = lane & 7, r0 = lane >> 3;
  float4 b4 = make_float4(0.f, 0.f, 0.f, 0.f), sc = b4, sh = b4;
  if (!init && bias) b4 = __ldg(reinterpret_cast<const float4 *>(bias) + q);
  if (e.dst) {
    sc = __ldg(reinterpret_cast<const float4 *>(e.scale + plane0) + q);
    sh = __ldg(reinterpret_cast<const float4 *>(e.shift + plane0) + q);
  }
#pragma unroll
  for (int i = 0; i < ROWS / 4; ++i) {
    const int r = 4 * i + r0;
    const long long row = row0 + r;
    if (row < n_out) {
      float4 v = *reinterpret_cast<const float4 *>(st + r * PITCH + 4 * q);
      if (init) {
        const float4 a = *reinterpret_cast<const float4 *>(init + row * init_stride + 4 * q);
        v.x += a.x, v.y += a.y, v.z += a.z, v.w += a.w;
      } else {
        v.x += b4.x, v.y += b4.y, v.z += b4.z, v.w += b4.w;
      }
      if (!e.skip_raw) *reinterpret_cast<float4 *>(out + row * out_stride + 4 * q) = v;
      if (e.dst) {
        float4 x = v, ysv = make_float4(0.f, 0.f, 0.f, 0.f);
        const int pe = e.pre_exist ? e.pre_exist[row] : -1;
        if (pe >= 0) {  // incremental form: add the saved input, subtract the saved activation
          const float4 a = *reinterpret_cast<const float4 *>(e.pre_in + (long long)pe * e.pre_in_stride + plane0 + 4 * q);
          x.x += a.x, x.y += a.y, x.z += a.z, x.w += a.w;
          const uint2 hq = *reinterpret_cast<const uint2 *>(static_cast<const __half *>(e.pre_out) + (long long)pe * e.pre_out_stride +
                                                            plane0 + 4 * q);
          const float2 f0 = __half22float2(*reinterpret_cast<const __half2 *>(&hq.x));
          const float2 f1 = __half22float2(*reinterpret_cast<const __half2 *>(&hq.y));
          ysv = make_float4(f0.x, f0.y, f1.x, f1.y);
        }
        float y0 = fmaf(x.x, sc.x, sh.x), y1 = fmaf(x.y, sc.y, sh.y), y2 = fmaf(x.z, sc.z, sh.z), y3 = fmaf(x.w, sc.w, sh.w);
        y0 = y0 > 0.f ? y0 : y0 * e.leak, y1 = y1 > 0.f ? y1 : y1 * e.leak;
        y2 = y2 > 0.f ? y2 : y2 * e.leak, y3 = y3 > 0.f ? y3 : y3 * e.leak;
        y0 -= ysv.x, y1 -= ysv.y, y2 -= ysv.z, y3 -= ysv.w;
        const __half2 lo = __floats2half2_rn(fminf(fmaxf(y0, -65504.f), 65504.f), fminf(fmaxf(y1, -65504.f), 65504.f));
        const __half2 hi = __floats2half2_rn(fminf(fmaxf(y2, -65504.f), 65504.f), fminf(fmaxf(y3, -65504.f), 65504.f));
        uint2 pk;
        pk.x = *reinterpret_cast<const unsigned int *>(&lo);
        pk.y = *reinterpret_cast<const unsigned int *>(&hi);
        *reinterpret_cast<uint2 *>(static_cast<__half *>(e.dst) + row * e.stride + plane0 + 4 * q) = pk;
      }
    }
  }
}

// true when store_pass may be used: 16-byte aligned fp32 rows, 8-byte aligned fp16 rows
__host__ __device__ __forceinline__ bool rows_vectorisable(const float *out, long long out_stride, const float *init,
                                                           long long init_stride, const float *bias, const EpiBn &e) {
  auto al = [](const void *p, unsigned a) { return (reinterpret_cast<unsigned long long>(p) & (a - 1)) == 0; };
  return al(out, 16) && out_stride % 4 == 0 && (!init || (al(init, 16) && init_stride % 4 == 0)) && (!bias || al(bias, 16)) &&
         (!e.dst || (al(e.dst, 8) && e.stride % 4 == 0 && al(e.scale, 16) && al(e.shift, 16))) &&
         (!e.pre_exist || (al(e.pre_in, 16) && e.pre_in_stride % 4 == 0 && al(e.pre_out, 8) && e.pre_out_stride % 4 == 0));
}

// TWO: a second set of gathered rows (SecondRows) follows the first through the same accumulators: the warp's slice of
// shared memory is refilled with the second map's addresses once the first reduction is done.
template <int CIN, int COUT, int NTR, int MINB, bool TWO>
__global__ void __launch_bounds__(kWarps * 32, MINB)
k_gather_mma_f16(const __half *__restrict__ in, long long in_stride, const int32_t *__restrict__ map, int K, long long n_out,
                 const uint4 *__restrict__ Wp, const float *__restrict__ bias, float *out, long long out_stride,
                 const float *init, long long init_stride, const EpiBn epi, const int vec, const SecondRows second) {
  constexpr int ROWS = 8 * NTR, MTC = COUT / 16;
  static_assert(kMaxK * ROWS * 8 >= ROWS * 36 * 4, "the epilogue stages a 32-plane pass in the warp's map slice");
  __shared__ unsigned long long s_map[kWarps][kMaxK * ROWS];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const long long row0 = ((long long)blockIdx.x * kWarps + warp) * ROWS;
  if (row0 >= n_out) return;
  unsigned long long *mp = s_map[warp];
  const bool perm = K == 27;
  float acc[MTC][NTR][4];
#pragma unroll
  for (int m = 0; m < MTC; ++m)
#pragma unroll
    for (int n = 0; n < NTR; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[m][n][i] = 0.f;
  constexpr int WK = (CIN / 32) * MTC * 2 * 32;  // uint4 per offset
  const uint4 *wl = Wp + lane;
#pragma unroll 1
  for (int src = 0; src < (TWO ? 2 : 1); ++src) {
  if (TWO && src == 1) __syncwarp();  // every lane has read the first map's addresses
  MapRegs<ROWS> regs;
  load_map<ROWS>(regs, row0, (TWO && src == 1) ? second.map : map, K, n_out, lane);
  unsigned int mask = publish_addr<ROWS>(regs, mp, K, lane,
                                         (TWO && src == 1) ? static_cast<const char *>(second.in) : reinterpret_cast<const char *>(in),
                                         ((TWO && src == 1) ? second.stride : in_stride) * 2, perm);
  if (mask) {
    FragH<CIN, NTR> f0, f1;
    int k0 = visit_offset(__ffs(mask) - 1, perm);
    mask &= mask - 1;
    load_rows_a<CIN, NTR>(f0, mp + k0 * ROWS, g, 16 * t);
    while (true) {
      int k1 = -1;
      if (mask) {
        k1 = visit_offset(__ffs(mask) - 1, perm);
        mask &= mask - 1;
        load_rows_a<CIN, NTR>(f1, mp + k1 * ROWS, g, 16 * t);
      }
      mma_rows_h<CIN, COUT, NTR>(acc, f0, wl + k0 * WK);
      if (k1 < 0) break;
      k0 = -1;
      if (mask) {
        k0 = visit_offset(__ffs(mask) - 1, perm);
        mask &= mask - 1;
        load_rows_a<CIN, NTR>(f0, mp + k0 * ROWS, g, 16 * t);
      }
      mma_rows_h<CIN, COUT, NTR>(acc, f1, wl + k1 * WK);
      if (k0 < 0) break;
    }
  }
  }
  if (TWO) __syncwarp();  // the slice becomes the epilogue's staging area
  if (vec) {
    float *st = reinterpret_cast<float *>(mp);
#pragma unroll
    for (int pass = 0; pass < MTC / 2; ++pass)
      store_pass<NTR>(acc[2 * pass], acc[2 * pass + 1], st, row0, n_out, bias ? bias + 32 * pass : nullptr, out + 32 * pass,
                      out_stride, init ? init + 32 * pass : nullptr, init_stride, lane, epi, 32 * pass);
  } else {
    store_acc<COUT, NTR>(acc, row0, n_out, bias, out, out_stride, init, init_stride, g, t, epi);
  }
}

// Wide layers on small grids (the deep levels of a UNet: a hundred to sixteen thousand rows, 96-224 planes).  There
// the tcgen05 kernel has too few 128-row tiles to fill the GPU, shares a tile's reduction among work items and needs a
// second launch to add the partial tiles.  Here a tile is 16 rows x a slab of 32 output planes (blockIdx.y), its
// reduction over the occupied offsets is run by KS warps (1, 2, 4 or 8: every KS-th occupied offset each), and the
// layer is one launch of rows/16 x n_out/32 x KS warps.  With one warp per tile a layer takes as long as its chain
// of 27 dependent gathers (0.4-0.5 us each: 20-30 us whatever the size) while most of the GPU idles; the launcher
// picks KS so that the GPU is covered.  The partial accumulators of warps 1 .. KS-1 are parked in shared memory and
// added by warp 0 in a fixed order (deterministic), which then runs the epilogue.
//
// Registers decide how many warps fit, so the gathered rows have ONE buffer (16 rows x n_in: 8 registers per 32 planes):
// as soon as the MMAs of a 32-plane chunk have been issued, the chunk's registers are reloaded with the same chunk of the
// warp's next offset, which then has the rest of this offset's MMAs to arrive.  The weight fragments of the next chunk
// are fetched while the MMAs of the current one are issued (two buffers of 16 registers).
constexpr int kSlabWarps = 8;

template <int C32> struct SlabRows {
  uint4 v[2][C32];
};

// chunk c of the rows at `mp_k` (16 addresses): lane (g, t) takes 16 bytes of rows g and g + 8
template <int C32>
__device__ __forceinline__ void slab_load_chunk(SlabRows<C32> &f, const unsigned long long *mp_k, int g, int lane_bytes, int c) {
#pragma unroll
  for (int n = 0; n < 2; ++n)
    f.v[n][c] = __ldg(reinterpret_cast<const uint4 *>(mp_k[n * 8 + g] + (unsigned long long)(lane_bytes + 64 * c)));
}

__device__ __forceinline__ void slab_load_w(uint4 (&a)[2][2], const uint4 *__restrict__ wk, int c, int mtc_total) {
#pragma unroll
  for (int m = 0; m < 2; ++m) {
    a[m][0] = __ldg(wk + ((c * mtc_total + m) * 2) * 32);
    a[m][1] = __ldg(wk + ((c * mtc_total + m) * 2 + 1) * 32);
  }
}

// One offset: MMAs of all chunks; after a chunk's MMAs its row registers are refilled from the next offset (mp_next,
// null at the end) and the weight fragments of the following chunk (of this offset, or chunk 0 of the next: wk_next)
// are already on their way.  P0: which weight buffer holds chunk 0 (alternates from offset to offset when C32 is odd).
template <int C32, int P0>
__device__ __forceinline__ void slab_offset(float (&acc)[2][2][4], SlabRows<C32> &f, uint4 (&a)[2][2][2], const uint4 *__restrict__ wk,
                                            const uint4 *__restrict__ wk_next, const unsigned long long *mp_next, int mtc_total,
                                            int g, int lane_bytes) {
#pragma unroll
  for (int c = 0; c < C32; ++c) {
    const int cur = (P0 + c) & 1, nxt = cur ^ 1;
    if (c + 1 < C32) slab_load_w(a[nxt], wk, c + 1, mtc_total);
    else if (wk_next) slab_load_w(a[nxt], wk_next, 0, mtc_total);
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
      for (int n = 0; n < 2; ++n) mma_m16n8k16_f16(acc[m][n], a[cur][m][0], f.v[n][c].x, f.v[n][c].y);
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
      for (int n = 0; n < 2; ++n) mma_m16n8k16_f16(acc[m][n], a[cur][m][1], f.v[n][c].z, f.v[n][c].w);
    if (mp_next) slab_load_chunk<C32>(f, mp_next, g, lane_bytes, c);
  }
}

template <int C32, int KS, bool TWO>
__global__ void __launch_bounds__(kSlabWarps * 32, 2)
k_gather_mma_f16_slab(const __half *__restrict__ in, long long in_stride, const int32_t *__restrict__ map, int K, long long n_out,
                      const uint4 *__restrict__ Wp, int Cout, const float *__restrict__ bias, float *out, long long out_stride,
                      const float *init, long long init_stride, const EpiBn epi, const int vec, const SecondRows second) {
  constexpr int ROWS = 16, TILES = kSlabWarps / KS;
  __shared__ unsigned long long s_map[kSlabWarps][kMaxK * ROWS];
  __shared__ float s_part[KS > 1 ? kSlabWarps : 1][16][32];  // [warp][accumulator element][lane]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int tile_local = warp / KS, split = warp % KS;
  const long long row0 = ((long long)blockIdx.x * TILES + tile_local) * ROWS;
  const bool live = row0 < n_out;
  if (KS == 1 && !live) return;  // with one warp per tile the warps never meet
  const int slab = blockIdx.y, mtc_total = Cout >> 4;
  unsigned long long *mp = s_map[warp];
  float acc[2][2][4];
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[m][n][i] = 0.f;
  if (live) {
    const bool perm = K == 27;
#pragma unroll 1
    for (int src = 0; src < (TWO ? 2 : 1); ++src) {  // TWO: the second set of rows follows through the same accumulators
    if (TWO && src == 1) __syncwarp();  // every lane has read the first map's addresses
    MapRegs<ROWS> regs;
    load_map<ROWS>(regs, row0, (TWO && src == 1) ? second.map : map, K, n_out, lane);
    const unsigned int all = publish_addr<ROWS>(
        regs, mp, K, lane, (TWO && src == 1) ? static_cast<const char *>(second.in) : reinterpret_cast<const char *>(in),
        ((TWO && src == 1) ? second.stride : in_stride) * 2, perm);
    unsigned int mask = all;
    if (KS > 1) {  // this warp's share: every KS-th occupied offset, counted from its own index
      mask = 0;
      int ord = 0;
      for (unsigned int m = all; m; m &= m - 1, ++ord)
        if (ord % KS == split) mask |= m & (0u - m);
    }
    const long long WK = (long long)C32 * mtc_total * 2 * 32;  // uint4 per offset
    const uint4 *wl = Wp + lane + (2 * slab) * 2 * 32;  // this slab's two 16-plane tiles inside a 32-plane block's fragments
    if (mask) {
      SlabRows<C32> f;
      uint4 a[2][2][2];
      int k = visit_offset(__ffs(mask) - 1, perm);
      mask &= mask - 1;
      const uint4 *wk = wl + k * WK;
      slab_load_w(a[0], wk, 0, mtc_total);
#pragma unroll
      for (int c = 0; c < C32; ++c) slab_load_chunk<C32>(f, mp + k * ROWS, g, 16 * t, c);
      while (true) {
        int kn = mask ? visit_offset(__ffs(mask) - 1, perm) : -1;
        mask &= mask - 1;
        slab_offset<C32, 0>(acc, f, a, wk, kn >= 0 ? wl + kn * WK : nullptr, kn >= 0 ? mp + kn * ROWS : nullptr, mtc_total, g, 16 * t);
        if (kn < 0) break;
        wk = wl + kn * WK;
        kn = mask ? visit_offset(__ffs(mask) - 1, perm) : -1;
        mask &= mask - 1;
        slab_offset<C32, (C32 & 1)>(acc, f, a, wk, kn >= 0 ? wl + kn * WK : nullptr, kn >= 0 ? mp + kn * ROWS : nullptr, mtc_total, g,
                                    16 * t);
        if (kn < 0) break;
        wk = wl + kn * WK;
      }
    }
    }
    if (TWO) __syncwarp();  // the slice becomes the epilogue's staging area
    if (KS > 1 && split != 0) {
#pragma unroll
      for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
          for (int i = 0; i < 4; ++i) s_part[warp][(m * 2 + n) * 4 + i][lane] = acc[m][n][i];
    }
  }
  if (KS > 1) {
    __syncthreads();
    if (!live || split != 0) return;
#pragma unroll 1
    for (int o = 1; o < KS; ++o)
#pragma unroll
      for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[m][n][i] += s_part[warp + o][(m * 2 + n) * 4 + i][lane];
  }
  if (vec)
    store_pass<2>(acc[0], acc[1], reinterpret_cast<float *>(mp), row0, n_out, bias ? bias + 32 * slab : nullptr, out + 32 * slab,
                  out_stride, init ? init + 32 * slab : nullptr, init_stride, lane, epi, 32 * slab);
  else
    store_acc<32, 2>(acc, row0, n_out, bias ? bias + 32 * slab : nullptr, out + 32 * slab, out_stride,
                     init ? init + 32 * slab : nullptr, init_stride, g, t, epi, 32 * slab);
}

// W [K][n_in][n_out] fp32 -> fp16 fragments [K][n_in/32][n_out/16][2][lane][8]: half e of (k, c, m, j, lane = 4g + t)
// is W[k][32c + 8t + 4j + 2(e >> 2) + (e & 1)][16m + g + 8((e >> 1) & 1)]
__global__ void k_pack_weights_f16(const float *__restrict__ W, __half *__restrict__ Wp, int Cin, int Cout, long long total) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int MTC = Cout / 16, C32 = Cin / 32;
  const int e = (int)(i & 7), lane = (int)((i >> 3) & 31), j = (int)((i >> 8) & 1);
  long long rest = i >> 9;
  const int m = (int)(rest % MTC);
  rest /= MTC;
  const int c = (int)(rest % C32);
  const long long k = rest / C32;
  const int g = lane >> 2, t = lane & 3;
  const int r = e >> 1, h = e & 1;  // register a0..a3 of the fragment, half inside it
  const int ci = 32 * c + 8 * t + 4 * j + 2 * (r >> 1) + h, co = 16 * m + g + 8 * (r & 1);
  Wp[i] = __float2half_rn(W[(k * Cin + ci) * Cout + co]);
}

// Layers with 1 to 4 input planes (the first layer of a network: colours, a constant one): the planes of a
// row fill k-slots 0..3 of one MMA, the other slots are zero, so an offset costs n_out / 16 MMAs per 8 rows and
// a 4-byte load per row.  The weights are read as they are (no packing), the hardware ignores their low
// mantissa bits.
template <int COUT, int NTR>
__global__ void __launch_bounds__(kWarps * 32)
k_gather_mma_tf32_small(const float *__restrict__ in, long long in_stride, const int32_t *__restrict__ map, int K, long long n_out,
                        const float *__restrict__ W, const float *__restrict__ bias, float *out, long long out_stride,
                        int Cin, const float *init, long long init_stride) {
  constexpr int ROWS = 8 * NTR, MTC = COUT / 16;
  __shared__ int s_map[kWarps][kMaxK * ROWS];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const long long row0 = ((long long)blockIdx.x * kWarps + warp) * ROWS;
  if (row0 >= n_out) return;
  int *mp = s_map[warp];
  MapRegs<ROWS> regs;
  load_map<ROWS>(regs, row0, map, K, n_out, lane);
  unsigned int mask = publish_map<ROWS>(regs, mp, K, lane);
  float acc[MTC][NTR][4];
#pragma unroll
  for (int m = 0; m < MTC; ++m)
#pragma unroll
    for (int n = 0; n < NTR; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[m][n][i] = 0.f;
  const bool plane_ok = t < Cin;
  while (mask) {
    const int k = __ffs(mask) - 1;
    mask &= mask - 1;
    float b[NTR];
#pragma unroll
    for (int n = 0; n < NTR; ++n) {
      const int s = mp[k * ROWS + n * 8 + g];
      b[n] = (s >= 0 && plane_ok) ? __ldg(in + (long long)s * in_stride + t) : 0.f;
    }
    const float *wk = W + ((long long)k * Cin + t) * COUT + g;
#pragma unroll
    for (int m = 0; m < MTC; ++m) {
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f);  // (plane t -> 16m + g, plane t -> 16m + g + 8, slots t + 4: unused)
      if (plane_ok) {
        a.x = __ldg(wk + 16 * m);
        a.y = __ldg(wk + 16 * m + 8);
      }
#pragma unroll
      for (int n = 0; n < NTR; ++n) mma_m16n8k8_tf32(acc[m][n], a, b[n], 0.f);
    }
  }
  store_acc<COUT, NTR>(acc, row0, n_out, bias, out, out_stride, init, init_stride, g, t);
}

// W [K][n_in][n_out] -> [K][n_in/16][n_out/16][2][lane][4], rounded to tf32 (round to nearest, ties away):
// element e of the float4 of (k, c, m, j, lane = 4g + t) is W[k][16c + 4t + 2j + (e >> 1)][16m + g + 8(e & 1)]
__global__ void k_pack_weights_mma(const float *__restrict__ W, float *__restrict__ Wp, int Cin, int Cout, long long total) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int MTC = Cout / 16, C16 = Cin / 16;
  const int e = (int)(i & 3), lane = (int)((i >> 2) & 31), j = (int)((i >> 7) & 1);
  long long rest = i >> 8;
  const int m = (int)(rest % MTC);
  rest /= MTC;
  const int c = (int)(rest % C16);
  const long long k = rest / C16;
  const int g = lane >> 2, t = lane & 3;
  const int ci = c * 16 + 4 * t + 2 * j + (e >> 1), co = m * 16 + g + 8 * (e & 1);
  const float w = W[(k * Cin + ci) * Cout + co];
  uint32_t u;
  asm("cvt.rna.tf32.f32 %0, %1;\n" : "=r"(u) : "f"(w));
  Wp[i] = __uint_as_float(u);
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

constexpr int max_planes() { return 64; }  // widest layer the warp-level kernels take
template <int CI, int CO, int NTR, int MINB>
void launch_warp(const float *in, int64_t in_stride, const int32_t *map, int K, int64_t n_out, const float *Wp,
                 const float *bias, float *out, int64_t out_stride, const float *init, int64_t init_stride, cudaStream_t s) {
  const long long tiles = (n_out + 8 * NTR - 1) / (8 * NTR);
  k_gather_mma_tf32<CI, CO, NTR, MINB><<<(unsigned)((tiles + kWarps - 1) / kWarps), kWarps * 32, 0, s>>>(
      in, in_stride, map, K, n_out, reinterpret_cast<const float4 *>(Wp), bias, out, out_stride, init, init_stride);
}

}  // namespace

// Decided by the shape alone, so that weights packed once stay valid for every call with that shape.
bool warp_mma_shape(int64_t K, int64_t Cin, int64_t Cout) {
  const int m = max_planes();
  if (K < 1 || K > kMaxK || Cin > m || Cout > m) return false;
  return (Cin == 16 || Cin == 32 || Cin == 64) && (Cout == 16 || Cout == 32 || Cout == 64);
}

int warp_mma_pack(const float *W, int64_t K, int64_t Cin, int64_t Cout, float *packed, cudaStream_t s) {
  const long long total = K * Cin * Cout;
  k_pack_weights_mma<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(W, packed, (int)Cin, (int)Cout, total);
  SCN_LAUNCHED();
  return SCN_OK;
}

int gather_mma_warp(const float *in, int64_t in_stride, const int32_t *map, int K, int64_t n_out, const float *W,
                    const float *bias, float *out, int64_t out_stride, int64_t Cin, int64_t Cout, const float *init,
                    int64_t init_stride, bool packed, cudaStream_t s, bool *handled) {
  *handled = false;
  if (!map && K != 1) return SCN_OK;
  if (!packed && Cin >= 1 && Cin <= 4 && K <= kMaxK && max_planes() > 0 && (Cout == 16 || Cout == 32 || Cout == 64)) {
    const long long tiles = (n_out + 31) / 32;
    const unsigned blocks = (unsigned)((tiles + kWarps - 1) / kWarps);
    if (Cout == 16)
      k_gather_mma_tf32_small<16, 4><<<blocks, kWarps * 32, 0, s>>>(in, in_stride, map, K, n_out, W, bias, out, out_stride,
                                                                   (int)Cin, init, init_stride);
    else if (Cout == 32)
      k_gather_mma_tf32_small<32, 4><<<blocks, kWarps * 32, 0, s>>>(in, in_stride, map, K, n_out, W, bias, out, out_stride,
                                                                   (int)Cin, init, init_stride);
    else
      k_gather_mma_tf32_small<64, 4><<<blocks, kWarps * 32, 0, s>>>(in, in_stride, map, K, n_out, W, bias, out, out_stride,
                                                                   (int)Cin, init, init_stride);
    SCN_LAUNCHED();
    *handled = true;
    return SCN_OK;
  }
  if (!warp_mma_shape(K, Cin, Cout)) return SCN_OK;
  if (in_stride % 4 != 0 || out_stride % 2 != 0 || !aligned16(in) || !aligned16(W) || !aligned16(out)) return SCN_OK;
  float *own = nullptr;
  const float *Wp = W;
  if (!packed) {
    SCN_TRY(dev_alloc_t(&own, (size_t)K * Cin * Cout, s));
    SCN_TRY(warp_mma_pack(W, K, Cin, Cout, own, s));
    Wp = own;
  }
#define SCN_WARP_LAUNCH(CI, CO, NTR, MINB) \
  launch_warp<CI, CO, NTR, MINB>(in, in_stride, map, K, n_out, Wp, bias, out, out_stride, init, init_stride, s)
  const int key = (int)Cin * 100 + (int)Cout;
  switch (key) {
    case 1616: SCN_WARP_LAUNCH(16, 16, 4, 4); break;
    case 1632: SCN_WARP_LAUNCH(16, 32, 4, 4); break;
    case 1664: SCN_WARP_LAUNCH(16, 64, 2, 4); break;
    case 3216: SCN_WARP_LAUNCH(32, 16, 4, 4); break;
    case 3232: SCN_WARP_LAUNCH(32, 32, 4, 4); break;
    case 3264: SCN_WARP_LAUNCH(32, 64, 2, 4); break;
    case 6416: SCN_WARP_LAUNCH(64, 16, 2, 4); break;
    case 6432: SCN_WARP_LAUNCH(64, 32, 2, 4); break;
    case 6464: SCN_WARP_LAUNCH(64, 64, 2, 3); break;
    default: dev_free(own, s); return SCN_OK;
  }
#undef SCN_WARP_LAUNCH
  dev_free(own, s);
  SCN_LAUNCHED();
  *handled = true;
  return SCN_OK;
}

static bool f16_shape(int64_t K, int64_t Cin, int64_t Cout) {
  return K >= 1 && K <= kMaxK && (Cin == 32 || Cin == 64) && (Cout == 32 || Cout == 64);
}
bool warp_mma_f16_shape(int64_t K, int64_t Cin, int64_t Cout) { return f16_shape(K, Cin, Cout); }

int warp_mma_pack_f16(const float *W, int64_t K, int64_t Cin, int64_t Cout, void *packed, cudaStream_t s) {
  if (!f16_shape(K, Cin, Cout)) return fail(SCN_E_INVALID, "shape cannot be packed for the fp16 kernel (planes 32 or 64)");
  if (!W || !packed) return fail(SCN_E_INVALID, "null pointer");
  const long long total = K * Cin * Cout;
  k_pack_weights_f16<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(W, static_cast<__half *>(packed), (int)Cin, (int)Cout, total);
  SCN_LAUNCHED();
  return SCN_OK;
}

// warp-fragment pack for any n_in multiple of 32 and n_out multiple of 32 (the slab kernel's weights)
int warp_mma_pack_f16_any(const float *W, int64_t K, int64_t Cin, int64_t Cout, void *packed, cudaStream_t s) {
  const long long total = K * Cin * Cout;
  k_pack_weights_f16<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(W, static_cast<__half *>(packed), (int)Cin, (int)Cout, total);
  SCN_LAUNCHED();
  return SCN_OK;
}

bool f16_second_rows_ok(int64_t K, int64_t Cin, int64_t Cout, int64_t n_out) {
  return K > 1 && (warp_mma_f16_shape(K, Cin, Cout) || (n_out <= g_slab_max_rows && warp_slab_f16_shape(K, Cin, Cout)));
}

bool warp_slab_f16_shape(int64_t K, int64_t Cin, int64_t Cout) {
  return K >= 1 && K <= kMaxK && Cin % 32 == 0 && Cin >= 96 && Cin <= 224 && Cout % 32 == 0 && Cout >= 32 && Cout <= 256;
}

// 0: the launcher chooses how many warps share a tile's reduction; 1, 2, 4, 8: fixed (scn_set_slab_share, a tuning aid)
int g_slab_share = 0;

static int check_second(const SecondRows *second, int K) {
  if (!second) return SCN_OK;
  if (!second->in || !second->map || K == 1) return fail(SCN_E_INVALID, "a second set of rows needs rows, a map and a filter volume above 1");
  if (second->stride % 8 != 0 || !aligned16(second->in))
    return fail(SCN_E_INVALID, "fp16 rows must be 16-byte aligned with a stride that is a multiple of 8 elements");
  return SCN_OK;
}

int gather_mma_slab_f16(const void *in, int64_t in_stride, const int32_t *map, int K, int64_t n_out, const void *Wp,
                        const float *bias, float *out, int64_t out_stride, int64_t Cin, int64_t Cout, const float *init,
                        int64_t init_stride, cudaStream_t s, const EpiBn *epi, const SecondRows *second) {
  const EpiBn e = epi ? *epi : EpiBn();
  if (!warp_slab_f16_shape(K, Cin, Cout)) return fail(SCN_E_INVALID, "shape not covered by the slab kernel");
  if (in_stride % 8 != 0 || !aligned16(in) || !aligned16(Wp))
    return fail(SCN_E_INVALID, "fp16 rows must be 16-byte aligned with a stride that is a multiple of 8 elements");
  SCN_TRY(check_second(second, K));
  const SecondRows two = second ? *second : SecondRows();
  const __half *inh = static_cast<const __half *>(in);
  const uint4 *W4 = static_cast<const uint4 *>(Wp);
  const long long tiles = (n_out + 15) / 16;
  const int vec = rows_vectorisable(out, out_stride, init, init_stride, bias, e) ? 1 : 0;
  // Warps that share a tile's reduction, from the number of tiles x slabs (warps when nothing is shared).  Measured on
  // the levels of a 255k-voxel room (us per layer with 1 / 2 / 4 / 8 warps): 14.6k rows 96->96 39 / 35 / 39 / 55,
  // 192->96 70 / 59 / 59 / 75; 3.5k rows 128->128 23 / 23 / 23 / 25; 2k rows 160->160 28 / 25 / 21 / 23;
  // 502 rows 192->192 33 / 23 / 14 / 14; 116 rows 224->224 35 / 23 / 16 / 12.
  const long long slabs = Cout / 32, lone = tiles * slabs;
  int ks = g_slab_share;
  if (ks != 1 && ks != 2 && ks != 4 && ks != 8) ks = lone >= 4000 ? 1 : lone >= 1000 ? 2 : lone >= 150 ? 4 : 8;
  const int tiles_per_block = kSlabWarps / ks;
  const dim3 grid((unsigned)((tiles + tiles_per_block - 1) / tiles_per_block), (unsigned)slabs);
#define SCN_SLAB_LAUNCH(C32, KS)                                                                                                    \
  do {                                                                                                                             \
    if (second)                                                                                                                    \
      k_gather_mma_f16_slab<C32, KS, true><<<grid, kSlabWarps * 32, 0, s>>>(inh, in_stride, map, K, n_out, W4, (int)Cout, bias, out, \
                                                                            out_stride, init, init_stride, e, vec, two);            \
    else                                                                                                                           \
      k_gather_mma_f16_slab<C32, KS, false><<<grid, kSlabWarps * 32, 0, s>>>(inh, in_stride, map, K, n_out, W4, (int)Cout, bias,    \
                                                                             out, out_stride, init, init_stride, e, vec, two);     \
  } while (0)
#define SCN_SLAB_KS(C32)                        \
  switch (ks) {                                 \
    case 1: SCN_SLAB_LAUNCH(C32, 1); break;     \
    case 2: SCN_SLAB_LAUNCH(C32, 2); break;     \
    case 4: SCN_SLAB_LAUNCH(C32, 4); break;     \
    default: SCN_SLAB_LAUNCH(C32, 8); break;    \
  }
  switch ((int)(Cin / 32)) {
    case 3: SCN_SLAB_KS(3); break;
    case 4: SCN_SLAB_KS(4); break;
    case 5: SCN_SLAB_KS(5); break;
    case 6: SCN_SLAB_KS(6); break;
    default: SCN_SLAB_KS(7); break;
  }
#undef SCN_SLAB_KS
#undef SCN_SLAB_LAUNCH
  SCN_LAUNCHED();
  return SCN_OK;
}

int gather_mma_warp_f16(const void *in, int64_t in_stride, const int32_t *map, int K, int64_t n_out, const void *Wp,
                        const float *bias, float *out, int64_t out_stride, int64_t Cin, int64_t Cout, const float *init,
                        int64_t init_stride, cudaStream_t s, const EpiBn *epi, const SecondRows *second) {
  const EpiBn e = epi ? *epi : EpiBn();
  SCN_TRY(check_second(second, K));
  const SecondRows two = second ? *second : SecondRows();
  if (!f16_shape(K, Cin, Cout)) return fail(SCN_E_INVALID, "the fp16 gather-GEMM takes 32 or 64 planes on either side");
  if (!map && K != 1) return fail(SCN_E_INVALID, "no map given for a filter volume above 1");
  if (in_stride % 8 != 0 || !aligned16(in) || !aligned16(Wp))
    return fail(SCN_E_INVALID, "fp16 rows must be 16-byte aligned with a stride that is a multiple of 8 elements");
  const __half *inh = static_cast<const __half *>(in);
  const uint4 *W4 = static_cast<const uint4 *>(Wp);
  const int vec = rows_vectorisable(out, out_stride, init, init_stride, bias, e) ? 1 : 0;
#define SCN_F16_LAUNCH(CI, CO, NTR, MINB)                                                                         \
  do {                                                                                                            \
    const long long tiles = (n_out + 8 * NTR - 1) / (8 * NTR);                                                    \
    if (second)                                                                                                   \
      k_gather_mma_f16<CI, CO, NTR, MINB, true><<<(unsigned)((tiles + kWarps - 1) / kWarps), kWarps * 32, 0, s>>>( \
          inh, in_stride, map, K, n_out, W4, bias, out, out_stride, init, init_stride, e, vec, two);              \
    else                                                                                                          \
      k_gather_mma_f16<CI, CO, NTR, MINB, false><<<(unsigned)((tiles + kWarps - 1) / kWarps), kWarps * 32, 0, s>>>( \
          inh, in_stride, map, K, n_out, W4, bias, out, out_stride, init, init_stride, e, vec, two);              \
  } while (0)
  if (Cin == 32 && Cout == 32) SCN_F16_LAUNCH(32, 32, 4, 5);
  else if (Cin == 32 && Cout == 64) SCN_F16_LAUNCH(32, 64, 4, 4);
  else if (Cin == 64 && Cout == 32) SCN_F16_LAUNCH(64, 32, 4, 4);
  else SCN_F16_LAUNCH(64, 64, 2, 4);
#undef SCN_F16_LAUNCH
  SCN_LAUNCHED();
  return SCN_OK;
}

}  // namespace scn
