// Warp-level gather-GEMM for narrow layers (n_in, n_out <= 64): rows gathered straight into registers.
//
//     out[o] = init(o) + sum_k in[ map[k][o] ] * W[k]           (same contract as the other gather-GEMM kernels)
//
// With 32 or 64 planes a reduction step carries too little arithmetic to pay for staging 128-row operand tiles
// in shared memory and driving them through tcgen05 from a single thread: that pipeline spends its time on
// barriers and descriptor traffic (measured: ~1300 cycles per 128-row step of 4 MMAs).  Here a warp owns 16 or 32
// consecutive output rows and all output planes, keeps the accumulator in registers and works through the
// offsets that have at least one neighbour among its rows:
//   * the rows' map entries [K][rows] are staged once in a warp-private slice of shared memory,
//   * for an offset, lane (g, t) (g = lane / 4, t = lane % 4) loads 16 bytes of rows g and g + 8 for every
//     16-plane chunk, straight from global memory through L1 (neighbouring rows of a tile share most of their
//     neighbours, so L1 catches the reuse); absent neighbours load nothing and contribute zeros,
//   * the four floats of such a load feed two mma.sync.m16n8k8 (tf32) as the k-slots (t, t + 4): the reduction
//     index is permuted so that no shuffle or shared-memory transpose is needed; the weights are packed once in
//     the matching order, [K][n_in / 16][n_out / 8][lane] float4, rounded to tf32, and read through L1,
//   * the loads of the next offset are issued before the MMAs of the current one (two register buffers).
// No barrier, no block-wide synchronisation, no scratch memory; skipping works at 16/32-row granularity instead
// of 128.  fp32 inputs are consumed as tf32 (low 13 mantissa bits ignored), accumulation is fp32.
#include "internal.h"
#include <stdlib.h>

namespace scn {

namespace {

constexpr int kWarps = 4;  // warps per block; every warp works alone
constexpr int kMaxK = 27;

__device__ __forceinline__ void mma_m16n8k8_tf32(float (&d)[4], float a0, float a1, float a2, float a3, float b0, float b1) {
  asm("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(__float_as_uint(a0)), "r"(__float_as_uint(a1)), "r"(__float_as_uint(a2)), "r"(__float_as_uint(a3)),
        "r"(__float_as_uint(b0)), "r"(__float_as_uint(b1)));
}

// gathered rows of one offset: [m-tile][row half: g, g + 8][16-plane chunk]
template <int CIN, int MT> struct Frag {
  float4 v[MT][2][CIN / 16];
};

template <int CIN, int MT>
__device__ __forceinline__ void load_rows(Frag<CIN, MT> &f, const int *mp_k, const float *__restrict__ in, long long in_stride,
                                          int g, int t) {
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int s = mp_k[mt * 16 + g + 8 * h];
      const float4 *p = reinterpret_cast<const float4 *>(in + (long long)(s >= 0 ? s : 0) * in_stride) + t;
#pragma unroll
      for (int c = 0; c < CIN / 16; ++c) f.v[mt][h][c] = s >= 0 ? __ldg(p + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
}

template <int CIN, int COUT, int MT>
__device__ __forceinline__ void mma_rows(float (&acc)[MT][COUT / 8][4], const Frag<CIN, MT> &f, const float4 *__restrict__ wk) {
  constexpr int NT = COUT / 8;
#pragma unroll
  for (int c = 0; c < CIN / 16; ++c)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const float4 b = __ldg(wk + (c * NT + nt) * 32);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        mma_m16n8k8_tf32(acc[mt][nt], f.v[mt][0][c].x, f.v[mt][1][c].x, f.v[mt][0][c].y, f.v[mt][1][c].y, b.x, b.y);
        mma_m16n8k8_tf32(acc[mt][nt], f.v[mt][0][c].z, f.v[mt][1][c].z, f.v[mt][0][c].w, f.v[mt][1][c].w, b.z, b.w);
      }
    }
}

template <int CIN, int COUT, int MT, int MINB>
__global__ void __launch_bounds__(kWarps * 32, MINB)
k_gather_mma_tf32(const float *__restrict__ in, long long in_stride, const int32_t *__restrict__ map, int K, long long n_out,
                  const float4 *__restrict__ Wp, const float *__restrict__ bias, float *__restrict__ out, long long out_stride,
                  int accumulate) {
  constexpr int ROWS = 16 * MT, NT = COUT / 8, C16 = CIN / 16;
  __shared__ int s_map[kWarps][kMaxK * ROWS];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const long long row0 = ((long long)blockIdx.x * kWarps + warp) * ROWS;
  if (row0 >= n_out) return;  // warps never synchronise with each other
  int *mp = s_map[warp];

  // stage the map entries of this warp's rows and note which offsets have any
  unsigned int mask = 0;
  if (map) {
    constexpr int PER = 32 / ROWS;  // offsets covered by one warp-wide load
    const int r = lane % ROWS, ksub = lane / ROWS;
    const bool row_ok = row0 + r < n_out;
    for (int k0 = 0; k0 < K; k0 += PER) {
      const int k = k0 + ksub;
      int v = -1;
      if (k < K && row_ok) v = __ldg(map + (long long)k * n_out + row0 + r);
      if (k < K) mp[k * ROWS + r] = v;
      const unsigned int b = __ballot_sync(0xffffffffu, v >= 0);
      if (PER == 2) {
        mask |= ((b & 0xffffu) ? 1u : 0u) << k0;
        mask |= ((b >> 16) ? 1u : 0u) << (k0 + 1);
      } else {
        mask |= (b ? 1u : 0u) << k0;
      }
    }
  } else {  // identity: row o reads row o
    if (lane < ROWS) mp[lane] = row0 + lane < n_out ? (int)(row0 + lane) : -1;
    mask = 1u;
  }
  __syncwarp();

  float acc[MT][NT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[mt][nt][i] = 0.f;

  const float4 *wl = Wp + lane;
  constexpr int WK = C16 * NT * 32;  // float4 per offset
  if (mask) {
    Frag<CIN, MT> f0, f1;
    int k0 = __ffs(mask) - 1;
    mask &= mask - 1;
    load_rows<CIN, MT>(f0, mp + k0 * ROWS, in, in_stride, g, t);
    while (true) {
      int k1 = -1;
      if (mask) {
        k1 = __ffs(mask) - 1;
        mask &= mask - 1;
        load_rows<CIN, MT>(f1, mp + k1 * ROWS, in, in_stride, g, t);
      }
      mma_rows<CIN, COUT, MT>(acc, f0, wl + (long long)k0 * WK);
      if (k1 < 0) break;
      k0 = -1;
      if (mask) {
        k0 = __ffs(mask) - 1;
        mask &= mask - 1;
        load_rows<CIN, MT>(f0, mp + k0 * ROWS, in, in_stride, g, t);
      }
      mma_rows<CIN, COUT, MT>(acc, f1, wl + (long long)k1 * WK);
      if (k0 < 0) break;
    }
  }

  // accumulator fragment: c0,c1 -> row g, planes 8nt + 2t, +1; c2,c3 -> row g + 8
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const long long row = row0 + mt * 16 + g + 8 * h;
      if (row < n_out) {
        float *o = out + row * out_stride + 2 * t;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          float2 v = make_float2(acc[mt][nt][2 * h], acc[mt][nt][2 * h + 1]);
          if (accumulate) {
            const float2 old = *reinterpret_cast<const float2 *>(o + 8 * nt);
            v.x += old.x;
            v.y += old.y;
          } else if (bias) {
            v.x += __ldg(bias + 8 * nt + 2 * t);
            v.y += __ldg(bias + 8 * nt + 2 * t + 1);
          }
          *reinterpret_cast<float2 *>(o + 8 * nt) = v;
        }
      }
    }
}

// W [K][n_in][n_out] -> [K][n_in/16][n_out/8][lane][4], rounded to tf32 (round to nearest, ties away)
__global__ void k_pack_weights_mma(const float *__restrict__ W, float *__restrict__ Wp, int Cin, int Cout, long long total) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int NT = Cout / 8, C16 = Cin / 16;
  const int j = (int)(i & 3), lane = (int)((i >> 2) & 31);
  long long rest = i >> 7;
  const int nt = (int)(rest % NT);
  rest /= NT;
  const int c = (int)(rest % C16);
  const long long k = rest / C16;
  const int g = lane >> 2, t = lane & 3;
  const int ci = c * 16 + 4 * t + j, co = nt * 8 + g;
  const float w = W[(k * Cin + ci) * Cout + co];
  uint32_t u;
  asm("cvt.rna.tf32.f32 %0, %1;\n" : "=r"(u) : "f"(w));
  Wp[i] = __uint_as_float(u);
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int max_planes() {
  static const int v = []() {
    const char *e = getenv("INSCONV_WARP_MMA_MAX");  // development aid: widest layer the warp-level kernel takes (0: off)
    return e ? atoi(e) : 64;
  }();
  return v;
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
                    const float *bias, float *out, int64_t out_stride, int64_t Cin, int64_t Cout, int accumulate, bool packed,
                    cudaStream_t s, bool *handled) {
  *handled = false;
  if (!warp_mma_shape(K, Cin, Cout)) return SCN_OK;
  if (!map && K != 1) return SCN_OK;
  if (in_stride % 4 != 0 || out_stride % 2 != 0 || !aligned16(in) || !aligned16(W) || !aligned16(out)) return SCN_OK;
  float *own = nullptr;
  const float *Wp = W;
  if (!packed) {
    SCN_TRY(dev_alloc_t(&own, (size_t)K * Cin * Cout, s));
    SCN_TRY(warp_mma_pack(W, K, Cin, Cout, own, s));
    Wp = own;
  }
#define SCN_WARP_LAUNCH(CI, CO, MT, MINB)                                                                             \
  do {                                                                                                                \
    const long long tiles = (n_out + 16 * MT - 1) / (16 * MT);                                                        \
    k_gather_mma_tf32<CI, CO, MT, MINB><<<(unsigned)((tiles + kWarps - 1) / kWarps), kWarps * 32, 0, s>>>(            \
        in, in_stride, map, K, n_out, reinterpret_cast<const float4 *>(Wp), bias, out, out_stride, accumulate);       \
  } while (0)
  const int key = (int)Cin * 100 + (int)Cout;
  switch (key) {
    case 1616: SCN_WARP_LAUNCH(16, 16, 2, 4); break;
    case 1632: SCN_WARP_LAUNCH(16, 32, 2, 4); break;
    case 1664: SCN_WARP_LAUNCH(16, 64, 1, 4); break;
    case 3216: SCN_WARP_LAUNCH(32, 16, 2, 4); break;
    case 3232: SCN_WARP_LAUNCH(32, 32, 2, 4); break;
    case 3264: SCN_WARP_LAUNCH(32, 64, 1, 4); break;
    case 6416: SCN_WARP_LAUNCH(64, 16, 1, 4); break;
    case 6432: SCN_WARP_LAUNCH(64, 32, 1, 4); break;
    case 6464: SCN_WARP_LAUNCH(64, 64, 1, 3); break;
    default: dev_free(own, s); return SCN_OK;
  }
#undef SCN_WARP_LAUNCH
  SCN_LAUNCHED();
  dev_free(own, s);
  *handled = true;
  return SCN_OK;
}

}  // namespace scn
