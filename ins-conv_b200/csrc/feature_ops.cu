// Feature kernels: output-stationary gather-GEMM (fp32 FFMA path), BatchNorm + leaky ReLU,
// InputLayer / OutputLayer reductions, and their incremental variants.
//
// Every convolution of the hot path is one launch of the same kernel:
//     out[o] = init(o) + sum_k  in[ map[k][o] ] * W[k]
// with map = the 27-offset neighbour map (submanifold), the 8-slot child map (stride-2
// convolution), the 8-slot parent map (deconvolution) or no map at all (1x1 NetworkInNetwork).
// A CTA owns a tile of consecutive output rows, loops over the offsets and channel chunks, and
// writes each output row exactly once: no atomics, no read-modify-write of the output, and the
// summation order is fixed, so results are deterministic.  Consecutive rows are consecutive in key
// order (x fastest), so the rows a tile gathers overlap heavily and are served from L2.
//
// Reference arithmetic restated here (paths relative to sparseconvnet/SCN/):
//   conv / deconv           CPU/Convolution.cpp:36-72, CPU/Deconvolution.cpp:8-44, CUDA/Convolution.cu:81-223
//   BatchNorm test mode     CUDA/BatchNormalization.cu:78-107, incremental :112-150
//   Input / Output layer    CUDA/IOLayers.cu:18-62, incremental :82-142
//   NetworkInNetwork        CUDA/NetworkInNetwork.cpp:9-25
#include "internal.h"
#include <cuda_fp16.h>

namespace scn {

static inline unsigned blocks_for(long long n, int t) { return (unsigned)((n + t - 1) / t); }
static inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// ---------------------------------------------------------------------------------------------
// gather-GEMM, fp32
// ---------------------------------------------------------------------------------------------
constexpr int kBK = 16;  // input channels staged per step

template <int TM, int TN, int RM, int RN>
__global__ void __launch_bounds__((TM / RM) * (TN / RN))
k_gather_gemm_f32(const float *__restrict__ in, long long in_stride, const int32_t *__restrict__ map, int K,
                  long long n_out, const float *__restrict__ W, const float *__restrict__ bias,
                  float *out, long long out_stride, int Cin, int Cout, const float *init, long long init_stride, int vecA,
                  int vecB) {
  constexpr int NT = (TM / RM) * (TN / RN);
  constexpr int CG = TN / RN;  // threads along the output channels
  static_assert(RM % 4 == 0 && RN == 4, "register tile is read as float4");
  __shared__ __align__(16) float As[kBK][TM + 4];
  __shared__ __align__(16) float Bs[kBK][TN];
  __shared__ int s_idx[TM];
  const int tid = threadIdx.x, tx = tid % CG, ty = tid / CG;
  const long long row0 = (long long)blockIdx.x * TM;
  const int n0 = blockIdx.y * TN;
  float acc[RM][RN];
#pragma unroll
  for (int i = 0; i < RM; ++i)
#pragma unroll
    for (int j = 0; j < RN; ++j) acc[i][j] = 0.f;

  for (int k = 0; k < K; ++k) {
    int any_local = 0;
    for (int r = tid; r < TM; r += NT) {
      const long long row = row0 + r;
      int v = -1;
      if (row < n_out) v = map ? __ldg(map + (long long)k * n_out + row) : (int)row;
      s_idx[r] = v;
      any_local |= (v >= 0);
    }
    if (!__syncthreads_or(any_local)) continue;  // no row of this tile has a neighbour at offset k
    const float *Wk = W + (long long)k * Cin * Cout;
    for (int c0 = 0; c0 < Cin; c0 += kBK) {
      // gathered rows, transposed to channel-major in shared memory
      for (int idx = tid; idx < TM * (kBK / 4); idx += NT) {
        const int r = idx / (kBK / 4), ch = idx % (kBK / 4);
        const int src = s_idx[r];
        const int c = c0 + ch * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (src >= 0 && c < Cin) {
          const float *p = in + (long long)src * in_stride + c;
          if (vecA && c + 3 < Cin) {
            v = __ldg(reinterpret_cast<const float4 *>(p));
          } else {
            v.x = __ldg(p);
            if (c + 1 < Cin) v.y = __ldg(p + 1);
            if (c + 2 < Cin) v.z = __ldg(p + 2);
            if (c + 3 < Cin) v.w = __ldg(p + 3);
          }
        }
        As[ch * 4 + 0][r] = v.x;
        As[ch * 4 + 1][r] = v.y;
        As[ch * 4 + 2][r] = v.z;
        As[ch * 4 + 3][r] = v.w;
      }
      // weight slab chunk [kBK][TN]
      for (int idx = tid; idx < kBK * (TN / 4); idx += NT) {
        const int kk = idx / (TN / 4), cn = (idx % (TN / 4)) * 4;
        const int ci = c0 + kk, co = n0 + cn;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (ci < Cin && co < Cout) {
          const float *p = Wk + (long long)ci * Cout + co;
          if (vecB && co + 3 < Cout) {
            v = __ldg(reinterpret_cast<const float4 *>(p));
          } else {
            v.x = __ldg(p);
            if (co + 1 < Cout) v.y = __ldg(p + 1);
            if (co + 2 < Cout) v.z = __ldg(p + 2);
            if (co + 3 < Cout) v.w = __ldg(p + 3);
          }
        }
        *reinterpret_cast<float4 *>(&Bs[kk][cn]) = v;
      }
      __syncthreads();
#pragma unroll
      for (int kk = 0; kk < kBK; ++kk) {
        float a[RM];
#pragma unroll
        for (int q = 0; q < RM / 4; ++q) {
          const float4 t = *reinterpret_cast<const float4 *>(&As[kk][ty * RM + q * 4]);
          a[q * 4 + 0] = t.x; a[q * 4 + 1] = t.y; a[q * 4 + 2] = t.z; a[q * 4 + 3] = t.w;
        }
        const float4 b = *reinterpret_cast<const float4 *>(&Bs[kk][tx * RN]);
#pragma unroll
        for (int i = 0; i < RM; ++i) {
          acc[i][0] = fmaf(a[i], b.x, acc[i][0]);
          acc[i][1] = fmaf(a[i], b.y, acc[i][1]);
          acc[i][2] = fmaf(a[i], b.z, acc[i][2]);
          acc[i][3] = fmaf(a[i], b.w, acc[i][3]);
        }
      }
      __syncthreads();
    }
  }
#pragma unroll
  for (int i = 0; i < RM; ++i) {
    const long long row = row0 + ty * RM + i;
    if (row >= n_out) continue;
#pragma unroll
    for (int j = 0; j < RN; ++j) {
      const int co = n0 + tx * RN + j;
      if (co >= Cout) continue;
      float v = acc[i][j];
      float *o = out + row * out_stride + co;
      if (init) v += init[row * init_stride + co];
      else if (bias) v += __ldg(bias + co);
      *o = v;
    }
  }
}

int gather_gemm_tf32(const float *in, int64_t in_stride, int64_t in_rows, const int32_t *map, int K, int64_t n_out, const float *W,
                     const float *bias, float *out, int64_t out_stride, int64_t Cin, int64_t Cout, const float *init,
                     int64_t init_stride, bool packed, cudaStream_t s, bool *handled);

int gather_gemm(const float *in, int64_t in_stride, int64_t in_rows, const int32_t *map, int K, int64_t n_out, const float *W,
                const float *bias, float *out, int64_t out_stride, int64_t Cin, int64_t Cout, const float *init,
                int64_t init_stride, int precision, cudaStream_t s) {
  if (n_out == 0) return SCN_OK;
  if (Cin <= 0 || Cout <= 0 || Cin > 65536 || Cout > 65536) return fail(SCN_E_INVALID, "bad plane count");
  if (precision != SCN_PREC_FP32 && precision != SCN_PREC_TF32 && precision != SCN_PREC_TF32_PACKED)
    return fail(SCN_E_INVALID, "unknown precision");
  if (precision != SCN_PREC_FP32) {
    bool handled = false;
    const bool packed = precision == SCN_PREC_TF32_PACKED;
    if (warp_mma_shape(K, Cin, Cout) || (Cin <= 4 && !packed)) {
      SCN_TRY(gather_mma_warp(in, in_stride, map, K, n_out, W, bias, out, out_stride, Cin, Cout, init, init_stride, packed, s,
                              &handled));
      if (handled) return SCN_OK;
      if (packed) return fail(SCN_E_INVALID, "packed weights given with an alignment the warp-level kernel does not take");
    }
    SCN_TRY(gather_gemm_tf32(in, in_stride, in_rows, map, K, n_out, W, bias, out, out_stride, Cin, Cout, init, init_stride,
                             packed, s, &handled));
    if (handled) return SCN_OK;
    if (precision == SCN_PREC_TF32_PACKED)
      return fail(SCN_E_INVALID, "packed weights given for a shape or alignment the tensor-core kernel does not take");
    // shapes the tensor-core kernel does not tile (n_in not a multiple of 8, ...) use the fp32 kernel,
    // which is at least as accurate.
  }
  const int vecA = aligned16(in) && (in_stride % 4 == 0);
  const int vecB = aligned16(W) && (Cout % 4 == 0);
  if (Cout <= 16) {
    dim3 grid(blocks_for(n_out, 128), 1);
    k_gather_gemm_f32<128, 16, 4, 4><<<grid, 128, 0, s>>>(in, in_stride, map, K, n_out, W, bias, out, out_stride,
                                                        (int)Cin, (int)Cout, init, init_stride, vecA, vecB);
  } else if (Cout <= 32) {
    dim3 grid(blocks_for(n_out, 64), 1);
    k_gather_gemm_f32<64, 32, 4, 4><<<grid, 128, 0, s>>>(in, in_stride, map, K, n_out, W, bias, out, out_stride,
                                                       (int)Cin, (int)Cout, init, init_stride, vecA, vecB);
  } else {
    dim3 grid(blocks_for(n_out, 64), blocks_for(Cout, 64));
    k_gather_gemm_f32<64, 64, 8, 4><<<grid, 128, 0, s>>>(in, in_stride, map, K, n_out, W, bias, out, out_stride,
                                                       (int)Cin, (int)Cout, init, init_stride, vecA, vecB);
  }
  SCN_LAUNCHED();
  return SCN_OK;
}

// ---------------------------------------------------------------------------------------------
// BatchNorm (running statistics) + leaky ReLU; optional incremental form
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float leaky(float v, float leak) { return v > 0.f ? v : v * leak; }

template <int VEC>
__global__ void k_bn(const float *__restrict__ in, long long in_stride, float *__restrict__ out, long long out_stride,
                     long long rows, int C, const float *__restrict__ mean, const float *__restrict__ var,
                     const float *__restrict__ gamma, const float *__restrict__ beta, float eps, float leak,
                     const int32_t *__restrict__ pre_exist, const float *__restrict__ pre_out,
                     const float *__restrict__ pre_in) {
  extern __shared__ float sm[];  // scale[C], shift[C]
  float *sw = sm, *sb = sm + C;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float w = (1.0f / sqrtf(var[c] + eps)) * (gamma ? gamma[c] : 1.f);
    sw[c] = w;
    sb[c] = (beta ? beta[c] : 0.f) - mean[c] * w;
  }
  __syncthreads();
  const int cv = C / VEC;
  const long long total = rows * cv;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / cv;
    const int c = (int)(i % cv) * VEC;
    const int pe = pre_exist ? pre_exist[row] : -1;
    if (VEC == 4) {
      float4 x = *reinterpret_cast<const float4 *>(in + row * in_stride + c);
      float4 y;
      float xs[4] = {x.x, x.y, x.z, x.w}, ys[4];
      float pi[4] = {0, 0, 0, 0}, po[4] = {0, 0, 0, 0};
      if (pe >= 0) {
        float4 a = *reinterpret_cast<const float4 *>(pre_in + (long long)pe * C + c);
        float4 b = *reinterpret_cast<const float4 *>(pre_out + (long long)pe * C + c);
        pi[0] = a.x; pi[1] = a.y; pi[2] = a.z; pi[3] = a.w;
        po[0] = b.x; po[1] = b.y; po[2] = b.z; po[3] = b.w;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float w = sw[c + j];
        const float o = w * xs[j] + sb[c + j];
        ys[j] = (pe >= 0) ? leaky(o + pi[j] * w, leak) - po[j] : leaky(o, leak);
      }
      y.x = ys[0]; y.y = ys[1]; y.z = ys[2]; y.w = ys[3];
      *reinterpret_cast<float4 *>(out + row * out_stride + c) = y;
    } else {
      const float w = sw[c];
      const float o = w * in[row * in_stride + c] + sb[c];
      float y;
      if (pe >= 0) y = leaky(o + pre_in[(long long)pe * C + c] * w, leak) - pre_out[(long long)pe * C + c];
      else y = leaky(o, leak);
      out[row * out_stride + c] = y;
    }
  }
}

// The same BatchNorm + leaky ReLU with the result rounded to fp16: the 16-bit rows are what the fp16 gather-GEMM
// of the following convolution reads (half the bytes per gathered row).  Eight planes per thread.
// Incremental form (pre_exist given): for a site that existed in the saved frame the result is the RESIDUAL of the
// activation, act(w (x + x_saved) + b) - y_saved (CUDA/BatchNormalization.cu:112-150), with y_saved read from the fp16
// rows the saved frame's BatchNorm wrote and x_saved from the fp32 rows it read.
__global__ void k_bn_f16out(const float *__restrict__ in, long long in_stride, __half *__restrict__ out, long long out_stride,
                            long long rows, int C, const float *__restrict__ mean, const float *__restrict__ var,
                            const float *__restrict__ gamma, const float *__restrict__ beta, float eps, float leak,
                            const int32_t *__restrict__ pre_exist, const __half *__restrict__ pre_out, long long pre_out_stride,
                            const float *__restrict__ pre_in, long long pre_in_stride, int affine_given) {
  extern __shared__ float sm[];  // scale[C], shift[C]
  float *sw = sm, *sb = sm + C;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    if (affine_given) {  // mean = scale, var = shift
      sw[c] = mean[c];
      sb[c] = var[c];
    } else {
      const float w = (1.0f / sqrtf(var[c] + eps)) * (gamma ? gamma[c] : 1.f);
      sw[c] = w;
      sb[c] = (beta ? beta[c] : 0.f) - mean[c] * w;
    }
  }
  __syncthreads();
  const int cv = C / 8;
  const long long total = rows * cv;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / cv;
    const int c = (int)(i % cv) * 8;
    const float4 x0 = *reinterpret_cast<const float4 *>(in + row * in_stride + c);
    const float4 x1 = *reinterpret_cast<const float4 *>(in + row * in_stride + c + 4);
    float xs[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
    float ys[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};  // what the saved frame held at this site (residual form)
    const int pe = pre_exist ? pre_exist[row] : -1;
    if (pe >= 0) {
      const float4 a0 = *reinterpret_cast<const float4 *>(pre_in + (long long)pe * pre_in_stride + c);
      const float4 a1 = *reinterpret_cast<const float4 *>(pre_in + (long long)pe * pre_in_stride + c + 4);
      xs[0] += a0.x, xs[1] += a0.y, xs[2] += a0.z, xs[3] += a0.w, xs[4] += a1.x, xs[5] += a1.y, xs[6] += a1.z, xs[7] += a1.w;
      const uint4 q = *reinterpret_cast<const uint4 *>(pre_out + (long long)pe * pre_out_stride + c);
      const __half2 *h = reinterpret_cast<const __half2 *>(&q);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(h[j]);
        ys[2 * j] = f.x;
        ys[2 * j + 1] = f.y;
      }
    }
    __align__(16) __half2 y[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      // values beyond fp16's range saturate at +-65504 instead of becoming infinities
      const float a = fminf(fmaxf(leaky(sw[c + 2 * j] * xs[2 * j] + sb[c + 2 * j], leak) - ys[2 * j], -65504.f), 65504.f);
      const float b =
          fminf(fmaxf(leaky(sw[c + 2 * j + 1] * xs[2 * j + 1] + sb[c + 2 * j + 1], leak) - ys[2 * j + 1], -65504.f), 65504.f);
      y[j] = __floats2half2_rn(a, b);
    }
    *reinterpret_cast<uint4 *>(out + row * out_stride + c) = *reinterpret_cast<const uint4 *>(y);
  }
}

// JoinTable followed by BatchNorm + leaky ReLU in one pass: joined[r] = [a[r] | b[r]] as fp32 rows (the shortcut of the
// block behind reads them) and rows16[r] = activation(joined[r] * scale + shift) as fp16 rows (the convolution behind the
// BatchNorm gathers them).  One thread per four planes of a row.
__global__ void k_join_bn_f16(const float *__restrict__ a, long long a_stride, int a_planes, const float *__restrict__ b,
                              long long b_stride, int b_planes, long long rows, float *__restrict__ joined, long long joined_stride,
                              const float *__restrict__ scale, const float *__restrict__ shift, float leak,
                              __half *__restrict__ rows16, long long rows16_stride) {
  const int groups = (a_planes + b_planes) >> 2;
  const long long total = rows * groups;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / groups;
    const int c = (int)(i - r * groups) << 2;
    const float4 v = c < a_planes ? __ldg(reinterpret_cast<const float4 *>(a + r * a_stride + c))
                                  : __ldg(reinterpret_cast<const float4 *>(b + r * b_stride + (c - a_planes)));
    *reinterpret_cast<float4 *>(joined + r * joined_stride + c) = v;
    const float4 sc = __ldg(reinterpret_cast<const float4 *>(scale + c)), sh = __ldg(reinterpret_cast<const float4 *>(shift + c));
    float y[4] = {fmaf(v.x, sc.x, sh.x), fmaf(v.y, sc.y, sh.y), fmaf(v.z, sc.z, sh.z), fmaf(v.w, sc.w, sh.w)};
#pragma unroll
    for (int j = 0; j < 4; ++j) y[j] = fminf(fmaxf(y[j] > 0.f ? y[j] : y[j] * leak, -65504.f), 65504.f);  // saturates like k_bn_f16out
    const __half2 lo = __floats2half2_rn(y[0], y[1]), hi = __floats2half2_rn(y[2], y[3]);
    uint2 packed;
    packed.x = *reinterpret_cast<const unsigned int *>(&lo);
    packed.y = *reinterpret_cast<const unsigned int *>(&hi);
    *reinterpret_cast<uint2 *>(rows16 + r * rows16_stride + c) = packed;
  }
}

int join_bn_forward_f16(const float *a, int64_t a_stride, int64_t a_planes, const float *b, int64_t b_stride, int64_t b_planes,
                        int64_t rows, float *joined, int64_t joined_stride, const float *scale, const float *shift, float leak,
                        void *rows16, int64_t rows16_stride, cudaStream_t s) {
  if (rows == 0) return SCN_OK;
  if (a_planes <= 0 || b_planes <= 0 || a_planes % 4 != 0 || b_planes % 4 != 0 || a_planes + b_planes > 4096)
    return fail(SCN_E_INVALID, "joined BatchNorm: plane counts must be positive multiples of 4, at most 4096 together");
  if (a_stride % 4 != 0 || b_stride % 4 != 0 || joined_stride % 4 != 0 || rows16_stride % 4 != 0 || !aligned16(a) || !aligned16(b) ||
      !aligned16(joined) || !aligned16(scale) || !aligned16(shift) || (reinterpret_cast<uintptr_t>(rows16) & 7))
    return fail(SCN_E_INVALID, "joined BatchNorm: rows must be 16-byte aligned with strides that are multiples of 4 elements");
  const long long work = rows * ((a_planes + b_planes) / 4);
  unsigned blocks = blocks_for(work, 256);
  if (blocks > 148u * 16u) blocks = 148u * 16u;
  k_join_bn_f16<<<blocks, 256, 0, s>>>(a, a_stride, (int)a_planes, b, b_stride, (int)b_planes, rows, joined, joined_stride, scale,
                                       shift, leak, static_cast<__half *>(rows16), rows16_stride);
  SCN_LAUNCHED();
  return SCN_OK;
}

int bn_forward_f16out(const float *in, int64_t in_stride, void *out, int64_t out_stride, int64_t rows, int64_t planes,
                      const float *mean, const float *var, const float *gamma, const float *beta, float eps, float leak,
                      cudaStream_t s, const int32_t *pre_exist, const void *pre_out, int64_t pre_out_stride, const float *pre_in,
                      int64_t pre_in_stride, bool affine_given) {
  if (rows == 0 || planes == 0) return SCN_OK;
  if (planes > 4096) return fail(SCN_E_INVALID, "BatchNorm over more than 4096 planes");
  if (planes % 8 != 0 || in_stride % 4 != 0 || out_stride % 8 != 0 || !aligned16(in) || !aligned16(out))
    return fail(SCN_E_INVALID, "fp16 BatchNorm output needs planes and the output stride to be multiples of 8 and 16-byte aligned rows");
  if (pre_exist && (!pre_out || !pre_in || pre_out_stride % 8 != 0 || pre_in_stride % 4 != 0 || !aligned16(pre_out) || !aligned16(pre_in)))
    return fail(SCN_E_INVALID, "incremental fp16 BatchNorm: saved rows must be 16-byte aligned (fp16 stride a multiple of 8, fp32 of 4)");
  const long long work = rows * (planes / 8);
  unsigned blocks = blocks_for(work, 256);
  if (blocks > 148u * 16u) blocks = 148u * 16u;
  k_bn_f16out<<<blocks, 256, (size_t)planes * 2 * sizeof(float), s>>>(in, in_stride, static_cast<__half *>(out), out_stride, rows,
                                                                      (int)planes, mean, var, gamma, beta, eps, leak, pre_exist,
                                                                      static_cast<const __half *>(pre_out), pre_out_stride, pre_in,
                                                                      pre_in_stride, affine_given ? 1 : 0);
  SCN_LAUNCHED();
  return SCN_OK;
}

int bn_forward(const float *in, int64_t in_stride, float *out, int64_t out_stride, int64_t rows, int64_t planes,
               const float *mean, const float *var, const float *gamma, const float *beta, float eps, float leak,
               const int32_t *pre_exist, const float *pre_out, const float *pre_in, cudaStream_t s) {
  if (rows == 0 || planes == 0) return SCN_OK;
  if (planes > 4096) return fail(SCN_E_INVALID, "BatchNorm over more than 4096 planes");
  const bool vec = planes % 4 == 0 && in_stride % 4 == 0 && out_stride % 4 == 0 && aligned16(in) && aligned16(out) &&
                   (!pre_exist || (aligned16(pre_in) && aligned16(pre_out)));
  const long long work = rows * (vec ? planes / 4 : planes);
  unsigned blocks = blocks_for(work, 256);
  if (blocks > 148u * 16u) blocks = 148u * 16u;
  const size_t smem = (size_t)planes * 2 * sizeof(float);
  if (vec)
    k_bn<4><<<blocks, 256, smem, s>>>(in, in_stride, out, out_stride, rows, (int)planes, mean, var, gamma, beta, eps,
                                     leak, pre_exist, pre_out, pre_in);
  else
    k_bn<1><<<blocks, 256, smem, s>>>(in, in_stride, out, out_stride, rows, (int)planes, mean, var, gamma, beta, eps,
                                     leak, pre_exist, pre_out, pre_in);
  SCN_LAUNCHED();
  return SCN_OK;
}


// ---------------------------------------------------------------------------------------------
// BatchNorm with batch statistics (train mode forward; CUDA/BatchNormalization.cu:14-72)
// ---------------------------------------------------------------------------------------------
// pass 1: per-plane sum and sum of squares.  A block owns a slab of rows; threads (32 planes x 8 rows)
// accumulate in fp32, the block reduces in shared memory and adds into fp64 totals.
__global__ void k_bn_stats(const float *__restrict__ in, long long in_stride, long long rows, int C,
                           long long rows_per_block, double *__restrict__ sums /*[2][C]*/) {
  __shared__ float s1[8][33], s2[8][33];
  const long long r0 = (long long)blockIdx.x * rows_per_block;
  const long long r1 = min(rows, r0 + rows_per_block);
  for (int c0 = 0; c0 < C; c0 += 32) {
    const int c = c0 + threadIdx.x;
    float a = 0.f, b = 0.f;
    if (c < C)
      for (long long r = r0 + threadIdx.y; r < r1; r += 8) {
        const float v = in[r * in_stride + c];
        a += v;
        b += v * v;
      }
    s1[threadIdx.y][threadIdx.x] = a;
    s2[threadIdx.y][threadIdx.x] = b;
    __syncthreads();
    if (threadIdx.y == 0 && c < C) {
      double ta = 0, tb = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        ta += s1[j][threadIdx.x];
        tb += s2[j][threadIdx.x];
      }
      atomicAdd(&sums[c], ta);
      atomicAdd(&sums[C + c], tb);
    }
    __syncthreads();
  }
}
// pass 2: mean, biased variance for the normalisation, running statistics (unbiased variance) updated in place
__global__ void k_bn_finalize(const double *__restrict__ sums, long long rows, int C, float eps, float momentum,
                              float *save_mean, float *save_invstd, float *running_mean, float *running_var,
                              float *batch_var) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const double mean = sums[c] / (double)rows;
  const double ss = sums[C + c] - mean * mean * (double)rows;  // sum of squared deviations
  if (save_mean) save_mean[c] = (float)mean;
  running_mean[c] = momentum * running_mean[c] + (1.f - momentum) * (float)mean;
  running_var[c] = momentum * running_var[c] + (1.f - momentum) * (float)(ss / (double)(rows - 1));
  const float var_b = (float)(ss / (double)rows);
  batch_var[c] = var_b;
  if (save_invstd) save_invstd[c] = 1.0f / sqrtf(var_b + eps);
  batch_var[C + c] = (float)mean;
}

int bn_forward_train(const float *in, int64_t in_stride, float *out, int64_t out_stride, int64_t rows, int64_t planes,
                     float *running_mean, float *running_var, float *save_mean, float *save_invstd, const float *gamma,
                     const float *beta, float eps, float momentum, float leak, cudaStream_t s) {
  if (rows == 0 || planes == 0) return SCN_OK;
  if (planes > 4096) return fail(SCN_E_INVALID, "BatchNorm over more than 4096 planes");
  double *sums = nullptr;
  float *stat = nullptr;  // [0..C): batch variance, [C..2C): batch mean
  SCN_TRY(dev_alloc_t(&sums, (size_t)planes * 2, s));
  SCN_TRY(dev_alloc_t(&stat, (size_t)planes * 2, s));
  SCN_CUDA(cudaMemsetAsync(sums, 0, (size_t)planes * 2 * sizeof(double), s));
  long long blocks = (rows + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  const long long rpb = (rows + blocks - 1) / blocks;
  k_bn_stats<<<(unsigned)blocks, dim3(32, 8), 0, s>>>(in, in_stride, rows, (int)planes, rpb, sums);
  SCN_LAUNCHED();
  k_bn_finalize<<<blocks_for(planes, 128), 128, 0, s>>>(sums, rows, (int)planes, eps, momentum, save_mean, save_invstd,
                                                        running_mean, running_var, stat);
  SCN_LAUNCHED();
  int r = bn_forward(in, in_stride, out, out_stride, rows, planes, stat + planes, stat, gamma, beta, eps, leak, nullptr,
                     nullptr, nullptr, s);
  dev_free(sums, s);
  dev_free(stat, s);
  return r;
}

// ---------------------------------------------------------------------------------------------
// InputLayer / OutputLayer
// ---------------------------------------------------------------------------------------------
// One thread per (site, plane).  Points of a site are added in ascending point index, the order of the
// reference's rule rows.  With pre_exist: residual of the voxel mean against the saved frame.
__global__ void k_input_fwd(const float *__restrict__ in, float *__restrict__ out, long long n, int planes,
                            const int32_t *__restrict__ off, const int32_t *__restrict__ item, int average,
                            const int32_t *__restrict__ pre_exist, const int32_t *__restrict__ pre_off,
                            const float *__restrict__ pre_out, const int32_t *__restrict__ pre_count) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n * planes) return;
  const long long r = i / planes;
  const int c = (int)(i % planes);
  const int b = off ? off[r] : (int)r, e = off ? off[r + 1] : (int)r + 1;
  const int cnt = e - b;
  int pe = -1, pre_cnt = 0;
  if (pre_exist) {
    pe = pre_exist[r];
    if (pe >= 0) pre_cnt = pre_count ? pre_count[pe] : pre_off ? pre_off[pe + 1] - pre_off[pe] : 1;
  }
  const float mult = (average && cnt > 0) ? 1.0f / (float)(cnt + pre_cnt) : 1.0f;
  float acc = 0.f;
  for (int j = b; j < e; ++j) acc += mult * in[(long long)item[j] * planes + c];
  if (pe >= 0) acc = acc + pre_out[(long long)pe * planes + c] * ((float)pre_cnt * mult - 1.0f);
  out[i] = acc;
}

// Grids whose sites have exactly one source each (the usual case: deduplicated voxels): one thread per (source, plane)
// writes the site's row; nothing is summed, so the order of the sources does not matter and no source list is needed.
__global__ void k_input_fwd_unique(const float *__restrict__ in, float *__restrict__ out, long long n_src, int planes,
                                   const int32_t *__restrict__ src_row, int average, const int32_t *__restrict__ pre_exist,
                                   const int32_t *__restrict__ pre_off, const float *__restrict__ pre_out,
                                   const int32_t *__restrict__ pre_count) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_src * planes) return;
  const long long p = i / planes;
  const int c = (int)(i % planes);
  const int r = src_row[p];
  int pe = -1, pre_cnt = 0;
  if (pre_exist) {
    pe = pre_exist[r];
    if (pe >= 0) pre_cnt = pre_count ? pre_count[pe] : pre_off ? pre_off[pe + 1] - pre_off[pe] : 1;
  }
  const float mult = average ? 1.0f / (float)(1 + pre_cnt) : 1.0f;
  float acc = 0.f;
  acc += mult * in[i];
  if (pe >= 0) acc = acc + pre_out[(long long)pe * planes + c] * ((float)pre_cnt * mult - 1.0f);
  out[(long long)r * planes + c] = acc;
}

__global__ void k_output_fwd(const float *__restrict__ in, float *__restrict__ out, long long n_pts, int planes,
                             const int32_t *__restrict__ src_row, const int32_t *__restrict__ pre_exist,
                             const float *__restrict__ pre_in) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_pts * planes) return;
  const long long p = i / planes;
  const int c = (int)(i % planes);
  const int r = src_row[p];
  float v = in[(long long)r * planes + c];
  if (pre_exist) {
    const int pe = pre_exist[r];
    if (pe >= 0) v += pre_in[(long long)pe * planes + c];
  }
  out[i] = v;
}

int input_forward(const Grid &g, const float *in, float *out, int64_t planes, int average, const int32_t *pre_exist,
                  const Grid *pre, const float *pre_out, cudaStream_t s) {
  if (g.n == 0 || planes == 0) return SCN_OK;
  if (!g.csr_off && g.n == g.n_src) {  // one source per site
    if (!g.src_row) return fail(SCN_E_STATE, "grid has no input rules");
    k_input_fwd_unique<<<blocks_for(g.n_src * planes, 256), 256, 0, s>>>(in, out, g.n_src, (int)planes, g.src_row, average, pre_exist,
                                                                       pre ? pre->csr_off : nullptr, pre_out,
                                                                       pre ? pre->site_count : nullptr);
    SCN_LAUNCHED();
    return SCN_OK;
  }
  if (!g.csr_item) return fail(SCN_E_STATE, "grid has no input rules");
  k_input_fwd<<<blocks_for(g.n * planes, 256), 256, 0, s>>>(in, out, g.n, (int)planes, g.csr_off, g.csr_item, average,
                                                          pre_exist, pre ? pre->csr_off : nullptr, pre_out,
                                                          pre ? pre->site_count : nullptr);
  SCN_LAUNCHED();
  return SCN_OK;
}

// the same, four planes per thread (planes a multiple of 4, 16-byte aligned rows): 16-byte loads and stores, one
// division per four values
__global__ void k_output_fwd4(const float4 *__restrict__ in, float4 *__restrict__ out, long long n_pts, int groups,
                              const int32_t *__restrict__ src_row, const int32_t *__restrict__ pre_exist,
                              const float4 *__restrict__ pre_in) {
  const long long total = n_pts * groups;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long p = i / groups;
    const int c = (int)(i - p * groups);
    const int r = __ldg(src_row + p);
    float4 v = __ldg(in + (long long)r * groups + c);
    if (pre_exist) {
      const int pe = __ldg(pre_exist + r);
      if (pe >= 0) {
        const float4 w = __ldg(pre_in + (long long)pe * groups + c);
        v.x += w.x;
        v.y += w.y;
        v.z += w.z;
        v.w += w.w;
      }
    }
    out[i] = v;
  }
}
int output_forward(const Grid &g, const float *in, float *out, int64_t planes, const int32_t *pre_exist,
                   const float *pre_in, cudaStream_t s) {
  if (g.n_src == 0 || planes == 0) return SCN_OK;
  if (planes % 4 == 0 && aligned16(in) && aligned16(out) && (!pre_exist || aligned16(pre_in))) {
    const long long work = g.n_src * (planes / 4);
    unsigned blocks = blocks_for(work, 256);
    if (blocks > 148u * 32u) blocks = 148u * 32u;
    k_output_fwd4<<<blocks, 256, 0, s>>>(reinterpret_cast<const float4 *>(in), reinterpret_cast<float4 *>(out), g.n_src,
                                         (int)(planes / 4), g.src_row, pre_exist, reinterpret_cast<const float4 *>(pre_in));
    SCN_LAUNCHED();
    return SCN_OK;
  }
  k_output_fwd<<<blocks_for(g.n_src * planes, 256), 256, 0, s>>>(in, out, g.n_src, (int)planes, g.src_row, pre_exist,
                                                               pre_in);
  SCN_LAUNCHED();
  return SCN_OK;
}

}  // namespace scn
