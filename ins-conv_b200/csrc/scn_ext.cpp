// The torch extension module `sparseconvnet.SCN`: the operator surface the sparseconvnet Python
// modules call, for dimension 3, forwarding to the C ABI of libinsconv_b200.so.
//
// It mirrors the hot-path subset of the reference's pybind module (sparseconvnet/SCN/pybind.cpp:13-33,
// 73-78, 97-102, 153-157, 173-189, 219-257, 304; prototypes in sparseconvnet/SCN/sparseconvnet.h):
// same function names, argument order and conventions -- sizes are CPU LongTensors, outputs arrive
// empty and are resized here, "no bias" is an empty tensor, convolutions return the multiply-add
// count.  Differences by design: errors raise Python exceptions instead of exiting the process, work
// is queued on torch's current CUDA stream, feature tensors must be CUDA fp32 (there is no CPU path),
// and the backward entry points exist only to fail with a clear message (inference only).
#include <torch/extension.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <cuda_runtime.h>

#include <stdexcept>
#include <string>

#include "insconv_b200.h"

namespace {

int g_precision = SCN_PREC_FP32;

void check(int status, const char *what) {
  if (status != SCN_OK)
    throw std::runtime_error(std::string(what) + ": " + scn_last_error() + " (status " + std::to_string(status) + ")");
}

void *stream_of(const at::Tensor &t) { return (void *)c10::cuda::getCurrentCUDAStream(t.device().index()).stream(); }

void need_cuda_f32(const at::Tensor &t, const char *name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor (this build has no CPU path)");
  TORCH_CHECK(t.scalar_type() == at::kFloat, name, " must be float32");
}

// A tensor that may be empty ("no bias"): when it has elements they must be CUDA float32 and `count` long, so that a
// module left on the CPU or built for other planes raises here instead of handing a bad pointer to a kernel.
void need_opt_cuda_f32(const at::Tensor &t, int64_t count, const char *name) {
  if (!t.defined() || t.numel() == 0) return;
  need_cuda_f32(t, name);
  TORCH_CHECK(t.numel() == count && t.is_contiguous(), name, " must hold ", count, " contiguous values; got ", t.numel());
}

// Feature rows must live on the sites the operator indexes them by: [rows of that grid, planes the weights take].
void need_rows(const at::Tensor &t, int64_t rows, int64_t planes, const char *name) {
  TORCH_CHECK(rows >= 0, name, ": Metadata has no grid at the spatial size these features are said to live on");
  TORCH_CHECK(t.dim() == 2 && t.size(0) == rows && t.size(1) == planes, name, " must be [", rows, ", ", planes, "]; got [",
              t.dim() == 2 ? t.size(0) : -1, ", ", t.dim() == 2 ? t.size(1) : -1, "]");
}

// Feature rows handed to a convolution: fp32, or fp16 as written by a BatchNorm in front of it ('fp16' precision).
// With fp16 rows the caller must hand in the matching fp16 weight pack (pack_weights_f16).
struct FeatArg {
  at::Tensor t;
  const float *ptr;
  bool half;
  FeatArg(const at::Tensor &x, const char *name) {
    TORCH_CHECK(x.is_cuda(), name, " must be a CUDA tensor (this build has no CPU path)");
    half = x.scalar_type() == at::kHalf;
    TORCH_CHECK(half || x.scalar_type() == at::kFloat, name, " must be float32 (or float16 rows from a BatchNorm)");
    t = x.contiguous();
    ptr = half ? reinterpret_cast<const float *>(t.data_ptr<at::Half>()) : t.data_ptr<float>();
  }
};

struct Size3 {
  int64_t v[3];
  explicit Size3(const at::Tensor &t) {
    TORCH_CHECK(t.numel() == 3, "only dimension 3 is supported; got a size of ", t.numel(), " elements");
    if (t.device().is_cpu() && t.scalar_type() == at::kLong && t.is_contiguous()) {
      for (int i = 0; i < 3; ++i) v[i] = t.data_ptr<int64_t>()[i];  // the usual case: no temporary tensor
    } else {
      auto c = t.to(at::kCPU, at::kLong).contiguous();
      for (int i = 0; i < 3; ++i) v[i] = c.data_ptr<int64_t>()[i];
    }
  }
};

const float *opt_ptr(const at::Tensor &t) { return t.numel() ? t.data_ptr<float>() : nullptr; }

void expect_filter(const at::Tensor &filt, int64_t want, const char *what) {
  if (filt.device().is_cpu() && filt.scalar_type() == at::kLong && filt.is_contiguous()) {
    for (int64_t i = 0; i < filt.numel(); ++i)
      TORCH_CHECK(filt.data_ptr<int64_t>()[i] == want, what, ": only filter size / stride ", want, " is supported");
    return;
  }
  auto c = filt.to(at::kCPU, at::kLong);
  for (int64_t i = 0; i < c.numel(); ++i)
    TORCH_CHECK(c.data_ptr<int64_t>()[i] == want, what, ": only filter size / stride ", want, " is supported");
}

// Weights for a convolution call: the caller's packed copy (made once by pack_weights) when the tensor-core
// path is selected and a matching copy was handed in, else the plain weights.
struct WeightArg {
  const float *ptr;
  int precision;
  WeightArg(const at::Tensor &w, const at::Tensor &packed, bool half_rows = false) {
    if (half_rows) {
      const int64_t vol = w.dim() == 3 ? w.size(0) : 1;
      TORCH_CHECK(packed.defined() && packed.is_cuda() && packed.scalar_type() == at::kHalf && packed.numel() > 0 &&
                      packed.numel() == scn_packed_size_f16(vol, w.size(w.dim() - 2), w.size(w.dim() - 1)),
                  "float16 feature rows need the float16 weight pack of this layer (pack_weights_f16)");
      ptr = reinterpret_cast<const float *>(packed.data_ptr<at::Half>());
      precision = SCN_PREC_F16;
      return;
    }
    if (g_precision == SCN_PREC_TF32 && packed.defined() && packed.numel() == w.numel() && packed.numel() > 0 &&
        packed.is_cuda() && packed.scalar_type() == at::kFloat) {
      ptr = packed.data_ptr<float>();
      precision = SCN_PREC_TF32_PACKED;
    } else {
      ptr = w.data_ptr<float>();
      precision = g_precision;
    }
  }
};

// The epilogue a convolution call may carry: addend (residual sum) and / or the BatchNorm + ReLU that follows the
// convolution in the network, written as fp16 rows into bn_out (resized here).  All tensors optional.
struct EpiArg {
  scn_epilogue e;
  bool any = false;
  EpiArg(const at::Tensor &addend, const at::Tensor &bn_scale, const at::Tensor &bn_shift, double bn_leak, at::Tensor &bn_out,
         bool skip_raw, int64_t rows, int64_t planes, const at::Tensor &bias) {
    memset(&e, 0, sizeof e);
    if (addend.defined() && addend.numel() > 0) {
      need_cuda_f32(addend, "addend");
      TORCH_CHECK(!bias.defined() || bias.numel() == 0, "the fused residual sum takes no bias");
      TORCH_CHECK(addend.dim() == 2 && addend.size(0) == rows && addend.size(1) == planes && addend.stride(1) == 1,
                  "addend must be [nActive, nOut] with unit plane stride");
      e.addend = addend.data_ptr<float>();
      e.addend_stride = addend.stride(0);
      any = true;
    }
    if (bn_scale.defined() && bn_scale.numel() > 0) {
      need_opt_cuda_f32(bn_scale, planes, "bn_scale");
      need_opt_cuda_f32(bn_shift, planes, "bn_shift");
      TORCH_CHECK(bn_shift.defined() && bn_shift.numel() == planes, "bn_shift must match bn_scale");
      TORCH_CHECK(bn_out.defined() && bn_out.scalar_type() == at::kHalf && bn_out.is_cuda(),
                  "bn_out must be a CUDA float16 tensor (it is resized here)");
      bn_out.resize_({rows, planes});
      e.bn_scale = bn_scale.data_ptr<float>();
      e.bn_shift = bn_shift.data_ptr<float>();
      e.bn_leakiness = bn_leak;
      e.bn_out = bn_out.data_ptr<at::Half>();
      e.bn_out_stride = planes;
      e.skip_raw = skip_raw ? 1 : 0;
      any = true;
    } else {
      TORCH_CHECK(!skip_raw, "skip_raw needs a fused BatchNorm output");
    }
  }
  // incremental form of the fused BatchNorm: the rows the saved frame's BatchNorm read (fp32) and wrote (fp16)
  void saved_rows(const at::Tensor &pre_in, const at::Tensor &pre_out, int64_t saved_rows_count, int64_t planes) {
    if (!e.bn_out) return;
    TORCH_CHECK(pre_in.defined() && pre_in.is_cuda() && pre_in.scalar_type() == at::kFloat && pre_in.dim() == 2 &&
                    pre_in.size(0) == saved_rows_count && pre_in.size(1) == planes && pre_in.stride(1) == 1,
                "bn_pre_in must be the saved float32 rows [saved sites, nOut]");
    TORCH_CHECK(pre_out.defined() && pre_out.is_cuda() && pre_out.scalar_type() == at::kHalf && pre_out.dim() == 2 &&
                    pre_out.size(0) == saved_rows_count && pre_out.size(1) == planes && pre_out.stride(1) == 1,
                "bn_pre_out must be the saved float16 rows [saved sites, nOut]");
    e.bn_pre_in = pre_in.data_ptr<float>();
    e.bn_pre_in_stride = pre_in.stride(0);
    e.bn_pre_out = pre_out.data_ptr<at::Half>();
    e.bn_pre_out_stride = pre_out.stride(0);
  }
  const scn_epilogue *get() const { return any ? &e : nullptr; }
};

class Metadata3 {
 public:
  Metadata3() { check(scn_metadata_create(&h_), "Metadata"); }
  ~Metadata3() { scn_metadata_destroy(h_); }
  Metadata3(const Metadata3 &) = delete;
  Metadata3 &operator=(const Metadata3 &) = delete;
  scn_metadata *h() const { return h_; }

  void clear() { check(scn_metadata_clear(h_, nullptr), "Metadata.clear"); }
  at::Tensor getSpatialLocations(at::Tensor spatialSize) {
    Size3 s(spatialSize);
    int64_t n = scn_metadata_n_active(h_, s.v);
    TORCH_CHECK(n >= 0, "Metadata has no grid at this spatial size");
    auto out = at::empty({n, 4}, at::TensorOptions().dtype(at::kLong).device(at::kCPU));
    check(scn_metadata_spatial_locations(h_, s.v, out.data_ptr<int64_t>(), (void *)c10::cuda::getCurrentCUDAStream().stream()),
          "getSpatialLocations");
    return out;
  }
  // int32 CUDA tensor [4, n]: x, y, z, batch of every site in row order, without leaving the device
  at::Tensor getSpatialLocationsDevice(at::Tensor spatialSize) {
    Size3 s(spatialSize);
    const int32_t *coords = nullptr;
    int64_t n = 0;
    check(scn_metadata_site_coords(h_, s.v, &coords, &n), "getSpatialLocationsDevice");
    auto out = at::empty({4, n}, at::TensorOptions().dtype(at::kInt).device(at::kCUDA));
    if (n) {
      auto stream = c10::cuda::getCurrentCUDAStream().stream();
      TORCH_CHECK(cudaMemcpyAsync(out.data_ptr<int>(), coords, (size_t)n * 16, cudaMemcpyDeviceToDevice, stream) ==
                      cudaSuccess,
                  "getSpatialLocationsDevice: copy failed");
    }
    return out;
  }
  int64_t getNActive(at::Tensor spatialSize) {
    Size3 s(spatialSize);
    return scn_metadata_n_active(h_, s.v);
  }
  // what the next InputLayer build on this object builds beyond the input scale / what the network then asked for
  void setBuildAhead(int neighbour_maps, int coarse_levels) {
    check(scn_metadata_set_build_ahead(h_, neighbour_maps, coarse_levels), "Metadata.setBuildAhead");
  }
  // row lists [4][cap] and their lengths [4] (CUDA int64) of the planes next to a slab's cuts: scn_halo_plane_lists
  std::pair<at::Tensor, at::Tensor> haloPlaneLists(at::Tensor spatialSize, int64_t lo, int64_t hi, bool left, bool right, int64_t cap) {
    Size3 s(spatialSize);
    auto opts = at::TensorOptions().dtype(at::kLong).device(at::kCUDA);
    auto lists = at::empty({4, cap}, opts), counts = at::empty({4}, opts);
    check(scn_halo_plane_lists(h_, s.v, (int)lo, (int)hi, left ? 1 : 0, right ? 1 : 0, cap, lists.data_ptr<int64_t>(),
                               counts.data_ptr<int64_t>(), (void *)c10::cuda::getCurrentCUDAStream().stream()),
          "Metadata.haloPlaneLists");
    return {lists, counts};
  }
  void setSiteCounts(at::Tensor counts) {
    TORCH_CHECK(counts.is_cuda() && counts.scalar_type() == at::kInt && counts.dim() == 1, "counts must be a CUDA int32 vector");
    auto c = counts.contiguous();
    check(scn_input_layer_set_site_counts(h_, c.data_ptr<int>(), c.numel(), (void *)c10::cuda::getCurrentCUDAStream().stream()),
          "Metadata.setSiteCounts");
  }
  void inherit(Metadata3 &previous) { check(scn_metadata_inherit(h_, previous.h()), "Metadata.inherit"); }
  std::pair<int, int> buildUsed() {
    int nm = 0, levels = 0;
    check(scn_metadata_build_used(h_, &nm, &levels), "Metadata.buildUsed");
    return {nm, levels};
  }

 private:
  scn_metadata *h_ = nullptr;
};

// ---- full-frame ops ------------------------------------------------------------------------------
double SubmanifoldConvolution_updateOutput(at::Tensor inputSize, at::Tensor filterSize, Metadata3 &m,
                                           at::Tensor input_features, at::Tensor output_features, at::Tensor weight,
                                           at::Tensor bias, int dilated_rate, at::Tensor packed, at::Tensor addend,
                                           at::Tensor bn_scale, at::Tensor bn_shift, double bn_leak, at::Tensor bn_out,
                                           bool skip_raw) {
  FeatArg fa(input_features, "input_features");
  need_cuda_f32(weight, "weight");
  TORCH_CHECK(dilated_rate == 1, "dilated submanifold convolutions are outside the hot path");
  TORCH_CHECK(weight.dim() == 3 && weight.size(0) == 27, "weight must be [27, nIn, nOut]");
  expect_filter(filterSize, 3, "SubmanifoldConvolution");
  c10::cuda::CUDAGuard guard(input_features.device());
  Size3 s(inputSize);
  const at::Tensor &in = fa.t;
  auto w = weight.contiguous();
  const int64_t n = scn_metadata_n_active(m.h(), s.v);
  TORCH_CHECK(n >= 0, "Metadata has no grid at this spatial size");
  need_rows(in, n, w.size(1), "input_features");
  need_opt_cuda_f32(bias, w.size(2), "bias");
  EpiArg epi(addend, bn_scale, bn_shift, bn_leak, bn_out, skip_raw, n, w.size(2), bias);
  if (!skip_raw) output_features.resize_({n, w.size(2)});
  double flops = 0;
  WeightArg wa(w, packed, fa.half);
  check(scn_ssc_forward_ex(m.h(), s.v, fa.ptr, in.size(1), skip_raw ? nullptr : output_features.data_ptr<float>(), w.size(2),
                           wa.ptr, opt_ptr(bias), w.size(1), w.size(2), wa.precision, epi.get(), stream_of(in), &flops),
        "SubmanifoldConvolution_updateOutput");
  return flops;
}

static double convolution_impl(at::Tensor inputSize, at::Tensor outputSize, at::Tensor filterSize, at::Tensor filterStride,
                               Metadata3 &m, at::Tensor input_features, at::Tensor output_features, at::Tensor weight,
                               at::Tensor bias, at::Tensor packed, at::Tensor bn_scale, at::Tensor bn_shift, double bn_leak,
                               at::Tensor bn_out, bool skip_raw, Metadata3 *pre_m, at::Tensor bn_pre_in, at::Tensor bn_pre_out) {
  FeatArg fa(input_features, "input_features");
  need_cuda_f32(weight, "weight");
  expect_filter(filterSize, 2, "Convolution");
  expect_filter(filterStride, 2, "Convolution");
  TORCH_CHECK(weight.dim() == 3 && weight.size(0) == 8, "weight must be [8, nIn, nOut]");
  c10::cuda::CUDAGuard guard(input_features.device());
  Size3 si(inputSize), so(outputSize);
  const at::Tensor &in = fa.t;
  auto w = weight.contiguous();
  need_rows(in, scn_metadata_n_active(m.h(), si.v), w.size(1), "input_features");
  need_opt_cuda_f32(bias, w.size(2), "bias");
  int64_t n = 0;
  check(scn_conv_prepare(m.h(), si.v, so.v, stream_of(in), &n), "Convolution_updateOutput");
  EpiArg epi(at::Tensor(), bn_scale, bn_shift, bn_leak, bn_out, skip_raw, n, w.size(2), bias);
  if (!skip_raw) output_features.resize_({n, w.size(2)});
  double flops = 0;
  WeightArg wa(w, packed, fa.half);
  if (pre_m && bn_pre_in.defined() && bn_pre_in.numel() > 0) {  // incremental form of the fused BatchNorm
    epi.saved_rows(bn_pre_in, bn_pre_out, scn_metadata_n_active(pre_m->h(), so.v), w.size(2));
    check(scn_incre_conv_forward_ex(m.h(), pre_m->h(), si.v, so.v, fa.ptr, in.size(1), output_features.data_ptr<float>(), w.size(2),
                                    wa.ptr, opt_ptr(bias), w.size(1), w.size(2), wa.precision, epi.get(), stream_of(in), &flops),
          "Incre_Convolution_updateOutput");
    return flops;
  }
  check(scn_conv_forward_ex(m.h(), si.v, so.v, fa.ptr, in.size(1), skip_raw ? nullptr : output_features.data_ptr<float>(),
                            w.size(2), wa.ptr, opt_ptr(bias), w.size(1), w.size(2), wa.precision, epi.get(),
                            stream_of(in), &flops),
        "Convolution_updateOutput");
  return flops;
}

double Convolution_updateOutput(at::Tensor inputSize, at::Tensor outputSize, at::Tensor filterSize,
                                at::Tensor filterStride, Metadata3 &m, at::Tensor input_features,
                                at::Tensor output_features, at::Tensor weight, at::Tensor bias, at::Tensor packed,
                                at::Tensor bn_scale, at::Tensor bn_shift, double bn_leak, at::Tensor bn_out, bool skip_raw) {
  return convolution_impl(inputSize, outputSize, filterSize, filterStride, m, input_features, output_features, weight, bias, packed,
                          bn_scale, bn_shift, bn_leak, bn_out, skip_raw, nullptr, at::Tensor(), at::Tensor());
}

double Deconvolution_updateOutput(at::Tensor inputSize, at::Tensor outputSize, at::Tensor filterSize,
                                  at::Tensor filterStride, Metadata3 &m, at::Tensor input_features,
                                  at::Tensor output_features, at::Tensor weight, at::Tensor bias, at::Tensor packed) {
  FeatArg fa(input_features, "input_features");
  need_cuda_f32(weight, "weight");
  expect_filter(filterSize, 2, "Deconvolution");
  expect_filter(filterStride, 2, "Deconvolution");
  c10::cuda::CUDAGuard guard(input_features.device());
  Size3 si(inputSize), so(outputSize);
  const at::Tensor &in = fa.t;
  auto w = weight.contiguous();
  const int64_t n = scn_metadata_n_active(m.h(), so.v);
  TORCH_CHECK(n >= 0, "Deconvolution: Metadata has no grid at the output spatial size");
  TORCH_CHECK(weight.dim() == 3 && weight.size(0) == 8, "weight must be [8, nIn, nOut]");
  need_rows(in, scn_metadata_n_active(m.h(), si.v), w.size(1), "input_features");
  need_opt_cuda_f32(bias, w.size(2), "bias");
  output_features.resize_({n, w.size(2)});
  double flops = 0;
  WeightArg wa(w, packed, fa.half);
  check(scn_deconv_forward(m.h(), si.v, so.v, fa.ptr, in.size(1), output_features.data_ptr<float>(),
                           w.size(2), wa.ptr, opt_ptr(bias), w.size(1), w.size(2), wa.precision,
                           stream_of(in), &flops),
        "Deconvolution_updateOutput");
  return flops;
}

void BatchNormalization_updateOutput(at::Tensor input_features, at::Tensor output_features, at::Tensor saveMean,
                                     at::Tensor saveInvStd, at::Tensor runningMean, at::Tensor runningVar,
                                     at::Tensor weight, at::Tensor bias, double eps, double momentum, bool train,
                                     double leakiness) {
  need_cuda_f32(input_features, "input_features");
  TORCH_CHECK(input_features.dim() == 2, "input_features must be [rows, planes]");
  need_cuda_f32(runningMean, "runningMean");
  need_cuda_f32(runningVar, "runningVar");
  need_opt_cuda_f32(runningMean, input_features.size(1), "runningMean");
  need_opt_cuda_f32(runningVar, input_features.size(1), "runningVar");
  need_opt_cuda_f32(weight, input_features.size(1), "weight");
  need_opt_cuda_f32(bias, input_features.size(1), "bias");
  c10::cuda::CUDAGuard guard(input_features.device());
  auto in = input_features.contiguous();
  if (output_features.scalar_type() == at::kHalf) {  // fp16 rows for the convolution that follows ('fp16' precision)
    TORCH_CHECK(!train, "float16 BatchNorm output is for inference with running statistics");
    output_features.resize_(in.sizes());
    if (in.numel() == 0) return;
    check(scn_bn_forward_f16(in.data_ptr<float>(), in.size(1), output_features.data_ptr<at::Half>(), in.size(1), in.size(0),
                             in.size(1), runningMean.data_ptr<float>(), runningVar.data_ptr<float>(), opt_ptr(weight),
                             opt_ptr(bias), eps, leakiness, stream_of(in)),
          "BatchNormalization_updateOutput");
    return;
  }
  output_features.resize_as_(in);
  if (in.numel() == 0) return;
  if (train) {  // batch statistics, running statistics updated in place (what demo.py exercises on its first frame)
    saveMean.resize_({in.size(1)});
    saveInvStd.resize_({in.size(1)});
    check(scn_bn_forward_train(in.data_ptr<float>(), in.size(1), output_features.data_ptr<float>(), in.size(1), in.size(0),
                               in.size(1), runningMean.data_ptr<float>(), runningVar.data_ptr<float>(),
                               saveMean.data_ptr<float>(), saveInvStd.data_ptr<float>(), opt_ptr(weight), opt_ptr(bias),
                               eps, momentum, leakiness, stream_of(in)),
          "BatchNormalization_updateOutput");
    return;
  }
  check(scn_bn_forward(in.data_ptr<float>(), in.size(1), output_features.data_ptr<float>(), in.size(1), in.size(0),
                       in.size(1), runningMean.data_ptr<float>(), runningVar.data_ptr<float>(), opt_ptr(weight),
                       opt_ptr(bias), eps, leakiness, stream_of(in)),
        "BatchNormalization_updateOutput");
}

// JoinTable of two tensors followed by the inference BatchNorm + leaky ReLU that consumes it, in one pass ('fp16'
// precision): joined <- [a | b] (float32), rows <- activation(joined * scale + shift) (float16)
void JoinTable_BatchNormalization_updateOutput(at::Tensor a, at::Tensor b, at::Tensor joined, at::Tensor scale, at::Tensor shift,
                                               double leakiness, at::Tensor rows) {
  need_cuda_f32(a, "a");
  need_cuda_f32(b, "b");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.size(0) == b.size(0), "a and b must be [rows, planes] on the same rows");
  const int64_t planes = a.size(1) + b.size(1);
  need_opt_cuda_f32(scale, planes, "scale");
  need_opt_cuda_f32(shift, planes, "shift");
  TORCH_CHECK(scale.numel() == planes && shift.numel() == planes, "scale and shift must have one entry per joined plane");
  TORCH_CHECK(joined.scalar_type() == at::kFloat && rows.scalar_type() == at::kHalf, "joined must be float32 and rows float16");
  c10::cuda::CUDAGuard guard(a.device());
  auto ac = a.contiguous(), bc = b.contiguous();
  joined.resize_({a.size(0), planes});
  rows.resize_({a.size(0), planes});
  if (a.size(0) == 0) return;
  check(scn_join_bn_forward_f16(ac.data_ptr<float>(), ac.size(1), ac.size(1), bc.data_ptr<float>(), bc.size(1), bc.size(1), ac.size(0),
                                joined.data_ptr<float>(), planes, scale.data_ptr<float>(), shift.data_ptr<float>(), leakiness,
                                rows.data_ptr<at::Half>(), planes, stream_of(ac)),
        "JoinTable_BatchNormalization_updateOutput");
}

double NetworkInNetwork_updateOutput(at::Tensor input_features, at::Tensor output_features, at::Tensor weight,
                                     at::Tensor bias, at::Tensor packed) {
  need_cuda_f32(input_features, "input_features");
  need_cuda_f32(weight, "weight");
  c10::cuda::CUDAGuard guard(input_features.device());
  auto in = input_features.contiguous();
  auto w = weight.contiguous();
  TORCH_CHECK(w.dim() == 2, "weight must be [nIn, nOut]");
  need_rows(in, in.dim() == 2 ? in.size(0) : -1, w.size(0), "input_features");
  need_opt_cuda_f32(bias, w.size(1), "bias");
  output_features.resize_({in.size(0), w.size(1)});
  double flops = 0;
  WeightArg wa(w, packed);
  check(scn_nin_forward(in.data_ptr<float>(), in.size(1), output_features.data_ptr<float>(), w.size(1), in.size(0),
                        wa.ptr, opt_ptr(bias), w.size(0), w.size(1), wa.precision, stream_of(in), &flops),
        "NetworkInNetwork_updateOutput");
  return flops;
}

// coords may be a CPU or a CUDA LongTensor [N,3] or [N,4]; a CUDA tensor is used in place (no bounce
// through the host).
// Grid builds on a stream of their own (overlap_grid_build): the site ranking and the coarse scales of frame t + 1 depend
// on that frame's coordinates only, so they can run while the last layers of frame t are still on the GPU, instead of
// behind them; the host, which waits for the site counts, is then not held up by frame t either.
struct BuildOverlap {
  bool on = false;
  int device = -1;
  cudaStream_t side = nullptr;
  cudaEvent_t inputs_ready = nullptr, built = nullptr;
};
BuildOverlap g_build_overlap;

// on: records "the inputs of the frames that follow are ready" on the current stream (the builds wait for that event,
// not for the stream's later work) and moves the builds of InputLayer_updateOutput to a side stream; off: back to the
// current stream.  The caller promises that coordinates handed over while this is on are complete at that event (inputs
// resident in device memory, or call again after queueing their copies).
void overlap_grid_build(bool on) {
  BuildOverlap &o = g_build_overlap;
  if (!on) {
    o.on = false;
    return;
  }
  int dev = 0;
  TORCH_CHECK(cudaGetDevice(&dev) == cudaSuccess, "overlap_grid_build: no CUDA device");
  if (o.device != dev) {
    TORCH_CHECK(o.device < 0, "overlap_grid_build serves one device per process");
    TORCH_CHECK(cudaStreamCreateWithFlags(&o.side, cudaStreamNonBlocking) == cudaSuccess &&
                    cudaEventCreateWithFlags(&o.inputs_ready, cudaEventDisableTiming) == cudaSuccess &&
                    cudaEventCreateWithFlags(&o.built, cudaEventDisableTiming) == cudaSuccess,
                "overlap_grid_build: could not create the side stream");
    o.device = dev;
  }
  TORCH_CHECK(cudaEventRecord(o.inputs_ready, c10::cuda::getCurrentCUDAStream(dev).stream()) == cudaSuccess,
              "overlap_grid_build: could not record the event");
  o.on = true;
}

void build_input(Metadata3 &m, at::Tensor spatialSize, at::Tensor input_coords, const at::Tensor &feats,
                 long batchSize, long mode, bool may_overlap = false) {
  TORCH_CHECK(input_coords.dim() == 2 && (input_coords.size(1) == 3 || input_coords.size(1) == 4),
              "coords must be N x 3 or N x 4");
  Size3 s(spatialSize);
  auto c = input_coords.to(at::kLong).contiguous();
  TORCH_CHECK(c.size(0) == feats.size(0), "coords and features disagree on the number of points");
  int64_t n = 0;
  const BuildOverlap &o = g_build_overlap;
  // only coordinates that are used as they are (no conversion queued on the current stream just now)
  const bool overlap = may_overlap && o.on && c.is_cuda() && c.is_same(input_coords) && c.device().index() == o.device;
  if (overlap) {
    cudaStream_t main = c10::cuda::getCurrentCUDAStream(o.device).stream();
    TORCH_CHECK(cudaStreamWaitEvent(o.side, o.inputs_ready, 0) == cudaSuccess, "InputLayer_updateOutput: stream wait failed");
    check(scn_input_layer_build(m.h(), s.v, c.data_ptr<int64_t>(), 0, c.size(0), (int)c.size(1), batchSize, (int)mode,
                                (void *)o.side, &n),
          "InputLayer_updateOutput");
    // the layers run on the current stream: behind the build
    TORCH_CHECK(cudaEventRecord(o.built, o.side) == cudaSuccess && cudaStreamWaitEvent(main, o.built, 0) == cudaSuccess,
                "InputLayer_updateOutput: stream wait failed");
    return;
  }
  check(scn_input_layer_build(m.h(), s.v, c.data_ptr<int64_t>(), c.is_cuda() ? 0 : 1, c.size(0), (int)c.size(1),
                              batchSize, (int)mode, stream_of(feats), &n),
        "InputLayer_updateOutput");
}

void InputLayer_updateOutput(Metadata3 &m, at::Tensor spatialSize, at::Tensor input_coords, at::Tensor input_features,
                             at::Tensor output_features, long batchSize, long mode) {
  need_cuda_f32(input_features, "input_features");
  c10::cuda::CUDAGuard guard(input_features.device());
  auto in = input_features.contiguous();
  build_input(m, spatialSize, input_coords, in, batchSize, mode, true);
  Size3 s(spatialSize);
  output_features.resize_({scn_metadata_n_active(m.h(), s.v), in.size(1)});
  check(scn_input_layer_forward(m.h(), in.data_ptr<float>(), output_features.data_ptr<float>(), in.size(1),
                                stream_of(in)),
        "InputLayer_updateOutput");
}

void OutputLayer_updateOutput(Metadata3 &m, at::Tensor input_features, at::Tensor output_features) {
  need_cuda_f32(input_features, "input_features");
  c10::cuda::CUDAGuard guard(input_features.device());
  auto in = input_features.contiguous();
  const int64_t n = scn_input_layer_n_points(m.h());
  TORCH_CHECK(n >= 0, "OutputLayer: Metadata has no input layer");
  TORCH_CHECK(in.dim() == 2 && in.size(0) == scn_metadata_input_n_active(m.h()),
              "input_features must have one row per site of the input scale");
  output_features.resize_({n, in.size(1)});
  check(scn_output_layer_forward(m.h(), in.data_ptr<float>(), output_features.data_ptr<float>(), in.size(1),
                                 stream_of(in)),
        "OutputLayer_updateOutput");
}

// ---- incremental ops -----------------------------------------------------------------------------
double Incre_SubmanifoldConvolution_updateOutput(at::Tensor inputSize, at::Tensor filterSize, Metadata3 &m,
                                                 at::Tensor input_features, at::Tensor output_features,
                                                 at::Tensor weight, at::Tensor bias, Metadata3 &pre_m,
                                                 at::Tensor pre_input_feats, at::Tensor packed, at::Tensor addend,
                                                 at::Tensor bn_scale, at::Tensor bn_shift, double bn_leak, at::Tensor bn_out,
                                                 at::Tensor bn_pre_in, at::Tensor bn_pre_out) {
  // fp32 residual rows with fp32 saved rows, or ('fp16' precision) both as fp16 rows with the fp16 weight pack
  FeatArg fin(input_features, "input_features"), fpre(pre_input_feats, "pre_input_feats");
  TORCH_CHECK(fin.half == fpre.half, "residual rows and saved rows must have the same type (both float32 or both float16)");
  expect_filter(filterSize, 3, "SubmanifoldConvolution");
  c10::cuda::CUDAGuard guard(input_features.device());
  Size3 s(inputSize);
  const at::Tensor &in = fin.t, &pre = fpre.t;
  auto w = weight.contiguous();
  const int64_t n = scn_metadata_n_active(m.h(), s.v);
  TORCH_CHECK(n >= 0, "Metadata has no grid at this spatial size");
  need_cuda_f32(weight, "weight");
  TORCH_CHECK(w.dim() == 3 && w.size(0) == 27, "weight must be [27, nIn, nOut]");
  need_rows(in, n, w.size(1), "input_features");
  need_rows(pre, scn_metadata_n_active(pre_m.h(), s.v), w.size(1), "pre_input_feats");
  need_opt_cuda_f32(bias, w.size(2), "bias");
  output_features.resize_({n, w.size(2)});
  double flops = 0;
  WeightArg wa(w, packed, fin.half);
  EpiArg epi(addend, bn_scale, bn_shift, bn_leak, bn_out, false, n, w.size(2), bias);
  epi.saved_rows(bn_pre_in, bn_pre_out, scn_metadata_n_active(pre_m.h(), s.v), w.size(2));
  check(scn_incre_ssc_forward_ex(m.h(), pre_m.h(), s.v, fin.ptr, in.size(1),
                                 output_features.data_ptr<float>(), w.size(2), wa.ptr, opt_ptr(bias),
                                 fpre.ptr, pre.size(1), w.size(1), w.size(2), wa.precision, epi.get(), stream_of(in),
                                 &flops),
        "Incre_SubmanifoldConvolution_updateOutput");
  return flops;
}

double Incre_Convolution_updateOutput(at::Tensor inputSize, at::Tensor outputSize, at::Tensor filterSize,
                                      at::Tensor filterStride, Metadata3 &m, at::Tensor input_features,
                                      at::Tensor output_features, at::Tensor weight, at::Tensor bias, at::Tensor packed,
                                      pybind11::object pre_m, at::Tensor bn_scale, at::Tensor bn_shift, double bn_leak,
                                      at::Tensor bn_out, at::Tensor bn_pre_in, at::Tensor bn_pre_out) {
  // a 2/2 convolution has no overlap between cells: the residual of the output is the convolution of
  // the residual (reference: CUDA/Convolution.cpp:83-113).  With pre_m and the saved rows, the incremental BatchNorm
  // behind the layer is formed in the epilogue.
  Metadata3 *pm = pre_m.is_none() ? nullptr : pre_m.cast<Metadata3 *>();
  return convolution_impl(inputSize, outputSize, filterSize, filterStride, m, input_features, output_features, weight, bias, packed,
                          bn_scale, bn_shift, bn_leak, bn_out, false, pm, bn_pre_in, bn_pre_out);
}

double Incre_Deconvolution_updateOutput(at::Tensor inputSize, at::Tensor outputSize, at::Tensor filterSize,
                                        at::Tensor filterStride, Metadata3 &m, at::Tensor input_features,
                                        at::Tensor output_features, at::Tensor weight, at::Tensor bias,
                                        Metadata3 &pre_m, at::Tensor pre_input_feats, at::Tensor packed) {
  FeatArg fin(input_features, "input_features"), fpre(pre_input_feats, "pre_input_feats");
  TORCH_CHECK(fin.half == fpre.half, "residual rows and saved rows must have the same type (both float32 or both float16)");
  c10::cuda::CUDAGuard guard(input_features.device());
  Size3 si(inputSize), so(outputSize);
  const at::Tensor &in = fin.t, &pre = fpre.t;
  auto w = weight.contiguous();
  const int64_t n = scn_metadata_n_active(m.h(), so.v);
  TORCH_CHECK(n >= 0, "Deconvolution: Metadata has no grid at the output spatial size");
  need_cuda_f32(weight, "weight");
  TORCH_CHECK(w.dim() == 3 && w.size(0) == 8, "weight must be [8, nIn, nOut]");
  need_rows(in, scn_metadata_n_active(m.h(), si.v), w.size(1), "input_features");
  need_rows(pre, scn_metadata_n_active(pre_m.h(), si.v), w.size(1), "pre_input_feats");
  need_opt_cuda_f32(bias, w.size(2), "bias");
  output_features.resize_({n, w.size(2)});
  double flops = 0;
  WeightArg wa(w, packed, fin.half);
  check(scn_incre_deconv_forward(m.h(), pre_m.h(), si.v, so.v, fin.ptr, in.size(1),
                                 output_features.data_ptr<float>(), w.size(2), wa.ptr, opt_ptr(bias),
                                 fpre.ptr, pre.size(1), w.size(1), w.size(2), wa.precision, stream_of(in),
                                 &flops),
        "Incre_Deconvolution_updateOutput");
  return flops;
}

void Incre_BatchNormalization_updateOutput(at::Tensor input_features, at::Tensor output_features, at::Tensor saveMean,
                                           at::Tensor saveInvStd, at::Tensor runningMean, at::Tensor runningVar,
                                           at::Tensor weight, at::Tensor bias, double eps, double momentum, bool train,
                                           double leakiness, Metadata3 &m, Metadata3 &pre_m,
                                           at::Tensor pre_output_feats, at::Tensor pre_input_feats,
                                           at::Tensor spatialSize) {
  need_cuda_f32(input_features, "input_features");
  (void)train;  // the incremental form always uses the running statistics (CUDA/BatchNormalization.cu:181-195)
  c10::cuda::CUDAGuard guard(input_features.device());
  Size3 s(spatialSize);
  auto in = input_features.contiguous();
  auto po = pre_output_feats.contiguous();
  auto pi = pre_input_feats.contiguous();
  // 'fp16' precision: an output tensor of type float16 asks for the residual as fp16 rows; the saved output then is
  // the fp16 tensor the saved frame's BatchNorm wrote
  const bool half_out = output_features.scalar_type() == at::kHalf;
  if (half_out) {
    TORCH_CHECK(po.is_cuda() && po.scalar_type() == at::kHalf, "pre_output_feats must be the saved float16 rows");
  } else {
    need_cuda_f32(po, "pre_output_feats");
  }
  need_cuda_f32(pi, "pre_input_feats");
  TORCH_CHECK(in.dim() == 2, "input_features must be [rows, planes]");
  need_rows(in, scn_metadata_n_active(m.h(), s.v), in.size(1), "input_features");
  need_rows(po, scn_metadata_n_active(pre_m.h(), s.v), in.size(1), "pre_output_feats");
  need_rows(pi, scn_metadata_n_active(pre_m.h(), s.v), in.size(1), "pre_input_feats");
  need_cuda_f32(runningMean, "runningMean");
  need_cuda_f32(runningVar, "runningVar");
  need_opt_cuda_f32(runningMean, in.size(1), "runningMean");
  need_opt_cuda_f32(runningVar, in.size(1), "runningVar");
  need_opt_cuda_f32(weight, in.size(1), "weight");
  need_opt_cuda_f32(bias, in.size(1), "bias");
  output_features.resize_(in.sizes());
  if (in.numel() == 0) return;
  if (half_out) {
    check(scn_incre_bn_forward_f16(m.h(), pre_m.h(), s.v, in.data_ptr<float>(), in.size(1), output_features.data_ptr<at::Half>(),
                                   in.size(1), in.size(1), runningMean.data_ptr<float>(), runningVar.data_ptr<float>(),
                                   opt_ptr(weight), opt_ptr(bias), eps, leakiness, po.data_ptr<at::Half>(), po.size(1),
                                   pi.data_ptr<float>(), pi.size(1), stream_of(in)),
          "Incre_BatchNormalization_updateOutput");
    return;
  }
  check(scn_incre_bn_forward(m.h(), pre_m.h(), s.v, in.data_ptr<float>(), in.size(1),
                             output_features.data_ptr<float>(), in.size(1), in.size(1), runningMean.data_ptr<float>(),
                             runningVar.data_ptr<float>(), opt_ptr(weight), opt_ptr(bias), eps, leakiness,
                             po.data_ptr<float>(), pi.data_ptr<float>(), stream_of(in)),
        "Incre_BatchNormalization_updateOutput");
}

void Incre_InputLayer_updateOutput(Metadata3 &m, at::Tensor spatialSize, at::Tensor input_coords,
                                   at::Tensor input_features, at::Tensor output_features, long batchSize, long mode,
                                   Metadata3 &pre_m, at::Tensor pre_output_feats) {
  need_cuda_f32(input_features, "input_features");
  need_cuda_f32(pre_output_feats, "pre_output_feats");
  c10::cuda::CUDAGuard guard(input_features.device());
  auto in = input_features.contiguous();
  auto po = pre_output_feats.contiguous();
  build_input(m, spatialSize, input_coords, in, batchSize, mode);
  Size3 s(spatialSize);
  need_rows(po, scn_metadata_n_active(pre_m.h(), s.v), in.size(1), "pre_output_feats");
  output_features.resize_({scn_metadata_n_active(m.h(), s.v), in.size(1)});
  check(scn_incre_input_layer_forward(m.h(), pre_m.h(), in.data_ptr<float>(), output_features.data_ptr<float>(),
                                      po.data_ptr<float>(), in.size(1), stream_of(in)),
        "Incre_InputLayer_updateOutput");
}

void Incre_OutputLayer_updateOutput(Metadata3 &m, at::Tensor input_features, at::Tensor output_features,
                                    Metadata3 &pre_m, at::Tensor pre_input_feats) {
  need_cuda_f32(input_features, "input_features");
  need_cuda_f32(pre_input_feats, "pre_input_feats");
  c10::cuda::CUDAGuard guard(input_features.device());
  auto in = input_features.contiguous();
  auto pi = pre_input_feats.contiguous();
  const int64_t n = scn_input_layer_n_points(m.h());
  TORCH_CHECK(n >= 0, "OutputLayer: Metadata has no input layer");
  TORCH_CHECK(in.dim() == 2 && in.size(0) == scn_metadata_input_n_active(m.h()),
              "input_features must have one row per site of the input scale");
  need_rows(pi, scn_metadata_input_n_active(pre_m.h()), in.size(1), "pre_input_feats");
  output_features.resize_({n, in.size(1)});
  check(scn_incre_output_layer_forward(m.h(), pre_m.h(), in.data_ptr<float>(), output_features.data_ptr<float>(),
                                       pi.data_ptr<float>(), in.size(1), stream_of(in)),
        "Incre_OutputLayer_updateOutput");
}

// Transposed copy of a convolution weight for the tensor-core kernels; an empty tensor when the shape is not
// one those kernels take.  weight: [volume, nIn, nOut] or [nIn, nOut].
at::Tensor pack_weights(at::Tensor weight) {
  need_cuda_f32(weight, "weight");
  auto w = weight.contiguous();
  const int64_t vol = w.dim() == 3 ? w.size(0) : 1, n_in = w.size(w.dim() - 2), n_out = w.size(w.dim() - 1);
  if (!scn_weights_packable(vol, n_in, n_out)) return at::empty({0}, w.options());
  c10::cuda::CUDAGuard guard(w.device());
  auto packed = at::empty_like(w);
  check(scn_pack_weights(w.data_ptr<float>(), vol, n_in, n_out, packed.data_ptr<float>(), stream_of(w)), "pack_weights");
  return packed;
}

// fp16 fragments for the convolutions that read fp16 rows (empty when the shape has no fp16 kernel)
at::Tensor pack_weights_f16(at::Tensor weight) {
  need_cuda_f32(weight, "weight");
  auto w = weight.contiguous();
  const int64_t vol = w.dim() == 3 ? w.size(0) : 1, n_in = w.size(w.dim() - 2), n_out = w.size(w.dim() - 1);
  const int64_t size = scn_packed_size_f16(vol, n_in, n_out);
  if (size <= 0) return at::empty({0}, w.options().dtype(at::kHalf));
  c10::cuda::CUDAGuard guard(w.device());
  auto packed = at::empty({size}, w.options().dtype(at::kHalf));
  check(scn_pack_weights_f16(w.data_ptr<float>(), vol, n_in, n_out, packed.data_ptr<at::Half>(), stream_of(w)),
        "pack_weights_f16");
  return packed;
}

// 'fp16' = tf32 kernels, plus fp16 rows between a BatchNorm and a narrow convolution behind it (the Python
// containers arrange that); the extension itself treats it as tf32.
bool g_half_rows = false;
void set_precision(const std::string &p) {
  if (p == "fp32") g_precision = SCN_PREC_FP32;
  else if (p == "tf32" || p == "fp16") g_precision = SCN_PREC_TF32;
  else throw std::runtime_error("precision must be 'fp32', 'tf32' or 'fp16'");
  g_half_rows = p == "fp16";
}
std::string get_precision() { return g_precision == SCN_PREC_TF32 ? (g_half_rows ? "fp16" : "tf32") : "fp32"; }

void no_backward(pybind11::args, pybind11::kwargs) {
  throw std::runtime_error("this build of sparseconvnet.SCN is inference only: backward passes are not part of the hot path");
}


// ---- label fusion (Result_3, ResultOfWeight: sparseconvnet/SCN/pybind.cpp:36-45, 275-282) ------------------------
// Same method names and argument meaning as the reference's classes; points may be CPU or CUDA LongTensors, scores CPU
// or CUDA float tensors (they are moved to the GPU, where the table lives); query results come back as the reference
// returns them, CPU LongTensors.
class LabelTable {
 public:
  // weight_classes < 0: a weight table whose vector length is taken from the first update
  LabelTable(int weight_classes, double maximum) : classes_(weight_classes), maximum_(maximum) {
    if (weight_classes >= 0) check(scn_labels_create(&h_, weight_classes, maximum), "label table");
  }
  ~LabelTable() { scn_labels_destroy(h_); }
  LabelTable(const LabelTable &) = delete;
  LabelTable &operator=(const LabelTable &) = delete;

  void update(at::Tensor ps, at::Tensor label) { apply(ps, label, false); }
  void set(at::Tensor ps, at::Tensor label) {
    if (ps.dim() == 1) {
      ps = ps.unsqueeze(0);
      label = label.unsqueeze(0);
    }
    apply(ps, label, true);
  }
  at::Tensor multiQuery(at::Tensor ps) {
    auto p = points(ps);
    auto out = at::empty({p.size(0)}, p.options());
    if (!h_) return out.fill_(-1).cpu();
    check(scn_labels_query(h_, p.data_ptr<int64_t>(), (int)p.size(1), p.size(0), out.data_ptr<int64_t>(), stream_of(p)),
          "multiQuery");
    sync_status(p);
    return out.cpu();
  }
  int64_t query(at::Tensor p) {
    TORCH_CHECK(p.dim() == 1, "query takes one point");
    return multiQuery(p.unsqueeze(0))[0].item<int64_t>();
  }
  at::Tensor get_all_points_labels() {
    auto opts = at::TensorOptions().dtype(at::kLong).device(at::kCUDA);
    if (!h_) return at::empty({0, 4}, at::TensorOptions().dtype(at::kLong));
    auto stream = (void *)c10::cuda::getCurrentCUDAStream().stream();
    int64_t n = 0;
    check(scn_labels_size(h_, &n, nullptr, stream), "get_all_points_labels");
    auto out = at::empty({n, 4}, opts);
    int64_t written = 0;
    check(scn_labels_dump(h_, out.data_ptr<int64_t>(), n, &written, stream), "get_all_points_labels");
    return out.narrow(0, 0, written).cpu();
  }
  void finalize(at::Tensor ps) {
    if (!h_) return;
    auto p = points(ps);
    check(scn_labels_finalize(h_, p.data_ptr<int64_t>(), (int)p.size(1), p.size(0), stream_of(p)), "finalize");
  }
  void clear() {
    if (h_) check(scn_labels_clear(h_, (void *)c10::cuda::getCurrentCUDAStream().stream()), "clear");
  }
  int64_t size() {
    if (!h_) return 0;
    int64_t n = 0;
    check(scn_labels_size(h_, &n, nullptr, (void *)c10::cuda::getCurrentCUDAStream().stream()), "size");
    return n;
  }
  int64_t rowsAppliedSerially() {
    if (!h_) return 0;
    int64_t n = 0, later = 0;
    check(scn_labels_size(h_, &n, &later, (void *)c10::cuda::getCurrentCUDAStream().stream()), "size");
    return later;
  }

 private:
  static at::Tensor points(const at::Tensor &ps) {
    TORCH_CHECK(ps.dim() == 2 && (ps.size(1) == 3 || ps.size(1) == 4) && ps.scalar_type() == at::kLong,
                "points must be a LongTensor [n, 3] or [n, 4]");
    return ps.to(at::kCUDA).contiguous();
  }
  void apply(const at::Tensor &ps, const at::Tensor &label, bool set) {
    auto p = points(ps);
    TORCH_CHECK(label.dim() == 2 && label.size(0) == p.size(0) && label.size(1) >= 1, "scores must be [n, classes]");
    auto sc = label.to(at::kCUDA, at::kFloat).contiguous();
    if (!h_) {  // weight table: the vector length is that of the first scores seen
      classes_ = (int)sc.size(1);
      check(scn_labels_create(&h_, classes_, maximum_), "label table");
    }
    auto fn = set ? scn_labels_set : scn_labels_update;
    check(fn(h_, p.data_ptr<int64_t>(), (int)p.size(1), p.size(0), sc.data_ptr<float>(), sc.stride(0), sc.size(1), stream_of(p)),
          set ? "set" : "update");
  }
  void sync_status(const at::Tensor &p) {
    int64_t n = 0;
    check(scn_labels_size(h_, &n, nullptr, stream_of(p)), "label table");
  }
  scn_labels *h_ = nullptr;
  int classes_;
  double maximum_;
};

// Result<3>: `int maximum` initialised from a float (resultHash.h:24-29) -- the default 0.7 is held as 0
class Result3 : public LabelTable {
 public:
  Result3() : LabelTable(0, (double)(int)0.7f) {}
  explicit Result3(float maximum) : LabelTable(0, (double)(int)maximum) {}
};
class ResultOfWeight3 : public LabelTable {
 public:
  ResultOfWeight3() : LabelTable(-1, 0.0) {}
};

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, mod) {
  mod.doc() = "B200 sparse-convolution operators behind the sparseconvnet.SCN interface (dimension 3)";
  // default of every optional tensor argument: an empty tensor (the interface's "no bias" convention), so that calls
  // with the reference's own argument lists work as they are
  const at::Tensor none = at::empty({0});
  pybind11::class_<Result3>(mod, "Result_3")
      .def(pybind11::init<>())
      .def(pybind11::init<float>())
      .def("set", &Result3::set)
      .def("query", &Result3::query)
      .def("multiQuery", &Result3::multiQuery)
      .def("clear", &Result3::clear)
      .def("update", &Result3::update)
      .def("get_all_points_labels", &Result3::get_all_points_labels)
      .def("finalize", &Result3::finalize)
      .def("size", &Result3::size)
      .def("rowsAppliedSerially", &Result3::rowsAppliedSerially);
  pybind11::class_<ResultOfWeight3>(mod, "ResultOfWeight")
      .def(pybind11::init<>())
      .def("query", &ResultOfWeight3::query)
      .def("multiQuery", &ResultOfWeight3::multiQuery)
      .def("clear", &ResultOfWeight3::clear)
      .def("update", &ResultOfWeight3::update)
      .def("get_all_points_labels", &ResultOfWeight3::get_all_points_labels)
      .def("finalize", &ResultOfWeight3::finalize)
      .def("size", &ResultOfWeight3::size);
  pybind11::class_<Metadata3>(mod, "Metadata_3")
      .def(pybind11::init<>())
      .def("clear", &Metadata3::clear)
      .def("getSpatialLocations", &Metadata3::getSpatialLocations)
      .def("getSpatialLocationsDevice", &Metadata3::getSpatialLocationsDevice)
      .def("getNActive", &Metadata3::getNActive)
      .def("setBuildAhead", &Metadata3::setBuildAhead)
      .def("buildUsed", &Metadata3::buildUsed)
      .def("inherit", &Metadata3::inherit)
      .def("setSiteCounts", &Metadata3::setSiteCounts)
      .def("haloPlaneLists", &Metadata3::haloPlaneLists)
      // The rest of the reference's Metadata interface (pybind.cpp:16-33).  The two setters only record a value that
      // the sample-by-sample builders below would read; those builders (and the dense / thresholded-tensor entry points)
      // feed the CPU SparseGrid path of the reference, which the GPU-grid hot path never takes: they exist here so that
      // code probing for them finds them, and say what they are when called.
      .def("setInputSpatialSize", [](Metadata3 &, at::Tensor) {})
      .def("setNormalGuideScale", [](Metadata3 &, int64_t) {});
  for (const char *name : {"batchAddSample", "setInputSpatialLocation", "setInputSpatialLocations",
                           "createMetadataForDenseToSparse", "sparsifyMetadata", "appendMetadata", "sparsifyCompare",
                           "addSampleFromThresholdedTensor", "generateRuleBooks3s2", "generateRuleBooks2s2",
                           "compareSparseHelper"}) {
    const std::string what = name;
    pybind11::setattr(mod.attr("Metadata_3"), name,
                      pybind11::cpp_function(
                          [what](pybind11::args, pybind11::kwargs) {
                            throw std::runtime_error("Metadata." + what +
                                                     " belongs to the reference's CPU sparse-grid path, which this build "
                                                     "does not have (scenes enter through InputLayer)");
                          },
                          pybind11::is_method(mod.attr("Metadata_3"))));
  }
  mod.def("SubmanifoldConvolution_updateOutput", &SubmanifoldConvolution_updateOutput, pybind11::arg("inputSize"), pybind11::arg("filterSize"), pybind11::arg("metadata"), pybind11::arg("input_features"), pybind11::arg("output_features"), pybind11::arg("weight"), pybind11::arg("bias"), pybind11::arg("dilated_rate"), pybind11::arg("packed") = none, pybind11::arg("addend") = none, pybind11::arg("bn_scale") = none, pybind11::arg("bn_shift") = none, pybind11::arg("bn_leak") = 0.0, pybind11::arg("bn_out") = none, pybind11::arg("skip_raw") = false);
  mod.def("Convolution_updateOutput", &Convolution_updateOutput, pybind11::arg("inputSize"), pybind11::arg("outputSize"), pybind11::arg("filterSize"), pybind11::arg("filterStride"), pybind11::arg("metadata"), pybind11::arg("input_features"), pybind11::arg("output_features"), pybind11::arg("weight"), pybind11::arg("bias"), pybind11::arg("packed") = none, pybind11::arg("bn_scale") = none, pybind11::arg("bn_shift") = none, pybind11::arg("bn_leak") = 0.0, pybind11::arg("bn_out") = none, pybind11::arg("skip_raw") = false);
  mod.def("Deconvolution_updateOutput", &Deconvolution_updateOutput, pybind11::arg("inputSize"), pybind11::arg("outputSize"), pybind11::arg("filterSize"), pybind11::arg("filterStride"), pybind11::arg("metadata"), pybind11::arg("input_features"), pybind11::arg("output_features"), pybind11::arg("weight"), pybind11::arg("bias"), pybind11::arg("packed") = none);
  mod.def("BatchNormalization_updateOutput", &BatchNormalization_updateOutput);
  mod.def("overlap_grid_build", &overlap_grid_build, pybind11::arg("on"));
  mod.def("JoinTable_BatchNormalization_updateOutput", &JoinTable_BatchNormalization_updateOutput);
  mod.def("NetworkInNetwork_updateOutput", &NetworkInNetwork_updateOutput, pybind11::arg("input_features"), pybind11::arg("output_features"), pybind11::arg("weight"), pybind11::arg("bias"), pybind11::arg("packed") = none);
  mod.def("InputLayer_updateOutput", &InputLayer_updateOutput);
  mod.def("OutputLayer_updateOutput", &OutputLayer_updateOutput);
  mod.def("Incre_SubmanifoldConvolution_updateOutput", &Incre_SubmanifoldConvolution_updateOutput, pybind11::arg("inputSize"), pybind11::arg("filterSize"), pybind11::arg("metadata"), pybind11::arg("input_features"), pybind11::arg("output_features"), pybind11::arg("weight"), pybind11::arg("bias"), pybind11::arg("pre_metadata"), pybind11::arg("pre_input_feats"), pybind11::arg("packed") = none, pybind11::arg("addend") = none, pybind11::arg("bn_scale") = none, pybind11::arg("bn_shift") = none, pybind11::arg("bn_leak") = 0.0, pybind11::arg("bn_out") = none, pybind11::arg("bn_pre_in") = none, pybind11::arg("bn_pre_out") = none);
  mod.def("Incre_Convolution_updateOutput", &Incre_Convolution_updateOutput, pybind11::arg("inputSize"), pybind11::arg("outputSize"), pybind11::arg("filterSize"), pybind11::arg("filterStride"), pybind11::arg("metadata"), pybind11::arg("input_features"), pybind11::arg("output_features"), pybind11::arg("weight"), pybind11::arg("bias"), pybind11::arg("packed") = none, pybind11::arg("pre_metadata") = pybind11::none(), pybind11::arg("bn_scale") = none, pybind11::arg("bn_shift") = none, pybind11::arg("bn_leak") = 0.0, pybind11::arg("bn_out") = none, pybind11::arg("bn_pre_in") = none, pybind11::arg("bn_pre_out") = none);
  mod.def("Incre_Deconvolution_updateOutput", &Incre_Deconvolution_updateOutput, pybind11::arg("inputSize"), pybind11::arg("outputSize"), pybind11::arg("filterSize"), pybind11::arg("filterStride"), pybind11::arg("metadata"), pybind11::arg("input_features"), pybind11::arg("output_features"), pybind11::arg("weight"), pybind11::arg("bias"), pybind11::arg("pre_metadata"), pybind11::arg("pre_input_feats"), pybind11::arg("packed") = none);
  mod.def("Incre_BatchNormalization_updateOutput", &Incre_BatchNormalization_updateOutput);
  mod.def("Incre_InputLayer_updateOutput", &Incre_InputLayer_updateOutput);
  mod.def("Incre_OutputLayer_updateOutput", &Incre_OutputLayer_updateOutput);
  mod.def("n_rulebook_bits", []() { return scn_n_rulebook_bits(); });
  mod.def("pack_weights", &pack_weights, "transposed weight copy for the tensor-core kernels (empty if not applicable)");
  mod.def("pack_weights_f16", &pack_weights_f16, "fp16 weight fragments for convolutions that read fp16 rows (empty if not applicable)");
  mod.def("set_precision", &set_precision, "arithmetic of the convolution kernels: 'fp32', 'tf32' or 'fp16'");
  mod.def("get_precision", &get_precision);
  mod.def("launch_count", []() { return scn_launch_count(); });
  mod.def("check_errors", []() { check(scn_check_errors((void *)c10::cuda::getCurrentCUDAStream().stream()), "check_errors"); },
          "synchronise the current stream and raise if a kernel flagged an asynchronous error");
  for (const char *name :
       {"SubmanifoldConvolution_backward", "Convolution_backward", "Deconvolution_backward",
        "BatchNormalization_backward", "NetworkInNetwork_updateGradInput", "NetworkInNetwork_accGradParameters",
        "InputLayer_updateGradInput", "OutputLayer_updateGradInput"})
    mod.def(name, &no_backward);
}
