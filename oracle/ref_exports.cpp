// extern "C" entry points over the reference's own host functions, for the ctypes binding in
// oracle/scn_ref.py.  TEST INFRASTRUCTURE: last part of the translation unit that build_ref.py assembles.
// Everything called here is the reference's code (Metadata<3>, cuda_* / cpu_* operators, rulebook
// builders), running on the CUDA-on-host emulation; this file only moves data in and out.
//
// Conventions: features are float32 row-major; sizes are cubic (one long per spatial size); an operator
// leaves its result in a per-thread slot that ref_result_* reads out; every function returns 0, or -1
// with ref_last_error() set (an exception from ATen or from the reference's code).
#include <string>

// The dynamic shared-memory array of _d_Convolution_GenerateOutputRules (CUDA/SubmanifoldRules_cuda.cu:749),
// declared there as `extern __shared__ uint32_t *address_list[]`: under the emulation an ordinary global.
uint32_t *address_list[64];

namespace {
thread_local std::string g_err;
thread_local at::Tensor g_out;            // float32 or int64 result
thread_local std::vector<Int> g_rules;    // flattened rulebook result

at::Tensor f32(const float *p, long rows, long cols) {
  at::Tensor t = at::empty({rows, cols}, at::kFloat);
  if (rows * cols) std::memcpy(t.data_ptr<float>(), p, sizeof(float) * rows * cols);
  return t;
}
at::Tensor f32v(const float *p, long n) {
  if (!p) return at::empty({0}, at::kFloat);
  at::Tensor t = at::empty({n}, at::kFloat);
  if (n) std::memcpy(t.data_ptr<float>(), p, sizeof(float) * n);
  return t;
}
at::Tensor cube(long s) { return at::full({3}, s, at::kLong); }
at::Tensor coords_tensor(const long *c, long n, long ncols) {
  at::Tensor t = at::empty({n, ncols}, at::kLong);
  if (n * ncols) std::memcpy(t.data_ptr<long>(), c, sizeof(long) * n * ncols);
  return t;
}
Metadata<3> &M(void *m) { return *static_cast<Metadata<3> *>(m); }
void flatten(const RuleBook &rb, int32_t *counts, size_t first = 0) {
  g_rules.clear();
  for (size_t k = first; k < rb.size(); ++k) {
    counts[k - first] = (int32_t)(rb[k].size() / 2);
    g_rules.insert(g_rules.end(), rb[k].begin(), rb[k].end());
  }
}
}  // namespace

#define REF_GUARD(...)                         \
  try {                                        \
    __VA_ARGS__;                               \
    return 0;                                  \
  } catch (const std::exception &e) {          \
    g_err = e.what();                          \
    return -1;                                 \
  }

extern "C" {

const char *ref_last_error() { return g_err.c_str(); }
void *ref_metadata_new() { return new Metadata<3>(); }
void ref_metadata_free(void *m) { delete static_cast<Metadata<3> *>(m); }

long ref_result_rows() { return g_out.dim() ? g_out.size(0) : 0; }
long ref_result_cols() { return g_out.dim() > 1 ? g_out.size(1) : 1; }
int ref_result_copy_f32(float *dst) {
  REF_GUARD(at::Tensor c = g_out.contiguous(); std::memcpy(dst, c.data_ptr<float>(), sizeof(float) * c.numel()))
}
int ref_result_copy_i64(long *dst) {
  REF_GUARD(at::Tensor c = g_out.contiguous(); std::memcpy(dst, c.data_ptr<long>(), sizeof(long) * c.numel()))
}
long ref_rules_size() { return (long)g_rules.size(); }
void ref_rules_copy(int32_t *dst) { std::memcpy(dst, g_rules.data(), sizeof(Int) * g_rules.size()); }

// ---- Metadata -------------------------------------------------------------------------------------
long ref_n_active(void *m, long spatial) {
  try {
    return M(m).getNActive(cube(spatial));
  } catch (const std::exception &e) {
    g_err = e.what();
    return -1;
  }
}
int ref_spatial_locations(void *m, long spatial) { REF_GUARD(g_out = M(m).getSpatialLocations(cube(spatial))) }
// rules[0] = {mode, maxActive, nIn, nOut}; rules[1] = nOut rows of (1 + maxActive)
int ref_input_rules(void *m, int32_t header[4]) {
  REF_GUARD(auto &rb = M(m).inputLayerRuleBook; for (int i = 0; i < 4; ++i) header[i] = rb[0][i]; g_rules = rb[1])
}
int ref_ssc_rulebook(void *m, long spatial, int32_t counts[27]) {
  REF_GUARD(flatten(M(m).getSubmanifoldRuleBook(cube(spatial), cube(3), true), counts))
}
int ref_conv_rulebook(void *m, long in_spatial, int32_t counts[8]) {
  REF_GUARD(flatten(M(m).getRuleBook(cube(in_spatial), cube(in_spatial / 2), cube(2), cube(2), true), counts))
}
int ref_incre_ssc_rulebook(void *m, void *pre, long spatial, int32_t counts[27]) {
  REF_GUARD(flatten(M(m).getIncreSubmanifoldRuleBook(cube(spatial), cube(3), true, 1, M(pre)), counts))
}
int ref_pre_exist(void *m, void *pre, long spatial, int32_t *dst, long n) {
  REF_GUARD(Int *map = M(m).getPreExistMaps(cube(spatial), M(pre)); std::memcpy(dst, map, sizeof(Int) * n))
}

// ---- the reference's GPU operators (cuda_*), kernels run by the emulation ---------------------------------
int ref_input_layer(void *m, long spatial, const long *coords, long n, long ncols, const float *feats, long planes,
                    long batch_size, long mode) {
  REF_GUARD(g_out = at::empty({0}, at::kFloat);
            cuda_InputLayer_updateOutput<float, 3>(M(m), cube(spatial), coords_tensor(coords, n, ncols), f32(feats, n, planes),
                                                   g_out, batch_size, mode))
}
int ref_incre_input_layer(void *m, long spatial, const long *coords, long n, long ncols, const float *feats, long planes,
                          long batch_size, long mode, void *pre, const float *pre_out, long pre_rows) {
  REF_GUARD(g_out = at::empty({0}, at::kFloat);
            cuda_Incre_InputLayer_updateOutput<float, 3>(M(m), cube(spatial), coords_tensor(coords, n, ncols),
                                                         f32(feats, n, planes), g_out, batch_size, mode, M(pre),
                                                         f32(pre_out, pre_rows, planes)))
}
int ref_output_layer(void *m, const float *in, long rows, long planes) {
  REF_GUARD(g_out = at::empty({0}, at::kFloat); cuda_OutputLayer_updateOutput<float, 3>(M(m), f32(in, rows, planes), g_out))
}
int ref_incre_output_layer(void *m, const float *in, long rows, long planes, void *pre, const float *pre_in, long pre_rows) {
  REF_GUARD(g_out = at::empty({0}, at::kFloat);
            cuda_Incre_OutputLayer_updateOutput<float, 3>(M(m), f32(in, rows, planes), g_out, M(pre),
                                                          f32(pre_in, pre_rows, planes)))
}
int ref_ssc(void *m, long spatial, const float *in, long rows, long n_in, const float *w, const float *bias, long n_out,
            double *flops) {
  REF_GUARD(g_out = at::empty({0}, at::kFloat);
            *flops = cuda_SubmanifoldConvolution_updateOutput<float, 3>(cube(spatial), cube(3), M(m), f32(in, rows, n_in), g_out,
                                                                        f32(w, 27 * n_in, n_out).view({27, n_in, n_out}),
                                                                        f32v(bias, n_out), 1))
}
int ref_incre_ssc(void *m, long spatial, const float *in, long rows, long n_in, const float *w, const float *bias, long n_out,
                  void *pre, const float *pre_in, long pre_rows, double *flops) {
  REF_GUARD(g_out = at::empty({0}, at::kFloat);
            *flops = cuda_Incre_SubmanifoldConvolution_updateOutput<float, 3>(
                cube(spatial), cube(3), M(m), f32(in, rows, n_in), g_out, f32(w, 27 * n_in, n_out).view({27, n_in, n_out}),
                f32v(bias, n_out), M(pre), f32(pre_in, pre_rows, n_in)))
}
int ref_conv(void *m, long in_spatial, const float *in, long rows, long n_in, const float *w, const float *bias, long n_out,
             int incremental, double *flops) {
  REF_GUARD(g_out = at::empty({0}, at::kFloat); at::Tensor x = f32(in, rows, n_in), wt = f32(w, 8 * n_in, n_out).view({8, n_in, n_out});
            *flops = incremental ? cuda_Incre_Convolution_updateOutput<float, 3>(cube(in_spatial), cube(in_spatial / 2), cube(2), cube(2),
                                                                                 M(m), x, g_out, wt, f32v(bias, n_out))
                                 : cuda_Convolution_updateOutput<float, 3>(cube(in_spatial), cube(in_spatial / 2), cube(2), cube(2), M(m),
                                                                           x, g_out, wt, f32v(bias, n_out)))
}
// in lives on the coarse scale `in_spatial`, out on 2 * in_spatial
int ref_deconv(void *m, long in_spatial, const float *in, long rows, long n_in, const float *w, const float *bias, long n_out,
               double *flops) {
  REF_GUARD(g_out = at::empty({0}, at::kFloat);
            *flops = cuda_Deconvolution_updateOutput<float, 3>(cube(in_spatial), cube(in_spatial * 2), cube(2), cube(2), M(m),
                                                               f32(in, rows, n_in), g_out, f32(w, 8 * n_in, n_out).view({8, n_in, n_out}),
                                                               f32v(bias, n_out)))
}
int ref_incre_deconv(void *m, long in_spatial, const float *in, long rows, long n_in, const float *w, const float *bias,
                     long n_out, void *pre, const float *pre_in, long pre_rows, double *flops) {
  REF_GUARD(g_out = at::empty({0}, at::kFloat);
            *flops = cuda_Incre_Deconvolution_updateOutput<float, 3>(
                cube(in_spatial), cube(in_spatial * 2), cube(2), cube(2), M(m), f32(in, rows, n_in), g_out,
                f32(w, 8 * n_in, n_out).view({8, n_in, n_out}), f32v(bias, n_out), M(pre), f32(pre_in, pre_rows, n_in)))
}
int ref_bn(const float *in, long rows, long planes, const float *mean, const float *var, const float *gamma, const float *beta,
           float eps, float momentum, int train, float leakiness, float *mean_out, float *var_out) {
  REF_GUARD(g_out = at::empty({0}, at::kFloat); at::Tensor rm = f32v(mean, planes), rv = f32v(var, planes);
            cuda_BatchNormalization_updateOutput<float>(f32(in, rows, planes), g_out, at::empty({planes}, at::kFloat),
                                                        at::empty({planes}, at::kFloat), rm, rv, f32v(gamma, planes),
                                                        f32v(beta, planes), eps, momentum, train != 0, leakiness);
            if (mean_out) std::memcpy(mean_out, rm.data_ptr<float>(), sizeof(float) * planes);
            if (var_out) std::memcpy(var_out, rv.data_ptr<float>(), sizeof(float) * planes))
}
int ref_incre_bn(const float *in, long rows, long planes, const float *mean, const float *var, const float *gamma,
                 const float *beta, float eps, float leakiness, void *m, void *pre, const float *pre_out, const float *pre_in,
                 long pre_rows, long spatial) {
  REF_GUARD(g_out = at::empty({0}, at::kFloat);
            cuda_Incre_BatchNormalization_updateOutput<float, 3>(
                f32(in, rows, planes), g_out, at::empty({planes}, at::kFloat), at::empty({planes}, at::kFloat), f32v(mean, planes),
                f32v(var, planes), f32v(gamma, planes), f32v(beta, planes), eps, 0.9f, false, leakiness, M(m), M(pre),
                f32(pre_out, pre_rows, planes), f32(pre_in, pre_rows, planes), cube(spatial)))
}
int ref_nin(const float *in, long rows, long n_in, const float *w, const float *bias, long n_out, double *flops) {
  REF_GUARD(g_out = at::empty({0}, at::kFloat);
            *flops = cuda_NetworkInNetwork_updateOutput<float>(f32(in, rows, n_in), g_out, f32(w, n_in, n_out), f32v(bias, n_out)))
}

// ---- the reference's CPU operators (cpu_*) on the same Metadata: gather -> mm -> scatter-add ------------------
int ref_cpu_ssc(void *m, long spatial, const float *in, long rows, long n_in, const float *w, const float *bias, long n_out,
                double *flops) {
  REF_GUARD(g_out = at::empty({0}, at::kFloat);
            *flops = cpu_SubmanifoldConvolution_updateOutput<float, 3>(cube(spatial), cube(3), M(m), f32(in, rows, n_in), g_out,
                                                                       f32(w, 27 * n_in, n_out).view({27, n_in, n_out}),
                                                                       f32v(bias, n_out)))
}
int ref_cpu_conv(void *m, long in_spatial, const float *in, long rows, long n_in, const float *w, const float *bias, long n_out,
                 double *flops) {
  REF_GUARD(g_out = at::empty({0}, at::kFloat);
            *flops = cpu_Convolution_updateOutput<float, 3>(cube(in_spatial), cube(in_spatial / 2), cube(2), cube(2), M(m),
                                                            f32(in, rows, n_in), g_out, f32(w, 8 * n_in, n_out).view({8, n_in, n_out}),
                                                            f32v(bias, n_out)))
}
int ref_cpu_deconv(void *m, long in_spatial, const float *in, long rows, long n_in, const float *w, const float *bias, long n_out,
                   double *flops) {
  REF_GUARD(g_out = at::empty({0}, at::kFloat);
            *flops = cpu_Deconvolution_updateOutput<float, 3>(cube(in_spatial), cube(in_spatial * 2), cube(2), cube(2), M(m),
                                                              f32(in, rows, n_in), g_out, f32(w, 8 * n_in, n_out).view({8, n_in, n_out}),
                                                              f32v(bias, n_out)))
}
int ref_cpu_bn(const float *in, long rows, long planes, const float *mean, const float *var, const float *gamma, const float *beta,
               float eps, float momentum, int train, float leakiness, float *mean_out, float *var_out) {
  REF_GUARD(g_out = at::empty({0}, at::kFloat); at::Tensor rm = f32v(mean, planes), rv = f32v(var, planes);
            cpu_BatchNormalization_updateOutput<float>(f32(in, rows, planes), g_out, at::empty({planes}, at::kFloat),
                                                       at::empty({planes}, at::kFloat), rm, rv, f32v(gamma, planes),
                                                       f32v(beta, planes), eps, momentum, train != 0, leakiness);
            if (mean_out) std::memcpy(mean_out, rm.data_ptr<float>(), sizeof(float) * planes);
            if (var_out) std::memcpy(var_out, rv.data_ptr<float>(), sizeof(float) * planes))
}
int ref_cpu_nin(const float *in, long rows, long n_in, const float *w, const float *bias, long n_out, double *flops) {
  REF_GUARD(g_out = at::empty({0}, at::kFloat);
            *flops = cpu_NetworkInNetwork_updateOutput<float>(f32(in, rows, n_in), g_out, f32(w, n_in, n_out), f32v(bias, n_out)))
}
// InputLayer_ForwardPass / OutputLayer arithmetic of CPU/IOLayers.cpp over the metadata's input rulebook
int ref_cpu_input_forward(void *m, const float *in, long rows, long planes) {
  REF_GUARD(auto &rb = M(m).inputLayerRuleBook; g_out = at::zeros({(long)rb[0][3], planes}, at::kFloat); at::Tensor x = f32(in, rows, planes);
            InputLayer_ForwardPass<float>(x.data_ptr<float>(), g_out.data_ptr<float>(), rb[0][3], rb[0][1], (Int)planes, &rb[1][0],
                                          rb[0][0] == 4))
}
int ref_cpu_output_forward(void *m, const float *in, long rows, long planes) {
  REF_GUARD(g_out = at::empty({0}, at::kFloat); cpu_OutputLayer_updateOutput<float, 3>(M(m), f32(in, rows, planes), g_out))
}


// ---- label fusion: Result<3> and ResultOfWeight<3> (Metadata/resultHash.h) -------------------------------
void *ref_result_new(float maximum) { return new Result<3>(maximum); }
void ref_result_free(void *r) { delete static_cast<Result<3> *>(r); }
int ref_result_update(void *r, const long *pts, long n, const float *scores, long classes) {
  REF_GUARD(static_cast<Result<3> *>(r)->update(coords_tensor(pts, n, 3), f32(scores, n, classes)))
}
int ref_result_set(void *r, const long *pts, long n, const float *scores, long classes) {
  REF_GUARD(static_cast<Result<3> *>(r)->set(coords_tensor(pts, n, 3), f32(scores, n, classes)))
}
int ref_result_multiquery(void *r, const long *pts, long n, long *out) {
  REF_GUARD(at::Tensor t = static_cast<Result<3> *>(r)->multiQuery(coords_tensor(pts, n, 3));
            std::memcpy(out, t.data_ptr<long>(), sizeof(long) * n))
}
long ref_result_size(void *r) { return (long)static_cast<Result<3> *>(r)->result.size(); }
int ref_result_all(void *r, long *out) {
  REF_GUARD(at::Tensor t = static_cast<Result<3> *>(r)->get_all_points_labels().contiguous();
            std::memcpy(out, t.data_ptr<long>(), sizeof(long) * t.numel()))
}
int ref_result_finalize(void *r, const long *pts, long n) { REF_GUARD(static_cast<Result<3> *>(r)->finalize(coords_tensor(pts, n, 3))) }
// the confidence of one voxel (not exposed by the reference's binding; read from its map for the comparison)
float ref_result_confidence(void *r, long x, long y, long z) {
  Point<3> p;
  p[0] = x, p[1] = y, p[2] = z;
  auto &m = static_cast<Result<3> *>(r)->result;
  auto it = m.find(p);
  return it == m.end() ? -1.f : it->second.second;
}

void *ref_weight_new() { return new ResultOfWeight<3>(); }
void ref_weight_free(void *r) { delete static_cast<ResultOfWeight<3> *>(r); }
int ref_weight_update(void *r, const long *pts, long n, const float *scores, long classes) {
  REF_GUARD(static_cast<ResultOfWeight<3> *>(r)->update(coords_tensor(pts, n, 3), f32(scores, n, classes).clone()))
}
int ref_weight_multiquery(void *r, const long *pts, long n, long *out) {
  REF_GUARD(at::Tensor t = static_cast<ResultOfWeight<3> *>(r)->multiQuery(coords_tensor(pts, n, 3));
            std::memcpy(out, t.data_ptr<long>(), sizeof(long) * n))
}
long ref_weight_size(void *r) { return (long)static_cast<ResultOfWeight<3> *>(r)->result.size(); }
int ref_weight_finalize(void *r, const long *pts, long n) {
  REF_GUARD(static_cast<ResultOfWeight<3> *>(r)->finalize(coords_tensor(pts, n, 3)))
}
}  // extern "C"
