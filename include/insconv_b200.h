/*
 * insconv_b200.h -- C ABI of the B200 (sm_100a) sparse-convolution hot path.
 *
 * This is the boundary a host language binds to.  Every entry point takes plain
 * pointers and sizes; nothing here mentions torch.  Unless a parameter is marked
 * HOST, every data pointer is a device pointer on the current CUDA device, and
 * `stream` is a cudaStream_t passed as void* (NULL = legacy default stream).
 *
 * Every function returns 0 on success and a negative SCN_E_* code otherwise;
 * scn_last_error() then returns a thread-local, human readable message.  No
 * entry point aborts the process, and there is no CPU fallback: without a
 * usable CUDA device every compute call fails with SCN_E_CUDA.
 *
 * Each declaration cites the interface of the reference implementation
 * (THU-luvision/INS-Conv, paths relative to sparseconvnet/SCN/) that it replaces.
 *
 * Conventions shared with the reference:
 *   - spatial sizes, filter sizes and strides are int64[3] HOST arrays;
 *   - feature matrices are row-major fp32 [rows, planes] with a row stride given
 *     in elements (stride == planes for contiguous tensors);
 *   - convolution weights are [volume, n_in, n_out] fp32, volume 27 (3x3x3
 *     submanifold, offset index (dx+1)*9 + (dy+1)*3 + (dz+1)) or 8 (2x2x2 / stride
 *     2, offset index (x&1)*4 + (y&1)*2 + (z&1));
 *   - "no bias" is a NULL pointer;
 *   - a site's row index is the rank of its packed key (batch, z, y, x) among the
 *     active sites of its scale, so row i is the i-th smallest key.
 */
#ifndef INSCONV_B200_H_
#define INSCONV_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define SCN_API __attribute__((visibility("default")))
#else
#define SCN_API
#endif

#define SCN_OK 0
#define SCN_E_INVALID (-1)   /* bad argument (size, mode, null pointer, range)          */
#define SCN_E_CUDA (-2)      /* a CUDA runtime call failed; message has the CUDA error  */
#define SCN_E_RANGE (-3)     /* coordinate / batch index outside the representable key  */
#define SCN_E_CAPACITY (-4)  /* scene bounding box or table larger than the build limit */
#define SCN_E_STATE (-5)     /* metadata has no grid / rulebook for the requested size  */
#define SCN_E_UNSUPPORTED (-6) /* feature of the reference outside the hot path         */

/* arithmetic used by the gather-GEMM kernels */
#define SCN_PREC_FP32 0      /* fp32 FFMA, fp32 accumulate (bit-for-bit deterministic)  */
#define SCN_PREC_TF32 1      /* tf32 tensor cores (tcgen05 with TMEM accumulators, or warp-level mma.sync for narrow layers), fp32 accumulate */
#define SCN_PREC_TF32_PACKED 2 /* as TF32, and `weight` already is the packed copy made by scn_pack_weights */
#define SCN_PREC_F16 3       /* scn_ssc/conv/deconv_forward only: `in` points to fp16 rows [n, n_in] (in_stride in fp16
                                elements; written by scn_bn_forward_f16) and `weight` to the fp16 copy made by
                                scn_pack_weights_f16; fp16 x fp16 products, fp32 accumulation, fp32 `out` */

/* Largest coordinate and batch index a key can hold. */
#define SCN_MAX_COORD 65534
#define SCN_MAX_BATCH 32766

typedef struct scn_metadata scn_metadata; /* opaque; replaces Metadata<3> (Metadata/Metadata.h:218-386) */

SCN_API const char *scn_last_error(void);
/* Library / build identification, e.g. "insconv_b200 sm_100a". */
SCN_API const char *scn_version(void);
/* Number of kernel launches issued by this library since load (all threads). */
SCN_API uint64_t scn_launch_count(void);
/* Tuning aid for the fp16 kernel of wide layers on small grids (16-row tiles, 32 output planes per warp): how many
 * warps share the reduction of one tile.  0 (default): chosen per launch from the number of tiles; 1, 2, 4, 8: fixed.
 * Results do not depend on it beyond the order of fp32 additions.  Process-wide. */
SCN_API int scn_set_slab_share(int warps);
/* Tuning aid: the row count up to which a wide fp16 layer runs that kernel instead of the tcgen05 kernel. */
SCN_API int scn_set_slab_max_rows(int64_t rows);
/* Synchronises `stream` and reports errors that kernels can only flag asynchronously (a bounded
 * wait inside a tensor-core kernel that ran out).  No counterpart in the reference, whose kernels
 * have no such waits. */
SCN_API int scn_check_errors(void *stream);
/* 32: width of a rulebook entry.  Replaces n_rulebook_bits (pybind.cpp:304). */
SCN_API int scn_n_rulebook_bits(void);

/* ---------------------------------------------------------------------------
 * Metadata: per-scale grids, rulebook caches, pre-exist maps.
 * Replaces class Metadata<3> and its pybind surface (pybind.cpp:13-33).
 * ------------------------------------------------------------------------- */
SCN_API int scn_metadata_create(scn_metadata **out);
SCN_API void scn_metadata_destroy(scn_metadata *m);
/* Metadata::clear (Metadata/Metadata.cpp:68-90). */
SCN_API int scn_metadata_clear(scn_metadata *m, void *stream);
/* Metadata::getNActive (Metadata/Metadata.h). Returns -1 when the scale is unknown. */
SCN_API int64_t scn_metadata_n_active(scn_metadata *m, const int64_t size[3]);
/* Metadata::getSpatialLocations (Metadata/Metadata.cpp:793-821): writes [n_active,4]
 * int64 rows (x,y,z,batch) in site order to `out` (HOST pointer). */
SCN_API int scn_metadata_spatial_locations(scn_metadata *m, const int64_t size[3], int64_t *out_host, void *stream);
/* Device pointers to a scale's site coordinates, SoA int32 [4][n] = x.., y.., z.., batch..
 * (the reference's _d_hash_points, CUDA/CUDPPWrapper.hpp:736-1010, plus the batch column). */
SCN_API int scn_metadata_site_coords(scn_metadata *m, const int64_t size[3], const int32_t **coords, int64_t *n);
/* Copies the scale's open-addressing table to HOST arrays of `capacity` entries
 * (capacity from a first call with keys == NULL).  Empty slots have key ~0.
 * The table is a second index beside the build's ranking structure (which serves the
 * rulebook builds): it is filled from the site coordinates by the first call of this
 * function or of scn_metadata_query on the scale, on `stream`, without a host round trip.
 * Key layout: batch<<48 | z<<32 | y<<16 | x.  This is the observable content of the
 * reference's Multival_Point_Hashtable (CUDA/CUDPPWrapper.hpp:736-1010): key -> row. */
SCN_API int scn_metadata_hash_dump(scn_metadata *m, const int64_t size[3], uint64_t *keys_host, int32_t *rows_host,
                           int64_t *capacity, void *stream);
/* Looks up `n` coordinates (device int32 SoA [4][n]) in the scale's table; rows[i] = site
 * row or -1.  Replaces Multival_Point_Hashtable::retrieve (CUDA/CUDPPWrapper.hpp:900-1010). */
SCN_API int scn_metadata_query(scn_metadata *m, const int64_t size[3], const int32_t *coords_soa, int64_t n,
                       int32_t *rows, void *stream);

/* ---------------------------------------------------------------------------
 * InputLayer / OutputLayer.
 * ------------------------------------------------------------------------- */
/* What scn_input_layer_build builds beyond the input scale.  A grid build ends with a host round trip (sizes must reach
 * the host); in the middle of a network that round trip first drains the queue of feature kernels.  A caller that knows
 * what its network will ask for has it built by the input layer, while the stream is still empty: the 3x3x3 neighbour
 * maps (their counts ride on the build's last round trip) and `coarse_levels` stride-2 scales, chained on the device
 * with one round trip for all of them.  neighbour_maps: 1 build them, 0 leave them to first use; coarse_levels: 0..16.
 * -1 in either place: no setting (the per-object setting falls back to the process default, the process default to
 * "nothing ahead").  scn_set_build_ahead sets the process default; scn_metadata_set_build_ahead sets it for the next
 * scn_input_layer_build on one metadata object; scn_metadata_build_used reports what the operators that ran on a
 * metadata object went on to ask for (neighbour maps yes/no, deepest stride-2 level), which is what a network should
 * pass for its next frame -- the Python InputLayer does exactly that, per network.  Results never depend on these
 * settings, only when the work is done.  No counterpart in the reference. */
SCN_API int scn_set_build_ahead(int neighbour_maps, int coarse_levels);
SCN_API int scn_metadata_set_build_ahead(scn_metadata *m, int neighbour_maps, int coarse_levels);
SCN_API int scn_metadata_build_used(scn_metadata *m, int *neighbour_maps, int *coarse_levels);
/* Hands the experience of the previous frame's metadata object to a new one: what its network asked for becomes the new
 * object's build-ahead setting, and the bounding box its input layer measured (with a margin) becomes the box the next
 * input-layer build lays its ranking bitmap out for -- keys, box and occupancy bits then come out of ONE pass over the
 * coordinates and the build has a single host round trip, at its end.  A frame that does not fit the inherited box is
 * built again with the box that pass measured; results never depend on what was inherited.  A metadata object that is
 * built on repeatedly inherits from itself.  No counterpart in the reference (which creates a fresh Metadata per frame,
 * sparseconvnet/ioLayers.py:54-57, and measures nothing ahead). */
SCN_API int scn_metadata_inherit(scn_metadata *m, const scn_metadata *previous);

/* Builds the finest grid from input points.  Replaces Metadata::inputLayer ->
 * inputLayerRulesSimple (Metadata/Metadata.cpp:442-463, Metadata/IOLayersRules.h:135-203)
 * and HashInputPointClouds / InsertAndCompactPointCloud (CUDA/CUDPPWrapper.hpp:668-796).
 * coords: int64 [n_in, ncols] rows (x,y,z[,batch]), ncols 3 or 4; HOST memory when
 * coords_on_host != 0, else device memory.  mode: 3 = sum, 4 = mean (the only modes
 * the reference's GPU grid accepts, IOLayersRules.h:141).  *n_active receives the
 * number of unique sites.  Synchronises `stream` (sizes must reach the host). */
SCN_API int scn_input_layer_build(scn_metadata *m, const int64_t size[3], const int64_t *coords, int coords_on_host,
                          int64_t n_in, int ncols, int64_t batch_size, int mode, void *stream,
                          int64_t *n_active);
/* out[site] = sum or mean of the features of its points, added in ascending point index.
 * Replaces cuda_InputLayer_updateOutput / InputLayer_fp_ (CUDA/IOLayers.cpp:34-96,
 * CUDA/IOLayers.cu:18-45).  in [n_in, planes], out [n_active, planes]. */
SCN_API int scn_input_layer_forward(scn_metadata *m, const float *in, float *out, int64_t planes, void *stream);
/* out[point] = in[site of point].  Replaces cuda_OutputLayer_updateOutput / InputLayer_bp_
 * (CUDA/IOLayers.cpp:123-145, CUDA/IOLayers.cu:48-76).  in [n_active, planes], out [n_in, planes]. */
SCN_API int scn_output_layer_forward(scn_metadata *m, const float *in, float *out, int64_t planes, void *stream);
/* Number of input points of the last scn_input_layer_build (rules[0][2], IOLayersRules.h:11-16). */
SCN_API int64_t scn_input_layer_n_points(scn_metadata *m);
/* Number of sites of the input scale (rules[0][3]; Metadata::inputNActive, Metadata/Metadata.h:278), -1 without an
 * input layer. */
SCN_API int64_t scn_metadata_input_n_active(scn_metadata *m);
/* States how many points each site of the input scale stands for (device int32 [n_active]) when that is not the number
 * of input rows that fell into it: a caller that keeps a scene as per-voxel sums hands in one row per voxel.  Only the
 * incremental input layer reads it, on the saved frame (the weight of the saved mean, CUDA/IOLayers.cu:88-92 takes it
 * from the saved rulebook's row).  No counterpart in the reference. */
SCN_API int scn_input_layer_set_site_counts(scn_metadata *m, const int32_t *counts, int64_t n, void *stream);
/* The InputLayer rulebook in the reference's padded layout (CUDA/IOLayers.cu:7-12):
 * header HOST int32[4] = {mode, maxActive, nIn, nOut}; rows HOST int32 [nOut, 1+maxActive]
 * = {count, point indices ascending..., zero padding}.  Call with rows == NULL to get the header. */
SCN_API int scn_input_layer_rules(scn_metadata *m, int32_t header_host[4], int32_t *rows_host, void *stream);

/* ---------------------------------------------------------------------------
 * Rulebooks (sorted rule pairs), for inspection and parity checks.
 * ------------------------------------------------------------------------- */
/* Submanifold 3x3x3 rulebook of a scale.  Replaces Metadata::getSubmanifoldRuleBook ->
 * SubmanifoldBuildObject (Metadata/Metadata.cpp:521-541, CUDA/SubmanifoldRules_cuda.cpp:38-228).
 * counts_host: HOST int64[27] pairs per offset.  pairs_host (may be NULL): HOST int32
 * [sum(counts), 2] rows (input_row, output_row), offsets concatenated in order, each offset
 * ascending in output_row. */
SCN_API int scn_ssc_rulebook(scn_metadata *m, const int64_t size[3], int64_t counts_host[27], int32_t *pairs_host,
                     void *stream);
/* Size-2 stride-2 rulebook between in_size and out_size = in_size/2, building the coarse grid
 * when needed.  Replaces Metadata::getRuleBook -> Convolution_InputSgToRulesAndOutputSg_FastDownSampleMode
 * (Metadata/Metadata.cpp:669-697, Metadata/ConvolutionRules.h:344-380).  counts_host: HOST int64[8];
 * pairs_host (may be NULL): HOST int32 [n_fine, 2] rows (fine_row, coarse_row), each offset ascending
 * in fine_row. */
SCN_API int scn_conv_rulebook(scn_metadata *m, const int64_t in_size[3], const int64_t out_size[3],
                      int64_t counts_host[8], int32_t *pairs_host, void *stream);

/* ---------------------------------------------------------------------------
 * Feature ops.  *flops receives the multiply-add count the reference returns
 * (pairs * n_in * n_out); may be NULL.
 * ------------------------------------------------------------------------- */
/* The tensor-core kernels read the weights in a layout of their own: transposed, [volume, n_out, n_in], for
 * the tcgen05 kernel; in mma.sync fragment order, rounded to tf32, for the warp-level kernel that takes the
 * narrow layers (n_in, n_out in {16, 32, 64}).  Which one applies depends on (volume, n_in, n_out) alone.
 * Normally every convolution call makes that copy itself; a caller whose weights do not change between calls
 * can make it once with this function (packed: device buffer of volume*n_in*n_out floats, contents opaque)
 * and pass it as `weight` with SCN_PREC_TF32_PACKED.  Only shapes these kernels accept can be packed:
 * scn_weights_packable() != 0 (narrow shapes as above, or n_in and n_out multiples of 32 with n_out <= 256).
 * No counterpart in the reference. */
SCN_API int scn_weights_packable(int64_t volume, int64_t n_in, int64_t n_out);
SCN_API int scn_pack_weights(const float *weight, int64_t volume, int64_t n_in, int64_t n_out, float *packed,
                             void *stream);

/* fp16 activations between a BatchNorm and the convolution that follows it (no counterpart in the reference, whose
 * features are fp32 throughout).  In the narrow layers the convolution is bound by the bytes it gathers, and
 * BatchNorm+ReLU output is well inside fp16's range; fp16 keeps 11 significant bits, one more than the tf32 the
 * other tensor-core kernels read.  scn_bn_forward_f16 writes the normalised rows as fp16 (out: [rows, planes] fp16,
 * out_stride in fp16 elements, planes and out_stride multiples of 8); scn_ssc/conv/deconv_forward with SCN_PREC_F16
 * read them.  Shapes: scn_weights_packable_f16() != 0 (n_in and n_out multiples of 32, n_out <= 224: planes 32 or
 * 64 on both sides run the warp-level kernel, the rest the tcgen05 kernel with kind::f16 and 64 planes per
 * reduction step); packed: scn_packed_size_f16() fp16 elements (n_in is padded to a multiple of 64 for the
 * tcgen05 layout), contents opaque. */
SCN_API int64_t scn_packed_size_f16(int64_t volume, int64_t n_in, int64_t n_out);
SCN_API int scn_weights_packable_f16(int64_t volume, int64_t n_in, int64_t n_out);
SCN_API int scn_pack_weights_f16(const float *weight, int64_t volume, int64_t n_in, int64_t n_out, void *packed,
                                 void *stream);
/* JoinTable (sparseconvnet/tables.py:44-55: torch.cat of the feature planes of two tensors on the same sites) followed
 * by the BatchNorm + leaky ReLU that consumes it (a UNet decoder: JoinTable, then a block whose branch starts with
 * BatchNormReLU), in one pass: joined = [a | b] as fp32 rows [rows, a_planes + b_planes] and
 * rows_f16 = activation(joined * scale + shift) as fp16 rows for the convolution behind the BatchNorm (scale, shift:
 * [a_planes + b_planes], gamma / sqrt(var + eps) and beta - mean * scale).  Plane counts multiples of 4; strides in
 * elements. */
SCN_API int scn_join_bn_forward_f16(const float *a, int64_t a_stride, int64_t a_planes, const float *b, int64_t b_stride,
                                    int64_t b_planes, int64_t rows, float *joined, int64_t joined_stride,
                                    const float *scale, const float *shift, double leakiness, void *rows_f16,
                                    int64_t rows_f16_stride, void *stream);
SCN_API int scn_bn_forward_f16(const float *in, int64_t in_stride, void *out, int64_t out_stride, int64_t rows,
                               int64_t planes, const float *running_mean, const float *running_var, const float *gamma,
                               const float *beta, double eps, double leakiness, void *stream);

/* Replaces cuda_SubmanifoldConvolution_updateOutput (CUDA/Convolution.cpp:152-218).
 * in [n, n_in], out [n, n_out] over the sites of `size`. */
SCN_API int scn_ssc_forward(scn_metadata *m, const int64_t size[3], const float *in, int64_t in_stride, float *out,
                    int64_t out_stride, const float *weight, const float *bias, int64_t n_in, int64_t n_out,
                    int precision, void *stream, double *flops);
/* out = addend + submanifold convolution(in), no bias: the residual sum of a ResNet block formed in the
 * convolution's epilogue instead of by a separate pass over both tensors.  addend [n, n_out] rows with stride
 * addend_stride; it may be `out` itself.  No counterpart in the reference, which adds with AddTable
 * (sparseconvnet/tables.py) after the convolution. */
SCN_API int scn_ssc_forward_add(scn_metadata *m, const int64_t size[3], const float *in, int64_t in_stride, float *out,
                        int64_t out_stride, const float *weight, const float *addend, int64_t addend_stride,
                        int64_t n_in, int64_t n_out, int precision, void *stream, double *flops);
/* What a convolution's epilogue does with a finished output row besides (or instead of) storing it.  No counterpart in
 * the reference, whose network runs AddTable (sparseconvnet/tables.py) and BatchNormalization
 * (CUDA/BatchNormalization.cu:78-107) as passes of their own over the whole tensor.
 *   addend      rows [n, n_out] (stride addend_stride) added to the result: the residual sum of a ResNet block.  With an
 *               addend no bias is applied.  It may be `out` itself.
 *   bn_scale, bn_shift, bn_leakiness, bn_out, bn_out_stride
 *               second output: leaky(v * bn_scale[c] + bn_shift[c]) of the finished value v (addend included) as fp16
 *               rows -- the BatchNorm + ReLU that follows in the network (scale = gamma / sqrt(var + eps), shift = beta -
 *               mean * scale), ready for the next convolution to gather.  Saturates at +-65504 like scn_bn_forward_f16.
 *               Available where the convolution itself reads fp16 rows (SCN_PREC_F16); bn_out 16-byte aligned,
 *               bn_out_stride a multiple of 8.
 *   skip_raw    1: the fp32 result is not stored (`out` may be NULL); only meaningful with bn_out. */
typedef struct scn_epilogue {
  const float *addend;
  int64_t addend_stride;
  const float *bn_scale;
  const float *bn_shift;
  double bn_leakiness;
  void *bn_out;
  int64_t bn_out_stride;
  int skip_raw;
  /* incremental operators only (scn_incre_*_forward_ex; must be NULL / 0 elsewhere): the rows the saved frame's
   * BatchNorm read (fp32, [saved sites, n_out]) and wrote (fp16).  With them the fused result is the RESIDUAL of the
   * activation, act((v + saved input) * scale + shift) - saved output, for sites that existed in the saved frame
   * (CUDA/BatchNormalization.cu:112-150) and act(v * scale + shift) for new ones. */
  const float *bn_pre_in;
  int64_t bn_pre_in_stride;
  const void *bn_pre_out;
  int64_t bn_pre_out_stride;
} scn_epilogue;
/* scn_ssc_forward / scn_conv_forward / scn_deconv_forward with an epilogue (epi == NULL: exactly those). */
SCN_API int scn_ssc_forward_ex(scn_metadata *m, const int64_t size[3], const float *in, int64_t in_stride, float *out,
                               int64_t out_stride, const float *weight, const float *bias, int64_t n_in, int64_t n_out,
                               int precision, const scn_epilogue *epi, void *stream, double *flops);
SCN_API int scn_conv_forward_ex(scn_metadata *m, const int64_t in_size[3], const int64_t out_size[3], const float *in,
                                int64_t in_stride, float *out, int64_t out_stride, const float *weight, const float *bias,
                                int64_t n_in, int64_t n_out, int precision, const scn_epilogue *epi, void *stream,
                                double *flops);
SCN_API int scn_deconv_forward_ex(scn_metadata *m, const int64_t in_size[3], const int64_t out_size[3], const float *in,
                                  int64_t in_stride, float *out, int64_t out_stride, const float *weight,
                                  const float *bias, int64_t n_in, int64_t n_out, int precision, const scn_epilogue *epi,
                                  void *stream, double *flops);
/* Makes sure the coarse grid and rulebook for in_size -> out_size exist and returns the coarse site
 * count (callers size the output with it).  Part of Metadata::getRuleBook (Metadata/Metadata.cpp:669-697). */
SCN_API int scn_conv_prepare(scn_metadata *m, const int64_t in_size[3], const int64_t out_size[3], void *stream,
                     int64_t *n_active_out);
/* Replaces cuda_Convolution_updateOutput (CUDA/Convolution.cpp:51-81); filter 2, stride 2. */
SCN_API int scn_conv_forward(scn_metadata *m, const int64_t in_size[3], const int64_t out_size[3], const float *in,
                     int64_t in_stride, float *out, int64_t out_stride, const float *weight, const float *bias,
                     int64_t n_in, int64_t n_out, int precision, void *stream, double *flops);
/* Replaces cuda_Deconvolution_updateOutput (CUDA/Deconvolution.cpp:28-58): in lives on the coarse
 * scale in_size, out on the fine scale out_size = 2*in_size. */
SCN_API int scn_deconv_forward(scn_metadata *m, const int64_t in_size[3], const int64_t out_size[3], const float *in,
                       int64_t in_stride, float *out, int64_t out_stride, const float *weight,
                       const float *bias, int64_t n_in, int64_t n_out, int precision, void *stream,
                       double *flops);
/* y = leaky(x * gamma/sqrt(var+eps) + beta - mean*gamma/sqrt(var+eps)); gamma/beta may be NULL.
 * Replaces cuda_BatchNormalization_updateOutput, test mode (CUDA/BatchNormalization.cpp:39-61,
 * CUDA/BatchNormalization.cu:78-107). */
SCN_API int scn_bn_forward(const float *in, int64_t in_stride, float *out, int64_t out_stride, int64_t rows,
                   int64_t planes, const float *running_mean, const float *running_var, const float *gamma,
                   const float *beta, double eps, double leakiness, void *stream);
/* Train-mode forward: batch statistics over the rows (biased variance for the normalisation), running
 * statistics updated in place as running = momentum*running + (1-momentum)*batch (unbiased variance),
 * save_mean / save_invstd (may be NULL) receive the batch mean and 1/sqrt(var+eps).  Replaces
 * BatchNormalization_f_train (CUDA/BatchNormalization.cu:14-72). */
SCN_API int scn_bn_forward_train(const float *in, int64_t in_stride, float *out, int64_t out_stride, int64_t rows,
                                 int64_t planes, float *running_mean, float *running_var, float *save_mean,
                                 float *save_invstd, const float *gamma, const float *beta, double eps,
                                 double momentum, double leakiness, void *stream);
/* out = in * weight (+ bias), weight [n_in, n_out].  Replaces cuda_NetworkInNetwork_updateOutput
 * (CUDA/NetworkInNetwork.cpp:9-25). */
SCN_API int scn_nin_forward(const float *in, int64_t in_stride, float *out, int64_t out_stride, int64_t rows,
                    const float *weight, const float *bias, int64_t n_in, int64_t n_out, int precision,
                    void *stream, double *flops);

/* The same 1x1 convolution as scn_nin_forward with SCN_PREC_TF32, for hosts that must not allocate.
 * It has no counterpart in the reference.  Some embedders run with a device-memory budget that is
 * handed out once at start-up (a perception process sharing its GPU with a mapping stack, a service
 * whose memory belongs to another framework's pool): for them a library call that reaches the device
 * allocator in steady state can fail late, stall on an implicit synchronisation, or break their
 * accounting.  This entry point calls no allocator of any kind.  The transposed copy of the weights
 * that the tensor-core kernel needs lives in a fixed 512 KiB buffer inside the library image (every GPU
 * that loads the library holds it until the process exits), which sets the limit:
 *   n_in * n_out <= 131072, n_in and n_out multiples of 32, n_out <= 256;
 * anything else is refused with SCN_E_CAPACITY or SCN_E_INVALID and a message.  Pointers must be
 * 16-byte aligned and strides multiples of 4 elements.
 * The first call on each device looks up the buffer's device address (a runtime query, made once per
 * device).  All calls share the one buffer: it is rewritten at the start of
 * every call (nothing in it has to be cleared), so two calls whose GPU work can overlap -- different
 * streams, or different threads -- race on it; keep them on one stream or serialise them. */
SCN_API int scn_nin_forward_noalloc(const float *in, int64_t in_stride, float *out, int64_t out_stride, int64_t rows,
                                    const float *weight, const float *bias, int64_t n_in, int64_t n_out,
                                    void *stream);

/* ---------------------------------------------------------------------------
 * Incremental ("Incre_*") path.  `m` holds only the sites touched by the new
 * points of this frame; `pre` is the metadata of the last full frame and the
 * pre_* matrices are the features saved on that frame.
 * ------------------------------------------------------------------------- */
/* pre_exist[row of m] = row in pre or -1, cached per scale.  Replaces Metadata::getPreExistMaps
 * (Metadata/Metadata.cpp:609-626).  *map receives a device pointer owned by m. */
SCN_API int scn_incre_pre_exist(scn_metadata *m, scn_metadata *pre, const int64_t size[3], const int32_t **map,
                        int64_t *n, void *stream);
/* Residual of the voxel means after merging the new points into the saved frame.  Replaces
 * cuda_Incre_InputLayer_updateOutput / InputLayer_inc_fp_ (CUDA/IOLayers.cpp:290-337,
 * CUDA/IOLayers.cu:82-106).  Call scn_input_layer_build(m, ...) first. */
SCN_API int scn_incre_input_layer_forward(scn_metadata *m, scn_metadata *pre, const float *in, float *out,
                                  const float *pre_out, int64_t planes, void *stream);
/* out[point] = in[site] + pre_in[pre site] when the site existed.  Replaces
 * cuda_Incre_OutputLayer_updateOutput / InputLayer_inc_bp_ (CUDA/IOLayers.cpp:339-368,
 * CUDA/IOLayers.cu:123-142). */
SCN_API int scn_incre_output_layer_forward(scn_metadata *m, scn_metadata *pre, const float *in, float *out,
                                   const float *pre_in, int64_t planes, void *stream);
/* Replaces cuda_Incre_SubmanifoldConvolution_updateOutput (CUDA/Convolution.cpp:221-303): the
 * submanifold convolution of the residual over m, plus, for sites of m absent from pre, the saved
 * features of their neighbours in pre (IncreSubmanifoldBuildObject, CUDA/SubmanifoldRules_cuda.cpp:233-472). */
SCN_API int scn_incre_ssc_forward(scn_metadata *m, scn_metadata *pre, const int64_t size[3], const float *in,
                          int64_t in_stride, float *out, int64_t out_stride, const float *weight,
                          const float *bias, const float *pre_in, int64_t pre_in_stride, int64_t n_in,
                          int64_t n_out, int precision, void *stream, double *flops);
/* The rule pairs (pre_row_of_neighbour, row_in_m) of the second term above, in the layout of
 * scn_ssc_rulebook.  Replaces Metadata::getIncreSubmanifoldRuleBook (Metadata/Metadata.cpp:543-565). */
SCN_API int scn_incre_ssc_rulebook(scn_metadata *m, scn_metadata *pre, const int64_t size[3], int64_t counts_host[27],
                           int32_t *pairs_host, void *stream);
/* Replaces cuda_Incre_Deconvolution_updateOutput (CUDA/Deconvolution.cpp:61-96,
 * CUDA/Deconvolution.cu:82-155): input row = residual (+ saved row when the coarse site existed
 * and the fine output site is new). */
SCN_API int scn_incre_deconv_forward(scn_metadata *m, scn_metadata *pre, const int64_t in_size[3],
                             const int64_t out_size[3], const float *in, int64_t in_stride, float *out,
                             int64_t out_stride, const float *weight, const float *bias, const float *pre_in,
                             int64_t pre_in_stride, int64_t n_in, int64_t n_out, int precision, void *stream,
                             double *flops);
/* Existing site: y = leaky(w*(x + pre_in) + b) - pre_out; new site: plain BN.  Replaces
 * cuda_Incre_BatchNormalization_updateOutput (CUDA/BatchNormalization.cpp:63-91,
 * CUDA/BatchNormalization.cu:112-150). */
SCN_API int scn_incre_bn_forward(scn_metadata *m, scn_metadata *pre, const int64_t size[3], const float *in,
                         int64_t in_stride, float *out, int64_t out_stride, int64_t planes,
                         const float *running_mean, const float *running_var, const float *gamma,
                         const float *beta, double eps, double leakiness, const float *pre_out,
                         const float *pre_in, void *stream);
/* The incremental BatchNorm of the 'fp16' precision: the residual is written as fp16 rows for the convolution behind it
 * (out: fp16 [n_active, planes], strides in elements), the saved frame's BatchNorm output is read as the fp16 rows that
 * frame wrote (pre_out), its input as fp32 rows (pre_in).  With SCN_PREC_F16, scn_incre_ssc_forward and
 * scn_incre_deconv_forward read both the residual rows and the saved rows as fp16 and take the fp16 weight pack. */
/* scn_incre_ssc_forward with an epilogue: addend = residual rows added to the result (the shortcut of a ResNet block);
 * bn_* = the incremental BatchNorm behind the layer formed in the convolution's epilogue (bn_pre_in / bn_pre_out given,
 * skip_raw 0).  scn_incre_conv_forward_ex: the stride-2 convolution of the residual (scn_conv_forward on the
 * incremental grid, CUDA/Convolution.cpp:83-113) with the same epilogue on the coarse scale. */
SCN_API int scn_incre_ssc_forward_ex(scn_metadata *m, scn_metadata *pre, const int64_t size[3], const float *in,
                                     int64_t in_stride, float *out, int64_t out_stride, const float *weight,
                                     const float *bias, const float *pre_in, int64_t pre_in_stride, int64_t n_in,
                                     int64_t n_out, int precision, const scn_epilogue *epi, void *stream, double *flops);
SCN_API int scn_incre_conv_forward_ex(scn_metadata *m, scn_metadata *pre, const int64_t in_size[3],
                                      const int64_t out_size[3], const float *in, int64_t in_stride, float *out,
                                      int64_t out_stride, const float *weight, const float *bias, int64_t n_in,
                                      int64_t n_out, int precision, const scn_epilogue *epi, void *stream, double *flops);
SCN_API int scn_incre_bn_forward_f16(scn_metadata *m, scn_metadata *pre, const int64_t size[3], const float *in,
                                     int64_t in_stride, void *out, int64_t out_stride, int64_t planes,
                                     const float *running_mean, const float *running_var, const float *gamma,
                                     const float *beta, double eps, double leakiness, const void *pre_out,
                                     int64_t pre_out_stride, const float *pre_in, int64_t pre_in_stride, void *stream);

/* ---- one scene on several GPUs: halo rows pushed into the neighbours' memory ------------------------------
 * The reference runs on one GPU; these entry points have no counterpart there.  A scene is cut into slabs along x,
 * one per GPU (one process each); after every convolution that reads neighbouring sites a rank overwrites the rows
 * of the plane beyond each of its cuts with the values their owner computed.  An scn_halo owns this rank's inbox
 * (device memory the two neighbours write into: per side two message slots of slot_bytes and a sequence number);
 * scn_halo_ipc_handle gives the 64-byte CUDA IPC handle to send to the neighbours, scn_halo_connect maps a
 * neighbour's inbox (side 0 = left, 1 = right; handle NULL = this rank's own inbox, i.e. the rank is its own
 * neighbour on that side).  All ranks must issue the same sequence of exchanges.
 *
 * scn_halo_exchange queues two kernels on `stream` and returns: rows is a device array [4][cap] of row indices
 * (send-left, send-right, receive-left, receive-right; both ranks at a cut list the plane's rows in the same order),
 * counts a device array [4] of how many entries of each list are used.  `a` (and `b`, optional) are row-major device
 * arrays patched in place, rows of a_row_bytes / b_row_bytes (multiples of 4).  Waiting for a neighbour is bounded
 * (scn_halo_set_spin_limit polls of 200 ns, default about one second): when it runs out the rows stay untouched and
 * scn_halo_status (which synchronises the stream) reports timed_out = 1; overflow = 1 says a plane did not fit a
 * slot and was cut short.  Both are cleared by reading them. */
typedef struct scn_halo scn_halo;
SCN_API int scn_halo_create(scn_halo **out, int64_t slot_bytes);
SCN_API void scn_halo_destroy(scn_halo *h);
SCN_API int scn_halo_ipc_handle(scn_halo *h, void *handle64);
SCN_API int scn_halo_connect(scn_halo *h, int side, const void *handle64);
SCN_API int scn_halo_set_spin_limit(scn_halo *h, int64_t polls);
SCN_API int scn_halo_exchange(scn_halo *h, const int64_t *rows, const int64_t *counts, int64_t cap, void *a,
                              int64_t a_row_bytes, void *b, int64_t b_row_bytes, void *stream);
SCN_API int scn_halo_status(scn_halo *h, int *timed_out, int *overflow, void *stream);
/* The row lists scn_halo_exchange takes, for a rank that owns the sites with lo <= x < hi of the scale `size`
 * (coordinates of that scale): lists [4][cap] int64 on the device = rows with x == lo, x == hi - 1, x == lo - 1,
 * x == hi, each ascending; counts [4] int64 on the device.  left / right: whether the rank has a neighbour on that side
 * (the lists of a side without one stay empty).  Two launches, no host round trip; entries beyond cap are dropped
 * and show as counts[i] > cap (which scn_halo_exchange reports as overflow). */
SCN_API int scn_halo_plane_lists(scn_metadata *m, const int64_t size[3], int lo, int hi, int left, int right, int64_t cap,
                                 int64_t *lists, int64_t *counts, void *stream);

/* ---- label fusion: the per-voxel vote table behind the network --------------------------------------------
 * Replaces Result<3> (Metadata/resultHash.h:22-138; bound as Result_3, pybind.cpp:36-45) and ResultOfWeight<3>
 * (resultHash.h:141-218; pybind.cpp:275-282): host hash maps there, a device-resident open-addressing table here.
 * weight_classes = 0: vote table, an entry is (label, confidence); > 0: weight table, an entry is a vector of that
 * many scores.  maximum: the cap of the confidence (the reference stores its float argument in an int member, so
 * its default 0.7 acts as 0; pass what the reference would hold).  points: device int64 [n, ncols], ncols 3 (x,y,z)
 * or 4 (+ batch index), coordinates in the library's key range; scores: device fp32 [n, classes] with the given row
 * stride.  Rows of one call that name the same voxel are applied in row order.
 *   update  vote: new voxel -> (argmax, max score); known voxel, same label -> confidence = min(maximum, confidence +
 *           score); other label -> confidence -= score, and below zero the label flips and the confidence changes
 *           sign (resultHash.h:62-98).  weight: new -> the row; known -> 0.5 * old + row (resultHash.h:146-158)
 *   set     vote table only: (argmax, confidence 0) whatever was there (resultHash.h:37-50)
 *   query   labels[i] = label (weight table: argmax of the vector) or -1 (multiQuery, resultHash.h:108-117)
 *   size    number of entries; synchronises the stream and reports coordinates outside the key range
 *           (SCN_E_RANGE) seen by earlier calls; rows_applied_serially (optional): rows of the last update that were
 *           not the first of their voxel
 *   dump    every entry as int64 (x, y, z, label), in no particular order (get_all_points_labels)
 *   finalize  keeps only the entries named by the points (resultHash.h:128-138) */
typedef struct scn_labels scn_labels;
SCN_API int scn_labels_create(scn_labels **out, int weight_classes, double maximum);
SCN_API void scn_labels_destroy(scn_labels *h);
SCN_API int scn_labels_clear(scn_labels *h, void *stream);
SCN_API int scn_labels_update(scn_labels *h, const int64_t *points, int ncols, int64_t n, const float *scores,
                              int64_t scores_stride, int64_t classes, void *stream);
SCN_API int scn_labels_set(scn_labels *h, const int64_t *points, int ncols, int64_t n, const float *scores,
                           int64_t scores_stride, int64_t classes, void *stream);
SCN_API int scn_labels_query(scn_labels *h, const int64_t *points, int ncols, int64_t n, int64_t *labels, void *stream);
SCN_API int scn_labels_size(scn_labels *h, int64_t *size, int64_t *rows_applied_serially, void *stream);
SCN_API int scn_labels_dump(scn_labels *h, int64_t *out, int64_t capacity_rows, int64_t *n_written, void *stream);
SCN_API int scn_labels_finalize(scn_labels *h, const int64_t *points, int ncols, int64_t n, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* INSCONV_B200_H_ */
