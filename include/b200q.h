/*
 * b200q — C ABI of the B200 (sm_100a) quantize / calibrate kernels.
 *
 * Every entry point takes plain device pointers and sizes, launches on the CUDA stream it is
 * given (a cudaStream_t passed as void*; NULL = legacy default stream), allocates nothing and
 * never synchronises (one exception, stated there: b200q_nvfp4_group_quantize_noalloc copies a
 * small table from pageable host memory).  The return value is B200Q_OK (0) or a negative b200q_status; on an
 * error nothing has been launched.  Pointers must be 16-byte aligned unless stated otherwise.
 *
 * The comment above each declaration names the interface of the reference (ModelOpt 0.40,
 * paths relative to the reference project root) that the entry point stands in for.
 */
#ifndef B200Q_H_
#define B200Q_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element type of floating tensors ("T" below) */
typedef enum { B200Q_F32 = 0, B200Q_F16 = 1, B200Q_BF16 = 2 } b200q_dtype;

typedef enum {
  B200Q_OK = 0,
  B200Q_ERR_NULL = -1,        /* a required pointer is NULL */
  B200Q_ERR_DTYPE = -2,       /* dtype code not one of b200q_dtype */
  B200Q_ERR_ALIGN = -3,       /* pointer not 16-byte aligned */
  B200Q_ERR_SHAPE = -4,       /* size not positive / not divisible by the block size */
  B200Q_ERR_ARG = -5,         /* other argument out of range (bits, flags, ...) */
  B200Q_ERR_CUDA = -6,        /* the CUDA runtime reported an error at launch */
  B200Q_ERR_UNSUPPORTED = -7, /* valid request the kernels do not cover */
  B200Q_ERR_TIMEOUT = -8,     /* a bounded device-side wait ran out */
  B200Q_ERR_CAPACITY = -9     /* request larger than the library's built-in scratch */
} b200q_status;

const char* b200q_strerror(int status);
int b200q_version(void);
/* number of SMs of the current device (grid sizing is a multiple of it) */
int b200q_sm_count(void);

/* ---------------------------------------------------------------- amax reductions --------- */

/* Running per-tensor abs-max: *amax_io = max(*amax_io, max|x|) as fp32 (zero it for a fresh
 * amax).  NaN in x makes the result NaN.  Replaces reduce_amax(axis=None)
 * (modelopt/torch/quantization/utils.py:155-188) and the running max of MaxCalibrator.collect
 * (modelopt/torch/quantization/calib/max.py:52-86). */
int b200q_amax_tensor(const void* x, int64_t n, int dtype, float* amax_io, void* stream);

/* Running abs-max over the outer and inner dimensions of x viewed as [outer, axis, inner]
 * (row-major): amax_io[a] = max(amax_io[a], max_{o,i} |x[o,a,i]|).  Replaces reduce_amax with a
 * reduce-axis list (utils.py:137-188) as used by per-channel MaxCalibrator (calib/max.py:62-63). */
int b200q_amax_axis(const void* x, int64_t outer, int64_t axis, int64_t inner, int dtype,
                    float* amax_io, void* stream);

/* Abs-max of each run of `block` contiguous elements: amax_out[b] (fp32, overwritten).
 * Replaces reduce_block_amax with block_sizes={-1: block} (utils.py:52-98). */
int b200q_amax_blocks(const void* x, int64_t nblocks, int block, int dtype, float* amax_out,
                      void* stream);

/* ---------------------------------------------------------------- integer fake quant ------ */

/* y = clamp(rint(x*scale), lo, bound)/scale with scale = bound/amax, bound = 2^(bits-1+unsigned)-1,
 * lo = -(bound + !narrow_range); amax < 2^-24 gives 0.  One fp32 amax for the whole tensor.
 * Replaces fake_tensor_quant of modelopt_cuda_ext
 * (modelopt/torch/quantization/src/tensor_quant_gpu.cu:43-98). */
int b200q_fake_int_tensor(const void* x, void* y, int64_t n, int dtype, const float* amax,
                          int num_bits, int is_unsigned, int narrow_range, void* stream);

/* Same arithmetic with amax[a] chosen by the middle index of x viewed as [outer, axis, inner].
 * Replaces fake_tensor_quant_with_axis (src/tensor_quant_gpu.cu:100-140). */
int b200q_fake_int_axis(const void* x, void* y, int64_t outer, int64_t axis, int64_t inner,
                        int dtype, const float* amax, int num_bits, int is_unsigned,
                        int narrow_range, void* stream);

/* Fused dynamic per-row quantisation of x[rows, cols]: the row abs-max is taken on chip and
 * used as amax of that row in the same pass; amax_out (fp32 [rows], may be NULL) receives it.
 * Replaces the reduce_amax + fake_tensor_quant_with_axis pair that TensorQuantizer issues for
 * dynamic / per-row / per-block integer quantisers
 * (modelopt/torch/quantization/nn/modules/tensor_quantizer.py:505-514,633-686). */
int b200q_fake_int_rows_dynamic(const void* x, void* y, int64_t rows, int64_t cols, int dtype,
                                float* amax_out, int num_bits, int is_unsigned,
                                int narrow_range, void* stream);

/* ---------------------------------------------------------------- FP8 E4M3 fake quant ----- */

/* y = T(float(e4m3_rn_satfinite(float(x)*scale))*inv), scale = 448/amax, inv = 1/scale;
 * amax == NULL casts without scaling.  Replaces fake_e4m3fy
 * (modelopt/torch/quantization/src/tensor_quant_gpu_fp8.cu:35-45,86-101). */
int b200q_fake_e4m3_tensor(const void* x, void* y, int64_t n, int dtype, const float* amax,
                           void* stream);

/* Per-channel form, x viewed as [outer, axis, inner].  Replaces fake_e4m3fy_with_axis
 * (src/tensor_quant_gpu_fp8.cu:47-84). */
int b200q_fake_e4m3_axis(const void* x, void* y, int64_t outer, int64_t axis, int64_t inner,
                         int dtype, const float* amax, void* stream);

/* ---------------------------------------------------------------- NVFP4 ------------------- */

/* flags for b200q_nvfp4_quantize */
enum {
  B200Q_NVFP4_GLOBAL_IS_SCALE2 = 1, /* `global` holds weights_scaling_factor_2, not amax */
  B200Q_NVFP4_SATURATE_SCALES = 2   /* block scales above the E4M3 range saturate to 448 (as the fake-quant
                                       path and the GEMM's activation quantiser do) instead of becoming the
                                       NaN code of the tensor cast: for data that can exceed a calibrated amax */
};

/* Two-level-scale NVFP4 real quantisation of nblocks runs of 16 contiguous elements:
 *   s2 = amax/2688 (or *global itself with B200Q_NVFP4_GLOBAL_IS_SCALE2), written to *s2_out
 *   scales[b] = e4m3(block_amax/(6*s2)) (0 -> 1.0; torch cast rule: >464 -> NaN code 0x7F),
 *               or scales_in[b] when scales_in != NULL
 *   code = sign<<3 | e2m1_rne(|x/(float(scales[b])*s2)|),  packed[j] = code[2j+1]<<4 | code[2j]
 * Replaces NVFP4QTensor.quantize / get_weights_scaling_factor / _cast_fp4
 * (modelopt/torch/quantization/qtensor/nvfp4_tensor.py:62-97,119-232). */
int b200q_nvfp4_quantize(const void* x, int64_t nblocks, int dtype, const float* global,
                         const uint8_t* scales_in, uint8_t* packed, uint8_t* scales,
                         float* s2_out, int flags, void* stream);

/* y = T(lut[code] * (float(scales[b]) * *s2)).  Replaces NVFP4QTensor.dequantize
 * (nvfp4_tensor.py:234-297) and the Triton fp4_dequantize
 * (modelopt/torch/quantization/triton/fp4_kernel.py:211-383). */
int b200q_nvfp4_dequantize(const uint8_t* packed, const uint8_t* scales, const float* s2,
                           void* y, int64_t nblocks, int dtype, void* stream);

/* NVFP4 fake quantisation: y = dequantize(quantize(x)) with the arithmetic above, block scale
 * cast saturating (min(.,448)), one pass, nothing stored but y.  Stands in for
 * dynamic_block_quantize_op with (2,1)/(4,3) formats
 * (modelopt/torch/quantization/tensor_quant.py:158-198; Triton fp4_fake_quant_block,
 * triton/fp4_kernel.py:45-208; fused_amax_convert, src/tensor_quant_mx.cu:239-391). */
int b200q_nvfp4_fake(const void* x, void* y, int64_t nblocks, int dtype, const float* amax,
                     void* stream);

/* One tensor of a grouped NVFP4 launch.  All pointers are device pointers. */
typedef struct {
  const void* x;        /* T [nblocks*16] */
  uint8_t* packed;      /* [nblocks*8]  */
  uint8_t* scales;      /* [nblocks]    */
  float* amax;          /* running abs-max slot of this tensor (in/out) */
  float* s2;            /* weights_scaling_factor_2 out */
  int64_t nblocks;      /* 16-element blocks in this tensor */
  int64_t tile_begin;   /* first tile of this tensor in the launch-wide tile numbering */
} b200q_nvfp4_desc;

/* elements one CTA tile of the grouped kernels covers (tile_begin is counted in these) */
int b200q_nvfp4_group_tile_elems(void);

/* Grouped launches over a device-resident descriptor table (n entries, tile_begin ascending,
 * total_tiles = tiles of all tensors).  `_amax` folds max|x| of each tensor into desc.amax;
 * `_quantize` then quantises every tensor from its desc.amax.  Two launches replace the
 * per-weight loop of pack_real_quantize_weight
 * (modelopt/torch/quantization/qtensor/base_qtensor.py:196-229). */
int b200q_nvfp4_group_amax(const b200q_nvfp4_desc* descs, int n, int64_t total_tiles, int dtype,
                           void* stream);
int b200q_nvfp4_group_quantize(const b200q_nvfp4_desc* descs, int n, int64_t total_tiles,
                               int dtype, void* stream);

/* Grouped NVFP4 quantisation (abs-max pass + quantise pass, same results as the two calls above)
 * for callers that are not allowed to allocate device memory where they quantise — an
 * inference-engine plugin inside its enqueue call, a service whose memory is handed out once at
 * start-up, a process under a hard memory cap.  This entry point has no counterpart in the
 * reference.  It calls no allocator of any kind: the descriptor table and the per-tensor abs-max
 * slots, which the other grouped calls expect from the caller, live in an array built into the
 * library (about 62 KB on every GPU that loads it, until the process exits).
 *   host_descs: HOST array of n descriptors; x, packed, scales, s2, nblocks are read (device
 *               pointers the caller owns), amax and tile_begin are ignored.
 *   n:          at most b200q_nvfp4_group_max_tensors_noalloc() (1024); more is refused with
 *               B200Q_ERR_CAPACITY and nothing is launched.
 * The first call made on a device looks up the array's device address (and keeps it for the life
 * of the process; after a cudaDeviceReset by the host application the next call asks again when its
 * first copy fails).  Make that first call before any stream capture begins anywhere in the
 * process.  The entry point itself must not be called on a capturing stream: the table is copied
 * from a buffer in the callee's stack frame, which a captured copy would outlive, so a capturing
 * stream is refused with B200Q_ERR_UNSUPPORTED before anything is enqueued.  Unlike the other entry
 * points this one may wait on the stream: the table goes to the device in chunks of 64
 * descriptors from pageable memory, and the runtime stages such a copy before it returns.
 * All calls on a device share the one array: the table is rewritten and the abs-max slots cleared
 * by every call, and two calls whose GPU work overlaps (different streams, different threads)
 * race on it — serialise them. */
int b200q_nvfp4_group_quantize_noalloc(const b200q_nvfp4_desc* host_descs, int n, int dtype,
                                       void* stream);
int b200q_nvfp4_group_max_tensors_noalloc(void);

/* ---------------------------------------------------------------- INT4 block -------------- */

/* INT4 (AWQ) block quantise + pack, arithmetic in T as the reference kernel does:
 *   scale = T(T(1/amax_T(block))*7) (or scales_in[b]);  u = roundf(clamp(x*scale,-8,7)+8)
 *   packed[j] = u[2j]<<4 | u[2j+1];  scales_out[b] = scale (T, may alias nothing, may be NULL).
 * Replaces INT4QTensor.quantize + INT4_quantize
 * (modelopt/torch/quantization/qtensor/int4_tensor.py:39-88; src/tensor_quant_gpu.cu:310-366). */
int b200q_int4_quantize(const void* x, int64_t nblocks, int block, int dtype,
                        const void* scales_in, void* scales_out, uint8_t* packed, void* stream);

/* y[2j] = T(hi-8)/scale, y[2j+1] = T(lo-8)/scale.  Replaces INT4_dequantize
 * (src/tensor_quant_gpu.cu:261-308). */
int b200q_int4_dequantize(const uint8_t* packed, const void* scales, void* y, int64_t nblocks,
                          int block, int dtype, void* stream);

/* ---------------------------------------------------------------- FP8 / INT8 real quant --- */

/* q = e4m3fn_torch_cast(T(x / scale[a])) over x viewed as [outer, axis, inner]; scales are T;
 * axis == 1 means one scale.  Replaces FP8QTensor.quantize
 * (modelopt/torch/quantization/qtensor/fp8_tensor.py:41-113). */
int b200q_fp8_quantize(const void* x, const void* scales, uint8_t* q, int64_t outer,
                       int64_t axis, int64_t inner, int dtype, void* stream);

/* q = int8(clamp(round_half_even(T(x / scale[a])), -128, 127)).  Replaces INT8QTensor.quantize
 * (modelopt/torch/quantization/qtensor/int8_tensor.py:35-89). */
int b200q_int8_quantize(const void* x, const void* scales, int8_t* q, int64_t outer,
                        int64_t axis, int64_t inner, int dtype, void* stream);

/* ---------------------------------------------------------------- histogram calibration --- */

/* counts[bin] += #{ i : bin = min(int(|x_i| * nbins / range_max), nbins-1), |x_i| <= range_max }
 * with 64-bit counters (|x| taken in fp32).  Replaces the abs/float/histc chain of
 * HistogramCalibrator.collect (modelopt/torch/quantization/calib/histogram.py:77-130). */
int b200q_hist_collect(const void* x, int64_t n, int dtype, int nbins, float range_max,
                       unsigned long long* counts, void* stream);

/* Entropy (KL-divergence) calibration on the device.  For every candidate i = start_bin, start_bin +
 * stride, ... <= nbins the first i bins are re-quantised into num_levels (a power of two,
 * 2^(bits-1+unsigned)) levels and KL(reference || candidate) is written to divergences[k]
 * (device, (nbins-start_bin)/stride + 1 doubles); *amax_out = edges[i*] (or i* x bin_width when
 * edges is NULL) for the LAST minimum i*.  Replaces _compute_amax_entropy
 * (modelopt/torch/quantization/calib/histogram.py:210-282), a host loop over scipy.stats.entropy. */
int b200q_hist_entropy(const unsigned long long* counts, int nbins, int num_levels, int start_bin, int stride,
                       const float* edges, float bin_width, double* divergences, float* amax_out,
                       void* stream);

/* Mean-squared-error calibration from a histogram: for every candidate i = start_bin, start_bin +
 * stride, ... < nbins the clip point is the centre of bin i, every bin centre is fake quantised to
 * +-bound integer levels and errors[k] = mean over bins of count * (q - centre)^2; *amax_out = the
 * centre of the FIRST minimum.  The documented algorithm of _compute_amax_mse
 * (modelopt/torch/quantization/calib/histogram.py:285-325). */
int b200q_hist_mse(const unsigned long long* counts, int nbins, const float* edges, double bound, int start_bin,
                   int stride, double* errors, float* amax_out, void* stream);

/* Open-ended collection for a calibrator whose range grows: bins continue past nbins - 1 at the
 * same width (range_max / nbins) up to `capacity` bins, so that later batches with larger values
 * need neither a new range nor a host round trip.  Samples beyond capacity bins, NaN and inf are
 * not binned; their number is added to *overflow.  counts has room for `capacity` bins.
 * Stands in for the range-extension branch of HistogramCalibrator.collect
 * (modelopt/torch/quantization/calib/histogram.py:119-130). */
int b200q_hist_collect_open(const void* x, int64_t n, int dtype, int nbins, float range_max, int capacity,
                            unsigned long long* counts, unsigned long long* overflow, void* stream);

/* The same binning with the range read from DEVICE memory when the kernel runs (*range_dev = right
 * edge of bin nbins - 1, e.g. the slot an abs-max kernel has just written or a value received from
 * another rank: no host round trip before the first batch), and with the counts added to n_dest
 * (1..4) histograms at once: calibrators that are handed the very same tensor (the q/k/v or the
 * gate/up input quantisers of a layer) share one pass over it.  counts[i] / overflow[i] are HOST arrays of
 * device pointers; every destination uses the same range.  A range that is not positive and finite puts
 * every non-zero element into the out-of-range counters.  The reference bins once per calibrator
 * (modelopt/torch/quantization/calib/histogram.py:77-130). */
int b200q_hist_collect_shared(const void* x, int64_t n, int dtype, int nbins, const float* range_dev,
                              int capacity, unsigned long long* const* counts,
                              unsigned long long* const* overflow, int n_dest, void* stream);

/* *amax_out = edge of the first bin whose cumulative share (float64 running sum of count/total)
 * reaches percentile/100: edges[i] when edges (fp32 [nbins+1]) is given, else bin_width*i.
 * Replaces _compute_amax_percentile (calib/histogram.py:328-343). */
int b200q_hist_percentile(const unsigned long long* counts, int nbins, const float* edges,
                          float bin_width, double percentile, float* amax_out, void* stream);

/* One histogram of a batched read-out (device-resident table, 8-byte aligned). */
typedef struct {
  const unsigned long long* counts;   /* [nbins] live counters */
  const float* edges;                 /* [nbins + 1] bin edges, or NULL: edge i = bin_width * i */
  float bin_width;
  int nbins;
} b200q_hist_desc;

/* The percentile read-out of n histograms in one launch (one CTA each): amax_out[i] as
 * b200q_hist_percentile gives for descs[i].  Replaces the per-quantiser loop over
 * _compute_amax_percentile in finish_stats_collection (calib/histogram.py:328-343,
 * model_calib.py:145-185). */
int b200q_hist_percentile_batch(const b200q_hist_desc* descs, int n, double percentile, float* amax_out,
                                void* stream);

/* ---------------------------------------------------------------- awq_lite search ---------- */

/* MSE calibration, all candidates in one pass: x (T, viewed as [outer, channels, inner], contiguous) is
 * read once and, taken as fp32, fake-quantised under each of the n_cand (<= 16) candidate amax values
 * cand_amax[s * channels + c] (fp32);
 *   loss_io[s * channels + c] += sum over the elements of channel c of (x - fq(x, cand))^2    (float64)
 * format 0: integer fake quant (num_bits / is_unsigned / narrow_range as b200q_fake_int_tensor);
 * format 1: FP8 E4M3 (b200q_fake_e4m3_tensor).  channels == 1 is the per-tensor case; otherwise inner
 * must be a multiple of the 16-byte pack and at least 32 packs (else B200Q_ERR_UNSUPPORTED).
 * Replaces the loop over candidates of MseCalibrator.collect — per candidate a fake-quant pass, a
 * squared error and a reduction (modelopt/torch/quantization/calib/mse.py:76-100). */
int b200q_mse_candidates(const void* x, int64_t outer, int64_t channels, int64_t inner, int dtype,
                         const float* cand_amax, int n_cand, int format, int num_bits, int is_unsigned,
                         int narrow_range, double* loss_io, void* stream);

/* One candidate of the awq_lite search, weight side: for w[rows, cols] and s[cols] (both T),
 *   v = T(w * s[col]);  amax = max|v| over each run of `block` elements of a row;
 *   y = T(fake_int(v, amax, num_bits, ...))      (integer fake quant as b200q_fake_int_tensor)
 * in one pass.  Replaces the pre_quant_scale multiply, block reshape, dynamic amax and
 * fake_tensor_quant_with_axis chain that TensorQuantizer.forward runs per alpha
 * (modelopt/torch/quantization/model_calib.py:671-685;
 *  nn/modules/tensor_quantizer.py:882-883,505-514,633-686). */
int b200q_awq_scale_fake_int(const void* w, const void* s, void* y, int64_t rows, int64_t cols,
                             int block, int dtype, int num_bits, int is_unsigned, int narrow_range,
                             void* stream);

/* *sum_io += sum_i float(T(a_i - b_i))^2 (float64 accumulator): the numerator of the awq_lite
 * loss (out - out_actual).float().pow(2).mean() (model_calib.py:623-627). */
int b200q_sq_diff_sum(const void* a, const void* b, int64_t n, int dtype, double* sum_io,
                      void* stream);

/* One candidate of the awq_lite search, evaluation side, on the tensor cores (tcgen05, TMEM):
 *   *sum_io += sum_{m,n} float(bf16(bf16(sum_k a[m,k]*b[n,k]) - ref[m,n]))^2
 * a [m,k], b [n,k], ref [m,n] bf16 row-major; m, n multiples of 128, k a multiple of 64 (other
 * shapes return B200Q_ERR_UNSUPPORTED).  The product is never written unless c_out (fp32 [m,n],
 * may be NULL) is given.  *status_io (device word, caller zeroes it) receives error bits if a
 * bounded wait inside the kernel ran out.  Replaces F.linear + update_loss of the search loop
 * (modelopt/torch/quantization/model_calib.py:623-627,671-685). */
int b200q_awq_gemm_sqerr(const void* a, const void* b, const void* ref, int64_t m, int64_t n,
                         int64_t k, double* sum_io, float* c_out, uint32_t* status_io, void* stream);

/* The same with the K extent split over `splits` (1..16) CTAs per output tile, for shapes with few
 * tiles and a long K (a down projection: 512 x 4096 x 14336).  Each CTA leaves an fp32 partial tile
 * in `workspace` (splits * m * n floats); the CTA of a tile that finishes last adds them in split
 * order, so the result does not depend on timing, and runs the same epilogue.  `counters` holds one
 * zeroed uint32 per 128 x 128 tile; the kernel leaves them zero again.  splits == 1 ignores both. */
int b200q_awq_gemm_sqerr_splitk(const void* a, const void* b, const void* ref, int64_t m, int64_t n,
                                int64_t k, int splits, float* workspace, uint32_t* counters,
                                double* sum_io, float* c_out, uint32_t* status_io, void* stream);

/* out[a, r, :] = T(x[r, :] * s[a, :]) for a = 0 .. n_alpha - 1: the activations of an awq_lite search
 * step under every candidate's input-side scale in one pass (x [rows, cols], s [n_alpha, cols], out
 * [n_alpha, rows, cols], all T; cols a multiple of 8, or 4 for fp32).  Replaces the pre_quant_scale
 * multiply of the input quantiser that the patched forward runs once per alpha
 * (modelopt/torch/quantization/model_calib.py:671-685; nn/modules/tensor_quantizer.py:882-883). */
int b200q_awq_scale_acts(const void* x, const void* s, void* out, int64_t rows, int64_t cols, int n_alpha,
                         int dtype, void* stream);

/* All candidates of one awq_lite search step (one layer, one calibration batch) in one persistent
 * launch on the tensor cores, with the weight-side producer fused into the GEMM's operand path:
 *   loss_io[a] += sum_{m,n} float(bf16(bf16(sum_k a_all[a][m,k] * fq_a(w)[n,k]) - ref[m,n]))^2
 *   fq_a(w) = per-`block` dynamic integer fake quant (as b200q_awq_scale_fake_int) of bf16(w * s_all[a])
 * a_all [n_alpha, m, k] = the activations times each candidate's inverse scale, w [n, k] the raw
 * weight (32-byte aligned), s_all [n_alpha, k], ref [m, n]: all bf16 row-major; loss_io float64
 * [n_alpha].  The scaled
 * and fake-quantised weight is formed in shared memory only.  block must be 128, k a multiple of
 * 128, n a multiple of 32 (other requests return B200Q_ERR_UNSUPPORTED); m is free.  c_out (fp32
 * [n_alpha, m, n], may be NULL) receives the products.  *status_io (device word, caller zeroes it)
 * receives error bits if a bounded wait inside the kernel ran out.  Replaces, for every alpha of
 * the grid at once, the body of the patched forward of awq_lite
 * (modelopt/torch/quantization/model_calib.py:671-685 with update_loss :623-627). */
int b200q_awq_search_fused(const void* a_all, const void* w, const void* s_all, const void* ref,
                           int n_alpha, int64_t m, int64_t n, int64_t k, int block, int num_bits,
                           int is_unsigned, int narrow_range, double* loss_io, float* c_out,
                           uint32_t* status_io, void* stream);

/* The same persistent CTA-pair kernel fed with weights that are ALREADY scaled and fake-quantised:
 *   loss_io[a] += sum_{m,n} float(bf16(bf16(sum_k a_all[a][m,k] * wq_all[a][n,k]) - ref[m,n]))^2
 * wq_all [n_alpha, n, k] bf16 (e.g. from b200q_awq_scale_fake_int, one candidate after the other), the
 * other arguments as above; k a multiple of 128, n a multiple of 32.  With n_alpha = 1 this is one
 * bf16 GEMM with the squared-error epilogue.  It is what the search uses for batches of several thousand
 * rows: the fused form above re-creates a candidate's weight once per 512-row slab, this form once per
 * candidate.  Same reference lines as b200q_awq_gemm_sqerr (model_calib.py:671-685,623-627). */
int b200q_awq_search_prequant(const void* a_all, const void* wq_all, const void* ref, int n_alpha,
                              int64_t m, int64_t n, int64_t k, double* loss_io, float* c_out,
                              uint32_t* status_io, void* stream);

/* NVFP4 with a block size other than 16 (any even size; NVFP4QTensor.quantize and
 * dynamic_block_quant take the block size as an argument, modelopt/torch/quantization/qtensor/
 * nvfp4_tensor.py:142-232, tensor_quant.py:158-198).  Same arithmetic and argument meaning as
 * b200q_nvfp4_quantize / _fake / _dequantize; one thread per block, no alignment requirement. */
int b200q_nvfp4_quantize_blocks(const void* x, int64_t nblocks, int block, int dtype, const float* global,
                                const uint8_t* scales_in, uint8_t* packed, uint8_t* scales, float* s2_out,
                                int flags, void* stream);
int b200q_nvfp4_fake_blocks(const void* x, void* y, int64_t nblocks, int block, int dtype, const float* amax,
                            void* stream);
int b200q_nvfp4_dequantize_blocks(const uint8_t* packed, const uint8_t* scales, const float* s2, void* y,
                                  int64_t nblocks, int block, int dtype, void* stream);

/* awq_clip block search.  w [rows, cols], x [ntok, cols] (the sampled calibration tokens) and
 * w_amax [rows * cols/block] (block abs-max, row-major) in `dtype`; ratios: nratios (<= 15) clip ratios
 * in device memory, fp32.  For every ratio r, row and block:
 *   loss[r][row][blk] += mean over tokens of float(T(cur - org))^2, where org / cur are the block's
 *   partial dot products T(sum_j T(x*w)) with the weights as they are / fake quantised (integer,
 *   num_bits) with block amax T(amax * ratio_r).  loss is fp32 [nratios, rows, cols/block], device.
 * Replaces the per-ratio loop of _clip_search (modelopt/torch/quantization/model_calib.py:875-915). */
int b200q_awq_clip_loss(const void* w, const void* x, const void* w_amax, const float* ratios, int nratios,
                        float* loss, int64_t rows, int64_t cols, int block, int ntok, int dtype,
                        int num_bits, int is_unsigned, int narrow_range, void* stream);

/* ---------------------------------------------------------------- rotation ------------------ */

/* Walsh-Hadamard transform (Sylvester order) of every row of x [rows, n], n a power of two <= 32768:
 *   y = T(float(T(H x)) * scale)   (sums in fp32; scale = 1/sqrt(n) gives the normalised transform).
 * Stands in for fast_hadamard_transform.hadamard_transform, a third-party CUDA package the
 * reference calls from normalized_hadamard_transform (modelopt/torch/quantization/nn/functional.py:75-109). */
int b200q_hadamard(const void* x, void* y, int64_t rows, int n, int dtype, float scale, void* stream);

/* ---------------------------------------------------------------- MX (E8M0-scaled) formats -- */

/* element formats of b200q_mx_fake (numbering of the reference's Types enum) */
enum { B200Q_MX_E4M3 = 0, B200Q_MX_E5M2 = 1, B200Q_MX_INT8 = 2, B200Q_MX_E2M1 = 6, B200Q_MX_E3M2 = 7,
       B200Q_MX_E2M3 = 8 };

/* MX fake quantisation over nblocks runs of `block` contiguous elements:
 *   unscale = 2^clamp(ceil(log2(block_amax / format_max)), -127, 127) (1 for amax 0/inf/NaN),
 *   y = T(sign(x) * round_to_format(|x| / unscale) * unscale), rounding to nearest even, saturating.
 * Replaces fused_amax_convert with an E8M0 scale format
 * (modelopt/torch/quantization/src/tensor_quant_mx.cu:36-54,105-137,239-294). */
int b200q_mx_fake(const void* x, void* y, int64_t nblocks, int block, int dtype, int elem_format,
                  void* stream);

/* MXFP4 real quantisation: scale byte = 127 + ceil(max(log2(block_amax/6), -127)), code =
 * (x > 0 ? 0 : 8) + number of E2M1 bounds strictly below |x / 2^e|, even element in the low nibble.
 * Replaces MXFP4QTensor.quantize (modelopt/torch/quantization/qtensor/mxfp4_tensor.py:38-81). */
int b200q_mxfp4_quantize(const void* x, int64_t nblocks, int block, int dtype, uint8_t* packed,
                         uint8_t* scales, void* stream);

/* ---------------------------------------------------------------- real-quant GEMMs ---------- */

/* FP8 per-tensor linear layer on the tensor cores (tcgen05 kind::f8f6f4, fp32 accumulation in TMEM):
 *   out[m, n] = T(sum_k a[m, k] * b[n, k] * (*scale_a) * (*scale_b) + bias[n])
 * a [m, k], b [n, k] E4M3 bytes, k contiguous; scale_a, scale_b device fp32 scalars (scale_b may be
 * NULL = 1); bias [n] of type T or NULL; out [m, n] of type T.  k a multiple of 16, n of 8; rows
 * beyond m or n are never read or written.  *status_io (device word, caller zeroes it) receives
 * error bits if a bounded wait inside the kernel ran out.  Replaces torch._scaled_mm in
 * _fp8_gemm_impl (modelopt/torch/quantization/backends/fp8_per_tensor_gemm.py:41-55). */
int b200q_fp8_gemm(const uint8_t* a, const uint8_t* b, const float* scale_a, const float* scale_b,
                   const void* bias, void* out, int64_t m, int64_t n, int64_t k, int dtype,
                   uint32_t* status_io, void* stream);

/* Test and tuning switch of b200q_fp8_gemm / b200q_nvfp4_gemm (no counterpart in the reference):
 * forces the CTA tile of every later launch in the process — 128 (128 x 128), 256 (128 x 256),
 * 512 (the largest tile) or 2 (128 x 128 with K shared by a cluster of two CTAs); 0 restores the
 * automatic choice.  Other values are ignored.  Returns the previous setting.  Not synchronised
 * with concurrent launches from other threads. */
int b200q_qgemm_tile_override(int tile);

/* The activation (or weight) operand of b200q_fp8_gemm: q = e4m3(clamp(x / *scale, -448, 448)),
 * *scale a device fp32 scalar, n elements.  round_quotient != 0 rounds the quotient to T before the
 * clamp, as the eager tensor expression does; 0 keeps it in fp32, as a fused graph of the same
 * expression does.  Replaces _to_fp8
 * (modelopt/torch/quantization/backends/fp8_per_tensor_gemm.py:35-37). */
int b200q_fp8_gemm_operand(const void* x, const float* scale, uint8_t* q, int64_t n, int dtype,
                           int round_quotient, void* stream);

/* NVFP4 linear layer on the tensor cores (tcgen05 kind::mxf4nvf4 with block scaling):
 *   out[m, n] = T(T(*alpha * sum_blk sfa[m, blk] * sfb[n, blk] * sum_{j<16} a[m, 16 blk + j] * b[n, 16 blk + j]) + bias[n])
 * a [m, k/2], b [n, k/2] packed E2M1 (even element in the low nibble); sfa, sfb E4M3 block scales
 * in the tiled order b200q_nvfp4_swizzle_scales writes; alpha device fp32 scalar (the product of
 * the two per-tensor scales); k a multiple of 32, n of 8.  Replaces torch.ops.trtllm.nvfp4_gemm
 * (modelopt/torch/quantization/backends/nvfp4_gemm.py:57-64). */
int b200q_nvfp4_gemm(const uint8_t* a, const uint8_t* b, const uint8_t* sfa, const uint8_t* sfb,
                     const float* alpha, const void* bias, void* out, int64_t m, int64_t n, int64_t k,
                     int dtype, uint32_t* status_io, void* stream);

/* Block scales [rows, cols] (one byte per 16 elements, row-major, as b200q_nvfp4_quantize writes
 * them) into 128-row x 4-scale tiles of 512 bytes: scale (r, c) goes to byte
 *   ((r / 128) * tiles_k + c / 4) * 512 + (r % 32) * 16 + ((r % 128) / 32) * 4 + c % 4,
 * tiles_k = 4 * ceil(cols / 16); rows are padded to 128 and cols to 16 with zeros, so `swizzled`
 * holds ceil(rows / 128) * tiles_k * 512 bytes.  For cols a multiple of 16 this is the scale order
 * of the block-scaled tensor-core instructions (the layout fp4_quantize of the reference's GEMM
 * backend returns, nvfp4_gemm.py:55). */
int b200q_nvfp4_swizzle_scales(const uint8_t* scales, uint8_t* swizzled, int64_t rows, int64_t cols,
                               void* stream);

/* ---------------------------------------------------------------- export packers ------------ */

/* INT4 weights in the checkpoint layout: q = clamp(round_half_even(w / scale[r, c/block]), -8, 7)
 * as a signed nibble, byte [r, c] of out[rows/2, cols] = q[2r, c] | q[2r+1, c] << 4.  scales is
 * [rows, cols/block], fp32 (scales_are_f32 != 0: the quotient is an fp32 division) or of type T
 * (the quotient is rounded to T).  Replaces pack_int4_in_uint8
 * (modelopt/torch/export/quant_utils.py:697-738). */
int b200q_int4_export_pack(const void* w, const void* scales, int scales_are_f32, uint8_t* out,
                           int64_t rows, int64_t cols, int block, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200Q_H_ */
