/*
 * aimet_b200 -- C ABI of the sm_100a quantization-simulation kernels.
 *
 * Every entry point takes plain device pointers and sizes, launches on the CUDA
 * stream it is given (a cudaStream_t passed as void*), never synchronises and
 * never allocates: outputs and scratch buffers are owned by the caller.  Every
 * function returns AB_OK (0) or a negative AB_ERR_* code; the message for the
 * last error of the calling thread is returned by aimet_b200_last_error().
 *
 * The citations name the aimet_torch interface each entry point stands behind
 * (paths relative to TrainingExtensions/torch/src/python/aimet_torch/).
 */
#ifndef AIMET_B200_H
#define AIMET_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AB_OK 0
#define AB_ERR_INVALID (-1)     /* bad argument (shape, dtype, null pointer) */
#define AB_ERR_UNSUPPORTED (-2) /* valid request this build has no kernel for */
#define AB_ERR_CUDA (-3)        /* a CUDA runtime call failed */
#define AB_ERR_SCRATCH (-4)     /* caller-provided scratch buffer is too small */
#define AB_ERR_DEVICE (-5)      /* a kernel reported a device-side time-out */

/* element types of tensors crossing the boundary */
#define AB_F32 0
#define AB_F16 1
#define AB_BF16 2
#define AB_F64 3

#define AB_MAX_DIMS 8

/*
 * How a row-major contiguous tensor maps onto its encoding parameters.
 * Along dim k every run of block[k] consecutive coordinates shares one
 * (scale, offset) pair: block[k] == size[k] broadcasts the parameter over the
 * dim, block[k] == 1 is per-channel, anything between is blockwise.  The
 * parameter arrays are row-major contiguous of shape size[k] / block[k].
 * (quantization/affine/backends/torch_builtins.py:119-162, 283-289 define the
 * same mapping through reshape + interleave.)
 */
typedef struct ab_layout {
    int32_t ndim;
    int32_t reserved;
    int64_t size[AB_MAX_DIMS];
    int64_t block[AB_MAX_DIMS];
} ab_layout;

int aimet_b200_version(void);
const char *aimet_b200_last_error(void);
/* Number of CUDA kernels this library has launched in this process (diagnostics). */
int64_t aimet_b200_launch_count(void);

/* ------------------------------------------------------------------------- *
 * Affine functionals.
 *   io_dtype       element type of x / y / grad tensors
 *   compute_dtype  the reference's "internal dtype": AB_F16 / AB_BF16 round
 *                  after every arithmetic step exactly like the aten chain the
 *                  reference runs in that dtype (torch_builtins.py:99-116, 268-300)
 *   param_dtype    element type of scale / offset / grad_scale / grad_offset
 *                  (AB_F32 or AB_F64)
 * ------------------------------------------------------------------------- */

/* out = clamp(round(x / scale) - offset, qmin, qmax)
 * replaces backends.quantize (quantization/affine/backends/utils.py:17-25,
 * torch_builtins.py:166-212, QuantizeFunc.forward :588-633) */
int aimet_b200_quantize(const void *x, void *y, const void *scale, const void *offset,
                        const ab_layout *layout, int io_dtype, int compute_dtype, int param_dtype,
                        int64_t qmin, int64_t qmax, void *stream);

/* out = (x + offset) * scale
 * replaces backends.dequantize (backends/utils.py:27-33, torch_builtins.py:537-571,
 * DequantizeFunc.forward :666-685) */
int aimet_b200_dequantize(const void *x, void *y, const void *scale, const void *offset,
                          const ab_layout *layout, int io_dtype, int compute_dtype, int param_dtype,
                          void *stream);

/* out = (clamp(round(x / scale - zps) - offset, qmin, qmax) + offset + zps) * scale
 * replaces backends.quantize_dequantize (backends/utils.py:35-44,
 * torch_builtins.py:216-302, QuantDequantFunc.forward :705-770) */
int aimet_b200_quantize_dequantize(const void *x, void *y, const void *scale, const void *offset,
                                   const ab_layout *layout, int io_dtype, int compute_dtype,
                                   int param_dtype, int64_t qmin, int64_t qmax,
                                   double zero_point_shift, void *stream);

/* out = (clamp(rint(x * (1 / scale)) + zp, qmin, qmax) - zp) * scale with zp = -(int)offset, all
 * in float32: the arithmetic of torch.fake_quantize_per_tensor_affine /
 * torch.fake_quantize_per_channel_affine, which backends.quantize_dequantize calls instead of
 * QuantDequantFunc when neither scale nor offset needs a gradient (torch_builtins.py:243-266,
 * _torch_fake_quantize :335-431).  scale / offset are float32; io_dtype is AB_F32, AB_F16 or
 * AB_BF16.  The backward pass passes grad_y where rint(x / scale) + zp lies inside [qmin, qmax]. */
int aimet_b200_fake_quantize(const void *x, void *y, const void *scale, const void *offset,
                             const ab_layout *layout, int io_dtype, int64_t qmin, int64_t qmax,
                             void *stream);
int aimet_b200_fake_quantize_backward(const void *x, const void *grad_y, const void *scale,
                                      const void *offset, const ab_layout *layout, int io_dtype,
                                      int64_t qmin, int64_t qmax, void *grad_x, void *stream);

/* Bytes of scratch the three backward entry points need for this layout. */
int64_t aimet_b200_backward_scratch_bytes(const ab_layout *layout, int io_dtype);

/* Backward passes.  grad_x / grad_scale / grad_offset may each be NULL when the
 * gradient is not wanted.  grad_scale / grad_offset have the parameters' shape
 * (the reference returns full-size tensors that autograd sums down to that
 * shape; the reduction is done here, deterministically).
 * QuantDequantFunc.backward (torch_builtins.py:772-831) */
int aimet_b200_quantize_dequantize_backward(const void *x, const void *grad_y, const void *scale,
                                            const void *offset, const ab_layout *layout,
                                            int io_dtype, int compute_dtype, int param_dtype,
                                            int64_t qmin, int64_t qmax, double zero_point_shift,
                                            void *grad_x, void *grad_scale, void *grad_offset,
                                            void *scratch, int64_t scratch_bytes, void *stream);
/* The same with the reference's experimental "pivot gradient spiking" (experimental/pgs.py,
 * torch_builtins.py:779-831): where |round(x/s - zps) - (x/s - zps)| > (1 - pgs_eps) / 2 (compared in
 * the internal dtype) the input gradient is grad_y * pgs_multiplier instead of grad_y.  Off when
 * pgs_eps == 0, pgs_multiplier == 1 or grad_x == NULL; scale / offset gradients are not affected. */
int aimet_b200_quantize_dequantize_backward_ex(const void *x, const void *grad_y, const void *scale,
                                               const void *offset, const ab_layout *layout,
                                               int io_dtype, int compute_dtype, int param_dtype,
                                               int64_t qmin, int64_t qmax, double zero_point_shift,
                                               double pgs_eps, double pgs_multiplier, void *grad_x,
                                               void *grad_scale, void *grad_offset, void *scratch,
                                               int64_t scratch_bytes, void *stream);
/* QuantizeFunc.backward (torch_builtins.py:637-659) */
int aimet_b200_quantize_backward(const void *x, const void *grad_y, const void *scale,
                                 const void *offset, const ab_layout *layout, int io_dtype,
                                 int compute_dtype, int param_dtype, int64_t qmin, int64_t qmax,
                                 void *grad_x, void *grad_scale, void *grad_offset, void *scratch,
                                 int64_t scratch_bytes, void *stream);
/* DequantizeFunc.backward (torch_builtins.py:689-701) */
int aimet_b200_dequantize_backward(const void *x, const void *grad_y, const void *scale,
                                   const void *offset, const ab_layout *layout, int io_dtype,
                                   int compute_dtype, int param_dtype, void *grad_x,
                                   void *grad_scale, void *grad_offset, void *scratch,
                                   int64_t scratch_bytes, void *stream);

/* No counterpart in the reference.  Same computation and results as
 * aimet_b200_quantize_dequantize_backward, for callers that cannot hand over a scratch buffer
 * because they are not allowed to allocate device memory where they run (an operator inside a
 * serving runtime that owns the allocator, a worker whose memory is all committed to a pool).
 * The reduction scratch is a fixed array inside the library instead:
 * aimet_b200_fixed_scratch_capacity() bytes (1 MiB), resident on every GPU that loads the library.
 * Layouts whose aimet_b200_backward_scratch_bytes() exceeds that are refused with AB_ERR_SCRATCH.
 * The first call on a device looks up the array's device address (a host-side runtime query, no
 * allocation); make that first call before starting any stream capture.  All calls on a device
 * share the array: calls whose kernels overlap on the GPU race, so keep them on one stream. */
int64_t aimet_b200_fixed_scratch_capacity(void);
int aimet_b200_quantize_dequantize_backward_fixed_scratch(
    const void *x, const void *grad_y, const void *scale, const void *offset, const ab_layout *layout,
    int io_dtype, int compute_dtype, int param_dtype, int64_t qmin, int64_t qmax,
    double zero_point_shift, void *grad_x, void *grad_scale, void *grad_offset, void *stream);

/* Floating-point fake-cast: y = fake_cast(clamp(x / scale, -maxval, maxval)) * scale, simulating a
 * float format with exponent_bits / mantissa_bits on a wider tensor; scale is float32 of the
 * layout's parameter shape (per-tensor, per-channel or blockwise).
 * replaces _float_quantize_dequantize (quantization/float/quantizer.py:619-705).
 *   in_dtype       dtype of x: io_dtype, or a 16-bit type with io_dtype AB_F32 (what type promotion
 *                  makes of a 16-bit tensor divided by a float32 scale with dimensions)
 *   io_dtype / compute_dtype  AB_F32, AB_F16 or AB_BF16: the dtype of y, in which every
 *                  step is evaluated and rounded as the reference's tensor operations are
 *   exponent_bias  bias of the format's exponent field (smallest normal number 2^(1 - bias))
 *   maxval         largest finite value of the format
 *   flags          1: formats without a torch dtype -- repeat fake_cast_to_ieee_float
 *                     (fp_quantization.py:157-214) step by step, else round to nearest even onto
 *                     the format's grid, subnormals included (_cast_decast :704-705)
 *                  2: the format has infinities: an infinite x / scale passes through (flag 1 only)
 *                  4: the format's zero is unsigned: zero results are +0 */
int aimet_b200_float_fake_cast(const void *x, void *y, const float *scale, const ab_layout *layout,
                               int in_dtype, int io_dtype, int compute_dtype, int32_t exponent_bits,
                               int32_t mantissa_bits, int32_t exponent_bias, double maxval,
                               int32_t flags, void *stream);

/* ------------------------------------------------------------------------- *
 * Calibration statistics.  The layout must reduce to (outer, channel, inner):
 * one statistic per parameter element, taken over everything that shares it.
 * ------------------------------------------------------------------------- */

int64_t aimet_b200_stats_scratch_bytes(const ab_layout *layout, int io_dtype);

/* min_out[c], max_out[c] in io_dtype.
 * finite_only == 0: torch.amin / torch.amax semantics, NaN propagates
 *   (_MinMaxObserver.collect_stats, quantization/encoding_analyzer.py:80-93)
 * finite_only == 1: +-inf and NaN are skipped; a slice with no finite value
 *   yields (+inf, -inf) (_HistogramObserver._get_min_max, :213-219) */
int aimet_b200_minmax(const void *x, const ab_layout *layout, int io_dtype, int finite_only,
                      void *min_out, void *max_out, void *scratch, int64_t scratch_bytes,
                      void *stream);

/* The same, as a running min / max over calls: min_io / max_io are read and updated (start them
 * at +inf / -inf).  Lets a calibration loop keep one pair of statistics on the device instead of
 * one pair per batch (_MinMaxObserver.merge_stats, encoding_analyzer.py:95-112). */
int aimet_b200_minmax_running(const void *x, const ab_layout *layout, int io_dtype, int finite_only,
                              void *min_io, void *max_io, void *scratch, int64_t scratch_bytes,
                              void *stream);

/* The same over a list of num_tensors tensors of one layout (a host array of device pointers):
 * the statistics run over all of them, and, where the layout is a single statistic over contiguous
 * tensors (a per-tensor quantizer's calibration batches), up to 32 tensors share one launch.
 * merge != 0 also takes in the values already in min_io / max_io. */
int aimet_b200_minmax_batches(const void *const *xs, int32_t num_tensors, const ab_layout *layout,
                              int io_dtype, int finite_only, int merge, void *min_io, void *max_io,
                              void *scratch, int64_t scratch_bytes, void *stream);

/* counts[c][b] (int64, overwritten): torch.histc binning of float(x) over
 * [lo[c], hi[c]], i.e. bin = (int)((x - lo) * num_bins / (hi - lo)) with x == hi
 * in the last bin and values outside [lo, hi] or NaN ignored; then the number of
 * x < below[c] is added to bin 0 and the number of x > above[c] to the last
 * bin, the comparison being made in io_dtype as the reference's tensor
 * comparison does.  lo / hi / below / above are float32[C].
 * (_HistogramObserver.collect_stats / merge_stats, encoding_analyzer.py:194-209, 313-323)
 * If fin_min / fin_max are non-NULL the finite-only min / max of each slice is
 * produced by the same pass (io_dtype, needs scratch as for aimet_b200_minmax). */
int aimet_b200_histogram(const void *x, const ab_layout *layout, int io_dtype, int32_t num_bins,
                         const float *lo, const float *hi, const float *below, const float *above,
                         int64_t *counts, void *fin_min, void *fin_max, void *scratch,
                         int64_t scratch_bytes, void *stream);

/* The same with options (flags, or-ed together):
 *   1  add to counts instead of overwriting them (several batches binned over one range, the
 *      second phase of a calibration whose range was agreed on first)
 *   2  fin_min / fin_max are running values over calls, as in aimet_b200_minmax_running */
int aimet_b200_histogram_ex(const void *x, const ab_layout *layout, int io_dtype, int32_t num_bins,
                            const float *lo, const float *hi, const float *below, const float *above,
                            int64_t *counts, void *fin_min, void *fin_max, int32_t flags,
                            void *scratch, int64_t scratch_bytes, void *stream);

/* The same over a list of tensors of one layout (see aimet_b200_minmax_batches), all binned over
 * the same range with the counts running over the list.  run_if_nonzero, if not NULL, holds one
 * device flag per histogram, read by the kernel: histograms whose flag is zero are left alone -- for
 * a pass that a preceding kernel may find unnecessary, decided without the host waiting. */
int aimet_b200_histogram_batches(const void *const *xs, int32_t num_tensors, const ab_layout *layout,
                                 int io_dtype, int32_t num_bins, const float *lo, const float *hi,
                                 const float *below, const float *above, int64_t *counts,
                                 void *fin_min, void *fin_max, int32_t flags,
                                 const int32_t *run_if_nonzero, void *scratch, int64_t scratch_bytes,
                                 void *stream);

/* Bin edges of histograms over [min, max] and what a histogram pass needs from them, one launch
 * for _HistogramObserver._create_bin_edges (encoding_analyzer.py:221-229): a degenerate range is
 * widened by 0.5 on each side in the statistics dtype (stat_dtype: AB_F32 / AB_F16 / AB_BF16),
 * edges = ticks * ((hi - lo) / num_bins) + lo.
 *   min, max      float32 [H] (the statistics, exact in stat_dtype)
 *   edges         float32 [H][num_bins + 1]
 *   lo, hi        float32 [H] first and last edge
 *   below, above  float32 [H] the same rounded to stat_dtype (for the outlier comparisons)
 *   range_limit   float32 [H][2] or NULL: edges -/+ (hi - lo) * growth_limit / 2 (:244-257) */
int aimet_b200_histogram_edges(const float *min, const float *max, int32_t num_hist, int32_t num_bins,
                               int stat_dtype, double growth_limit, float *edges, float *lo, float *hi,
                               float *below, float *above, float *range_limit, void *stream);

/* Moves accumulated histograms into the range that also covers a new batch, one launch for
 * what _HistogramObserver.merge_stats (encoding_analyzer.py:231-323) does with tensor
 * expressions: updated range = batch range clamped between the growth limit and the current
 * edges; counts of a source bin that straddles a destination edge are split proportionally
 * (first part rounded half to even); new edges = ticks * step + lo.  All float32.
 *   new_min/new_max   [H]   finite range of the new batch
 *   cur_min/cur_max   [H]   range of the accumulated histograms
 *   cur_edges         [H][num_bins + 1], cur_hist [H][num_bins]
 *   range_limit       [H][2] growth limit (lower, upper)
 *   out_min/out_max   [H]   updated range
 *   out_carry         [H][num_bins] the accumulated counts in the bins of the updated range
 *                     (a copy of cur_hist where the range did not change)
 *   out_edges         [H][num_bins + 1] edges of the updated range */
int aimet_b200_histogram_merge(const float *new_min, const float *new_max, const float *cur_min,
                               const float *cur_max, const float *cur_edges, const float *cur_hist,
                               const float *range_limit, int32_t num_hist, int32_t num_bins,
                               float *out_min, float *out_max, float *out_carry, float *out_edges,
                               void *stream);

/* The same, and out_moved [H] (int32, may be NULL) = 1 where the updated range no longer ends at
 * the current edges, i.e. where counts taken over the current edges are not the counts over the
 * updated range; out_range [H][4] (may be NULL) = first edge, last edge of the updated range and
 * the two rounded to stat_dtype (what a histogram pass over the updated range takes as lo, hi,
 * below, above). */
int aimet_b200_histogram_merge_ex(const float *new_min, const float *new_max, const float *cur_min,
                                  const float *cur_max, const float *cur_edges, const float *cur_hist,
                                  const float *range_limit, int32_t num_hist, int32_t num_bins,
                                  float *out_min, float *out_max, float *out_carry, float *out_edges,
                                  int32_t *out_moved, float *out_range, int stat_dtype, void *stream);

/* One update of a single (per-tensor) accumulated histogram with a new batch, everything a call of
 * _HistogramObserver.collect_stats + merge_stats does (encoding_analyzer.py:194-323), enqueued by
 * one call: the batch is binned against the current range while its own finite min / max are
 * found; the accumulated counts move into the range that also covers the batch (growth limit
 * applied); only if that range differs from the current one is the batch binned again, over the
 * new range (decided on the device); the two are added.
 *   cur_hist [num_bins], cur_edges [num_bins + 1], cur_min, cur_max [1]: the state before
 *   cur_range [4]: first edge, last edge, and the two rounded to the tensor dtype
 *   range_limit [2]: the growth limits of the range (-inf / +inf when there is none)
 *   new_*: the state after (must not overlap the state before);  batch_min / batch_max [1] in the
 *   tensor dtype;  counts, redo int64 [num_bins], carry float32 [num_bins], moved int32 [1]: work
 *   buffers;  scratch as for aimet_b200_histogram */
int aimet_b200_histogram_update(const void *x, const ab_layout *layout, int io_dtype, int32_t num_bins,
                                const float *cur_hist, const float *cur_edges, const float *cur_min,
                                const float *cur_max, const float *cur_range, const float *range_limit,
                                float *new_hist, float *new_edges, float *new_min, float *new_max,
                                float *new_range, void *batch_min, void *batch_max, int64_t *counts,
                                int64_t *redo, float *carry, int32_t *moved, void *scratch,
                                int64_t scratch_bytes, void *stream);

/* hist_out[h][b] = carry[h][b] + (moved[h] ? redo : counts)[h][b] as float32: the last step of a
 * sequential update (encoding_analyzer.py:313-323), taking the batch's counts from the pass that is
 * valid for the updated range. */
int aimet_b200_histogram_combine(const int64_t *counts, const int64_t *redo, const float *carry,
                                 const int32_t *moved, int32_t num_hist, int32_t num_bins,
                                 float *hist_out, void *stream);

/* Expected clipping + rounding noise of every (delta, offset) candidate against
 * a histogram, and the arg-min per histogram.
 *   hist        float32 [H][num_bins]
 *   edge0/width float32 [H]: first bin edge and bin width (bin_edges[1]-bin_edges[0])
 *   deltas      float32 [H][num_cand]
 *   offsets     float32 [H][num_cand] or, if offsets_per_hist == 0, [num_cand]
 *   noise_out   float32 [H][num_cand]
 *   best_out    int32   [H]  (lowest index among equal minima)
 * _LpNormEncodingAnalyzer._estimate_clip_and_quant_noise / _select_best_candidates
 * (encoding_analyzer.py:822-899); the error of a bin is |quantized midpoint - midpoint|^p times
 * its count, times gamma where the midpoint was clipped */
int aimet_b200_sqnr_sweep(const float *hist, const float *edge0, const float *width,
                          const float *deltas, const float *offsets, int32_t offsets_per_hist,
                          int32_t num_hist, int32_t num_bins, int32_t num_cand, double num_steps,
                          double gamma, double p, float *noise_out, int32_t *best_out, void *stream);

/* The whole SQNR / TF-enhanced range search in two launches: the candidates are formed on the
 * device with the reference's operations in the reference's order, evaluated against the
 * histogram, and the winner's range min = offset * delta, max = min + num_steps * delta is written.
 * _pick_test_candidates, _clamp_delta_offset_values, _select_best_candidates,
 * compute_encodings_from_stats (encoding_analyzer.py:700-899).
 *   hist          float32 [H][num_bins];  edges float32 [H][num_bins + 1]
 *   stat_min/max  float32 [H] observed range (exact in stat_dtype, the dtype of the statistics)
 *   asymmetric: num_deltas deltas x (num_base_offsets + 1) offsets; base_offsets float32
 *     [num_base_offsets] is round(arange(-num_steps, step, step)), step = num_steps / (O - 2), the
 *     observed offset is appended;  symmetric: num_deltas deltas, offset floor(-num_steps / 2)
 *   noise_out     float32 [H][num_cand];  deltas_out / offsets_out float32 [H][num_cand] or both NULL
 *   enc_min_out / enc_max_out float32 [H];  best_out int32 [H] (lowest index among equal minima) */
int aimet_b200_sqnr_encodings(const float *hist, const float *edges, const float *stat_min,
                              const float *stat_max, const float *base_offsets,
                              int32_t num_base_offsets, int32_t num_deltas, int32_t symmetric,
                              int stat_dtype, int32_t num_hist, int32_t num_bins, double num_steps,
                              double gamma, double p, double min_scale, float *noise_out, float *deltas_out,
                              float *offsets_out, float *enc_min_out, float *enc_max_out,
                              int32_t *best_out, void *stream);

/* ------------------------------------------------------------------------- *
 * SeqMSE reconstruction loss of a Linear layer for all candidates and all
 * input-channel blocks at once:
 *   out[c][n][b][0] = sum_m f(x[m,Kb] . w[n,Kb],  xq[m,Kb] . wq[c][n,Kb])
 * where Kb are the K / num_blocks input channels of block b, and f is the
 * squared difference (loss_kind 0, 2, 3) or the absolute difference (1).
 * loss_kind 2 also returns out[..][1] = sum of squares of the second product,
 * loss_kind 3 the sum of squares of the first product (what neg_sqnr needs as
 * its signal: the Linear path passes (xw, xqwq), seq_mse.py:440-454, the Conv2d
 * path (xqwq, xw), _base/seq_mse.py:705-720).
 *   x, xq  [M][K] row-major, io_dtype AB_BF16 or AB_F16;  w [N][K];  wq [C][N][K]
 *   out    float32 [C][N][num_blocks][nvals], nvals = 2 for loss_kind 2 and 3, else 1
 *   lowp_epilogue != 0 rounds both products and f() to io_dtype the way the
 *   reference's half-precision aten chain does.
 *   has_reference == 0 drops the first product (x and w are not read): the loss
 *   is f(0, xq . wq), which a caller that has formed differences itself uses.
 * With num_blocks > 1 the channels of one block must be a multiple of 16.
 * SequentialMse._compute_linear_loss (seq_mse.py:403-482).
 * The contraction runs on the 5th-generation tensor cores (tcgen05, TMEM
 * accumulators, TMA-fed operands).  status is a device int32 the kernel sets to
 * non-zero if one of its bounded waits gives up. */
int64_t aimet_b200_seqmse_blocks_scratch_bytes(int64_t M, int64_t N, int64_t K, int32_t num_blocks,
                                               int32_t num_cand);
int aimet_b200_seqmse_linear_loss_blocks(const void *x, const void *xq, const void *w, const void *wq,
                                         int64_t M, int64_t N, int64_t K, int32_t num_blocks,
                                         int32_t num_cand, int io_dtype, int loss_kind,
                                         int lowp_epilogue, int has_reference, float *out,
                                         int32_t *status, void *scratch, int64_t scratch_bytes,
                                         void *stream);
/* The same with num_blocks == 1 and has_reference == 1: out is float32 [C][N][nvals]. */
int64_t aimet_b200_seqmse_scratch_bytes(int64_t M, int64_t N, int64_t K, int32_t num_cand);
int aimet_b200_seqmse_linear_loss(const void *x, const void *xq, const void *w, const void *wq,
                                  int64_t M, int64_t N, int64_t K, int32_t num_cand, int io_dtype,
                                  int loss_kind, int lowp_epilogue, float *out, int32_t *status,
                                  void *scratch, int64_t scratch_bytes, void *stream);
/* No counterpart in the reference (its GEMMs are library calls without device-side waits).
 * Launches one warp that waits, with the kernel's bounded wait, on a barrier nothing completes:
 * after limit_us microseconds the wait gives up, *status becomes 3 and the kernel returns.  Lets
 * a host check the give-up path of the SeqMSE kernel's waits without provoking any fault. */
int aimet_b200_seqmse_wait_selftest(int32_t *status, int64_t limit_us, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* AIMET_B200_H */
