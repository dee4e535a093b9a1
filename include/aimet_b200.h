/*
 * aimet_b200 -- C ABI of the B200 (sm_100a) quantization-simulation hot path.
 *
 * Drop-in boundary for the arithmetic layer of AIMET's quantsim:
 *   - libpymo / "v1" semantics  (DlQuantization C++: clamp -> divide -> round-half-away -> dequantize)
 *   - aimet_torch "v2" semantics (torch_builtins: divide -> round-half-even -> offset -> clamp -> dequantize)
 *
 * Conventions
 *   - Every entry point returns 0 (AQ_OK) or a negative aq_status_t; nothing throws.
 *   - Pointers named d_* are DEVICE pointers on the current CUDA device; h_* are host pointers.
 *   - Nothing here allocates or frees device memory, and nothing synchronises the device unless the
 *     comment says so.  Scratch memory is caller-owned ("workspace").
 *   - `stream` is a cudaStream_t passed as void*; NULL means the legacy default stream.
 *   - Element counts and strides are 64-bit.
 *   - Channel geometry: for a contiguous tensor of n elements, element i belongs to encoding
 *     channel (i / inner) % num_ch.  Per-tensor: num_ch = 1.  Per-output-channel conv weight
 *     [C,I,kh,kw]: num_ch = C, inner = I*kh*kw.  Blockwise [O, I] with block B on the input dim and
 *     scales [O, I/B]: num_ch = O*I/B, inner = B.  NCHW activations per channel: num_ch = C, inner = H*W.
 *
 * Reference citations are paths inside the AIMET 1.35 source tree.
 */
#ifndef AIMET_B200_H_
#define AIMET_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C"
{
#endif

typedef enum
{
    AQ_OK              = 0,
    AQ_ERR_INVALID_ARG = -1, /* NULL pointer, negative size, bad enum, misaligned workspace ... */
    AQ_ERR_UNSUPPORTED = -2, /* combination not implemented (e.g. stochastic rounding) */
    AQ_ERR_CUDA        = -3, /* a CUDA runtime call or launch failed; see aq_last_cuda_error() */
    AQ_ERR_WORKSPACE   = -4, /* workspace missing or too small */
    AQ_ERR_TOO_LARGE   = -5  /* size beyond a documented maximum */
} aq_status_t;

typedef enum
{
    AQ_F32  = 0,
    AQ_F16  = 1,
    AQ_BF16 = 2
} aq_dtype_t;

/* Mirrors DlQuantization::RoundingMode (ModelOptimizations/DlQuantization/include/DlQuantization/Quantization.hpp:145-149).
 * Stochastic rounding is not reproducible in the reference (rand()/clock()-seeded curand) and is rejected here. */
typedef enum
{
    AQ_ROUND_NEAREST    = 0,
    AQ_ROUND_STOCHASTIC = 1
} aq_rounding_t;

/* Mirrors DlQuantization::TfEncoding (Quantization.hpp:113-120). */
typedef struct
{
    double min;
    double max;
    double delta;
    double offset;
    int bw;
} aq_encoding_t;

#define AQ_PDF_SIZE 512 /* DlQuantization PDF_SIZE, src/math_functions.hpp:80 */

/* Device-resident TF-Enhanced histogram state (one per quantizer).
 * Replaces DlQuantization::PDF::xLeft plus the per-call bucket geometry of UpdatePdf
 * (src/math_functions.hpp:59-67, src/math_functions.cpp:264-268). */
typedef struct
{
    double x_left[AQ_PDF_SIZE]; /* bucket left edges */
    float bucket_size;          /* (float)(x_left[1]-x_left[0]) */
    float pdf_offset;           /* (float)x_left[0] / bucket_size */
    int32_t initialized;        /* 0 until a batch with (min,max) != (0,0) was seen */
    int32_t reserved;
} aq_tfe_state_t;

/* ------------------------------------------------------------------------------------------------
 * Library / error helpers
 * ---------------------------------------------------------------------------------------------- */
int aq_version(void);
const char* aq_status_string(int status);
/* Text of the last CUDA error seen by this thread inside the library ("" if none). */
const char* aq_last_cuda_error(void);
/* Number of kernel launches issued by the library in this process (for launch accounting). */
int64_t aq_launch_count(void);

/* ------------------------------------------------------------------------------------------------
 * Host-side encoding arithmetic (no GPU involved)
 * ---------------------------------------------------------------------------------------------- */

/* Replaces TensorQuantizationSim<float>::fillEncodingInfo / generateScaleOffset
 * (ModelOptimizations/DlQuantization/src/TensorQuantizationSim.cpp:62-92) and gateMinMax
 * (src/quantization_utils.cpp:145-156). */
int aq_fill_encoding(int bw, double enc_min, double enc_max, aq_encoding_t* h_out);

/* Replaces getComputedEncodings (src/quantization_utils.cpp:58-143). */
int aq_computed_encodings(int bw, double min, double max, int symmetric, int strict_symmetric, int unsigned_symmetric,
                          aq_encoding_t* h_out);

/* Replaces TfEncodingAnalyzer<float>::computeEncoding (src/TfEncodingAnalyzer.cpp:80-101) given the
 * accumulated running min / max. */
int aq_minmax_encoding(int bw, double stat_min, double stat_max, int symmetric, int strict_symmetric,
                       int unsigned_symmetric, aq_encoding_t* h_out);

/* ------------------------------------------------------------------------------------------------
 * libpymo-semantics fake-quant (fp32 only, like the reference)
 * ---------------------------------------------------------------------------------------------- */

/* Replaces TensorQuantizationSim<float>::quantizeDequantizeTensor
 * (src/TensorQuantizationSim.cpp:94-114 -> src/trim_functions.cpp:93-113,173-182; GPU kernel
 * src/trim_functions.cu:46-60).  The grid is re-derived from (enc_min, enc_max, bw) on every call. */
int aq_qdq_per_tensor(const float* d_in, float* d_out, int64_t n, double enc_min, double enc_max, int bw,
                      int rounding_mode, void* stream);

/* Replaces TensorQuantizationSim<float>::quantizeTensor (src/TensorQuantizationSim.cpp:116-126 ->
 * src/trim_functions.cpp:202-218; GPU kernel src/trim_functions.cu:62-76).  Integer codes in a float container. */
int aq_quantize_per_tensor(const float* d_in, float* d_out, int64_t n, double enc_min, double enc_max, int bw,
                           int rounding_mode, int shift_to_signed, void* stream);

/* Replaces AimetTensorQuantizer::quantizeDequantizePerChannel
 * (TrainingExtensions/torch/src/AimetTensorQuantizer.cpp:256-307) together with
 * TensorQuantizationSim<float>::quantizeDequantizeTensorPerChannel (src/TensorQuantizationSim.cpp:287-317,
 * src/trim_functions.cpp:697-709, kernel src/trim_functions.cu:78-92).
 * d_enc_min / d_enc_max: raw (un-gated) per-channel float min/max, num_ch entries, on the device.
 * num_steps: 2^bw-1, minus one when channel 0 is value-symmetric (the caller decides, as the reference's host
 * code does).  Gating, delta = (max-min)/num_steps and offset = round-half-even(min/delta) happen in the kernel
 * in fp32, in the reference's operation order. */
int aq_qdq_per_channel(const float* d_in, float* d_out, int64_t n, int64_t num_ch, int64_t inner,
                       const float* d_enc_min, const float* d_enc_max, double num_steps, int rounding_mode,
                       void* stream);

/* Replaces quantizeDequantizeBroadcast (src/trim_functions.cpp:633-687, kernel src/trim_functions.cu:96-122;
 * contract in include/DlQuantization/Quantization.hpp:152-222).  Encodings are used as given.
 * h_in_strides / h_enc_strides: HOST arrays of ndims (<= 8) element strides; encoding strides are 0 on
 * broadcast dimensions. */
int aq_qdq_broadcast(const float* d_in, float* d_out, int64_t n, int64_t ndims, const int64_t* h_in_strides,
                     const int64_t* h_enc_strides, const float* d_enc_min, const float* d_enc_max,
                     const float* d_enc_delta, const float* d_enc_offset, void* stream);

/* Everything the v2 min/max calibration does after the reduction, for `count` encodings in one launch:
 *   1. _MinMaxObserver.merge_stats (aimet_torch/v2/quantization/encoding_analyzer.py:112-128): d_running_minmax
 *      ([2, count]: mins, then maxs) takes torch.minimum / torch.maximum with d_batch_minmax, or adopts it when
 *      running_valid = 0 (skipped when d_running_minmax is NULL);
 *   2. MinMaxEncodingAnalyzer.compute_encodings_from_stats (encoding_analyzer.py:340-386) on the batch range -- or on
 *      the running range when d_batch_minmax is NULL -- in the reference's operation order and with the roundings of
 *      statistics held in stats_dtype (AQ_F32 / AQ_F16 / AQ_BF16);
 *   3. the quantizer's scale = (max - min) / num_steps and offset = round(min / scale) - qmin (0 when symmetric)
 *      (aimet_torch/v2/quantization/affine/quantizer.py:222-246), in float32.
 * Inputs hold float32 values that are exactly representable in stats_dtype (what aq_minmax yields on such a tensor).
 * d_out: [4, count] = encoding min, encoding max, scale, offset.  The reference runs about 25 small tensor operations
 * per quantizer for this. */
int aq_v2_minmax_encoding(const float* d_batch_minmax, float* d_running_minmax, int running_valid, int stats_dtype,
                          int64_t count, double num_steps, int symmetric, double qmin, float* d_out, void* stream);

/* 16-bit float fake-quantization: out = (float) (half) in, round to nearest even.  Replaces
 * quantizeDequantizeFp16Gpu (src/Fp16Quantization.cpp:46-50, kernel src/trim_functions.cu:135-148) and the
 * tensor.half().float() pair of the v1 wrappers (aimet_torch/v1/tensor_quantizer.py:1104-1107). */
int aq_qdq_fp16(const float* d_in, float* d_out, int64_t n, void* stream);

/* Integer codes in integer containers.  Replaces TensorQuantizationSim<float>::quantizeTensorPacked ->
 * quantizeToFxpPackedCpu (src/TensorQuantizationSim.cpp:128-139, src/trim_functions.cpp:220-385; CPU only, four host
 * threads in the reference).  The grid is re-derived from (enc_min, enc_max, bw) as in aq_qdq_per_tensor, but clamp,
 * divide, offset and round are evaluated in double.  bw in {1, 2, 4, 8, 16, 32}; one code per container of
 * max(bw, 8) bits: uint8 / uint16 / uint32, or -- with shift_to_signed, which subtracts 2^(bw-1) - 1 -- int8 / int16 /
 * int32 (sub-byte signed codes are masked to their low bw bits).  d_out: n containers, naturally aligned. */
int aq_quantize_packed(const float* d_in, void* d_out, int64_t n, double enc_min, double enc_max, int bw,
                       int rounding_mode, int shift_to_signed, void* stream);

/* Inverse: replaces TensorQuantizationSim<float>::dequantizeTensor -> dequantizeFromPackedFxpCpu
 * (src/TensorQuantizationSim.cpp:210-219, src/trim_functions.cpp:388-605): out = (float)(delta * (code + offset)) in
 * double, codes read from the containers described above (signed sub-byte codes sign-extended). */
int aq_dequantize_packed(const void* d_in, float* d_out, int64_t n, double enc_min, double enc_max, int bw,
                         int shift_to_signed, void* stream);

/* Straight-through backward of the v1 wrappers: dx = g * [enc_min <= x <= enc_max], per tensor
 * (num_ch = 1) or per channel.  Replaces compute_dloss_by_dx
 * (TrainingExtensions/torch/src/python/aimet_torch/v1/quantsim_straight_through_grad.py:91-118).
 * d_enc_min / d_enc_max hold num_ch floats on the device. */
int aq_ste_backward_v1(const float* d_x, const float* d_grad, float* d_dx, int64_t n, int64_t num_ch, int64_t inner,
                       const float* d_enc_min, const float* d_enc_max, void* stream);

/* ------------------------------------------------------------------------------------------------
 * v2-semantics affine fake-quant (fp32 / fp16 / bf16 storage, fp32 internal math)
 * ---------------------------------------------------------------------------------------------- */

#define AQ_V2_OUT_QDQ   0 /* y = (clamp(round(x/s) - o, qmin, qmax) + o) * s */
#define AQ_V2_OUT_CODES 1 /* y =  clamp(round(x/s) - o, qmin, qmax)          */

#define AQ_V2_INTERNAL_F64 2 /* value of narrow_internal: float64 arithmetic */

/* Replaces QuantDequantFunc.forward / QuantizeFunc.forward
 * (TrainingExtensions/torch/src/python/aimet_torch/v2/quantization/affine/backends/torch_builtins.py:290-327,208-236).
 * d_scale / d_offset: num_ch fp32 values on the device (already cast to the internal dtype by the caller).
 * d_mask (may be NULL): one byte per element, 1 where qmin <= round(x/s) - o <= qmax.
 * narrow_internal selects the arithmetic dtype, following the reference's rule (torch_builtins.py:60-87,162-171):
 * 0 = fp32 intermediates; 1 = every intermediate rounded to the storage dtype (what the reference does for
 * quantize()/dequantize() and, for quantize_dequantize(), whenever that dtype is precise enough for the grid);
 * AQ_V2_INTERNAL_F64 = float64 intermediates, for grids of 2^24 steps or more (32-bit quantizers), where qmin / qmax
 * need not be exact in fp32. */
int aq_v2_quantize(const void* d_x, void* d_y, uint8_t* d_mask, int dtype, int64_t n, int64_t num_ch, int64_t inner,
                   const float* d_scale, const float* d_offset, double qmin, double qmax, int out_kind,
                   int narrow_internal, void* stream);

/* Replaces DequantizeFunc.forward (torch_builtins.py:251-276): y = (x + o) * s. */
int aq_v2_dequantize(const void* d_x, void* d_y, int dtype, int64_t n, int64_t num_ch, int64_t inner,
                     const float* d_scale, const float* d_offset, int narrow_internal, void* stream);

/* Replaces the scale / offset gradients of QuantDequantFunc.backward (torch_builtins.py:334-343), element-wise and
 * un-reduced like the reference (the caller's autograd sums over the broadcast dimensions):
 *   dscale = g * (clamp(round(x/s), o+qmin, o+qmax) - (x/s)*mask),  doffset = g * ((1-mask) * s).
 * d_dscale / d_doffset: n floats each; either may be NULL. */
int aq_v2_qdq_backward_params(const void* d_x, const void* d_grad, const uint8_t* d_mask, float* d_dscale,
                              float* d_doffset, int dtype, int64_t n, int64_t num_ch, int64_t inner,
                              const float* d_scale, const float* d_offset, double qmin, double qmax, void* stream);

/* The same gradients already summed over everything an encoding is broadcast along: d_dscale / d_doffset receive
 * num_ch floats each (either may be NULL), i.e. what autograd's reduction of the reference's un-reduced returns
 * yields (torch_builtins.py:334-343 followed by sum_to_size).  The element-wise terms are the reference's; the order in
 * which they are added is not (torch does not specify its own), so results agree to summation tolerance.  Reads
 * 2 * sizeof(T) + 1 bytes per element and writes none, against 17 + 8 for the un-reduced form plus a reduction. */
int aq_v2_qdq_backward_params_reduced(const void* d_x, const void* d_grad, const uint8_t* d_mask, float* d_dscale,
                                      float* d_doffset, int dtype, int64_t n, int64_t num_ch, int64_t inner,
                                      const float* d_scale, const float* d_offset, double qmin, double qmax,
                                      void* stream);

/* Replaces the tensor-gradient of QuantDequantFunc.backward (torch_builtins.py:329-344): dx = grad * mask.
 * d_mask holds one byte per element, 0 or 1 (what aq_v2_quantize writes, and how a bool tensor is stored). */
int aq_v2_qdq_backward(const void* d_grad, const uint8_t* d_mask, void* d_dx, int dtype, int64_t n, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Statistics
 * ---------------------------------------------------------------------------------------------- */

/* Bytes of scratch aq_minmax needs for this geometry (0 is possible). */
int64_t aq_minmax_workspace_bytes(int64_t n, int64_t num_ch, int64_t inner);

/* One fused pass producing min and max per encoding channel.
 * Replaces GetMin + GetMax (src/math_functions.cpp:61-100,327-347; thrust versions src/math_functions.cu:52-64)
 * and the v2 observer reduction (aimet_torch/v2/quantization/encoding_analyzer.py:100-104 with
 * aimet_torch/v2/utils.py:69-90).
 * d_out_min / d_out_max: num_ch floats each (values of 16-bit inputs are exact in fp32).
 * propagate_nan = 0: NaNs are ignored (std::min/std::max folds of the reference C++);
 * propagate_nan = 1: any NaN in a channel makes both outputs NaN (torch.min / torch.max).
 * accumulate != 0 folds the result into the values already in d_out_min / d_out_max (running statistics over
 * batches: the accumulation of TfEncodingAnalyzer::updateStats, src/TfEncodingAnalyzer.cpp:59-71, and of
 * _MinMaxObserver.merge_stats, encoding_analyzer.py:106-122) instead of overwriting them.
 * An empty channel yields +inf / -inf.  d_workspace must be 256-byte aligned and zero-filled before its first
 * use; the library leaves it reusable. */
int aq_minmax(const void* d_x, int dtype, int64_t n, int64_t num_ch, int64_t inner, float* d_out_min,
              float* d_out_max, int propagate_nan, int accumulate, void* d_workspace, int64_t workspace_bytes,
              void* stream);

/* Size of the scratch that aq_minmax_static keeps inside the library image (per GPU that loads the library). */
#define AQ_MINMAX_STATIC_SCRATCH_BYTES (1 << 20)

/* aq_minmax for callers that must not allocate device memory.  (It has no counterpart in the reference, which
 * always allocates its scratch through an allocator callback.)  Think of an inference runtime whose device arena
 * was sized and frozen at start-up, or an operator callback that a host framework runs with allocation switched
 * off: such a caller has nowhere to get the workspace that aq_minmax asks for.  Here the scratch is a fixed array
 * of AQ_MINMAX_STATIC_SCRATCH_BYTES inside the library; the caller passes only the input and the two outputs.
 *   - Same results as aq_minmax(..., accumulate = 0, ...): one min and one max per encoding channel.
 *   - Returns AQ_ERR_TOO_LARGE when the call would touch more scratch than the array holds.  Whole-tensor
 *     statistics always fit.  Per-channel / per-block statistics whose rows each map to one output (n / inner ==
 *     num_ch and rows short enough not to be split) write straight to the outputs and fit at any size; the others
 *     keep one (min, max) pair per (row, segment) in the scratch and fit up to about 130,000 such pairs.  The limit
 *     is never looser than aq_minmax_workspace_bytes(n, num_ch, inner) <= AQ_MINMAX_STATIC_SCRATCH_BYTES.
 *   - Calls no cudaMalloc / cudaFree and no allocating library routine.  The first call on each device looks the
 *     array's device address up (cudaGetSymbolAddress, with that device current); make that first call before
 *     any stream capture begins.  That look-up may run on several host threads at once (they store the same
 *     address).
 *   - All calls on a device share the one array and it keeps the previous call's contents; the entry point clears
 *     the part that has to start at zero on `stream` itself.  Calls that overlap on the GPU (different streams,
 *     no ordering between them) race on the scratch: serialise them. */
int aq_minmax_static(const void* d_x, int dtype, int64_t n, int64_t num_ch, int64_t inner, float* d_out_min,
                     float* d_out_max, int propagate_nan, void* stream);

/* Builds the bucket grid from a batch's (min,max) held on the device; leaves the state un-initialised when both
 * are zero.  Replaces the first-batch branch of UpdatePdf and InitializePdf<float>
 * (src/math_functions.cpp:207-262).  d_minmax: {min, max} floats on the device.  No-op if already initialised. */
int aq_tfe_init_grid(const float* d_minmax, aq_tfe_state_t* d_state, void* stream);

/* One batch of the 512-bucket histogram: bucket = round-half-away(x / bucket_size - pdf_offset), samples outside
 * [0, 512) are dropped.  Replaces GetHistogram_cpu / histogramCountKernel + histogramReduceSumKernel
 * (src/math_functions.cpp:367-384, src/math_functions.cu:125-211).
 * d_hist: 512 uint32 counters, ADDED to (zero them for a fresh batch).  d_count (may be NULL): one int64 that is
 * set to n when the state is initialised and to 0 otherwise (the reference skips such batches).
 * d_state must be 16-byte aligned (any block from cudaMalloc is); d_hists rows likewise in aq_tfe_pdf_replay. */
int aq_tfe_histogram(const float* d_x, int64_t n, const aq_tfe_state_t* d_state, uint32_t* d_hist, int64_t* d_count,
                     void* stream);

/* Most batches one aq_tfe_histogram_many call takes. */
#define AQ_TFE_HIST_MANY 16

/* aq_tfe_histogram for m batches that are all resident already (1 <= m <= AQ_TFE_HIST_MANY), in ONE launch: batch b
 * (h_d_x[b], h_n[b] elements) is added into row d_hists + b * row_stride * 512 and sets d_counts[b * row_stride]
 * (row_stride = 1: adjacent rows; a rank of a data-parallel calibration that owns every R-th batch passes R).  The reference has no such
 * call -- TfEnhancedEncodingAnalyzer::updateStats (src/TfEnhancedEncodingAnalyzer.cpp:60-76) takes one tensor at a
 * time -- but a calibration that holds a list of batches gives the same rows this way without the gap between
 * launches, which at 51 MB per batch is a third of the time.  h_d_x and h_n are HOST arrays (of device pointers and
 * of element counts); they are read before the call returns.
 * d_gate (may be NULL): one int32 on the device; when it holds 0 the batches are dropped (counts 0, rows untouched),
 * exactly as when the state is not initialised.  See aq_tfe_select_grid. */
int aq_tfe_histogram_many(const float* const* h_d_x, const int64_t* h_n, int m, int64_t row_stride,
                          const aq_tfe_state_t* d_state, uint32_t* d_hists, int64_t* d_counts, const int32_t* d_gate,
                          void* stream);

/* Bytes of scratch for aq_tfe_offer_grid (zero-filled before first use, 256-byte aligned, left reusable). */
int64_t aq_tfe_offer_grid_workspace_bytes(void);

/* Offers a batch as the one that defines the bucket grid: min and max of d_x in one pass and, in the same launch, the
 * grid set-up from them.  Replaces GetMin + GetMax + InitializePdf in the first-batch branch of UpdatePdf
 * (src/math_functions.cpp:207-262), which the reference runs as two tensor passes, two host read-backs and host
 * arithmetic.  When the state is initialised already the launch returns without touching d_x, so a caller that has
 * not yet learned on the host whether the grid exists can keep offering batches without waiting for the device.
 * d_range (may be NULL): 3 floats {min, max, 1.0f} of the batch, {0, 0, 1} when the pass was skipped.
 * init = 0: only report the range, leave the state alone (grid agreement across ranks, aq_tfe_select_grid). */
int aq_tfe_offer_grid(const float* d_x, int64_t n, aq_tfe_state_t* d_state, float* d_range, int init,
                      void* d_workspace, int64_t workspace_bytes, void* stream);

/* Grid agreement of a data-parallel calibration, decided on the device.  d_ranges: num_ranks triples {min, max,
 * present} of the batches of one round in global order (an all-gather of every rank's d_range; present = 0 for a rank
 * without a batch).  The first present batch whose (min, max) is not (0, 0) defines the grid -- the rule of the
 * sequential reference (src/math_functions.cpp:248-262) applied to the round.  *d_gate becomes 1 when this rank's
 * batch of the round counts and 0 when it must be dropped (no grid yet, or an all-zero batch that precedes the
 * defining one).  No-op with *d_gate = 1 when the state is initialised already.  The reference calibrates in one
 * process and has no counterpart. */
int aq_tfe_select_grid(const float* d_ranges, int num_ranks, int rank, aq_tfe_state_t* d_state, int32_t* d_gate,
                       void* stream);

/* Replays the running mean pdf <- (pdf*k + hist/cnt)/(k+1) over `num_batches` per-batch histograms in order,
 * skipping rows whose count is 0.  Replaces the accumulation loop of UpdatePdf (src/math_functions.cpp:278-287).
 * d_hists: [num_batches, 512] uint32; d_counts: [num_batches] int64; d_pdf: 512 doubles (overwritten);
 * d_iterations: one int32 (overwritten with the number of batches used). */
int aq_tfe_pdf_replay(const uint32_t* d_hists, const int64_t* d_counts, int64_t num_batches, double* d_pdf,
                      int32_t* d_iterations, void* stream);

/* Bytes of scratch for aq_tfe_search. */
int64_t aq_tfe_search_workspace_bytes(void);

/* SQNR grid search; one warp per candidate (delta, offset).  Replaces
 * TfEnhancedEncodingAnalyzer<float>::computeEncoding (src/TfEnhancedEncodingAnalyzer.cpp:78-397).
 * stats_updated: whether any batch was ever offered (selects the all-zero-data encoding when the state is still
 * un-initialised).  d_out_encoding: 5 doubles {min, max, delta, offset, bw} on the device. */
int aq_tfe_search(const aq_tfe_state_t* d_state, const double* d_pdf, int stats_updated, int bw, int symmetric,
                  int strict_symmetric, int unsigned_symmetric, double* d_out_encoding, void* d_workspace,
                  int64_t workspace_bytes, void* stream);

/* aq_tfe_pdf_replay followed by aq_tfe_search in one call: everything TfEnhancedEncodingAnalyzer<float>::computeEncoding
 * (src/TfEnhancedEncodingAnalyzer.cpp:78-113) does after the last updateStats, from the per-batch rows to the
 * encoding.  d_stats_updated (may be NULL): the "any batch was ever offered" flag as an int32 on the device
 * (non-zero = yes), used instead of `stats_updated` when given -- for ranks of a data-parallel calibration, which
 * learn it from the exchanged buffer without a host read.  Workspace as for aq_tfe_search. */
int aq_tfe_compute_encoding(const aq_tfe_state_t* d_state, const uint32_t* d_hists, const int64_t* d_counts,
                            int64_t num_batches, double* d_pdf, int32_t* d_iterations, int stats_updated,
                            const int32_t* d_stats_updated, int bw, int symmetric, int strict_symmetric,
                            int unsigned_symmetric, double* d_out_encoding, void* d_workspace, int64_t workspace_bytes,
                            void* stream);

/* The percentile analyzer on the same per-batch rows: aq_tfe_pdf_replay, then
 * PercentileEncodingAnalyzer<float>::computeEncoding (src/PercentileEncodingAnalyzer.cpp:79-194): the range that holds
 * `percentile` percent of the probability mass from either side, widened to include zero, then the grid of
 * getComputedEncodings (src/quantization_utils.cpp:58-143).  percentile = 100 keeps the observed range.  Statistics
 * (state, rows, counts) are those of aq_tfe_offer_grid / aq_tfe_histogram: the reference's percentile, MSE and
 * TF-Enhanced analyzers all collect the same 512-bucket PDF.  d_stats_updated as for aq_tfe_compute_encoding. */
int aq_tfe_percentile_encoding(const aq_tfe_state_t* d_state, const uint32_t* d_hists, const int64_t* d_counts,
                               int64_t num_batches, double* d_pdf, int32_t* d_iterations, int stats_updated,
                               const int32_t* d_stats_updated, double percentile, int bw, int symmetric,
                               int strict_symmetric, int unsigned_symmetric, double* d_out_encoding, void* stream);

/* Bytes of scratch for aq_tfe_mse_encoding (any content; 256-byte aligned). */
int64_t aq_tfe_mse_workspace_bytes(void);

/* The MSE analyzer on the same per-batch rows: aq_tfe_pdf_replay, then MseEncodingAnalyzer<float>::computeEncoding
 * (src/MseEncodingAnalyzer.cpp:78-267): every (negative-or-zero edge, positive-or-zero edge) pair of the buckets
 * inside the observed range is a candidate range; its cost is the PDF-weighted squared fake-quantization error of the
 * bucket centres (sequential float sum in the reference's order); the first candidate of least cost wins and goes
 * through getComputedEncodings.  The reference evaluates its up to 66,564 candidates one by one on the host; here
 * each gets a thread.  Statistics and d_stats_updated as for aq_tfe_compute_encoding. */
int aq_tfe_mse_encoding(const aq_tfe_state_t* d_state, const uint32_t* d_hists, const int64_t* d_counts,
                        int64_t num_batches, double* d_pdf, int32_t* d_iterations, int stats_updated,
                        const int32_t* d_stats_updated, int bw, int symmetric, int strict_symmetric,
                        int unsigned_symmetric, double* d_out_encoding, void* d_workspace, int64_t workspace_bytes,
                        void* stream);

/* ------------------------------------------------------------------------------------------------
 * aimet_torch v2 histogram statistics (_HistogramObserver) and SQNR range search (SqnrEncodingAnalyzer)
 * ---------------------------------------------------------------------------------------------- */

#define AQ_V2HIST_MAX_BINS 4096 /* the reference's default is 2048 */

/* One histogram of the v2 observer in device memory: this header, then float histogram[bins], then
 * float bin_edges[bins + 1] -- the fields of _Histogram (aimet_torch/v2/quantization/encoding_analyzer.py:57-62).
 * Counts are float32 because the reference keeps them in a float32 tensor (torch.histc output). */
typedef struct
{
    float min;           /* smallest finite value seen */
    float max;           /* largest finite value seen */
    int32_t initialized; /* 0 = no statistics yet */
    int32_t error;       /* 1 = a batch held no finite value (the reference raises ValueError for it) */
} aq_v2hist_head_t;

#define AQ_V2HIST_BYTES(bins) (sizeof(aq_v2hist_head_t) + (size_t) (2 * (bins) + 1) * sizeof(float))

/* Bytes of scratch for aq_v2hist_collect / aq_v2hist_merge (any content; 256-byte aligned). */
int64_t aq_v2hist_scratch_bytes(void);

/* _HistogramObserver.collect_stats for one histogram (encoding_analyzer.py:145-182): finite min / max of the batch,
 * bin edges over that range, torch.histc counts (bin rule of the CPU operator: bin = min(bins - 1,
 * floor(((x - lo) * bins) / (hi - lo))) in float32, elements outside [lo, hi] and NaN ignored), -inf / +inf and
 * stragglers beyond the last edge folded into the end bins.  d_x: `n` elements of `dtype`, dense.  d_batch receives
 * the batch's own _Histogram.  Three launches reading d_x twice; no host synchronisation. */
int aq_v2hist_collect(const void* d_x, int dtype, int64_t n, int bins, aq_v2hist_head_t* d_batch, void* d_scratch,
                      void* stream);

/* _HistogramObserver.merge_stats for one histogram (encoding_analyzer.py:212-262).  state_has_stats = 0: the state
 * adopts d_batch.  Otherwise the range grows to cover both, the old counts are re-binned with the reference's
 * split-and-round rule (sequential float32 additions in the reference's order), and the batch is counted again at the
 * widened range (one pass over d_x: the batch's finite min / max come from d_batch).  d_updates: bins floats of
 * scratch. */
int aq_v2hist_merge(const void* d_x, int dtype, int64_t n, int bins, aq_v2hist_head_t* d_state,
                    const aq_v2hist_head_t* d_batch, int state_has_stats, void* d_scratch, float* d_updates,
                    void* stream);

/* Bytes of scratch for aq_v2hist_sqnr (zero-filled before first use, 256-byte aligned, left reusable). */
int64_t aq_v2hist_sqnr_workspace_bytes(void);

/* SqnrEncodingAnalyzer.compute_encodings_from_stats for one histogram (encoding_analyzer.py:577-725): candidate
 * (delta, offset) pairs -- num_deltas deltas times, when asymmetric, the num_offsets offsets of d_offsets plus the
 * observed offset, each clamped to the observed range; symmetric: d_offsets holds the single offset
 * (-num_steps) // 2 --, the clipping / rounding noise of each over the bin mid-points with the clipped bins weighted
 * by gamma, and the first candidate of least noise.  One warp per candidate.  d_out: {min, max} as float32. */
int aq_v2hist_sqnr(const aq_v2hist_head_t* d_stats, int bins, double num_steps, int symmetric, int num_deltas,
                   const float* d_offsets, int num_offsets, double gamma, float* d_out, void* d_workspace,
                   int64_t workspace_bytes, void* stream);

/* The same three steps for `rows` histograms at once -- a per-channel observer, which the reference serves with a
 * Python loop over channels (encoding_analyzer.py:158-182, 219-262, 586-600).  d_x: rows x n_per_row elements, row r
 * dense at d_x + r * n_per_row (callers move the encoding axes to the front first).  Statistics blocks are
 * block_stride bytes apart (>= AQ_V2HIST_BYTES(bins), a multiple of 16).  d_scratch: rows x
 * aq_v2hist_scratch_bytes(); d_updates: rows x bins floats; d_workspace: rows x aq_v2hist_sqnr_workspace_bytes()
 * (zero-filled before first use); d_out: rows x {min, max}.  rows <= 65535.  One set of launches whatever `rows` is. */
int aq_v2hist_collect_rows(const void* d_x, int dtype, int64_t n_per_row, int rows, int bins,
                           aq_v2hist_head_t* d_batches, int64_t block_stride, void* d_scratch, void* stream);
int aq_v2hist_merge_rows(const void* d_x, int dtype, int64_t n_per_row, int rows, int bins, aq_v2hist_head_t* d_states,
                         const aq_v2hist_head_t* d_batches, int64_t block_stride, int state_has_stats, void* d_scratch,
                         float* d_updates, void* stream);
/* aq_v2hist_collect_rows followed by aq_v2hist_merge_rows of the same batch (what update_stats does,
 * encoding_analyzer.py:283-291), with one counting pass that fills both the batch's own histograms (d_batches) and
 * the histograms over the widened range: two passes over d_x instead of three. */
int aq_v2hist_update_rows(const void* d_x, int dtype, int64_t n_per_row, int rows, int bins, aq_v2hist_head_t* d_states,
                          aq_v2hist_head_t* d_batches, int64_t block_stride, int state_has_stats, void* d_scratch,
                          float* d_updates, void* stream);
/* The same statistics when the batches of one calibration are spread over several workers (one per GPU) and the result
 * must be the sequential one, bit for bit.  merge_stats is sequential (encoding_analyzer.py:212-262): batch b is counted
 * over the range that batches 0..b cover together and the old counts are re-binned, with rounding, each time the range
 * grows.  So: (1) aq_v2hist_range_rows -- finite min / max of one batch (one pass), 4 words per histogram: min bits, max
 * bits, "has a finite value", 1; the workers exchange the records of all batches (a record of zeros = no such batch, so
 * an integer sum over buffers in which every worker fills only its own rows is a valid exchange); (2)
 * aq_v2hist_plan_batches -- from all n_batches x rows records, in batch order, the range every batch is counted over
 * (8 floats per batch and histogram: lo, hi, batch min, batch max, any_finite, first, present, 0); (3)
 * aq_v2hist_count_rows -- one batch counted over its plan's range (second pass): bins + 2 integer words per histogram
 * (bins, below / -inf, above / +inf), ADDED to d_counts (one launch; the table starts zero-filled, which the exchange by
 * integer sum needs anyway); the workers exchange the counts the same way; (4) aq_v2hist_replay_batches --
 * collect_stats of the first batch and merge_stats of every later one from the counts, in batch order, one launch.
 * d_states receives what _HistogramObserver.stats holds after the same batches fed one by one; a batch without a finite
 * value sets `error` (the reference raises ValueError for it). */
int aq_v2hist_range_rows(const void* d_x, int dtype, int64_t n_per_row, int rows, int32_t* d_range, void* d_scratch,
                         void* stream);
int aq_v2hist_plan_batches(const int32_t* d_ranges, int n_batches, int rows, int bins, float* d_plans, void* stream);
int aq_v2hist_count_rows(const void* d_x, int dtype, int64_t n_per_row, int rows, int bins, const float* d_plan,
                         uint32_t* d_counts, void* stream);
/* aq_v2hist_range_rows / aq_v2hist_count_rows for a list of m equally shaped batches in one call (d_xs: HOST array of m
 * device pointers, NULL = no batch at that position): batch i writes the record / counts that start i * stride words
 * into the table it is given and, for the counts, reads the plan i * plan_stride floats into d_plans -- with the
 * strides of a worker's share of the global tables (world_size x the size of one batch's entry) a worker fills its
 * rows of the exchange tables directly. */
int aq_v2hist_range_many(const void* const* d_xs, int m, int dtype, int64_t n_per_row, int rows, int32_t* d_ranges,
                         int64_t stride_words, void* d_scratch, void* stream);
int aq_v2hist_count_many(const void* const* d_xs, int m, int dtype, int64_t n_per_row, int rows, int bins,
                         const float* d_plans, int64_t plan_stride, uint32_t* d_counts, int64_t count_stride,
                         void* stream);
int aq_v2hist_replay_batches(const uint32_t* d_counts, const float* d_plans, int n_batches, int rows, int bins,
                             aq_v2hist_head_t* d_states, int64_t block_stride, void* stream);
int aq_v2hist_sqnr_rows(const aq_v2hist_head_t* d_stats, int64_t block_stride, int rows, int bins, double num_steps,
                        int symmetric, int num_deltas, const float* d_offsets, int num_offsets, double gamma,
                        float* d_out, void* d_workspace, int64_t workspace_bytes, void* stream);

/* aq_v2hist_sqnr_rows plus what the quantizer derives from the chosen range while it calibrates (affine/quantizer.py:
 * 222-246, 317-374): min / max cast to stats_dtype, then float32 scale = (max - min) / num_steps and offset =
 * round(min / scale) - qmin (0 when symmetric).  d_out: rows x {min, max, scale, offset}. */
int aq_v2hist_sqnr_encode_rows(const aq_v2hist_head_t* d_stats, int64_t block_stride, int rows, int bins, double num_steps,
                               int symmetric, int num_deltas, const float* d_offsets, int num_offsets, double gamma,
                               int stats_dtype, double qmin, float* d_out, void* d_workspace, int64_t workspace_bytes,
                               void* stream);

#ifdef __cplusplus
}
#endif
#endif /* AIMET_B200_H_ */
