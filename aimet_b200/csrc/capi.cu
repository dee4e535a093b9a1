// extern "C" surface of libaimet_b200.so: argument validation, host-side encoding arithmetic and dispatch into
// the kernels.  No torch types, no allocation, no implicit synchronisation.
#include <float.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>

#include "common.cuh"
#include "encoding_math.cuh"
#include "kernels.h"

namespace aq
{
// ---- launch accounting / error text ----------------------------------------------------------------
static std::atomic<int64_t> g_launches {0};
static thread_local char g_cuda_error[256] = "";

bool pdl_enabled()
{
    static const bool on = getenv("AQ_NO_PDL") == nullptr;
    return on;
}

void note_launch()
{
    g_launches.fetch_add(1, std::memory_order_relaxed);
}
int cuda_fail(cudaError_t e)
{
    strncpy(g_cuda_error, cudaGetErrorString(e), sizeof(g_cuda_error) - 1);
    g_cuda_error[sizeof(g_cuda_error) - 1] = 0;
    return AQ_ERR_CUDA;
}
int check_launch()
{
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? AQ_OK : cuda_fail(e);
}

// ---- host arithmetic ---------------------------------------------------------------------------------
static void fill_encoding(int bw, double mn, double mx, aq_encoding_t* e)
{
    mn = hmin(mn, 0.0);
    mx = hmax(mx, 0.0);
    mx = hmax(mx, mn + 1e-5);
    double steps = pow(2.0, (double) (uint8_t) bw) - 1.0;
    if (mn == -mx)
        steps -= 1.0;
    e->bw     = bw;
    e->delta  = (mx - mn) / steps;
    e->offset = round(mn / e->delta);
    e->min    = e->offset * e->delta;
    e->max    = e->delta * steps + e->min;
}

static inline bool bad_geom(int64_t n, int64_t num_ch, int64_t inner)
{
    return n < 0 || num_ch < 1 || inner < 1 || (num_ch > 1 && (n % inner) != 0);
}
}   // namespace aq

using namespace aq;

extern "C"
{
int aq_version(void)
{
    return 100;
}

const char* aq_status_string(int s)
{
    switch (s)
    {
    case AQ_OK: return "ok";
    case AQ_ERR_INVALID_ARG: return "invalid argument";
    case AQ_ERR_UNSUPPORTED: return "unsupported combination";
    case AQ_ERR_CUDA: return "CUDA error";
    case AQ_ERR_WORKSPACE: return "workspace missing or too small";
    case AQ_ERR_TOO_LARGE: return "size beyond the documented maximum";
    default: return "unknown status";
    }
}

const char* aq_last_cuda_error(void)
{
    return g_cuda_error;
}

int64_t aq_launch_count(void)
{
    return g_launches.load(std::memory_order_relaxed);
}

int aq_fill_encoding(int bw, double enc_min, double enc_max, aq_encoding_t* h_out)
{
    if (!h_out || bw < 1 || bw > 32)
        return AQ_ERR_INVALID_ARG;
    fill_encoding(bw, enc_min, enc_max, h_out);
    return AQ_OK;
}

int aq_computed_encodings(int bw, double mn, double mx, int symmetric, int strict, int unsigned_sym,
                          aq_encoding_t* h_out)
{
    if (!h_out || bw < 1 || bw > 32)
        return AQ_ERR_INVALID_ARG;
    computed_encodings(bw, mn, mx, symmetric != 0, strict != 0, unsigned_sym != 0, h_out);
    return AQ_OK;
}

int aq_minmax_encoding(int bw, double stat_min, double stat_max, int symmetric, int strict, int unsigned_sym,
                       aq_encoding_t* h_out)
{
    if (!h_out || bw < 1 || bw > 32)
        return AQ_ERR_INVALID_ARG;
    const double mn = hmin(0.0, stat_min);
    double mx       = hmax(0.0, stat_max);
    mx              = hmax(mx, mn + 0.01);
    computed_encodings(bw, mn, mx, symmetric != 0, strict != 0, unsigned_sym != 0, h_out);
    return AQ_OK;
}

int aq_qdq_per_tensor(const float* d_in, float* d_out, int64_t n, double enc_min, double enc_max, int bw,
                      int rounding_mode, void* stream)
{
    if (n < 0 || (n > 0 && (!d_in || !d_out)) || bw < 1 || bw > 32)
        return AQ_ERR_INVALID_ARG;
    if (rounding_mode != AQ_ROUND_NEAREST)
        return AQ_ERR_UNSUPPORTED;
    aq_encoding_t e;
    fill_encoding(bw, enc_min, enc_max, &e);
    return pymo_per_tensor(d_in, d_out, n, (float) e.min, (float) e.max, (float) e.delta, (float) e.offset, 0, 0.0f,
                           (cudaStream_t) stream);
}

int aq_quantize_per_tensor(const float* d_in, float* d_out, int64_t n, double enc_min, double enc_max, int bw,
                           int rounding_mode, int shift_to_signed, void* stream)
{
    if (n < 0 || (n > 0 && (!d_in || !d_out)) || bw < 1 || bw > 32)
        return AQ_ERR_INVALID_ARG;
    if (rounding_mode != AQ_ROUND_NEAREST)
        return AQ_ERR_UNSUPPORTED;
    aq_encoding_t e;
    fill_encoding(bw, enc_min, enc_max, &e);
    unsigned int shift = 0;
    if (shift_to_signed)
        shift = (unsigned int) pow(2.0, (double) (bw - 1));
    return pymo_per_tensor(d_in, d_out, n, (float) e.min, (float) e.max, (float) e.delta, (float) e.offset, 1,
                           (float) shift, (cudaStream_t) stream);
}

int aq_v2_minmax_encoding(const float* d_batch_minmax, float* d_running_minmax, int running_valid, int stats_dtype,
                          int64_t count, double num_steps, int symmetric, double qmin, float* d_out, void* stream)
{
    if (count < 0 || (!d_batch_minmax && !d_running_minmax) || !d_out || !(num_steps > 0) || stats_dtype < AQ_F32 ||
        stats_dtype > AQ_BF16 || (!d_batch_minmax && !running_valid))
        return AQ_ERR_INVALID_ARG;
    return v2_minmax_encode(d_batch_minmax, d_running_minmax, running_valid, stats_dtype, count, num_steps, symmetric, qmin,
                            d_out, (cudaStream_t) stream);
}

int aq_qdq_fp16(const float* d_in, float* d_out, int64_t n, void* stream)
{
    if (n < 0 || (n > 0 && (!d_in || !d_out)))
        return AQ_ERR_INVALID_ARG;
    return fp16_qdq(d_in, d_out, n, (cudaStream_t) stream);
}

static inline bool packed_bw_ok(int bw)
{
    return bw == 1 || bw == 2 || bw == 4 || bw == 8 || bw == 16 || bw == 32;
}

int aq_quantize_packed(const float* d_in, void* d_out, int64_t n, double enc_min, double enc_max, int bw,
                       int rounding_mode, int shift_to_signed, void* stream)
{
    if (n < 0 || (n > 0 && (!d_in || !d_out)) || !packed_bw_ok(bw) || ((uintptr_t) d_out % (bw > 16 ? 4 : (bw > 8 ? 2 : 1))))
        return AQ_ERR_INVALID_ARG;
    if (rounding_mode != AQ_ROUND_NEAREST)
        return AQ_ERR_UNSUPPORTED;
    aq_encoding_t e;
    fill_encoding(bw, enc_min, enc_max, &e);
    return packed_quantize(d_in, d_out, n, e.min, e.max, e.delta, e.offset, bw, shift_to_signed != 0,
                           (cudaStream_t) stream);
}

int aq_dequantize_packed(const void* d_in, float* d_out, int64_t n, double enc_min, double enc_max, int bw,
                         int shift_to_signed, void* stream)
{
    if (n < 0 || (n > 0 && (!d_in || !d_out)) || !packed_bw_ok(bw) || ((uintptr_t) d_in % (bw > 16 ? 4 : (bw > 8 ? 2 : 1))))
        return AQ_ERR_INVALID_ARG;
    aq_encoding_t e;
    fill_encoding(bw, enc_min, enc_max, &e);
    return packed_dequantize(d_in, d_out, n, e.delta, e.offset, bw, shift_to_signed != 0, (cudaStream_t) stream);
}

int aq_qdq_per_channel(const float* d_in, float* d_out, int64_t n, int64_t num_ch, int64_t inner,
                       const float* d_enc_min, const float* d_enc_max, double num_steps, int rounding_mode,
                       void* stream)
{
    if (bad_geom(n, num_ch, inner) || (n > 0 && (!d_in || !d_out)) || !d_enc_min || !d_enc_max || !(num_steps >= 1))
        return AQ_ERR_INVALID_ARG;
    if (rounding_mode != AQ_ROUND_NEAREST)
        return AQ_ERR_UNSUPPORTED;
    return pymo_per_channel(d_in, d_out, n, num_ch, inner, d_enc_min, d_enc_max, nullptr, nullptr, (float) num_steps,
                            1, (cudaStream_t) stream);
}

int aq_qdq_broadcast(const float* d_in, float* d_out, int64_t n, int64_t ndims, const int64_t* h_in_strides,
                     const int64_t* h_enc_strides, const float* d_enc_min, const float* d_enc_max,
                     const float* d_enc_delta, const float* d_enc_offset, void* stream)
{
    if (n < 0 || ndims < 1 || ndims > 8 || !h_in_strides || !h_enc_strides || (n > 0 && (!d_in || !d_out)) ||
        !d_enc_min || !d_enc_max || !d_enc_delta || !d_enc_offset)
        return AQ_ERR_INVALID_ARG;
    for (int64_t d = 0; d < ndims; ++d)
        if (h_in_strides[d] < 1 || h_enc_strides[d] < 0)
            return AQ_ERR_INVALID_ARG;
    // Fast path: the non-broadcast dimensions form one contiguous group [first, last] whose encodings are laid out
    // row-major, i.e. enc_stride[d] * inner == in_stride[d] with inner = in_stride[last].  Then the encoding
    // index is (i / inner) % num_ch and the staged per-channel kernel applies.
    int first = -1, last = -1;
    for (int d = 0; d < ndims; ++d)
        if (h_enc_strides[d] != 0)
        {
            if (first < 0)
                first = d;
            last = d;
        }
    if (first >= 0)
    {
        const int64_t inner = h_in_strides[last];
        bool fast           = true;
        for (int d = first; d <= last; ++d)
            if (h_enc_strides[d] * inner != h_in_strides[d])
                fast = false;
        const int64_t span = (first == 0) ? n : h_in_strides[first - 1];
        if (fast && span % inner == 0 && n % inner == 0 && (n / inner) % (span / inner) == 0)
            return pymo_per_channel(d_in, d_out, n, span / inner, inner, d_enc_min, d_enc_max, d_enc_delta,
                                    d_enc_offset, 0.0f, 0, (cudaStream_t) stream);
    }
    BroadcastArgs a;
    a.in = d_in, a.out = d_out, a.n = n, a.ndims = (int) ndims;
    for (int d = 0; d < 8; ++d)
    {
        a.in_strides[d]  = d < ndims ? h_in_strides[d] : 1;
        a.enc_strides[d] = d < ndims ? h_enc_strides[d] : 0;
        a.in_m64[d]      = magic64(a.in_strides[d]);
    }
    a.mn = d_enc_min, a.mx = d_enc_max, a.dl = d_enc_delta, a.of = d_enc_offset;
    return pymo_broadcast(a, (cudaStream_t) stream);
}

int aq_ste_backward_v1(const float* d_x, const float* d_grad, float* d_dx, int64_t n, int64_t num_ch, int64_t inner,
                       const float* d_enc_min, const float* d_enc_max, void* stream)
{
    if (bad_geom(n, num_ch, inner) || (n > 0 && (!d_x || !d_grad || !d_dx)) || !d_enc_min || !d_enc_max)
        return AQ_ERR_INVALID_ARG;
    SteArgs a;
    a.x = d_x, a.g = d_grad, a.dx = d_dx, a.n = n, a.enc_min = d_enc_min, a.enc_max = d_enc_max;
    a.geom.num_ch = num_ch, a.geom.inner = inner;
    return ste_v1(a, (cudaStream_t) stream);
}

int aq_v2_quantize(const void* d_x, void* d_y, uint8_t* d_mask, int dtype, int64_t n, int64_t num_ch, int64_t inner,
                   const float* d_scale, const float* d_offset, double qmin, double qmax, int out_kind,
                   int narrow_internal, void* stream)
{
    if (bad_geom(n, num_ch, inner) || (n > 0 && (!d_x || !d_y)) || !d_scale || !d_offset || qmin > qmax ||
        (out_kind != AQ_V2_OUT_QDQ && out_kind != AQ_V2_OUT_CODES) || dtype < AQ_F32 || dtype > AQ_BF16)
        return AQ_ERR_INVALID_ARG;
    // the grid bounds must be exact in the internal dtype (the caller checks representability like the reference)
    if (narrow_internal != AQ_V2_INTERNAL_F64 && ((double) (float) qmin != qmin || (double) (float) qmax != qmax))
        return AQ_ERR_UNSUPPORTED;
    V2Args a;
    a.x = d_x, a.y = d_y, a.mask = d_mask, a.n = n, a.scale = d_scale, a.offset = d_offset;
    a.qmin = (float) qmin, a.qmax = (float) qmax, a.out_kind = out_kind, a.dequant_only = 0;
    a.qmin_wide = qmin, a.qmax_wide = qmax;
    a.geom.num_ch = num_ch, a.geom.inner = inner;
    return v2_launch(a, dtype, narrow_internal, (cudaStream_t) stream);
}

int aq_v2_dequantize(const void* d_x, void* d_y, int dtype, int64_t n, int64_t num_ch, int64_t inner,
                     const float* d_scale, const float* d_offset, int narrow_internal, void* stream)
{
    if (bad_geom(n, num_ch, inner) || (n > 0 && (!d_x || !d_y)) || !d_scale || !d_offset || dtype < AQ_F32 ||
        dtype > AQ_BF16)
        return AQ_ERR_INVALID_ARG;
    V2Args a;
    a.x = d_x, a.y = d_y, a.mask = nullptr, a.n = n, a.scale = d_scale, a.offset = d_offset;
    a.qmin = 0, a.qmax = 0, a.qmin_wide = 0, a.qmax_wide = 0, a.out_kind = AQ_V2_OUT_QDQ, a.dequant_only = 1;
    a.geom.num_ch = num_ch, a.geom.inner = inner;
    return v2_launch(a, dtype, narrow_internal, (cudaStream_t) stream);
}

int aq_v2_qdq_backward_params(const void* d_x, const void* d_grad, const uint8_t* d_mask, float* d_dscale,
                              float* d_doffset, int dtype, int64_t n, int64_t num_ch, int64_t inner,
                              const float* d_scale, const float* d_offset, double qmin, double qmax, void* stream)
{
    if (bad_geom(n, num_ch, inner) || (n > 0 && (!d_x || !d_grad || !d_mask)) || (!d_dscale && !d_doffset) ||
        !d_scale || !d_offset || qmin > qmax || dtype < AQ_F32 || dtype > AQ_BF16)
        return AQ_ERR_INVALID_ARG;
    V2GradArgs a;
    a.x = d_x, a.grad = d_grad, a.mask = d_mask, a.dscale = d_dscale, a.doffset = d_doffset, a.n = n;
    a.scale = d_scale, a.offset = d_offset, a.qmin = (float) qmin, a.qmax = (float) qmax;
    a.geom.num_ch = num_ch, a.geom.inner = inner;
    return v2_param_grad(a, dtype, 0, (cudaStream_t) stream);
}

int aq_v2_qdq_backward_params_reduced(const void* d_x, const void* d_grad, const uint8_t* d_mask, float* d_dscale,
                                      float* d_doffset, int dtype, int64_t n, int64_t num_ch, int64_t inner,
                                      const float* d_scale, const float* d_offset, double qmin, double qmax,
                                      void* stream)
{
    if (bad_geom(n, num_ch, inner) || (n > 0 && (!d_x || !d_grad || !d_mask)) || (!d_dscale && !d_doffset) ||
        !d_scale || !d_offset || qmin > qmax || dtype < AQ_F32 || dtype > AQ_BF16)
        return AQ_ERR_INVALID_ARG;
    V2GradArgs a;
    a.x = d_x, a.grad = d_grad, a.mask = d_mask, a.dscale = d_dscale, a.doffset = d_doffset, a.n = n;
    a.scale = d_scale, a.offset = d_offset, a.qmin = (float) qmin, a.qmax = (float) qmax;
    a.geom.num_ch = num_ch, a.geom.inner = inner;
    return v2_param_grad(a, dtype, 1, (cudaStream_t) stream);
}

int aq_v2_qdq_backward(const void* d_grad, const uint8_t* d_mask, void* d_dx, int dtype, int64_t n, void* stream)
{
    if (n < 0 || (n > 0 && (!d_grad || !d_mask || !d_dx)) || dtype < AQ_F32 || dtype > AQ_BF16)
        return AQ_ERR_INVALID_ARG;
    return v2_backward(d_grad, d_mask, d_dx, dtype, n, (cudaStream_t) stream);
}

int64_t aq_minmax_workspace_bytes(int64_t n, int64_t num_ch, int64_t inner)
{
    if (bad_geom(n, num_ch, inner))
        return AQ_ERR_INVALID_ARG;
    return minmax_workspace_bytes(n, num_ch, inner);
}

int aq_minmax(const void* d_x, int dtype, int64_t n, int64_t num_ch, int64_t inner, float* d_out_min,
              float* d_out_max, int propagate_nan, int accumulate, void* d_workspace, int64_t workspace_bytes,
              void* stream)
{
    if (bad_geom(n, num_ch, inner) || (n > 0 && !d_x) || !d_out_min || !d_out_max || dtype < AQ_F32 ||
        dtype > AQ_BF16)
        return AQ_ERR_INVALID_ARG;
    if (num_ch > 1 && n / inner % num_ch != 0)
        return AQ_ERR_INVALID_ARG;
    if (!d_workspace || ((uintptr_t) d_workspace % 256) != 0)
        return AQ_ERR_WORKSPACE;
    return minmax_dispatch(d_x, dtype, n, num_ch, inner, d_out_min, d_out_max, propagate_nan, accumulate, d_workspace,
                           workspace_bytes, (cudaStream_t) stream);
}

int aq_minmax_static(const void* d_x, int dtype, int64_t n, int64_t num_ch, int64_t inner, float* d_out_min,
                     float* d_out_max, int propagate_nan, void* stream)
{
    if (bad_geom(n, num_ch, inner) || (n > 0 && !d_x) || !d_out_min || !d_out_max || dtype < AQ_F32 ||
        dtype > AQ_BF16)
        return AQ_ERR_INVALID_ARG;
    if (num_ch > 1 && n / inner % num_ch != 0)
        return AQ_ERR_INVALID_ARG;
    return minmax_static(d_x, dtype, n, num_ch, inner, d_out_min, d_out_max, propagate_nan, (cudaStream_t) stream);
}

int aq_tfe_init_grid(const float* d_minmax, aq_tfe_state_t* d_state, void* stream)
{
    if (!d_minmax || !d_state)
        return AQ_ERR_INVALID_ARG;
    return tfe_init_grid(d_minmax, d_state, (cudaStream_t) stream);
}

int aq_tfe_histogram(const float* d_x, int64_t n, const aq_tfe_state_t* d_state, uint32_t* d_hist, int64_t* d_count,
                     void* stream)
{
    if (n < 0 || (n > 0 && !d_x) || !d_state || !d_hist)
        return AQ_ERR_INVALID_ARG;
    if (((uintptr_t) d_state % 16) || ((uintptr_t) d_x % 4) || ((uintptr_t) d_hist % 4) || ((uintptr_t) d_count % 8))
        return AQ_ERR_INVALID_ARG;   // the kernels use 16-byte loads of the state
    if (n > 0x7fffffffLL)
        return AQ_ERR_TOO_LARGE;   // the reference counts elements in an int; so does the PDF replay
    return tfe_histogram(d_x, n, d_state, d_hist, d_count, nullptr, (cudaStream_t) stream);
}

int aq_tfe_histogram_many(const float* const* h_d_x, const int64_t* h_n, int m, int64_t row_stride,
                          const aq_tfe_state_t* d_state, uint32_t* d_hists, int64_t* d_counts, const int32_t* d_gate,
                          void* stream)
{
    if (m < 1 || m > AQ_TFE_HIST_MANY || row_stride < 1 || !h_d_x || !h_n || !d_state || !d_hists)
        return AQ_ERR_INVALID_ARG;
    if (((uintptr_t) d_state % 16) || ((uintptr_t) d_hists % 4) || ((uintptr_t) d_counts % 8) || ((uintptr_t) d_gate % 4))
        return AQ_ERR_INVALID_ARG;
    for (int b = 0; b < m; ++b)
    {
        if (h_n[b] < 0 || (h_n[b] > 0 && !h_d_x[b]) || ((uintptr_t) h_d_x[b] % 4))
            return AQ_ERR_INVALID_ARG;
        if (h_n[b] > 0x7fffffffLL)
            return AQ_ERR_TOO_LARGE;
    }
    return tfe_histogram_many(h_d_x, h_n, m, row_stride, d_state, d_hists, d_counts, d_gate, (cudaStream_t) stream);
}

int64_t aq_tfe_offer_grid_workspace_bytes(void)
{
    return 256 + (int64_t) kNumSMs * 4 * (int64_t) sizeof(float2);
}

int aq_tfe_offer_grid(const float* d_x, int64_t n, aq_tfe_state_t* d_state, float* d_range, int init,
                      void* d_workspace, int64_t workspace_bytes, void* stream)
{
    if (n < 0 || (n > 0 && !d_x) || !d_state || ((uintptr_t) d_x % 4) || ((uintptr_t) d_state % 16) ||
        ((uintptr_t) d_range % 4))
        return AQ_ERR_INVALID_ARG;
    if (n > 0x7fffffffLL)
        return AQ_ERR_TOO_LARGE;
    if (!d_workspace || ((uintptr_t) d_workspace % 256) != 0)
        return AQ_ERR_WORKSPACE;
    return tfe_offer_grid(d_x, n, d_state, d_range, init, d_workspace, workspace_bytes, (cudaStream_t) stream);
}

int aq_tfe_select_grid(const float* d_ranges, int num_ranks, int rank, aq_tfe_state_t* d_state, int32_t* d_gate,
                       void* stream)
{
    if (!d_ranges || num_ranks < 1 || rank < 0 || rank >= num_ranks || !d_state || !d_gate ||
        ((uintptr_t) d_ranges % 4) || ((uintptr_t) d_state % 16) || ((uintptr_t) d_gate % 4))
        return AQ_ERR_INVALID_ARG;
    return tfe_select_grid(d_ranges, num_ranks, rank, d_state, d_gate, (cudaStream_t) stream);
}

int aq_tfe_pdf_replay(const uint32_t* d_hists, const int64_t* d_counts, int64_t num_batches, double* d_pdf,
                      int32_t* d_iterations, void* stream)
{
    if (num_batches < 0 || (num_batches > 0 && (!d_hists || !d_counts)) || !d_pdf || !d_iterations)
        return AQ_ERR_INVALID_ARG;
    if (((uintptr_t) d_hists % 16) || ((uintptr_t) d_counts % 8) || ((uintptr_t) d_pdf % 8))
        return AQ_ERR_INVALID_ARG;   // rows are fetched with 16-byte asynchronous copies
    return tfe_pdf_replay(d_hists, d_counts, num_batches, d_pdf, d_iterations, (cudaStream_t) stream);
}

int64_t aq_tfe_search_workspace_bytes(void)
{
    return tfe_search_workspace_bytes();
}

int aq_tfe_search(const aq_tfe_state_t* d_state, const double* d_pdf, int stats_updated, int bw, int symmetric,
                  int strict, int unsigned_sym, double* d_out_encoding, void* d_workspace, int64_t workspace_bytes,
                  void* stream)
{
    if (!d_state || !d_pdf || !d_out_encoding || bw < 1 || bw > 32)
        return AQ_ERR_INVALID_ARG;
    if (!d_workspace || ((uintptr_t) d_workspace % 256) != 0)
        return AQ_ERR_WORKSPACE;
    return tfe_search(d_state, d_pdf, stats_updated, nullptr, bw, symmetric, strict, unsigned_sym, d_out_encoding,
                      d_workspace, workspace_bytes, (cudaStream_t) stream);
}

int aq_tfe_compute_encoding(const aq_tfe_state_t* d_state, const uint32_t* d_hists, const int64_t* d_counts,
                            int64_t num_batches, double* d_pdf, int32_t* d_iterations, int stats_updated,
                            const int32_t* d_stats_updated, int bw, int symmetric, int strict, int unsigned_sym,
                            double* d_out_encoding, void* d_workspace, int64_t workspace_bytes, void* stream)
{
    if (!d_state || !d_out_encoding || bw < 1 || bw > 32 || ((uintptr_t) d_stats_updated % 4))
        return AQ_ERR_INVALID_ARG;
    if (!d_workspace || ((uintptr_t) d_workspace % 256) != 0)
        return AQ_ERR_WORKSPACE;
    const int rc = aq_tfe_pdf_replay(d_hists, d_counts, num_batches, d_pdf, d_iterations, stream);
    if (rc != AQ_OK)
        return rc;
    return tfe_search(d_state, d_pdf, stats_updated, d_stats_updated, bw, symmetric, strict, unsigned_sym,
                      d_out_encoding, d_workspace, workspace_bytes, (cudaStream_t) stream);
}

int aq_tfe_percentile_encoding(const aq_tfe_state_t* d_state, const uint32_t* d_hists, const int64_t* d_counts,
                               int64_t num_batches, double* d_pdf, int32_t* d_iterations, int stats_updated,
                               const int32_t* d_stats_updated, double percentile, int bw, int symmetric, int strict,
                               int unsigned_sym, double* d_out_encoding, void* stream)
{
    if (!d_state || !d_out_encoding || bw < 1 || bw > 32 || ((uintptr_t) d_stats_updated % 4) ||
        !(percentile >= 0.0 && percentile <= 100.0))
        return AQ_ERR_INVALID_ARG;
    const int rc = aq_tfe_pdf_replay(d_hists, d_counts, num_batches, d_pdf, d_iterations, stream);
    if (rc != AQ_OK)
        return rc;
    return tfe_percentile(d_state, d_pdf, stats_updated, d_stats_updated, (float) percentile, bw, symmetric, strict,
                          unsigned_sym, d_out_encoding, (cudaStream_t) stream);
}

int64_t aq_tfe_mse_workspace_bytes(void)
{
    return tfe_mse_workspace_bytes();
}

int aq_tfe_mse_encoding(const aq_tfe_state_t* d_state, const uint32_t* d_hists, const int64_t* d_counts,
                        int64_t num_batches, double* d_pdf, int32_t* d_iterations, int stats_updated,
                        const int32_t* d_stats_updated, int bw, int symmetric, int strict, int unsigned_sym,
                        double* d_out_encoding, void* d_workspace, int64_t workspace_bytes, void* stream)
{
    if (!d_state || !d_out_encoding || bw < 1 || bw > 32 || ((uintptr_t) d_stats_updated % 4))
        return AQ_ERR_INVALID_ARG;
    if (!d_workspace || ((uintptr_t) d_workspace % 256) != 0 || workspace_bytes < tfe_mse_workspace_bytes())
        return AQ_ERR_WORKSPACE;
    const int rc = aq_tfe_pdf_replay(d_hists, d_counts, num_batches, d_pdf, d_iterations, stream);
    if (rc != AQ_OK)
        return rc;
    return tfe_mse(d_state, d_pdf, stats_updated, d_stats_updated, bw, symmetric, strict, unsigned_sym, d_out_encoding,
                   d_workspace, (cudaStream_t) stream);
}

int64_t aq_v2hist_scratch_bytes(void)
{
    return v2hist_scratch_bytes();
}

static inline bool bad_v2hist(const void* d_x, int dtype, int64_t n, int bins, const void* a, const void* b)
{
    return n < 0 || (n > 0 && !d_x) || dtype < AQ_F32 || dtype > AQ_BF16 || bins < 1 || bins > AQ_V2HIST_MAX_BINS ||
           !a || !b || ((uintptr_t) a % 16) || ((uintptr_t) b % 256);
}

int aq_v2hist_collect(const void* d_x, int dtype, int64_t n, int bins, aq_v2hist_head_t* d_batch, void* d_scratch,
                      void* stream)
{
    if (bad_v2hist(d_x, dtype, n, bins, d_batch, d_scratch))
        return AQ_ERR_INVALID_ARG;
    return v2hist_collect(d_x, dtype, n, bins, d_batch, d_scratch, (cudaStream_t) stream);
}

int aq_v2hist_merge(const void* d_x, int dtype, int64_t n, int bins, aq_v2hist_head_t* d_state,
                    const aq_v2hist_head_t* d_batch, int state_has_stats, void* d_scratch, float* d_updates,
                    void* stream)
{
    if (bad_v2hist(d_x, dtype, n, bins, d_state, d_scratch) || !d_batch || !d_updates)
        return AQ_ERR_INVALID_ARG;
    return v2hist_merge(d_x, dtype, n, bins, d_state, d_batch, state_has_stats, d_scratch, d_updates,
                        (cudaStream_t) stream);
}

static inline bool bad_v2hist_rows(int rows, int64_t block_stride, int bins)
{
    return rows < 1 || block_stride < (int64_t) AQ_V2HIST_BYTES(bins) || (block_stride % 16) != 0;
}

int aq_v2hist_collect_rows(const void* d_x, int dtype, int64_t n_per_row, int rows, int bins,
                           aq_v2hist_head_t* d_batches, int64_t block_stride, void* d_scratch, void* stream)
{
    if (bad_v2hist(d_x, dtype, n_per_row, bins, d_batches, d_scratch) || bad_v2hist_rows(rows, block_stride, bins))
        return AQ_ERR_INVALID_ARG;
    return v2hist_collect_rows(d_x, dtype, n_per_row, rows, bins, d_batches, block_stride, d_scratch,
                               (cudaStream_t) stream);
}

int aq_v2hist_merge_rows(const void* d_x, int dtype, int64_t n_per_row, int rows, int bins, aq_v2hist_head_t* d_states,
                         const aq_v2hist_head_t* d_batches, int64_t block_stride, int state_has_stats, void* d_scratch,
                         float* d_updates, void* stream)
{
    if (bad_v2hist(d_x, dtype, n_per_row, bins, d_states, d_scratch) || !d_batches || !d_updates ||
        bad_v2hist_rows(rows, block_stride, bins))
        return AQ_ERR_INVALID_ARG;
    return v2hist_merge_rows(d_x, dtype, n_per_row, rows, bins, d_states, d_batches, block_stride, state_has_stats,
                             d_scratch, d_updates, (cudaStream_t) stream);
}

int aq_v2hist_update_rows(const void* d_x, int dtype, int64_t n_per_row, int rows, int bins, aq_v2hist_head_t* d_states,
                          aq_v2hist_head_t* d_batches, int64_t block_stride, int state_has_stats, void* d_scratch,
                          float* d_updates, void* stream)
{
    if (bad_v2hist(d_x, dtype, n_per_row, bins, d_states, d_scratch) || !d_batches || !d_updates ||
        bad_v2hist_rows(rows, block_stride, bins))
        return AQ_ERR_INVALID_ARG;
    return v2hist_update_rows(d_x, dtype, n_per_row, rows, bins, d_states, d_batches, block_stride, state_has_stats,
                              d_scratch, d_updates, (cudaStream_t) stream);
}

int aq_v2hist_range_rows(const void* d_x, int dtype, int64_t n_per_row, int rows, int32_t* d_range, void* d_scratch,
                         void* stream)
{
    if (!d_x || !d_range || !d_scratch || n_per_row < 1 || rows < 1 ||
        (dtype != AQ_F32 && dtype != AQ_F16 && dtype != AQ_BF16))
        return AQ_ERR_INVALID_ARG;
    return v2hist_range_rows(d_x, dtype, n_per_row, rows, d_range, d_scratch, (cudaStream_t) stream);
}

int aq_v2hist_plan_batches(const int32_t* d_ranges, int n_batches, int rows, int bins, float* d_plans, void* stream)
{
    if (!d_ranges || !d_plans || n_batches < 1 || rows < 1 || bins < 1 || bins > AQ_V2HIST_MAX_BINS)
        return AQ_ERR_INVALID_ARG;
    return v2hist_plan_batches(d_ranges, n_batches, rows, bins, d_plans, (cudaStream_t) stream);
}

int aq_v2hist_count_rows(const void* d_x, int dtype, int64_t n_per_row, int rows, int bins, const float* d_plan,
                         uint32_t* d_counts, void* stream)
{
    if (!d_x || !d_plan || !d_counts || n_per_row < 1 || rows < 1 || bins < 1 ||
        bins > AQ_V2HIST_MAX_BINS || (dtype != AQ_F32 && dtype != AQ_F16 && dtype != AQ_BF16))
        return AQ_ERR_INVALID_ARG;
    return v2hist_count_rows(d_x, dtype, n_per_row, rows, bins, d_plan, d_counts, (cudaStream_t) stream);
}

int aq_v2hist_range_many(const void* const* d_xs, int m, int dtype, int64_t n_per_row, int rows, int32_t* d_ranges,
                         int64_t stride_words, void* d_scratch, void* stream)
{
    if (!d_xs || m < 1 || !d_ranges || !d_scratch || n_per_row < 1 || rows < 1 || stride_words < 4 * (int64_t) rows ||
        (dtype != AQ_F32 && dtype != AQ_F16 && dtype != AQ_BF16))
        return AQ_ERR_INVALID_ARG;
    return v2hist_range_many(d_xs, m, dtype, n_per_row, rows, d_ranges, stride_words, d_scratch, (cudaStream_t) stream);
}

int aq_v2hist_count_many(const void* const* d_xs, int m, int dtype, int64_t n_per_row, int rows, int bins,
                         const float* d_plans, int64_t plan_stride, uint32_t* d_counts, int64_t count_stride,
                         void* stream)
{
    if (!d_xs || m < 1 || !d_plans || !d_counts || n_per_row < 1 || rows < 1 || bins < 1 ||
        bins > AQ_V2HIST_MAX_BINS || plan_stride < 8 * (int64_t) rows || count_stride < (int64_t) rows * (bins + 2) ||
        (dtype != AQ_F32 && dtype != AQ_F16 && dtype != AQ_BF16))
        return AQ_ERR_INVALID_ARG;
    return v2hist_count_many(d_xs, m, dtype, n_per_row, rows, bins, d_plans, plan_stride, d_counts, count_stride,
                             (cudaStream_t) stream);
}

int aq_v2hist_replay_batches(const uint32_t* d_counts, const float* d_plans, int n_batches, int rows, int bins,
                             aq_v2hist_head_t* d_states, int64_t block_stride, void* stream)
{
    if (!d_counts || !d_plans || !d_states || n_batches < 1 || bins < 1 || bins > AQ_V2HIST_MAX_BINS ||
        bad_v2hist_rows(rows, block_stride, bins))
        return AQ_ERR_INVALID_ARG;
    return v2hist_replay_batches(d_counts, d_plans, n_batches, rows, bins, d_states, block_stride, (cudaStream_t) stream);
}

int aq_v2hist_sqnr_rows(const aq_v2hist_head_t* d_stats, int64_t block_stride, int rows, int bins, double num_steps,
                        int symmetric, int num_deltas, const float* d_offsets, int num_offsets, double gamma,
                        float* d_out, void* d_workspace, int64_t workspace_bytes, void* stream)
{
    if (!d_stats || bins < 1 || bins > AQ_V2HIST_MAX_BINS || !(num_steps > 0) || num_deltas < 2 || !d_offsets ||
        num_offsets < 1 || !d_out || bad_v2hist_rows(rows, block_stride, bins))
        return AQ_ERR_INVALID_ARG;
    if (!d_workspace || ((uintptr_t) d_workspace % 256) != 0)
        return AQ_ERR_WORKSPACE;
    return v2hist_sqnr_rows(d_stats, block_stride, rows, bins, num_steps, symmetric, num_deltas, d_offsets, num_offsets,
                            gamma, d_out, d_workspace, workspace_bytes, (cudaStream_t) stream);
}

int aq_v2hist_sqnr_encode_rows(const aq_v2hist_head_t* d_stats, int64_t block_stride, int rows, int bins, double num_steps,
                               int symmetric, int num_deltas, const float* d_offsets, int num_offsets, double gamma,
                               int stats_dtype, double qmin, float* d_out, void* d_workspace, int64_t workspace_bytes,
                               void* stream)
{
    if (!d_stats || bins < 1 || bins > AQ_V2HIST_MAX_BINS || !(num_steps > 0) || num_deltas < 2 || !d_offsets ||
        num_offsets < 1 || !d_out || bad_v2hist_rows(rows, block_stride, bins) || stats_dtype < AQ_F32 ||
        stats_dtype > AQ_BF16)
        return AQ_ERR_INVALID_ARG;
    if (!d_workspace || ((uintptr_t) d_workspace % 256) != 0)
        return AQ_ERR_WORKSPACE;
    return v2hist_sqnr_rows(d_stats, block_stride, rows, bins, num_steps, symmetric, num_deltas, d_offsets, num_offsets,
                            gamma, d_out, d_workspace, workspace_bytes, (cudaStream_t) stream, 4, stats_dtype, qmin);
}

int64_t aq_v2hist_sqnr_workspace_bytes(void)
{
    return v2hist_sqnr_workspace_bytes();
}

int aq_v2hist_sqnr(const aq_v2hist_head_t* d_stats, int bins, double num_steps, int symmetric, int num_deltas,
                   const float* d_offsets, int num_offsets, double gamma, float* d_out, void* d_workspace,
                   int64_t workspace_bytes, void* stream)
{
    if (!d_stats || bins < 1 || bins > AQ_V2HIST_MAX_BINS || !(num_steps > 0) || num_deltas < 2 || !d_offsets ||
        num_offsets < 1 || !d_out)
        return AQ_ERR_INVALID_ARG;
    if (!d_workspace || ((uintptr_t) d_workspace % 256) != 0)
        return AQ_ERR_WORKSPACE;
    return v2hist_sqnr(d_stats, bins, num_steps, symmetric, num_deltas, d_offsets, num_offsets, gamma, d_out,
                       d_workspace, workspace_bytes, (cudaStream_t) stream);
}

}   // extern "C"