// TF-Enhanced SQNR grid search on the device: one warp per candidate (delta, offset).
//
// Follows DlQuantization/src/TfEnhancedEncodingAnalyzer.cpp (DTYPE = float): candidate lists :177-253,
// clamping :149-175, observed range :255-291, cost :293-355, first-strict-minimum selection :115-147 and the
// final encoding :357-397.  The mixed float/double arithmetic and the ascending-bucket summation order of the
// reference are kept, because near-tie candidates would otherwise flip: the 512 per-bucket terms of a candidate
// are computed by the warp's lanes in parallel, but each of the three cost sums is added up in bucket order by a
// single lane.
#include <float.h>
#include <limits.h>
#include <math.h>

#include "common.cuh"
#include "encoding_math.cuh"
#include "kernels.h"

namespace aq
{

constexpr int kAsymDeltas  = 17;
constexpr int kAsymOffsets = 21;
constexpr int kAsymSlots   = kAsymDeltas * kAsymOffsets + 1;   // 358
constexpr int kSymSlots    = 128;                              // loop runs 101 (or 100/102) times
constexpr int kMaxSlots    = 384;
constexpr int kSearchWarps = 4;                                // warps (= candidates) per CTA

struct SearchWs
{
    unsigned int ticket;
    int pad[3];
    double cost[kMaxSlots];
    float delta[kMaxSlots];
    int offset[kMaxSlots];
    int valid[kMaxSlots];
};

int64_t tfe_search_workspace_bytes()
{
    return (int64_t) ((sizeof(SearchWs) + 255) / 256 * 256);
}

// double -> int like x86-64 cvttsd2si: out of range or NaN gives INT_MIN
__device__ __forceinline__ int to_int_x86(double v)
{
    if (!(v > -2147483649.0 && v < 2147483648.0))
        return INT_MIN;
    return (int) v;
}
__device__ __forceinline__ int to_int_x86(float v)
{
    if (!(v >= -2147483648.0f && v < 2147483648.0f))
        return INT_MIN;
    return (int) v;
}
// std::max(a,b) = (a<b)?b:a ; std::min(a,b) = (b<a)?b:a
template <typename T>
__device__ __forceinline__ T smax(T a, T b)
{
    return (a < b) ? b : a;
}
template <typename T>
__device__ __forceinline__ T smin(T a, T b)
{
    return (b < a) ? b : a;
}

// _clampToObservedMinMax (:149-175)
__device__ bool clamp_candidate(float obs_min, float obs_max, float steps, float& delta, int& offset)
{
    float t_min = smax(__fmul_rn(delta, (float) offset), -FLT_MAX);
    float t_max = smin(__fmul_rn(delta, __fadd_rn((float) offset, steps)), FLT_MAX);
    if (t_min < obs_min && t_max > obs_max)
        return false;
    t_min = smax(obs_min, t_min);
    t_max = smin(obs_max, t_max);
    if (t_min == t_max)
        return false;
    delta  = __double2float_rn(__ddiv_rn(__dsub_rn((double) t_max, (double) t_min), (double) steps));
    offset = to_int_x86(round_half_away(__fdiv_rn(t_min, delta)));
    return true;
}

struct SearchArgs
{
    const aq_tfe_state_t* st;
    const double* pdf;
    int stats_updated, bw, symmetric, strict, unsigned_sym;
    const int32_t* stats_updated_dev;   // when not null: the flag lives on the device (non-zero = updated)
    float steps;   // (float)(2^bw - 1), computed on the host
    double* out;   // {min, max, delta, offset, bw}
    SearchWs* ws;
    int slots;
};

__global__ void __launch_bounds__(kSearchWarps * 32) tfe_search_kernel(SearchArgs a)
{
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int slot = blockIdx.x * kSearchWarps + warp;
    __shared__ double s_term[kSearchWarps][AQ_PDF_SIZE];   // bottom-saturation or in-range term of a bucket
    __shared__ double s_top[kSearchWarps][AQ_PDF_SIZE];    // top-saturation term (ranges may overlap, see below)
    __shared__ bool s_last;

    const int initialized = a.st->initialized;
    float steps           = a.steps;

    if (!initialized)
    {
        // computeEncoding (:78-107): no PDF yet
        if (blockIdx.x == 0 && threadIdx.x == 0)
        {
            double e[5] = {0, 0, 0, 0, 0};
            if (a.stats_updated_dev ? (*a.stats_updated_dev != 0) : (a.stats_updated != 0))
            {
                const double d = __ddiv_rn(2.0, (double) (int) steps);
                const double o = floor(__ddiv_rn(-1.0, d));
                e[0]           = __dmul_rn(o, d);
                e[1]           = __dadd_rn(e[0], __dmul_rn((double) (int) steps, d));
                e[2]           = d;
                e[3]           = o;
                e[4]           = a.bw;
            }
            for (int i = 0; i < 5; ++i)
                a.out[i] = e[i];
        }
        return;
    }

    // ---- observed range (_findRangeOfAggregateStats :255-291), computed redundantly by every warp -----------
    const double* __restrict__ xl  = a.st->x_left;
    const double* __restrict__ pdf = a.pdf;
    int first = AQ_PDF_SIZE, last = 0;
    for (int i = lane; i < AQ_PDF_SIZE; i += 32)
        if (pdf[i] > 0)
        {
            first = min(first, i);
            last  = max(last, i);
        }
    first = __reduce_min_sync(0xffffffffu, first);
    last  = __reduce_max_sync(0xffffffffu, last);
    float obs_mn = (first < AQ_PDF_SIZE) ? (float) xl[first] : (float) xl[0];
    float obs_mx = (last > 0) ? (float) xl[last] : (float) xl[AQ_PDF_SIZE - 1];
    obs_mn       = smin(obs_mn, 0.0f);
    obs_mx       = smax(obs_mx, 0.0f);
    obs_mx       = smax(obs_mx, __fadd_rn(obs_mn, (float) 0.01));

    // ---- this warp's candidate ------------------------------------------------------------------------------
    float c_delta = 0.f;
    int c_offset  = 0;
    bool valid    = false;
    if (a.symmetric)
    {
        if (a.strict)
            steps = __fsub_rn(steps, 1.0f);
        float delta_max;
        int t_off;
        if (obs_mn == 0.0f && a.unsigned_sym)
        {
            delta_max = __fdiv_rn(obs_mx, steps);
            t_off     = 0;
        }
        else
        {
            const float amax = smax(fabsf(obs_mx), fabsf(obs_mn));
            delta_max        = __double2float_rn(__ddiv_rn((double) amax, __ddiv_rn((double) steps, 2.0)));
            t_off            = (int) floorf(__fdiv_rn(-steps, 2.0f));
        }
        // for (float f = 1/100; f <= 1 + 1/100; f += 1/100): float accumulation through double, replayed literally
        float f = (float) (1.0 / 100);
        int k   = 0;
        while ((double) f <= 1 + 1.0 / 100 && k < slot)
        {
            f = __double2float_rn(__dadd_rn((double) f, 1.0 / 100));
            ++k;
        }
        if (k == slot && (double) f <= 1 + 1.0 / 100)
        {
            c_delta  = __fmul_rn(f, delta_max);
            c_offset = t_off;
            valid    = true;
        }
    }
    else
    {
        // _pickTestCandidatesAsymmetric (:177-214)
        const float obs_delta = __double2float_rn(__ddiv_rn(__dsub_rn((double) obs_mx, (double) obs_mn), (double) steps));
        const int obs_off     = to_int_x86(round_half_away(__fdiv_rn(obs_mn, obs_delta)));
        const float g_min     = smax(__fmul_rn(obs_delta, (float) obs_off), -FLT_MAX);
        const float g_max     = smin(__fmul_rn(obs_delta, __fadd_rn((float) obs_off, steps)), FLT_MAX);
        if (slot == kAsymSlots - 1)
        {
            c_delta  = obs_delta;
            c_offset = obs_off;
            valid    = true;
        }
        else if (slot < kAsymSlots - 1)
        {
            const int di  = slot / kAsymOffsets;   // f = (di + 1) / 16, exact in float
            const int oi  = slot - di * kAsymOffsets;
            const float f = (float) (di + 1) * 0.0625f;
            c_delta       = __fmul_rn(f, obs_delta);
            c_offset      = to_int_x86(__dadd_rn((double) (-steps), __dmul_rn(__ddiv_rn((double) steps, 20.0), (double) oi)));
            valid         = clamp_candidate(g_min, g_max, steps, c_delta, c_offset);
        }
    }

    // ---- cost (_quantAndSatCost :293-355) -------------------------------------------------------------------
    double cost = DBL_MAX;
    if (valid)
    {
        const float min_val   = __fmul_rn(c_delta, (float) c_offset);
        const float step_size = a.steps;
        const float max_val   = __fmul_rn(c_delta, __fadd_rn((float) c_offset, step_size));
        const float pdf_start = (float) xl[0];
        const double pdf_step = __dsub_rn(xl[1], xl[0]);
        const double half     = __ddiv_rn(pdf_step, 2.0);
        int min_ind = to_int_x86(floor(__ddiv_rn((double) __fsub_rn(min_val, pdf_start), pdf_step)));
        min_ind     = smin(smax(0, min_ind), AQ_PDF_SIZE - 1);
        int max_ind = to_int_x86(floor(__ddiv_rn((double) __fsub_rn(max_val, pdf_start), pdf_step)));
        max_ind     = smin(smax(0, max_ind), AQ_PDF_SIZE - 1);
        const float min_mid =
            __double2float_rn(__dadd_rn(__dadd_rn((double) pdf_start, __dmul_rn((double) min_ind, pdf_step)), half));
        const float max_mid =
            __double2float_rn(__dadd_rn(__dadd_rn((double) pdf_start, __dmul_rn((double) max_ind, pdf_step)), half));
        // The reference runs three loops: i < min_ind (bottom), i >= max_ind (top), min_ind <= i < max_ind (middle).
        // When max_ind < min_ind (a float overflow in the index arithmetic collapses max_ind to 0) a bucket is
        // counted in BOTH saturation sums, so the two are kept in separate arrays.
        for (int i = lane; i < AQ_PDF_SIZE; i += 32)
        {
            const double mid = __dadd_rn(__dadd_rn((double) pdf_start, __dmul_rn((double) i, pdf_step)), half);
            double low       = 0.0;
            if (i < min_ind)
            {
                const double d = __dsub_rn(mid, (double) min_mid);
                low            = __dmul_rn(pdf[i], __dmul_rn(d, d));
            }
            else if (i < max_ind)
            {
                const float fv = __double2float_rn(mid);
                const int q    = to_int_x86(round_half_away(__fsub_rn(__fdiv_rn(fv, c_delta), (float) c_offset)));
                const float dq = __fmul_rn(c_delta, (float) (int) ((unsigned) q + (unsigned) c_offset));
                const double d = (double) __fsub_rn(fv, dq);
                low            = __dmul_rn(pdf[i], __dmul_rn(d, d));
            }
            s_term[warp][i] = low;
            double top      = 0.0;
            if (i >= max_ind)
            {
                const double d = __dsub_rn(mid, (double) max_mid);
                top            = __dmul_rn(pdf[i], __dmul_rn(d, d));
            }
            s_top[warp][i] = top;
        }
        __syncwarp();
        // three ordered sums, one lane each
        double part = 0.0;
        if (lane == 0)
            for (int i = 0; i < min_ind; ++i)
                part = __dadd_rn(part, s_term[warp][i]);
        else if (lane == 1)
            for (int i = max_ind; i < AQ_PDF_SIZE; ++i)
                part = __dadd_rn(part, s_top[warp][i]);
        else if (lane == 2)
            for (int i = min_ind; i < max_ind; ++i)
                part = __dadd_rn(part, s_term[warp][i]);
        const double bottom = __shfl_sync(0xffffffffu, part, 0);
        const double top    = __shfl_sync(0xffffffffu, part, 1);
        const double quant  = __shfl_sync(0xffffffffu, part, 2);
        const double sqnr   = __dadd_rn(__dmul_rn((double) 3.0f, __dadd_rn(bottom, top)), quant);
        cost                = smin(sqnr, DBL_MAX);
    }
    if (lane == 0 && slot < a.slots)
    {
        a.ws->cost[slot]   = cost;
        a.ws->delta[slot]  = c_delta;
        a.ws->offset[slot] = c_offset;
        a.ws->valid[slot]  = valid ? 1 : 0;
        __threadfence();
    }

    // ---- last CTA picks the first strict minimum and writes the encoding ----------------------------------------
    __syncthreads();
    if (threadIdx.x == 0)
    {
        __threadfence();
        const unsigned int t = atomicAdd(&a.ws->ticket, 1u);
        s_last               = (t == gridDim.x - 1);
    }
    __syncthreads();
    if (!s_last)
        return;
    __threadfence();
    if (warp == 0)
    {
        double best = DBL_MAX;
        int best_i  = INT_MAX;
        for (int i = lane; i < a.slots; i += 32)
        {
            const double c = __ldcg(&a.ws->cost[i]);
            const int v    = __ldcg(&a.ws->valid[i]);
            if (v && c < best)   // strict: keeps the earliest slot of this lane among equals
            {
                best   = c;
                best_i = i;
            }
        }
        // across lanes: smaller cost wins, equal costs -> smaller slot index (= the reference's first strict minimum)
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
        {
            const double oc = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi    = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (oc < best || (oc == best && oi < best_i))
            {
                best   = oc;
                best_i = oi;
            }
        }
        if (lane == 0)
        {
            float b_delta = -1.0f;
            int b_offset  = -1;
            if (best_i != INT_MAX && best < DBL_MAX)
            {
                b_delta  = __ldcg(&a.ws->delta[best_i]);
                b_offset = __ldcg(&a.ws->offset[best_i]);
            }
            const float b_min = smax(__fmul_rn(b_delta, (float) b_offset), -FLT_MAX);
            const float b_max = smin(__fmul_rn(b_delta, __fadd_rn((float) b_offset, steps)), FLT_MAX);
            a.out[0]          = (double) b_min;
            a.out[1]          = (double) b_max;
            a.out[2]          = (double) b_delta;
            a.out[3]          = (double) b_offset;
            a.out[4]          = (double) a.bw;
            a.ws->ticket      = 0;
        }
    }
}

int tfe_search(const aq_tfe_state_t* st, const double* pdf, int stats_updated, const int32_t* stats_updated_dev, int bw,
               int symmetric, int strict, int unsigned_sym, double* out, void* ws, int64_t ws_bytes, cudaStream_t stream)
{
    if (ws_bytes < tfe_search_workspace_bytes())
        return AQ_ERR_WORKSPACE;
    SearchArgs a;
    a.st = st, a.pdf = pdf, a.stats_updated = stats_updated, a.stats_updated_dev = stats_updated_dev, a.bw = bw;
    a.symmetric = symmetric, a.strict = strict, a.unsigned_sym = unsigned_sym;
    a.out = out, a.ws = static_cast<SearchWs*>(ws);
    a.steps         = (float) (pow(2.0, (double) bw) - 1.0);
    a.slots         = symmetric ? kSymSlots : kAsymSlots;
    const int grid  = (a.slots + kSearchWarps - 1) / kSearchWarps;
    launch_pdl(tfe_search_kernel, (unsigned) grid, kSearchWarps * 32, 0, stream, a);
    note_launch();
    return check_launch();
}

// ---- percentile analyzer on the same statistics ----------------------------------------------------------------
// PercentileEncodingAnalyzer<float>::computeEncoding (DlQuantization/src/PercentileEncodingAnalyzer.cpp:79-194) with
// findOriginalRange<float> (src/math_functions.cpp:404-438).  512 buckets and a serial cumulative sum whose order the
// result depends on: one thread does it, in the reference's mixed float / double arithmetic.
__global__ void tfe_percentile_kernel(const aq_tfe_state_t* __restrict__ st, const double* __restrict__ pdf,
                                      int stats_updated, const int32_t* __restrict__ stats_updated_dev, float percentile,
                                      int bw, int symmetric, int strict, int unsigned_sym, double* __restrict__ out)
{
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x != 0 || blockIdx.x != 0)
        return;
    float num_steps = (float) (ldexp(1.0, bw) - 1.0);
    if (symmetric && strict)
        num_steps = __fsub_rn(num_steps, 1.0f);
    if (!st->initialized)
    {
        double e[5] = {0, 0, 0, 0, 0};
        if (stats_updated_dev ? (*stats_updated_dev != 0) : (stats_updated != 0))
        {
            const double d = __ddiv_rn(2.0, (double) (int) num_steps);
            const double o = floor(__ddiv_rn(-1.0, d));
            e[0]           = __dmul_rn(o, d);
            e[1]           = __dadd_rn(e[0], __dmul_rn((double) (int) num_steps, d));
            e[2] = d, e[3] = o, e[4] = bw;
        }
        for (int i = 0; i < 5; ++i)
            out[i] = e[i];
        return;
    }
    const double* __restrict__ xl = st->x_left;
    float min_val = (float) xl[0], max_val = (float) xl[AQ_PDF_SIZE - 1];
    for (int i = 0; i < AQ_PDF_SIZE; ++i)
        if (pdf[i] > 0)
        {
            min_val = (float) xl[i];
            break;
        }
    for (int i = AQ_PDF_SIZE - 1; i > 0; --i)
        if (pdf[i] > 0)
        {
            max_val = (float) xl[i];
            break;
        }
    min_val = smin(min_val, 0.0f);
    max_val = smax(max_val, 0.0f);
    max_val = smax(max_val, __fadd_rn(min_val, (float) 0.01));
    float a_min = min_val, a_max = max_val;
    if (percentile != 100.0f)
    {
        const float bin_width = (float) __dsub_rn(xl[1], xl[0]);
        float p_min           = (float) xl[0];
        float p_max           = (float) __dadd_rn(xl[AQ_PDF_SIZE - 1], (double) bin_width);
        const float left      = __fsub_rn(1.0f, __fdiv_rn(percentile, 100.0f));
        const float right     = __fdiv_rn(percentile, 100.0f);
        // cumulative distribution, summed in bucket order; the first bucket reaching `left` gives the lower bound,
        // the last bucket still below `right` (and below the observed maximum) the upper one
        double cdf = 0.0;
        bool have_min = false;
        int top = -1;
        for (int i = 0; i < AQ_PDF_SIZE; ++i)
        {
            cdf = (i == 0) ? pdf[0] : __dadd_rn(pdf[i], cdf);
            if (!have_min && cdf >= (double) left)
            {
                p_min    = (float) xl[i];
                have_min = true;
            }
            if (cdf < (double) right && xl[i] < (double) max_val)
                top = i;
        }
        if (top >= 0)
            p_max = (float) __dadd_rn(xl[top], (double) bin_width);
        if (p_min == p_max)
            p_max = __fadd_rn(p_max, bin_width);
        a_min = p_min, a_max = p_max;
    }
    a_min = smin(a_min, 0.0f);
    a_max = smax(a_max, 0.0f);
    aq_encoding_t e;
    computed_encodings(bw, (double) a_min, (double) a_max, symmetric != 0, strict != 0, unsigned_sym != 0, &e);
    out[0] = e.min, out[1] = e.max, out[2] = e.delta, out[3] = e.offset, out[4] = (double) bw;
}

int tfe_percentile(const aq_tfe_state_t* st, const double* pdf, int stats_updated, const int32_t* stats_updated_dev,
                   float percentile, int bw, int symmetric, int strict, int unsigned_sym, double* out, cudaStream_t stream)
{
    launch_pdl(tfe_percentile_kernel, 1, 32, 0, stream, st, pdf, stats_updated, stats_updated_dev, percentile, bw,
               symmetric, strict, unsigned_sym, out);
    note_launch();
    return check_launch();
}

// ---- MSE analyzer on the same statistics -------------------------------------------------------------------------
// MseEncodingAnalyzer<float>::computeEncoding (DlQuantization/src/MseEncodingAnalyzer.cpp:78-267): every pair of a
// negative-or-zero and a positive-or-zero bucket edge inside the observed range is a (min, max) candidate -- up to
// 66,564 of them, which the reference walks one after the other on the host; its cost is the PDF-weighted squared
// fake-quantization error of the bucket centres, a sequential float sum over up to 513 centres whose order the result
// depends on.  Here: one thread prepares the lists in the reference's float arithmetic, one thread per candidate
// runs the reference's sum in order, one CTA takes the first candidate of least cost.
constexpr int kMseMaxEdges = AQ_PDF_SIZE + 8;
constexpr int kMseMaxCands = (AQ_PDF_SIZE / 2 + 2) * (AQ_PDF_SIZE / 2 + 2);   // (a + 1)(b + 1) with a + b <= 514
constexpr int kMseThreads  = 128;

struct MseWs
{
    int n_min, n_max, num_centers, done;
    float fallback_min, fallback_max;
    float pad[2];
    float mins[kMseMaxEdges + 1], maxs[kMseMaxEdges + 1];
    float centers[kMseMaxEdges], center_pdf[kMseMaxEdges];
    float cost[kMseMaxCands];
};

int64_t tfe_mse_workspace_bytes()
{
    return (int64_t) ((sizeof(MseWs) + 255) / 256 * 256);
}

__global__ void tfe_mse_prepare_kernel(const aq_tfe_state_t* __restrict__ st, const double* __restrict__ pdf,
                                       int stats_updated, const int32_t* __restrict__ stats_updated_dev, int bw,
                                       int symmetric, int strict, MseWs* __restrict__ ws, double* __restrict__ out)
{
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x != 0 || blockIdx.x != 0)
        return;
    ws->n_min = ws->n_max = ws->num_centers = 0;
    ws->done  = 0;
    float num_steps = (float) (ldexp(1.0, bw) - 1.0);
    if (symmetric && strict)
        num_steps = __fsub_rn(num_steps, 1.0f);
    if (!st->initialized)
    {
        double e[5] = {0, 0, 0, 0, 0};
        if (stats_updated_dev ? (*stats_updated_dev != 0) : (stats_updated != 0))
        {
            const double d = __ddiv_rn(2.0, (double) (int) num_steps);
            const double o = floor(__ddiv_rn(-1.0, d));
            e[0]           = __dmul_rn(o, d);
            e[1]           = __dadd_rn(e[0], __dmul_rn((double) (int) num_steps, d));
            e[2] = d, e[3] = o, e[4] = bw;
        }
        for (int i = 0; i < 5; ++i)
            out[i] = e[i];
        ws->done = 1;
        return;
    }
    const double* __restrict__ xl = st->x_left;
    const float bin_width = (float) __dsub_rn(xl[1], xl[0]);
    const float hist_min  = (float) xl[0];
    const float hist_max  = (float) __dadd_rn(xl[AQ_PDF_SIZE - 1], (double) bin_width);
    // findOriginalRange<float> (src/math_functions.cpp:404-438)
    float min_val = (float) xl[0], max_val = (float) xl[AQ_PDF_SIZE - 1];
    for (int i = 0; i < AQ_PDF_SIZE; ++i)
        if (pdf[i] > 0)
        {
            min_val = (float) xl[i];
            break;
        }
    for (int i = AQ_PDF_SIZE - 1; i > 0; --i)
        if (pdf[i] > 0)
        {
            max_val = (float) xl[i];
            break;
        }
    min_val = smin(min_val, 0.0f);
    max_val = smax(max_val, 0.0f);
    max_val = smax(max_val, __fadd_rn(min_val, (float) 0.01));
    max_val = __fadd_rn(max_val, bin_width);
    ws->fallback_min = min_val, ws->fallback_max = max_val;
    // bucket edges inside the observed range (a running float sum in the reference), split by sign as they come
    int n_min = 0, n_max = 0, num_edges = 1;
    if (min_val < 0)
        ws->mins[n_min++] = min_val;
    else if (min_val > 0)
        ws->maxs[n_max++] = min_val;
    float e = hist_min;
    for (int it = 0; it < kMseMaxEdges - 1 && e <= hist_max; ++it, e = __fadd_rn(e, bin_width))
    {
        if (e >= min_val && e <= max_val)
        {
            ++num_edges;
            if (e < 0)
                ws->mins[n_min++] = e;
            else if (e > 0)
                ws->maxs[n_max++] = e;
        }
    }
    ws->mins[n_min++] = 0.0f;
    ws->maxs[n_max++] = 0.0f;
    // bucket centres and the PDF value under each
    const float pdf_start = (float) xl[0];
    const int num_centers = num_edges - 1;
    float c = 0.0f;
    for (int i = 0; i < num_centers; ++i)
    {
        c       = i == 0 ? __fadd_rn(min_val, __fdiv_rn(bin_width, 2.0f)) : __fadd_rn(c, bin_width);
        int idx = to_int_x86(floorf(__fdiv_rn(__fsub_rn(c, pdf_start), bin_width)));
        idx     = min(max(0, idx), AQ_PDF_SIZE - 1);
        ws->centers[i]    = c;
        ws->center_pdf[i] = (float) pdf[idx];
    }
    ws->n_min = n_min, ws->n_max = n_max, ws->num_centers = num_centers;
}

__global__ void __launch_bounds__(kMseThreads) tfe_mse_cost_kernel(MseWs* __restrict__ ws, int bw, int symmetric,
                                                                   int strict, int unsigned_sym)
{
    pdl_launch_dependents();
    pdl_wait();
    const int n_max = ws->n_max;
    const int cands = ws->n_min * n_max - 1;   // the last pair is {0, 0}
    const int cand  = blockIdx.x * kMseThreads + threadIdx.x;
    if (ws->done || cand >= cands)
        return;
    const float c_min = ws->mins[cand / n_max], c_max = ws->maxs[cand % n_max];
    aq_encoding_t enc;
    computed_encodings(bw, (double) c_min, (double) c_max, symmetric != 0, strict != 0, unsigned_sym != 0, &enc);
    const int n = ws->num_centers;
    float err   = 0.0f;
    for (int i = 0; i < n; ++i)
    {
        const float v       = ws->centers[i];
        const float clamped = smax(c_min, smin(v, c_max));
        const int quantized = to_int_x86(round(__dsub_rn(__ddiv_rn((double) clamped, enc.delta), enc.offset)));
        const float dequant = (float) __dmul_rn(enc.delta, __dadd_rn((double) quantized, enc.offset));
        const double d      = (double) __fsub_rn(v, dequant);
        err = (float) __dadd_rn((double) err, __dmul_rn((double) ws->center_pdf[i], __dmul_rn(d, d)));
    }
    ws->cost[cand] = err;
}

__global__ void __launch_bounds__(256) tfe_mse_select_kernel(MseWs* __restrict__ ws, int bw, int symmetric, int strict,
                                                             int unsigned_sym, double* __restrict__ out)
{
    pdl_launch_dependents();
    pdl_wait();
    if (ws->done)
        return;
    const int n_max = ws->n_max;
    const int cands = ws->n_min * n_max - 1;
    // `if (mse < mseMin)` walking the candidates in order from FLT_MAX: the first candidate of least cost; NaN never wins
    float best = FLT_MAX;
    int best_i = INT_MAX;
    for (int i = threadIdx.x; i < cands; i += 256)
    {
        const float v = ws->cost[i];
        if (v < best)
            best = v, best_i = i;
    }
    __shared__ float s_v[256];
    __shared__ int s_i[256];
    s_v[threadIdx.x] = best, s_i[threadIdx.x] = best_i;
    __syncthreads();
    if (threadIdx.x != 0)
        return;
    for (int t = 1; t < 256; ++t)
        if (s_i[t] != INT_MAX && (s_v[t] < best || (s_v[t] == best && s_i[t] < best_i)))
            best = s_v[t], best_i = s_i[t];
    float a_min = ws->fallback_min, a_max = ws->fallback_max;
    if (best_i != INT_MAX)
        a_min = ws->mins[best_i / n_max], a_max = ws->maxs[best_i % n_max];
    a_min = smin(a_min, 0.0f);
    a_max = smax(a_max, 0.0f);
    aq_encoding_t e;
    computed_encodings(bw, (double) a_min, (double) a_max, symmetric != 0, strict != 0, unsigned_sym != 0, &e);
    out[0] = e.min, out[1] = e.max, out[2] = e.delta, out[3] = e.offset, out[4] = (double) bw;
}

int tfe_mse(const aq_tfe_state_t* st, const double* pdf, int stats_updated, const int32_t* stats_updated_dev, int bw,
            int symmetric, int strict, int unsigned_sym, double* out, void* ws, cudaStream_t stream)
{
    MseWs* w = static_cast<MseWs*>(ws);
    launch_pdl(tfe_mse_prepare_kernel, 1, 32, 0, stream, st, pdf, stats_updated, stats_updated_dev, bw, symmetric, strict,
               w, out);
    note_launch();
    launch_pdl(tfe_mse_cost_kernel, (unsigned) ((kMseMaxCands + kMseThreads - 1) / kMseThreads), kMseThreads, 0, stream, w,
               bw, symmetric, strict, unsigned_sym);
    note_launch();
    launch_pdl(tfe_mse_select_kernel, 1, 256, 0, stream, w, bw, symmetric, strict, unsigned_sym, out);
    note_launch();
    return check_launch();
}

}   // namespace aq
