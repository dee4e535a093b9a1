/*
 * TEST INFRASTRUCTURE ONLY -- never imported, linked or executed by the product path.
 *
 * Plain-C, single-threaded CPU restatement of the libpymo ("v1") arithmetic of AIMET's
 * quantization-simulation hot path.  Every function cites the reference file:line it follows
 * (paths relative to the AIMET 1.35 source tree).  It exists so that GPU parity tests have a
 * checker that travels to machines where the reference checkout is absent.
 *
 * PINNED: tests/test_oracle_pin.py checks this file bit-for-bit against (a) the reference's own
 * known-answer vectors from ModelOptimizations/DlQuantization/test/Test*.cpp and (b) the unmodified
 * reference sources compiled into oracle/_ref/libaimet_ref.so (when that library is present), and
 * tests/golden/ holds fixtures generated from (b).
 *
 * Build: gcc -std=c11 -O2 -fPIC -ffp-contract=off -shared libpymo_oracle.c -lm
 * (no FMA contraction: the reference's default x86-64 build evaluates a*b+c in two roundings).
 */
#include <float.h>
#include <limits.h>
#include <math.h>
#include <stdint.h>
#include <string.h>

#define ORC_PDF_SIZE 512

/* std::max(a,b) = (a<b)?b:a and std::min(a,b) = (b<a)?b:a -- the argument order decides what a NaN or a
 * signed zero does, so the restatement keeps the reference's argument order at every call site. */
#define STD_MAX(a, b) (((a) < (b)) ? (b) : (a))
#define STD_MIN(a, b) (((b) < (a)) ? (b) : (a))

/* double -> int the way x86-64 cvttsd2si does it (out of range / NaN -> INT_MIN). */
static int to_int_x86_d(double v)
{
    if (!(v > -2147483649.0 && v < 2147483648.0))
        return INT_MIN;
    return (int) v;
}
static int to_int_x86_f(float v)
{
    if (!(v >= -2147483648.0f && v < 2147483648.0f))
        return INT_MIN;
    return (int) v;
}

/* ---------------------------------------------------------------------------------------------
 * A1. Per-tensor grid.  TensorQuantizationSim.cpp:62-92 (generateScaleOffset / fillEncodingInfo),
 *     quantization_utils.cpp:145-156 (gateMinMax), trim_functions.cpp:61-73 (computeDelta/Offset).
 *     out4 = {min, max, delta, offset} in double.
 * ------------------------------------------------------------------------------------------- */
void orc_fill_encoding(int bw, double enc_min, double enc_max, double* out4)
{
    /* gateMinMax: keep zero inside, keep a 1e-5 wide range */
    enc_min = STD_MIN(enc_min, 0.0);
    enc_max = STD_MAX(enc_max, 0.0);
    enc_max = STD_MAX(enc_max, enc_min + 1e-5);
    double steps = pow(2.0, (double) (uint8_t) bw) - 1.0;
    if (enc_min == -enc_max)
        steps -= 1.0; /* strict-symmetric detected by value */
    double delta  = (enc_max - enc_min) / steps;
    double offset = round(enc_min / delta);
    out4[0]       = offset * delta;
    out4[1]       = delta * steps + out4[0];
    out4[2]       = delta;
    out4[3]       = offset;
}

/* Element function.  trim_functions.cpp:140-171 (quantizeValueCpu + dequantizeValueCpu), DTYPE=float. */
static inline float quantize_value(float x, float mn, float mx, float delta, float offset)
{
    float t = fmaxf(fminf(x, mx), mn);
    t       = t / delta - offset;
    return roundf(t);
}
static inline float dequantize_value(float q, float delta, float offset)
{
    return delta * (q + offset);
}

/* TensorQuantizationSim.cpp:94-114 -> trim_functions.cpp:173-182 */
void orc_qdq_per_tensor(const float* in, int64_t n, float* out, double enc_min, double enc_max, int bw)
{
    double e[4];
    orc_fill_encoding(bw, enc_min, enc_max, e);
    const float mn = (float) e[0], mx = (float) e[1], d = (float) e[2], o = (float) e[3];
    for (int64_t i = 0; i < n; ++i)
        out[i] = dequantize_value(quantize_value(in[i], mn, mx, d, o), d, o);
}

/* TensorQuantizationSim.cpp:116-126 -> trim_functions.cpp:202-218 (codes kept in a float container) */
void orc_quantize_per_tensor(const float* in, int64_t n, float* out, double enc_min, double enc_max, int bw,
                             int shift_to_signed)
{
    double e[4];
    orc_fill_encoding(bw, enc_min, enc_max, e);
    const float mn = (float) e[0], mx = (float) e[1], d = (float) e[2], o = (float) e[3];
    unsigned int shift = 0;
    if (shift_to_signed)
        shift = (unsigned int) pow(2.0, (double) (bw - 1));
    for (int64_t i = 0; i < n; ++i)
    {
        float q = quantize_value(in[i], mn, mx, d, o);
        out[i]  = q - (float) shift;
    }
}

/* ---------------------------------------------------------------------------------------------
 * A2. Per-channel grid, derived in fp32 exactly as the torch ops in
 *     TrainingExtensions/torch/src/AimetTensorQuantizer.cpp:236-254,271-299 do on CPU:
 *     gate (zero inside, +1e-5f), delta = (max-min)/steps (true fp32 division),
 *     offset = round-half-to-even(min/delta).  steps loses one iff channel 0 has min == -max
 *     (decided on the double values, :289-294).
 * ------------------------------------------------------------------------------------------- */
void orc_per_channel_grid(const double* enc_min, const double* enc_max, int64_t num_ch, int bw, float* g_min,
                          float* g_max, float* g_delta, float* g_offset)
{
    double steps = pow(2.0, (double) bw) - 1.0;
    if (num_ch > 0 && enc_min[0] == -enc_max[0])
        steps -= 1.0;
    const float fsteps = (float) steps;
    for (int64_t c = 0; c < num_ch; ++c)
    {
        float mn = (float) enc_min[c], mx = (float) enc_max[c];
        mn       = mn < 0.0f ? mn : 0.0f; /* torch::minimum(min, 0) */
        mx       = mx > 0.0f ? mx : 0.0f; /* torch::maximum(max, 0) */
        float lo = mn + 1e-5f;
        mx       = mx > lo ? mx : lo;
        float d  = (mx - mn) / fsteps;
        float o  = nearbyintf(mn / d); /* at::round = half to even */
        g_min[c] = mn, g_max[c] = mx, g_delta[c] = d, g_offset[c] = o;
    }
}

/* trim_functions.cpp:697-709 (quantizeDequantizePerChannelCpu) */
void orc_qdq_per_channel(const float* in, int64_t num_ch, int64_t n, int64_t per_ch, float* out, const float* g_min,
                         const float* g_max, const float* g_delta, const float* g_offset)
{
    for (int64_t i = 0; i < n; ++i)
    {
        int64_t c = (i / per_ch) % num_ch;
        out[i]    = dequantize_value(quantize_value(in[i], g_min[c], g_max[c], g_delta[c], g_offset[c]), g_delta[c],
                                     g_offset[c]);
    }
}

/* trim_functions.cpp:633-660 (quantizeDequantizeBroadcastCpu): encoding index by stride walk */
void orc_qdq_broadcast(const float* in, float* out, int64_t n, int64_t ndims, const int64_t* in_strides,
                       const int64_t* enc_strides, const float* g_min, const float* g_max, const float* g_delta,
                       const float* g_offset)
{
    for (int64_t i = 0; i < n; ++i)
    {
        int64_t e = 0, rem = i;
        for (int64_t d = 0; d < ndims; ++d)
        {
            int64_t k = rem / in_strides[d];
            rem -= k * in_strides[d];
            e += enc_strides[d] * k;
        }
        out[i] = dequantize_value(quantize_value(in[i], g_min[e], g_max[e], g_delta[e], g_offset[e]), g_delta[e],
                                  g_offset[e]);
    }
}

/* v1 straight-through backward: dx = g * [min <= x <= max]
 * TrainingExtensions/torch/src/python/aimet_torch/v1/quantsim_straight_through_grad.py:91-118 */
void orc_ste_bwd(const float* x, const float* g, int64_t n, float enc_min, float enc_max, float* dx)
{
    for (int64_t i = 0; i < n; ++i)
        dx[i] = g[i] * ((enc_min <= x[i] && x[i] <= enc_max) ? 1.0f : 0.0f);
}

/* ---------------------------------------------------------------------------------------------
 * A3. MinMax ("TF") analyzer.
 * ------------------------------------------------------------------------------------------- */
/* math_functions.cpp:327-347 (GetMax_cpu / GetMin_cpu): std::max/std::min folds, NaN never enters */
void orc_min_max(const float* in, int64_t n, float* out2)
{
    float mn = (float) INFINITY, mx = -(float) INFINITY; /* (float)+-DBL_MAX */
    for (int64_t i = 0; i < n; ++i)
    {
        mx = STD_MAX(mx, in[i]);
        mn = STD_MIN(mn, in[i]);
    }
    out2[0] = mn, out2[1] = mx;
}

/* quantization_utils.cpp:58-143 (getComputedEncodings). out4 = {min,max,delta,offset} */
void orc_computed_encodings(int bw, double mn, double mx, int symmetric, int strict, int unsigned_sym, double* out4)
{
    double steps = pow(2.0, (double) (uint8_t) bw) - 1.0;
    if (symmetric && strict)
        steps -= 1.0;
    if (isinf(mn))
        mn = -(double) FLT_MAX;
    if (isinf(mx))
        mx = (double) FLT_MAX;

    double e_min, e_max, delta, offset;
    if (symmetric && (mn < 0.0 || !unsigned_sym))
    {
        double a           = STD_MAX(fabs(mx), fabs(mn));
        unsigned int n_pos = (unsigned int) floor(steps / 2.0);
        delta              = a / n_pos;
        offset             = -ceil(steps / 2.0);
        e_min              = STD_MAX(offset * delta, -(double) FLT_MAX);
        e_max              = STD_MIN(delta * n_pos, (double) FLT_MAX);
    }
    else
    {
        delta = (mx - mn) / steps;
        if (mn < 0 && mx > 0)
        {
            double bz = round(-mn / delta);
            bz        = STD_MIN(steps, STD_MAX(0.0, bz));
            offset    = -bz;
            double p  = delta * offset;
            if (p >= -(double) FLT_MAX && p <= (double) FLT_MAX)
                e_min = p;
            else
                e_min = -(double) FLT_MAX;
            e_max = mx - mn + e_min;
            if (e_max > (double) FLT_MAX)
                e_max = (double) FLT_MAX;
        }
        else
        {
            offset = round(mn / delta);
            e_min  = mn;
            e_max  = mx;
        }
    }
    out4[0] = e_min, out4[1] = e_max, out4[2] = delta, out4[3] = offset;
}

/* TfEncodingAnalyzer.cpp:80-101 (computeEncoding) on running stats in double */
void orc_minmax_encoding(int bw, double stat_min, double stat_max, int symmetric, int strict, int unsigned_sym,
                         double* out4)
{
    double mn = STD_MIN(0.0, stat_min);
    double mx = STD_MAX(0.0, stat_max);
    mx        = STD_MAX(mx, mn + 0.01);
    orc_computed_encodings(bw, mn, mx, symmetric, strict, unsigned_sym, out4);
}

/* ---------------------------------------------------------------------------------------------
 * A4. 512-bucket PDF.
 * ------------------------------------------------------------------------------------------- */
/* math_functions.cpp:207-241 (InitializePdf<float>, signed_vals=true) */
void orc_pdf_init(float min_val, float max_val, double* x_left)
{
    if (min_val == max_val)
    {
        max_val = STD_MAX(max_val, min_val + 0.01f);
    }
    float center = (max_val + min_val) / 2.0f;
    float lo     = center - 3.0f * (center - min_val);
    float hi     = center + 3.0f * (max_val - center);
    lo           = STD_MAX(-FLT_MAX, lo);
    hi           = STD_MIN(FLT_MAX, hi);
    double bucket = ((double) hi - (double) lo) / ORC_PDF_SIZE;
    for (int i = 0; i < ORC_PDF_SIZE; ++i)
        x_left[i] = (double) lo + i * bucket;
}

/* Bucket geometry narrowed to float: math_functions.cpp:264-268 */
void orc_pdf_geometry(const double* x_left, float* bucket_size, float* pdf_offset)
{
    float bs     = (float) (x_left[1] - x_left[0]);
    float mn     = (float) x_left[0];
    *bucket_size = bs;
    *pdf_offset  = mn / bs;
}

/* math_functions.cpp:367-384 (GetHistogram_cpu, signed).  Adds into hist[512]. */
void orc_hist512(const float* in, int64_t n, float bucket_size, float pdf_offset, uint32_t* hist)
{
    for (int64_t i = 0; i < n; ++i)
    {
        int idx = to_int_x86_f(roundf(in[i] / bucket_size - pdf_offset));
        if (idx >= 0 && idx < ORC_PDF_SIZE)
            hist[idx] += 1;
    }
}

/* Running mean of per-batch PDFs: math_functions.cpp:278-287.  cnt is the full element count. */
void orc_pdf_accumulate(const uint32_t* hist, int64_t cnt, double* pdf, int* iterations)
{
    const int it = *iterations;
    for (int i = 0; i < ORC_PDF_SIZE; ++i)
    {
        double prob = (double) hist[i] / (double) (int) cnt;
        pdf[i]      = (pdf[i] * it + prob) / (it + 1);
    }
    *iterations = it + 1;
}

/* math_functions.cpp:243-288 (UpdatePdf<float>): state = x_left[512], pdf[512], *initialized, *iterations.
 * hist_out (may be NULL) receives this batch's raw counts. Returns 1 if the batch was consumed, 0 if it was the
 * all-zero batch that the reference skips before the PDF exists. */
int orc_update_pdf(const float* in, int64_t n, double* x_left, double* pdf, int* initialized, int* iterations,
                   uint32_t* hist_out)
{
    if (!*initialized)
    {
        float mm[2];
        orc_min_max(in, n, mm);
        if (mm[0] == 0 && mm[1] == 0)
            return 0;
        orc_pdf_init(mm[0], mm[1], x_left);
        memset(pdf, 0, ORC_PDF_SIZE * sizeof(double));
        *iterations  = 0;
        *initialized = 1;
    }
    float bs, po;
    orc_pdf_geometry(x_left, &bs, &po);
    uint32_t hist[ORC_PDF_SIZE];
    memset(hist, 0, sizeof(hist));
    orc_hist512(in, n, bs, po, hist);
    orc_pdf_accumulate(hist, n, pdf, iterations);
    if (hist_out)
        memcpy(hist_out, hist, sizeof(hist));
    return 1;
}

/* ---------------------------------------------------------------------------------------------
 * A5. TF-Enhanced search (TfEnhancedEncodingAnalyzer.cpp, DTYPE=float).
 * ------------------------------------------------------------------------------------------- */
/* :293-355 (_quantAndSatCost) */
double orc_tfe_cost(const double* x_left, const double* pdf, int bw, float delta, int offset)
{
    float min_val   = delta * (float) offset;
    float step_size = (float) (pow(2.0, (double) bw) - 1.0);
    float max_val   = delta * ((float) offset + step_size);
    float pdf_start = (float) x_left[0];
    double pdf_step = x_left[1] - x_left[0];

    int min_ind = to_int_x86_d(floor((double) (min_val - pdf_start) / pdf_step));
    min_ind     = STD_MIN(STD_MAX(0, min_ind), ORC_PDF_SIZE - 1);
    int max_ind = to_int_x86_d(floor((double) (max_val - pdf_start) / pdf_step));
    max_ind     = STD_MIN(STD_MAX(0, max_ind), ORC_PDF_SIZE - 1);

    double sat_bottom = 0;
    float min_mid     = (float) ((double) pdf_start + (min_ind * pdf_step) + pdf_step / 2);
    for (int i = 0; i < min_ind; ++i)
    {
        double mid = (double) pdf_start + i * pdf_step + pdf_step / 2;
        double d   = mid - (double) min_mid;
        sat_bottom += pdf[i] * (d * d);
    }
    double sat_top = 0;
    float max_mid  = (float) ((double) pdf_start + (max_ind * pdf_step) + pdf_step / 2);
    for (int i = max_ind; i < ORC_PDF_SIZE; ++i)
    {
        double mid = (double) pdf_start + i * pdf_step + pdf_step / 2;
        double d   = mid - (double) max_mid;
        sat_top += pdf[i] * (d * d);
    }
    double quant = 0;
    for (int i = min_ind; i < max_ind; ++i)
    {
        float fv  = (float) ((double) pdf_start + i * pdf_step + pdf_step / 2);
        int q     = to_int_x86_f(roundf(fv / delta - (float) offset));
        float dq  = delta * (float) (int) ((unsigned) q + (unsigned) offset); /* wraps like the x86 build */
        double d  = (double) (fv - dq);
        quant += pdf[i] * (d * d);
    }
    double cost = (double) 3.0f * (sat_bottom + sat_top) + quant;
    return STD_MIN(cost, DBL_MAX);
}

/* :255-291 (_findRangeOfAggregateStats) */
static void tfe_observed_range(const double* x_left, const double* pdf, float* out_min, float* out_max)
{
    float mn = (float) x_left[0];
    float mx = (float) x_left[ORC_PDF_SIZE - 1];
    for (int i = 0; i < ORC_PDF_SIZE; ++i)
        if (pdf[i] > 0)
        {
            mn = (float) x_left[i];
            break;
        }
    for (int i = ORC_PDF_SIZE - 1; i > 0; --i)
        if (pdf[i] > 0)
        {
            mx = (float) x_left[i];
            break;
        }
    mn       = STD_MIN(mn, 0.0f);
    mx       = STD_MAX(mx, 0.0f);
    mx       = STD_MAX(mx, mn + (float) 0.01);
    *out_min = mn, *out_max = mx;
}

/* :149-175 (_clampToObservedMinMax) */
static int tfe_clamp(float obs_min, float obs_max, float steps, float* test_delta, int* test_offset)
{
    float t_min = STD_MAX(*test_delta * (float) *test_offset, -FLT_MAX);
    float t_max = STD_MIN(*test_delta * ((float) *test_offset + steps), FLT_MAX);
    if (t_min < obs_min && t_max > obs_max)
        return 0;
    t_min = STD_MAX(obs_min, t_min);
    t_max = STD_MIN(obs_max, t_max);
    if (t_min == t_max)
        return 0;
    *test_delta  = (float) (((double) t_max - (double) t_min) / (double) steps);
    *test_offset = to_int_x86_f(roundf(t_min / *test_delta));
    return 1;
}

#define ORC_MAX_CAND 512

/* :177-253 candidate lists; returns the count, in the reference's push order (= tie-break order) */
int orc_tfe_candidates(const double* x_left, const double* pdf, int bw, int symmetric, int strict, int unsigned_sym,
                       float* cand_delta, int* cand_offset)
{
    float mn, mx;
    tfe_observed_range(x_left, pdf, &mn, &mx);
    float steps = (float) (pow(2.0, (double) bw) - 1.0);
    int n       = 0;
    if (symmetric)
    {
        if (strict)
            steps -= 1.0f;
        float delta_max;
        int t_off;
        if (mn == 0.0f && unsigned_sym)
        {
            delta_max = mx / steps;
            t_off     = 0;
        }
        else
        {
            float a   = STD_MAX(fabsf(mx), fabsf(mn));
            delta_max = (float) ((double) a / ((double) steps / 2.0));
            t_off     = (int) floorf(-steps / 2.0f);
        }
        for (float f = (float) (1.0 / 100); (double) f <= 1 + 1.0 / 100; f = (float) ((double) f + 1.0 / 100))
        {
            if (n >= ORC_MAX_CAND)
                break;
            cand_delta[n]  = f * delta_max;
            cand_offset[n] = t_off;
            ++n;
        }
    }
    else
    {
        float obs_delta = (float) (((double) mx - (double) mn) / (double) steps);
        int obs_off     = to_int_x86_f(roundf(mn / obs_delta));
        float obs_min   = STD_MAX(obs_delta * (float) obs_off, -FLT_MAX);
        float obs_max   = STD_MIN(obs_delta * ((float) obs_off + steps), FLT_MAX);
        float delta_max = obs_delta;
        for (float f = (float) (1.0 / 16); (double) f <= 1 + 1.0 / 16; f = (float) ((double) f + 1.0 / 16))
        {
            for (int i = 0; i <= 20; ++i)
            {
                float td = f * delta_max;
                int to   = to_int_x86_d((double) (-steps) + (double) steps / 20.0 * i);
                if (!tfe_clamp(obs_min, obs_max, steps, &td, &to))
                    continue;
                cand_delta[n]  = td;
                cand_offset[n] = to;
                ++n;
            }
        }
        cand_delta[n]  = obs_delta;
        cand_offset[n] = obs_off;
        ++n;
    }
    return n;
}

/* :78-147, :357-397 (computeEncoding / getComputedEncodings / _findBestCandidate).
 * out5 = {min,max,delta,offset,bw}.  initialized: PDF exists; stats_updated: updateStats was ever called. */
void orc_tfe_compute(const double* x_left, const double* pdf, int initialized, int stats_updated, int bw, int symmetric,
                     int strict, int unsigned_sym, double* out5)
{
    memset(out5, 0, 5 * sizeof(double));
    float steps = (float) (pow(2.0, (double) bw) - 1.0);
    if (!initialized)
    {
        if (stats_updated)
        {
            double mn = -1, mx = 1;
            double d  = (mx - mn) / (int) steps;
            double o  = floor(mn / d);
            out5[0]   = o * d;
            out5[1]   = out5[0] + (int) steps * d;
            out5[2]   = d;
            out5[3]   = o;
            out5[4]   = bw;
        }
        return;
    }
    float cd[ORC_MAX_CAND];
    int co[ORC_MAX_CAND];
    int n = orc_tfe_candidates(x_left, pdf, bw, symmetric, strict, unsigned_sym, cd, co);
    if (symmetric && strict)
        steps -= 1.0f;
    float best_delta = -1;
    int best_offset  = -1;
    double best_cost = DBL_MAX;
    for (int k = 0; k < n; ++k)
    {
        double c = orc_tfe_cost(x_left, pdf, bw, cd[k], co[k]);
        if (c < best_cost)
        {
            best_cost = c, best_delta = cd[k], best_offset = co[k];
        }
    }
    float b_min = STD_MAX(best_delta * (float) best_offset, -FLT_MAX);
    float b_max = STD_MIN(best_delta * ((float) best_offset + steps), FLT_MAX);
    out5[0]     = b_min;
    out5[1]     = b_max;
    out5[2]     = best_delta;
    out5[3]     = best_offset;
    out5[4]     = bw;
}

/* ---------------------------------------------------------------------------------------------
 * A6. Percentile analyzer on the same 512-bucket PDF (DTYPE = float).
 * ------------------------------------------------------------------------------------------- */
/* math_functions.cpp:404-438 (findOriginalRange<float>) */
static void orc_original_range(const double* x_left, const double* pdf, float* mn_out, float* mx_out)
{
    float mn = (float) x_left[0];
    float mx = (float) x_left[ORC_PDF_SIZE - 1];
    for (int i = 0; i < ORC_PDF_SIZE; ++i)
        if (pdf[i] > 0)
        {
            mn = (float) x_left[i];
            break;
        }
    for (int i = ORC_PDF_SIZE - 1; i > 0; --i)
        if (pdf[i] > 0)
        {
            mx = (float) x_left[i];
            break;
        }
    mn = STD_MIN(mn, 0.0f);
    mx = STD_MAX(mx, 0.0f);
    mx = STD_MAX(mx, mn + (float) 0.01);
    *mn_out = mn, *mx_out = mx;
}

/* PercentileEncodingAnalyzer.cpp:79-194 (computeEncoding + _computePercentileRange).
 * out5 = {min, max, delta, offset, bw}; initialized = whether the PDF exists. */
void orc_percentile_compute(const double* x_left, const double* pdf, int initialized, int stats_updated, float percentile,
                            int bw, int symmetric, int strict, int unsigned_sym, double* out5)
{
    for (int i = 0; i < 5; ++i)
        out5[i] = 0;
    float num_steps = (float) (pow(2, bw) - 1);
    if (symmetric && strict)
        num_steps -= 1;
    if (!initialized)
    {
        if (stats_updated)
        {
            double e_min = -1, e_max = 1;
            double delta  = (e_max - e_min) / (int) num_steps;
            double offset = floor(e_min / delta);
            e_min         = offset * delta;
            e_max         = e_min + (int) num_steps * delta;
            out5[0] = e_min, out5[1] = e_max, out5[2] = delta, out5[3] = offset, out5[4] = bw;
        }
        return;
    }
    float min_val, max_val;
    orc_original_range(x_left, pdf, &min_val, &max_val);
    float a_min = min_val, a_max = max_val;
    if (percentile != 100.0f)
    {
        const float bin_width = (float) (x_left[1] - x_left[0]);
        float hist_min        = (float) x_left[0];
        float hist_max        = (float) (x_left[ORC_PDF_SIZE - 1] + bin_width);
        float p_min = hist_min, p_max = hist_max;
        double cdf[ORC_PDF_SIZE];
        cdf[0] = pdf[0];
        for (int i = 1; i < ORC_PDF_SIZE; ++i)
            cdf[i] = pdf[i] + cdf[i - 1];
        float left = 1 - percentile / 100;
        for (int i = 0; i < ORC_PDF_SIZE; ++i)
            if (cdf[i] >= left)
            {
                p_min = (float) x_left[i];
                break;
            }
        float right = percentile / 100;
        for (int i = ORC_PDF_SIZE - 1; i >= 0; --i)
            if (cdf[i] < right && x_left[i] < max_val)
            {
                p_max = (float) (x_left[i] + bin_width);
                break;
            }
        if (p_min == p_max)
            p_max += bin_width;
        a_min = p_min, a_max = p_max;
    }
    a_min = STD_MIN(a_min, 0.0f);
    a_max = STD_MAX(a_max, 0.0f);
    orc_computed_encodings(bw, a_min, a_max, symmetric, strict, unsigned_sym, out5);
    out5[4] = bw;
}

/* ---------------------------------------------------------------------------------------------
 * A6b. MSE analyzer on the same 512-bucket PDF (DTYPE = float).
 * ------------------------------------------------------------------------------------------- */
/* MseEncodingAnalyzer.cpp:246-267 (_computeMSECost) */
static float orc_mse_cost(int bw, const float* centers, const float* center_pdf, int num_centers, float c_min,
                          float c_max, int symmetric, int strict, int unsigned_sym)
{
    double enc[5];
    orc_computed_encodings(bw, c_min, c_max, symmetric, strict, unsigned_sym, enc);
    const double delta = enc[2], offset = enc[3];
    float err = 0;
    for (int i = 0; i < num_centers; ++i)
    {
        float v        = centers[i];
        float clamped  = STD_MAX(c_min, STD_MIN(v, c_max));
        int quantized  = (int) round(clamped / delta - offset);
        float dequant  = (float) (delta * (quantized + offset));
        err            = (float) (err + center_pdf[i] * pow(v - dequant, 2));
    }
    return err;
}

/* MseEncodingAnalyzer.cpp:78-213 (computeEncoding, _minimizeMSE, _pickMinMaxCandidatesMSECalib) */
void orc_mse_compute(const double* x_left, const double* pdf, int initialized, int stats_updated, int bw, int symmetric,
                     int strict, int unsigned_sym, double* out5)
{
    for (int i = 0; i < 5; ++i)
        out5[i] = 0;
    float num_steps = (float) (pow(2, bw) - 1);
    if (symmetric && strict)
        num_steps -= 1;
    if (!initialized)
    {
        if (stats_updated)
        {
            double e_min = -1, e_max = 1;
            double delta  = (e_max - e_min) / (int) num_steps;
            double offset = floor(e_min / delta);
            e_min         = offset * delta;
            e_max         = e_min + (int) num_steps * delta;
            out5[0] = e_min, out5[1] = e_max, out5[2] = delta, out5[3] = offset, out5[4] = bw;
        }
        return;
    }
    const float bin_width = (float) (x_left[1] - x_left[0]);
    float hist_min        = (float) x_left[0];
    float hist_max        = (float) (x_left[ORC_PDF_SIZE - 1] + bin_width);
    float min_val, max_val;
    orc_original_range(x_left, pdf, &min_val, &max_val);
    max_val = max_val + bin_width;
    float edges[ORC_PDF_SIZE + 8];
    int num_edges = 0;
    edges[num_edges++] = min_val;
    for (float i = hist_min; i <= hist_max; i += bin_width)
        if (i >= min_val && i <= max_val && num_edges < ORC_PDF_SIZE + 8)
            edges[num_edges++] = i;
    float mins[ORC_PDF_SIZE + 9], maxs[ORC_PDF_SIZE + 9];
    int n_min = 0, n_max = 0;
    for (int k = 0; k < num_edges; ++k)
    {
        if (edges[k] < 0)
            mins[n_min++] = edges[k];
        else if (edges[k] > 0)
            maxs[n_max++] = edges[k];
    }
    mins[n_min++] = 0, maxs[n_max++] = 0;
    const float pdf_start = (float) x_left[0];
    const float pdf_step  = (float) (x_left[1] - x_left[0]);
    const int num_centers = num_edges - 1;
    float centers[ORC_PDF_SIZE + 8], center_pdf[ORC_PDF_SIZE + 8];
    for (int i = 0; i < num_centers; ++i)
    {
        centers[i] = i == 0 ? min_val + bin_width / 2 : centers[i - 1] + bin_width;
        int idx    = (int) floorf((centers[i] - pdf_start) / pdf_step);
        idx        = STD_MIN(STD_MAX(0, idx), ORC_PDF_SIZE - 1);
        center_pdf[i] = (float) pdf[idx];
    }
    float mse_min = FLT_MAX;
    float best_min = min_val, best_max = max_val;
    for (int a = 0; a < n_min; ++a)
        for (int b = 0; b < n_max; ++b)
        {
            if (a == n_min - 1 && b == n_max - 1)
                break;   /* {0, 0} is not a candidate */
            float mse = orc_mse_cost(bw, centers, center_pdf, num_centers, mins[a], maxs[b], symmetric, strict, unsigned_sym);
            if (mse < mse_min)
                mse_min = mse, best_min = mins[a], best_max = maxs[b];
        }
    best_min = STD_MIN(best_min, 0.0f);
    best_max = STD_MAX(best_max, 0.0f);
    orc_computed_encodings(bw, best_min, best_max, symmetric, strict, unsigned_sym, out5);
    out5[4] = bw;
}

/* ---------------------------------------------------------------------------------------------
 * A7. Integer codes in integer containers.
 * ------------------------------------------------------------------------------------------- */
/* trim_functions.cpp:220-385 (quantizeToFxpPackedCpu, ROUND_NEAREST).  enc4 = {min, max, delta, offset} as
 * orc_fill_encoding gives them.  out holds n containers of max(bw, 8) bits. */
void orc_quantize_packed(const float* in, int64_t n, const double* enc4, int bw, int shift_to_signed, void* out)
{
    const double e_min = enc4[0], e_max = enc4[1], delta = enc4[2], offset = enc4[3];
    for (int64_t i = 0; i < n; ++i)
    {
        double q = STD_MAX(STD_MIN((double) in[i], e_max), e_min);
        q        = q / delta - offset;
        q        = round(q);
        if (!shift_to_signed)
        {
            if (bw < 8)
            {
                uint8_t small         = (uint8_t) q;
                ((uint8_t*) out)[i] = (uint8_t) STD_MAX(STD_MIN((double) small, (double) (pow(2, bw) - 1)), 0.0);
            }
            else if (bw == 8)
                ((uint8_t*) out)[i] = (uint8_t) STD_MAX(STD_MIN(q, 255.0), 0.0);
            else if (bw == 16)
                ((uint16_t*) out)[i] = (uint16_t) STD_MAX(STD_MIN(q, 65535.0), 0.0);
            else
                ((uint32_t*) out)[i] = (uint32_t) STD_MAX(STD_MIN(q, 4294967295.0), 0.0);
        }
        else
        {
            q -= pow(2, bw - 1) - 1;
            if (bw < 8)
            {
                int8_t small       = (int8_t) q;
                ((int8_t*) out)[i] = small & (int8_t) (pow(2, bw) - 1);
            }
            else if (bw == 8)
                ((int8_t*) out)[i] = (int8_t) STD_MAX(STD_MIN(q, 127.0), -128.0);
            else if (bw == 16)
                ((int16_t*) out)[i] = (int16_t) STD_MAX(STD_MIN(q, 32767.0), -32768.0);
            else
                ((int32_t*) out)[i] = (int32_t) STD_MAX(STD_MIN(q, 2147483647.0), -2147483648.0);
        }
    }
}

/* trim_functions.cpp:388-605 (dequantizeFromPackedFxpCpu) */
void orc_dequantize_packed(const void* in, int64_t n, const double* enc4, int bw, int is_signed, float* out)
{
    const double delta = enc4[2], offset = enc4[3];
    for (int64_t i = 0; i < n; ++i)
    {
        double code;
        if (!is_signed)
            code = bw <= 8 ? (double) ((const uint8_t*) in)[i] : (bw == 16 ? (double) ((const uint16_t*) in)[i] : (double) ((const uint32_t*) in)[i]);
        else if (bw < 8)
        {
            int8_t b = ((const int8_t*) in)[i];
            code     = (b & (int8_t) pow(2, bw - 1)) ? (double) (int8_t) (~((int8_t) pow(2, bw) - 1) | b) : (double) b;
        }
        else
            code = bw == 8 ? (double) ((const int8_t*) in)[i] : (bw == 16 ? (double) ((const int16_t*) in)[i] : (double) ((const int32_t*) in)[i]);
        out[i] = (float) (delta * (code + offset));
    }
}

