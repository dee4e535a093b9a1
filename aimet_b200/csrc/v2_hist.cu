// aimet_torch v2 histogram statistics and SQNR range search on the device.
//
// Follows aimet_torch/v2/quantization/encoding_analyzer.py: _HistogramObserver.collect_stats (:145-182), merge_stats
// (:212-262), _create_bin_edges (:194-203), _get_bin_num (:205-208) and SqnrEncodingAnalyzer (:577-725).  That code is
// a sequence of float32 tensor operations; every operation here is the same IEEE float32 operation in the same order
// (explicit round-to-nearest intrinsics, no contraction), so histograms, bin edges, candidates and the chosen
// (delta, offset) come out with the reference's bits.  Two things are decided outside that file:
//   * torch.histc.  The bin rule of the installed CPU operator was derived by experiment (values on, just below and
//     just above every boundary): elements outside [lo, hi] and NaN are ignored, an element goes to bin
//     min(bins - 1, floor(fl(fl((x - lo) * bins) / (hi - lo)))), and equal bounds are replaced by (lo - 1, hi + 1).
//     tests/golden/histc_rule.npz holds the boundary-value fixtures this rule is locked to.
//   * the reduction order of torch.sum over the bins of a candidate's noise, which torch does not specify.  The
//     float32 terms are the reference's; they are accumulated in double and rounded to float32 once, so only
//     candidates whose noise agrees to the last float32 bit can be ordered differently.
#include <float.h>
#include <limits.h>
#include <math.h>
#include <stddef.h>

#include "common.cuh"
#include "kernels.h"
#include <type_traits>

namespace aq
{

constexpr int kV2HistThreads  = 256;
constexpr int kV2HistMaxParts = 1024;
constexpr int kV2HistUnroll   = 4;
constexpr int kV2HistQueue    = 1024;   // packets a CTA can put aside for the exact rule
constexpr float kEps32        = 1.1920928955078125e-07f;   // torch.finfo(torch.float32).eps

// Scratch of one collect / merge sequence (device memory, caller-owned):
//   uint32 counts[AQ_V2HIST_MAX_BINS + 2]   bins, then "below lo", then "above hi"
//   uint32 counts2[...]                     a second set for the fused collect + merge
//   float2 partials[kV2HistMaxParts]        per-CTA finite (min, max)
//   float  plan[8]                          lo, hi, batch_min, batch_max, any_finite, pad...
struct V2HistScratch
{
    uint32_t counts[AQ_V2HIST_MAX_BINS + 2];
    uint32_t pad[2];
    uint32_t counts2[AQ_V2HIST_MAX_BINS + 2];   // the same batch counted over the widened range (fused update)
    uint32_t pad2[2];
    float2 partials[kV2HistMaxParts];
    float plan[8];   // lo, hi, batch_min, batch_max, any_finite, widened lo, widened hi
};

// Several histograms per launch (per-channel observers): blockIdx.y is the histogram; these are the distances between
// consecutive histograms' inputs, scratch areas, statistics blocks and re-binning buffers.  All zero for one histogram.
// Where the counting kernel reads its range and adds its counts when that is not the scratch area: one batch's rows of
// a plan table (8 floats per histogram) and of a counts table (bins + 2 words per histogram).  Null = scratch.
struct V2HDirect
{
    const float* plan;
    uint32_t* counts;
};

struct V2HRows
{
    int64_t x_stride;     // elements
    int64_t sc_stride;    // bytes
    int64_t st_stride;    // bytes
    int64_t upd_stride;   // floats
};
template <typename P>
__device__ __forceinline__ P* v2h_row(P* base, int64_t stride_bytes)
{
    return reinterpret_cast<P*>(reinterpret_cast<char*>(const_cast<typename std::remove_const<P>::type*>(base)) +
                                (int64_t) blockIdx.y * stride_bytes);
}

int64_t v2hist_scratch_bytes()
{
    return (int64_t) ((sizeof(V2HistScratch) + 255) / 256 * 256);
}

__device__ __forceinline__ float* v2h_hist(aq_v2hist_head_t* s)
{
    return reinterpret_cast<float*>(s + 1);
}
__device__ __forceinline__ float* v2h_edges(aq_v2hist_head_t* s, int nb)
{
    return reinterpret_cast<float*>(s + 1) + nb;
}

// ---- pass 1: min / max over the finite elements -----------------------------------------------------------------
template <typename T, int VEC>
__global__ void __launch_bounds__(kV2HistThreads) v2h_finite_minmax_kernel(const T* __restrict__ x, int64_t n,
                                                                           float2* __restrict__ partials, V2HRows rw)
{
    pdl_launch_dependents();
    pdl_wait();
    x += (int64_t) blockIdx.y * rw.x_stride;
    partials = v2h_row(partials, rw.sc_stride);
    float mn = INFINITY, mx = -INFINITY;
    auto take = [&](float f) {
        if (fabsf(f) <= FLT_MAX)   // false for NaN and +-Inf
        {
            mn = fminf(mn, f);
            mx = fmaxf(mx, f);
        }
    };
    const int64_t npack  = n / VEC;
    const int64_t stride = (int64_t) gridDim.x * kV2HistThreads;
    int64_t p            = (int64_t) blockIdx.x * kV2HistThreads + threadIdx.x;
    // kV2HistUnroll packets in flight per thread (one at a time left the pass latency-bound at a quarter of the
    // memory bandwidth); the last, partial group is issued together as well
    for (; p + (kV2HistUnroll - 1) * stride < npack; p += kV2HistUnroll * stride)
    {
        Pack<T, VEC> v[kV2HistUnroll];
#pragma unroll
        for (int u = 0; u < kV2HistUnroll; ++u)
            v[u] = load_pack<T, VEC>(x + (p + u * stride) * VEC);
#pragma unroll
        for (int u = 0; u < kV2HistUnroll; ++u)
#pragma unroll
            for (int e = 0; e < VEC; ++e)
                take(to_f32<T>(v[u].v[e]));
    }
    {
        Pack<T, VEC> v[kV2HistUnroll - 1];
#pragma unroll
        for (int u = 0; u < kV2HistUnroll - 1; ++u)
            if (p + u * stride < npack)
                v[u] = load_pack<T, VEC>(x + (p + u * stride) * VEC);
#pragma unroll
        for (int u = 0; u < kV2HistUnroll - 1; ++u)
            if (p + u * stride < npack)
#pragma unroll
                for (int e = 0; e < VEC; ++e)
                    take(to_f32<T>(v[u].v[e]));
    }
    if (blockIdx.x == 0 && threadIdx.x < (int) (n - npack * VEC))
        take(to_f32<T>(x[npack * VEC + threadIdx.x]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
    {
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    __shared__ float s_mn[kV2HistThreads / 32], s_mx[kV2HistThreads / 32];
    if ((threadIdx.x & 31) == 0)
        s_mn[threadIdx.x >> 5] = mn, s_mx[threadIdx.x >> 5] = mx;
    __syncthreads();
    if (threadIdx.x == 0)
    {
        for (int w = 1; w < kV2HistThreads / 32; ++w)
            mn = fminf(mn, s_mn[w]), mx = fmaxf(mx, s_mx[w]);
        partials[blockIdx.x] = make_float2(mn, mx);
    }
}

// ---- plan: fold the partials, decide the range the histogram pass uses, clear the counters -------------------------
// merge = 0: the batch alone (collect_stats): range = first and last bin edge of _create_bin_edges(min, max).
// merge = 1: the widened range of merge_stats: [min(batch, state), max(batch, state)].
__global__ void __launch_bounds__(kV2HistThreads) v2h_plan_kernel(V2HistScratch* __restrict__ sc, int nparts, int nb,
                                                                  int merge, const aq_v2hist_head_t* __restrict__ state,
                                                                  const aq_v2hist_head_t* __restrict__ batch, V2HRows rw)
{
    pdl_launch_dependents();
    pdl_wait();
    sc    = v2h_row(sc, rw.sc_stride);
    state = state ? v2h_row(state, rw.st_stride) : nullptr;
    batch = batch ? v2h_row(batch, rw.st_stride) : nullptr;
    float mn = INFINITY, mx = -INFINITY;
    if (batch)
    {
        // the batch's own statistics already hold its finite min / max: no second pass over the data for them
        if (!batch->error)
            mn = batch->min, mx = batch->max;
    }
    else
    {
        for (int i = threadIdx.x; i < nparts; i += kV2HistThreads)
        {
            mn = fminf(mn, sc->partials[i].x);
            mx = fmaxf(mx, sc->partials[i].y);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
    {
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    __shared__ float s_mn[kV2HistThreads / 32], s_mx[kV2HistThreads / 32];
    if ((threadIdx.x & 31) == 0)
        s_mn[threadIdx.x >> 5] = mn, s_mx[threadIdx.x >> 5] = mx;
    for (int i = threadIdx.x; i < nb + 2; i += kV2HistThreads)
    {
        sc->counts[i] = 0;
        if (merge == 2)
            sc->counts2[i] = 0;
    }
    __syncthreads();
    if (threadIdx.x != 0)
        return;
    for (int w = 1; w < kV2HistThreads / 32; ++w)
        mn = fminf(mn, s_mn[w]), mx = fmaxf(mx, s_mx[w]);
    const bool any = mn <= mx;
    float lo, hi;
    if (!any)
    {
        lo = 0.0f, hi = 1.0f;   // nothing finite: the caller is told through any_finite; counters stay meaningless
        mn = mx = 0.0f;
    }
    else if (merge != 1)
    {
        float a = mn, b = mx;
        if (a == b)
            a = __fsub_rn(a, 0.5f), b = __fadd_rn(b, 0.5f);
        const float step = __fdiv_rn(__fsub_rn(b, a), (float) nb);
        lo               = __fadd_rn(__fmul_rn(0.0f, step), a);
        hi               = __fadd_rn(__fmul_rn((float) nb, step), a);
    }
    else
    {
        // Python min(new, cur) / max(new, cur): the second argument wins only when it is strictly smaller / larger
        lo = (state->min < mn) ? state->min : mn;
        hi = (state->max > mx) ? state->max : mx;
    }
    sc->plan[0] = lo, sc->plan[1] = hi, sc->plan[2] = mn, sc->plan[3] = mx, sc->plan[4] = any ? 1.0f : 0.0f;
    if (merge == 2)
    {
        // fused collect + merge: the widened range as well (with nothing finite in the batch it is never used for bins)
        sc->plan[5] = any ? ((state->min < mn) ? state->min : mn) : 0.0f;
        sc->plan[6] = any ? ((state->max > mx) ? state->max : mx) : 1.0f;
    }
}

// ---- pass 2: counts with the torch.histc bin rule, plus the elements below lo and above hi ------------------------
// DUAL: the batch is counted over its own range AND over the widened range of the merge in the same pass.
// The exact bin rule, out of line: it runs for about one element in a thousand.
__device__ __noinline__ float v2h_exact_quotient_floor(float t, float w)
{
    return floorf(__fdiv_rn(t, w));
}

template <typename T, int VEC, bool DUAL>
__global__ void __launch_bounds__(kV2HistThreads) v2h_count_kernel(const T* __restrict__ x, int64_t n,
                                                                   V2HistScratch* __restrict__ sc, int nb, V2HRows rw,
                                                                   V2HDirect direct)
{
    pdl_launch_dependents();
    extern __shared__ uint32_t s_cnt[];   // nb + 2 (twice with DUAL)
    __shared__ long long s_queue[kV2HistQueue];   // packets put aside for the exact rule
    __shared__ int s_queued;
    for (int i = threadIdx.x; i < (DUAL ? 2 : 1) * (nb + 2); i += kV2HistThreads)
        s_cnt[i] = 0;
    if (threadIdx.x == 0)
        s_queued = 0;   // (the barrier below comes before the first push)
    pdl_wait();
    x += (int64_t) blockIdx.y * rw.x_stride;
    sc = v2h_row(sc, rw.sc_stride);
    // range and counters: the scratch area's, or (sharded calibration) a row of the caller's plan and counts tables
    const float* __restrict__ plan = direct.plan ? direct.plan + (int64_t) blockIdx.y * 8 : sc->plan;
    uint32_t* __restrict__ out     = direct.counts ? direct.counts + (int64_t) blockIdx.y * (nb + 2) : sc->counts;
    float lo = plan[0], hi = plan[1];
    const float cmp_lo = lo, cmp_hi = hi;
    if (lo == hi)
        lo = __fsub_rn(lo, 1.0f), hi = __fadd_rn(hi, 1.0f);   // torch.histc's own rule for equal bounds
    const float width = __fsub_rn(hi, lo);
    const float nbf   = (float) nb;
    float lo2 = 0.0f, hi2 = 0.0f, cmp_lo2 = 0.0f, cmp_hi2 = 0.0f, width2 = 1.0f;
    if (DUAL)
    {
        lo2 = plan[5], hi2 = plan[6];
        cmp_lo2 = lo2, cmp_hi2 = hi2;
        if (lo2 == hi2)
            lo2 = __fsub_rn(lo2, 1.0f), hi2 = __fadd_rn(hi2, 1.0f);
        width2 = __fsub_rn(hi2, lo2);
    }
    uint32_t* s_cnt2 = s_cnt + (nb + 2);
    __syncthreads();
    // bin = min(nb - 1, floor(((f - lo) * nb) / width)) needs the correctly rounded quotient only when it lies next to an
    // integer: the product with the rounded reciprocal differs from it by less than 2^-22 |q|.  The sweep bins with the
    // reciprocal and tests a whole packet at once; a packet with an element inside that band around an integer (about
    // one element in a thousand) is not counted but queued, and the CTA counts the queued packets with the exact rule
    // after its sweep.  A queue that overflows (data sitting on the bin edges, e.g. values that are already quantized)
    // makes the CTA drop what it has and count its whole share with the exact rule.
    const float rwidth = __frcp_rn(width), rwidth2 = __frcp_rn(width2);
    auto exact_bin = [&](float f, float lo_, float w_) {
        const int b = (int) v2h_exact_quotient_floor(__fmul_rn(__fsub_rn(f, lo_), nbf), w_);
        return b < nb - 1 ? b : nb - 1;
    };
    // Fast bin of one element; `worst` collects, over a packet, |frac(qf) - 0.5| + 2^-22 qf: above 0.5 means that some
    // quotient is within its band of an integer (unsure).  floor(qf) for 0 <= qf < 2^22 comes from two additions
    // instead of the conversion unit: with h = qf - 0.5 (exact), RN(h + 1.5 * 2^23) - 1.5 * 2^23 is the integer nearest
    // to h, i.e. floor(qf) unless qf is an integer (a tie), and integers are unsure anyway; h minus that integer is
    // frac(qf) - 0.5, exactly.  A quotient of exactly 0 (an element equal to lo, e.g. the zeros of a post-ReLU batch)
    // gives 0.5 + 0, which counts as sure: it is bin 0 under either form.  The test itself may round as it likes (a
    // fused multiply-add): the band has half an ulp of the quotient to spare.  NaN, from an infinite element, is
    // ignored by the maximum: such an element is never binned.
    constexpr float kMagic   = 12582912.0f;
    constexpr int kMagicBits = 0x4B400000;
    auto fast_bin = [&](float f, float lo_, float rw_, float& worst) {
        const float qf = __fmul_rn(__fmul_rn(__fsub_rn(f, lo_), nbf), rw_);
        const float h  = __fsub_rn(qf, 0.5f);
        const float u  = __fadd_rn(h, kMagic);
        const float e  = __fsub_rn(h, __fsub_rn(u, kMagic));
        worst          = fmaxf(worst, __fmaf_rn(qf, 2.384185791015625e-07f, fabsf(e)));
        const int b    = __float_as_int(u) - kMagicBits;
        return b < nb - 1 ? b : nb - 1;
    };
    // An element inside [lo, hi] is never beyond the edges the end bins are judged by (the two pairs differ only when
    // the bounds are equal, and then every finite element equals them), so the tests are exclusive.
    auto put = [&](uint32_t* cnt, float f, int b, uint32_t k, float lo_, float hi_, float clo, float chi) {
        if (f >= lo_ && f <= hi_)
            atomicAdd(&cnt[b], k);
        else if (f < clo)
            atomicAdd(&cnt[nb], k);
        else if (f > chi)
            atomicAdd(&cnt[nb + 1], k);
    };
    auto take_n = [&](float f, uint32_t k) {
        put(s_cnt, f, exact_bin(f, lo, width), k, lo, hi, cmp_lo, cmp_hi);
        if (DUAL)
            put(s_cnt2, f, exact_bin(f, lo2, width2), k, lo2, hi2, cmp_lo2, cmp_hi2);
    };
    // Exact zeros (half of a post-ReLU activation) would all land on one counter: they are tallied in a register and
    // added once per thread at the end.
    uint32_t zeros = 0;
    auto take = [&](float f) {
        if (f == 0.0f)
            ++zeros;
        else
            take_n(f, 1u);
    };
    // The same for two elements at a time (two float32 lanes per instruction); every operation rounds as in fast_bin.
    const f32x2_t k_nb = pair(nbf, nbf), k_half = pair(0.5f, 0.5f), k_magic = pair(kMagic, kMagic);
    const f32x2_t k_band = pair(2.384185791015625e-07f, 2.384185791015625e-07f);
    auto fast_bin2 = [&](float f0, float f1, float lo_, float rw_, float& worst, int& b0, int& b1) {
        const f32x2_t qf = mul2(mul2(sub2(pair(f0, f1), pair(lo_, lo_)), k_nb), pair(rw_, rw_));
        const f32x2_t h  = sub2(qf, k_half);
        const f32x2_t u  = add2(h, k_magic);
        const f32x2_t fl = sub2(u, k_magic);
        // |e| + band = max(band + e, band - e) with e = h - fl
        float p0, p1, n0, n1, u0, u1;
        unpair(fma2(qf, k_band, sub2(h, fl)), p0, p1);
        unpair(fma2(qf, k_band, sub2(fl, h)), n0, n1);
        asm("max.f32 %0, %0, %1, %2;" : "+f"(worst) : "f"(p0), "f"(p1));
        asm("max.f32 %0, %0, %1, %2;" : "+f"(worst) : "f"(n0), "f"(n1));
        unpair(u, u0, u1);
        b0 = __float_as_int(u0) - kMagicBits;
        b1 = __float_as_int(u1) - kMagicBits;
        b0 = b0 < nb - 1 ? b0 : nb - 1;
        b1 = b1 < nb - 1 ? b1 : nb - 1;
    };
    // counter += 1 under a predicate, without a branch
    auto count_if = [&](uint32_t* counter, bool on) {
        const unsigned a = (unsigned) __cvta_generic_to_shared(counter);
        asm volatile("{ .reg .pred q; setp.ne.u32 q, %1, 0; @q red.shared.add.u32 [%0], 1; }" ::"r"(a), "r"((unsigned) on)
                     : "memory");
    };
    auto take_packet = [&](const Pack<T, VEC>& v, int64_t p) {
        float f[VEC];
        int b[VEC], b2[VEC];
        float worst = 0.0f;
#pragma unroll
        for (int e = 0; e < VEC; ++e)
            f[e] = to_f32<T>(v.v[e]);
        if (VEC == 1)
        {
            b[0] = fast_bin(f[0], lo, rwidth, worst);
            if (DUAL)
                b2[0] = fast_bin(f[0], lo2, rwidth2, worst);
        }
        else
        {
#pragma unroll
            for (int e = 0; e + 1 < VEC; e += 2)
            {
                fast_bin2(f[e], f[e + 1], lo, rwidth, worst, b[e], b[e + 1]);
                if (DUAL)
                    fast_bin2(f[e], f[e + 1], lo2, rwidth2, worst, b2[e], b2[e + 1]);
            }
        }
        // the packet's smallest and largest element, NaN if it holds one: a packet that is not wholly inside the
        // range(s) -- an infinity, a NaN, the one element beyond a rounded last edge -- is left to the exact pass too,
        // so that the sweep needs no range test per element
        float vmin = f[0], vmax = f[0];
#pragma unroll
        for (int e = 1; e < VEC; e += 2)
        {
            const float g = f[e + 1 < VEC ? e + 1 : e];
            asm("min.NaN.f32 %0, %0, %1, %2;" : "+f"(vmin) : "f"(f[e]), "f"(g));
            asm("max.NaN.f32 %0, %0, %1, %2;" : "+f"(vmax) : "f"(f[e]), "f"(g));
        }
        bool sure = worst <= 0.5f && vmin >= lo && vmax <= hi;
        if (DUAL)
            sure = sure && vmin >= lo2 && vmax <= hi2;
        if (!sure)
        {
            const int slot = atomicAdd(&s_queued, 1);
            if ((unsigned) slot < (unsigned) kV2HistQueue)
                s_queue[slot] = p;
            return;
        }
#pragma unroll
        for (int e = 0; e < VEC; ++e)
        {
            const bool nz = f[e] != 0.0f;
            if (DUAL)
            {
                // two counters per element: skipping both for a zero is worth a branch
                if (nz)
                {
                    atomicAdd(&s_cnt[b[e]], 1u);
                    atomicAdd(&s_cnt2[b2[e]], 1u);
                }
                else
                    ++zeros;
            }
            else
            {
                zeros += nz ? 0u : 1u;
                count_if(&s_cnt[b[e]], nz);
            }
        }
    };
    const int64_t npack  = n / VEC;
    const int64_t stride = (int64_t) gridDim.x * kV2HistThreads;
    int64_t p            = (int64_t) blockIdx.x * kV2HistThreads + threadIdx.x;
    for (; p + (kV2HistUnroll - 1) * stride < npack; p += kV2HistUnroll * stride)
    {
        Pack<T, VEC> v[kV2HistUnroll];
#pragma unroll
        for (int u = 0; u < kV2HistUnroll; ++u)
            v[u] = load_pack<T, VEC>(x + (p + u * stride) * VEC);
#pragma unroll
        for (int u = 0; u < kV2HistUnroll; ++u)
            take_packet(v[u], p + u * stride);
    }
    {
        Pack<T, VEC> v[kV2HistUnroll - 1];
#pragma unroll
        for (int u = 0; u < kV2HistUnroll - 1; ++u)
            if (p + u * stride < npack)
                v[u] = load_pack<T, VEC>(x + (p + u * stride) * VEC);
#pragma unroll
        for (int u = 0; u < kV2HistUnroll - 1; ++u)
            if (p + u * stride < npack)
                take_packet(v[u], p + u * stride);
    }
    if (blockIdx.x == 0 && threadIdx.x < (int) (n - npack * VEC))
        take(to_f32<T>(x[npack * VEC + threadIdx.x]));
    __syncthreads();
    const int queued = s_queued;
    if (queued <= kV2HistQueue)
    {
        for (int i = threadIdx.x; i < queued; i += kV2HistThreads)
        {
            const Pack<T, VEC> v = load_pack<T, VEC>(x + s_queue[i] * VEC);
#pragma unroll 1
            for (int e = 0; e < VEC; ++e)
                take(to_f32<T>(v.v[e]));
        }
    }
    else
    {
        // start over, exactly (block-uniform)
        for (int i = threadIdx.x; i < (DUAL ? 2 : 1) * (nb + 2); i += kV2HistThreads)
            s_cnt[i] = 0;
        zeros = 0;
        __syncthreads();
        for (int64_t q = (int64_t) blockIdx.x * kV2HistThreads + threadIdx.x; q < npack; q += stride)
        {
            const Pack<T, VEC> v = load_pack<T, VEC>(x + q * VEC);
#pragma unroll 1
            for (int e = 0; e < VEC; ++e)
                take(to_f32<T>(v.v[e]));
        }
        if (blockIdx.x == 0 && threadIdx.x < (int) (n - npack * VEC))
            take(to_f32<T>(x[npack * VEC + threadIdx.x]));
    }
    if (zeros)
        take_n(0.0f, zeros);
    __syncthreads();
    for (int i = threadIdx.x; i < nb + 2; i += kV2HistThreads)
    {
        if (s_cnt[i])
            atomicAdd(&out[i], s_cnt[i]);
        if (DUAL && s_cnt2[i])
            atomicAdd(&sc->counts2[i], s_cnt2[i]);
    }
}

// _create_bin_edges(min, max): arange(0, bins + 1) * step + min with step = (max - min) / bins, after widening equal
// bounds by 0.5 on either side.
__device__ __forceinline__ void v2h_write_edges(float mn, float mx, int nb, float* __restrict__ edges)
{
    if (mx == mn)
        mn = __fsub_rn(mn, 0.5f), mx = __fadd_rn(mx, 0.5f);
    const float step = __fdiv_rn(__fsub_rn(mx, mn), (float) nb);
    for (int i = threadIdx.x; i <= nb; i += blockDim.x)
        edges[i] = __fadd_rn(__fmul_rn((float) i, step), mn);
}

// ---- collect_stats: the batch's own _Histogram ---------------------------------------------------------------------
// One CTA; counts = bins, then "below the first edge", then "above the last edge".
__device__ __forceinline__ void v2h_collect_step(const uint32_t* __restrict__ counts, float mn, float mx, bool any, int nb,
                                                 aq_v2hist_head_t* __restrict__ out)
{
    float* hist = v2h_hist(out);
    for (int i = threadIdx.x; i < nb; i += kV2HistThreads)
    {
        float h = (float) counts[i];
        if (i == 0)
            h = __fadd_rn(h, (float) counts[nb]);          // histogram[0]  += sum(x < bin_edges[0])
        if (i == nb - 1)
            h = __fadd_rn(h, (float) counts[nb + 1]);      // histogram[-1] += sum(x > bin_edges[-1])
        hist[i] = h;
    }
    v2h_write_edges(mn, mx, nb, v2h_edges(out, nb));
    if (threadIdx.x == 0)
    {
        out->min = mn, out->max = mx;
        out->initialized = 1;
        out->error       = any ? 0 : 1;
    }
}

__global__ void __launch_bounds__(kV2HistThreads) v2h_finish_collect_kernel(const V2HistScratch* __restrict__ sc, int nb,
                                                                            aq_v2hist_head_t* __restrict__ out, V2HRows rw)
{
    pdl_launch_dependents();
    pdl_wait();
    sc  = v2h_row(sc, rw.sc_stride);
    out = v2h_row(out, rw.st_stride);
    v2h_collect_step(sc->counts, sc->plan[2], sc->plan[3], sc->plan[4] != 0.0f, nb, out);
}

// torch.minimum: NaN wins
__device__ __forceinline__ float torch_minimum(float a, float b)
{
    return (a != a || b != b) ? NAN : (a < b ? a : b);
}
__device__ __forceinline__ int v2h_bin_num(float width, float cur_min, float data, int nb)
{
    // _get_bin_num: ((data - curr_min) / bin_width).to(int32) clipped to bins - 1
    const float idx = __fdiv_rn(__fsub_rn(data, cur_min), width);
    int b;
    if (!(idx > -2147483648.0f && idx < 2147483648.0f))
        b = INT_MIN;   // what the x86 float->int32 conversion gives for NaN and out-of-range values
    else
        b = (int) idx;
    return b < nb - 1 ? b : nb - 1;
}

// ---- merge_stats: state <- state re-binned to the widened range + the batch counted at that range -----------------
// The re-binning is two sequential scatter loops over the bins in the reference (float additions whose order matters
// once counts pass 2^24): one thread walks them in the same order; the rest is element-wise.
// The old counts moved into the bins of the widened range (merge_stats, encoding_analyzer.py:229-249): two sequential
// scatter loops whose float additions happen in the reference's order.  One thread; `updates` starts at zero.
__device__ __forceinline__ void v2h_rebin_serial(const float* __restrict__ hist, float* __restrict__ updates, float cmin,
                                                 float cmax, float umin, float umax, int nb)
{
    const float dest_w = __fdiv_rn(__fsub_rn(umax, umin), (float) nb);
    const float src_w  = __fdiv_rn(__fsub_rn(cmax, cmin), (float) nb);
    for (int i = 0; i < nb; ++i)
    {
        const float src_start = __fadd_rn(cmin, __fmul_rn(src_w, (float) i));
        const int dest        = v2h_bin_num(dest_w, umin, src_start, nb);
        const float dest_end  = __fadd_rn(umin, __fmul_rn(dest_w, (float) (dest + 1)));
        const float split     = rintf(__fmul_rn(__fdiv_rn(__fsub_rn(dest_end, src_start), src_w), hist[i]));
        const float upd       = torch_minimum(split, hist[i]);
        if (dest >= 0)
            updates[dest] = __fadd_rn(updates[dest], upd);
    }
    for (int i = 0; i < nb; ++i)
    {
        // recomputed rather than stored: the same operations give the same values
        const float src_start = __fadd_rn(cmin, __fmul_rn(src_w, (float) i));
        const int dest        = v2h_bin_num(dest_w, umin, src_start, nb);
        const float dest_end  = __fadd_rn(umin, __fmul_rn(dest_w, (float) (dest + 1)));
        const float split     = rintf(__fmul_rn(__fdiv_rn(__fsub_rn(dest_end, src_start), src_w), hist[i]));
        const float upd       = torch_minimum(split, hist[i]);
        if (upd < hist[i])
        {
            const int other = v2h_bin_num(dest_w, umin, __fadd_rn(src_start, dest_w), nb);
            if (other >= 0)
                updates[other] = __fadd_rn(updates[other], __fsub_rn(hist[i], upd));
        }
    }
}

// One CTA.  counts: the batch counted over [umin, umax] (bins, then -inf, then +inf elements).
__device__ __forceinline__ void v2h_merge_step(const uint32_t* __restrict__ counts, float umin, float umax, bool any,
                                               int nb, aq_v2hist_head_t* __restrict__ state, float* __restrict__ updates)
{
    float* hist      = v2h_hist(state);
    const float cmin = state->min, cmax = state->max;
    const bool same  = (umin == cmin) && (umax == cmax);
    if (same)
    {
        for (int i = threadIdx.x; i < nb; i += kV2HistThreads)
            updates[i] = hist[i];
    }
    else
    {
        for (int i = threadIdx.x; i < nb; i += kV2HistThreads)
            updates[i] = 0.0f;
    }
    __syncthreads();
    if (!same && threadIdx.x == 0)
        v2h_rebin_serial(hist, updates, cmin, cmax, umin, umax, nb);
    __syncthreads();
    for (int i = threadIdx.x; i < nb; i += kV2HistThreads)
    {
        float h = __fadd_rn((float) counts[i], updates[i]);
        if (i == 0)
            h = __fadd_rn(h, (float) counts[nb]);        // expanded[0]  += sum(x == -inf)
        if (i == nb - 1)
            h = __fadd_rn(h, (float) counts[nb + 1]);    // expanded[-1] += sum(x == +inf)
        hist[i] = h;
    }
    v2h_write_edges(umin, umax, nb, v2h_edges(state, nb));
    __syncthreads();
    if (threadIdx.x == 0)
    {
        state->min = umin, state->max = umax;
        if (!any)
            state->error = 1;
    }
}

__global__ void __launch_bounds__(kV2HistThreads) v2h_merge_kernel(const V2HistScratch* __restrict__ sc, int nb,
                                                                   aq_v2hist_head_t* __restrict__ state,
                                                                   float* __restrict__ updates /* nb floats */, V2HRows rw,
                                                                   int dual)
{
    pdl_launch_dependents();
    pdl_wait();
    sc      = v2h_row(sc, rw.sc_stride);
    state   = v2h_row(state, rw.st_stride);
    updates += (int64_t) blockIdx.y * rw.upd_stride;
    // after a fused pass the widened range and its counts sit in the second set
    const uint32_t* __restrict__ counts = dual ? sc->counts2 : sc->counts;
    const float umin = dual ? sc->plan[5] : sc->plan[0], umax = dual ? sc->plan[6] : sc->plan[1];
    if (dual && sc->plan[4] == 0.0f)
    {
        // nothing finite in the batch: the reference raises; here the state is flagged and left as it is
        if (threadIdx.x == 0)
            state->error = 1;
        return;
    }
    v2h_merge_step(counts, umin, umax, sc->plan[4] != 0.0f, nb, state, updates);
}

// The tail of a fused update in one launch: the batch's own statistics from the first set of counters, then the merge
// from the second set (they write different blocks).
__global__ void __launch_bounds__(kV2HistThreads) v2h_finish_update_kernel(const V2HistScratch* __restrict__ sc, int nb,
                                                                           aq_v2hist_head_t* __restrict__ batch,
                                                                           aq_v2hist_head_t* __restrict__ state,
                                                                           float* __restrict__ updates, V2HRows rw)
{
    pdl_launch_dependents();
    pdl_wait();
    sc    = v2h_row(sc, rw.sc_stride);
    batch = v2h_row(batch, rw.st_stride);
    state = v2h_row(state, rw.st_stride);
    updates += (int64_t) blockIdx.y * rw.upd_stride;
    const bool any = sc->plan[4] != 0.0f;
    v2h_collect_step(sc->counts, sc->plan[2], sc->plan[3], any, nb, batch);
    if (!any)
    {
        // nothing finite in the batch: the reference raises; here the state is flagged and left as it is
        if (threadIdx.x == 0)
            state->error = 1;
        return;
    }
    v2h_merge_step(sc->counts2, sc->plan[5], sc->plan[6], true, nb, state, updates);
}

__global__ void __launch_bounds__(kV2HistThreads) v2h_copy_kernel(const aq_v2hist_head_t* __restrict__ src, int nb,
                                                                  aq_v2hist_head_t* __restrict__ dst, V2HRows rw)
{
    pdl_launch_dependents();
    pdl_wait();
    src = v2h_row(src, rw.st_stride);
    dst = v2h_row(dst, rw.st_stride);
    const float* s = reinterpret_cast<const float*>(src + 1);
    float* d       = reinterpret_cast<float*>(dst + 1);
    for (int i = threadIdx.x; i < 2 * nb + 1; i += kV2HistThreads)
        d[i] = s[i];
    if (threadIdx.x == 0)
        *dst = *src;
}

// ---- launchers ------------------------------------------------------------------------------------------------------
// Grid of the counting kernel: CTAs walk their share with a grid stride, so the grid is one resident wave over all rows
// -- as many CTAs per SM as the instantiation's registers and this launch's shared memory allow.
template <typename T, int V, bool DUAL>
static int64_t v2h_count_grid(int64_t n, int rows, size_t smem)
{
    static int per_sm        = 0;
    static size_t per_sm_for = 0;
    if (per_sm == 0 || per_sm_for != smem)
    {
        int v = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&v, v2h_count_kernel<T, V, DUAL>, kV2HistThreads, smem) !=
                cudaSuccess || v < 1)
            v = 4;
        per_sm = v, per_sm_for = smem;
    }
    int64_t blocks = (n + (int64_t) kV2HistThreads * V * 4 - 1) / ((int64_t) kV2HistThreads * V * 4);
    int64_t cap    = (int64_t) kNumSMs * per_sm / rows;
    cap            = cap < 1 ? 1 : cap;
    return blocks > cap ? cap : (blocks < 1 ? 1 : blocks);
}

// rows histograms of n elements each (row r starts at x + r * n), one grid row per histogram.
template <typename T>
static int v2h_passes(const T* x, int64_t n, int rows, int nb, int merge, const aq_v2hist_head_t* state,
                      const aq_v2hist_head_t* batch, V2HistScratch* sc, const V2HRows& rw, cudaStream_t st)
{
    const int vec      = pick_vec<T>(x, nullptr, nullptr, rows > 1 ? n : 0);
    int64_t blocks     = (n + (int64_t) kV2HistThreads * vec * 4 - 1) / ((int64_t) kV2HistThreads * vec * 4);
    int64_t cap        = (int64_t) kNumSMs * 6 / rows;   // about one resident wave over all rows
    cap                = cap < 1 ? 1 : cap;
    blocks             = blocks > cap ? cap : (blocks < 1 ? 1 : blocks);
    const int nparts   = (int) (blocks < kV2HistMaxParts ? blocks : kV2HistMaxParts);
    const size_t smem  = (size_t) (nb + 2) * sizeof(uint32_t);
    const unsigned ry  = (unsigned) rows;
#define AQ_V2H(V)                                                                                                    \
    if (!batch)                                                                                                      \
    {                                                                                                                \
        launch_pdl(v2h_finite_minmax_kernel<T, V>, dim3((unsigned) nparts, ry), kV2HistThreads, 0, st, x, n,         \
                   sc->partials, rw);                                                                                \
        note_launch();                                                                                               \
    }                                                                                                                \
    launch_pdl(v2h_plan_kernel, dim3(1, ry), kV2HistThreads, 0, st, sc, nparts, nb, merge, state, batch, rw);        \
    note_launch();                                                                                                   \
    if (merge == 2)                                                                                                  \
        launch_pdl(v2h_count_kernel<T, V, true>, dim3((unsigned) v2h_count_grid<T, V, true>(n, rows, 2 * smem), ry), \
                   kV2HistThreads, 2 * smem, st, x, n, sc, nb, rw, V2HDirect {nullptr, nullptr});                    \
    else                                                                                                             \
        launch_pdl(v2h_count_kernel<T, V, false>, dim3((unsigned) v2h_count_grid<T, V, false>(n, rows, smem), ry),   \
                   kV2HistThreads, smem, st, x, n, sc, nb, rw, V2HDirect {nullptr, nullptr});                        \
    note_launch();
    if (vec >= 4 && sizeof(T) == 4)
    {
        AQ_V2H(4)
    }
    else if (vec >= 8)
    {
        AQ_V2H((sizeof(T) == 2 ? 8 : 4))
    }
    else
    {
        AQ_V2H(1)
    }
#undef AQ_V2H
    return check_launch();
}

static int v2h_passes_any(const void* x, int dtype, int64_t n, int rows, int nb, int merge,
                          const aq_v2hist_head_t* state, const aq_v2hist_head_t* batch, V2HistScratch* sc,
                          const V2HRows& rw, cudaStream_t st)
{
    switch (dtype)
    {
    case AQ_F32: return v2h_passes<float>((const float*) x, n, rows, nb, merge, state, batch, sc, rw, st);
    case AQ_F16: return v2h_passes<__half>((const __half*) x, n, rows, nb, merge, state, batch, sc, rw, st);
    case AQ_BF16:
        return v2h_passes<__nv_bfloat16>((const __nv_bfloat16*) x, n, rows, nb, merge, state, batch, sc, rw, st);
    default: return AQ_ERR_INVALID_ARG;
    }
}

// The two data passes on their own (sharded calibration runs them at different times).
template <typename T>
static void v2h_geometry(const T* x, int64_t n, int rows, int* vec, int64_t* blocks, int* nparts)
{
    *vec        = pick_vec<T>(x, nullptr, nullptr, rows > 1 ? n : 0);
    int64_t b   = (n + (int64_t) kV2HistThreads * *vec * 4 - 1) / ((int64_t) kV2HistThreads * *vec * 4);
    int64_t cap = (int64_t) kNumSMs * 6 / rows;
    cap         = cap < 1 ? 1 : cap;
    b           = b > cap ? cap : (b < 1 ? 1 : b);
    *blocks     = b;
    *nparts     = (int) (b < kV2HistMaxParts ? b : kV2HistMaxParts);
}

template <typename T>
static int v2h_minmax_only(const T* x, int64_t n, int rows, V2HistScratch* sc, const V2HRows& rw, int* nparts,
                           cudaStream_t st)
{
    int vec;
    int64_t blocks;
    v2h_geometry<T>(x, n, rows, &vec, &blocks, nparts);
    const dim3 grid((unsigned) *nparts, (unsigned) rows);
    if (vec >= 4 && sizeof(T) == 4)
        launch_pdl(v2h_finite_minmax_kernel<T, 4>, grid, kV2HistThreads, 0, st, x, n, sc->partials, rw);
    else if (vec >= 8)
        launch_pdl(v2h_finite_minmax_kernel<T, (sizeof(T) == 2 ? 8 : 4)>, grid, kV2HistThreads, 0, st, x, n, sc->partials,
                   rw);
    else
        launch_pdl(v2h_finite_minmax_kernel<T, 1>, grid, kV2HistThreads, 0, st, x, n, sc->partials, rw);
    note_launch();
    return check_launch();
}

template <typename T>
static int v2h_count_only(const T* x, int64_t n, int rows, int nb, const V2HRows& rw, V2HDirect direct, cudaStream_t st)
{
    V2HistScratch* sc = nullptr;
    int vec, nparts;
    int64_t blocks;
    v2h_geometry<T>(x, n, rows, &vec, &blocks, &nparts);
    const size_t smem = (size_t) (nb + 2) * sizeof(uint32_t);
    const unsigned ry = (unsigned) rows;
    constexpr int kWide = sizeof(T) == 2 ? 8 : 4;
    if (vec >= 4 && sizeof(T) == 4)
        launch_pdl(v2h_count_kernel<T, 4, false>, dim3((unsigned) v2h_count_grid<T, 4, false>(n, rows, smem), ry),
                   kV2HistThreads, smem, st, x, n, sc, nb, rw, direct);
    else if (vec >= 8)
        launch_pdl(v2h_count_kernel<T, kWide, false>, dim3((unsigned) v2h_count_grid<T, kWide, false>(n, rows, smem), ry),
                   kV2HistThreads, smem, st, x, n, sc, nb, rw, direct);
    else
        launch_pdl(v2h_count_kernel<T, 1, false>, dim3((unsigned) v2h_count_grid<T, 1, false>(n, rows, smem), ry),
                   kV2HistThreads, smem, st, x, n, sc, nb, rw, direct);
    note_launch();
    return check_launch();
}

static int v2h_minmax_any(const void* x, int dtype, int64_t n, int rows, V2HistScratch* sc, const V2HRows& rw, int* nparts,
                          cudaStream_t st)
{
    switch (dtype)
    {
    case AQ_F32: return v2h_minmax_only<float>((const float*) x, n, rows, sc, rw, nparts, st);
    case AQ_F16: return v2h_minmax_only<__half>((const __half*) x, n, rows, sc, rw, nparts, st);
    case AQ_BF16: return v2h_minmax_only<__nv_bfloat16>((const __nv_bfloat16*) x, n, rows, sc, rw, nparts, st);
    default: return AQ_ERR_INVALID_ARG;
    }
}

static int v2h_count_any(const void* x, int dtype, int64_t n, int rows, int nb, const V2HRows& rw, V2HDirect direct,
                         cudaStream_t st)
{
    switch (dtype)
    {
    case AQ_F32: return v2h_count_only<float>((const float*) x, n, rows, nb, rw, direct, st);
    case AQ_F16: return v2h_count_only<__half>((const __half*) x, n, rows, nb, rw, direct, st);
    case AQ_BF16: return v2h_count_only<__nv_bfloat16>((const __nv_bfloat16*) x, n, rows, nb, rw, direct, st);
    default: return AQ_ERR_INVALID_ARG;
    }
}

int v2hist_collect_rows(const void* x, int dtype, int64_t n, int rows, int nb, aq_v2hist_head_t* batch,
                        int64_t block_stride, void* scratch, cudaStream_t st)
{
    if (rows < 1 || rows > 65535)
        return AQ_ERR_TOO_LARGE;
    V2HistScratch* sc = static_cast<V2HistScratch*>(scratch);
    const V2HRows rw {rows > 1 ? n : 0, rows > 1 ? v2hist_scratch_bytes() : 0, rows > 1 ? block_stride : 0, 0};
    int rc = v2h_passes_any(x, dtype, n, rows, nb, 0, nullptr, nullptr, sc, rw, st);
    if (rc != AQ_OK)
        return rc;
    launch_pdl(v2h_finish_collect_kernel, dim3(1, (unsigned) rows), kV2HistThreads, 0, st, (const V2HistScratch*) sc, nb,
               batch, rw);
    note_launch();
    return check_launch();
}

int v2hist_merge_rows(const void* x, int dtype, int64_t n, int rows, int nb, aq_v2hist_head_t* state,
                      const aq_v2hist_head_t* batch, int64_t block_stride, int state_has_stats, void* scratch,
                      float* updates, cudaStream_t st)
{
    if (rows < 1 || rows > 65535)
        return AQ_ERR_TOO_LARGE;
    const V2HRows rw {rows > 1 ? n : 0, rows > 1 ? v2hist_scratch_bytes() : 0, rows > 1 ? block_stride : 0,
                      rows > 1 ? (int64_t) nb : 0};
    if (!state_has_stats)
    {
        // merge_stats on an empty observer adopts the batch's statistics as they are
        launch_pdl(v2h_copy_kernel, dim3(1, (unsigned) rows), kV2HistThreads, 0, st, batch, nb, state, rw);
        note_launch();
        return check_launch();
    }
    V2HistScratch* sc = static_cast<V2HistScratch*>(scratch);
    int rc            = v2h_passes_any(x, dtype, n, rows, nb, 1, state, batch, sc, rw, st);
    if (rc != AQ_OK)
        return rc;
    launch_pdl(v2h_merge_kernel, dim3(1, (unsigned) rows), kV2HistThreads, 0, st, (const V2HistScratch*) sc, nb, state,
               updates, rw, 0);
    note_launch();
    return check_launch();
}

// collect_stats + merge_stats of one batch in two passes over the data instead of three: finite min / max, then ONE
// counting pass that fills the batch's own histogram and the histogram over the widened range.
int v2hist_update_rows(const void* x, int dtype, int64_t n, int rows, int nb, aq_v2hist_head_t* state,
                       aq_v2hist_head_t* batch, int64_t block_stride, int state_has_stats, void* scratch,
                       float* updates, cudaStream_t st)
{
    if (!state_has_stats)
    {
        int rc = v2hist_collect_rows(x, dtype, n, rows, nb, batch, block_stride, scratch, st);
        if (rc != AQ_OK)
            return rc;
        return v2hist_merge_rows(x, dtype, n, rows, nb, state, batch, block_stride, 0, scratch, updates, st);
    }
    if (rows < 1 || rows > 65535)
        return AQ_ERR_TOO_LARGE;
    V2HistScratch* sc = static_cast<V2HistScratch*>(scratch);
    const V2HRows rw {rows > 1 ? n : 0, rows > 1 ? v2hist_scratch_bytes() : 0, rows > 1 ? block_stride : 0,
                      rows > 1 ? (int64_t) nb : 0};
    int rc = v2h_passes_any(x, dtype, n, rows, nb, 2, state, nullptr, sc, rw, st);
    if (rc != AQ_OK)
        return rc;
    launch_pdl(v2h_finish_update_kernel, dim3(1, (unsigned) rows), kV2HistThreads, 0, st, (const V2HistScratch*) sc, nb,
               batch, state, updates, rw);
    note_launch();
    return check_launch();
}

int v2hist_collect(const void* x, int dtype, int64_t n, int nb, aq_v2hist_head_t* batch, void* scratch, cudaStream_t st)
{
    return v2hist_collect_rows(x, dtype, n, 1, nb, batch, 0, scratch, st);
}

int v2hist_merge(const void* x, int dtype, int64_t n, int nb, aq_v2hist_head_t* state, const aq_v2hist_head_t* batch,
                 int state_has_stats, void* scratch, float* updates, cudaStream_t st)
{
    return v2hist_merge_rows(x, dtype, n, 1, nb, state, batch, 0, state_has_stats, scratch, updates, st);
}

// =================================================================================================
// The same statistics with the batches of one calibration spread over several workers (one per GPU).
//
// merge_stats is sequential: batch b is counted over the range that batches 0..b cover together, and the old counts
// are re-binned, with rounding, each time that range grows (encoding_analyzer.py:223-262).  To get the sequential
// result bit for bit from workers that each hold a share of the batches:
//   1. every worker takes the finite min / max of each of its batches (one pass)        -> aq_v2hist_range_rows
//      and the workers exchange those few words;
//   2. every worker derives, for every batch, the range it has to be counted over        -> aq_v2hist_plan_batches
//      (a sequential scan in batch order with Python's min / max tie rules);
//   3. every worker counts its own batches over their ranges (second pass)              -> aq_v2hist_count_rows
//      and the workers exchange the integer counts (bins + 2 words per batch);
//   4. every worker replays collect_stats / merge_stats in batch order from the counts  -> aq_v2hist_replay_batches
//      -- the float additions and the re-binning happen in the reference's order.
// A range record is 4 words: min and max (float bits), "has a finite value", "present".  A record of zeros is a batch
// that does not exist (workers with fewer batches than others), so that records and counts can be exchanged by an
// integer sum over buffers in which every worker fills only its own rows.
// A plan is 8 floats: lo, hi (the range to count over), batch min, batch max, any_finite, first, present, pad.
// =================================================================================================
__global__ void __launch_bounds__(kV2HistThreads) v2h_range_kernel(const V2HistScratch* __restrict__ sc, int nparts,
                                                                   int32_t* __restrict__ range, V2HRows rw)
{
    pdl_launch_dependents();
    pdl_wait();
    sc = v2h_row(sc, rw.sc_stride);
    range += (int64_t) blockIdx.y * 4;
    float mn = INFINITY, mx = -INFINITY;
    for (int i = threadIdx.x; i < nparts; i += kV2HistThreads)
    {
        mn = fminf(mn, sc->partials[i].x);
        mx = fmaxf(mx, sc->partials[i].y);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
    {
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    __shared__ float s_mn[kV2HistThreads / 32], s_mx[kV2HistThreads / 32];
    if ((threadIdx.x & 31) == 0)
        s_mn[threadIdx.x >> 5] = mn, s_mx[threadIdx.x >> 5] = mx;
    __syncthreads();
    if (threadIdx.x != 0)
        return;
    for (int w = 1; w < kV2HistThreads / 32; ++w)
        mn = fminf(mn, s_mn[w]), mx = fmaxf(mx, s_mx[w]);
    const bool any = mn <= mx;
    range[0] = __float_as_int(any ? mn : 0.0f);
    range[1] = __float_as_int(any ? mx : 0.0f);
    range[2] = any ? 1 : 0;
    range[3] = 1;
}

// One CTA per histogram walks the batches in order: the records of a stretch of batches are staged in shared memory
// by all threads, one thread scans them (the scan is a chain of a few compares per batch), all threads write the plans.
constexpr int kV2HistPlanChunk = 512;
__global__ void __launch_bounds__(kV2HistThreads) v2h_plan_batches_kernel(const int32_t* __restrict__ ranges, int n_batches,
                                                                          int rows, int nb, float* __restrict__ plans)
{
    pdl_launch_dependents();
    pdl_wait();
    __shared__ int32_t s_rg[kV2HistPlanChunk * 4];
    __shared__ float s_pl[kV2HistPlanChunk * 8];
    const int r = blockIdx.y;
    bool have = false;   // thread 0's scan state, carried from chunk to chunk
    float smin = 0.0f, smax = 0.0f;
    for (int b0 = 0; b0 < n_batches; b0 += kV2HistPlanChunk)
    {
        const int m = n_batches - b0 < kV2HistPlanChunk ? n_batches - b0 : kV2HistPlanChunk;
        for (int i = threadIdx.x; i < m * 4; i += kV2HistThreads)
            s_rg[i] = ranges[((int64_t) (b0 + (i >> 2)) * rows + r) * 4 + (i & 3)];
        __syncthreads();
        if (threadIdx.x == 0)
        {
            for (int k = 0; k < m; ++k)
            {
                const int32_t* rg  = s_rg + k * 4;
                float* pl          = s_pl + k * 8;
                const bool present = rg[3] != 0, any = rg[2] != 0;
                const float mn = __int_as_float(rg[0]), mx = __int_as_float(rg[1]);
                float lo = 0.0f, hi = 1.0f;
                bool first = false;
                if (present && any)
                {
                    if (!have)
                    {
                        // collect_stats: first and last edge of _create_bin_edges(min, max)
                        float a0 = mn, b1 = mx;
                        if (a0 == b1)
                            a0 = __fsub_rn(a0, 0.5f), b1 = __fadd_rn(b1, 0.5f);
                        const float step = __fdiv_rn(__fsub_rn(b1, a0), (float) nb);
                        lo               = __fadd_rn(__fmul_rn(0.0f, step), a0);
                        hi               = __fadd_rn(__fmul_rn((float) nb, step), a0);
                        smin = mn, smax = mx;
                        have = first = true;
                    }
                    else
                    {
                        // Python min(new, cur) / max(new, cur): the second argument wins only when strictly smaller /
                        // larger
                        lo   = (smin < mn) ? smin : mn;
                        hi   = (smax > mx) ? smax : mx;
                        smin = lo, smax = hi;
                    }
                }
                pl[0] = lo, pl[1] = hi, pl[2] = mn, pl[3] = mx;
                pl[4] = any ? 1.0f : 0.0f, pl[5] = first ? 1.0f : 0.0f, pl[6] = present ? 1.0f : 0.0f, pl[7] = 0.0f;
            }
        }
        __syncthreads();
        for (int i = threadIdx.x; i < m * 8; i += kV2HistThreads)
            plans[((int64_t) (b0 + (i >> 3)) * rows + r) * 8 + (i & 7)] = s_pl[i];
        __syncthreads();
    }
}

// One CTA per histogram replays the batches in order.  The running histogram lives in registers (bin i of thread t is
// t + 256 j) and only a change of range goes through shared memory, where one thread re-bins the old counts in the
// reference's order; a batch inside the current range costs one coalesced read of its counts and one addition per bin,
// with no barrier.  Bin edges are written once, at the end (they follow from min / max alone).
constexpr int kV2HistPerThread   = (AQ_V2HIST_MAX_BINS + kV2HistThreads - 1) / kV2HistThreads;
constexpr int kV2HistReplayChunk = 256;   // batches whose plans are staged in shared memory at a time
__global__ void __launch_bounds__(kV2HistThreads) v2h_replay_kernel(const uint32_t* __restrict__ counts,
                                                                    const float* __restrict__ plans, int n_batches, int rows,
                                                                    int nb, aq_v2hist_head_t* __restrict__ state,
                                                                    int64_t st_stride)
{
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float s_hist[AQ_V2HIST_MAX_BINS], s_upd[AQ_V2HIST_MAX_BINS];
    __shared__ float s_plan[kV2HistReplayChunk * 8];
    const int r = blockIdx.y;
    state       = v2h_row(state, st_stride);
    float h[kV2HistPerThread];
    uint32_t nxt[kV2HistPerThread];   // the next batch's counts, fetched while this batch is folded in
    uint32_t nxt_below = 0, nxt_above = 0;
#pragma unroll
    for (int j = 0; j < kV2HistPerThread; ++j)
        h[j] = 0.0f, nxt[j] = 0;
    auto fetch = [&](int b) {
        const uint32_t* cn = counts + ((int64_t) b * rows + r) * (nb + 2);
#pragma unroll
        for (int j = 0; j < kV2HistPerThread; ++j)
        {
            const int i = threadIdx.x + j * kV2HistThreads;
            if (i < nb)
                nxt[j] = cn[i];
        }
        nxt_below = cn[nb], nxt_above = cn[nb + 1];
    };
    float smin = 0.0f, smax = 0.0f;
    int initialized = 0, error = 0;
    fetch(0);
    for (int b = 0; b < n_batches; ++b)
    {
        if (b % kV2HistReplayChunk == 0)
        {
            // the plans of the next stretch of batches, staged by all threads
            __syncthreads();
            const int m = n_batches - b < kV2HistReplayChunk ? n_batches - b : kV2HistReplayChunk;
            for (int i = threadIdx.x; i < m * 8; i += kV2HistThreads)
                s_plan[i] = plans[((int64_t) (b + (i >> 3)) * rows + r) * 8 + (i & 7)];
            __syncthreads();
        }
        const float* pl = s_plan + (b % kV2HistReplayChunk) * 8;
        uint32_t cur[kV2HistPerThread];
#pragma unroll
        for (int j = 0; j < kV2HistPerThread; ++j)
            cur[j] = nxt[j];
        const float below = (float) nxt_below, above = (float) nxt_above;
        if (b + 1 < n_batches)
            fetch(b + 1);
        if (pl[6] == 0.0f)
            continue;
        if (pl[4] == 0.0f)
        {
            error = 1;   // a batch without a finite value: the reference raises ValueError when it meets it
            continue;
        }
        const bool first = pl[5] != 0.0f;
        const float umin = first ? pl[2] : pl[0], umax = first ? pl[3] : pl[1];
        if (first)
            initialized = 1;
        else if (!(umin == smin && umax == smax))
        {
            // block-uniform: the range grows
#pragma unroll
            for (int j = 0; j < kV2HistPerThread; ++j)
            {
                const int i = threadIdx.x + j * kV2HistThreads;
                if (i < nb)
                    s_hist[i] = h[j], s_upd[i] = 0.0f;
            }
            __syncthreads();
            if (threadIdx.x == 0)
                v2h_rebin_serial(s_hist, s_upd, smin, smax, umin, umax, nb);
            __syncthreads();
#pragma unroll
            for (int j = 0; j < kV2HistPerThread; ++j)
            {
                const int i = threadIdx.x + j * kV2HistThreads;
                if (i < nb)
                    h[j] = s_upd[i];
            }
        }
        // collect_stats: float(counts), then the elements beyond the edges; merge_stats: float(counts) + re-binned old
        // counts, then the infinities -- the same additions in the same order (the first batch has no old counts)
#pragma unroll
        for (int j = 0; j < kV2HistPerThread; ++j)
        {
            const int i = threadIdx.x + j * kV2HistThreads;
            if (i < nb)
            {
                float v = first ? (float) cur[j] : __fadd_rn((float) cur[j], h[j]);
                if (i == 0)
                    v = __fadd_rn(v, below);
                if (i == nb - 1)
                    v = __fadd_rn(v, above);
                h[j] = v;
            }
        }
        smin = umin, smax = umax;
    }
    float* hist = v2h_hist(state);
#pragma unroll
    for (int j = 0; j < kV2HistPerThread; ++j)
    {
        const int i = threadIdx.x + j * kV2HistThreads;
        if (i < nb)
            hist[i] = h[j];
    }
    v2h_write_edges(smin, smax, nb, v2h_edges(state, nb));
    if (threadIdx.x == 0)
    {
        state->min = smin, state->max = smax;
        state->initialized = initialized;
        state->error       = error;
    }
}

int v2hist_range_rows(const void* x, int dtype, int64_t n, int rows, int32_t* range, void* scratch, cudaStream_t st)
{
    if (rows < 1 || rows > 65535)
        return AQ_ERR_TOO_LARGE;
    V2HistScratch* sc = static_cast<V2HistScratch*>(scratch);
    const V2HRows rw {rows > 1 ? n : 0, rows > 1 ? v2hist_scratch_bytes() : 0, 0, 0};
    int nparts = 0;
    int rc     = v2h_minmax_any(x, dtype, n, rows, sc, rw, &nparts, st);
    if (rc != AQ_OK)
        return rc;
    launch_pdl(v2h_range_kernel, dim3(1, (unsigned) rows), kV2HistThreads, 0, st, (const V2HistScratch*) sc, nparts, range,
               rw);
    note_launch();
    return check_launch();
}

int v2hist_plan_batches(const int32_t* ranges, int n_batches, int rows, int nb, float* plans, cudaStream_t st)
{
    if (n_batches < 1 || rows < 1)
        return AQ_ERR_INVALID_ARG;
    if (rows > 65535)
        return AQ_ERR_TOO_LARGE;
    launch_pdl(v2h_plan_batches_kernel, dim3(1, (unsigned) rows), kV2HistThreads, 0, st, ranges, n_batches, rows, nb,
               plans);
    note_launch();
    return check_launch();
}

int v2hist_count_rows(const void* x, int dtype, int64_t n, int rows, int nb, const float* plan, uint32_t* counts,
                      cudaStream_t st)
{
    if (rows < 1 || rows > 65535)
        return AQ_ERR_TOO_LARGE;
    const V2HRows rw {rows > 1 ? n : 0, 0, 0, 0};
    return v2h_count_any(x, dtype, n, rows, nb, rw, V2HDirect {plan, counts}, st);
}

// The two passes for a list of equally shaped batches (one host call per pass: the launches of consecutive batches
// queue back to back).  Batch i writes record / counts number i * stride of the tables it is given.
int v2hist_range_many(const void* const* xs, int m, int dtype, int64_t n, int rows, int32_t* ranges, int64_t stride_words,
                      void* scratch, cudaStream_t st)
{
    for (int i = 0; i < m; ++i)
    {
        if (!xs[i])
            continue;
        const int rc = v2hist_range_rows(xs[i], dtype, n, rows, ranges + (int64_t) i * stride_words, scratch, st);
        if (rc != AQ_OK)
            return rc;
    }
    return AQ_OK;
}

int v2hist_count_many(const void* const* xs, int m, int dtype, int64_t n, int rows, int nb, const float* plans,
                      int64_t plan_stride, uint32_t* counts, int64_t count_stride, cudaStream_t st)
{
    for (int i = 0; i < m; ++i)
    {
        if (!xs[i])
            continue;
        const int rc = v2hist_count_rows(xs[i], dtype, n, rows, nb, plans + (int64_t) i * plan_stride,
                                         counts + (int64_t) i * count_stride, st);
        if (rc != AQ_OK)
            return rc;
    }
    return AQ_OK;
}

int v2hist_replay_batches(const uint32_t* counts, const float* plans, int n_batches, int rows, int nb,
                          aq_v2hist_head_t* states, int64_t block_stride, cudaStream_t st)
{
    if (rows < 1 || rows > 65535)
        return AQ_ERR_TOO_LARGE;
    if (n_batches < 1)
        return AQ_ERR_INVALID_ARG;
    launch_pdl(v2h_replay_kernel, dim3(1, (unsigned) rows), kV2HistThreads, 0, st, counts, plans, n_batches, rows, nb,
               states, rows > 1 ? block_stride : (int64_t) 0);
    note_launch();
    return check_launch();
}

// =================================================================================================
// SQNR search (SqnrEncodingAnalyzer.compute_encodings_from_stats for one histogram)
// =================================================================================================
constexpr int kSqnrWarps = 4;

struct SqnrArgs
{
    const aq_v2hist_head_t* stats;
    int nb;
    float num_steps;        // float32(num_steps)
    float min_gap;          // float32(eps * num_steps)
    int symmetric;
    int num_deltas;
    int num_offsets;        // entries of `offsets` (asymmetric: the fixed grid; the observed offset is appended)
    const float* offsets;   // device; symmetric: one entry, (-num_steps) // 2
    float gamma;
    float* noise;           // [candidates] workspace
    unsigned int* ticket;   // workspace, zero on entry, left zero
    float* out;             // {min, max}
    int64_t st_stride;      // bytes between the statistics blocks of consecutive histograms (blockIdx.y)
    int64_t ws_stride;      // bytes between their workspaces; results are out_width floats apart
    int out_width;          // 2: {min, max};  4: {min, max, scale, offset} of a quantizer with lower code bound qmin,
    int stats_dtype;        //    min / max first rounded to the statistics dtype as the reference's cast does
    float qmin;
};

__device__ __forceinline__ void sqnr_candidate(const SqnrArgs& a, float min_v, float max_v, int cand, float& delta,
                                               float& offset)
{
    const float ns = a.num_steps;
    if (a.symmetric)
    {
        // _pick_test_candidates_symmetric (:639-652)
        const float m         = fmaxf(max_v, -min_v);
        const float max_delta = __fdiv_rn(__fmul_rn(2.0f, m), ns);
        const float k         = (float) (cand + 1);
        delta                 = fmaxf(__fdiv_rn(__fmul_rn(max_delta, k), (float) (a.num_deltas - 1)), kEps32);
        offset                = a.offsets[0];
        return;
    }
    // _pick_test_candidates_asymmetric (:613-637) + _clamp_delta_offset_values (:654-672)
    const int per_delta   = a.num_offsets + 1;
    const int di          = cand / per_delta;
    const int oi          = cand - di * per_delta;
    const float max_delta = __fdiv_rn(__fsub_rn(max_v, min_v), ns);
    const float obs_off   = rintf(__fdiv_rn(min_v, max_delta));
    const float obs_min   = __fmul_rn(max_delta, obs_off);
    const float obs_max   = __fadd_rn(obs_min, __fmul_rn(max_delta, ns));
    const float td        = __fdiv_rn(__fmul_rn(max_delta, (float) (di + 1)), (float) (a.num_deltas - 1));
    const float to        = oi < a.num_offsets ? a.offsets[oi] : obs_off;
    float t_min           = __fmul_rn(td, to);
    float t_max           = __fadd_rn(t_min, __fmul_rn(td, ns));
    t_min                 = fmaxf(obs_min, t_min);   // torch.max / torch.min: finite operands here
    t_max                 = fminf(obs_max, t_max);
    delta                 = fmaxf(__fdiv_rn(__fsub_rn(t_max, t_min), ns), kEps32);
    offset                = rintf(__fdiv_rn(t_min, delta));
}

__global__ void __launch_bounds__(kSqnrWarps * 32) v2h_sqnr_kernel(SqnrArgs a)
{
    pdl_launch_dependents();
    pdl_wait();
    a.stats  = v2h_row(a.stats, a.st_stride);
    a.ticket = v2h_row(a.ticket, a.ws_stride);
    a.noise  = v2h_row(a.noise, a.ws_stride);
    a.out += a.out_width * (int64_t) blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int per_delta  = a.symmetric ? 1 : a.num_offsets + 1;
    const int candidates = a.num_deltas * per_delta;
    const int cand       = blockIdx.x * kSqnrWarps + warp;
    __shared__ bool s_last;
    const aq_v2hist_head_t* st = a.stats;
    const float* hist  = reinterpret_cast<const float*>(st + 1);
    const float* edges = hist + a.nb;
    // _pick_test_candidates (:602-611)
    float min_v = fminf(st->min, 0.0f);
    float max_v = fmaxf(st->max, 0.0f);
    max_v       = fmaxf(max_v, __fadd_rn(min_v, a.min_gap));
    if (cand < candidates)
    {
        float delta, offset;
        sqnr_candidate(a, min_v, max_v, cand, delta, offset);
        // _estimate_clip_and_quant_noise (:688-725)
        const float hd   = __fsub_rn(edges[1], edges[0]);
        const float mid0 = __fadd_rn(edges[0], __fdiv_rn(hd, 2.0f));
        double sum       = 0.0;
        for (int i = lane; i < a.nb; i += 32)
        {
            const float mid = __fadd_rn(mid0, __fmul_rn(hd, (float) i));
            float q         = rintf(__fsub_rn(__fdiv_rn(mid, delta), offset));
            const bool clip = (q < 0.0f) || (q > a.num_steps);
            if (q == q)   // torch.clamp keeps NaN
                q = fminf(fmaxf(q, 0.0f), a.num_steps);
            const float qdq = __fmul_rn(__fadd_rn(q, offset), delta);
            const float d   = __fsub_rn(qdq, mid);
            float err       = __fmul_rn(__fmul_rn(d, d), hist[i]);
            if (a.gamma != 1.0f && clip)
                err = __fmul_rn(err, a.gamma);
            sum += (double) err;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
            sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (lane == 0)
            a.noise[cand] = (float) sum;
    }
    __syncthreads();
    if (threadIdx.x == 0)
    {
        __threadfence();
        const unsigned int t = atomicAdd(a.ticket, 1u);
        s_last               = (t == gridDim.x - 1);
    }
    __syncthreads();
    if (!s_last || warp != 0)
        return;
    __threadfence();
    // torch.min over the flattened (delta, offset) grid: the first smallest value
    float best = INFINITY;
    int best_i = INT_MAX;
    bool nan   = false;
    for (int i = lane; i < candidates; i += 32)
    {
        const float v = __ldcg(&a.noise[i]);
        if (v != v)
        {
            if (!nan || i < best_i)
                best_i = nan ? min(best_i, i) : i;
            nan = true;
        }
        else if (!nan && (v < best || (v == best && i < best_i)))
        {
            best   = v;
            best_i = i;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
    {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi   = __shfl_xor_sync(0xffffffffu, best_i, o);
        const int on   = __shfl_xor_sync(0xffffffffu, (int) nan, o);
        if (on && (!nan || oi < best_i))
            nan = true, best_i = oi;
        else if (!on && !nan && (ov < best || (ov == best && oi < best_i)))
            best = ov, best_i = oi;
    }
    if (lane == 0)
    {
        float delta = 0.0f, offset = 0.0f;
        if (best_i != INT_MAX)
            sqnr_candidate(a, min_v, max_v, best_i, delta, offset);
        float mn = __fmul_rn(offset, delta);
        float mx = __fadd_rn(mn, __fmul_rn(a.num_steps, delta));
        if (a.out_width == 4)
        {
            // what the quantizer derives from the returned range (affine/quantizer.py:222-246): the range in the
            // statistics dtype, then float32 scale = (max - min) / num_steps and offset = round(min / scale) - qmin
            if (a.stats_dtype == AQ_F16)
                mn = __half2float(__float2half_rn(mn)), mx = __half2float(__float2half_rn(mx));
            else if (a.stats_dtype == AQ_BF16)
                mn = __bfloat162float(__float2bfloat16_rn(mn)), mx = __bfloat162float(__float2bfloat16_rn(mx));
            const float scale = __fdiv_rn(__fsub_rn(mx, mn), a.num_steps);
            a.out[2]          = scale;
            a.out[3]          = a.symmetric ? 0.0f : __fsub_rn(rintf(__fdiv_rn(mn, scale)), a.qmin);
        }
        a.out[0]  = mn;
        a.out[1]  = mx;
        *a.ticket = 0;
    }
}

int64_t v2hist_sqnr_workspace_bytes()
{
    return 256 + 4096 * (int64_t) sizeof(float);
}

int v2hist_sqnr_rows(const aq_v2hist_head_t* stats, int64_t block_stride, int rows, int nb, double num_steps,
                     int symmetric, int num_deltas, const float* offsets, int num_offsets, double gamma, float* out,
                     void* ws, int64_t ws_bytes, cudaStream_t st, int out_width, int stats_dtype, double qmin)
{
    SqnrArgs a;
    a.out_width = out_width, a.stats_dtype = stats_dtype, a.qmin = (float) qmin;
    a.stats = stats, a.nb = nb, a.num_steps = (float) num_steps;
    a.min_gap   = (float) ((double) kEps32 * num_steps);
    a.symmetric = symmetric, a.num_deltas = num_deltas, a.num_offsets = num_offsets, a.offsets = offsets;
    a.gamma     = (float) gamma;
    a.ticket    = static_cast<unsigned int*>(ws);
    a.noise     = reinterpret_cast<float*>(static_cast<char*>(ws) + 256);
    a.out       = out;
    a.st_stride = rows > 1 ? block_stride : 0;
    a.ws_stride = rows > 1 ? v2hist_sqnr_workspace_bytes() : 0;
    const int candidates = num_deltas * (symmetric ? 1 : num_offsets + 1);
    if (rows < 1 || rows > 65535)
        return AQ_ERR_TOO_LARGE;
    if (candidates < 1 || candidates > 4096 || ws_bytes < (int64_t) rows * v2hist_sqnr_workspace_bytes())
        return candidates > 4096 ? AQ_ERR_TOO_LARGE : AQ_ERR_WORKSPACE;
    const int grid = (candidates + kSqnrWarps - 1) / kSqnrWarps;
    launch_pdl(v2h_sqnr_kernel, dim3((unsigned) grid, (unsigned) rows), kSqnrWarps * 32, 0, st, a);
    note_launch();
    return check_launch();
}

int v2hist_sqnr(const aq_v2hist_head_t* stats, int nb, double num_steps, int symmetric, int num_deltas,
                const float* offsets, int num_offsets, double gamma, float* out, void* ws, int64_t ws_bytes,
                cudaStream_t st)
{
    return v2hist_sqnr_rows(stats, 0, 1, nb, num_steps, symmetric, num_deltas, offsets, num_offsets, gamma, out, ws,
                            ws_bytes, st, 2, AQ_F32, 0.0);
}

}   // namespace aq
