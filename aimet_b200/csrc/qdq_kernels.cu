// Fake-quant element kernels for sm_100a: quantize-dequantize / quantize / dequantize forward and the
// straight-through backward, at per-tensor, per-channel and blockwise granularity.
//
// All kernels are HBM-bound streaming kernels: one CTA owns one contiguous chunk of
// THREADS * VEC * UNROLL elements, every thread issues UNROLL independent 16-byte (VEC-wide) loads before
// it computes, and the per-channel / per-block encodings of the chunk are staged once in shared memory.
//
// Results must match the CPU reference bit for bit, and the reference divides (x / scale).  An IEEE division
// costs ~10 instructions, which makes these kernels issue-bound (most of all the 16-bit ones, which carry twice
// the elements per byte), so the hot loop multiplies by the correctly rounded reciprocal instead and *proves*
// per packet that this cannot have changed a rounded integer: product and true quotient differ by at most 3 ulp,
// so they can only round differently when the product lies within a small guard band of a rounding boundary.
// A packet with an element inside the band (about one element in ten thousand for 8-bit grids), or with
// anything non-finite, is recomputed out of line with the reference formula itself.
// The file is compiled with -fmad=false; every fused multiply-add below is explicit.
#include "common.cuh"
#include "kernels.h"

namespace aq
{

constexpr int kThreads = 256;
#ifndef AQ_UNROLL8
#define AQ_UNROLL8 2
#endif
#ifndef AQ_UNROLL4
#define AQ_UNROLL4 4
#endif
#ifndef AQ_UNROLL8_PER_TENSOR
#define AQ_UNROLL8_PER_TENSOR 2
#endif
// 16-byte packets in flight per thread, by packet width in elements (8 = 16-bit types)
template <int VEC>
__host__ __device__ constexpr int unroll_of()
{
    return VEC == 8 ? AQ_UNROLL8 : AQ_UNROLL4;
}
// v2 forward with one encoding for the whole tensor and 16-bit elements: two ADJACENT packets per thread, moved as one
// 32-byte access each way (measured on a [4096,11008] bf16 weight: 29.0 us; one 16-byte packet per thread 31.3 us; two
// interleaved 16-byte packets per thread 34.1 us).
template <int VEC, int PER_CH>
__host__ __device__ constexpr int v2_unroll()
{
    return (VEC == 8 && PER_CH == 0) ? AQ_UNROLL8_PER_TENSOR : unroll_of<VEC>();
}
constexpr int kMaxRuns = 1026;   // chunk / inner + 2 with VEC | inner  (see make_geom)

template <int VEC>
__host__ __device__ constexpr int chunk_elems()
{
    return kThreads * VEC * unroll_of<VEC>();
}

constexpr float kMagicRne = 12582912.0f;               // 1.5 * 2^23: (t + M) - M == rint(t) for |t| < 2^22
constexpr float kTwo23f   = 8388608.0f;
constexpr float kUlp24    = 5.9604644775390625e-08f;   // 2^-24

// -------------------------------------------------------------------------------------------------
// Run bookkeeping shared by the per-channel kernels
// -------------------------------------------------------------------------------------------------
struct RunCtx
{
    int64_t r0;     // index of the first run met by this CTA
    int64_t loc0;   // offset of the CTA's first element inside run r0
    int nruns;      // runs met by this CTA
    int64_t ch0;    // channel of run r0
};

// Integer divisions below run once per CTA but in every thread; tensors below 2^32 elements replace them by one
// multiply-high each (a 64-bit division costs about as many instructions as a thread's whole element work).
template <int VEC>
__device__ __forceinline__ RunCtx make_run_ctx(const ChanGeom& g, int64_t base, int64_t n)
{
    RunCtx c;
    if (g.small)
        c.r0 = (int64_t) div_m64((uint32_t) base, g.inner_m64);
    else
        c.r0 = base / g.inner;
    c.loc0            = base - c.r0 * g.inner;
    int64_t remaining = n - base;
    int64_t span      = remaining < (int64_t) chunk_elems<VEC>() ? remaining : (int64_t) chunk_elems<VEC>();
    if (g.mode == 2)
        c.nruns = (c.loc0 + span - 1 >= g.inner) ? 2 : 1;
    else
        c.nruns = (int) local_run(g, (uint32_t) (c.loc0 + span - 1)) + 1;
    if (g.small)
        c.ch0 = (int64_t) ((uint32_t) c.r0 - div_m64((uint32_t) c.r0, g.ch_m64) * (uint32_t) g.num_ch);
    else
        c.ch0 = c.r0 % g.num_ch;
    return c;
}

// Channel of the lr-th run met by the CTA (lr < kMaxRuns).
__device__ __forceinline__ int64_t run_channel(const ChanGeom& g, const RunCtx& c, int lr)
{
    int64_t ch = c.ch0 + lr;
    if (ch >= g.num_ch)
    {
        ch -= g.num_ch;
        if (ch >= g.num_ch)
            ch = ((uint64_t) ch <= 0xffffffffull) ? (int64_t) ((uint32_t) ch % (uint32_t) g.num_ch) : ch % g.num_ch;
    }
    return ch;
}

__device__ __forceinline__ uint32_t run_of(const ChanGeom& g, const RunCtx& c, uint32_t off)
{
    // branch-free; mode 2 compares in 64 bits because inner may exceed 2^32 there
    const uint32_t loc        = (uint32_t) c.loc0 + off;
    const uint32_t by_compare = (c.loc0 + (int64_t) off >= g.inner) ? 1u : 0u;
    return g.mode == 1 ? __umulhi(loc, g.magic) : (g.mode == 2 ? by_compare : loc);
}

template <>
__device__ __forceinline__ uint8_t from_f32<uint8_t>(float v)   // padding value of partial mask packets
{
    return (uint8_t) v;
}

template <typename T>
__device__ __forceinline__ float narrow(float v)
{
    return to_f32<T>(from_f32<T>(v));
}

// -------------------------------------------------------------------------------------------------
// Packet <-> fp32 conversion (pairs of 16-bit values convert with one instruction)
// -------------------------------------------------------------------------------------------------
template <typename T, int VEC>
__device__ __forceinline__ void unpack(const Pack<T, VEC>& p, float (&f)[VEC])
{
#pragma unroll
    for (int e = 0; e < VEC; ++e)
        f[e] = to_f32<T>(p.v[e]);
}
template <typename T, int VEC>
__device__ __forceinline__ void repack(const float (&f)[VEC], Pack<T, VEC>& p)
{
#pragma unroll
    for (int e = 0; e < VEC; ++e)
        p.v[e] = from_f32<T>(f[e]);
}
#define AQ_PAIRWISE(T, T2, TO2, FROM2)                                                                               \
    template <>                                                                                                      \
    __device__ __forceinline__ void unpack<T, 8>(const Pack<T, 8>& p, float(&f)[8])                                  \
    {                                                                                                                \
        const T2* q = reinterpret_cast<const T2*>(&p);                                                               \
        for (int e = 0; e < 4; ++e)                                                                                  \
        {                                                                                                            \
            const float2 v = TO2(q[e]);                                                                              \
            f[2 * e] = v.x, f[2 * e + 1] = v.y;                                                                      \
        }                                                                                                            \
    }                                                                                                                \
    template <>                                                                                                      \
    __device__ __forceinline__ void repack<T, 8>(const float(&f)[8], Pack<T, 8>& p)                                  \
    {                                                                                                                \
        T2* q = reinterpret_cast<T2*>(&p);                                                                           \
        for (int e = 0; e < 4; ++e)                                                                                  \
            q[e] = FROM2(f[2 * e], f[2 * e + 1]);                                                                    \
    }                                                                                                                \
    template <>                                                                                                      \
    __device__ __forceinline__ void unpack<T, 4>(const Pack<T, 4>& p, float(&f)[4])                                  \
    {                                                                                                                \
        const T2* q = reinterpret_cast<const T2*>(&p);                                                               \
        for (int e = 0; e < 2; ++e)                                                                                  \
        {                                                                                                            \
            const float2 v = TO2(q[e]);                                                                              \
            f[2 * e] = v.x, f[2 * e + 1] = v.y;                                                                      \
        }                                                                                                            \
    }                                                                                                                \
    template <>                                                                                                      \
    __device__ __forceinline__ void repack<T, 4>(const float(&f)[4], Pack<T, 4>& p)                                  \
    {                                                                                                                \
        T2* q = reinterpret_cast<T2*>(&p);                                                                           \
        for (int e = 0; e < 2; ++e)                                                                                  \
            q[e] = FROM2(f[2 * e], f[2 * e + 1]);                                                                    \
    }
AQ_PAIRWISE(__half, __half2, __half22float2, __floats2half2_rn)
AQ_PAIRWISE(__nv_bfloat16, __nv_bfloat162, __bfloat1622float2, __floats2bfloat162_rn)
#undef AQ_PAIRWISE

__device__ __forceinline__ float clamp_keep_nan(float r, float lo, float hi)
{
    // torch.clamp keeps NaN: min.NaN / max.NaN
    float q;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(q) : "f"(r), "f"(lo));
    asm("min.NaN.f32 %0, %1, %2;" : "=f"(q) : "f"(q), "f"(hi));
    return q;
}

// max(a, |b|, |c|), NaN if any operand is NaN
__device__ __forceinline__ float max3_abs_nan(float a, float b, float c)
{
    float r;
    asm("max.NaN.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(fabsf(b)), "f"(fabsf(c)));
    return r;
}

// =================================================================================================
// Chunk load / store
// =================================================================================================
// Offset of a thread's u-th packet inside the CTA's chunk.  Interleaved: packet u of all threads is one contiguous
// stretch.  Adjacent (ADJ): a thread's packets follow one another, so that they share an encoding when the run
// length is a multiple of U * VEC.
template <int VEC, int U, bool ADJ>
__device__ __forceinline__ uint32_t packet_offset(int u)
{
    return ADJ ? (uint32_t) (threadIdx.x * U + u) * VEC : (uint32_t) (u * kThreads + threadIdx.x) * VEC;
}

template <typename T, int VEC, int U, bool ADJ = false>
__device__ __forceinline__ void load_chunk(const T* __restrict__ x, int64_t base, int64_t n, Pack<T, VEC> (&v)[U],
                                           bool (&full)[U])
{
#pragma unroll
    for (int u = 0; u < U; ++u)
    {
        const int64_t idx = base + (int64_t) packet_offset<VEC, U, ADJ>(u);
        full[u]           = idx + VEC <= n;
        if (full[u])
            v[u] = load_pack<T, VEC>(x + idx);
        else
        {
#pragma unroll
            for (int e = 0; e < VEC; ++e)
                v[u].v[e] = (idx + e < n) ? x[idx + e] : from_f32<T>(0.0f);
        }
    }
}

template <typename T, int VEC>
__device__ __forceinline__ void store_packet(T* __restrict__ y, int64_t idx, int64_t n, const Pack<T, VEC>& v, bool full)
{
    if (full)
        store_pack<T, VEC>(y + idx, v);
    else
    {
#pragma unroll
        for (int e = 0; e < VEC; ++e)
            if (idx + e < n)
                y[idx + e] = v.v[e];
    }
}

// Two adjacent 16-byte packets of one thread as ONE 32-byte access (sm_100 ld / st.global.v8.b32): with the adjacent
// layout a warp's 16-byte accesses cover every 32-byte sector only half, two instructions per sector; the wide form
// touches whole sectors once.  The address must be 32-byte aligned.
template <typename T, int VEC>
__device__ __forceinline__ void load_pack_pair(const T* p, Pack<T, VEC>& a, Pack<T, VEC>& b)
{
    static_assert(sizeof(Pack<T, VEC>) == 16, "16-byte packets only");
    uint32_t* ra = reinterpret_cast<uint32_t*>(&a);
    uint32_t* rb = reinterpret_cast<uint32_t*>(&b);
    asm volatile("ld.global.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(ra[0]), "=r"(ra[1]), "=r"(ra[2]), "=r"(ra[3]), "=r"(rb[0]), "=r"(rb[1]), "=r"(rb[2]), "=r"(rb[3])
                 : "l"(p));
}
template <typename T, int VEC>
__device__ __forceinline__ void store_pack_pair(T* p, const Pack<T, VEC>& a, const Pack<T, VEC>& b)
{
    static_assert(sizeof(Pack<T, VEC>) == 16, "16-byte packets only");
    const uint32_t* ra = reinterpret_cast<const uint32_t*>(&a);
    const uint32_t* rb = reinterpret_cast<const uint32_t*>(&b);
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(ra[0]), "r"(ra[1]), "r"(ra[2]),
                 "r"(ra[3]), "r"(rb[0]), "r"(rb[1]), "r"(rb[2]), "r"(rb[3])
                 : "memory");
}

// =================================================================================================
// libpymo semantics: quantizeValueCpu + dequantizeValueCpu (DlQuantization/src/trim_functions.cpp:140-171)
//   t = fmax(fmin(x, max), min);  u = t / delta - offset;  q = roundf(u);  y = delta * (q + offset)
// =================================================================================================
struct PymoSlot
{
    float mn, mx, dl, of;
    float rdl;    // RN(1 / delta)
    float c;      // 1.5 - offset
    float eps;    // 0.5 - guard band, or 0 when the reciprocal form cannot be trusted for this grid
};

struct PymoArgs
{
    const float* in;
    float* out;
    int64_t n;
    // per-tensor (host-derived grid, narrowed to float like the reference does at the call boundary)
    float mn, mx, delta, offset;
    // per-channel
    const float* enc_min;      // raw min/max (derive = 1) or gated min/max (derive = 0)
    const float* enc_max;
    const float* enc_delta;    // derive = 0 only
    const float* enc_offset;   // derive = 0 only
    float num_steps;
    int derive;
    float shift;   // subtracted from codes (quantize only)
    ChanGeom geom;
};

// Fast form: s = t * RN(1/delta) + (1.5 - offset) approximates u + 1.5 (one FMA); floor(s) is read from the
// mantissa after a round-down add of 2^23, so q = floor(u + 0.5) = roundf(u) for u > -0.5.
// |s - (u + 1.5)| <= 2^-24 (2|t/delta| + |c| + |s| + |u|) <= 2^-24 (3|of| + 4 umax + 6): that is the guard band.
__device__ __forceinline__ void pymo_finish(PymoSlot& k)
{
    k.rdl = __frcp_rn(k.dl);
    k.c   = 1.5f - k.of;
    const float ulo    = __fsub_rn(__fdiv_rn(k.mn, k.dl), k.of);   // smallest / largest u the clamp lets through
    const float uhi    = __fsub_rn(__fdiv_rn(k.mx, k.dl), k.of);
    const float umax   = fmaxf(fabsf(ulo), fabsf(uhi));
    const float margin = 1.25f * kUlp24 * (3.0f * fabsf(k.of) + 4.0f * umax + 6.0f);
    const bool sane    = (ulo > -1.0f) && (umax < 4194304.0f) && (margin < 0.25f) && (fabsf(k.of) < 4194304.0f);
    k.eps              = sane ? 0.5f - margin : 0.0f;   // any NaN makes `sane` false
}

__device__ __forceinline__ PymoSlot pymo_load(const PymoArgs& a, int64_t ch)
{
    PymoSlot k;
    k.mn = a.enc_min[ch], k.mx = a.enc_max[ch];
    if (a.derive)
    {
        // AimetTensorQuantizer.cpp:236-254: gate, delta, offset in fp32 (offset: half to even)
        k.mn     = k.mn < 0.0f ? k.mn : 0.0f;
        k.mx     = k.mx > 0.0f ? k.mx : 0.0f;
        float lo = __fadd_rn(k.mn, 1e-5f);
        k.mx     = k.mx > lo ? k.mx : lo;
        k.dl     = __fdiv_rn(__fsub_rn(k.mx, k.mn), a.num_steps);
        k.of     = rintf(__fdiv_rn(k.mn, k.dl));
    }
    else
    {
        k.dl = a.enc_delta[ch];
        k.of = a.enc_offset[ch];
    }
    pymo_finish(k);
    return k;
}

template <int VEC, bool CODES>
__device__ __forceinline__ void pymo_exact_packet(const Pack<float, VEC>& in, Pack<float, VEC>& out, PymoSlot k, float shift)
{
#pragma unroll
    for (int e = 0; e < VEC; ++e)
    {
        const float t = fmaxf(fminf(in.v[e], k.mx), k.mn);
        const float q = round_half_away(__fsub_rn(__fdiv_rn(t, k.dl), k.of));
        out.v[e]      = CODES ? __fsub_rn(q, shift) : __fmul_rn(k.dl, __fadd_rn(q, k.of));
    }
}

template <int VEC, bool PER_CH, bool CODES>
__global__ void __launch_bounds__(kThreads) pymo_qdq_kernel(PymoArgs a)
{
    pdl_launch_dependents();
    pdl_wait();
    constexpr int CHUNK = chunk_elems<VEC>();
    const int64_t base  = (int64_t) blockIdx.x * CHUNK;
    __shared__ PymoSlot s_slot[PER_CH ? kMaxRuns : 1];
    RunCtx rc {0, 0, 1, 0};
    PymoSlot k0;
    // the element loads go out first; the encodings are staged while they are in flight
    Pack<float, VEC> v[unroll_of<VEC>()];
    bool full[unroll_of<VEC>()];
    load_chunk<float, VEC, unroll_of<VEC>()>(a.in, base, a.n, v, full);
    if (PER_CH)
    {
        rc = make_run_ctx<VEC>(a.geom, base, a.n);
        for (int lr = threadIdx.x; lr < rc.nruns; lr += kThreads)
            s_slot[lr] = pymo_load(a, run_channel(a.geom, rc, lr));
        __syncthreads();
    }
    else
    {
        k0.mn = a.mn, k0.mx = a.mx, k0.dl = a.delta, k0.of = a.offset;
        pymo_finish(k0);
    }
    const float shift = a.shift;
#pragma unroll
    for (int u = 0; u < unroll_of<VEC>(); ++u)
    {
        const uint32_t off = (uint32_t) (u * kThreads + threadIdx.x) * VEC;
        PymoSlot k         = k0;
        if (PER_CH)
            k = s_slot[run_of(a.geom, rc, off)];   // VEC | inner: one run per packet
        Pack<float, VEC> r;
        bool ok = true;
#pragma unroll
        for (int e = 0; e < VEC; ++e)
        {
            const float t  = fmaxf(fminf(v[u].v[e], k.mx), k.mn);
            const float s  = fmaf(t, k.rdl, k.c);
            const float s2 = __fadd_rd(s, kTwo23f);
            const float g  = s - (s2 - 8388607.5f);
            ok             = ok && (fabsf(g) < k.eps);
            const float q  = s2 - 8388609.0f;   // floor(s) - 1
            r.v[e]         = CODES ? __fsub_rn(q, shift) : __fmul_rn(k.dl, __fadd_rn(q, k.of));
        }
        if (!ok)
            pymo_exact_packet<VEC, CODES>(v[u], r, k, shift);
        store_packet<float, VEC>(a.out, base + off, a.n, r, full[u]);
    }
}

template <bool PER_CH>
static int launch_pymo(PymoArgs a, int vec, bool codes, cudaStream_t st)
{
    if (a.n == 0)
        return AQ_OK;
#define AQ_LAUNCH(V)                                                                                                 \
    {                                                                                                                \
        a.geom       = make_geom(a.geom.num_ch, a.geom.inner, chunk_elems<V>(), a.n);                                     \
        int64_t grid = (a.n + chunk_elems<V>() - 1) / chunk_elems<V>();                                              \
        if (codes)                                                                                                   \
            launch_pdl(pymo_qdq_kernel<V, PER_CH, true>, (unsigned) grid, kThreads, 0, st, a);                                 \
        else                                                                                                         \
            launch_pdl(pymo_qdq_kernel<V, PER_CH, false>, (unsigned) grid, kThreads, 0, st, a);                                \
    }
    switch (vec)
    {
    case 4: AQ_LAUNCH(4) break;
    case 2: AQ_LAUNCH(2) break;
    default: AQ_LAUNCH(1) break;
    }
#undef AQ_LAUNCH
    note_launch();
    return check_launch();
}

int pymo_per_tensor(const float* in, float* out, int64_t n, float mn, float mx, float delta, float offset,
                    int codes_only, float shift, cudaStream_t st)
{
    PymoArgs a {};
    a.in = in, a.out = out, a.n = n;
    a.mn = mn, a.mx = mx, a.delta = delta, a.offset = offset;
    a.shift       = shift;
    a.geom.num_ch = 1, a.geom.inner = n > 0 ? n : 1;
    return launch_pymo<false>(a, pick_vec<float>(in, out, nullptr, 0), codes_only != 0, st);
}

int pymo_per_channel(const float* in, float* out, int64_t n, int64_t num_ch, int64_t inner, const float* enc_min,
                     const float* enc_max, const float* enc_delta, const float* enc_offset, float num_steps,
                     int derive, cudaStream_t st)
{
    PymoArgs a {};
    a.in = in, a.out = out, a.n = n;
    a.enc_min = enc_min, a.enc_max = enc_max, a.enc_delta = enc_delta, a.enc_offset = enc_offset;
    a.num_steps = num_steps, a.derive = derive;
    a.geom.num_ch = num_ch, a.geom.inner = inner;
    return launch_pymo<true>(a, pick_vec<float>(in, out, nullptr, inner), false, st);
}

// -------------------------------------------------------------------------------------------------
// General broadcast QDQ (stride walk), libpymo semantics.  Rarely-used fallback for encodings that do not
// reduce to (i / inner) % num_ch; one element per thread per step, exact division.
// -------------------------------------------------------------------------------------------------
// Encodings whose layout does not reduce to channel = (i / inner) % num_ch (broadcast dimensions between encoded
// ones).  A thread takes VEC consecutive elements with one 16-byte load and store; the encoding index of each comes
// from a per-dimension decomposition of its flat index -- for tensors below 2^32 elements with multiply-high by
// precomputed magic numbers (a 64-bit division costs as many instructions as everything else here together).
template <int VEC, bool SMALL>
__global__ void __launch_bounds__(kThreads) pymo_broadcast_kernel(BroadcastArgs a)
{
    pdl_launch_dependents();
    pdl_wait();
    const int64_t first = ((int64_t) blockIdx.x * kThreads + threadIdx.x) * VEC;
    if (first >= a.n)
        return;
    const bool full = first + VEC <= a.n;
    Pack<float, VEC> v, r;
    if (full)
        v = load_pack<float, VEC>(a.in + first);
    else
    {
#pragma unroll
        for (int e = 0; e < VEC; ++e)
            v.v[e] = first + e < a.n ? a.in[first + e] : 0.0f;
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e)
    {
        int64_t enc = 0;
        if (SMALL)
        {
            uint32_t rem = (uint32_t) (first + e);
#pragma unroll
            for (int d = 0; d < 8; ++d)
                if (d < a.ndims)
                {
                    const uint32_t k = div_m64(rem, a.in_m64[d]);
                    rem -= k * (uint32_t) a.in_strides[d];
                    enc += a.enc_strides[d] * (int64_t) k;
                }
        }
        else
        {
            int64_t rem = first + e;
            for (int d = 0; d < a.ndims; ++d)
            {
                const int64_t k = rem / a.in_strides[d];
                rem -= k * a.in_strides[d];
                enc += a.enc_strides[d] * k;
            }
        }
        if (!full && first + e >= a.n)
            enc = 0;
        const float dl = __ldg(a.dl + enc), of = __ldg(a.of + enc);
        const float t  = fmaxf(fminf(v.v[e], __ldg(a.mx + enc)), __ldg(a.mn + enc));
        const float q  = round_half_away(__fsub_rn(__fdiv_rn(t, dl), of));
        r.v[e]         = __fmul_rn(dl, __fadd_rn(q, of));
    }
    if (full)
        store_pack<float, VEC>(a.out + first, r);
    else
    {
#pragma unroll
        for (int e = 0; e < VEC; ++e)
            if (first + e < a.n)
                a.out[first + e] = r.v[e];
    }
}

int pymo_broadcast(const BroadcastArgs& a, cudaStream_t st)
{
    if (a.n == 0)
        return AQ_OK;
    const bool small = (uint64_t) a.n <= 0xffffffffull;
    const int vec    = pick_vec<float>(a.in, a.out, nullptr, 0) >= 4 ? 4 : 1;
    const int64_t blocks = (a.n + (int64_t) kThreads * vec - 1) / ((int64_t) kThreads * vec);
#define AQ_BC(V, S) launch_pdl(pymo_broadcast_kernel<V, S>, (unsigned) blocks, kThreads, 0, st, a)
    if (vec == 4)
        small ? AQ_BC(4, true) : AQ_BC(4, false);
    else
        small ? AQ_BC(1, true) : AQ_BC(1, false);
#undef AQ_BC
    note_launch();
    return check_launch();
}

// =================================================================================================
// v2 semantics: torch_builtins.py:303-313 (QuantDequantFunc / QuantizeFunc) and :264-266 (DequantizeFunc)
//   r = round_half_even(x / s) - o;  mask = qmin <= r <= qmax;  q = clamp(r, qmin, qmax);  y = (q + o) * s
// =================================================================================================
struct V2Slot
{
    float s, o, rs;
    float eps;   // 0.5 - guard band of the reciprocal form for this encoding
};
constexpr float kBandPerUnit = 2.384185791015625e-07f;   // 2^-22 = 4 ulp of 1.0

// RN(x/s) and RN(x * RN(1/s)) differ by at most 3 ulp of the quotient t, i.e. by less than 2^-22 |t|.  Wherever the
// rounded value can matter (within one step of the clamp range) |t| <= T = max(|qmin + o|, |qmax + o|) + 1, so a
// guard band of 2^-22 T around every half-integer is enough; outside that range both forms clamp to the same bound.
__device__ __forceinline__ V2Slot v2_slot(float s, float o, float qmin, float qmax)
{
    V2Slot k;
    k.s  = s;
    k.o  = o;
    k.rs = __frcp_rn(k.s);
    const float T      = fmaxf(fabsf(__fadd_rn(qmin, k.o)), fabsf(__fadd_rn(qmax, k.o))) + 1.0f;
    const float margin = kBandPerUnit * T;
    // One band for the whole encoding.  (For grids of 2^11 steps or more, e.g. 16-bit activations, a band sized
    // for the largest quotient would send a percent of all elements to the exact path; the kernel is then built
    // with WIDE and takes the band from each element's own quotient instead, 2^-22 (|t| + 1), at the price of two
    // more packed operations per pair, and ignores eps.)
    k.eps = (margin < 0.25f) ? 0.5f - margin : 0.0f;   // NaN -> 0: always the exact path
    return k;
}
__device__ __forceinline__ V2Slot v2_load(const float* scale, const float* offset, int64_t ch, float qmin, float qmax)
{
    return v2_slot(scale[ch], offset[ch], qmin, qmax);
}

// Reference formula for one packet (also the only path when intermediates are kept in the storage dtype).
template <typename T, int VEC, bool NARROW, bool CODES>
__device__ __forceinline__ void v2_exact_packet(const float (&x)[VEC], float (&y)[VEC], uint8_t (&m)[VEC], V2Slot k, float qmin,
                                             float qmax)
{
#pragma unroll
    for (int e = 0; e < VEC; ++e)
    {
        float r = __fdiv_rn(x[e], k.s);
        if (NARROW)
            r = narrow<T>(r);   // fp32 arithmetic + one rounding == the narrow operation (24 >= 2p + 2)
        r = rintf(r);
        r = __fsub_rn(r, k.o);
        if (NARROW)
            r = narrow<T>(r);
        const float q = clamp_keep_nan(r, qmin, qmax);
        m[e]          = (q == r) ? 1 : 0;
        if (CODES)
            y[e] = q;
        else
        {
            float v = __fadd_rn(q, k.o);
            if (NARROW)
                v = narrow<T>(v);
            y[e] = __fmul_rn(v, k.s);
        }
    }
}

// MODE: 0 = fast fp32-internal quantize(-dequantize); 1 = exact / narrow-internal quantize(-dequantize); 2 = dequantize
// PER_CH: 0 = one encoding; 1 = the encodings of the runs met by the CTA are staged in shared memory (few, long
// runs); 2 = every thread fetches the one encoding its adjacent packets share (many short runs per tile, e.g.
// blocks of 64: staging would cost a barrier and a slot per run).
// WIDE (fast mode only): the grid has 2^11 steps or more and the guard band follows each element's quotient.
template <typename T, int VEC, int PER_CH, int MODE, bool NARROW, bool CODES, bool MASK, bool WIDE>
__global__ void __launch_bounds__(kThreads) v2_kernel(V2Args a)
{
    pdl_launch_dependents();
    pdl_wait();
    constexpr int U     = v2_unroll<VEC, PER_CH>();
    constexpr int CHUNK = kThreads * VEC * U;
    const int64_t base  = (int64_t) blockIdx.x * CHUNK;
    const int64_t hi    = a.n;
    const float qmin = a.qmin, qmax = a.qmax;
    __shared__ V2Slot s_slot[PER_CH == 1 ? kMaxRuns : 1];
    RunCtx rc {0, 0, 1, 0};
    V2Slot k0;
    // adjacent packets: blockwise (one encoding per thread) and the 16-bit per-tensor form (for its 32-byte accesses)
    // (the fp32 per-tensor form measured no better with it: 11.0 against 9.9 us for 25.7 MB, equal at 256 MB)
    constexpr bool ADJ = PER_CH == 2 || (PER_CH == 0 && VEC == 8 && U == 2);
    if (!PER_CH)
        k0 = v2_load(a.scale, a.offset, 0, qmin, qmax);
    // per channel: the element loads go out first and the encodings are fetched while they are in flight
    Pack<T, VEC> v[U];
    bool full[U];
    // adjacent layout, two 16-byte packets per thread, both inside the tensor, 32-byte aligned tensors: one 32-byte
    // access each way (the mask, when there is one, keeps its narrower packets)
    constexpr bool kPairable = ADJ && U % 2 == 0 && sizeof(Pack<T, VEC>) == 16;
    bool paired              = false;
    if constexpr (kPairable)
    {
        const int64_t first = base + (int64_t) packet_offset<VEC, U, true>(0);
        paired              = a.wide_ok && first + U * VEC <= hi;
        if (paired)
        {
#pragma unroll
            for (int u = 0; u < U; u += 2)
            {
                load_pack_pair<T, VEC>(static_cast<const T*>(a.x) + first + u * VEC, v[u], v[u + 1]);
                full[u] = full[u + 1] = true;
            }
        }
    }
    if (!paired)
        load_chunk<T, VEC, U, ADJ>(static_cast<const T*>(a.x), base, hi, v, full);
    Pack<T, VEC> held;   // the first packet's result, kept until its neighbour is ready
    if (PER_CH == 1)
    {
        rc = make_run_ctx<VEC>(a.geom, base, hi);
        for (int lr = threadIdx.x; lr < rc.nruns; lr += kThreads)
            s_slot[lr] = v2_load(a.scale, a.offset, run_channel(a.geom, rc, lr), qmin, qmax);
        __syncthreads();
    }
    if (PER_CH == 2)
    {
        // the thread's packets are adjacent and the run length is a multiple of U * VEC: one encoding per thread,
        // fetched straight from global memory (neighbouring lanes read the same words)
        const int64_t first = base + packet_offset<VEC, U, true>(0);
        int64_t ch          = 0;
        if (first < hi)
        {
            if (a.geom.small)
            {
                const uint32_t run = div_m64((uint32_t) first, a.geom.inner_m64);
                ch = a.geom.wraps ? (int64_t) (run - div_m64(run, a.geom.ch_m64) * (uint32_t) a.geom.num_ch) : (int64_t) run;
            }
            else
                ch = (first / a.geom.inner) % a.geom.num_ch;
        }
        k0 = v2_slot(__ldg(a.scale + ch), __ldg(a.offset + ch), qmin, qmax);
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
    {
        const uint32_t off = packet_offset<VEC, U, ADJ>(u);
        const int64_t idx  = base + off;
        V2Slot k           = k0;
        if (PER_CH == 1)
            k = s_slot[run_of(a.geom, rc, off)];
        float x[VEC], y[VEC];
        uint8_t m[VEC];
        unpack<T, VEC>(v[u], x);
        if (MODE == 2)
        {
            // DequantizeFunc: (x + o) * s, in the storage dtype
#pragma unroll
            for (int e = 0; e < VEC; ++e)
            {
                float r = __fadd_rn(x[e], k.o);
                if (NARROW)
                    r = narrow<T>(r);
                y[e] = __fmul_rn(r, k.s);
            }
        }
        else if (MODE == 1)
            v2_exact_packet<T, VEC, NARROW, CODES>(x, y, m, k, qmin, qmax);
        else
        {
            bool ok = true;
            if (VEC == 1)
            {
                const float t = __fmul_rn(x[0], k.rs);
                float r       = __fsub_rn(__fadd_rn(t, kMagicRne), kMagicRne);
                const float d = fabsf(__fsub_rn(t, r));
                ok = !WIDE ? (d < k.eps)   // false for NaN / Inf
                           : (__fadd_rn(d, __fmul_rn(kBandPerUnit, fabsf(t))) < 0.5f - 2.0f * kBandPerUnit);
                r             = __fsub_rn(r, k.o);
                const float q = clamp_keep_nan(r, qmin, qmax);
                if (MASK)
                    m[0] = (q == r) ? 1 : 0;
                y[0] = CODES ? q : __fmul_rn(__fadd_rn(q, k.o), k.s);
            }
            else
            {
                const f32x2_t rs2 = pair(k.rs, k.rs), o2 = pair(k.o, k.o), s2 = pair(k.s, k.s);
                const f32x2_t magic = pair(kMagicRne, kMagicRne);
                constexpr bool per_element = WIDE;
                const f32x2_t band_p = pair(kBandPerUnit, kBandPerUnit), band_n = pair(-kBandPerUnit, -kBandPerUnit);
                float worst = 0.0f;   // largest distance of a product from its rounded value; NaN for NaN / Inf
#pragma unroll
                for (int e = 0; e + 1 < VEC; e += 2)
                {
                    const f32x2_t t = mul2(pair(x[e], x[e + 1]), rs2);
                    f32x2_t r       = sub2(add2(t, magic), magic);
                    float d0, d1, r0, r1;
                    const f32x2_t d = sub2(t, r);
                    if (per_element)
                    {
                        // |d| + 2^-22 |t| = max(|d + 2^-22 t|, |d - 2^-22 t|)
                        float u0, u1, w0, w1;
                        unpair(fma2(t, band_p, d), u0, u1);
                        unpair(fma2(t, band_n, d), w0, w1);
                        worst = max3_abs_nan(max3_abs_nan(worst, u0, u1), w0, w1);
                    }
                    else
                    {
                        unpair(d, d0, d1);
                        worst = max3_abs_nan(worst, d0, d1);
                    }
                    unpair(sub2(r, o2), r0, r1);
                    const float q0 = clamp_keep_nan(r0, qmin, qmax), q1 = clamp_keep_nan(r1, qmin, qmax);
                    if (MASK)
                        m[e] = (q0 == r0) ? 1 : 0, m[e + 1] = (q1 == r1) ? 1 : 0;
                    if (CODES)
                        y[e] = q0, y[e + 1] = q1;
                    else
                        unpair(mul2(add2(pair(q0, q1), o2), s2), y[e], y[e + 1]);
                }
                ok = worst < (per_element ? 0.5f - 2.0f * kBandPerUnit : k.eps);
            }
            if (!ok)
                v2_exact_packet<T, VEC, false, CODES>(x, y, m, k, qmin, qmax);
        }
        Pack<T, VEC> r;
        repack<T, VEC>(y, r);
        bool stored = false;
        if constexpr (kPairable)
        {
            if (paired)
            {
                if ((u & 1) == 0)
                    held = r;
                else
                    store_pack_pair<T, VEC>(static_cast<T*>(a.y) + (idx - VEC), held, r);
                stored = true;
            }
        }
        if (!stored)
            store_packet<T, VEC>(static_cast<T*>(a.y), idx, hi, r, full[u]);
        if (MASK)
        {
            Pack<uint8_t, VEC> mp;
#pragma unroll
            for (int e = 0; e < VEC; ++e)
                mp.v[e] = m[e];
            store_packet<uint8_t, VEC>(a.mask, idx, hi, mp, full[u]);
        }
    }
}

template <typename T, int VEC, int PER_CH>
static void launch_v2_variant(const V2Args& a, bool narrow, cudaStream_t st)
{
    constexpr int64_t chunk = (int64_t) kThreads * VEC * v2_unroll<VEC, PER_CH>();
    const int64_t grid      = (a.n + chunk - 1) / chunk;
    const unsigned g        = (unsigned) grid;
    const bool codes = a.out_kind == AQ_V2_OUT_CODES, mask = a.mask != nullptr;
    const bool wide = (a.qmax - a.qmin) >= 2048.0f;
#define AQ_K(MODE, NARROW, CODES, MASK, WIDE)                                                                        \
    launch_pdl(v2_kernel<T, VEC, PER_CH, MODE, NARROW, CODES, MASK, WIDE>, g, kThreads, 0, st, a)
#define AQ_K0(CODES, MASK) (wide ? AQ_K(0, false, CODES, MASK, true) : AQ_K(0, false, CODES, MASK, false))
    if (a.dequant_only)
    {
        if (narrow)
            AQ_K(2, true, false, false, false);
        else
            AQ_K(2, false, false, false, false);
    }
    else if (narrow)
    {
        if (codes)
            mask ? AQ_K(1, true, true, true, false) : AQ_K(1, true, true, false, false);
        else
            mask ? AQ_K(1, true, false, true, false) : AQ_K(1, true, false, false, false);
    }
    else
    {
        if (codes)
            mask ? AQ_K0(true, true) : AQ_K0(true, false);
        else
            mask ? AQ_K0(false, true) : AQ_K0(false, false);
    }
#undef AQ_K0
#undef AQ_K
}

template <typename T, bool PER_CH>
static int launch_v2_vec(V2Args a, int vec, bool narrow, cudaStream_t st)
{
    // more than 16 runs per tile, each a whole number of thread shares: per-thread encoding loads instead of
    // shared-memory staging (block 64 on a [4096,11008] bf16 weight: 40.9 us per thread, 50.2 us staged; forcing 6 or 8
    // CTAs per SM on the per-thread form spilled and ended at 42 us; moving a thread's two adjacent packets as one 32-byte
    // access brought it to 36.6 us)
#define AQ_LAUNCH(V)                                                                                                 \
    {                                                                                                                \
        a.geom = make_geom(a.geom.num_ch, a.geom.inner, chunk_elems<V>(), a.n);                                      \
        if (PER_CH && a.geom.inner * 16 < chunk_elems<V>() && a.geom.inner % (unroll_of<V>() * V) == 0)              \
            launch_v2_variant<T, V, PER_CH ? 2 : 0>(a, narrow, st);                                                  \
        else                                                                                                         \
            launch_v2_variant<T, V, PER_CH ? 1 : 0>(a, narrow, st);                                                  \
    }
    if (sizeof(T) == 2 && vec == 8)
        AQ_LAUNCH((sizeof(T) == 2 ? 8 : 4))
    else if (vec >= 4)
        AQ_LAUNCH(4)
    else
        AQ_LAUNCH(1)
#undef AQ_LAUNCH
    note_launch();
    return check_launch();
}

template <typename T>
static int launch_v2_t(V2Args a, bool narrow, cudaStream_t st)
{
    const bool per_ch = a.geom.num_ch > 1;
    a.wide_ok         = ((uintptr_t) a.x % 32 == 0 && (uintptr_t) a.y % 32 == 0) ? 1 : 0;
    // the mask is written with VEC-byte packets, so it constrains the width like the tensors do
    int vec = pick_vec<T>(a.x, a.y, nullptr, per_ch ? a.geom.inner : 0);
    while (vec > 1 && a.mask && ((uintptr_t) a.mask % vec))
        vec >>= 1;
    if (per_ch)
        return launch_v2_vec<T, true>(a, vec, narrow, st);
    return launch_v2_vec<T, false>(a, vec, narrow, st);
}

// Grids of 2^24 steps or more (a 32-bit quantizer): the reference evaluates the same expressions in float64
// (torch_builtins.py:162-171).  A plain element-per-thread kernel with IEEE double arithmetic; such grids are rare and
// the kernel is division-bound, not memory-bound.
template <typename T>
__global__ void __launch_bounds__(256) v2_f64_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                     uint8_t* __restrict__ mask, int64_t n, const float* __restrict__ scale,
                                                     const float* __restrict__ offset, double qmin, double qmax,
                                                     int codes, int64_t num_ch, int64_t inner)
{
    pdl_launch_dependents();
    pdl_wait();
    for (int64_t i = (int64_t) blockIdx.x * 256 + threadIdx.x; i < n; i += (int64_t) gridDim.x * 256)
    {
        const int64_t ch = num_ch > 1 ? (i / inner) % num_ch : 0;
        const double s = (double) scale[ch], o = (double) offset[ch];
        const double r = __dsub_rn(rint(__ddiv_rn((double) to_f32<T>(x[i]), s)), o);
        if (mask)
            mask[i] = (r >= qmin && r <= qmax) ? 1 : 0;
        const double q = fmin(fmax(r, qmin), qmax);   // NaN stays NaN in torch.clamp; fmin / fmax would drop it
        const double c = (r != r) ? r : q;
        const double out = codes ? c : __dmul_rn(__dadd_rn(c, o), s);
        y[i] = from_f32<T>(__double2float_rn(out));
    }
}

template <typename T>
static int launch_v2_f64(const V2Args& a, cudaStream_t st)
{
    int64_t blocks = (a.n + 255) / 256;
    if (blocks > (int64_t) kNumSMs * 8)
        blocks = (int64_t) kNumSMs * 8;
    launch_pdl(v2_f64_kernel<T>, (unsigned) blocks, 256, 0, st, (const T*) a.x, (T*) a.y, a.mask, a.n, a.scale, a.offset,
               a.qmin_wide, a.qmax_wide, a.out_kind == AQ_V2_OUT_CODES ? 1 : 0, a.geom.num_ch, a.geom.inner);
    note_launch();
    return check_launch();
}

int v2_launch(V2Args a, int dtype, int narrow_internal, cudaStream_t st)
{
    if (a.n == 0)
        return AQ_OK;
    if (narrow_internal == AQ_V2_INTERNAL_F64)
    {
        if (a.dequant_only)
            return AQ_ERR_UNSUPPORTED;
        switch (dtype)
        {
        case AQ_F32: return launch_v2_f64<float>(a, st);
        case AQ_BF16: return launch_v2_f64<__nv_bfloat16>(a, st);
        case AQ_F16: return launch_v2_f64<__half>(a, st);
        default: return AQ_ERR_INVALID_ARG;
        }
    }
    switch (dtype)
    {
    case AQ_F32: return launch_v2_t<float>(a, false, st);
    case AQ_BF16: return launch_v2_t<__nv_bfloat16>(a, narrow_internal != 0, st);
    case AQ_F16: return launch_v2_t<__half>(a, narrow_internal != 0, st);
    default: return AQ_ERR_INVALID_ARG;
    }
}

// -------------------------------------------------------------------------------------------------
// 16-bit float fake-quantization: out = float(half(in))  (quantizeDequantizeFp16Kernel, trim_functions.cu:135-148)
// -------------------------------------------------------------------------------------------------
template <int VEC>
__global__ void __launch_bounds__(kThreads) fp16_qdq_kernel(const float* __restrict__ in, float* __restrict__ out, int64_t n)
{
    pdl_launch_dependents();
    pdl_wait();
    const int64_t idx = ((int64_t) blockIdx.x * kThreads + threadIdx.x) * VEC;
    if (idx + VEC <= n)
    {
        const Pack<float, VEC> v = load_pack<float, VEC>(in + idx);
        Pack<float, VEC> r;
#pragma unroll
        for (int e = 0; e < VEC; ++e)
            r.v[e] = __half2float(__float2half_rn(v.v[e]));
        store_pack<float, VEC>(out + idx, r);
    }
    else
    {
        for (int64_t i = idx; i < n; ++i)
            out[i] = __half2float(__float2half_rn(in[i]));
    }
}

int fp16_qdq(const float* in, float* out, int64_t n, cudaStream_t st)
{
    if (n == 0)
        return AQ_OK;
    const int vec = pick_vec<float>(in, out, nullptr, 0) >= 4 ? 4 : 1;
    const int64_t grid = (n + (int64_t) kThreads * vec - 1) / ((int64_t) kThreads * vec);
    if (vec == 4)
        launch_pdl(fp16_qdq_kernel<4>, (unsigned) grid, kThreads, 0, st, in, out, n);
    else
        launch_pdl(fp16_qdq_kernel<1>, (unsigned) grid, kThreads, 0, st, in, out, n);
    note_launch();
    return check_launch();
}

// -------------------------------------------------------------------------------------------------
// Integer codes in integer containers (libpymo "packed" form)
// -------------------------------------------------------------------------------------------------
// quantizeToFxpPackedCpu / dequantizeFromPackedFxpCpu (DlQuantization/src/trim_functions.cpp:220-605): unlike the
// float-container path these evaluate clamp, divide, offset and round in DOUBLE from the double-precision encoding, and
// store one code per container of max(bw, 8) bits (uint8/16/32, or int8/16/32 when shifted to signed by 2^(bw-1) - 1;
// sub-byte widths keep one value per byte, the signed ones masked to their low bw bits).
template <typename OUT>
__device__ __forceinline__ OUT packed_store_cast(double v, double lo, double hi)
{
    const double c = (hi < v) ? hi : v;          // std::min(v, hi)
    const double d = (c < lo) ? lo : c;          // std::max(., lo)
    return (d == d) ? (OUT) d : (OUT) 0;
}

template <typename OUT>
__global__ void __launch_bounds__(256) packed_quantize_kernel(const float* __restrict__ in, OUT* __restrict__ out,
                                                              int64_t n, double e_min, double e_max, double delta,
                                                              double offset, int bw, int to_signed)
{
    pdl_launch_dependents();
    pdl_wait();
    const double shift = to_signed ? ldexp(1.0, bw - 1) - 1.0 : 0.0;
    const double top   = ldexp(1.0, bw) - 1.0;
    for (int64_t i = (int64_t) blockIdx.x * 256 + threadIdx.x; i < n; i += (int64_t) gridDim.x * 256)
    {
        const double x = (double) in[i];
        double q       = (e_max < x) ? e_max : x;    // std::min(x, max)
        q              = (q < e_min) ? e_min : q;    // std::max(., min)
        q              = round(__dsub_rn(__ddiv_rn(q, delta), offset));
        if (!to_signed)
        {
            if (bw < 8)
            {
                const uint8_t small = (q == q) ? (uint8_t) q : (uint8_t) 0;
                out[i]              = (OUT) packed_store_cast<uint8_t>((double) small, 0.0, top);
            }
            else
                out[i] = packed_store_cast<OUT>(q, 0.0, bw == 8 ? 255.0 : (bw == 16 ? 65535.0 : 4294967295.0));
        }
        else
        {
            q = __dsub_rn(q, shift);
            if (bw < 8)
            {
                const int8_t small = (q == q) ? (int8_t) q : (int8_t) 0;
                out[i]             = (OUT) (small & (int8_t) (int) top);
            }
            else
                out[i] = packed_store_cast<OUT>(q, bw == 8 ? -128.0 : (bw == 16 ? -32768.0 : -2147483648.0),
                                                bw == 8 ? 127.0 : (bw == 16 ? 32767.0 : 2147483647.0));
        }
    }
}

template <typename IN>
__global__ void __launch_bounds__(256) packed_dequantize_kernel(const IN* __restrict__ in, float* __restrict__ out,
                                                                int64_t n, double delta, double offset, int bw,
                                                                int is_signed)
{
    pdl_launch_dependents();
    pdl_wait();
    for (int64_t i = (int64_t) blockIdx.x * 256 + threadIdx.x; i < n; i += (int64_t) gridDim.x * 256)
    {
        double code = (double) in[i];
        if (is_signed && bw < 8)
        {
            // one value per byte, sign-extended from its low bw bits
            const int8_t b = (int8_t) in[i];
            code           = (b & (int8_t) (1 << (bw - 1))) ? (double) (int8_t) (~((int8_t) ((1 << bw) - 1)) | b) : (double) b;
        }
        out[i] = (float) __dmul_rn(delta, __dadd_rn(code, offset));
    }
}

static unsigned packed_grid(int64_t n)
{
    int64_t blocks = (n + 255) / 256;
    if (blocks > (int64_t) kNumSMs * 16)
        blocks = (int64_t) kNumSMs * 16;
    return (unsigned) (blocks < 1 ? 1 : blocks);
}

int packed_quantize(const float* in, void* out, int64_t n, double e_min, double e_max, double delta, double offset, int bw,
                    int to_signed, cudaStream_t st)
{
    if (n == 0)
        return AQ_OK;
#define AQ_PQ(OUT)                                                                                                   \
    launch_pdl(packed_quantize_kernel<OUT>, packed_grid(n), 256, 0, st, in, (OUT*) out, n, e_min, e_max, delta, offset, \
               bw, to_signed)
    if (bw <= 8)
    {
        if (to_signed)
            AQ_PQ(int8_t);
        else
            AQ_PQ(uint8_t);
    }
    else if (bw == 16)
    {
        if (to_signed)
            AQ_PQ(int16_t);
        else
            AQ_PQ(uint16_t);
    }
    else
    {
        if (to_signed)
            AQ_PQ(int32_t);
        else
            AQ_PQ(uint32_t);
    }
#undef AQ_PQ
    note_launch();
    return check_launch();
}

int packed_dequantize(const void* in, float* out, int64_t n, double delta, double offset, int bw, int is_signed,
                      cudaStream_t st)
{
    if (n == 0)
        return AQ_OK;
#define AQ_PD(IN)                                                                                                    \
    launch_pdl(packed_dequantize_kernel<IN>, packed_grid(n), 256, 0, st, (const IN*) in, out, n, delta, offset, bw,    \
               is_signed)
    if (bw <= 8)
    {
        if (is_signed)
            AQ_PD(int8_t);
        else
            AQ_PD(uint8_t);
    }
    else if (bw == 16)
    {
        if (is_signed)
            AQ_PD(int16_t);
        else
            AQ_PD(uint16_t);
    }
    else
    {
        if (is_signed)
            AQ_PD(int32_t);
        else
            AQ_PD(uint32_t);
    }
#undef AQ_PD
    note_launch();
    return check_launch();
}

// -------------------------------------------------------------------------------------------------
// Backward kernels
// -------------------------------------------------------------------------------------------------

template <typename T>
struct PairOf
{
    using type                       = float2;
    static constexpr uint32_t one_bits = 0;
};
template <>
struct PairOf<__half>
{
    using type                       = __half2;
    static constexpr uint32_t one_bits = 0x3c00u;
};
template <>
struct PairOf<__nv_bfloat16>
{
    using type                       = __nv_bfloat162;
    static constexpr uint32_t one_bits = 0x3f80u;
};

// v2: dx = grad * mask  (torch_builtins.py:342).  Mask bytes are 0 or 1 (as aq_v2_quantize writes them).
// One packet per thread and 8 CTAs per SM: with four packets per thread the kernel needed 48 registers (5 CTAs per SM)
// and a 25.7 MB gradient took 13.4 us; this form takes 10.1 us there and the same 89.6 us as before at 256 MB.
#ifndef AQ_BWD_MINB
#define AQ_BWD_MINB 8
#endif
#ifndef AQ_BWD_UNROLL
#define AQ_BWD_UNROLL 1
#endif
template <int VEC>
__host__ __device__ constexpr int bwd_unroll()
{
    return VEC == 8 ? AQ_UNROLL8 : AQ_BWD_UNROLL;
}
template <typename T, int VEC>
__global__ void __launch_bounds__(kThreads, AQ_BWD_MINB) v2_bwd_kernel(const T* __restrict__ g,
                                                                       const uint8_t* __restrict__ mask,
                                                                       T* __restrict__ dx, int64_t n)
{
    pdl_launch_dependents();
    pdl_wait();
    constexpr int U     = bwd_unroll<VEC>();
    constexpr int CHUNK = kThreads * VEC * U;
    const int64_t base  = (int64_t) blockIdx.x * CHUNK;
    Pack<T, VEC> v[U];
    Pack<uint8_t, VEC> m[U];
    bool full[U];
    load_chunk<T, VEC, U>(g, base, n, v, full);
    load_chunk<uint8_t, VEC, U>(mask, base, n, m, full);
#pragma unroll
    for (int u = 0; u < U; ++u)
    {
        const int64_t idx = base + (int64_t) (u * kThreads + threadIdx.x) * VEC;
        Pack<T, VEC> r;
        if constexpr (sizeof(T) == 2 && VEC == 8)
        {
            // grad * bool with two lanes per instruction: the 0 / 1 mask bytes of a pair are spread to 16-bit lanes
            // and scaled to the bit pattern of 1.0, then one packed multiply in the storage type (x * 1 and x * 0
            // are exact there, and -0 / Inf / NaN behave as in the reference product).
            using T2            = typename PairOf<T>::type;
            const uint32_t one  = PairOf<T>::one_bits;
            const uint32_t* mw  = reinterpret_cast<const uint32_t*>(&m[u]);
            const uint32_t* gw  = reinterpret_cast<const uint32_t*>(&v[u]);
            uint32_t* rw        = reinterpret_cast<uint32_t*>(&r);
#pragma unroll
            for (int j = 0; j < 4; ++j)
            {
                const uint32_t sel = __byte_perm(mw[j >> 1], 0u, (j & 1) ? 0x4342u : 0x4140u) * one;
                const T2 prod      = __hmul2(*reinterpret_cast<const T2*>(&gw[j]), *reinterpret_cast<const T2*>(&sel));
                rw[j]              = *reinterpret_cast<const uint32_t*>(&prod);
            }
        }
        else
        {
            float f[VEC];
            unpack<T, VEC>(v[u], f);
#pragma unroll
            for (int e = 0; e < VEC; ++e)
            {
                // grad * bool: x*1 and x*0 are exact in any dtype (-0 and NaN behave as in the reference product)
                f[e] = __fmul_rn(f[e], m[u].v[e] ? 1.0f : 0.0f);
            }
            repack<T, VEC>(f, r);
        }
        store_packet<T, VEC>(dx, idx, n, r, full[u]);
    }
}

template <typename T>
static int launch_v2_bwd(const void* g, const uint8_t* mask, void* dx, int64_t n, cudaStream_t st)
{
    int vec = pick_vec<T>(g, dx, nullptr, 0);
    while (vec > 1 && ((uintptr_t) mask % vec))
        vec >>= 1;
#define AQ_LAUNCH(V)                                                                                                 \
    {                                                                                                                \
        const int64_t chunk = (int64_t) kThreads * V * bwd_unroll<V>();                                              \
        int64_t grid        = (n + chunk - 1) / chunk;                                                               \
        launch_pdl(v2_bwd_kernel<T, V>, (unsigned) grid, kThreads, 0, st, (const T*) g, mask, (T*) dx, n);                    \
    }
    if (sizeof(T) == 2 && vec == 8)
        AQ_LAUNCH((sizeof(T) == 2 ? 8 : 4))
    else if (vec >= 4)
        AQ_LAUNCH(4)
    else
        AQ_LAUNCH(1)
#undef AQ_LAUNCH
    note_launch();
    return check_launch();
}

int v2_backward(const void* g, const uint8_t* mask, void* dx, int dtype, int64_t n, cudaStream_t st)
{
    if (n == 0)
        return AQ_OK;
    switch (dtype)
    {
    case AQ_F32: return launch_v2_bwd<float>(g, mask, dx, n, st);
    case AQ_F16: return launch_v2_bwd<__half>(g, mask, dx, n, st);
    case AQ_BF16: return launch_v2_bwd<__nv_bfloat16>(g, mask, dx, n, st);
    default: return AQ_ERR_INVALID_ARG;
    }
}

// v2 encoding gradients (torch_builtins.py:334-343):
//   ds = g * (clamp(round(x/s), o + qmin, o + qmax) - (x/s) * mask)      do = g * ((1 - mask) * s)
// REDUCE = false: element-wise and un-reduced exactly like the reference returns them (its autograd sums over the
// broadcast dimensions afterwards).  REDUCE = true: that sum is taken here -- per thread over its packets, per CTA
// in shared memory (one slot per run of a channel inside the CTA's chunk), then one floating-point atomic per run into
// the per-channel result -- so the two full-size fp32 tensors (8 bytes per element written, 8 read back) never exist.
// The summation order differs from torch's, which is not specified either; the terms are identical.
template <typename T, int VEC, bool PER_CH, bool REDUCE>
__global__ void __launch_bounds__(kThreads) v2_param_grad_kernel(V2GradArgs a)
{
    pdl_launch_dependents();
    pdl_wait();
    constexpr int CHUNK = chunk_elems<VEC>();
    const int64_t base  = (int64_t) blockIdx.x * CHUNK;
    __shared__ float s_sc[PER_CH ? kMaxRuns : 1], s_of[PER_CH ? kMaxRuns : 1];
    __shared__ float s_ds[(PER_CH && REDUCE) ? kMaxRuns : kThreads / 32], s_do[(PER_CH && REDUCE) ? kMaxRuns : kThreads / 32];
    RunCtx rc {0, 0, 1, 0};
    float sc0 = 0.f, of0 = 0.f;
    Pack<T, VEC> xv[unroll_of<VEC>()], gv[unroll_of<VEC>()];
    Pack<uint8_t, VEC> mv[unroll_of<VEC>()];
    bool full[unroll_of<VEC>()];
    load_chunk<T, VEC, unroll_of<VEC>()>(static_cast<const T*>(a.x), base, a.n, xv, full);
    load_chunk<T, VEC, unroll_of<VEC>()>(static_cast<const T*>(a.grad), base, a.n, gv, full);
    load_chunk<uint8_t, VEC, unroll_of<VEC>()>(a.mask, base, a.n, mv, full);
    if (PER_CH)
    {
        rc = make_run_ctx<VEC>(a.geom, base, a.n);
        for (int lr = threadIdx.x; lr < rc.nruns; lr += kThreads)
        {
            const int64_t ch = run_channel(a.geom, rc, lr);
            s_sc[lr]         = a.scale[ch];
            s_of[lr]         = a.offset[ch];
            if (REDUCE)
                s_ds[lr] = 0.0f, s_do[lr] = 0.0f;
        }
        __syncthreads();
    }
    else
    {
        sc0 = __ldg(a.scale);
        of0 = __ldg(a.offset);
    }
    float tot_s = 0.0f, tot_o = 0.0f;   // per-thread sums (per-tensor encodings)
#pragma unroll
    for (int u = 0; u < unroll_of<VEC>(); ++u)
    {
        const uint32_t off = (uint32_t) (u * kThreads + threadIdx.x) * VEC;
        const int64_t idx  = base + off;
        float sc = sc0, of = of0;
        uint32_t lr = 0;
        if (PER_CH)
        {
            lr = run_of(a.geom, rc, off);
            sc = s_sc[lr], of = s_of[lr];
        }
        const float lo = __fadd_rn(of, a.qmin), hi = __fadd_rn(of, a.qmax);
        Pack<float, VEC> ds, dof;
        float ps = 0.0f, po = 0.0f;
#pragma unroll
        for (int e = 0; e < VEC; ++e)
        {
            const float g = to_f32<T>(gv[u].v[e]);
            const float m = mv[u].v[e] ? 1.0f : 0.0f;
            const float t = __fdiv_rn(to_f32<T>(xv[u].v[e]), sc);
            const float c = clamp_keep_nan(rintf(t), lo, hi);
            ds.v[e]       = __fmul_rn(g, __fsub_rn(c, __fmul_rn(t, m)));
            dof.v[e]      = __fmul_rn(g, __fmul_rn(1.0f - m, sc));
            if (REDUCE && (full[u] || idx + e < a.n))
                ps += ds.v[e], po += dof.v[e];
        }
        if (REDUCE)
        {
            if (PER_CH)
            {
                // A warp's 32 packets are consecutive, so they nearly always lie in one run: the warp adds them up with
                // shuffles and issues one shared atomic (thirty-two floating-point atomics on one shared address
                // serialise: rows of 2304 elements ran at 0.06 of the copy bandwidth that way).
                const bool active     = idx < a.n;
                const unsigned livems = __ballot_sync(0xffffffffu, active);
                if (livems)
                {
                    const int leader   = __ffs(livems) - 1;
                    const uint32_t lrl = __shfl_sync(0xffffffffu, lr, leader);
                    if (__all_sync(0xffffffffu, !active || lr == lrl))
                    {
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1)
                        {
                            ps += __shfl_xor_sync(0xffffffffu, ps, o);
                            po += __shfl_xor_sync(0xffffffffu, po, o);
                        }
                        if ((threadIdx.x & 31) == leader)
                        {
                            if (a.dscale)
                                atomicAdd(&s_ds[lrl], ps);
                            if (a.doffset)
                                atomicAdd(&s_do[lrl], po);
                        }
                    }
                    else if (active)
                    {
                        if (a.dscale)
                            atomicAdd(&s_ds[lr], ps);
                        if (a.doffset)
                            atomicAdd(&s_do[lr], po);
                    }
                }
            }
            else
                tot_s += ps, tot_o += po;
        }
        else
        {
            if (a.dscale)
                store_packet<float, VEC>(a.dscale, idx, a.n, ds, full[u]);
            if (a.doffset)
                store_packet<float, VEC>(a.doffset, idx, a.n, dof, full[u]);
        }
    }
    if (!REDUCE)
        return;
    if (PER_CH)
    {
        __syncthreads();
        for (int lr = threadIdx.x; lr < rc.nruns; lr += kThreads)
        {
            const int64_t ch = run_channel(a.geom, rc, lr);
            if (a.dscale && s_ds[lr] != 0.0f)
                atomicAdd(&a.dscale[ch], s_ds[lr]);
            if (a.doffset && s_do[lr] != 0.0f)
                atomicAdd(&a.doffset[ch], s_do[lr]);
        }
    }
    else
    {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
        {
            tot_s += __shfl_xor_sync(0xffffffffu, tot_s, o);
            tot_o += __shfl_xor_sync(0xffffffffu, tot_o, o);
        }
        if ((threadIdx.x & 31) == 0)
            s_ds[threadIdx.x >> 5] = tot_s, s_do[threadIdx.x >> 5] = tot_o;
        __syncthreads();
        if (threadIdx.x == 0)
        {
            float bs = 0.0f, bo = 0.0f;
            for (int w = 0; w < kThreads / 32; ++w)
                bs += s_ds[w], bo += s_do[w];
            if (a.dscale)
                atomicAdd(a.dscale, bs);
            if (a.doffset)
                atomicAdd(a.doffset, bo);
        }
    }
}

template <typename T>
static int launch_param_grad(V2GradArgs a, bool reduce, cudaStream_t st)
{
    const bool per_ch = a.geom.num_ch > 1;
    int vec           = pick_vec<T>(a.x, a.grad, nullptr, per_ch ? a.geom.inner : 0);
    if (vec > 4)
        vec = 4;   // fp32 outputs: 4 elements = 16 bytes
    while (vec > 1 && (((uintptr_t) a.mask % vec) ||
                       (!reduce && (((uintptr_t) a.dscale % (4 * vec)) || ((uintptr_t) a.doffset % (4 * vec))))))
        vec >>= 1;
    if (reduce)
    {
        // the sums start from zero (the outputs are small: one float per encoding)
        cudaError_t e = cudaSuccess;
        if (a.dscale)
            e = cudaMemsetAsync(a.dscale, 0, sizeof(float) * (size_t) a.geom.num_ch, st);
        if (e == cudaSuccess && a.doffset)
            e = cudaMemsetAsync(a.doffset, 0, sizeof(float) * (size_t) a.geom.num_ch, st);
        if (e != cudaSuccess)
            return cuda_fail(e);
    }
#define AQ_LAUNCH(V, PC, RD)                                                                                         \
    {                                                                                                                \
        a.geom       = make_geom(a.geom.num_ch, a.geom.inner, chunk_elems<V>(), a.n);                                     \
        int64_t grid = (a.n + chunk_elems<V>() - 1) / chunk_elems<V>();                                              \
        launch_pdl(v2_param_grad_kernel<T, V, PC, RD>, (unsigned) grid, kThreads, 0, st, a);                         \
    }
#define AQ_PICK(RD)                                                                                                  \
    if (per_ch)                                                                                                      \
    {                                                                                                                \
        if (vec == 4)                                                                                                \
            AQ_LAUNCH(4, true, RD)                                                                                   \
        else                                                                                                         \
            AQ_LAUNCH(1, true, RD)                                                                                   \
    }                                                                                                                \
    else                                                                                                             \
    {                                                                                                                \
        if (vec == 4)                                                                                                \
            AQ_LAUNCH(4, false, RD)                                                                                  \
        else                                                                                                         \
            AQ_LAUNCH(1, false, RD)                                                                                  \
    }
    if (reduce)
    {
        AQ_PICK(true)
    }
    else
    {
        AQ_PICK(false)
    }
#undef AQ_PICK
#undef AQ_LAUNCH
    note_launch();
    return check_launch();
}

int v2_param_grad(V2GradArgs a, int dtype, int reduce, cudaStream_t st)
{
    if (a.n == 0 && !reduce)
        return AQ_OK;
    switch (dtype)
    {
    case AQ_F32: return launch_param_grad<float>(a, reduce != 0, st);
    case AQ_F16: return launch_param_grad<__half>(a, reduce != 0, st);
    case AQ_BF16: return launch_param_grad<__nv_bfloat16>(a, reduce != 0, st);
    default: return AQ_ERR_INVALID_ARG;
    }
}

// v1: dx = g * [enc_min <= x <= enc_max], mask recomputed from the saved input
// (aimet_torch/v1/quantsim_straight_through_grad.py:91-118)
template <int VEC, bool PER_CH>
__global__ void __launch_bounds__(kThreads) ste_v1_kernel(SteArgs a)
{
    pdl_launch_dependents();
    pdl_wait();
    constexpr int CHUNK = chunk_elems<VEC>();
    const int64_t base  = (int64_t) blockIdx.x * CHUNK;
    __shared__ float s_mn[PER_CH ? kMaxRuns : 1], s_mx[PER_CH ? kMaxRuns : 1];
    RunCtx rc {0, 0, 1, 0};
    float mn0 = 0.f, mx0 = 0.f;
    Pack<float, VEC> xv[unroll_of<VEC>()], gv[unroll_of<VEC>()];
    bool full[unroll_of<VEC>()];
    load_chunk<float, VEC, unroll_of<VEC>()>(a.x, base, a.n, xv, full);
    load_chunk<float, VEC, unroll_of<VEC>()>(a.g, base, a.n, gv, full);
    if (PER_CH)
    {
        rc = make_run_ctx<VEC>(a.geom, base, a.n);
        for (int lr = threadIdx.x; lr < rc.nruns; lr += kThreads)
        {
            const int64_t ch = run_channel(a.geom, rc, lr);
            s_mn[lr]         = a.enc_min[ch];
            s_mx[lr]         = a.enc_max[ch];
        }
        __syncthreads();
    }
    else
    {
        mn0 = __ldg(a.enc_min);
        mx0 = __ldg(a.enc_max);
    }
#pragma unroll
    for (int u = 0; u < unroll_of<VEC>(); ++u)
    {
        const uint32_t off = (uint32_t) (u * kThreads + threadIdx.x) * VEC;
        float mn = mn0, mx = mx0;
        if (PER_CH)
        {
            const uint32_t lr = run_of(a.geom, rc, off);
            mn = s_mn[lr], mx = s_mx[lr];
        }
#pragma unroll
        for (int e = 0; e < VEC; ++e)
        {
            const float x = xv[u].v[e];
            gv[u].v[e]    = __fmul_rn(gv[u].v[e], (mn <= x && x <= mx) ? 1.0f : 0.0f);
        }
        store_packet<float, VEC>(a.dx, base + off, a.n, gv[u], full[u]);
    }
}

int ste_v1(SteArgs a, cudaStream_t st)
{
    if (a.n == 0)
        return AQ_OK;
    const bool per_ch = a.geom.num_ch > 1;
    const int vec     = pick_vec<float>(a.x, a.g, a.dx, per_ch ? a.geom.inner : 0);
#define AQ_LAUNCH(V, PC)                                                                                             \
    {                                                                                                                \
        a.geom       = make_geom(a.geom.num_ch, a.geom.inner, chunk_elems<V>(), a.n);                                     \
        int64_t grid = (a.n + chunk_elems<V>() - 1) / chunk_elems<V>();                                              \
        launch_pdl(ste_v1_kernel<V, PC>, (unsigned) grid, kThreads, 0, st, a);                                               \
    }
    if (per_ch)
    {
        if (vec == 4)
            AQ_LAUNCH(4, true)
        else
            AQ_LAUNCH(1, true)
    }
    else
    {
        if (vec == 4)
            AQ_LAUNCH(4, false)
        else
            AQ_LAUNCH(1, false)
    }
#undef AQ_LAUNCH
    note_launch();
    return check_launch();
}

}   // namespace aq
