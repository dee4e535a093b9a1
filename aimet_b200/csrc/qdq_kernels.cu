// Fake-quant element kernels for sm_100a: quantize-dequantize / quantize / dequantize forward and the
// straight-through backward, at per-tensor, per-channel and blockwise granularity.
//
// All kernels are HBM-bound streaming kernels: one CTA owns one contiguous chunk of
// THREADS * VEC * UNROLL elements, every thread issues UNROLL independent 16-byte (VEC-wide) loads before
// it computes, and the per-channel / per-block encodings of the chunk are staged once in shared memory.
//
// Results must match the CPU reference bit for bit, and the reference divides (x / scale).  An IEEE division
// costs ~10 instructions, which would make the 16-bit kernels issue-bound, so the hot loop multiplies by the
// correctly rounded reciprocal instead and *proves* per element that this cannot change the rounded integer:
// the product and the true quotient differ by a few ulps, so they can only round to different integers when
// the product lies within a small margin of a rounding boundary.  Elements inside that margin (about one in
// ten thousand for 8-bit grids), and anything non-finite, take the exact division.  The file is compiled with
// -fmad=false; every fused multiply-add below is explicit.
#include "common.cuh"
#include "kernels.h"

namespace aq
{

constexpr int kThreads = 256;
constexpr int kUnroll  = 4;
constexpr int kMaxRuns = 1026;   // chunk / inner + 2 with VEC | inner  (see make_geom)

template <int VEC>
__host__ __device__ constexpr int chunk_elems()
{
    return kThreads * VEC * kUnroll;
}

constexpr float kMagicRne = 12582912.0f;   // 1.5 * 2^23: (t + M) - M == rint(t) for |t| < 2^22
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
};

template <int VEC>
__device__ __forceinline__ RunCtx make_run_ctx(const ChanGeom& g, int64_t base, int64_t n)
{
    RunCtx c;
    c.r0              = base / g.inner;
    c.loc0            = base - c.r0 * g.inner;
    int64_t remaining = n - base;
    int64_t span      = remaining < (int64_t) chunk_elems<VEC>() ? remaining : (int64_t) chunk_elems<VEC>();
    c.nruns           = (int) ((c.loc0 + span - 1) / g.inner) + 1;
    return c;
}

__device__ __forceinline__ uint32_t run_of(const ChanGeom& g, const RunCtx& c, uint32_t off)
{
    if (g.mode == 2)
        return (c.loc0 + (int64_t) off) >= g.inner ? 1u : 0u;
    return local_run(g, (uint32_t) c.loc0 + off);
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

// =================================================================================================
// Element operators.  Each has a Slot (per-channel constants, staged in shared memory or held in registers for
// per-tensor work), `load(ch)` to build it, and `apply(x, slot, in_range)`.
// =================================================================================================

// ---- libpymo: quantizeValueCpu + dequantizeValueCpu (DlQuantization/src/trim_functions.cpp:140-171) -------------
//   t = fmax(fmin(x, max), min);  u = t / delta - offset;  q = roundf(u);  y = delta * (q + offset)
struct PymoOp
{
    // per-tensor (host-derived grid, narrowed to float like the reference does at the call boundary)
    float mn, mx, delta, offset;
    // per-channel
    const float* enc_min;      // raw min/max (derive = 1) or gated min/max (derive = 0)
    const float* enc_max;
    const float* enc_delta;    // derive = 0 only
    const float* enc_offset;   // derive = 0 only
    float num_steps;
    int derive;
    float shift;       // subtracted from codes (quantize only)
    int codes_only;    // 1: emit integer codes, 0: quantize-dequantize

    struct Slot
    {
        float mn, mx, dl, of;
        float rdl;    // RN(1 / delta)
        float c;      // 0.5 - offset
        float eps;    // 0.5 - margin, or 0 when the reciprocal form cannot be trusted for this grid
    };

    __device__ __forceinline__ static void finish(Slot& k)
    {
        k.rdl = __frcp_rn(k.dl);
        k.c   = 0.5f - k.of;
        // u ranges over [~0, (max-min)/delta]; |s - (u + 0.5)| <= 2^-24 (2|q| + |c| + |s| + |u|) with
        // |q| <= |of| + |u|, so 2^-24 (3|of| + 4 umax + 2), plus a quarter for second-order terms
        const float umax   = fabsf(__fdiv_rn(__fsub_rn(k.mx, k.mn), k.dl));
        const float margin = 1.25f * kUlp24 * (3.0f * fabsf(k.of) + 4.0f * umax + 2.0f);
        k.eps              = (margin < 0.25f && umax < 4194304.0f) ? 0.5f - margin : 0.0f;   // NaN -> 0
        if (!(k.eps > 0.0f))
            k.eps = 0.0f;
    }

    __device__ __forceinline__ Slot scalar_slot() const
    {
        Slot k;
        k.mn = mn, k.mx = mx, k.dl = delta, k.of = offset;
        finish(k);
        return k;
    }

    __device__ __forceinline__ Slot load(int64_t ch) const
    {
        Slot k;
        k.mn = enc_min[ch], k.mx = enc_max[ch];
        if (derive)
        {
            // AimetTensorQuantizer.cpp:236-254: gate, delta, offset in fp32 (offset: half to even)
            k.mn     = k.mn < 0.0f ? k.mn : 0.0f;
            k.mx     = k.mx > 0.0f ? k.mx : 0.0f;
            float lo = __fadd_rn(k.mn, 1e-5f);
            k.mx     = k.mx > lo ? k.mx : lo;
            k.dl     = __fdiv_rn(__fsub_rn(k.mx, k.mn), num_steps);
            k.of     = rintf(__fdiv_rn(k.mn, k.dl));
        }
        else
        {
            k.dl = enc_delta[ch];
            k.of = enc_offset[ch];
        }
        finish(k);
        return k;
    }

    template <bool NARROW>
    __device__ __forceinline__ float apply(float x, const Slot& k, bool& in_range) const
    {
        in_range      = true;
        const float t = fmaxf(fminf(x, k.mx), k.mn);
        // fast: s ~ u + 0.5; q = floor(s) read from the mantissa after a round-down add of 2^23
        const float s  = fmaf(t, k.rdl, k.c);
        const float s2 = __fadd_rd(s, kTwo23f);
        float q        = s2 - kTwo23f;
        const float g  = s - (s2 - 8388607.5f);
        if (!(fabsf(g) < k.eps) || s < 0.0f)
        {
            // near a rounding boundary (or a degenerate grid): the reference formula itself
            q = round_half_away(__fsub_rn(__fdiv_rn(t, k.dl), k.of));
        }
        if (codes_only)
            return __fsub_rn(q, shift);
        return __fmul_rn(k.dl, __fadd_rn(q, k.of));
    }
};

// ---- v2: torch_builtins.py:303-313 (QuantDequantFunc / QuantizeFunc) and :264-266 (DequantizeFunc) -------------
//   r = round_half_even(x / s) - o;  mask = qmin <= r <= qmax;  q = clamp(r, qmin, qmax);  y = (q + o) * s
struct V2Op
{
    const float* scale;
    const float* offset;
    float qmin, qmax;
    int out_kind;
    int dequant_only;

    struct Slot
    {
        float s, o, rs;
    };

    __device__ __forceinline__ Slot load(int64_t ch) const
    {
        Slot k;
        k.s  = scale[ch];
        k.o  = offset[ch];
        k.rs = __frcp_rn(k.s);
        return k;
    }
    __device__ __forceinline__ Slot scalar_slot() const
    {
        return load(0);
    }

    template <typename T, bool NARROW>
    __device__ __forceinline__ float apply_t(float x, const Slot& k, bool& in_range) const
    {
        if (dequant_only)
        {
            in_range = true;
            float r  = __fadd_rn(x, k.o);
            if (NARROW)
                r = narrow<T>(r);
            return __fmul_rn(r, k.s);
        }
        float r;
        if (NARROW)
        {
            // the storage dtype is also the arithmetic dtype: every step is rounded to it.  fp32 arithmetic
            // followed by one rounding equals the narrow operation (24 >= 2p + 2 for p = 11 and p = 8).
            r = narrow<T>(__fdiv_rn(x, k.s));
            r = rintf(r);
            r = narrow<T>(__fsub_rn(r, k.o));
        }
        else
        {
            // RN(x/s) and RN(x * RN(1/s)) differ by at most 3 ulp, so they round to different integers only if
            // the product is within 3 ulp of a half-integer; 4 ulp = 2^-22 |t| is used as the guard band.
            const float t = __fmul_rn(x, k.rs);
            r             = __fsub_rn(__fadd_rn(t, kMagicRne), kMagicRne);
            const float d = __fsub_rn(t, r);
            if (!(fabsf(d) < fmaf(fabsf(t), -4.0f * kUlp24, 0.5f)))
                r = rintf(__fdiv_rn(x, k.s));   // also taken for NaN / Inf / |t| >= 2^21
            r = __fsub_rn(r, k.o);
        }
        // torch.clamp keeps NaN: min.NaN / max.NaN
        float q;
        asm("max.NaN.f32 %0, %1, %2;" : "=f"(q) : "f"(r), "f"(qmin));
        asm("min.NaN.f32 %0, %1, %2;" : "=f"(q) : "f"(q), "f"(qmax));
        in_range = (q == r);   // false for NaN, like (qmin <= r) & (r <= qmax)
        if (out_kind == AQ_V2_OUT_CODES)
            return q;
        float y = __fadd_rn(q, k.o);
        if (NARROW)
            y = narrow<T>(y);
        return __fmul_rn(y, k.s);
    }
};

// =================================================================================================
// Streaming skeleton
// =================================================================================================
template <typename T, int VEC>
__device__ __forceinline__ void load_chunk(const T* __restrict__ x, int64_t base, int64_t n, Pack<T, VEC> (&v)[kUnroll],
                                           bool (&full)[kUnroll])
{
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
    {
        const int64_t idx = base + (int64_t) (u * kThreads + threadIdx.x) * VEC;
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

struct PymoArgs
{
    const float* in;
    float* out;
    int64_t n;
    PymoOp op;
    ChanGeom geom;
};

template <int VEC, bool PER_CH>
__global__ void __launch_bounds__(kThreads) pymo_qdq_kernel(PymoArgs a)
{
    constexpr int CHUNK = chunk_elems<VEC>();
    const int64_t base  = (int64_t) blockIdx.x * CHUNK;
    __shared__ PymoOp::Slot s_slot[PER_CH ? kMaxRuns : 1];
    RunCtx rc {0, 0, 1};
    PymoOp::Slot k0;
    if (PER_CH)
    {
        rc = make_run_ctx<VEC>(a.geom, base, a.n);
        for (int lr = threadIdx.x; lr < rc.nruns; lr += kThreads)
            s_slot[lr] = a.op.load((rc.r0 + lr) % a.geom.num_ch);
        __syncthreads();
    }
    else
        k0 = a.op.scalar_slot();

    Pack<float, VEC> v[kUnroll];
    bool full[kUnroll];
    load_chunk<float, VEC>(a.in, base, a.n, v, full);
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
    {
        const uint32_t off = (uint32_t) (u * kThreads + threadIdx.x) * VEC;
        PymoOp::Slot k     = k0;
        if (PER_CH)
            k = s_slot[run_of(a.geom, rc, off)];   // VEC | inner: one run per packet
#pragma unroll
        for (int e = 0; e < VEC; ++e)
        {
            bool dummy;
            v[u].v[e] = a.op.apply<false>(v[u].v[e], k, dummy);
        }
        store_packet<float, VEC>(a.out, base + off, a.n, v[u], full[u]);
    }
}

template <bool PER_CH>
static int launch_pymo(PymoArgs a, int vec, cudaStream_t st)
{
    if (a.n == 0)
        return AQ_OK;
#define AQ_LAUNCH(V)                                                                                                 \
    {                                                                                                                \
        a.geom       = make_geom(a.geom.num_ch, a.geom.inner, chunk_elems<V>());                                     \
        int64_t grid = (a.n + chunk_elems<V>() - 1) / chunk_elems<V>();                                              \
        pymo_qdq_kernel<V, PER_CH><<<(unsigned) grid, kThreads, 0, st>>>(a);                                         \
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
    a.op.mn = mn, a.op.mx = mx, a.op.delta = delta, a.op.offset = offset;
    a.op.codes_only = codes_only, a.op.shift = shift;
    a.geom.num_ch = 1, a.geom.inner = n > 0 ? n : 1;
    return launch_pymo<false>(a, pick_vec<float>(in, out, nullptr, 0), st);
}

int pymo_per_channel(const float* in, float* out, int64_t n, int64_t num_ch, int64_t inner, const float* enc_min,
                     const float* enc_max, const float* enc_delta, const float* enc_offset, float num_steps,
                     int derive, cudaStream_t st)
{
    PymoArgs a {};
    a.in = in, a.out = out, a.n = n;
    a.op.enc_min = enc_min, a.op.enc_max = enc_max, a.op.enc_delta = enc_delta, a.op.enc_offset = enc_offset;
    a.op.num_steps = num_steps, a.op.derive = derive;
    a.geom.num_ch = num_ch, a.geom.inner = inner;
    return launch_pymo<true>(a, pick_vec<float>(in, out, nullptr, inner), st);
}

// -------------------------------------------------------------------------------------------------
// General broadcast QDQ (stride walk), libpymo semantics.  Rarely-used fallback for encodings that do not
// reduce to (i / inner) % num_ch; one element per thread per step, exact division.
// -------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) pymo_broadcast_kernel(BroadcastArgs a)
{
    const int64_t stride = (int64_t) gridDim.x * kThreads;
    for (int64_t i = (int64_t) blockIdx.x * kThreads + threadIdx.x; i < a.n; i += stride)
    {
        int64_t e = 0, rem = i;
        for (int d = 0; d < a.ndims; ++d)
        {
            const int64_t k = rem / a.in_strides[d];
            rem -= k * a.in_strides[d];
            e += a.enc_strides[d] * k;
        }
        const float dl = a.dl[e], of = a.of[e];
        const float t  = fmaxf(fminf(a.in[i], a.mx[e]), a.mn[e]);
        const float q  = round_half_away(__fsub_rn(__fdiv_rn(t, dl), of));
        a.out[i]       = __fmul_rn(dl, __fadd_rn(q, of));
    }
}

int pymo_broadcast(const BroadcastArgs& a, cudaStream_t st)
{
    if (a.n == 0)
        return AQ_OK;
    int64_t blocks = (a.n + kThreads - 1) / kThreads;
    int64_t cap    = (int64_t) kNumSMs * 8 * 4;
    pymo_broadcast_kernel<<<(unsigned) (blocks < cap ? blocks : cap), kThreads, 0, st>>>(a);
    note_launch();
    return check_launch();
}

// -------------------------------------------------------------------------------------------------
// v2-semantics quantize / quantize-dequantize (+ optional clamp mask) and dequantize
// -------------------------------------------------------------------------------------------------
template <typename T, int VEC, bool PER_CH, bool NARROW>
__global__ void __launch_bounds__(kThreads) v2_kernel(V2Args a)
{
    constexpr int CHUNK = chunk_elems<VEC>();
    const int64_t base  = (int64_t) blockIdx.x * CHUNK;
    V2Op op;
    op.scale = a.scale, op.offset = a.offset, op.qmin = a.qmin, op.qmax = a.qmax;
    op.out_kind = a.out_kind, op.dequant_only = a.dequant_only;
    __shared__ V2Op::Slot s_slot[PER_CH ? kMaxRuns : 1];
    RunCtx rc {0, 0, 1};
    V2Op::Slot k0;
    if (PER_CH)
    {
        rc = make_run_ctx<VEC>(a.geom, base, a.n);
        for (int lr = threadIdx.x; lr < rc.nruns; lr += kThreads)
            s_slot[lr] = op.load((rc.r0 + lr) % a.geom.num_ch);
        __syncthreads();
    }
    else
        k0 = op.scalar_slot();

    Pack<T, VEC> v[kUnroll];
    bool full[kUnroll];
    load_chunk<T, VEC>(static_cast<const T*>(a.x), base, a.n, v, full);
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
    {
        const uint32_t off = (uint32_t) (u * kThreads + threadIdx.x) * VEC;
        const int64_t idx  = base + off;
        V2Op::Slot k       = k0;
        if (PER_CH)
            k = s_slot[run_of(a.geom, rc, off)];
        Pack<uint8_t, VEC> m;
#pragma unroll
        for (int e = 0; e < VEC; ++e)
        {
            bool in_range;
            const float r = op.apply_t<T, NARROW>(to_f32<T>(v[u].v[e]), k, in_range);
            v[u].v[e]     = from_f32<T>(r);
            m.v[e]        = in_range ? 1 : 0;
        }
        store_packet<T, VEC>(static_cast<T*>(a.y), idx, a.n, v[u], full[u]);
        if (a.mask)
            store_packet<uint8_t, VEC>(a.mask, idx, a.n, m, full[u]);
    }
}

template <typename T, bool PER_CH, bool NARROW>
static int launch_v2_vec(V2Args a, int vec, cudaStream_t st)
{
#define AQ_LAUNCH(V)                                                                                                 \
    {                                                                                                                \
        a.geom       = make_geom(a.geom.num_ch, a.geom.inner, chunk_elems<V>());                                     \
        int64_t grid = (a.n + chunk_elems<V>() - 1) / chunk_elems<V>();                                              \
        v2_kernel<T, V, PER_CH, NARROW><<<(unsigned) grid, kThreads, 0, st>>>(a);                                    \
    }
    if (sizeof(T) == 2 && vec == 8)
        AQ_LAUNCH((sizeof(T) == 2 ? 8 : 4))
    else if (vec == 4)
        AQ_LAUNCH(4)
    else if (vec == 2)
        AQ_LAUNCH(2)
    else
        AQ_LAUNCH(1)
#undef AQ_LAUNCH
    note_launch();
    return check_launch();
}

template <typename T, bool NARROW>
static int launch_v2_t(V2Args a, cudaStream_t st)
{
    const bool per_ch = a.geom.num_ch > 1;
    // the mask is written with VEC-byte packets, so it constrains the width like the tensors do
    int vec = pick_vec<T>(a.x, a.y, nullptr, per_ch ? a.geom.inner : 0);
    while (vec > 1 && a.mask && ((uintptr_t) a.mask % vec))
        vec >>= 1;
    if (per_ch)
        return launch_v2_vec<T, true, NARROW>(a, vec, st);
    return launch_v2_vec<T, false, NARROW>(a, vec, st);
}

int v2_launch(V2Args a, int dtype, int narrow_internal, cudaStream_t st)
{
    if (a.n == 0)
        return AQ_OK;
    switch (dtype)
    {
    case AQ_F32: return launch_v2_t<float, false>(a, st);
    case AQ_BF16:
        return narrow_internal ? launch_v2_t<__nv_bfloat16, true>(a, st) : launch_v2_t<__nv_bfloat16, false>(a, st);
    case AQ_F16: return narrow_internal ? launch_v2_t<__half, true>(a, st) : launch_v2_t<__half, false>(a, st);
    default: return AQ_ERR_INVALID_ARG;
    }
}

// -------------------------------------------------------------------------------------------------
// Backward kernels
// -------------------------------------------------------------------------------------------------

// v2: dx = grad * mask  (torch_builtins.py:342)
template <typename T, int VEC>
__global__ void __launch_bounds__(kThreads) v2_bwd_kernel(const T* __restrict__ g, const uint8_t* __restrict__ mask,
                                                          T* __restrict__ dx, int64_t n)
{
    constexpr int CHUNK = chunk_elems<VEC>();
    const int64_t base  = (int64_t) blockIdx.x * CHUNK;
    Pack<T, VEC> v[kUnroll];
    Pack<uint8_t, VEC> m[kUnroll];
    bool full[kUnroll];
    load_chunk<T, VEC>(g, base, n, v, full);
    load_chunk<uint8_t, VEC>(mask, base, n, m, full);
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
    {
        const int64_t idx = base + (int64_t) (u * kThreads + threadIdx.x) * VEC;
#pragma unroll
        for (int e = 0; e < VEC; ++e)
        {
            // grad * bool: x*1 and x*0 are exact in any dtype (-0 and NaN behave as in the reference product)
            const float p = __fmul_rn(to_f32<T>(v[u].v[e]), m[u].v[e] ? 1.0f : 0.0f);
            v[u].v[e]     = from_f32<T>(p);
        }
        store_packet<T, VEC>(dx, idx, n, v[u], full[u]);
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
        int64_t grid = (n + chunk_elems<V>() - 1) / chunk_elems<V>();                                                \
        v2_bwd_kernel<T, V><<<(unsigned) grid, kThreads, 0, st>>>((const T*) g, mask, (T*) dx, n);                    \
    }
    if (sizeof(T) == 2 && vec == 8)
        AQ_LAUNCH((sizeof(T) == 2 ? 8 : 4))
    else if (vec == 4)
        AQ_LAUNCH(4)
    else if (vec == 2)
        AQ_LAUNCH(2)
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

// v2 encoding gradients, element-wise and un-reduced exactly like the reference (autograd sums the broadcast
// dimensions afterwards), torch_builtins.py:334-343:
//   ds = g * (clamp(round(x/s), o + qmin, o + qmax) - (x/s) * mask)      do = g * ((1 - mask) * s)
template <typename T, int VEC, bool PER_CH>
__global__ void __launch_bounds__(kThreads) v2_param_grad_kernel(V2GradArgs a)
{
    constexpr int CHUNK = chunk_elems<VEC>();
    const int64_t base  = (int64_t) blockIdx.x * CHUNK;
    __shared__ float s_sc[PER_CH ? kMaxRuns : 1], s_of[PER_CH ? kMaxRuns : 1];
    RunCtx rc {0, 0, 1};
    float sc0 = 0.f, of0 = 0.f;
    if (PER_CH)
    {
        rc = make_run_ctx<VEC>(a.geom, base, a.n);
        for (int lr = threadIdx.x; lr < rc.nruns; lr += kThreads)
        {
            const int64_t ch = (rc.r0 + lr) % a.geom.num_ch;
            s_sc[lr]         = a.scale[ch];
            s_of[lr]         = a.offset[ch];
        }
        __syncthreads();
    }
    else
    {
        sc0 = __ldg(a.scale);
        of0 = __ldg(a.offset);
    }
    Pack<T, VEC> xv[kUnroll], gv[kUnroll];
    Pack<uint8_t, VEC> mv[kUnroll];
    bool full[kUnroll];
    load_chunk<T, VEC>(static_cast<const T*>(a.x), base, a.n, xv, full);
    load_chunk<T, VEC>(static_cast<const T*>(a.grad), base, a.n, gv, full);
    load_chunk<uint8_t, VEC>(a.mask, base, a.n, mv, full);
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
    {
        const uint32_t off = (uint32_t) (u * kThreads + threadIdx.x) * VEC;
        const int64_t idx  = base + off;
        float sc = sc0, of = of0;
        if (PER_CH)
        {
            const uint32_t lr = run_of(a.geom, rc, off);
            sc = s_sc[lr], of = s_of[lr];
        }
        const float lo = __fadd_rn(of, a.qmin), hi = __fadd_rn(of, a.qmax);
        Pack<float, VEC> ds, dof;
#pragma unroll
        for (int e = 0; e < VEC; ++e)
        {
            const float g = to_f32<T>(gv[u].v[e]);
            const float m = mv[u].v[e] ? 1.0f : 0.0f;
            const float t = __fdiv_rn(to_f32<T>(xv[u].v[e]), sc);
            float c       = rintf(t);
            asm("max.NaN.f32 %0, %1, %2;" : "=f"(c) : "f"(c), "f"(lo));
            asm("min.NaN.f32 %0, %1, %2;" : "=f"(c) : "f"(c), "f"(hi));
            ds.v[e]  = __fmul_rn(g, __fsub_rn(c, __fmul_rn(t, m)));
            dof.v[e] = __fmul_rn(g, __fmul_rn(1.0f - m, sc));
        }
        if (a.dscale)
            store_packet<float, VEC>(a.dscale, idx, a.n, ds, full[u]);
        if (a.doffset)
            store_packet<float, VEC>(a.doffset, idx, a.n, dof, full[u]);
    }
}

template <typename T>
static int launch_param_grad(V2GradArgs a, cudaStream_t st)
{
    const bool per_ch = a.geom.num_ch > 1;
    int vec           = pick_vec<T>(a.x, a.grad, nullptr, per_ch ? a.geom.inner : 0);
    if (vec > 4)
        vec = 4;   // fp32 outputs: 4 elements = 16 bytes
    while (vec > 1 && (((uintptr_t) a.mask % vec) || ((uintptr_t) a.dscale % (4 * vec)) ||
                       ((uintptr_t) a.doffset % (4 * vec))))
        vec >>= 1;
#define AQ_LAUNCH(V, PC)                                                                                             \
    {                                                                                                                \
        a.geom       = make_geom(a.geom.num_ch, a.geom.inner, chunk_elems<V>());                                     \
        int64_t grid = (a.n + chunk_elems<V>() - 1) / chunk_elems<V>();                                              \
        v2_param_grad_kernel<T, V, PC><<<(unsigned) grid, kThreads, 0, st>>>(a);                                     \
    }
    if (per_ch)
    {
        if (vec == 4)
            AQ_LAUNCH(4, true)
        else if (vec == 2)
            AQ_LAUNCH(2, true)
        else
            AQ_LAUNCH(1, true)
    }
    else
    {
        if (vec == 4)
            AQ_LAUNCH(4, false)
        else if (vec == 2)
            AQ_LAUNCH(2, false)
        else
            AQ_LAUNCH(1, false)
    }
#undef AQ_LAUNCH
    note_launch();
    return check_launch();
}

int v2_param_grad(V2GradArgs a, int dtype, cudaStream_t st)
{
    if (a.n == 0)
        return AQ_OK;
    switch (dtype)
    {
    case AQ_F32: return launch_param_grad<float>(a, st);
    case AQ_F16: return launch_param_grad<__half>(a, st);
    case AQ_BF16: return launch_param_grad<__nv_bfloat16>(a, st);
    default: return AQ_ERR_INVALID_ARG;
    }
}

// v1: dx = g * [enc_min <= x <= enc_max], mask recomputed from the saved input
// (aimet_torch/v1/quantsim_straight_through_grad.py:91-118)
template <int VEC, bool PER_CH>
__global__ void __launch_bounds__(kThreads) ste_v1_kernel(SteArgs a)
{
    constexpr int CHUNK = chunk_elems<VEC>();
    const int64_t base  = (int64_t) blockIdx.x * CHUNK;
    __shared__ float s_mn[PER_CH ? kMaxRuns : 1], s_mx[PER_CH ? kMaxRuns : 1];
    RunCtx rc {0, 0, 1};
    float mn0 = 0.f, mx0 = 0.f;
    if (PER_CH)
    {
        rc = make_run_ctx<VEC>(a.geom, base, a.n);
        for (int lr = threadIdx.x; lr < rc.nruns; lr += kThreads)
        {
            const int64_t ch = (rc.r0 + lr) % a.geom.num_ch;
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
    Pack<float, VEC> xv[kUnroll], gv[kUnroll];
    bool full[kUnroll];
    load_chunk<float, VEC>(a.x, base, a.n, xv, full);
    load_chunk<float, VEC>(a.g, base, a.n, gv, full);
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
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
        a.geom       = make_geom(a.geom.num_ch, a.geom.inner, chunk_elems<V>());                                     \
        int64_t grid = (a.n + chunk_elems<V>() - 1) / chunk_elems<V>();                                              \
        ste_v1_kernel<V, PC><<<(unsigned) grid, kThreads, 0, st>>>(a);                                               \
    }
    if (per_ch)
    {
        if (vec == 4)
            AQ_LAUNCH(4, true)
        else if (vec == 2)
            AQ_LAUNCH(2, true)
        else
            AQ_LAUNCH(1, true)
    }
    else
    {
        if (vec == 4)
            AQ_LAUNCH(4, false)
        else if (vec == 2)
            AQ_LAUNCH(2, false)
        else
            AQ_LAUNCH(1, false)
    }
#undef AQ_LAUNCH
    note_launch();
    return check_launch();
}

}   // namespace aq
