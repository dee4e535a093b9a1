// Fake-quant element kernels for sm_100a: quantize-dequantize / quantize / dequantize forward and the
// straight-through backward, at per-tensor, per-channel and blockwise granularity.
//
// All kernels are HBM-bound streaming kernels: one CTA owns one contiguous chunk of
// THREADS * VEC * UNROLL elements, every thread issues UNROLL independent 16-byte (VEC-wide) loads before
// it computes, and per-channel / per-block encodings of the chunk are staged once in shared memory.
// Arithmetic is IEEE: correctly rounded division, no FMA contraction (the file is compiled with -fmad=false),
// because results must match the CPU reference bit for bit.
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

// -------------------------------------------------------------------------------------------------
// Element arithmetic
// -------------------------------------------------------------------------------------------------

// libpymo: quantizeValueCpu + dequantizeValueCpu (DlQuantization/src/trim_functions.cpp:140-171).
__device__ __forceinline__ float pymo_code(float x, float mn, float mx, float delta, float offset)
{
    float t = fmaxf(fminf(x, mx), mn);
    t       = __fsub_rn(__fdiv_rn(t, delta), offset);
    return round_half_away(t);
}
__device__ __forceinline__ float pymo_dequant(float q, float delta, float offset)
{
    return __fmul_rn(delta, __fadd_rn(q, offset));
}

__device__ __forceinline__ float round_f16(float v)
{
    return __half2float(__float2half_rn(v));
}

// v2: torch_builtins.py:303-313.  Returns the code (or the dequantized value) and the in-range flag.
template <bool HALF_INTERNAL>
__device__ __forceinline__ float v2_element(float x, float s, float o, float qmin, float qmax, int out_kind,
                                            bool& in_range)
{
    float r = __fdiv_rn(x, s);
    if (HALF_INTERNAL)
        r = round_f16(r);
    r = rintf(r);   // half to even; exact in fp16 too
    r = __fsub_rn(r, o);
    if (HALF_INTERNAL)
        r = round_f16(r);
    in_range = (qmin <= r) && (r <= qmax);
    // torch.clamp keeps NaN
    float q = r < qmin ? qmin : (r > qmax ? qmax : r);
    if (out_kind == AQ_V2_OUT_CODES)
        return q;
    float y = __fadd_rn(q, o);
    if (HALF_INTERNAL)
        y = round_f16(y);
    y = __fmul_rn(y, s);
    return y;
}

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
    c.r0             = base / g.inner;
    c.loc0           = base - c.r0 * g.inner;
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

// -------------------------------------------------------------------------------------------------
// libpymo-semantics QDQ / quantize-to-codes
// -------------------------------------------------------------------------------------------------
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
    float shift;       // subtracted from codes (quantize only)
    int codes_only;    // 1: emit integer codes, 0: quantize-dequantize
    ChanGeom geom;
};

template <int VEC, bool PER_CH>
__global__ void __launch_bounds__(kThreads) pymo_qdq_kernel(PymoArgs a)
{
    constexpr int CHUNK = chunk_elems<VEC>();
    const int64_t base  = (int64_t) blockIdx.x * CHUNK;
    __shared__ float s_mn[PER_CH ? kMaxRuns : 1], s_mx[PER_CH ? kMaxRuns : 1], s_dl[PER_CH ? kMaxRuns : 1],
        s_of[PER_CH ? kMaxRuns : 1];
    RunCtx rc {0, 0, 1};
    if (PER_CH)
    {
        rc = make_run_ctx<VEC>(a.geom, base, a.n);
        for (int lr = threadIdx.x; lr < rc.nruns; lr += kThreads)
        {
            const int64_t ch = (rc.r0 + lr) % a.geom.num_ch;
            float mn = a.enc_min[ch], mx = a.enc_max[ch], dl, of;
            if (a.derive)
            {
                // AimetTensorQuantizer.cpp:236-254: gate, delta, offset in fp32 (offset: half to even)
                mn = mn < 0.0f ? mn : 0.0f;
                mx = mx > 0.0f ? mx : 0.0f;
                float lo = __fadd_rn(mn, 1e-5f);
                mx       = mx > lo ? mx : lo;
                dl       = __fdiv_rn(__fsub_rn(mx, mn), a.num_steps);
                of       = rintf(__fdiv_rn(mn, dl));
            }
            else
            {
                dl = a.enc_delta[ch];
                of = a.enc_offset[ch];
            }
            s_mn[lr] = mn, s_mx[lr] = mx, s_dl[lr] = dl, s_of[lr] = of;
        }
        __syncthreads();
    }

    Pack<float, VEC> v[kUnroll];
    bool full[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
    {
        const int64_t idx = base + (int64_t) (u * kThreads + threadIdx.x) * VEC;
        full[u]           = idx + VEC <= a.n;
        if (full[u])
            v[u] = load_pack<float, VEC>(a.in + idx);
        else
        {
#pragma unroll
            for (int e = 0; e < VEC; ++e)
                v[u].v[e] = (idx + e < a.n) ? a.in[idx + e] : 0.0f;
        }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
    {
        const uint32_t off = (uint32_t) (u * kThreads + threadIdx.x) * VEC;
        const int64_t idx  = base + off;
        float mn = a.mn, mx = a.mx, dl = a.delta, of = a.offset;
        if (PER_CH)
        {
            const uint32_t lr = run_of(a.geom, rc, off);   // VEC | inner: one run per packet
            mn = s_mn[lr], mx = s_mx[lr], dl = s_dl[lr], of = s_of[lr];
        }
#pragma unroll
        for (int e = 0; e < VEC; ++e)
        {
            float q   = pymo_code(v[u].v[e], mn, mx, dl, of);
            v[u].v[e] = a.codes_only ? __fsub_rn(q, a.shift) : pymo_dequant(q, dl, of);
        }
        if (full[u])
            store_pack<float, VEC>(a.out + idx, v[u]);
        else
        {
#pragma unroll
            for (int e = 0; e < VEC; ++e)
                if (idx + e < a.n)
                    a.out[idx + e] = v[u].v[e];
        }
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
    a.mn = mn, a.mx = mx, a.delta = delta, a.offset = offset;
    a.codes_only = codes_only, a.shift = shift;
    a.geom.num_ch = 1, a.geom.inner = n > 0 ? n : 1;
    return launch_pymo<false>(a, pick_vec<float>(in, out, nullptr, 0), st);
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
    return launch_pymo<true>(a, pick_vec<float>(in, out, nullptr, inner), st);
}

// -------------------------------------------------------------------------------------------------
// General broadcast QDQ (stride walk), libpymo semantics.  Rarely-used fallback for encodings that do not
// reduce to (i / inner) % num_ch; one element per thread per step.
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
        a.out[i] = pymo_dequant(pymo_code(a.in[i], a.mn[e], a.mx[e], dl, of), dl, of);
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

template <typename T, int VEC, bool PER_CH, bool HALF_INTERNAL>
__global__ void __launch_bounds__(kThreads) v2_kernel(V2Args a)
{
    constexpr int CHUNK = chunk_elems<VEC>();
    const int64_t base  = (int64_t) blockIdx.x * CHUNK;
    const T* __restrict__ x = static_cast<const T*>(a.x);
    T* __restrict__ y       = static_cast<T*>(a.y);
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

    Pack<T, VEC> v[kUnroll];
    bool full[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
    {
        const int64_t idx = base + (int64_t) (u * kThreads + threadIdx.x) * VEC;
        full[u]           = idx + VEC <= a.n;
        if (full[u])
            v[u] = load_pack<T, VEC>(x + idx);
        else
        {
#pragma unroll
            for (int e = 0; e < VEC; ++e)
                v[u].v[e] = (idx + e < a.n) ? x[idx + e] : from_f32<T>(0.0f);
        }
    }
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
        Pack<uint8_t, VEC> m;
#pragma unroll
        for (int e = 0; e < VEC; ++e)
        {
            const float xv = to_f32<T>(v[u].v[e]);
            float r;
            if (a.dequant_only)
            {
                // DequantizeFunc: (x + o) * s   (torch_builtins.py:264-266)
                r = __fadd_rn(xv, of);
                if (HALF_INTERNAL)
                    r = round_f16(r);
                r      = __fmul_rn(r, sc);
                m.v[e] = 1;
            }
            else
            {
                bool in_range;
                r      = v2_element<HALF_INTERNAL>(xv, sc, of, a.qmin, a.qmax, a.out_kind, in_range);
                m.v[e] = in_range ? 1 : 0;
            }
            v[u].v[e] = from_f32<T>(r);
        }
        if (full[u])
        {
            store_pack<T, VEC>(y + idx, v[u]);
            if (a.mask)
                store_pack<uint8_t, VEC>(a.mask + idx, m);
        }
        else
        {
#pragma unroll
            for (int e = 0; e < VEC; ++e)
                if (idx + e < a.n)
                {
                    y[idx + e] = v[u].v[e];
                    if (a.mask)
                        a.mask[idx + e] = m.v[e];
                }
        }
    }
}

template <typename T, bool PER_CH, bool HALF_INTERNAL>
static int launch_v2_vec(V2Args a, int vec, cudaStream_t st)
{
#define AQ_LAUNCH(V)                                                                                                 \
    {                                                                                                                \
        a.geom       = make_geom(a.geom.num_ch, a.geom.inner, chunk_elems<V>());                                     \
        int64_t grid = (a.n + chunk_elems<V>() - 1) / chunk_elems<V>();                                              \
        v2_kernel<T, V, PER_CH, HALF_INTERNAL><<<(unsigned) grid, kThreads, 0, st>>>(a);                             \
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

template <typename T, bool HALF_INTERNAL>
static int launch_v2_t(V2Args a, cudaStream_t st)
{
    const bool per_ch = a.geom.num_ch > 1;
    // the mask is written with VEC-byte packets, so it constrains the width like the tensors do
    int vec = pick_vec<T>(a.x, a.y, nullptr, per_ch ? a.geom.inner : 0);
    while (vec > 1 && a.mask && ((uintptr_t) a.mask % vec))
        vec >>= 1;
    if (per_ch)
        return launch_v2_vec<T, true, HALF_INTERNAL>(a, vec, st);
    return launch_v2_vec<T, false, HALF_INTERNAL>(a, vec, st);
}

int v2_launch(V2Args a, int dtype, int internal_f16, cudaStream_t st)
{
    if (a.n == 0)
        return AQ_OK;
    switch (dtype)
    {
    case AQ_F32: return launch_v2_t<float, false>(a, st);
    case AQ_BF16: return launch_v2_t<__nv_bfloat16, false>(a, st);
    case AQ_F16:
        return internal_f16 ? launch_v2_t<__half, true>(a, st) : launch_v2_t<__half, false>(a, st);
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
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
    {
        const int64_t idx = base + (int64_t) (u * kThreads + threadIdx.x) * VEC;
        full[u]           = idx + VEC <= n;
        if (full[u])
        {
            v[u] = load_pack<T, VEC>(g + idx);
            m[u] = load_pack<uint8_t, VEC>(mask + idx);
        }
        else
        {
#pragma unroll
            for (int e = 0; e < VEC; ++e)
            {
                v[u].v[e] = (idx + e < n) ? g[idx + e] : from_f32<T>(0.0f);
                m[u].v[e] = (idx + e < n) ? mask[idx + e] : 0;
            }
        }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
    {
        const int64_t idx = base + (int64_t) (u * kThreads + threadIdx.x) * VEC;
#pragma unroll
        for (int e = 0; e < VEC; ++e)
        {
            // grad * bool: the product in the tensor's own dtype (x*1 and x*0 are exact, NaN*0 stays NaN)
            const float p = __fmul_rn(to_f32<T>(v[u].v[e]), m[u].v[e] ? 1.0f : 0.0f);
            v[u].v[e]     = from_f32<T>(p);
        }
        if (full[u])
            store_pack<T, VEC>(dx + idx, v[u]);
        else
        {
#pragma unroll
            for (int e = 0; e < VEC; ++e)
                if (idx + e < n)
                    dx[idx + e] = v[u].v[e];
        }
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
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
    {
        const int64_t idx = base + (int64_t) (u * kThreads + threadIdx.x) * VEC;
        full[u]           = idx + VEC <= a.n;
        if (full[u])
        {
            xv[u] = load_pack<float, VEC>(a.x + idx);
            gv[u] = load_pack<float, VEC>(a.g + idx);
        }
        else
        {
#pragma unroll
            for (int e = 0; e < VEC; ++e)
            {
                xv[u].v[e] = (idx + e < a.n) ? a.x[idx + e] : 0.0f;
                gv[u].v[e] = (idx + e < a.n) ? a.g[idx + e] : 0.0f;
            }
        }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
    {
        const uint32_t off = (uint32_t) (u * kThreads + threadIdx.x) * VEC;
        const int64_t idx  = base + off;
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
        if (full[u])
            store_pack<float, VEC>(a.dx + idx, gv[u]);
        else
        {
#pragma unroll
            for (int e = 0; e < VEC; ++e)
                if (idx + e < a.n)
                    a.dx[idx + e] = gv[u].v[e];
        }
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
