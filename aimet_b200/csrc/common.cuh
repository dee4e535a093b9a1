// Shared device helpers for the aimet_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/aimet_b200.h"

namespace aq
{

constexpr int kNumSMs = 148;   // B200: 2 dies x 74 SMs

// ---- launch accounting / error capture (defined in capi.cu) -----------------------------------
void note_launch();
int check_launch();                 // cudaGetLastError -> AQ_OK / AQ_ERR_CUDA
int cuda_fail(cudaError_t e);       // records the text, returns AQ_ERR_CUDA

// ---- programmatic dependent launch -------------------------------------------------------------------------
// Back-to-back launches of these short kernels (8-12 us of DRAM time each) lose 2-3 us per launch to the gap between
// the end of one grid and the start of the next.  Kernels launched through launch_pdl() may be scheduled while the
// previous grid of the stream is still draining: every kernel first tells the scheduler that its dependents may
// launch (pdl_launch_dependents), does whatever needs no global input (shared-memory setup), and only then waits
// for the previous grid to complete and flush (pdl_wait) -- so data dependencies through global memory are kept.
// Both instructions are no-ops in a grid that was launched normally.
__device__ __forceinline__ void pdl_launch_dependents()
{
    asm volatile("griddepcontrol.launch_dependents;");
}
__device__ __forceinline__ void pdl_wait()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

bool pdl_enabled();   // capi.cu: false when AQ_NO_PDL is set in the environment

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, unsigned block, size_t smem, cudaStream_t st,
                              Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim            = grid;
    cfg.blockDim           = dim3(block, 1, 1);
    cfg.dynamicSmemBytes   = smem;
    cfg.stream             = st;
    cudaLaunchAttribute attr[1];
    attr[0].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs                                          = attr;
    cfg.numAttrs                                       = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// ---- storage <-> fp32 ---------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v)
{
    return v;
}
template <>
__device__ __forceinline__ float to_f32<__half>(__half v)
{
    return __half2float(v);
}
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v)
{
    return __bfloat162float(v);
}

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v)
{
    return v;
}
template <>
__device__ __forceinline__ __half from_f32<__half>(float v)
{
    return __float2half_rn(v);
}
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v)
{
    return __float2bfloat16_rn(v);
}

// ---- VEC-wide packets: one aligned load / store instruction of up to 16 bytes -------------------
template <typename T, int VEC>
struct alignas(sizeof(T) * VEC) Pack
{
    T v[VEC];
};

template <typename T, int VEC>
__device__ __forceinline__ Pack<T, VEC> load_pack(const T* p)
{
    return *reinterpret_cast<const Pack<T, VEC>*>(p);
}
template <typename T, int VEC>
__device__ __forceinline__ void store_pack(T* p, const Pack<T, VEC>& v)
{
    *reinterpret_cast<Pack<T, VEC>*>(p) = v;
}

// Largest power-of-two vector width (in elements, <= 16 bytes) that both the pointers' alignment and a
// divisibility constraint `multiple_of` allow.
template <typename T>
inline int pick_vec(const void* a, const void* b, const void* c, int64_t multiple_of)
{
    int vec = 16 / (int) sizeof(T);
    auto ok = [&](int v) {
        const uintptr_t bytes = (uintptr_t) v * sizeof(T);
        if (a && ((uintptr_t) a % bytes))
            return false;
        if (b && ((uintptr_t) b % bytes))
            return false;
        if (c && ((uintptr_t) c % bytes))
            return false;
        if (multiple_of > 0 && (multiple_of % v))
            return false;
        return true;
    };
    while (vec > 1 && !ok(vec))
        vec >>= 1;
    return vec;
}

// ---- exact rounding helpers -------------------------------------------------------------------
// C roundf(): nearest, ties away from zero.  t - trunc(t) is exact, so the tie test is exact.
__device__ __forceinline__ float round_half_away(float t)
{
    float r = truncf(t);
    float d = t - r;
    if (fabsf(d) >= 0.5f)
        r += copysignf(1.0f, t);
    return r;
}

// ---- channel geometry ---------------------------------------------------------------------------
// Element i of a contiguous tensor belongs to encoding channel (i / inner) % num_ch.
// A CTA covers a contiguous chunk, so it meets at most chunk/inner + 2 consecutive "runs" of `inner` elements;
// their parameters are staged in shared memory and a run is found with one 32-bit multiply-high.
struct ChanGeom
{
    int64_t inner;
    int64_t num_ch;
    uint32_t magic;   // ceil(2^32 / inner) when 1 < inner < 2^16, else 0
    int mode;         // 0: inner == 1 (run = local offset), 1: magic multiply, 2: inner so large that a chunk
                      //    meets at most two runs (compare)
    // exact division of a 32-bit value by inner / num_ch with one 64-bit multiply-high: ceil(2^64 / d) for d > 1
    // (0 stands for d == 1).  Only used when the tensor has fewer than 2^32 elements (`small`).
    uint64_t inner_m64, ch_m64;
    int small;
    int wraps;   // 0 when every run is its own channel (n / inner <= num_ch), so that channel == run
};

inline uint64_t magic64(int64_t d)
{
    if (d <= 1)
        return 0;
    const unsigned __int128 one = (unsigned __int128) 1 << 64;
    return (uint64_t) ((one + (unsigned __int128) d - 1) / (unsigned __int128) d);
}

inline ChanGeom make_geom(int64_t num_ch, int64_t inner, int64_t chunk, int64_t n = -1)
{
    ChanGeom g;
    g.inner  = inner;
    g.num_ch = num_ch;
    g.magic  = 0;
    if (inner == 1)
        g.mode = 0;
    else if (inner >= chunk)
        g.mode = 2;
    else
    {
        // local offsets are < inner + chunk <= 2*chunk <= 2^15 and inner < chunk <= 2^14, so
        // floor(loc/inner) == umulhi(loc, ceil(2^32/inner)) exactly (loc * inner < 2^32).
        g.mode  = 1;
        g.magic = (uint32_t) ((0x100000000ull + (uint64_t) inner - 1) / (uint64_t) inner);
    }
    g.small     = (n >= 0 && (uint64_t) n <= 0xffffffffull) ? 1 : 0;
    g.inner_m64 = magic64(inner);
    g.ch_m64    = magic64(num_ch);
    g.wraps     = (n < 0 || inner <= 0 || (n + inner - 1) / inner > num_ch) ? 1 : 0;
    return g;
}

// floor(v / d) for v < 2^32 and 1 <= d < 2^32, m = magic64(d): v * (m * d - 2^64) < 2^64 keeps the product's error
// below one step of 1 / d.
__device__ __forceinline__ uint32_t div_m64(uint32_t v, uint64_t m)
{
    return m ? (uint32_t) __umul64hi((uint64_t) v, m) : v;
}

// Run index of local offset `loc` (< inner + chunk) for modes 0 and 1.
__device__ __forceinline__ uint32_t local_run(const ChanGeom& g, uint32_t loc)
{
    return g.mode == 1 ? __umulhi(loc, g.magic) : loc;
}

// -------------------------------------------------------------------------------------------------
// Two fp32 lanes per instruction (sm_100 add/sub/mul.f32x2, round-to-nearest, no flush): the 16-bit kernels carry
// twice the elements per byte and are issue-bound with one lane per instruction.
// -------------------------------------------------------------------------------------------------
typedef unsigned long long f32x2_t;
__device__ __forceinline__ f32x2_t pair(float lo, float hi)
{
    f32x2_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpair(f32x2_t v, float& lo, float& hi)
{
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2_t mul2(f32x2_t a, f32x2_t b)
{
    f32x2_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2_t add2(f32x2_t a, f32x2_t b)
{
    f32x2_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2_t sub2(f32x2_t a, f32x2_t b)
{
    f32x2_t r;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2_t fma2(f32x2_t a, f32x2_t b, f32x2_t c)
{
    f32x2_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

}   // namespace aq
