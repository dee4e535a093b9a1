// Calibration statistics kernels for sm_100a: fused min/max reductions (per tensor / per channel / per block)
// and the 512-bucket TF-Enhanced histogram.  All are single-pass, HBM-bound streaming reads.
#include <float.h>
#include <stddef.h>

#include <atomic>
#include <type_traits>

#include "common.cuh"
#include "kernels.h"

namespace aq
{

// =================================================================================================
// min / max
// =================================================================================================

template <bool PROP>
__device__ __forceinline__ float min_op(float a, float b)
{
    if (PROP)
    {
        float r;
        asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
        return r;
    }
    return fminf(a, b);
}
template <bool PROP>
__device__ __forceinline__ float max_op(float a, float b)
{
    if (PROP)
    {
        float r;
        asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
        return r;
    }
    return fmaxf(a, b);
}

template <bool PROP, int WIDTH>
__device__ __forceinline__ void group_reduce(float& mn, float& mx)
{
#pragma unroll
    for (int o = WIDTH / 2; o > 0; o >>= 1)
    {
        mn = min_op<PROP>(mn, __shfl_xor_sync(0xffffffffu, mn, o, WIDTH));
        mx = max_op<PROP>(mx, __shfl_xor_sync(0xffffffffu, mx, o, WIDTH));
    }
}

// Folds one packet into (mn, mx).  16-bit packets are reduced two lanes per instruction in their own type first
// (min / max select one of their operands, so the type they run in cannot change the result).
template <typename T, int VEC, bool PROP>
__device__ __forceinline__ void fold_pack(const Pack<T, VEC>& v, float& mn, float& mx)
{
    if constexpr (sizeof(T) == 2 && VEC >= 4)
    {
        using T2     = typename std::conditional<std::is_same<T, __half>::value, __half2, __nv_bfloat162>::type;
        const T2* q  = reinterpret_cast<const T2*>(&v);
        T2 lo = q[0], hi = q[0];
#pragma unroll
        for (int e = 1; e < VEC / 2; ++e)
        {
            lo = PROP ? __hmin2_nan(lo, q[e]) : __hmin2(lo, q[e]);
            hi = PROP ? __hmax2_nan(hi, q[e]) : __hmax2(hi, q[e]);
        }
        mn = min_op<PROP>(mn, min_op<PROP>(to_f32<T>(lo.x), to_f32<T>(lo.y)));
        mx = max_op<PROP>(mx, max_op<PROP>(to_f32<T>(hi.x), to_f32<T>(hi.y)));
    }
    else
    {
#pragma unroll
        for (int e = 0; e < VEC; ++e)
        {
            const float f = to_f32<T>(v.v[e]);
            mn            = min_op<PROP>(mn, f);
            mx            = max_op<PROP>(mx, f);
        }
    }
}

static_assert(offsetof(aq_tfe_state_t, bucket_size) % 16 == 0 && offsetof(aq_tfe_state_t, pdf_offset) == offsetof(aq_tfe_state_t, bucket_size) + 4 &&
                  offsetof(aq_tfe_state_t, initialized) == offsetof(aq_tfe_state_t, bucket_size) + 8,
              "the histogram kernel reads bucket_size, pdf_offset and initialized with one 16-byte load");
constexpr int kMaxDevices = 64;   // per-device bookkeeping tables
constexpr int kMmThreads = 512;   // resident form, 4 CTAs per SM (large tensors)
constexpr int kMmMidThreads = 768;   // resident form, 2 CTAs per SM (medium tensors)
constexpr int kMmTileThreads = 256;   // one-tile-per-CTA form (small tensors)
constexpr int kMmUnroll  = 4;
constexpr int kTensorGridCap = 6 * kNumSMs;   // most CTAs (= partials) a whole-tensor reduction ever uses
constexpr int64_t kMmMidBytes = 96ll << 20;   // largest input the 2-CTA-per-SM resident form takes

// ---- whole-tensor reduction: warp shuffles, last CTA folds the partials ------------------------------------
// workspace layout: [0] uint32 ticket counter (must be 0 on entry; the kernel leaves it 0),
//                   [64 ...) float2 partials, one per CTA.
// Every thread sweeps packets p, p + stride, ...; kMmUnroll of them are in flight at once and the last, partial
// group is issued together as well (never one load at a time).  Small and medium tensors get one group per thread
// (grid = number of tiles, so the whole tensor is requested at once); large ones a resident grid that loops.
template <typename T, int VEC, bool PROP, int THREADS>
__global__ void __launch_bounds__(THREADS) minmax_tensor_kernel(const T* __restrict__ x, int64_t n,
                                                                float* __restrict__ out_min,
                                                                float* __restrict__ out_max,
                                                                unsigned int* __restrict__ ticket,
                                                                float2* __restrict__ partials, int accumulate)
{
    pdl_launch_dependents();
    pdl_wait();
    float mn = INFINITY, mx = -INFINITY;
    const int64_t npack  = n / VEC;
    const int64_t stride = (int64_t) gridDim.x * THREADS;
    int64_t p            = (int64_t) blockIdx.x * THREADS + threadIdx.x;
    for (; p + (kMmUnroll - 1) * stride < npack; p += kMmUnroll * stride)
    {
        Pack<T, VEC> v[kMmUnroll];
#pragma unroll
        for (int u = 0; u < kMmUnroll; ++u)
            v[u] = load_pack<T, VEC>(x + (p + u * stride) * VEC);
#pragma unroll
        for (int u = 0; u < kMmUnroll; ++u)
            fold_pack<T, VEC, PROP>(v[u], mn, mx);
    }
    {
        // partial group: up to kMmUnroll - 1 packets, all in flight together
        Pack<T, VEC> v[kMmUnroll - 1];
#pragma unroll
        for (int u = 0; u < kMmUnroll - 1; ++u)
            if (p + u * stride < npack)
                v[u] = load_pack<T, VEC>(x + (p + u * stride) * VEC);
#pragma unroll
        for (int u = 0; u < kMmUnroll - 1; ++u)
            if (p + u * stride < npack)
                fold_pack<T, VEC, PROP>(v[u], mn, mx);
    }
    // ragged tail (fewer than VEC elements)
    if (blockIdx.x == 0 && threadIdx.x < (int) (n - npack * VEC))
    {
        const float f = to_f32<T>(x[npack * VEC + threadIdx.x]);
        mn            = min_op<PROP>(mn, f);
        mx            = max_op<PROP>(mx, f);
    }

    group_reduce<PROP, 32>(mn, mx);
    __shared__ float s_mn[THREADS / 32], s_mx[THREADS / 32];
    __shared__ bool s_last;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0)
        s_mn[warp] = mn, s_mx[warp] = mx;
    __syncthreads();
    if (warp == 0)
    {
        mn = lane < THREADS / 32 ? s_mn[lane] : INFINITY;
        mx = lane < THREADS / 32 ? s_mx[lane] : -INFINITY;
        group_reduce<PROP, 32>(mn, mx);
        if (lane == 0)
        {
            partials[blockIdx.x] = make_float2(mn, mx);
            __threadfence();
            const unsigned int t = atomicAdd(ticket, 1u);
            s_last               = (t == gridDim.x - 1);
        }
    }
    __syncthreads();
    if (!s_last)
        return;
    __threadfence();
    mn = INFINITY, mx = -INFINITY;
    for (int i = threadIdx.x; i < (int) gridDim.x; i += THREADS)
    {
        const float2 q = __ldcg(&partials[i]);
        mn             = min_op<PROP>(mn, q.x);
        mx             = max_op<PROP>(mx, q.y);
    }
    group_reduce<PROP, 32>(mn, mx);
    __syncthreads();
    if (lane == 0)
        s_mn[warp] = mn, s_mx[warp] = mx;
    __syncthreads();
    if (warp == 0)
    {
        mn = lane < THREADS / 32 ? s_mn[lane] : INFINITY;
        mx = lane < THREADS / 32 ? s_mx[lane] : -INFINITY;
        group_reduce<PROP, 32>(mn, mx);
        if (lane == 0)
        {
            if (PROP && (mn != mn || mx != mx))
                mn = mx = NAN;
            if (accumulate)
            {
                mn = min_op<PROP>(out_min[0], mn);
                mx = max_op<PROP>(out_max[0], mx);
            }
            out_min[0] = mn;
            out_max[0] = mx;
            *ticket    = 0;   // ready for the next call on this stream
        }
    }
}

// ---- rows: the tensor is R = n / inner contiguous rows; row r belongs to channel r % num_ch ----------------
// A group of GS lanes reduces one (row, segment) pair.  Results go to `part_*[row * nseg + seg]`.
template <typename T, int VEC, int GS, bool PROP>
__global__ void __launch_bounds__(256) minmax_rows_kernel(const T* __restrict__ x, int64_t rows, int64_t inner,
                                                          int nseg, int64_t seg_len /* elements, multiple of VEC */,
                                                          float* __restrict__ part_min, float* __restrict__ part_max,
                                                          int accumulate /* only with direct output */)
{
    pdl_launch_dependents();
    pdl_wait();
    const int lane_in_group  = threadIdx.x % GS;
    const int64_t group      = ((int64_t) blockIdx.x * 256 + threadIdx.x) / GS;
    const int64_t num_groups = (int64_t) gridDim.x * 256 / GS;
    const int64_t items      = rows * nseg;
    if (nseg == 1 && inner <= (int64_t) GS * VEC)
    {
        // Short rows (block scales, small kernels): one packet per lane covers a row, so the loads in flight come
        // from kMmUnroll different rows instead of from one row's sweep.
        const bool lane_has = (int64_t) (lane_in_group + 1) * VEC <= inner;
        for (int64_t it = group; it < rows; it += (int64_t) kMmUnroll * num_groups)
        {
            Pack<T, VEC> v[kMmUnroll];
#pragma unroll
            for (int u = 0; u < kMmUnroll; ++u)
            {
                const int64_t r = it + u * num_groups;
                if (r < rows && lane_has)
                    v[u] = load_pack<T, VEC>(x + r * inner + lane_in_group * VEC);
            }
#pragma unroll
            for (int u = 0; u < kMmUnroll; ++u)
            {
                const int64_t r = it + u * num_groups;
                float mn = INFINITY, mx = -INFINITY;
                if (r < rows && lane_has)
                    fold_pack<T, VEC, PROP>(v[u], mn, mx);
                group_reduce<PROP, GS>(mn, mx);
                if (r < rows && lane_in_group == 0)
                {
                    if (PROP && (mn != mn || mx != mx))
                        mn = mx = NAN;
                    if (accumulate)
                    {
                        mn = min_op<PROP>(part_min[r], mn);
                        mx = max_op<PROP>(part_max[r], mx);
                    }
                    part_min[r] = mn;
                    part_max[r] = mx;
                }
            }
        }
        return;
    }
    for (int64_t it = group; it < items; it += num_groups)
    {
        const int64_t row = it / nseg;
        const int seg     = (int) (it - row * nseg);
        const int64_t beg = (int64_t) seg * seg_len;
        int64_t end       = beg + seg_len;
        if (end > inner)
            end = inner;
        const T* __restrict__ rp = x + row * inner;
        float mn = INFINITY, mx = -INFINITY;
        int64_t e = beg + (int64_t) lane_in_group * VEC;
        for (; e + (int64_t) (kMmUnroll - 1) * GS * VEC + VEC <= end; e += (int64_t) kMmUnroll * GS * VEC)
        {
            Pack<T, VEC> v[kMmUnroll];
#pragma unroll
            for (int u = 0; u < kMmUnroll; ++u)
                v[u] = load_pack<T, VEC>(rp + e + (int64_t) u * GS * VEC);
#pragma unroll
            for (int u = 0; u < kMmUnroll; ++u)
                fold_pack<T, VEC, PROP>(v[u], mn, mx);
        }
        for (; e + VEC <= end; e += (int64_t) GS * VEC)
            fold_pack<T, VEC, PROP>(load_pack<T, VEC>(rp + e), mn, mx);
        // VEC divides inner and seg_len, so no ragged tail exists inside a row.
        group_reduce<PROP, GS>(mn, mx);
        if (lane_in_group == 0)
        {
            if (PROP && (mn != mn || mx != mx))
                mn = mx = NAN;
            if (accumulate)
            {
                mn = min_op<PROP>(part_min[it], mn);
                mx = max_op<PROP>(part_max[it], mx);
            }
            part_min[it] = mn;
            part_max[it] = mx;
        }
    }
}

// Folds partials [outer, num_ch, nseg] -> [num_ch].
template <bool PROP>
__global__ void __launch_bounds__(256) minmax_fold_kernel(const float* __restrict__ part_min,
                                                          const float* __restrict__ part_max, int64_t outer,
                                                          int64_t num_ch, int nseg, float* __restrict__ out_min,
                                                          float* __restrict__ out_max, int accumulate)
{
    pdl_launch_dependents();
    pdl_wait();
    const int64_t c = (int64_t) blockIdx.x * 256 + threadIdx.x;
    if (c >= num_ch)
        return;
    float mn = INFINITY, mx = -INFINITY;
    for (int64_t o = 0; o < outer; ++o)
        for (int s = 0; s < nseg; ++s)
        {
            const int64_t i = (o * num_ch + c) * nseg + s;
            mn              = min_op<PROP>(mn, part_min[i]);
            mx              = max_op<PROP>(mx, part_max[i]);
        }
    if (PROP && (mn != mn || mx != mx))
        mn = mx = NAN;
    if (accumulate)
    {
        mn = min_op<PROP>(out_min[c], mn);
        mx = max_op<PROP>(out_max[c], mx);
    }
    out_min[c] = mn;
    out_max[c] = mx;
}

// Empty tensor with several channels: every channel reports the identity of min / max.
__global__ void __launch_bounds__(256) minmax_fill_empty_kernel(float* __restrict__ out_min, float* __restrict__ out_max,
                                                                int64_t num_ch)
{
    pdl_launch_dependents();
    pdl_wait();
    for (int64_t c = (int64_t) blockIdx.x * 256 + threadIdx.x; c < num_ch; c += (int64_t) gridDim.x * 256)
    {
        out_min[c] = INFINITY;
        out_max[c] = -INFINITY;
    }
}

struct RowsPlan
{
    int64_t rows, outer;
    int nseg;
    int64_t seg_len;
    int gs;
    bool direct;   // partials ARE the outputs (outer == 1, nseg == 1)
};

static RowsPlan plan_rows(int64_t n, int64_t num_ch, int64_t inner, int vec)
{
    RowsPlan p;
    p.rows  = n / inner;
    p.outer = p.rows / num_ch;
    // lanes per row: enough to cover the row once with VEC-wide loads, capped at a warp
    int64_t packs = inner / vec;
    int gs        = 1;
    while (gs < 32 && gs < packs)
        gs <<= 1;
    p.gs = gs;
    // Split long rows only when there are too few of them to give every SM half its warps: a split costs a second
    // launch for the fold, which outweighs the better balance from about 90 MB down.
    const int64_t target_items = (int64_t) kNumSMs * 32;
    int nseg                   = 1;
    if (gs == 32 && p.rows < target_items)
    {
        int64_t want     = (target_items + p.rows - 1) / p.rows;
        int64_t max_segs = packs / (32 * kMmUnroll);   // keep >= one unrolled sweep per segment
        if (max_segs < 1)
            max_segs = 1;
        nseg = (int) (want < max_segs ? want : max_segs);
        if (nseg > 4096)
            nseg = 4096;
    }
    int64_t seg_len = (inner + nseg - 1) / nseg;
    seg_len         = (seg_len + vec - 1) / vec * vec;
    nseg            = (int) ((inner + seg_len - 1) / seg_len);
    p.nseg          = nseg;
    p.seg_len       = seg_len;
    p.direct        = (p.outer == 1 && nseg == 1);
    return p;
}

// Whole-tensor grid.  Every CTA ends by taking a ticket and waiting for the answer, and a CTA slot held through that
// round trip delays the CTA queued behind it, so the grid is always one that is resident at once:
//   tile form  -- one tile (kMmTileThreads x kMmUnroll packets) per CTA while those CTAs fit one wave;
//   mid form   -- 2 CTAs of kMmMidThreads per SM that loop (25.7 MB fp32: 7.8 us against 9.5 us for 1568 tiles);
//   large form -- 4 CTAs of kMmThreads per SM that loop.
enum MmForm { kMmTile = 0, kMmMid = 1, kMmLarge = 2 };
static int tensor_grid(int64_t n, int vec, int elem_bytes, MmForm& form)
{
    const int64_t per_tile = (int64_t) kMmTileThreads * vec * kMmUnroll;
    int64_t tiles          = (n + per_tile - 1) / per_tile;
    if (tiles < 1)
        tiles = 1;
    if (tiles <= kTensorGridCap)
    {
        form = kMmTile;
        return (int) tiles;
    }
    form = n * elem_bytes <= kMmMidBytes ? kMmMid : kMmLarge;
    return form == kMmMid ? kNumSMs * 2 : kNumSMs * 4;
}

template <typename T>
static int vec_for(const void* x, int64_t multiple_of)
{
    return pick_vec<T>(x, nullptr, nullptr, multiple_of);
}

static int dtype_vec(const void* x, int dtype, int64_t multiple_of)
{
    switch (dtype)
    {
    case AQ_F32: return vec_for<float>(x, multiple_of);
    case AQ_F16: return vec_for<__half>(x, multiple_of);
    case AQ_BF16: return vec_for<__nv_bfloat16>(x, multiple_of);
    default: return 0;
    }
}

int64_t minmax_workspace_bytes(int64_t n, int64_t num_ch, int64_t inner)
{
    if (num_ch <= 1)
        return 256 + (int64_t) kTensorGridCap * sizeof(float2);
    if (n / inner == 0)
        return 256;   // no rows: nothing to plan (the outputs are filled directly)
    // worst case over vector widths: vec = 1 gives the most segments
    int64_t worst = 0;
    for (int vec = 1; vec <= 8; vec <<= 1)
    {
        if (inner % vec)
            continue;
        RowsPlan p  = plan_rows(n, num_ch, inner, vec);
        int64_t b   = 2 * p.rows * p.nseg * (int64_t) sizeof(float);
        worst       = b > worst ? b : worst;
    }
    return worst + 256;
}

template <typename T, int VEC, bool PROP>
static void launch_rows_gs(const T* x, const RowsPlan& p, int64_t inner, float* pmin, float* pmax, int acc,
                           cudaStream_t st)
{
    const int64_t items     = p.rows * p.nseg;
    const int64_t per_block = 256 / p.gs;
    int64_t blocks          = (items + per_block - 1) / per_block;
    const int64_t cap       = (int64_t) kNumSMs * 6;   // one resident wave (6 CTAs of 256 threads per SM at 40 registers)
    if (blocks > cap)
        blocks = cap;
#define AQ_GS(G)                                                                                                     \
    case G:                                                                                                          \
        launch_pdl(minmax_rows_kernel<T, VEC, G, PROP>, (unsigned) blocks, 256, 0, st, x, p.rows, inner, p.nseg,     \
                   p.seg_len, pmin, pmax, acc);                                                                      \
        break;
    switch (p.gs)
    {
        AQ_GS(1)
        AQ_GS(2)
        AQ_GS(4)
        AQ_GS(8)
        AQ_GS(16)
    default:
        launch_pdl(minmax_rows_kernel<T, VEC, 32, PROP>, (unsigned) blocks, 256, 0, st, x, p.rows, inner, p.nseg,
                   p.seg_len, pmin, pmax, acc);
    }
#undef AQ_GS
    note_launch();
}

template <typename T, bool PROP>
static int minmax_t(const T* x, int64_t n, int64_t num_ch, int64_t inner, float* out_min, float* out_max,
                    int accumulate, void* ws, int64_t ws_bytes, cudaStream_t st)
{
    if (num_ch <= 1)
    {
        const int vec = vec_for<T>(x, 0);
        MmForm form;
        const int grid = tensor_grid(n, vec, (int) sizeof(T), form);
        if (ws_bytes < 256 + (int64_t) grid * (int64_t) sizeof(float2))
            return AQ_ERR_WORKSPACE;
        unsigned int* ticket = static_cast<unsigned int*>(ws);
        float2* partials     = reinterpret_cast<float2*>(static_cast<char*>(ws) + 256);
#define AQ_MM(V)                                                                                                     \
    if (form == kMmTile)                                                                                             \
        launch_pdl(minmax_tensor_kernel<T, V, PROP, kMmTileThreads>, (unsigned) grid, kMmTileThreads, 0, st, x, n,   \
                   out_min, out_max, ticket, partials, accumulate);                                                  \
    else if (form == kMmMid)                                                                                         \
        launch_pdl(minmax_tensor_kernel<T, V, PROP, kMmMidThreads>, (unsigned) grid, kMmMidThreads, 0, st, x, n,     \
                   out_min, out_max, ticket, partials, accumulate);                                                  \
    else                                                                                                             \
        launch_pdl(minmax_tensor_kernel<T, V, PROP, kMmThreads>, (unsigned) grid, kMmThreads, 0, st, x, n, out_min,  \
                   out_max, ticket, partials, accumulate);
        switch (vec)
        {
        case 8: AQ_MM((sizeof(T) == 2 ? 8 : 4)) break;
        case 4: AQ_MM(4) break;
        case 2: AQ_MM(2) break;
        default: AQ_MM(1)
        }
#undef AQ_MM
        note_launch();
        return check_launch();
    }
    if (n / inner == 0)
    {
        // no rows at all: min over nothing is +inf, max is -inf; running statistics stay as they are
        if (accumulate)
            return AQ_OK;
        int64_t blocks = (num_ch + 255) / 256;
        if (blocks > kNumSMs)
            blocks = kNumSMs;
        launch_pdl(minmax_fill_empty_kernel, (unsigned) blocks, 256, 0, st, out_min, out_max, num_ch);
        note_launch();
        return check_launch();
    }
    const int vec = vec_for<T>(x, inner);
    RowsPlan p    = plan_rows(n, num_ch, inner, vec);
    float *pmin = out_min, *pmax = out_max;
    if (!p.direct)
    {
        // the first 256 bytes hold the whole-tensor kernel's ticket counter and must stay untouched
        const int64_t need = 256 + 2 * p.rows * p.nseg * (int64_t) sizeof(float);
        if (ws_bytes < need)
            return AQ_ERR_WORKSPACE;
        pmin = reinterpret_cast<float*>(static_cast<char*>(ws) + 256);
        pmax = pmin + p.rows * p.nseg;
    }
    switch (vec)
    {
    case 8: launch_rows_gs<T, (sizeof(T) == 2 ? 8 : 4), PROP>(x, p, inner, pmin, pmax, p.direct ? accumulate : 0, st); break;
    case 4: launch_rows_gs<T, 4, PROP>(x, p, inner, pmin, pmax, p.direct ? accumulate : 0, st); break;
    case 2: launch_rows_gs<T, 2, PROP>(x, p, inner, pmin, pmax, p.direct ? accumulate : 0, st); break;
    default: launch_rows_gs<T, 1, PROP>(x, p, inner, pmin, pmax, p.direct ? accumulate : 0, st);
    }
    int rc = check_launch();
    if (rc != AQ_OK || p.direct)
        return rc;
    launch_pdl(minmax_fold_kernel<PROP>, (unsigned) ((num_ch + 255) / 256), 256, 0, st, (const float*) pmin,
               (const float*) pmax, p.outer, num_ch, p.nseg, out_min, out_max, accumulate);
    note_launch();
    return check_launch();
}

int minmax_dispatch(const void* x, int dtype, int64_t n, int64_t num_ch, int64_t inner, float* out_min,
                    float* out_max, int propagate_nan, int accumulate, void* ws, int64_t ws_bytes, cudaStream_t st)
{
#define AQ_T(T)                                                                                                      \
    (propagate_nan                                                                                                   \
         ? minmax_t<T, true>((const T*) x, n, num_ch, inner, out_min, out_max, accumulate, ws, ws_bytes, st)         \
         : minmax_t<T, false>((const T*) x, n, num_ch, inner, out_min, out_max, accumulate, ws, ws_bytes, st))
    switch (dtype)
    {
    case AQ_F32: return AQ_T(float);
    case AQ_F16: return AQ_T(__half);
    case AQ_BF16: return AQ_T(__nv_bfloat16);
    default: return AQ_ERR_INVALID_ARG;
    }
#undef AQ_T
}

// -------------------------------------------------------------------------------------------------
// Min/max without caller scratch.
//
// Some hosts of this library may not allocate device memory at the point where they need statistics: an
// inference runtime whose memory arena was sized and frozen at start-up, an operator callback that another
// framework runs with allocation disabled, or a process that has handed all device memory to a pool it does not
// own.  For them the reduction scratch lives in this fixed array inside the library image.  Every GPU that loads
// the library holds these bytes until the process exits; all calls on a device share them, so two calls that
// overlap on the GPU (different streams) race, and the array keeps whatever the previous call left behind.
// -------------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_minmax_static_scratch[AQ_MINMAX_STATIC_SCRATCH_BYTES];

// Scratch bytes the call would really touch (the public size query is a worst case over vector widths and always
// charges row partials; a plan whose rows are written straight to the outputs needs only the ticket area).
static int64_t minmax_scratch_need(const void* x, int dtype, int64_t n, int64_t num_ch, int64_t inner)
{
    if (num_ch <= 1)
    {
        MmForm form;
        return 256 + (int64_t) tensor_grid(n, dtype_vec(x, dtype, 0), dtype == AQ_F32 ? 4 : 2, form) * (int64_t) sizeof(float2);
    }
    if (n / inner == 0)
        return 256;
    const RowsPlan p = plan_rows(n, num_ch, inner, dtype_vec(x, dtype, inner));
    return p.direct ? 256 : 256 + 2 * p.rows * p.nseg * (int64_t) sizeof(float);
}

int minmax_static(const void* x, int dtype, int64_t n, int64_t num_ch, int64_t inner, float* out_min, float* out_max,
                  int propagate_nan, cudaStream_t st)
{
    if (minmax_scratch_need(x, dtype, n, num_ch, inner) > (int64_t) AQ_MINMAX_STATIC_SCRATCH_BYTES)
        return AQ_ERR_TOO_LARGE;
    // In host code the array's name is only a handle; the address the kernels need comes from the runtime, once per
    // device, with that device current.  Entries are written once with the same value by whichever thread gets there
    // first, so relaxed atomics are enough.
    static std::atomic<void*> scratch_of_device[kMaxDevices];
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess)
        return cuda_fail(e);
    if (dev < 0 || dev >= kMaxDevices)
        return AQ_ERR_UNSUPPORTED;
    void* scratch = scratch_of_device[dev].load(std::memory_order_relaxed);
    if (!scratch)
    {
        e = cudaGetSymbolAddress(&scratch, g_minmax_static_scratch);
        if (e != cudaSuccess)
            return cuda_fail(e);
        scratch_of_device[dev].store(scratch, std::memory_order_relaxed);
    }
    // The whole-tensor kernel expects its ticket counter (first 256 bytes) to be zero; nothing else has to be.
    e = cudaMemsetAsync(scratch, 0, 256, st);
    if (e != cudaSuccess)
        return cuda_fail(e);
    return minmax_dispatch(x, dtype, n, num_ch, inner, out_min, out_max, propagate_nan, 0, scratch,
                           (int64_t) AQ_MINMAX_STATIC_SCRATCH_BYTES, st);
}

// =================================================================================================
// TF-Enhanced: bucket grid, 512-bucket histogram, PDF replay
// =================================================================================================

// InitializePdf<float> + the geometry lines of UpdatePdf (DlQuantization/src/math_functions.cpp:207-268), run by the
// first AQ_PDF_SIZE threads of one CTA (all threads of the CTA must call it: it contains a barrier).  Leaves the
// state alone when it is initialised already or when the batch is all zeros (the reference waits for the next one).
__device__ __forceinline__ void tfe_grid_from_range(float mn, float mx, aq_tfe_state_t* __restrict__ st)
{
    if (st->initialized || (mn == 0.0f && mx == 0.0f))
        return;   // uniform over the CTA: both operands are the same for every thread
    if (mn == mx)
    {
        const float alt = __fadd_rn(mn, 0.01f);
        mx              = mx < alt ? alt : mx;
    }
    const float center = __fdiv_rn(__fadd_rn(mx, mn), 2.0f);
    float lo           = __fsub_rn(center, __fmul_rn(3.0f, __fsub_rn(center, mn)));
    float hi           = __fadd_rn(center, __fmul_rn(3.0f, __fsub_rn(mx, center)));
    lo                 = (-FLT_MAX < lo) ? lo : -FLT_MAX;
    hi                 = (hi < FLT_MAX) ? hi : FLT_MAX;
    const double bucket = __ddiv_rn(__dsub_rn((double) hi, (double) lo), (double) AQ_PDF_SIZE);
    const int i         = threadIdx.x;
    if (i < AQ_PDF_SIZE)
        st->x_left[i] = __dadd_rn((double) lo, __dmul_rn((double) i, bucket));
    __syncthreads();
    if (i == 0)
    {
        const double x0 = __dadd_rn((double) lo, __dmul_rn(0.0, bucket));
        const double x1 = __dadd_rn((double) lo, __dmul_rn(1.0, bucket));
        const float bs  = __double2float_rn(__dsub_rn(x1, x0));
        const float m0  = __double2float_rn(x0);
        st->bucket_size = bs;
        st->pdf_offset  = __fdiv_rn(m0, bs);
        __threadfence();
        st->initialized = 1;
    }
}

__global__ void __launch_bounds__(AQ_PDF_SIZE) tfe_init_grid_kernel(const float* __restrict__ minmax,
                                                                    aq_tfe_state_t* __restrict__ st)
{
    pdl_launch_dependents();
    pdl_wait();
    tfe_grid_from_range(minmax[0], minmax[1], st);
}

// ---- range of a batch, fused with the grid set-up -------------------------------------------------------------
// One launch does what the reference's first-batch branch of UpdatePdf does with GetMin + GetMax + InitializePdf:
// a single min/max pass over the batch, and the last CTA to finish builds the bucket grid from the result.  Once
// the state is initialised the launch returns at once (a few microseconds instead of a pass over the tensor), so a
// caller that does not yet KNOW on the host whether the grid exists can keep offering batches without waiting
// for the device.  With `range` the (min, max, 1.0f) triple of the batch is also written out -- (0, 0, 1) when the
// pass was skipped -- for callers that agree on the grid across ranks; `init` = 0 leaves the state alone.
// workspace layout as for minmax_tensor_kernel.
constexpr int kOfferThreads = 512;
__global__ void __launch_bounds__(kOfferThreads, 4) tfe_offer_grid_kernel(const float* __restrict__ x, int64_t n,
                                                                       aq_tfe_state_t* __restrict__ st,
                                                                       float* __restrict__ range, int init,
                                                                       unsigned int* __restrict__ ticket,
                                                                       float2* __restrict__ partials)
{
    pdl_launch_dependents();
    pdl_wait();
    if (st->initialized)
    {
        if (range && blockIdx.x == 0 && threadIdx.x == 0)
            range[0] = 0.0f, range[1] = 0.0f, range[2] = 1.0f;
        return;
    }
    float mn = INFINITY, mx = -INFINITY;
    const bool vec4      = ((uintptr_t) x % 16) == 0;
    const int64_t npack  = vec4 ? n / 4 : 0;
    const int64_t stride = (int64_t) gridDim.x * kOfferThreads;
    int64_t p            = (int64_t) blockIdx.x * kOfferThreads + threadIdx.x;
    for (; p + (kMmUnroll - 1) * stride < npack; p += kMmUnroll * stride)
    {
        Pack<float, 4> v[kMmUnroll];
#pragma unroll
        for (int u = 0; u < kMmUnroll; ++u)
            v[u] = load_pack<float, 4>(x + (p + u * stride) * 4);
#pragma unroll
        for (int u = 0; u < kMmUnroll; ++u)
            fold_pack<float, 4, false>(v[u], mn, mx);
    }
    {
        Pack<float, 4> v[kMmUnroll - 1];
#pragma unroll
        for (int u = 0; u < kMmUnroll - 1; ++u)
            if (p + u * stride < npack)
                v[u] = load_pack<float, 4>(x + (p + u * stride) * 4);
#pragma unroll
        for (int u = 0; u < kMmUnroll - 1; ++u)
            if (p + u * stride < npack)
                fold_pack<float, 4, false>(v[u], mn, mx);
    }
    // what the packets did not cover: the ragged tail, or everything when the base address is not 16-byte aligned
    for (int64_t i = npack * 4 + (int64_t) blockIdx.x * kOfferThreads + threadIdx.x; i < n; i += stride)
    {
        mn = fminf(mn, x[i]);
        mx = fmaxf(mx, x[i]);
    }
    group_reduce<false, 32>(mn, mx);
    __shared__ float s_mn[kOfferThreads / 32], s_mx[kOfferThreads / 32];
    __shared__ bool s_last;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0)
        s_mn[warp] = mn, s_mx[warp] = mx;
    __syncthreads();
    if (warp == 0)
    {
        mn = lane < kOfferThreads / 32 ? s_mn[lane] : INFINITY;
        mx = lane < kOfferThreads / 32 ? s_mx[lane] : -INFINITY;
        group_reduce<false, 32>(mn, mx);
        if (lane == 0)
        {
            partials[blockIdx.x] = make_float2(mn, mx);
            __threadfence();
            const unsigned int t = atomicAdd(ticket, 1u);
            s_last               = (t == gridDim.x - 1);
        }
    }
    __syncthreads();
    if (!s_last)
        return;
    __threadfence();
    mn = INFINITY, mx = -INFINITY;
    for (int i = threadIdx.x; i < (int) gridDim.x; i += kOfferThreads)
    {
        const float2 q = __ldcg(&partials[i]);
        mn             = fminf(mn, q.x);
        mx             = fmaxf(mx, q.y);
    }
    group_reduce<false, 32>(mn, mx);
    __syncthreads();
    if (lane == 0)
        s_mn[warp] = mn, s_mx[warp] = mx;
    __syncthreads();
    mn = INFINITY, mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < kOfferThreads / 32; ++w)   // every thread needs the result: the grid set-up is CTA-wide
    {
        mn = fminf(mn, s_mn[w]);
        mx = fmaxf(mx, s_mx[w]);
    }
    if (threadIdx.x == 0)
    {
        *ticket = 0;   // ready for the next call on this stream
        if (range)
            range[0] = mn, range[1] = mx, range[2] = 1.0f;
    }
    if (init)
        tfe_grid_from_range(mn, mx, st);
}

// Grid agreement across ranks, decided on the device: `ranges` holds one (min, max, present) triple per rank for the
// batches of one round (global order inside a round = rank order).  The first present batch whose (min, max) is
// not (0, 0) defines the grid (DlQuantization/src/math_functions.cpp:248-262).  `gate` tells this rank whether its own
// batch of the round counts: an all-zero batch that precedes the defining one was dropped by the sequential
// reference before the grid existed, so it must be dropped here too.
__global__ void __launch_bounds__(AQ_PDF_SIZE) tfe_select_grid_kernel(const float* __restrict__ ranges, int num_ranks,
                                                                      int rank, aq_tfe_state_t* __restrict__ st,
                                                                      int32_t* __restrict__ gate)
{
    pdl_launch_dependents();
    pdl_wait();
    if (st->initialized)
    {
        if (threadIdx.x == 0)
            *gate = 1;
        return;
    }
    int chosen = -1;
    for (int r = 0; r < num_ranks; ++r)
    {
        const float mn = ranges[3 * r], mx = ranges[3 * r + 1], present = ranges[3 * r + 2];
        if (present != 0.0f && !(mn == 0.0f && mx == 0.0f))
        {
            chosen = r;
            break;
        }
    }
    if (threadIdx.x == 0)
        *gate = (chosen >= 0 && rank >= chosen) ? 1 : 0;
    if (chosen >= 0)
        tfe_grid_from_range(ranges[3 * chosen], ranges[3 * chosen + 1], st);
}

// Bucket of one sample: (int) roundf(x / bucket_size - pdf_offset), valid when inside [0, 512).
// For t > -0.5 the half-away rounding equals floor(t + 0.5); adding with round-down keeps the sum from being
// rounded up across an integer, so floor() of it is exact.  NaN and t <= -0.5 fail the first test.
__device__ __forceinline__ bool bucket_of(float x, float bs, float po, int& k)
{
    const float t = __fsub_rn(__fdiv_rn(x, bs), po);
    k             = __float2int_rd(__fadd_rd(t, 0.5f));
    return (t > -0.5f) && ((unsigned) k < (unsigned) AQ_PDF_SIZE);
}

// ---- lane-private layout ------------------------------------------------------------------------------------
// counters[bucket][lane]: a lane only ever touches shared-memory bank `lane`, so one warp-wide atomic never has
// a bank conflict or a same-address collision, whatever the data looks like (post-ReLU spikes, a few hot
// buckets, ...).  Row 512 is a trash row for samples that fall outside the grid, which keeps the hot loop free
// of branches.  513 rows x 32 lanes x 4 B = 65,664 B per CTA; two persistent CTAs of 1024 threads per SM.
constexpr int kLaneHistThreads = 1024;
constexpr int kLaneHistRows    = AQ_PDF_SIZE + 1;
constexpr int kLaneHistBytes   = kLaneHistRows * 32 * (int) sizeof(uint32_t);
constexpr float kTwo23         = 8388608.0f;
constexpr uint32_t kTwo23Bits  = 0x4B000000u;

// Hot-loop bucket computation without a division and without conversion instructions.
//   s  = x * (1/bucket_size) + (1.5 - pdf_offset)      one FMA; approximates t + 1.5 with t = x/bs - po
//   s2 = RD(s + 2^23)                                   its low mantissa bits now hold floor(s)
//   g  = s - (s2 - (2^23 - 0.5))                        fractional part minus one half (both steps exact)
// The exact formula round_half_away(RN(RN(x/bs) - po)) changes value only where t + 1.5 crosses an integer, and
// |s - (t + 1.5)| < margin (see hist_margin), so when |g| < 0.5 - margin the bucket is floor(s) - 1 for certain.
// Everything else (near a boundary, NaN, Inf) is reported through `sure = false`; the caller takes that one
// sample back out of the counters and redoes it with the exact division formula.
// Returns the row to increment (512 = trash row for samples outside the grid).
__device__ __forceinline__ uint32_t bucket_row_fast(float x, float rbs, float c, float eps, bool& sure)
{
    const float s  = fmaf(x, rbs, c);
    const float s2 = __fadd_rd(s, kTwo23);
    const float g  = s - (s2 - 8388607.5f);
    sure           = fabsf(g) < eps;   // false for NaN
    return min(__float_as_uint(s2) - (kTwo23Bits + 1u), (uint32_t) AQ_PDF_SIZE);
}

// counters[row][lane] += 1 / -= 1 with a 32-bit shared-window address (one LEA + one RED per sample)
__device__ __forceinline__ void lane_hist_inc(uint32_t base, uint32_t row)
{
    asm volatile("red.shared.add.u32 [%0], 1;" ::"r"(base + (row << 7)));
}
__device__ __forceinline__ void lane_hist_dec(uint32_t base, uint32_t row)
{
    asm volatile("red.shared.add.s32 [%0], -1;" ::"r"(base + (row << 7)));
}

// Bound of |s - (t + 1.5)| for every sample whose approximate position s lies within [0, 515]:
//   exact path:  RN(x/bs) = q(1+e1),  t = (RN(x/bs) - po)(1+e2)
//   fast path:   rbs = (1/bs)(1+e3),  c = (1.5-po)(1+e4),  s = (x*rbs + c)(1+e5)          |e_i| <= 2^-24
//   => |s - (t+1.5)| <= 2^-24 (2|q| + |c| + |s| + |t|),  |q| <= |po| + 515,  |c| <= |po| + 1.5,  |s|,|t| <= 515
//   <= 2^-24 (3|po| + 2062); a quarter more is added for the second-order terms.
// Samples farther out cannot come back into the grid through this error as long as the margin stays below a
// quarter bucket, which the kernel checks.
__host__ __device__ inline float hist_margin(float po)
{
    return 1.25f * 5.9604644775390625e-08f /* 2^-24 */ * (3.0f * fabsf(po) + 2062.0f);
}

constexpr int kLaneUnroll = 4;

// Packets that held an unsure sample are not repaired inside the hot loop (any call or long branch body there
// costs registers that the two-CTAs-per-SM budget does not have); the index of their group goes to a small
// shared-memory queue and the CTA repairs them together after its sweep.  About one group of 16 samples in 170 is
// queued on ordinary data.
constexpr int kFixQueue        = 4096;
constexpr int kLaneHistSmem    = kLaneHistBytes + kFixQueue * (int) sizeof(uint32_t);

// Repair of one queued packet: re-read it (it has just passed through L2), take every unsure sample's fast-path count
// back out and count it with the exact formula instead.
__device__ __forceinline__ void hist_fix_packet(const float4* __restrict__ x4, uint32_t q, uint32_t base, float rbs,
                                                float c, float eps, float bs, float po)
{
    const float4 w   = __ldg(x4 + q);
    const float f[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int e = 0; e < 4; ++e)
    {
        bool sure;
        const uint32_t row = bucket_row_fast(f[e], rbs, c, eps, sure);
        if (!sure)
        {
            lane_hist_dec(base, row);
            int k;
            if (bucket_of(f[e], bs, po, k))
                lane_hist_inc(base, (uint32_t) k);
        }
    }
}

// Up to AQ_TFE_HIST_MANY batches per launch, each into its own row.  The launch overhead (about 1.3 us of the 13 us a
// 51 MB batch takes as a launch of its own) is paid once per launch, and -- with the work split described at the kernel
// -- so is most of the stop at the end of a sweep, measured with cycle stamps at 51 MB per batch: 1.35 us until the
// CTA's slowest warp arrives, 1.7 us to repair the ~30 queued packets (a dependent re-read), 1.0 us to fold (0.6 us
// with 128-bit shared loads), which the other CTA of the SM only partly covers.  16 batches per launch: 8.9 us per
// batch (0.90 of the copy bandwidth) against 12.8 us (0.62) for one batch per launch.
// Other forms that avoid the stop were built and measured slower: one CTA per SM with a dedicated fold warp and two
// counter sets (32 warps cannot keep the SM busy: 3.9 TB/s even without any atomics), repair in place from the
// registers or through a queue of sample values (both make the compiler spill inside the hot loop at 32 registers),
// counters shared by the CTA with per-set tickets instead of a barrier (same-address reductions cost nothing on this
// GPU, but the per-thread recount calls are slower than the joint repair), and repairing straight in the batch's
// global row so that the re-read runs under the fold and one barrier goes away (bit-identical, but the packet and
// flag kept across the fold cost the sweep its registers: 13.0 us per batch against 11.6 us; as a function that is
// not inlined, 13.3 us).
struct HistJob
{
    const float* x[AQ_TFE_HIST_MANY];
    int64_t n[AQ_TFE_HIST_MANY];
    int m;
    int64_t row_stride;   // rows between consecutive batches of the launch (1 = adjacent rows)
    uint32_t* hist;    // row of batch 0; batch b adds into hist + b * row_stride * 512
    int64_t* count;    // may be null; batch b sets count[b * row_stride]
    const int32_t* gate;   // may be null; *gate == 0 drops the batches (count 0, rows untouched)
    int slices;            // S: CTAs that share one batch (interleaved, 1024 packets at a time)
    int items;             // k: (batch, slice) pairs per CTA; m * S == k * gridDim.x
};

// A batch that does not start on a 16-byte boundary (a view into a larger buffer) has up to three leading elements
// before its first aligned packet; they are counted one by one like the ragged tail.
__device__ __forceinline__ int hist_lead(const float* x, int64_t n)
{
    return (int) min((int64_t) ((0u - (uint32_t) ((uintptr_t) x >> 2)) & 3u), n);
}

// Work split: a batch is swept by S CTAs that interleave 1024 packets at a time (so its bytes arrive as one sequential
// stream), and a CTA takes k (batch, slice) pairs, m * S = k * gridDim.x with the smallest such k = m / gcd(m, gridDim.x):
// 16 batches on 296 CTAs give S = 37 and k = 2, i.e. a CTA stops to repair and fold twice per launch.  When every CTA
// took a slice of every batch (S = gridDim.x, k = m) it stopped 16 times, and those stops were a quarter of the
// kernel's time.  Contiguous shares of the concatenated batches (one or two stops, but 296 distant streams) were
// measured too: 11.2 us per 51 MB batch against 11.6 us -- the sweep itself is slower that way.
__global__ void __launch_bounds__(kLaneHistThreads, 2) tfe_hist_lane_kernel(const __grid_constant__ HistJob job,
                                                                            const aq_tfe_state_t* __restrict__ st)
{
    pdl_launch_dependents();
    extern __shared__ uint32_t s_lane_hist[];   // [513][32] counters, then the repair queue
    uint32_t* s_queue = s_lane_hist + kLaneHistRows * 32;
    __shared__ uint32_t s_queued;
    __shared__ float s_bs, s_po;   // only the exact formula (rare paths) needs them: kept out of the registers
    {
        // shared-memory setup needs no global input: it overlaps the tail of the previous grid
        uint4* z = reinterpret_cast<uint4*>(s_lane_hist);
        for (int i = threadIdx.x; i < kLaneHistRows * 32 / 4; i += kLaneHistThreads)
            z[i] = make_uint4(0, 0, 0, 0);
        if (threadIdx.x == 0)
            s_queued = 0;
    }
    const uint32_t stride = (uint32_t) job.slices * kLaneHistThreads;
    // Bringing a slice's first packets into L2 may start before the previous grid has finished even if that grid is
    // still writing them: L2 is the point of coherence, a line fetched early is simply updated by the later stores.
    auto prefetch_head = [&](int item) {
        const int b       = item / job.slices;
        const uint32_t p0 = (uint32_t) (item - b * job.slices) * kLaneHistThreads + threadIdx.x;
        const int lead    = hist_lead(job.x[b], job.n[b]);
        const float4* h4  = reinterpret_cast<const float4*>(job.x[b] + lead);
        const uint32_t np = (uint32_t) ((job.n[b] - lead) / 4);
#pragma unroll
        for (int u = 0; u < kLaneUnroll; ++u)
            if (p0 + u * stride < np)
                asm volatile("prefetch.global.L2 [%0];" ::"l"(h4 + (p0 + u * stride)));
    };
    prefetch_head(blockIdx.x);
    pdl_wait();
    // bucket_size, pdf_offset and the initialized flag sit in one aligned 16-byte group: one load, one round trip
    const int4 tail = *reinterpret_cast<const int4*>(&st->bucket_size);
    int initialized = tail.z;
    if (job.gate && *job.gate == 0)
        initialized = 0;
    if (blockIdx.x == 0 && threadIdx.x < job.m && job.count)
        job.count[threadIdx.x * job.row_stride] = initialized ? job.n[threadIdx.x] : 0;
    if (!initialized)
        return;
    if (threadIdx.x == 0)
        s_bs = __int_as_float(tail.x), s_po = __int_as_float(tail.y);
    __syncthreads();
    const float margin = hist_margin(__int_as_float(tail.y));
    // A margin of a quarter bucket or more means the grid sits so far from zero that the reciprocal form is
    // useless: eps = 0 marks every packet unsure, the queue overflows and the CTA takes the exact sweep below.
    const float eps = margin < 0.25f ? 0.5f - margin : 0.0f;
    const float rbs = __frcp_rn(__int_as_float(tail.x));
    const float c   = 1.5f - __int_as_float(tail.y);
    const uint32_t base = (uint32_t) __cvta_generic_to_shared(s_lane_hist + (threadIdx.x & 31));

    // Per sample: FFMA, 3 FADD, FMNMX, VIADDMNMX, LEA, RED.  `worst` collects max |g| of the group; a NaN (from a
    // NaN / Inf sample) is dropped by fmaxf, which is fine: such a sample went to the trash row, and the exact
    // formula drops it too.
#define AQ_HIST_SAMPLE(X)                                                                                            \
    {                                                                                                                \
        const float s_  = fmaf((X), rbs, c);                                                                         \
        const float s2_ = __fadd_rd(s_, kTwo23);                                                                     \
        worst           = fmaxf(worst, fabsf(s_ - (s2_ - 8388607.5f)));                                              \
        lane_hist_inc(base, min(__float_as_uint(s2_) - (kTwo23Bits + 1u), (uint32_t) AQ_PDF_SIZE));                  \
    }
#define AQ_HIST_PACKET(V)                                                                                            \
    {                                                                                                                \
        AQ_HIST_SAMPLE((V).x) AQ_HIST_SAMPLE((V).y) AQ_HIST_SAMPLE((V).z) AQ_HIST_SAMPLE((V).w)                      \
    }
#define AQ_HIST_QUEUE()                                                                                              \
    if (!(worst < eps))                                                                                              \
    {                                                                                                                \
        const uint32_t slot = atomicAdd(&s_queued, 1u);                                                              \
        if (slot < (uint32_t) kFixQueue)                                                                             \
            s_queue[slot] = p;                                                                                       \
    }
    for (int it = 0; it < job.items; ++it)
    {
        const int item                = (int) blockIdx.x + it * (int) gridDim.x;
        const int b                   = item / job.slices;
        const uint32_t first          = (uint32_t) (item - b * job.slices) * kLaneHistThreads;
        const float* __restrict__ x0  = job.x[b];
        const int lead                = hist_lead(x0, job.n[b]);
        const float4* __restrict__ x4 = reinterpret_cast<const float4*>(x0 + lead);
        const uint32_t npack          = (uint32_t) ((job.n[b] - lead) / 4);
        const bool more               = it + 1 < job.items;
        // Packet indices within a batch fit 32 bits (n <= 2^31 elements).  Every thread sweeps packets p, p + stride,
        // ... of its slice; kLaneUnroll of them are in flight at once; the last, partial group is issued together as
        // well.
        uint32_t p = first + threadIdx.x;
        if (npack >= (kLaneUnroll - 1) * stride)
        {
            const uint32_t last_full = npack - (kLaneUnroll - 1) * stride;   // p < last_full: a full group fits
            for (; p < last_full; p += kLaneUnroll * stride)
            {
                float4 v[kLaneUnroll];
#pragma unroll
                for (int u = 0; u < kLaneUnroll; ++u)
                    v[u] = __ldcs(x4 + (p + u * stride));
                float worst = 0.0f;
#pragma unroll
                for (int u = 0; u < kLaneUnroll; ++u)
                    AQ_HIST_PACKET(v[u])
                AQ_HIST_QUEUE()
            }
        }
        {
            // partial group: up to kLaneUnroll - 1 packets
            float4 v[kLaneUnroll - 1];
#pragma unroll
            for (int u = 0; u < kLaneUnroll - 1; ++u)
                if (p + u * stride < npack)
                    v[u] = __ldcs(x4 + (p + u * stride));
            float worst = 0.0f;
#pragma unroll
            for (int u = 0; u < kLaneUnroll - 1; ++u)
                if (p + u * stride < npack)
                    AQ_HIST_PACKET(v[u])
            AQ_HIST_QUEUE()
        }
        // the next slice's first packets travel to L2 while this one is being repaired and folded
        if (more)
            prefetch_head(item + (int) gridDim.x);
        __syncthreads();
        const uint32_t queued = s_queued;
        if (queued <= (uint32_t) kFixQueue)
        {
            // one queued group = up to kLaneUnroll packets; (entry, packet) pairs are spread over the threads
            for (uint32_t i = threadIdx.x; i < queued * kLaneUnroll; i += kLaneHistThreads)
            {
                const uint32_t q = s_queue[i / kLaneUnroll] + (i % kLaneUnroll) * stride;
                if (q < npack)
                    hist_fix_packet(x4, q, base, rbs, c, eps, s_bs, s_po);
            }
        }
        else
        {
            // Queue overflow (adversarial data sitting on bucket boundaries): throw this CTA's counts away and redo
            // its slice with the exact formula.
            __syncthreads();
            for (int i = threadIdx.x; i < kLaneHistRows * 32; i += kLaneHistThreads)
                s_lane_hist[i] = 0;
            __syncthreads();
            for (uint32_t q = first + threadIdx.x; q < npack; q += stride)
            {
                const float4 w   = __ldg(x4 + q);
                const float f[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                for (int e = 0; e < 4; ++e)
                {
                    int k;
                    if (bucket_of(f[e], s_bs, s_po, k))
                        lane_hist_inc(base, (uint32_t) k);
                }
            }
        }
        __syncthreads();
        // Fold the 32 lane copies of each bucket and add the sums to the batch's global row.  Two threads per bucket,
        // each sums 16 copies (and leaves them zero for the next segment); the column order is rotated by the bucket
        // index so that the 32 lanes of a warp (16 buckets x 2 halves) touch 32 different banks at every step.  CTAs
        // start at rotated buckets so that they do not all hit the same global counter at the same moment.
        {
            const int rot   = (blockIdx.x * 37) & (AQ_PDF_SIZE - 1);
            const int bk    = ((threadIdx.x >> 1) + rot) & (AQ_PDF_SIZE - 1);
            const int half  = threadIdx.x & 1;
            uint32_t* row   = s_lane_hist + (bk << 5) + (half << 4);
            uint32_t sum    = 0;
            // four 16-byte loads per thread; the order is rotated by the bucket index so that the eight threads of a
            // quarter warp (4 buckets x 2 halves) touch eight different groups of four banks
#pragma unroll
            for (int k = 0; k < 4; ++k)
            {
                uint4* q      = reinterpret_cast<uint4*>(row) + ((k + bk) & 3);
                const uint4 w = *q;
                sum += w.x + w.y + w.z + w.w;
                if (more)
                    *q = make_uint4(0, 0, 0, 0);
            }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            if (half == 0 && sum)
                atomicAdd(&job.hist[b * job.row_stride * AQ_PDF_SIZE + bk], sum);
            if (more)
            {
                // the trash row and the queue counter start the next segment at zero as well
                if (threadIdx.x < 32)
                    s_lane_hist[(AQ_PDF_SIZE << 5) + threadIdx.x] = 0;
                if (threadIdx.x == 32)
                    s_queued = 0;
                __syncthreads();
            }
        }
    }   // (batch, slice) pairs
    if (blockIdx.x == 0)
    {
        // Elements outside the aligned packets -- up to three before the first one of a batch (a view that does not
        // start on a 16-byte boundary) and up to three after the last -- go straight to the batch's row.
        for (int b = 0; b < job.m; ++b)
        {
            const float* x0  = job.x[b];
            const int lead   = hist_lead(x0, job.n[b]);
            const int64_t np = (job.n[b] - lead) / 4;
            const int ragged = (int) (job.n[b] - lead - np * 4);
            const int t      = threadIdx.x;
            int k;
            if (t < lead + ragged && bucket_of(t < lead ? x0[t] : x0[lead + np * 4 + (t - lead)], s_bs, s_po, k))
                atomicAdd(&job.hist[b * job.row_stride * AQ_PDF_SIZE + k], 1u);
        }
    }
#undef AQ_HIST_SAMPLE
#undef AQ_HIST_PACKET
#undef AQ_HIST_QUEUE
}


static int hist_lane_attributes()
{
    static std::atomic<bool> attr_set[kMaxDevices];   // function attributes are per device
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess)
        return cuda_fail(e);
    if (dev < 0 || dev >= kMaxDevices || !attr_set[dev])
    {
        e = cudaFuncSetAttribute(tfe_hist_lane_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kLaneHistSmem);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(tfe_hist_lane_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                     cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess)
            return cuda_fail(e);
        if (dev >= 0 && dev < kMaxDevices)
            attr_set[dev] = true;
    }
    return AQ_OK;
}

int tfe_histogram_many(const float* const* xs, const int64_t* ns, int m, int64_t row_stride, const aq_tfe_state_t* st,
                       uint32_t* hist, int64_t* count, const int32_t* gate, cudaStream_t stream)
{
    int64_t n_total = 0;
    for (int b = 0; b < m; ++b)
        n_total += ns[b];
    const int rc = hist_lane_attributes();
    if (rc != AQ_OK)
        return rc;
    HistJob job;
    for (int b = 0; b < AQ_TFE_HIST_MANY; ++b)
    {
        job.x[b] = b < m ? xs[b] : nullptr;
        job.n[b] = b < m ? ns[b] : 0;
    }
    job.m = m, job.row_stride = row_stride, job.hist = hist, job.count = count, job.gate = gate;
    int64_t per_block = (int64_t) kLaneHistThreads * 4 * kLaneUnroll;
    int64_t blocks    = (n_total + per_block - 1) / per_block;
    int64_t cap       = (int64_t) kNumSMs * 2;   // two resident 1024-thread CTAs per SM (32 registers, 64 KiB each)
    if (blocks > cap)
        blocks = cap;
    if (blocks < 1)
        blocks = 1;
    // Two ways to split m batches over the CTAs: (a) cut the grid to a multiple of m, one slice per CTA and one stop
    // per launch, with up to m - 1 CTAs idle; (b) the full grid with the smallest k such that m * S == k * blocks.
    // The cheaper one by a simple model (a stop costs about 3 us, the sweep runs at about 6 TB/s): measured at 51 MB
    // per batch, (a) wins for 3, 5, 7, 15 batches (15: 9.0 against 11.9 us per batch), (b) for 16 (8.96 against 9.12).
    auto gcd = [](int a, int b) {
        while (b)
        {
            const int t = a % b;
            a = b, b = t;
        }
        return a;
    };
    if (blocks >= m)
    {
        const double sweep_us = (double) n_total * 4.0 / 6.0e6, stop_us = 3.0;
        const int64_t cut     = (blocks / m) * m;
        const double cost_cut  = sweep_us * (double) blocks / (double) cut + stop_us;
        const double cost_full = sweep_us + stop_us * (m / gcd(m, (int) blocks));
        if (cost_cut < cost_full)
            blocks = cut;
    }
    int g = m, r = (int) blocks;
    while (r)
    {
        const int t = g % r;
        g = r, r = t;
    }
    job.items  = m / g;
    job.slices = (int) (blocks / g);
    launch_pdl(tfe_hist_lane_kernel, (unsigned) blocks, kLaneHistThreads, kLaneHistSmem, stream, job, st);
    note_launch();
    return check_launch();
}

int tfe_histogram(const float* x, int64_t n, const aq_tfe_state_t* st, uint32_t* hist, int64_t* count,
                  const int32_t* gate, cudaStream_t stream)
{
    return tfe_histogram_many(&x, &n, 1, 1, st, hist, count, gate, stream);
}

int tfe_offer_grid(const float* x, int64_t n, aq_tfe_state_t* st, float* range, int init, void* ws, int64_t ws_bytes,
                   cudaStream_t stream)
{
    // resident grid (every CTA first looks at the state: an offer that is not needed costs one small wave)
    int64_t blocks = (n + (int64_t) kOfferThreads * 4 * kMmUnroll - 1) / ((int64_t) kOfferThreads * 4 * kMmUnroll);
    if (blocks > (int64_t) kNumSMs * 4)
        blocks = (int64_t) kNumSMs * 4;
    if (blocks < 1)
        blocks = 1;
    if (ws_bytes < 256 + blocks * (int64_t) sizeof(float2))
        return AQ_ERR_WORKSPACE;
    launch_pdl(tfe_offer_grid_kernel, (unsigned) blocks, kOfferThreads, 0, stream, x, n, st, range, init,
               static_cast<unsigned int*>(ws), reinterpret_cast<float2*>(static_cast<char*>(ws) + 256));
    note_launch();
    return check_launch();
}

int tfe_select_grid(const float* ranges, int num_ranks, int rank, aq_tfe_state_t* st, int32_t* gate,
                    cudaStream_t stream)
{
    launch_pdl(tfe_select_grid_kernel, 1, AQ_PDF_SIZE, 0, stream, ranges, num_ranks, rank, st, gate);
    note_launch();
    return check_launch();
}

int tfe_init_grid(const float* minmax, aq_tfe_state_t* st, cudaStream_t stream)
{
    launch_pdl(tfe_init_grid_kernel, 1, AQ_PDF_SIZE, 0, stream, minmax, st);
    note_launch();
    return check_launch();
}

// Correctly rounded a / b from y = RN(1 / b): two residual corrections.  After the first one q is within one ulp
// of a / b, and for such a q Markstein's theorem gives RN(q + (a - b q) y) = RN(a / b).  Five dependent fused
// operations instead of the ~20 of a full division; b must be a positive normal number, a zero or normal.
__device__ __forceinline__ double div_by_rcp(double a, double b, double y)
{
    double q = __dmul_rn(a, y);
    q        = __fma_rn(__fma_rn(-b, q, a), y, q);
    return __fma_rn(__fma_rn(-b, q, a), y, q);
}

constexpr int kReplayThreads = 64;    // buckets per CTA: 8 CTAs cover the 512 buckets (2,048 rows: 77 us; with 128: 85 us)
constexpr int kReplayChunk   = 64;    // rows per shared-memory stage
constexpr int kReplayGroup   = 16;    // rows folded between two checks of the speculation
constexpr int kReplaySmem    = 2 * kReplayChunk * kReplayThreads * (int) sizeof(uint32_t);

// Running mean of per-batch PDFs, batch order preserved (DlQuantization/src/math_functions.cpp:278-287):
// pdf <- (pdf * k + hist / count) / (k + 1) for every batch with a non-zero count.  The chain over k is serial per
// bucket and a CTA's two warps sit on schedulers of their own, so the kernel is built to keep a warp's instruction stream short
// and free of branches:
//  * rows arrive through a two-stage cp.async ring (64 rows x this CTA's 64 buckets per stage);
//  * per stage the CTA prepares, per row, count, RN(1/count), k, k + 1 and RN(1/(k + 1)); both divisions then use
//    div_by_rcp (bit-identical to IEEE division).  A dropped row (count 0, or past the end of the table) is encoded
//    as (1, 0, 1, 1, 1): its probability evaluates to 0 and the mean step to (acc * 1 + 0) / 1 = acc, so the fold
//    needs no test per row;
//  * inside a group of rows the chain runs on the quotient after ONE correction while the second correction is
//    evaluated beside it; the second one is the correctly rounded quotient, so when the two agree for every row of
//    the group the result stands, otherwise the group is folded again with the full sequence.
// A count whose low 32 bits are zero (the reference divides by (int) count) takes the plain-division path.
__global__ void __launch_bounds__(kReplayThreads) tfe_pdf_replay_kernel(const uint32_t* __restrict__ hists,
                                                                        const int64_t* __restrict__ counts,
                                                                        int64_t num_batches, double* __restrict__ pdf,
                                                                        int32_t* __restrict__ iterations)
{
    pdl_launch_dependents();
    pdl_wait();
    constexpr int CH = kReplayChunk, G = kReplayGroup;
    extern __shared__ __align__(16) unsigned char replay_dyn[];
    uint32_t(*buf)[CH][kReplayThreads] = reinterpret_cast<uint32_t(*)[CH][kReplayThreads]>(replay_dyn);
    __shared__ __align__(8) int64_t s_c[2][CH];
    __shared__ double s_d[CH], s_rd[CH], s_k[CH], s_b[CH], s_rb[CH];
    __shared__ int s_warp[kReplayThreads / 32];
    __shared__ int s_odd;
    const int t = threadIdx.x;
    const int i = blockIdx.x * kReplayThreads + t;
    auto issue  = [&](int stage, int64_t c0) {
        const int rows = (int) ((num_batches - c0 < CH) ? (num_batches - c0) : CH);
        constexpr int LPR = kReplayThreads / 4;     // lanes that copy one row's slice, 16 bytes per lane
#pragma unroll 4
        for (int pass = 0; pass < CH / 4; ++pass)   // four rows per pass
        {
            const int r = pass * 4 + t / LPR;
            if (r < rows)
            {
                const unsigned dst  = (unsigned) __cvta_generic_to_shared(&buf[stage][r][(t % LPR) * 4]);
                const uint32_t* src = hists + (c0 + r) * AQ_PDF_SIZE + blockIdx.x * kReplayThreads + (t % LPR) * 4;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
            }
        }
        if (t < rows)
        {
            const unsigned dst = (unsigned) __cvta_generic_to_shared(&s_c[stage][t]);
            asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(counts + c0 + t) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (t == 0)
        s_odd = 0;
    issue(0, 0);
    double acc  = 0.0;
    int it_base = 0;
    int chunk   = 0;
    for (int64_t c0 = 0; c0 < num_batches; c0 += CH, ++chunk)
    {
        const int stage = chunk & 1;
        const int rows  = (int) ((num_batches - c0 < CH) ? (num_batches - c0) : CH);
        if (c0 + CH < num_batches)
        {
            issue(stage ^ 1, c0 + CH);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        }
        else
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        // ---- per-row preparation: thread t owns row c0 + t ----
        const int64_t cnt   = (t < rows) ? s_c[stage][t] : 0;
        const bool live     = cnt != 0;
        const unsigned mask = __ballot_sync(0xffffffffu, live);
        if ((t & 31) == 0)
            s_warp[t >> 5] = __popc(mask);
        __syncthreads();
        int before = __popc(mask & ((1u << (t & 31)) - 1u));
        int total  = 0;
#pragma unroll
        for (int w = 0; w < kReplayThreads / 32; ++w)
        {
            if (w < (t >> 5))
                before += s_warp[w];
            total += s_warp[w];
        }
        if (t < CH)
        {
            if (live)
            {
                const int it   = it_base + before;
                const double d = (double) (int) cnt;
                if (d == 0.0)
                    s_odd = 1;
                s_d[t]  = d;
                s_rd[t] = __drcp_rn(d);
                s_k[t]  = (double) it;
                s_b[t]  = (double) (it + 1);
                s_rb[t] = __drcp_rn((double) (it + 1));
            }
            else
            {
                s_d[t] = s_k[t] = s_b[t] = s_rb[t] = 1.0;
                s_rd[t]                            = 0.0;
            }
        }
        __syncthreads();
        if (s_odd)
        {
            for (int r = 0; r < rows; ++r)
                if (s_c[stage][r] != 0)
                    acc = __ddiv_rn(__dadd_rn(__dmul_rn(acc, s_k[r]), __ddiv_rn((double) buf[stage][r][t], s_d[r])), s_b[r]);
        }
        else
        {
            for (int j0 = 0; j0 < CH; j0 += G)
            {
                double prob[G];
#pragma unroll
                for (int u = 0; u < G; ++u)
                    prob[u] = div_by_rcp((double) buf[stage][j0 + u][t], s_d[j0 + u], s_rd[j0 + u]);
                const double acc0 = acc;
                bool redo         = false;
#pragma unroll
                for (int u = 0; u < G; ++u)
                {
                    const double b = s_b[j0 + u], y = s_rb[j0 + u];
                    const double a = __dadd_rn(__dmul_rn(acc, s_k[j0 + u]), prob[u]);
                    double q       = __dmul_rn(a, y);
                    q              = __fma_rn(__fma_rn(-b, q, a), y, q);
                    redo |= __fma_rn(__fma_rn(-b, q, a), y, q) != q;
                    acc = q;
                }
                if (redo)
                {
                    acc = acc0;
#pragma unroll
                    for (int u = 0; u < G; ++u)
                        acc = div_by_rcp(__dadd_rn(__dmul_rn(acc, s_k[j0 + u]), prob[u]), s_b[j0 + u], s_rb[j0 + u]);
                }
            }
        }
        it_base += total;
        __syncthreads();
        if (t == 0)
            s_odd = 0;
    }
    pdf[i] = acc;
    if (i == 0)
        *iterations = it_base;
}

int tfe_pdf_replay(const uint32_t* hists, const int64_t* counts, int64_t num_batches, double* pdf,
                   int32_t* iterations, cudaStream_t stream)
{
    static std::atomic<bool> attr_set[kMaxDevices];   // function attributes are per device
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess)
        return cuda_fail(e);
    if (dev < 0 || dev >= kMaxDevices || !attr_set[dev])
    {
        e = cudaFuncSetAttribute(tfe_pdf_replay_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kReplaySmem);
        if (e != cudaSuccess)
            return cuda_fail(e);
        if (dev >= 0 && dev < kMaxDevices)
            attr_set[dev] = true;
    }
    launch_pdl(tfe_pdf_replay_kernel, AQ_PDF_SIZE / kReplayThreads, kReplayThreads, kReplaySmem, stream, hists, counts,
               num_batches, pdf, iterations);
    note_launch();
    return check_launch();
}

// -------------------------------------------------------------------------------------------------
// aimet_torch v2 min/max calibration, the part after the reduction: merge of the batch range into the running range,
// MinMaxEncodingAnalyzer.compute_encodings_from_stats (aimet_torch/v2/quantization/encoding_analyzer.py:325-386) and the
// quantizer's scale / offset (affine/quantizer.py:222-246) for `count` encodings in one launch.  The reference spends
// about 25 small tensor operations per quantizer on this; every one of them is element-wise, so each encoding is one
// thread here, evaluated in the reference's operation order and -- for 16-bit statistics -- with its roundings: the
// statistics and the first quotient live in the statistics dtype, everything after the comparison with the minimum
// scale is float32 (the adjustment term is a float32 tensor, which promotes the rest).
// -------------------------------------------------------------------------------------------------
template <int DT>
__device__ __forceinline__ float round_to(float v)
{
    if (DT == AQ_F16)
        return __half2float(__float2half_rn(v));
    if (DT == AQ_BF16)
        return __bfloat162float(__float2bfloat16_rn(v));
    return v;
}
__device__ __forceinline__ float nan_min(float a, float b)   // torch.minimum: NaN wins
{
    return (a != a || b != b) ? NAN : fminf(a, b);
}
__device__ __forceinline__ float nan_max(float a, float b)
{
    return (a != a || b != b) ? NAN : fmaxf(a, b);
}

template <int DT>
__global__ void __launch_bounds__(256) v2_minmax_encode_kernel(const float* __restrict__ batch /* [2, count] or null */,
                                                               float* __restrict__ running /* [2, count] or null */,
                                                               int running_valid, int64_t count, float num_steps,
                                                               float steps_in_dt, float pos_steps, float neg_steps,
                                                               int symmetric, float qmin, float type_max,
                                                               float* __restrict__ out /* [4, count] */)
{
    pdl_launch_dependents();
    pdl_wait();
    const int64_t i = (int64_t) blockIdx.x * 256 + threadIdx.x;
    if (i >= count)
        return;
    float mn, mx;
    if (batch)
    {
        mn = batch[i], mx = batch[count + i];
        if (running)
        {
            // merge_stats: torch.minimum / torch.maximum with the running range (or adopt the batch)
            const float rmn = running_valid ? nan_min(running[i], mn) : mn;
            const float rmx = running_valid ? nan_max(running[count + i], mx) : mx;
            running[i] = rmn, running[count + i] = rmx;
        }
    }
    else
        mn = running[i], mx = running[count + i];
    const float eps  = 1.1920928955078125e-07f;   // torch.finfo(torch.float32).eps
    const float min0 = (mn != mn) ? mn : fminf(mn, 0.0f);
    const float max0 = (mx != mx) ? mx : fmaxf(mx, 0.0f);
    const float diff = round_to<DT>(__fdiv_rn(round_to<DT>(__fsub_rn(max0, min0)), steps_in_dt));
    const float adj  = (diff < eps) ? eps : 0.0f;
    float umin, umax;
    if (symmetric)
    {
        umax              = __fadd_rn(max0, __fmul_rn(pos_steps, adj));
        umin              = __fsub_rn(min0, __fmul_rn(neg_steps, adj));
        const float delta = nan_max(__fdiv_rn(umax, pos_steps), __fdiv_rn(-umin, neg_steps));
        umin              = __fmul_rn(-neg_steps, delta);
        umax              = __fmul_rn(pos_steps, delta);
    }
    else
    {
        umax = __fadd_rn(max0, __fmul_rn(num_steps, adj));
        umin = min0;
    }
    // clamp to the statistics dtype's range (NaN stays NaN), then the cast to that dtype
    const float emax = round_to<DT>((umax == umax) ? fminf(umax, type_max) : umax);
    const float emin = round_to<DT>((umin == umin) ? fmaxf(umin, -type_max) : umin);
    const float scale = __fdiv_rn(__fsub_rn(emax, emin), num_steps);
    const float offset = symmetric ? 0.0f : __fsub_rn(rintf(__fdiv_rn(emin, scale)), qmin);
    out[i] = emin, out[count + i] = emax, out[2 * count + i] = scale, out[3 * count + i] = offset;
}

int v2_minmax_encode(const float* batch, float* running, int running_valid, int dtype, int64_t count, double num_steps,
                     int symmetric, double qmin, float* out, cudaStream_t st)
{
    if (count == 0)
        return AQ_OK;
    const float ns  = (float) num_steps;
    const float pos = (float) floor(num_steps / 2.0), neg = (float) ceil(num_steps / 2.0);
    // the divisor of the first quotient is a tensor of the statistics dtype in the reference's arithmetic
    float ns_dt = ns, tmax = FLT_MAX;
    if (dtype == AQ_F16)
        ns_dt = __half2float(__float2half_rn(ns)), tmax = 65504.0f;
    else if (dtype == AQ_BF16)
        ns_dt = __bfloat162float(__float2bfloat16_rn(ns)), tmax = 3.3895313892515355e38f;
    const unsigned grid = (unsigned) ((count + 255) / 256);
#define AQ_ENC(DT)                                                                                                   \
    launch_pdl(v2_minmax_encode_kernel<DT>, grid, 256, 0, st, batch, running, running_valid, count, ns, ns_dt, pos, neg, \
               symmetric, (float) qmin, tmax, out)
    switch (dtype)
    {
    case AQ_F32: AQ_ENC(AQ_F32); break;
    case AQ_F16: AQ_ENC(AQ_F16); break;
    case AQ_BF16: AQ_ENC(AQ_BF16); break;
    default: return AQ_ERR_INVALID_ARG;
    }
#undef AQ_ENC
    note_launch();
    return check_launch();
}

}   // namespace aq
