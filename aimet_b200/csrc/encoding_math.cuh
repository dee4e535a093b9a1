// Encoding arithmetic shared by the host entry points and the device-side analyzers: the same double-precision
// operations in the same order as the reference, so that both sides give the reference's bits.
#pragma once

#include <float.h>
#include <math.h>

#include "common.cuh"

namespace aq
{
// std::max / std::min with the reference's argument order (decides NaN and signed-zero behaviour)
__host__ __device__ inline double hmax(double a, double b)
{
    return (a < b) ? b : a;
}
__host__ __device__ inline double hmin(double a, double b)
{
    return (b < a) ? b : a;
}

// getComputedEncodings (DlQuantization/src/quantization_utils.cpp:58-143)
__host__ __device__ inline void computed_encodings(int bw, double mn, double mx, bool sym, bool strict,
                                                   bool unsigned_sym, aq_encoding_t* e)
{
    double steps = ldexp(1.0, (int) (uint8_t) bw) - 1.0;   // 2^bw exactly, on the host and on the device
    if (sym && strict)
        steps -= 1.0;
    e->bw = bw;
    if (isinf(mn))
        mn = -(double) FLT_MAX;
    if (isinf(mx))
        mx = (double) FLT_MAX;
    if (sym && (mn < 0.0 || !unsigned_sym))
    {
        const double amax      = hmax(fabs(mx), fabs(mn));
        const unsigned int pos = (unsigned int) floor(steps / 2.0);
        e->delta               = amax / pos;
        e->offset              = -ceil(steps / 2.0);
        e->min                 = hmax(e->offset * e->delta, -(double) FLT_MAX);
        e->max                 = hmin(e->delta * pos, (double) FLT_MAX);
        return;
    }
    e->delta = (mx - mn) / steps;
    if (mn < 0 && mx > 0)
    {
        double zero_code = round(-mn / e->delta);
        zero_code        = hmin(steps, hmax(0.0, zero_code));
        e->offset        = -zero_code;
        const double lo  = e->delta * e->offset;
        e->min           = (lo >= -(double) FLT_MAX && lo <= (double) FLT_MAX) ? lo : -(double) FLT_MAX;
        e->max           = mx - mn + e->min;
        if (e->max > (double) FLT_MAX)
            e->max = (double) FLT_MAX;
    }
    else
    {
        e->offset = round(mn / e->delta);
        e->min    = mn;
        e->max    = mx;
    }
}
}   // namespace aq
