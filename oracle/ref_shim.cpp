// TEST INFRASTRUCTURE ONLY -- not part of the shipped product path.
//
// Thin extern "C" wrapper over the *unmodified* AIMET DlQuantization CPU sources
// (ModelOptimizations/DlQuantization/src/*.cpp).  The Makefile next to this file
// compiles those sources where they lie in the reference checkout together with
// this shim into oracle/_ref/libaimet_ref.so.  Nothing from the reference is
// copied into this repository; this file only calls its public C++ entry points
// so that Python tests (ctypes) can drive them.
//
// Used for: (1) pinning the C restatement in libpymo_oracle.c, (2) generating
// the golden fixtures under tests/golden, (3) the timed CPU baseline.

#include <cstdint>
#include <cstring>
#include <tuple>
#include <vector>

#include "DlQuantization/Quantization.hpp"
#include "TensorQuantizationSim.h"
#include "TfEncodingAnalyzer.h"
#include "MseEncodingAnalyzer.h"
#include "PercentileEncodingAnalyzer.h"
#include "TfEnhancedEncodingAnalyzer.h"
#include "math_functions.hpp"
#include "quantization_utils.hpp"
#include "trim_functions.hpp"

using namespace DlQuantization;

namespace
{
void storeEncoding(const TfEncoding& e, double* out5)
{
    out5[0] = e.min;
    out5[1] = e.max;
    out5[2] = e.delta;
    out5[3] = e.offset;
    out5[4] = (double) e.bw;
}
}   // namespace

extern "C"
{
// TensorQuantizationSim<float>::fillEncodingInfo (TensorQuantizationSim.cpp:84-92)
void ref_fill_encoding(int bw, double encMin, double encMax, double* out5)
{
    TensorQuantizationSim<float> sim;
    TfEncoding e;
    sim.fillEncodingInfo(e, (uint8_t) bw, encMin, encMax);
    storeEncoding(e, out5);
}

// TensorQuantizationSim<float>::quantizeDequantizeTensor (TensorQuantizationSim.cpp:94-114), CPU mode.
void ref_qdq_per_tensor(const float* in, int64_t n, float* out, double encMin, double encMax, int bw)
{
    TensorQuantizationSim<float> sim;
    sim.quantizeDequantizeTensor(in, (size_t) n, out, encMin, encMax, (uint8_t) bw, ROUND_NEAREST, false);
}

// TensorQuantizationSim<float>::quantizeTensor (TensorQuantizationSim.cpp:116-126), CPU mode.
void ref_quantize_per_tensor(const float* in, int64_t n, float* out, double encMin, double encMax, int bw,
                             int shiftToSigned)
{
    TensorQuantizationSim<float> sim;
    sim.quantizeTensor(in, (size_t) n, out, encMin, encMax, (uint8_t) bw, ROUND_NEAREST, false, shiftToSigned != 0);
}

// TensorQuantizationSim<float>::quantizeDequantizeTensorPerChannel (TensorQuantizationSim.cpp:287-317), CPU mode.
// The four encoding arrays are used as given (the caller derives them, as AimetTensorQuantizer.cpp:256-307 does).
void ref_qdq_per_channel(const float* in, int64_t numChannel, int64_t numElement, int64_t numElementPerChannel,
                         float* out, float* encMin, float* encMax, float* encDelta, float* encOffset)
{
    TensorQuantizationSim<float> sim;
    sim.quantizeDequantizeTensorPerChannel(in, (size_t) numChannel, (size_t) numElement,
                                           (size_t) numElementPerChannel, out, encMin, encMax, encDelta, encOffset,
                                           ROUND_NEAREST, false);
}

// quantizeDequantizeBroadcastCpu (trim_functions.cpp:633-660).
void ref_qdq_broadcast(const float* in, float* out, int64_t numElement, int64_t numDims, const int64_t* inputStrides,
                       const int64_t* encodingStrides, const float* encMin, const float* encMax,
                       const float* encDelta, const float* encOffset)
{
    quantizeDequantizeBroadcastCpu<float>(in, out, numElement, numDims, inputStrides, encodingStrides, encMin, encMax,
                                          encDelta, encOffset);
}

// getComputedEncodings (quantization_utils.cpp:58-143).
void ref_computed_encodings(int bw, double mn, double mx, int symmetric, int strict, int unsignedSym, double* out5)
{
    TfEncoding e = getComputedEncodings((uint8_t) bw, mn, mx, symmetric != 0, strict != 0, unsignedSym != 0);
    e.bw         = bw;
    storeEncoding(e, out5);
}

// GetMin / GetMax (math_functions.cpp:61-100, 327-347), CPU mode.
void ref_min_max(const float* in, int64_t n, float* out2)
{
    out2[0] = GetMin(in, (int) n, COMP_MODE_CPU);
    out2[1] = GetMax(in, (int) n, COMP_MODE_CPU);
}

// ---- TfEncodingAnalyzer<float> (MinMax) -------------------------------------------------------
void* ref_tf_new()
{
    return new TfEncodingAnalyzer<float>();
}
void ref_tf_free(void* h)
{
    delete static_cast<TfEncodingAnalyzer<float>*>(h);
}
void ref_tf_update(void* h, const float* in, int64_t n)
{
    static_cast<TfEncodingAnalyzer<float>*>(h)->updateStats(in, (size_t) n, COMP_MODE_CPU);
}
void ref_tf_compute(void* h, int bw, int symmetric, int strict, int unsignedSym, double* out5)
{
    TfEncoding e = static_cast<TfEncodingAnalyzer<float>*>(h)->computeEncoding((uint8_t) bw, symmetric != 0,
                                                                              strict != 0, unsignedSym != 0);
    e.bw         = bw;
    storeEncoding(e, out5);
}

// ---- TfEnhancedEncodingAnalyzer<float> ---------------------------------------------------------
void* ref_tfe_new()
{
    return new TfEnhancedEncodingAnalyzer<float>();
}
void ref_tfe_free(void* h)
{
    delete static_cast<TfEnhancedEncodingAnalyzer<float>*>(h);
}
void ref_tfe_update(void* h, const float* in, int64_t n)
{
    static_cast<TfEnhancedEncodingAnalyzer<float>*>(h)->updateStats(in, (size_t) n, COMP_MODE_CPU);
}
void ref_tfe_compute(void* h, int bw, int symmetric, int strict, int unsignedSym, double* out5)
{
    TfEncoding e = static_cast<TfEnhancedEncodingAnalyzer<float>*>(h)->computeEncoding(
        (uint8_t) bw, symmetric != 0, strict != 0, unsignedSym != 0);
    storeEncoding(e, out5);
}
// Returns the number of buckets written (0 when the PDF is not initialised yet, else 512).
int ref_tfe_histogram(void* h, double* xLeft, double* pdf)
{
    auto v = static_cast<TfEnhancedEncodingAnalyzer<float>*>(h)->getStatsHistogram();
    for (size_t i = 0; i < v.size(); ++i)
    {
        xLeft[i] = std::get<0>(v[i]);
        pdf[i]   = std::get<1>(v[i]);
    }
    return (int) v.size();
}

// One UpdatePdf step (math_functions.cpp:243-288) on a caller-held PDF given as raw arrays.
// xLeft/pdf hold 512 doubles; *initialized says whether xLeft is valid; *iterations is the running count.
void ref_update_pdf(const float* in, int64_t n, double* xLeft, double* pdf, int* initialized, int* iterations)
{
    PDF p;
    if (*initialized)
    {
        p.xLeft.assign(xLeft, xLeft + PDF_SIZE);
        p.pdf.assign(pdf, pdf + PDF_SIZE);
        p.iterations = *iterations;
    }
    else
    {
        p.iterations = 0;
    }
    UpdatePdf(in, (int) n, COMP_MODE_CPU, true, p, nullptr);
    if (p.xLeft.size() == (size_t) PDF_SIZE)
    {
        std::memcpy(xLeft, p.xLeft.data(), PDF_SIZE * sizeof(double));
        std::memcpy(pdf, p.pdf.data(), PDF_SIZE * sizeof(double));
        *initialized = 1;
        *iterations  = p.iterations;
    }
}

// ---- PercentileEncodingAnalyzer<float> ---------------------------------------------------------
void* ref_pct_new()
{
    return new PercentileEncodingAnalyzer<float>();
}
void ref_pct_free(void* h)
{
    delete static_cast<PercentileEncodingAnalyzer<float>*>(h);
}
void ref_pct_update(void* h, const float* in, int64_t n)
{
    static_cast<PercentileEncodingAnalyzer<float>*>(h)->updateStats(in, (size_t) n, COMP_MODE_CPU);
}
void ref_pct_set_percentile(void* h, float percentile)
{
    static_cast<PercentileEncodingAnalyzer<float>*>(h)->setPercentileValue(percentile);
}
void ref_pct_compute(void* h, int bw, int symmetric, int strict, int unsignedSym, double* out5)
{
    TfEncoding e = static_cast<PercentileEncodingAnalyzer<float>*>(h)->computeEncoding(
        (uint8_t) bw, symmetric != 0, strict != 0, unsignedSym != 0);
    storeEncoding(e, out5);
}

// ---- MseEncodingAnalyzer<float> ----------------------------------------------------------------
void* ref_mse_new()
{
    return new MseEncodingAnalyzer<float>();
}
void ref_mse_free(void* h)
{
    delete static_cast<MseEncodingAnalyzer<float>*>(h);
}
void ref_mse_update(void* h, const float* in, int64_t n)
{
    static_cast<MseEncodingAnalyzer<float>*>(h)->updateStats(in, (size_t) n, COMP_MODE_CPU);
}
void ref_mse_compute(void* h, int bw, int symmetric, int strict, int unsignedSym, double* out5)
{
    TfEncoding e = static_cast<MseEncodingAnalyzer<float>*>(h)->computeEncoding((uint8_t) bw, symmetric != 0,
                                                                                strict != 0, unsignedSym != 0);
    storeEncoding(e, out5);
}

// TensorQuantizationSim<float>::quantizeTensorPacked / dequantizeTensor (TensorQuantizationSim.cpp:128-139,210-219).
// out must hold n containers of max(bw, 8) bits.
void ref_quantize_packed(const float* in, int64_t n, void* out, double encMin, double encMax, int bw, int shiftToSigned)
{
    TensorQuantizationSim<float> sim;
    std::vector<uint8_t> packed;
    sim.quantizeTensorPacked(in, (size_t) n, packed, encMin, encMax, (uint8_t) bw, ROUND_NEAREST, false,
                             shiftToSigned != 0);
    std::memcpy(out, packed.data(), packed.size());
}
void ref_dequantize_packed(const void* in, int64_t n, float* out, double encMin, double encMax, int bw, int shiftToSigned)
{
    TensorQuantizationSim<float> sim;
    sim.dequantizeTensor(static_cast<const uint8_t*>(in), (size_t) n, out, encMin, encMax, (uint8_t) bw,
                         shiftToSigned != 0);
}

// computeMinMaxRangeFromDeltaOffset / computeDeltaAndOffsetFromMinMax (quantization_utils.cpp:158-228) the way
// TensorQuantizer::computePartialEncoding picks between them (TensorQuantizer.cpp:327-343).  enc5 is in/out;
// returns 1 when the reference throws.
int ref_partial_encoding(int bw, double* enc5, int symmetric, int unsignedSym, int strict)
{
    TfEncoding e;
    e.min = enc5[0], e.max = enc5[1], e.delta = enc5[2], e.offset = enc5[3], e.bw = (int) enc5[4];
    try
    {
        if (e.min == 0 && e.max == 0)
            computeMinMaxRangeFromDeltaOffset((uint8_t) bw, e, symmetric != 0, unsignedSym != 0, strict != 0);
        else if (e.delta == 0)
            computeDeltaAndOffsetFromMinMax((uint8_t) bw, e, symmetric != 0, unsignedSym != 0, strict != 0);
        else
            return 1;
    }
    catch (...)
    {
        return 1;
    }
    storeEncoding(e, enc5);
    return 0;
}

}   // extern "C"
