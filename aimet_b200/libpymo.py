"""Drop-in for the native objects behind AIMET's v1 quantsim: ``aimet_common.libpymo`` (enums, ``TfEncoding``,
``TensorQuantizer``) and ``aimet_common.AimetTensorQuantizer.AimetTensorQuantizer``.

Same class and method names, argument meaning and error behaviour as the pybind objects declared in
``ModelOptimizations/PyModelOptimizations/PyModelOptimizations.cpp:147-260`` and
``TrainingExtensions/torch/src/AimetTensorQuantizer.cpp:75-331`` -- but every tensor operation runs on the
B200 through the C ABI, statistics stay resident on the device between batches, and nothing runs on the CPU:
``use_cuda=False`` or a CPU tensor raises ``RuntimeError`` instead of silently taking another path.
"""
from __future__ import annotations

import enum
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import ops


class ComputationMode(enum.IntEnum):
    COMP_MODE_CPU = 0
    COMP_MODE_GPU = 1


class QuantizationMode(enum.IntEnum):
    QUANTIZATION_TF = 0
    QUANTIZATION_TF_ENHANCED = 1
    QUANTIZATION_RANGE_LEARNING = 2
    QUANTIZATION_PERCENTILE = 3
    QUANTIZATION_MSE = 4
    QUANTIZATION_ENTROPY = 5


class RoundingMode(enum.IntEnum):
    ROUND_NEAREST = 0
    ROUND_STOCHASTIC = 1


class TensorQuantizerOpMode(enum.IntEnum):
    updateStats = 0
    oneShotQuantizeDequantize = 1
    quantizeDequantize = 2
    passThrough = 3


# pybind's export_values(): the enumerators are also module attributes
for _e in (ComputationMode, QuantizationMode, RoundingMode):
    globals().update(_e.__members__)


class TfEncoding:
    """Mirror of DlQuantization::TfEncoding (read/write fields ``min, max, delta, offset, bw``)."""
    __slots__ = ("min", "max", "delta", "offset", "bw")

    def __init__(self, min: float = 0.0, max: float = 0.0, delta: float = 0.0, offset: float = 0.0, bw: int = 0):
        self.min, self.max, self.delta, self.offset, self.bw = min, max, delta, offset, bw

    @classmethod
    def _from_c(cls, e) -> "TfEncoding":
        return cls(e.min, e.max, e.delta, e.offset, int(e.bw))

    def __repr__(self):
        return f"TfEncoding(min={self.min}, max={self.max}, delta={self.delta}, offset={self.offset}, bw={self.bw})"


_SUPPORTED_SCHEMES = (QuantizationMode.QUANTIZATION_TF, QuantizationMode.QUANTIZATION_TF_ENHANCED,
                      QuantizationMode.QUANTIZATION_RANGE_LEARNING, QuantizationMode.QUANTIZATION_PERCENTILE,
                      QuantizationMode.QUANTIZATION_MSE)


def _require_gpu(t: torch.Tensor, use_cuda: bool, what: str):
    if not use_cuda or not t.is_cuda:
        raise RuntimeError(f"aimet_b200: {what} needs use_cuda=True and a CUDA tensor; there is no CPU path")
    if t.dtype != torch.float32:
        raise RuntimeError(f"aimet_b200: {what} takes float32 tensors (callers upcast, as with the reference)")


def _dense(t: torch.Tensor) -> torch.Tensor:
    """The element kernels work on raw storage: keep the tensor's own dense layout (the reference does
    ``input.contiguous(input.suggest_memory_format())``), copy only when it is a strided view."""
    if t.is_contiguous() or (t.dim() == 4 and t.is_contiguous(memory_format=torch.channels_last)) or \
            (t.dim() == 5 and t.is_contiguous(memory_format=torch.channels_last_3d)):
        return t
    return t.contiguous()


class _MinMaxStats:
    """Running min / max on the device (TfEncodingAnalyzer, DlQuantization/src/TfEncodingAnalyzer.cpp:59-101)."""

    def __init__(self):
        self.acc: Optional[torch.Tensor] = None   # float32 [2, 1] on the device

    def update(self, x: torch.Tensor):
        if self.acc is None or self.acc.device != x.device:
            self.acc = torch.tensor([[float("inf")], [float("-inf")]], dtype=torch.float32, device=x.device)
        ops.minmax(x, 1, None, propagate_nan=False, out=self.acc, accumulate=True)

    def compute(self, bw, symmetric, strict, unsigned_sym) -> TfEncoding:
        mn, mx = (float(v) for v in self.acc.reshape(-1).tolist())
        # the reference starts its running stats at +-DBL_MAX and narrows through float: an analyzer that only
        # ever saw empty tensors reports +-inf, which the encoding math maps to +-FLT_MAX as well
        return TfEncoding._from_c(ops.minmax_encoding(bw, mn, mx, symmetric, strict, unsigned_sym))

    def histogram(self):
        raise RuntimeError("aimet_b200: the TF (min/max) analyzer keeps no histogram")


class _TfEnhancedStats:
    """512-bucket PDF statistics on the device (TfEnhancedEncodingAnalyzer,
    DlQuantization/src/TfEnhancedEncodingAnalyzer.cpp:60-113)."""

    def __init__(self, percentile_of=None, mse=False):
        self.dev: Optional[ops.TfeDeviceState] = None
        self.updated = False
        #: True for the MSE analyzer (MseEncodingAnalyzer.cpp, same statistics)
        self.mse = mse
        #: None for TF-Enhanced; for the percentile analyzer (PercentileEncodingAnalyzer.cpp, same statistics) a
        #: callable returning the percentile currently set on the owning quantizer
        self.percentile_of = percentile_of

    def update(self, x: torch.Tensor):
        if self.dev is None:
            self.dev = ops.TfeDeviceState(x.device)
        self.updated = True
        st = self.dev
        if not st.poll_initialized():
            # first batch(es): the grid comes from this batch's min/max, unless it is all zeros.  The device decides
            # (one launch: min/max pass + grid setup, which returns at once when a grid exists); the host only stops
            # offering when an asynchronous read of the flag has come back, so no call waits for the GPU.
            st.offer_grid(x)
            st.start_probe()
        st.add_batch(x)

    def compute(self, bw, symmetric, strict, unsigned_sym) -> TfEncoding:
        if self.mse:
            e = self.dev.mse_encoding(self.updated, bw, symmetric, strict, unsigned_sym).tolist()
        elif self.percentile_of is not None:
            e = self.dev.percentile_encoding(self.updated, self.percentile_of(), bw, symmetric, strict,
                                             unsigned_sym).tolist()
        else:
            e = self.dev.compute_encoding(self.updated, bw, symmetric, strict, unsigned_sym).tolist()
        return TfEncoding(e[0], e[1], e[2], e[3], int(e[4]))

    def histogram(self) -> List[Tuple[float, float]]:
        st = self.dev
        if st is None or not st.is_initialized():
            return []
        st.replay()
        return list(zip(st.x_left().tolist(), st.pdf.tolist()))


class AimetTensorQuantizer:
    """Mirror of the torch-extension class ``AimetTensorQuantizer``
    (TrainingExtensions/torch/src/AimetTensorQuantizer.cpp:75-331)."""

    def __init__(self, quantizationScheme: QuantizationMode):
        self._scheme = QuantizationMode(quantizationScheme)
        if self._scheme not in _SUPPORTED_SCHEMES:
            raise RuntimeError(f"aimet_b200: quantization scheme {self._scheme.name} is outside the accelerated path "
                               "(TF, TF-Enhanced, percentile and MSE are implemented)")
        self._isEncodingValid = False
        self._stats = self._new_stats()

    def _new_stats(self):
        if self._scheme == QuantizationMode.QUANTIZATION_TF_ENHANCED:
            return _TfEnhancedStats()
        if self._scheme == QuantizationMode.QUANTIZATION_PERCENTILE:
            return _TfEnhancedStats(percentile_of=self.getPercentileValue)
        if self._scheme == QuantizationMode.QUANTIZATION_MSE:
            return _TfEnhancedStats(mse=True)
        return _MinMaxStats()

    # -- statistics ----------------------------------------------------------------------------------
    def resetEncodingStats(self):
        self._isEncodingValid = False
        self._stats = self._new_stats()

    def updateStats(self, input: torch.Tensor, use_cuda: bool):
        _require_gpu(input, use_cuda, "updateStats")
        self._isEncodingValid = True
        self._stats.update(_dense(input))

    def getEncoding(self, bitwidth: int, useSymmetricEncodings: bool, useStrictSymmetric: bool,
                    useUnsignedSymmetric: bool) -> Tuple[TfEncoding, bool]:
        if not self._isEncodingValid:
            return TfEncoding(), False
        enc = self._stats.compute(int(bitwidth), bool(useSymmetricEncodings), bool(useStrictSymmetric),
                                  bool(useUnsignedSymmetric))
        return enc, True

    def getStatsHistogram(self) -> List[Tuple[float, float]]:
        return self._stats.histogram()

    def setPercentileValue(self, percentile: float):
        """Kept for the percentile scheme; the other analyzers ignore it, as in the reference."""
        self._percentile = float(percentile)

    def getPercentileValue(self) -> float:
        return getattr(self, "_percentile", 100.0)

    # -- fake-quant ------------------------------------------------------------------------------------
    def quantizeDequantize(self, input: torch.Tensor, encoding: TfEncoding, roundingMode: RoundingMode,
                           use_cuda: bool) -> torch.Tensor:
        _require_gpu(input, use_cuda, "quantizeDequantize")
        return ops.qdq_per_tensor(_dense(input), encoding.min, encoding.max, encoding.bw, int(roundingMode))

    def quantize(self, input: torch.Tensor, encoding: TfEncoding, roundingMode: RoundingMode, use_cuda: bool,
                 shiftToSigned: bool) -> torch.Tensor:
        _require_gpu(input, use_cuda, "quantize")
        return ops.quantize_per_tensor(_dense(input), encoding.min, encoding.max, encoding.bw, shiftToSigned,
                                       int(roundingMode))

    def makeDeltaOffsetTensor(self, device, encodings: Sequence[TfEncoding]) -> Tuple[torch.Tensor, torch.Tensor]:
        vals = torch.tensor([[e.delta for e in encodings], [e.offset for e in encodings]], dtype=torch.float32)
        vals = vals.to(device)
        return vals[0], vals[1]

    def quantizeDequantizePerChannel(self, input: torch.Tensor, encodings: Sequence[TfEncoding], numChannel: int,
                                     numElement: int, numElementPerChannel: int, roundingMode: RoundingMode,
                                     useCuda: bool) -> torch.Tensor:
        return quantize_dequantize_per_channel(input, encodings, numChannel, numElement, numElementPerChannel,
                                               roundingMode, useCuda)


def quantize_dequantize_per_channel(input: torch.Tensor, encodings: Sequence[TfEncoding], numChannel: int,
                                    numElement: int, numElementPerChannel: int, roundingMode: RoundingMode,
                                    useCuda: bool) -> torch.Tensor:
    """AimetTensorQuantizer::quantizeDequantizePerChannel (TrainingExtensions/torch/src/AimetTensorQuantizer.cpp:256-307):
    the per-channel grid is derived from the encodings' (min, max) inside the kernel."""
    _require_gpu(input, useCuda, "quantizeDequantizePerChannel")
    if len(encodings) != numChannel:
        raise RuntimeError("aimet_b200: one encoding per channel is required")
    x = input.contiguous()
    if x.numel() != numElement:
        raise RuntimeError("aimet_b200: numElement does not match the tensor")
    mm = torch.tensor([[e.min for e in encodings], [e.max for e in encodings]], dtype=torch.float32)
    mm = mm.to(x.device, non_blocking=True)
    steps = 2.0 ** encodings[0].bw - 1
    if encodings[0].min == -encodings[0].max:
        steps -= 1
    return ops.qdq_per_channel(x, mm[0], mm[1], numChannel, numElementPerChannel, steps, int(roundingMode))


class TensorQuantizer:
    """Mirror of ``libpymo.TensorQuantizer`` (numpy in / numpy out; PyTensorQuantizer.cpp:43-77 over
    DlQuantization/src/TensorQuantizer.cpp).  Host arrays are staged to the GPU, processed there and copied
    back: this is the end-to-end path with host buffers."""

    def __init__(self, quantScheme: QuantizationMode, roundingMode: RoundingMode, device: str = "cuda"):
        self._q = AimetTensorQuantizer(quantScheme)
        self._scheme = QuantizationMode(quantScheme)
        self.roundingMode = RoundingMode(roundingMode)
        self.isEncodingValid = False
        self._strict = False
        self._unsigned = False
        self._device = torch.device(device)

    def _to_dev(self, a: np.ndarray) -> torch.Tensor:
        t = torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32))
        return t.to(self._device, non_blocking=True)

    def updateStats(self, tensor: np.ndarray, useCuda: bool = True):
        self._q.updateStats(self._to_dev(tensor), True)

    def computeEncoding(self, bitwidth: int, useSymmetricEncodings: bool) -> TfEncoding:
        enc, valid = self._q.getEncoding(bitwidth, useSymmetricEncodings, self._strict, self._unsigned)
        self.isEncodingValid = valid
        return enc

    def quantizeDequantize(self, inputTensor: np.ndarray, outputTensor: np.ndarray, encodingMin: float,
                           encodingMax: float, bitwidth: int, useCuda: bool = True):
        y = ops.qdq_per_tensor(self._to_dev(inputTensor), encodingMin, encodingMax, bitwidth, int(self.roundingMode))
        outputTensor.reshape(-1)[:] = y.reshape(-1).cpu().numpy()

    def quantizeTensorPacked(self, inputTensor: np.ndarray, encodingMin: float, encodingMax: float, bw: int,
                             roundMode: RoundingMode = RoundingMode.ROUND_NEAREST, useCuda: bool = True,
                             useStrictSymmetric: bool = False) -> np.ndarray:
        """Integer codes in uint8/16/32 containers (int8/16/32 when ``useStrictSymmetric`` shifts them to signed):
        DlQuantization/src/TensorQuantizer.cpp:179-186.  The reference returns the bytes of that array."""
        codes = ops.quantize_packed(self._to_dev(inputTensor), encodingMin, encodingMax, bw, useStrictSymmetric,
                                    int(roundMode))
        return codes.cpu().numpy()

    def dequantize(self, codes: np.ndarray, encodingMin: float, encodingMax: float, bw: int,
                   useStrictSymmetric: bool = False) -> np.ndarray:
        """Inverse of ``quantizeTensorPacked`` (DlQuantization/src/TensorQuantizer.cpp:217-223)."""
        t = torch.from_numpy(np.ascontiguousarray(codes)).to(self._device, non_blocking=True)
        return ops.dequantize_packed(t, encodingMin, encodingMax, bw, useStrictSymmetric).cpu().numpy()

    def resetEncodingStats(self):
        self._q.resetEncodingStats()
        self.isEncodingValid = False

    def setQuantScheme(self, scheme: QuantizationMode):
        self._scheme = QuantizationMode(scheme)
        self._q = AimetTensorQuantizer(self._scheme)

    def getQuantScheme(self) -> QuantizationMode:
        return self._scheme

    def setStrictSymmetric(self, flag: bool):
        self._strict = bool(flag)

    def getStrictSymmetric(self) -> bool:
        return self._strict

    def setUnsignedSymmetric(self, flag: bool):
        self._unsigned = bool(flag)

    def getUnsignedSymmetric(self) -> bool:
        return self._unsigned

    def getStatsHistogram(self):
        return self._q.getStatsHistogram()

    def setPercentileValue(self, percentile: float):
        self._q.setPercentileValue(percentile)

    def getPercentileValue(self) -> float:
        return self._q.getPercentileValue()

    def computePartialEncoding(self, bw: int, encoding: TfEncoding, useSymmetricEncodings: bool,
                               useUnsignedSymmetric: bool, useStrictSymmetric: bool) -> None:
        """Fills in the missing half of ``encoding`` in place (DlQuantization/src/TensorQuantizer.cpp:327-343):
        (min, max) from (delta, offset) when min == max == 0, (delta, offset) from (min, max) when delta == 0."""
        compute_partial_encoding(bw, encoding, useSymmetricEncodings, useUnsignedSymmetric, useStrictSymmetric)


def compute_partial_encoding(bw: int, encoding: TfEncoding, use_symmetric: bool, use_unsigned_symmetric: bool,
                             use_strict_symmetric: bool) -> None:
    """``computeMinMaxRangeFromDeltaOffset`` / ``computeDeltaAndOffsetFromMinMax``
    (DlQuantization/src/quantization_utils.cpp:158-228); host arithmetic in double, as in the reference."""
    import math
    if encoding.min == 0 and encoding.max == 0:
        if encoding.bw == 0:
            raise ValueError("Encodings must have a valid non-zero bitwidth")
        if encoding.delta == 0 and encoding.offset > 0:
            raise ValueError("Encoding must have a valid non-zero delta/offset if min and max are zero")
        steps = 2.0 ** bw - 1
        if use_symmetric and use_strict_symmetric:
            steps -= 1
        encoding.min = encoding.offset * encoding.delta
        if use_symmetric and (encoding.min < 0.0 or not use_unsigned_symmetric):
            encoding.max = encoding.delta * math.floor(steps / 2)
        else:
            encoding.max = encoding.delta * steps + encoding.min
    elif encoding.delta == 0:
        if encoding.bw == 0:
            raise ValueError("Encodings must have a valid non-zero bitwidth")
        if encoding.delta != 0 and encoding.offset != 0:
            raise ValueError("Encoding delta and offset must be zero to use this function")
        e = ops.computed_encodings(int(bw), encoding.min, encoding.max, use_symmetric, use_strict_symmetric,
                                   use_unsigned_symmetric)
        encoding.delta, encoding.offset, encoding.bw = e.delta, e.offset, int(e.bw)
    else:
        raise RuntimeError("Cannot determine how to compute partial encoding")


class EncodingAnalyzerForPython:
    """Mirror of ``libpymo.EncodingAnalyzerForPython`` (DlQuantization/src/EncodingAnalyzerForPython.cpp:54-92): numpy
    in, ``(TfEncoding, is_valid)`` out.  The array is staged to the GPU and the statistics stay there."""

    def __init__(self, quantizationScheme: QuantizationMode, device: str = "cuda"):
        self._q = AimetTensorQuantizer(quantizationScheme)
        self._device = torch.device(device)

    def updateStats(self, input: np.ndarray, use_cuda: bool = True):
        t = torch.from_numpy(np.ascontiguousarray(input, dtype=np.float32)).to(self._device, non_blocking=True)
        self._q.updateStats(t, True)

    def computeEncoding(self, bitwidth: int, isSymmetric: bool, useStrictSymmetric: bool,
                        useUnsignedSymmetric: bool) -> Tuple[TfEncoding, bool]:
        return self._q.getEncoding(bitwidth, isSymmetric, useStrictSymmetric, useUnsignedSymmetric)


class TensorQuantizationSimForPython:
    """Mirror of ``libpymo.TensorQuantizationSimForPython`` (DlQuantization/src/TensorQuantizationSimForPython.cpp:54-79):
    ``quantizeDequantize(array, encoding, roundingMode[, bitwidth], use_cuda) -> array``."""

    def __init__(self, device: str = "cuda"):
        self._device = torch.device(device)

    def quantizeDequantize(self, input: np.ndarray, encoding: TfEncoding, roundingMode: RoundingMode, *rest):
        if len(rest) == 2:
            bitwidth = int(rest[0])
        elif len(rest) == 1:
            bitwidth = int(encoding.bw)
        else:
            raise TypeError("quantizeDequantize(input, encoding, roundingMode, [bitwidth,] use_cuda)")
        t = torch.from_numpy(np.ascontiguousarray(input, dtype=np.float32)).to(self._device, non_blocking=True)
        y = ops.qdq_per_tensor(t, encoding.min, encoding.max, bitwidth, int(roundingMode))
        return y.cpu().numpy().reshape(np.shape(input))
