"""TEST INFRASTRUCTURE ONLY: CPU checkers for the parity tests.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may import this
package.  The product package never does.

Two libraries are wrapped with ctypes + numpy:

* ``liboracle.so``   - our plain-C restatement (``libpymo_oracle.c``), always buildable (``make oracle``).
* ``libaimet_ref.so`` - the unmodified reference DlQuantization CPU sources behind ``ref_shim.cpp``
  (``make ref``); exists only where the reference checkout was available at build time.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from typing import Optional

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(_HERE, "_build", "liboracle.so")
REF_SO = os.path.join(_HERE, "_ref", "libaimet_ref.so")
PDF_SIZE = 512


def reference_root(ref_root: Optional[str] = None) -> Optional[str]:
    """Where a checkout of the reference lies: the argument, else ``AIMET_REFERENCE_ROOT``, else a directory named
    ``reference`` next to this repository.  None when there is none (the fixtures under tests/golden then stand in)."""
    for root in (ref_root, os.environ.get("AIMET_REFERENCE_ROOT"),
                 os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")):
        if root and os.path.isdir(os.path.join(root, "ModelOptimizations", "DlQuantization", "src")):
            return root
    return None


def build(ref_root: Optional[str] = None) -> None:
    """Compile the C restatement; also the reference shim when a reference checkout is found (reference_root)."""
    subprocess.run(["make", "-s", "-C", _HERE, "oracle"], check=True)
    root = reference_root(ref_root)
    if root is not None:
        subprocess.run(["make", "-s", "-C", _HERE, "ref", f"REF_ROOT={root}"], check=True)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a, t):
    return a.ctypes.data_as(C.POINTER(t))


_PF, _PD, _PU, _PI, _PL = (C.POINTER(C.c_float), C.POINTER(C.c_double), C.POINTER(C.c_uint32),
                           C.POINTER(C.c_int), C.POINTER(C.c_int64))


class Oracle:
    """ctypes view of liboracle.so (the C restatement)."""

    def __init__(self, path: str = ORACLE_SO):
        if not os.path.exists(path):
            build()
        L = self.lib = C.CDLL(path)
        L.orc_fill_encoding.argtypes = [C.c_int, C.c_double, C.c_double, _PD]
        L.orc_qdq_per_tensor.argtypes = [_PF, C.c_int64, _PF, C.c_double, C.c_double, C.c_int]
        L.orc_quantize_per_tensor.argtypes = [_PF, C.c_int64, _PF, C.c_double, C.c_double, C.c_int, C.c_int]
        L.orc_per_channel_grid.argtypes = [_PD, _PD, C.c_int64, C.c_int, _PF, _PF, _PF, _PF]
        L.orc_qdq_per_channel.argtypes = [_PF, C.c_int64, C.c_int64, C.c_int64, _PF, _PF, _PF, _PF, _PF]
        L.orc_qdq_broadcast.argtypes = [_PF, _PF, C.c_int64, C.c_int64, _PL, _PL, _PF, _PF, _PF, _PF]
        L.orc_ste_bwd.argtypes = [_PF, _PF, C.c_int64, C.c_float, C.c_float, _PF]
        L.orc_min_max.argtypes = [_PF, C.c_int64, _PF]
        L.orc_computed_encodings.argtypes = [C.c_int, C.c_double, C.c_double, C.c_int, C.c_int, C.c_int, _PD]
        L.orc_minmax_encoding.argtypes = [C.c_int, C.c_double, C.c_double, C.c_int, C.c_int, C.c_int, _PD]
        L.orc_pdf_init.argtypes = [C.c_float, C.c_float, _PD]
        L.orc_pdf_geometry.argtypes = [_PD, _PF, _PF]
        L.orc_hist512.argtypes = [_PF, C.c_int64, C.c_float, C.c_float, _PU]
        L.orc_pdf_accumulate.argtypes = [_PU, C.c_int64, _PD, _PI]
        L.orc_update_pdf.argtypes = [_PF, C.c_int64, _PD, _PD, _PI, _PI, _PU]
        L.orc_update_pdf.restype = C.c_int
        L.orc_tfe_cost.argtypes = [_PD, _PD, C.c_int, C.c_float, C.c_int]
        L.orc_tfe_cost.restype = C.c_double
        L.orc_tfe_candidates.argtypes = [_PD, _PD, C.c_int, C.c_int, C.c_int, C.c_int, _PF, _PI]
        L.orc_tfe_candidates.restype = C.c_int
        L.orc_tfe_compute.argtypes = [_PD, _PD, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _PD]
        L.orc_quantize_packed.argtypes = [_PF, C.c_int64, _PD, C.c_int, C.c_int, C.c_void_p]
        L.orc_dequantize_packed.argtypes = [C.c_void_p, C.c_int64, _PD, C.c_int, C.c_int, _PF]
        L.orc_mse_compute.argtypes = [_PD, _PD, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _PD]
        L.orc_percentile_compute.argtypes = [_PD, _PD, C.c_int, C.c_int, C.c_float, C.c_int, C.c_int, C.c_int, C.c_int, _PD]

    # --- QDQ -------------------------------------------------------------------------------------
    def fill_encoding(self, bw, mn, mx):
        out = np.zeros(4, np.float64)
        self.lib.orc_fill_encoding(bw, mn, mx, _p(out, C.c_double))
        return out

    def qdq_per_tensor(self, x, mn, mx, bw):
        x = _f32(x)
        out = np.empty_like(x)
        self.lib.orc_qdq_per_tensor(_p(x, C.c_float), x.size, _p(out, C.c_float), mn, mx, bw)
        return out

    def quantize_per_tensor(self, x, mn, mx, bw, shift_to_signed=False):
        x = _f32(x)
        out = np.empty_like(x)
        self.lib.orc_quantize_per_tensor(_p(x, C.c_float), x.size, _p(out, C.c_float), mn, mx, bw,
                                         int(shift_to_signed))
        return out

    def per_channel_grid(self, mins, maxs, bw):
        mins = np.ascontiguousarray(mins, np.float64)
        maxs = np.ascontiguousarray(maxs, np.float64)
        n = mins.size
        g = [np.empty(n, np.float32) for _ in range(4)]
        self.lib.orc_per_channel_grid(_p(mins, C.c_double), _p(maxs, C.c_double), n, bw,
                                      *[_p(a, C.c_float) for a in g])
        return g

    def qdq_per_channel(self, x, num_ch, per_ch, g_min, g_max, g_delta, g_offset):
        x = _f32(x)
        out = np.empty_like(x)
        g = [_f32(a) for a in (g_min, g_max, g_delta, g_offset)]
        self.lib.orc_qdq_per_channel(_p(x, C.c_float), num_ch, x.size, per_ch, _p(out, C.c_float),
                                     *[_p(a, C.c_float) for a in g])
        return out

    def qdq_broadcast(self, x, in_strides, enc_strides, g_min, g_max, g_delta, g_offset):
        x = _f32(x)
        out = np.empty_like(x)
        ins = np.ascontiguousarray(in_strides, np.int64)
        ens = np.ascontiguousarray(enc_strides, np.int64)
        g = [_f32(a) for a in (g_min, g_max, g_delta, g_offset)]
        self.lib.orc_qdq_broadcast(_p(x, C.c_float), _p(out, C.c_float), x.size, ins.size, _p(ins, C.c_int64),
                                   _p(ens, C.c_int64), *[_p(a, C.c_float) for a in g])
        return out

    def ste_bwd(self, x, g, mn, mx):
        x, g = _f32(x), _f32(g)
        out = np.empty_like(x)
        self.lib.orc_ste_bwd(_p(x, C.c_float), _p(g, C.c_float), x.size, mn, mx, _p(out, C.c_float))
        return out

    # --- MinMax ----------------------------------------------------------------------------------
    def min_max(self, x):
        x = _f32(x)
        out = np.zeros(2, np.float32)
        self.lib.orc_min_max(_p(x, C.c_float), x.size, _p(out, C.c_float))
        return out

    def computed_encodings(self, bw, mn, mx, symmetric=False, strict=False, unsigned_sym=False):
        out = np.zeros(4, np.float64)
        self.lib.orc_computed_encodings(bw, mn, mx, int(symmetric), int(strict), int(unsigned_sym),
                                        _p(out, C.c_double))
        return out

    def minmax_encoding(self, bw, stat_min, stat_max, symmetric=False, strict=False, unsigned_sym=False):
        out = np.zeros(4, np.float64)
        self.lib.orc_minmax_encoding(bw, stat_min, stat_max, int(symmetric), int(strict), int(unsigned_sym),
                                     _p(out, C.c_double))
        return out

    # --- TF-Enhanced -----------------------------------------------------------------------------
    def pdf_init(self, mn, mx):
        x_left = np.zeros(PDF_SIZE, np.float64)
        self.lib.orc_pdf_init(mn, mx, _p(x_left, C.c_double))
        return x_left

    def pdf_geometry(self, x_left):
        bs, po = C.c_float(), C.c_float()
        self.lib.orc_pdf_geometry(_p(x_left, C.c_double), C.byref(bs), C.byref(po))
        return np.float32(bs.value), np.float32(po.value)

    def hist512(self, x, bucket_size, pdf_offset):
        x = _f32(x)
        h = np.zeros(PDF_SIZE, np.uint32)
        self.lib.orc_hist512(_p(x, C.c_float), x.size, bucket_size, pdf_offset, _p(h, C.c_uint32))
        return h

    @staticmethod
    def packed_dtype(bw, signed):
        return {(8, False): np.uint8, (8, True): np.int8, (16, False): np.uint16, (16, True): np.int16,
                (32, False): np.uint32, (32, True): np.int32}[(max(int(bw), 8), bool(signed))]

    def quantize_packed(self, x, mn, mx, bw, shift_to_signed=False):
        x = _f32(x)
        enc = np.ascontiguousarray(self.fill_encoding(bw, mn, mx), np.float64)
        out = np.zeros(x.shape, self.packed_dtype(bw, shift_to_signed))
        self.lib.orc_quantize_packed(_p(x, C.c_float), x.size, _p(enc, C.c_double), int(bw), int(shift_to_signed),
                                     out.ctypes.data_as(C.c_void_p))
        return out

    def dequantize_packed(self, codes, mn, mx, bw, shift_to_signed=False):
        codes = np.ascontiguousarray(codes)
        enc = np.ascontiguousarray(self.fill_encoding(bw, mn, mx), np.float64)
        out = np.zeros(codes.shape, np.float32)
        self.lib.orc_dequantize_packed(codes.ctypes.data_as(C.c_void_p), codes.size, _p(enc, C.c_double), int(bw),
                                       int(shift_to_signed), _p(out, C.c_float))
        return out

    def percentile_compute(self, x_left, pdf, initialized, stats_updated, percentile, bw, symmetric=False,
                           strict=False, unsigned_sym=False):
        out = np.zeros(5, np.float64)
        x_left = np.ascontiguousarray(x_left, np.float64)
        pdf = np.ascontiguousarray(pdf, np.float64)
        self.lib.orc_percentile_compute(_p(x_left, C.c_double), _p(pdf, C.c_double), int(initialized),
                                        int(stats_updated), float(percentile), int(bw), int(symmetric), int(strict),
                                        int(unsigned_sym), _p(out, C.c_double))
        return out

    def mse_compute(self, x_left, pdf, initialized, stats_updated, bw, symmetric=False, strict=False,
                    unsigned_sym=False):
        out = np.zeros(5, np.float64)
        x_left = np.ascontiguousarray(x_left, np.float64)
        pdf = np.ascontiguousarray(pdf, np.float64)
        self.lib.orc_mse_compute(_p(x_left, C.c_double), _p(pdf, C.c_double), int(initialized), int(stats_updated),
                                 int(bw), int(symmetric), int(strict), int(unsigned_sym), _p(out, C.c_double))
        return out

    def tfe_cost(self, x_left, pdf, bw, delta, offset):
        return self.lib.orc_tfe_cost(_p(x_left, C.c_double), _p(pdf, C.c_double), bw, delta, offset)

    def tfe_candidates(self, x_left, pdf, bw, symmetric=False, strict=False, unsigned_sym=False):
        cd = np.zeros(512, np.float32)
        co = np.zeros(512, np.int32)
        n = self.lib.orc_tfe_candidates(_p(x_left, C.c_double), _p(pdf, C.c_double), bw, int(symmetric), int(strict),
                                        int(unsigned_sym), _p(cd, C.c_float), _p(co, C.c_int))
        return cd[:n].copy(), co[:n].copy()


class OracleTfeAnalyzer:
    """TF-Enhanced analyzer state machine on top of the C restatement (mirrors
    DlQuantization/src/TfEnhancedEncodingAnalyzer.cpp:60-113)."""

    def __init__(self, oracle: Oracle):
        self.o = oracle
        self.x_left = np.zeros(PDF_SIZE, np.float64)
        self.pdf = np.zeros(PDF_SIZE, np.float64)
        self.initialized = C.c_int(0)
        self.iterations = C.c_int(0)
        self.stats_updated = False
        self.batch_hists = []

    def update(self, x):
        x = _f32(x)
        self.stats_updated = True
        h = np.zeros(PDF_SIZE, np.uint32)
        used = self.o.lib.orc_update_pdf(_p(x, C.c_float), x.size, _p(self.x_left, C.c_double),
                                         _p(self.pdf, C.c_double), C.byref(self.initialized),
                                         C.byref(self.iterations), _p(h, C.c_uint32))
        if used:
            self.batch_hists.append(h)
        return bool(used)

    def compute(self, bw, symmetric=False, strict=False, unsigned_sym=False):
        out = np.zeros(5, np.float64)
        self.o.lib.orc_tfe_compute(_p(self.x_left, C.c_double), _p(self.pdf, C.c_double), self.initialized.value,
                                   int(self.stats_updated), bw, int(symmetric), int(strict), int(unsigned_sym),
                                   _p(out, C.c_double))
        return out


    def compute_percentile(self, percentile, bw, symmetric=False, strict=False, unsigned_sym=False):
        """The percentile analyzer's encoding from the same statistics (PercentileEncodingAnalyzer.cpp:79-194)."""
        return self.o.percentile_compute(self.x_left, self.pdf, self.initialized.value, self.stats_updated, percentile,
                                         bw, symmetric, strict, unsigned_sym)


    def compute_mse(self, bw, symmetric=False, strict=False, unsigned_sym=False):
        """The MSE analyzer's encoding from the same statistics (MseEncodingAnalyzer.cpp:78-267)."""
        return self.o.mse_compute(self.x_left, self.pdf, self.initialized.value, self.stats_updated, bw, symmetric,
                                  strict, unsigned_sym)


class Reference:
    """ctypes view of libaimet_ref.so (the reference's own CPU code). ``available()`` says whether it exists."""

    @staticmethod
    def available(path: str = REF_SO) -> bool:
        return os.path.exists(path)

    def __init__(self, path: str = REF_SO):
        L = self.lib = C.CDLL(path)
        L.ref_fill_encoding.argtypes = [C.c_int, C.c_double, C.c_double, _PD]
        L.ref_qdq_per_tensor.argtypes = [_PF, C.c_int64, _PF, C.c_double, C.c_double, C.c_int]
        L.ref_quantize_per_tensor.argtypes = [_PF, C.c_int64, _PF, C.c_double, C.c_double, C.c_int, C.c_int]
        L.ref_qdq_per_channel.argtypes = [_PF, C.c_int64, C.c_int64, C.c_int64, _PF, _PF, _PF, _PF, _PF]
        L.ref_qdq_broadcast.argtypes = [_PF, _PF, C.c_int64, C.c_int64, _PL, _PL, _PF, _PF, _PF, _PF]
        L.ref_computed_encodings.argtypes = [C.c_int, C.c_double, C.c_double, C.c_int, C.c_int, C.c_int, _PD]
        L.ref_min_max.argtypes = [_PF, C.c_int64, _PF]
        for name in ("ref_tf_new", "ref_tfe_new"):
            getattr(L, name).restype = C.c_void_p
        for name in ("ref_tf_free", "ref_tfe_free"):
            getattr(L, name).argtypes = [C.c_void_p]
        for name in ("ref_tf_update", "ref_tfe_update"):
            getattr(L, name).argtypes = [C.c_void_p, _PF, C.c_int64]
        for name in ("ref_tf_compute", "ref_tfe_compute"):
            getattr(L, name).argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, _PD]
        L.ref_tfe_histogram.argtypes = [C.c_void_p, _PD, _PD]
        L.ref_tfe_histogram.restype = C.c_int
        L.ref_update_pdf.argtypes = [_PF, C.c_int64, _PD, _PD, _PI, _PI]
        if hasattr(L, "ref_pct_new"):
            L.ref_pct_new.restype = C.c_void_p
            L.ref_pct_free.argtypes = [C.c_void_p]
            L.ref_pct_update.argtypes = [C.c_void_p, _PF, C.c_int64]
            L.ref_pct_set_percentile.argtypes = [C.c_void_p, C.c_float]
            L.ref_pct_compute.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, _PD]
            L.ref_mse_new.restype = C.c_void_p
            L.ref_mse_free.argtypes = [C.c_void_p]
            L.ref_mse_update.argtypes = [C.c_void_p, _PF, C.c_int64]
            L.ref_mse_compute.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, _PD]
            L.ref_quantize_packed.argtypes = [_PF, C.c_int64, C.c_void_p, C.c_double, C.c_double, C.c_int, C.c_int]
            L.ref_dequantize_packed.argtypes = [C.c_void_p, C.c_int64, _PF, C.c_double, C.c_double, C.c_int, C.c_int]
            L.ref_partial_encoding.argtypes = [C.c_int, _PD, C.c_int, C.c_int, C.c_int]
            L.ref_partial_encoding.restype = C.c_int

    def fill_encoding(self, bw, mn, mx):
        out = np.zeros(5, np.float64)
        self.lib.ref_fill_encoding(bw, mn, mx, _p(out, C.c_double))
        return out[:4]

    def qdq_per_tensor(self, x, mn, mx, bw):
        x = _f32(x)
        out = np.empty_like(x)
        self.lib.ref_qdq_per_tensor(_p(x, C.c_float), x.size, _p(out, C.c_float), mn, mx, bw)
        return out

    def quantize_per_tensor(self, x, mn, mx, bw, shift_to_signed=False):
        x = _f32(x)
        out = np.empty_like(x)
        self.lib.ref_quantize_per_tensor(_p(x, C.c_float), x.size, _p(out, C.c_float), mn, mx, bw,
                                         int(shift_to_signed))
        return out

    def qdq_per_channel(self, x, num_ch, per_ch, g_min, g_max, g_delta, g_offset):
        x = _f32(x)
        out = np.empty_like(x)
        g = [_f32(a).copy() for a in (g_min, g_max, g_delta, g_offset)]
        self.lib.ref_qdq_per_channel(_p(x, C.c_float), num_ch, x.size, per_ch, _p(out, C.c_float),
                                     *[_p(a, C.c_float) for a in g])
        return out

    def qdq_broadcast(self, x, in_strides, enc_strides, g_min, g_max, g_delta, g_offset):
        x = _f32(x)
        out = np.empty_like(x)
        ins = np.ascontiguousarray(in_strides, np.int64)
        ens = np.ascontiguousarray(enc_strides, np.int64)
        g = [_f32(a) for a in (g_min, g_max, g_delta, g_offset)]
        self.lib.ref_qdq_broadcast(_p(x, C.c_float), _p(out, C.c_float), x.size, ins.size, _p(ins, C.c_int64),
                                   _p(ens, C.c_int64), *[_p(a, C.c_float) for a in g])
        return out

    def computed_encodings(self, bw, mn, mx, symmetric=False, strict=False, unsigned_sym=False):
        out = np.zeros(5, np.float64)
        self.lib.ref_computed_encodings(bw, mn, mx, int(symmetric), int(strict), int(unsigned_sym),
                                        _p(out, C.c_double))
        return out[:4]

    def min_max(self, x):
        x = _f32(x)
        out = np.zeros(2, np.float32)
        self.lib.ref_min_max(_p(x, C.c_float), x.size, _p(out, C.c_float))
        return out

    def batch_hist(self, x, x_left):
        """Raw uint32[512] counts of one batch on a given bucket grid, recovered exactly from one
        UpdatePdf step on an empty PDF (pdf[i] = hist[i]/cnt when iterations == 0)."""
        x = _f32(x)
        xl = np.array(x_left, np.float64)
        pdf = np.zeros(PDF_SIZE, np.float64)
        init, it = C.c_int(1), C.c_int(0)
        self.lib.ref_update_pdf(_p(x, C.c_float), x.size, _p(xl, C.c_double), _p(pdf, C.c_double), C.byref(init),
                                C.byref(it))
        return np.rint(pdf * x.size).astype(np.uint32)


class RefAnalyzer:
    """Owns one reference analyzer object: kind 'tf' (MinMax), 'tfe' (TF-Enhanced), 'pct' (percentile) or 'mse'."""

    def __init__(self, ref: Reference, kind: str):
        self.ref, self.kind = ref, kind
        self.h = getattr(ref.lib, f"ref_{kind}_new")()

    def __del__(self):
        if getattr(self, "h", None):
            getattr(self.ref.lib, f"ref_{self.kind}_free")(self.h)
            self.h = None

    def update(self, x):
        x = _f32(x)
        getattr(self.ref.lib, f"ref_{self.kind}_update")(self.h, _p(x, C.c_float), x.size)

    def compute(self, bw, symmetric=False, strict=False, unsigned_sym=False):
        out = np.zeros(5, np.float64)
        getattr(self.ref.lib, f"ref_{self.kind}_compute")(self.h, bw, int(symmetric), int(strict), int(unsigned_sym),
                                                          _p(out, C.c_double))
        return out

    def set_percentile(self, percentile: float):
        self.ref.lib.ref_pct_set_percentile(self.h, float(percentile))

    def histogram(self):
        xl = np.zeros(PDF_SIZE, np.float64)
        pdf = np.zeros(PDF_SIZE, np.float64)
        n = self.ref.lib.ref_tfe_histogram(self.h, _p(xl, C.c_double), _p(pdf, C.c_double))
        return (xl, pdf) if n else (None, None)
