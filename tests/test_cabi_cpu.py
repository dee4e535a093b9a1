"""CPU-side checks of the C ABI: the shared library loads, exports every function that include/aimet_b200.h
declares (and nothing in the header is missing from the Python binding), and the host-only encoding arithmetic
matches the oracle bit for bit.  No kernel is launched here."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from _data import assert_bits_equal

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    text = open(os.path.join(ROOT, "include", "aimet_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(aq_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_function():
    from aimet_b200 import _lib
    names = header_functions()
    assert len(names) >= 20
    lib = C.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in the header but not exported"
    assert sorted(_lib.SIGNATURES) == names, "Python binding and header disagree"


def test_no_torch_types_in_header():
    text = open(os.path.join(ROOT, "include", "aimet_b200.h")).read()
    code = re.sub(r"/\*.*?\*/", "", text, flags=re.S)   # declarations only; comments cite reference paths
    assert "at::" not in code and "torch" not in code.lower() and "Tensor" not in code


def test_version_and_status_strings():
    from aimet_b200._lib import lib
    assert lib.aq_version() >= 100
    assert lib.aq_status_string(0) == b"ok"
    assert b"invalid" in lib.aq_status_string(-1)


def test_host_encoding_arithmetic_matches_oracle(oracle):
    from aimet_b200 import ops
    for mn, mx, bw in [(-0.46, 0.72, 8), (0.5, 1.0, 8), (0.5, 0.5, 8), (-0.5, -0.1, 8), (-5, 10, 3), (-5, 5, 3),
                       (-1.3, 2.7, 4), (-3, 3, 16), (0, 0, 8)]:
        e = ops.fill_encoding(bw, mn, mx)
        assert_bits_equal(np.array([e.min, e.max, e.delta, e.offset]), oracle.fill_encoding(bw, mn, mx))
    for bw in (4, 8, 16):
        for mn, mx in [(-1.5, 3.2), (0, 4.4), (-3, 0), (-2, 2), (-1e-3, 1e-3), (-np.inf, 5), (0, 0.01), (2.0, 7.0)]:
            for flags in [(0, 0, 0), (1, 0, 0), (1, 1, 0), (1, 0, 1)]:
                e = ops.computed_encodings(bw, mn, mx, *flags)
                assert_bits_equal(np.array([e.min, e.max, e.delta, e.offset]),
                                  oracle.computed_encodings(bw, mn, mx, *flags))
                e = ops.minmax_encoding(bw, mn, mx, *flags)
                assert_bits_equal(np.array([e.min, e.max, e.delta, e.offset]),
                                  oracle.minmax_encoding(bw, mn, mx, *flags))
                assert e.bw == bw


def test_argument_validation_without_gpu():
    from aimet_b200._lib import lib
    # invalid arguments are rejected before any CUDA call
    assert lib.aq_qdq_per_tensor(None, None, 10, -1.0, 1.0, 8, 0, None) == -1
    assert lib.aq_qdq_per_tensor(None, None, 0, -1.0, 1.0, 8, 1, None) == -2      # stochastic rounding
    assert lib.aq_qdq_per_tensor(None, None, -1, -1.0, 1.0, 8, 0, None) == -1
    assert lib.aq_v2_quantize(None, None, None, 0, 8, 1, 8, None, None, 0.0, 255.0, 0, 0, None) == -1
    assert lib.aq_minmax(None, 0, 8, 3, 3, None, None, 0, 0, None, 0, None) == -1   # 8 % 3 != 0
    assert lib.aq_tfe_search(None, None, 0, 8, 0, 0, 0, None, None, 0, None) == -1
    assert lib.aq_minmax_workspace_bytes(1 << 20, 1, 1 << 20) >= 256
    assert lib.aq_tfe_search_workspace_bytes() % 256 == 0


def test_python_layers_refuse_cpu_tensors():
    import torch
    from aimet_b200 import libpymo, ops
    import aimet_b200.v2.backend as b200
    x = torch.randn(16)
    with pytest.raises(RuntimeError):
        ops.qdq_per_tensor(x, -1, 1, 8)
    with pytest.raises(RuntimeError):
        ops.minmax(x)
    with pytest.raises(RuntimeError):
        b200.quantize_dequantize(x, torch.ones(1), torch.zeros(1), 0, 255)
    with pytest.raises(RuntimeError):
        libpymo.AimetTensorQuantizer(libpymo.QUANTIZATION_TF).updateStats(x, True)


def test_v2_geometry_resolution():
    """Pure host logic: how tensor layouts and encoding shapes map to (num_ch, inner)."""
    import torch
    from aimet_b200.v2.backend import resolve_geometry
    g = resolve_geometry(torch.empty(512, 256, 3, 3), (512, 1, 1, 1), None)
    assert (g.num_ch, g.inner, g.order) == (512, 2304, None)
    g = resolve_geometry(torch.empty(8, 16, 14, 14), (1, 16, 1, 1), None)
    assert (g.num_ch, g.inner) == (16, 196)
    g = resolve_geometry(torch.empty(8, 16, 14, 14).contiguous(memory_format=torch.channels_last), (1, 16, 1, 1), None)
    assert (g.num_ch, g.inner) == (16, 1)            # channels are innermost in NHWC memory
    g = resolve_geometry(torch.empty(4096, 11008), (4096, 172), (-1, 64))
    assert (g.num_ch, g.inner) == (4096 * 172, 64)
    g = resolve_geometry(torch.empty(64, 32, 3, 3), (64, 8, 1, 1), (1, 4, -1, -1))
    assert (g.num_ch, g.inner) == (64 * 8, 4 * 9)
    g = resolve_geometry(torch.empty(10, 20), (1,), None)
    assert (g.num_ch, g.inner) == (1, 200)
    g = resolve_geometry(torch.empty(4, 5, 3), (4, 1, 3), None)
    assert g.order is not None and (g.num_ch, g.inner) == (12, 5)
