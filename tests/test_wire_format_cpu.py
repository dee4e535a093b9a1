"""Tensor subclasses that carry an encoding: which operations keep it, drop it or return a plain tensor.  Expected
classes come from the reference's own QuantizedTensor / DequantizedTensor (tests/golden/v2_wire_format.json, see
gen_golden.py); no kernel runs here, so the rules are checked without a GPU."""
import importlib.util
import json
import os

import pytest
import torch

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
FIX = json.load(open(os.path.join(GOLDEN, "v2_wire_format.json")))


def _ops():
    spec = importlib.util.spec_from_file_location("_gen_golden", os.path.join(GOLDEN, "gen_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.wire_format_ops()


@pytest.mark.parametrize("tag,shape", [("pertensor", ()), ("perchannel", (4, 1))])
def test_encoding_propagation_rules(tag, shape):
    from aimet_b200.v2.qtensor import DequantizedTensor
    from aimet_b200.v2.quantizer import AffineEncoding
    x = torch.randn(4, 6).as_subclass(DequantizedTensor)
    x.encoding = AffineEncoding(torch.full(shape, 0.1), torch.full(shape, -128.0), 0, 255)
    for name, fn in _ops():
        want = FIX["ops"][f"{tag}/{name}"]
        got = fn(x)
        assert type(got).__name__ == want["class"], (tag, name)
        assert (getattr(got, "encoding", None) is not None) == want["has_encoding"], (tag, name)
    assert x.encoding is not None   # none of the operations touched the source tensor


def test_integer_dtype_is_rejected():
    from aimet_b200.v2.qtensor import QuantizedTensor
    from aimet_b200.v2.quantizer import AffineEncoding
    q = torch.arange(4.0).as_subclass(QuantizedTensor)
    q.encoding = AffineEncoding(torch.tensor(0.5), torch.tensor(0.0), 0, 255)
    with pytest.raises(RuntimeError, match="non-floating point"):
        q.to(torch.int32)
    with pytest.raises(RuntimeError):
        QuantizedTensor(torch.arange(4))
    assert q.quantize() is q


def test_missing_encoding_raises():
    from aimet_b200.v2.qtensor import DequantizedTensor, EncodingError
    x = torch.randn(3).as_subclass(DequantizedTensor)
    with pytest.raises(EncodingError):
        x.quantize()
    with pytest.raises(EncodingError):
        x.quantized_repr()
    assert x.dequantize() is x


def test_grid_properties_follow_reference_rules():
    from aimet_b200.v2.quantizer import AffineEncoding
    s, o = torch.tensor(1.0), torch.tensor(0.0)
    assert AffineEncoding(s, o, 0, 255).dtype == torch.uint8 and AffineEncoding(s, o, -128, 127).dtype == torch.int8
    assert AffineEncoding(s, o, -100, 27).dtype == torch.int8 and AffineEncoding(s, o, 0, 65535).dtype == torch.int32
    assert AffineEncoding(s, o, -32768, 32767).dtype == torch.int16
    assert AffineEncoding(s, o, -8, 7).bitwidth == 4 and AffineEncoding(s, o, -8, 7).signed
    with pytest.raises(RuntimeError, match="undefined"):
        AffineEncoding(s, o, -100, 27).bitwidth   # pylint: disable=expression-not-assigned
    with pytest.raises(RuntimeError, match="floating point"):
        AffineEncoding(s, o, 0, 255).to(torch.int8)
