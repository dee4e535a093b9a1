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


@pytest.mark.parametrize("cls_name", ["QuantizedTensor", "DequantizedTensor"])
def test_copies_keep_class_and_encoding(cls_name):
    """Deep copies (copy.deepcopy, pickle) are tensors of the same class with a copy of the encoding; a shallow copy
    shares storage and the encoding object (the reference's test_tensor.py:511-564)."""
    import copy
    import pickle
    from aimet_b200.v2 import qtensor
    from aimet_b200.v2.quantizer import AffineEncoding
    cls = getattr(qtensor, cls_name)
    for data in (torch.randn(5, 5), torch.nn.Parameter(torch.randn(5, 5))):
        t = data.detach().clone().as_subclass(cls)
        t.encoding = AffineEncoding(torch.tensor(0.1), torch.tensor(-10.0), 8)   # (bitwidth[, signed]) form
        assert (t.encoding.qmin, t.encoding.qmax) == (0, 255) and not t.encoding.signed
        for deep in (copy.deepcopy, lambda v: pickle.loads(pickle.dumps(v))):
            c = deep(t)
            assert type(c) is cls and torch.equal(c, t) and c.data_ptr() != t.data_ptr()
            assert c.requires_grad == t.requires_grad and c.dtype == t.dtype and c.stride() == t.stride()
            assert c.encoding is not t.encoding and torch.equal(c.encoding.scale, t.encoding.scale)
            assert c.encoding.bitwidth == t.encoding.bitwidth and c.encoding.signed == t.encoding.signed
        c = copy.copy(t)
        assert type(c) is cls and c.data_ptr() == t.data_ptr() and c.encoding is t.encoding


def test_encoding_constructor_forms():
    from aimet_b200.v2.quantizer import AffineEncoding
    s, o = torch.tensor(0.5), torch.tensor(0.0)
    assert (AffineEncoding(s, o, 4, True).qmin, AffineEncoding(s, o, 4, True).qmax) == (-8, 7)
    assert (AffineEncoding(s, o, -100, 27).qmin, AffineEncoding(s, o, -100, 27).qmax) == (-100, 27)
    e = AffineEncoding(s, o, bitwidth=8, signed=False, symmetry=True, block_size=(1, 4))
    assert (e.qmin, e.qmax, e.symmetry, e.block_size) == (0, 255, True, (1, 4))
    with pytest.raises(ValueError):
        AffineEncoding(s, o, 5, 5)
    with pytest.raises(TypeError):
        AffineEncoding(s, o, 0, 255, nonsense=1)

