"""Encodings as exported dictionaries, and quantizer outputs that carry their encoding, against the reference's own
classes (tests/golden/v2_wire_format.json; calibration inputs from v2_quantizer.npz -- both written by gen_golden.py)."""
import json
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
FIX = json.load(open(os.path.join(GOLDEN, "v2_wire_format.json")))
DATA = np.load(os.path.join(GOLDEN, "v2_quantizer.npz"))

CASES = {
    "pt_a8": ("qdq", ((), 8, False), {}), "pt_s4_codes": ("q", ((), 4, True), {}),
    "pc_w8": ("qdq", ((6, 1, 1, 1), 8, True), {}), "pc_axis1_qminqmax": ("qdq", ((1, 5, 1, 1), -100, 27, False), {}),
    "blk_w4": ("qdq", ((12, 4), 4, True), {"block_size": (-1, 8)}), "pt_a16": ("qdq", ((), 16, False), {}),
}


def _calibrated(name):
    from aimet_b200.v2.quantizer import Quantize, QuantizeDequantize
    kind, args, kwargs = CASES[name]
    q = (QuantizeDequantize if kind == "qdq" else Quantize)(*args, **kwargs).cuda()
    with torch.no_grad(), q.compute_encodings():
        b = 0
        while f"{name}/batch{b}" in DATA:
            q(torch.from_numpy(DATA[f"{name}/batch{b}"]).cuda())
            b += 1
    return q, torch.from_numpy(DATA[f"{name}/probe"]).cuda()


@pytest.mark.parametrize("name", sorted(CASES))
def test_legacy_encodings_and_tensor_subclasses(name):
    from aimet_b200.v2.qtensor import DequantizedTensor, QuantizedTensor
    want = FIX["quantizers"][name]
    q, probe = _calibrated(name)
    enc = q.get_encoding()
    assert str(enc.dtype) == want["encoding_dtype"]
    with torch.no_grad():
        y = q(probe)
    rep = y.quantized_repr()
    assert type(rep) is torch.Tensor and str(rep.dtype) == want["quantized_repr_dtype"]
    assert rep.flatten().tolist() == want["quantized_repr"]
    if "legacy_error" in want:
        with pytest.raises(RuntimeError):
            q.get_legacy_encodings()
        return
    assert type(y).__name__ == want["out_class"] and isinstance(y, (QuantizedTensor, DequantizedTensor))
    assert enc.granularity == want["granularity"] and enc.bitwidth == want["bitwidth"] and enc.signed == want["signed"]
    assert q.get_legacy_encodings() == want["legacy"]   # floats compare exactly: same fp32 values widened to double
    dq = y.dequantize()
    assert isinstance(dq, DequantizedTensor) and dq.encoding is not None
    assert dq.as_subclass(torch.Tensor).flatten().tolist() == want["dequantized"]
    rq = dq.quantize()
    assert isinstance(rq, QuantizedTensor)
    assert rq.as_subclass(torch.Tensor).flatten().tolist() == want["requantized"]


@pytest.mark.parametrize("name", sorted(n for n in CASES if "legacy" in FIX["quantizers"][n]))
def test_legacy_encodings_reimport(name):
    from aimet_b200.v2.quantizer import Quantize, QuantizeDequantize
    want = FIX["quantizers"][name]
    kind, args, kwargs = CASES[name]
    q2 = (QuantizeDequantize if kind == "qdq" else Quantize)(args[0], 8, False, **kwargs).cuda()
    q2.set_legacy_encodings(want["legacy"])
    r = want["reimport"]
    assert (q2.qmin, q2.qmax, q2.symmetric) == (r["qmin"], r["qmax"], r["symmetric"])
    assert q2.min.flatten().tolist() == r["min"] and q2.max.flatten().tolist() == r["max"]
    assert q2.get_scale().flatten().tolist() == r["scale"] and q2.get_offset().flatten().tolist() == r["offset"]
    assert q2.get_legacy_encodings() == r["legacy"]


def test_plain_outputs_switch():
    q, probe = _calibrated("pt_a8")
    q.plain_outputs = True
    assert type(q(probe)) is torch.Tensor


def test_sim_export_and_load_round_trip(tmp_path):
    """Encodings written by one simulation and loaded into a fresh one reproduce its outputs bit for bit; the loaded
    quantizers are frozen against a later calibration; strict / partial behave as documented."""
    from aimet_b200.v2.quantsim import QuantizationSimModel
    torch.manual_seed(3)
    model = torch.nn.Sequential(torch.nn.Conv2d(3, 8, 3), torch.nn.ReLU(), torch.nn.Conv2d(8, 4, 3)).cuda().eval()
    x = torch.randn(4, 3, 16, 16, device="cuda")
    sim = QuantizationSimModel(model, x, quant_scheme="post_training_tf")
    sim.compute_encodings(lambda m, _: m(x))
    path = sim.export_encodings(str(tmp_path), "net")
    saved = json.load(open(path))
    assert set(saved) == {"version", "activation_encodings", "param_encodings", "excluded_layers"}
    assert len(saved["param_encodings"]["0.weight"]) == 8 and saved["param_encodings"]["0.weight"][0]["is_symmetric"] == "True"
    assert all(set(v) <= {"input", "output"} for v in saved["activation_encodings"].values())
    want = sim.model(x)

    sim2 = QuantizationSimModel(model, x, quant_scheme="post_training_tf")
    sim2.load_encodings(path, allow_overwrite=False)
    assert torch.equal(sim2.model(x), want)
    sim2.compute_encodings(lambda m, _: m(x * 3))   # frozen: calibration must not move anything
    assert torch.equal(sim2.model(x), want)

    bad = dict(saved, param_encodings=dict(saved["param_encodings"], **{"nope.weight": saved["param_encodings"]["0.weight"]}))
    with pytest.raises(RuntimeError, match="nope.weight"):
        QuantizationSimModel(model, x, quant_scheme="post_training_tf").load_encodings(bad)
    sim3 = QuantizationSimModel(model, x, quant_scheme="post_training_tf")
    only_params = {"param_encodings": saved["param_encodings"], "activation_encodings": {}}
    sim3.load_encodings(only_params, partial=False)   # activation quantizers are removed
    assert not sim3.activation_quantizers
    assert sim3.model(x).shape == want.shape
