"""Generates the golden fixtures in this directory from the REFERENCE ITSELF (run where a reference checkout and
oracle/_ref exist; the fixtures are committed so that the tests need neither).

    python tests/golden/gen_golden.py /path/to/aimet        (or AIMET_REFERENCE_ROOT=/path/to/aimet)

* v2_backend.npz   - aimet_torch v2 ``torch_builtins`` (loaded by file path, CPU) on seeded inputs:
                     quantize / quantize_dequantize / dequantize outputs, clamp masks (from dx with unit grads),
                     and un-reduced-then-summed scale / offset gradients.
* v2_minmax.npz    - aimet_torch v2 ``MinMaxEncodingAnalyzer`` encodings (CPU).
* v2_quantizer.npz - aimet_torch v2 ``Quantize`` / ``QuantizeDequantize`` modules (affine/quantizer.py loaded by path,
                     CPU): outputs inside the calibration context (dynamic encodings), calibrated min / max /
                     scale / offset, outputs after calibration.
* v2_wire_format.json - the legacy encoding dicts (``get_legacy_encodings``), their re-import
                     (``set_legacy_encodings``), ``quantized_repr`` / ``dequantize`` of quantizer outputs and the class /
                     encoding that results from operations on them, from the reference's own quantizer and tensor
                     classes (CPU).
* v1_range_learning.npz - aimet_torch v1 learned-grid functions ``calculate_forward_pass`` / ``calculate_gradients``
                     (v1/quantsim_straight_through_grad.py loaded by path, CPU): outputs, dx, min / max gradients.
* v2_backend_reference_tests.npz - the data of the reference's OWN backend test file
                     (test/python/v2/quantization/affine/backends/test_backend.py, loaded by path): its six
                     known-answer vector sets, its block-quantization cases, and the inputs / expected values of its
                     gradient-comparison tests as that file builds them (same seed, same helpers), with the expected
                     values computed on CPU by the reference's plain-autograd modules and by ``torch_builtins``.
* v2_sqnr.npz      - aimet_torch v2 ``SqnrEncodingAnalyzer`` / ``_HistogramObserver`` (encoding_analyzer.py loaded by path,
                     CPU): per-batch histograms, the merged histogram / bin edges / min / max after every update,
                     dynamic and final encodings for several grids; includes the tensors of the reference's own
                     histogram tests.
* histc_rule.npz   - the installed ``torch.histc`` CPU operator on values on, just below and just above every bin
                     boundary (the operator is third-party code: its bin rule is pinned by execution).
* v1_ste.npz       - aimet_torch v1 straight-through gradient ``compute_dloss_by_dx`` (same file, CPU): per tensor
                     and per channel on axis 0 / 1, with inputs exactly on the encoding bounds.
* libpymo.npz      - the reference DlQuantization CPU code (oracle/_ref): per-tensor QDQ / codes, TF and
                     TF-Enhanced encodings, per-batch histograms, on seeded inputs.
"""
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def load_reference_v2(ref_root: str):
    """Loads the three hot-path files of aimet_torch.v2 by path.  The package itself cannot be imported here
    (it pulls in bokeh, onnx, spconv ...), so empty parent packages and an identity stub for the ONNX symbolic
    decorator are registered first."""
    at = os.path.join(ref_root, "TrainingExtensions", "torch", "src", "python", "aimet_torch")
    for name in ("aimet_torch", "aimet_torch.v2", "aimet_torch.v2.quantization", "aimet_torch.v2.quantization.affine",
                 "aimet_torch.v2.quantization.affine.backends", "aimet_torch.v2.experimental",
                 "aimet_torch.v2.experimental.onnx"):
        if name not in sys.modules:
            m = types.ModuleType(name)
            m.__path__ = []
            sys.modules[name] = m
    exp = types.ModuleType("aimet_torch.v2.experimental.onnx._export")
    exp.register_symbolic = lambda sym: (lambda fn: fn)
    for n in ("quantize_symbolic", "dequantize_symbolic", "quantize_dequantize_symbolic"):
        setattr(exp, n, None)
    sys.modules[exp.__name__] = exp
    sys.modules["aimet_torch.v2.experimental.onnx"]._export = exp

    def load(modname, relpath):
        spec = importlib.util.spec_from_file_location(modname, os.path.join(at, relpath))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[modname] = mod
        spec.loader.exec_module(mod)
        return mod

    utils = load("aimet_torch.v2.utils", "v2/utils.py")
    tb = load("aimet_torch.v2.quantization.affine.backends.torch_builtins",
              "v2/quantization/affine/backends/torch_builtins.py")
    ea = load("aimet_torch.v2.quantization.encoding_analyzer", "v2/quantization/encoding_analyzer.py")
    return utils, tb, ea


def v2_cases():
    """(name, tensor, scale, offset, qmin, qmax, block_size) -- small, seeded, with ties and out-of-range values."""
    g = torch.Generator().manual_seed(1234)
    cases = []

    def rnd(*shape, s=1.0):
        return torch.randn(*shape, generator=g) * s

    ties = torch.tensor([0.25, 0.75, 1.25, -0.25, -0.75, 63.75, -64.25, 1000.0, -1000.0, 0.0])
    for dt in (torch.float32, torch.float16, torch.bfloat16):
        for bw, signed in ((8, False), (8, True), (4, True), (16, False)):
            steps = 2 ** bw - 1
            qmin, qmax = (-(steps + 1) // 2, steps // 2) if signed else (0, steps)
            x = torch.cat([rnd(300, s=3.0), ties]).to(dt)
            scale = torch.tensor(0.5 if bw < 16 else 0.001)
            offset = torch.tensor(0.0 if signed else float(-(steps // 2)))
            cases.append((f"pt_{str(dt)[6:]}_b{bw}{'s' if signed else 'u'}", x, scale, offset, qmin, qmax, None))
    # per-channel (axis 0) conv-like weight and per-channel on axis 1 of an activation
    w = rnd(6, 4, 3, 3, s=0.2)
    sc = (w.abs().amax(dim=(1, 2, 3), keepdim=True) / 127)
    cases.append(("pc_w_f32", w, sc, torch.zeros_like(sc), -128, 127, None))
    a = rnd(3, 5, 4, 2, s=2.0)
    sc = torch.linspace(0.01, 0.05, 5).view(1, 5, 1, 1)
    of = torch.tensor([-128., -100., -90., -128., -5.]).view(1, 5, 1, 1)
    cases.append(("pc_act_axis1_f32", a, sc, of, 0, 255, None))
    cases.append(("pc_act_axis1_cl_f32", a.contiguous(memory_format=torch.channels_last), sc, of, 0, 255, None))
    # blockwise [O, I] with block 8 on the input dim, W4 symmetric, bf16 (the LLM weight case, scaled down)
    wb = (rnd(12, 32, s=0.02)).to(torch.bfloat16)
    sb = (wb.float().view(12, 4, 8).abs().amax(dim=2) / 7).clamp_min(1e-6)
    cases.append(("blk_bf16_w4", wb, sb, torch.zeros_like(sb), -8, 7, (-1, 8)))
    cases.append(("blk_f32_w4", wb.float(), sb, torch.zeros_like(sb), -8, 7, (1, 8)))
    # conv weight blocked on input channels: [O, I, kh, kw], block (1, 4, -1, -1)
    wc = rnd(4, 8, 3, 3, s=0.1)
    sc4 = (wc.view(4, 2, 4, 3, 3).abs().amax(dim=(2, 3, 4)) / 7).view(4, 2, 1, 1)
    cases.append(("blk_conv_f32", wc, sc4, torch.zeros_like(sc4), -8, 7, (1, 4, -1, -1)))
    # encodings interleaved with broadcast dims: scale [4,1,3]
    t3 = rnd(4, 5, 3)
    s3 = torch.linspace(0.02, 0.2, 12).view(4, 1, 3)
    cases.append(("interleaved_f32", t3, s3, torch.full_like(s3, -100.0), 0, 255, None))
    return cases


def gen_v2(ref_root: str):
    _, tb, ea = load_reference_v2(ref_root)
    out = {}
    for name, x, scale, offset, qmin, qmax, bs in v2_cases():
        out[f"{name}/x"] = x.float().numpy()
        out[f"{name}/dtype"] = np.array(str(x.dtype))
        out[f"{name}/scale"] = scale.numpy()
        out[f"{name}/offset"] = offset.numpy()
        out[f"{name}/q"] = np.array([qmin, qmax])
        out[f"{name}/block"] = np.array(bs if bs is not None else [], dtype=np.int64)
        out[f"{name}/channels_last"] = np.array(x.dim() == 4 and not x.is_contiguous())
        xr = x.clone().requires_grad_(True)
        sr = scale.clone().requires_grad_(True)
        orr = offset.clone().requires_grad_(True)
        y = tb.quantize_dequantize(xr, sr, orr, qmin, qmax, bs)
        gy = torch.randn(y.shape, generator=torch.Generator().manual_seed(7)).to(y.dtype)
        y.backward(gy)
        out[f"{name}/qdq"] = y.detach().float().numpy()
        out[f"{name}/gy"] = gy.float().numpy()
        out[f"{name}/dx"] = xr.grad.float().numpy()
        out[f"{name}/dscale"] = sr.grad.float().numpy()
        out[f"{name}/doffset"] = orr.grad.float().numpy()
        ones = torch.ones_like(x)
        xm = x.clone().requires_grad_(True)
        tb.quantize_dequantize(xm, scale, offset, qmin, qmax, bs).backward(ones)
        out[f"{name}/mask"] = (xm.grad.float().numpy() != 0)
        if tb._is_grid_representable(x.dtype, qmin, qmax):
            q = tb.quantize(x, scale, offset, qmin, qmax, bs)
            out[f"{name}/codes"] = q.float().numpy()
            out[f"{name}/deq"] = tb.dequantize(q, scale, offset, bs).float().numpy()
    np.savez_compressed(os.path.join(HERE, "v2_backend.npz"), **out)

    mm = {}
    k = 0
    for dt in (torch.float32, torch.bfloat16):
        for shape, enc_shape in (((64, 33), (1,)), ((8, 4, 3, 3), (8, 1, 1, 1)), ((6, 16), (6, 2))):
            for steps, sym in ((255, False), (255, True), (15, True), (65535, False)):
                g = torch.Generator().manual_seed(100 + k)
                x = (torch.randn(*shape, generator=g) * 2 + (0.5 if not sym else 0)).to(dt)
                if enc_shape == (6, 2):
                    an = ea.MinMaxEncodingAnalyzer((6, 2, 1))
                    xin = x.view(6, 2, 8)
                else:
                    an = ea.MinMaxEncodingAnalyzer(enc_shape)
                    xin = x
                an.update_stats(xin)
                an.update_stats(xin * 0.5 + 0.1)
                mn, mx = an.compute_encodings(steps, sym)
                mm[f"c{k}/x"] = x.float().numpy()
                mm[f"c{k}/meta"] = np.array([str(dt), str(list(enc_shape)), str(steps), str(int(sym))])
                mm[f"c{k}/min"] = mn.float().numpy()
                mm[f"c{k}/max"] = mx.float().numpy()
                k += 1
    np.savez_compressed(os.path.join(HERE, "v2_minmax.npz"), **mm)


def load_reference_quantizer(ref_root: str):
    """Loads aimet_torch/v2/quantization/affine/quantizer.py and what it imports, by path (after load_reference_v2)."""
    at = os.path.join(ref_root, "TrainingExtensions", "torch", "src", "python", "aimet_torch")

    def load(modname, relpath, pkg=False):
        path = os.path.join(at, relpath)
        spec = importlib.util.spec_from_file_location(modname, path,
                                                      submodule_search_locations=[os.path.dirname(path)] if pkg else None)
        mod = importlib.util.module_from_spec(spec)
        sys.modules[modname] = mod
        spec.loader.exec_module(mod)
        return mod

    q = "aimet_torch.v2.quantization"
    load(q + ".affine.backends.utils", "v2/quantization/affine/backends/utils.py")
    load(q + ".affine.backends", "v2/quantization/affine/backends/__init__.py", pkg=True)
    benc = load(q + ".base.encoding", "v2/quantization/base/encoding.py")
    base = types.ModuleType(q + ".base")
    base.__path__ = []
    sys.modules[q + ".base"] = base
    base.EncodingBase = benc.EncodingBase
    base.QuantizerBase = load(q + ".base.quantizer", "v2/quantization/base/quantizer.py").QuantizerBase
    load(q + ".affine._utils", "v2/quantization/affine/_utils.py")
    aenc = load(q + ".affine.encoding", "v2/quantization/affine/encoding.py")
    load(q + ".tensor", "v2/quantization/tensor.py")
    sys.modules[q + ".affine"].AffineEncoding = aenc.AffineEncoding
    sys.modules[q + ".affine"].VectorEncoding = getattr(aenc, "VectorEncoding", None)
    return load(q + ".affine.quantizer", "v2/quantization/affine/quantizer.py")


def quantizer_cases():
    """(name, kind, ctor args, ctor kwargs, calibration batches, probe input)."""
    g = torch.Generator().manual_seed(77)

    def rnd(*shape, s=1.0):
        return torch.randn(*shape, generator=g) * s

    return [
        ("pt_a8", "qdq", ((), 8, False), {}, [rnd(4, 8, 5, 5, s=k) for k in (1.0, 2.5, 0.5)], rnd(4, 8, 5, 5, s=3.0)),
        ("pt_s4_codes", "q", ((), 4, True), {}, [rnd(64, 33, s=k) for k in (0.3, 0.2)], rnd(64, 33, s=0.4)),
        ("pc_w8", "qdq", ((6, 1, 1, 1), 8, True), {}, [rnd(6, 4, 3, 3, s=0.2)], rnd(6, 4, 3, 3, s=0.25)),
        ("pc_axis1_qminqmax", "qdq", ((1, 5, 1, 1), -100, 27, False), {}, [rnd(3, 5, 4, 2, s=k) for k in (1.0, 2.0)],
         rnd(3, 5, 4, 2, s=2.0)),
        ("blk_w4", "qdq", ((12, 4), 4, True), {"block_size": (-1, 8)}, [rnd(12, 32, s=0.02)], rnd(12, 32, s=0.03)),
        ("blk_w4_bf16", "qdq", ((12, 4), 4, True), {"block_size": (1, 8)}, [rnd(12, 32, s=0.02).to(torch.bfloat16)],
         rnd(12, 32, s=0.03).to(torch.bfloat16)),
        ("pt_a16", "qdq", ((), 16, False), {}, [rnd(2048, s=k) for k in (1.0, 4.0)], rnd(2048, s=5.0)),
        # grouped blocks (LPBQ): 4-bit blocks of 8 decompressed to 8 bits, groups of 2 blocks / all blocks of a row
        ("gbq_w4_g2", "gbq", ((12, 4), 4, True, 8), {"block_size": (-1, 8), "block_grouping": (1, 2)},
         [rnd(12, 32, s=0.02)], rnd(12, 32, s=0.03)),
        ("gbq_w4_all", "gbq", ((12, 4), 4, True, 8), {"block_size": (1, 8), "block_grouping": (1, -1)},
         [rnd(12, 32, s=0.05)], rnd(12, 32, s=0.05)),
        ("gbq_w4_rows", "gbq", ((12, 4), 4, True, 6), {"block_size": (1, 8), "block_grouping": (3, 4)},
         [rnd(12, 32, s=0.02) * torch.linspace(0.2, 3.0, 12).view(12, 1)], rnd(12, 32, s=0.03)),
    ]


def gen_quantizer(ref_root: str):
    load_reference_v2(ref_root)
    rq = load_reference_quantizer(ref_root)
    out = {}
    for name, kind, args, kwargs, batches, probe in quantizer_cases():
        q = {"qdq": rq.QuantizeDequantize, "q": rq.Quantize, "gbq": rq.GroupedBlockQuantizeDequantize}[kind](*args, **kwargs)
        with torch.no_grad():
            with q.compute_encodings():
                for b, x in enumerate(batches):
                    out[f"{name}/batch{b}"] = x.float().numpy()
                    out[f"{name}/dyn{b}"] = q(x).as_subclass(torch.Tensor).float().numpy()
            out[f"{name}/min"] = q.min.detach().numpy()
            out[f"{name}/max"] = q.max.detach().numpy()
            out[f"{name}/scale"] = q.get_scale().detach().numpy()
            out[f"{name}/offset"] = q.get_offset().detach().numpy()
            out[f"{name}/probe"] = probe.float().numpy()
            out[f"{name}/out"] = q(probe).as_subclass(torch.Tensor).float().numpy()
            if kind == "gbq":
                out[f"{name}/per_channel_scale"] = q.get_per_channel_scale().numpy()
                out[f"{name}/integer_scale"] = q.get_per_block_integer_scale().numpy()
        out[f"{name}/dtype"] = np.array(str(probe.dtype))
    np.savez_compressed(os.path.join(HERE, "v2_quantizer.npz"), **out)


def wire_format_ops():
    """(name, function) -- operations applied to a quantizer output; the fixture records what class and encoding the
    reference's tensor subclasses give the result."""
    return [
        ("float16", lambda t: t.to(torch.float16)), ("double", lambda t: t.double()),
        ("contiguous", lambda t: t.contiguous()),
        ("view", lambda t: t.view(-1)), ("getitem", lambda t: t[0]), ("permute", lambda t: t.permute(1, 0)),
        ("flatten_fn", lambda t: torch.flatten(t)), ("chunk", lambda t: t.chunk(2)[1]),
        ("add", lambda t: t + 1.0), ("radd", lambda t: torch.ones(()) + t), ("mul_tensor", lambda t: t * t),
        ("relu", lambda t: torch.relu(t)), ("add_", lambda t: t.clone().add_(1.0)),
        ("clone", lambda t: t.clone()), ("detach", lambda t: t.detach()),
    ]


def gen_wire_format(ref_root: str):
    """v2_wire_format.json: legacy encoding dicts, their re-import, and tensor-subclass behaviour, all produced by the
    reference's own ``Quantize`` / ``QuantizeDequantize`` / ``QuantizedTensor`` classes (CPU)."""
    import json
    load_reference_v2(ref_root)
    rq = load_reference_quantizer(ref_root)
    out = {"quantizers": {}, "ops": {}}
    for name, kind, args, kwargs, batches, probe in quantizer_cases():
        if batches[0].dtype != torch.float32 or kind == "gbq":
            continue
        cls = rq.QuantizeDequantize if kind == "qdq" else rq.Quantize
        q = cls(*args, **kwargs)
        with torch.no_grad():
            with q.compute_encodings():
                for x in batches:
                    q(x)
            enc = q.get_encoding()
            y = q(probe)
            try:
                legacy = q.get_legacy_encodings()
            except RuntimeError:
                # a grid that is not a power of two has no bit-width, hence no legacy form
                out["quantizers"][name] = {"legacy_error": "RuntimeError", "encoding_dtype": str(enc.dtype),
                                           "quantized_repr": y.quantized_repr().flatten().tolist(),
                                           "quantized_repr_dtype": str(y.quantized_repr().dtype)}
                continue
            rec = {"legacy": legacy, "encoding_dtype": str(enc.dtype), "granularity": enc.granularity,
                   "bitwidth": enc.bitwidth, "signed": bool(enc.signed), "out_class": type(y).__name__,
                   "quantized_repr": y.quantized_repr().flatten().tolist(),
                   "quantized_repr_dtype": str(y.quantized_repr().dtype),
                   "dequantized": y.dequantize().as_subclass(torch.Tensor).flatten().tolist(),
                   "requantized": y.dequantize().quantize().as_subclass(torch.Tensor).flatten().tolist()}
            # a fresh quantizer of the same shape takes the exported dicts back
            q2 = cls(args[0], 8, False, **kwargs)   # grid and symmetry come from the dicts
            q2.set_legacy_encodings(legacy)
            rec["reimport"] = {"qmin": q2.qmin, "qmax": q2.qmax, "symmetric": bool(q2.symmetric),
                               "min": q2.min.flatten().tolist(), "max": q2.max.flatten().tolist(),
                               "scale": q2.get_scale().flatten().tolist(), "offset": q2.get_offset().flatten().tolist(),
                               "legacy": q2.get_legacy_encodings()}
        out["quantizers"][name] = rec
    # propagation rules on a per-tensor and a per-channel output
    g = torch.Generator().manual_seed(5)
    x = torch.randn(4, 6, generator=g)
    for tag, shape in (("pertensor", ()), ("perchannel", (4, 1))):
        q = rq.QuantizeDequantize(shape, 8, False)
        with torch.no_grad():
            with q.compute_encodings():
                q(x)
            y = q(x)
            for op, fn in wire_format_ops():
                r = fn(y)
                out["ops"][f"{tag}/{op}"] = {"class": type(r).__name__,
                                             "has_encoding": bool(getattr(r, "encoding", None) is not None)}
    with open(os.path.join(HERE, "v2_wire_format.json"), "w") as f:
        json.dump(out, f, sort_keys=True)


def range_learning_cases():
    """(name, tensor, encoding_min, encoding_max, bitwidth, symmetric, strict, unsigned, channel_axis)."""
    g = torch.Generator().manual_seed(4242)

    def rnd(*shape, s=1.0):
        return torch.randn(*shape, generator=g) * s

    x = rnd(5, 6, 7, 3, s=2.0)
    w = rnd(8, 4, 3, 3, s=0.3)
    pc_min = -torch.linspace(0.3, 0.9, 8)
    pc_max = torch.linspace(0.4, 1.0, 8)
    return [
        ("pt_a8", x, torch.tensor([-3.3]), torch.tensor([4.1]), 8, False, False, False, 0),
        ("pt_a4", x, torch.tensor([-1.0]), torch.tensor([2.0]), 4, False, False, False, 0),
        ("pt_s8", x, torch.tensor([-3.5]), torch.tensor([3.5]), 8, True, False, False, 0),
        ("pt_s8_strict", x, torch.tensor([-3.5]), torch.tensor([3.5]), 8, True, True, False, 0),
        ("pt_u8_unsigned_sym", x.abs(), torch.tensor([0.0]), torch.tensor([5.0]), 8, True, False, True, 0),
        ("pc_w8_sym", w, -pc_max, pc_max, 8, True, False, False, 0),
        ("pc_w8_asym", w, pc_min, pc_max, 8, False, False, False, 0),
        ("pc_axis1_a8", x, -torch.linspace(1, 3, 6), torch.linspace(2, 4, 6), 8, False, False, False, 1),
        ("bias_1d", rnd(8, s=0.5), pc_min, pc_max, 8, False, False, False, 0),
        ("pt_a16", x, torch.tensor([-6.0]), torch.tensor([7.0]), 16, False, False, False, 0),
        ("pt_a8_bf16", x.to(torch.bfloat16), torch.tensor([-3.3]).to(torch.bfloat16),
         torch.tensor([4.1]).to(torch.bfloat16), 8, False, False, False, 0),
        ("pt_a16_bf16", x.to(torch.bfloat16), torch.tensor([-6.0]).to(torch.bfloat16),
         torch.tensor([7.0]).to(torch.bfloat16), 16, False, False, False, 0),
    ]


def gen_range_learning(ref_root: str):
    at = os.path.join(ref_root, "TrainingExtensions", "torch", "src", "python", "aimet_torch")
    for name in ("aimet_torch", "aimet_torch.v1"):
        if name not in sys.modules:
            m = types.ModuleType(name)
            m.__path__ = []
            sys.modules[name] = m

    def load(modname, relpath):
        spec = importlib.util.spec_from_file_location(modname, os.path.join(at, relpath))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[modname] = mod
        spec.loader.exec_module(mod)
        return mod

    load("aimet_torch.v1.tensor_factory_utils", "v1/tensor_factory_utils.py")
    gf = load("aimet_torch.v1.quantsim_straight_through_grad", "v1/quantsim_straight_through_grad.py")
    out = {}
    gen = torch.Generator().manual_seed(99)
    for name, x, emin, emax, bw, sym, strict, unsigned, axis in range_learning_cases():
        q = types.SimpleNamespace(bitwidth=bw, use_symmetric_encodings=sym, use_strict_symmetric=strict,
                                  is_unsigned_symmetric=unsigned, channel_axis=axis)
        gy = torch.randn(x.shape, generator=gen).to(x.dtype)
        with torch.no_grad():
            y, inter = gf.calculate_forward_pass(x, q, emin, emax)
            dx = inter.mask_tensor * gy
            # the function receives the tensor as the forward pass used it (float32 after the 16-bit upcast)
            xin = x.float() if (x.dtype != torch.float32 and bw >= 16) else x
            gin = gy.float() if (x.dtype != torch.float32 and bw >= 16) else gy
            dmin, dmax = gf.calculate_gradients(xin, gin, inter, axis)
        out[f"{name}/x"] = x.float().numpy()
        out[f"{name}/gy"] = gy.float().numpy()
        out[f"{name}/min"] = emin.float().numpy()
        out[f"{name}/max"] = emax.float().numpy()
        out[f"{name}/cfg"] = np.array([bw, int(sym), int(strict), int(unsigned), axis])
        out[f"{name}/dtype"] = np.array(str(x.dtype))
        out[f"{name}/y"] = y.float().numpy()
        out[f"{name}/dx"] = dx.float().numpy()
        out[f"{name}/dmin"] = dmin.float().numpy()
        out[f"{name}/dmax"] = dmax.float().numpy()
    np.savez_compressed(os.path.join(HERE, "v1_range_learning.npz"), **out)


def gen_reference_backend_tests(ref_root: str):
    """Data of the reference's backend test file, so that its cases can be replayed where the file itself is absent."""
    import random
    _, tb, _ = load_reference_v2(ref_root)
    if "aimet_torch.v2.quantization.affine" in sys.modules:
        sys.modules["aimet_torch.v2.quantization"].affine = sys.modules["aimet_torch.v2.quantization.affine"]
    path = os.path.join(ref_root, "TrainingExtensions", "torch", "test", "python", "v2", "quantization", "affine",
                        "backends", "test_backend.py")
    spec = importlib.util.spec_from_file_location("reference_test_backend", path)
    T = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(T)
    out = {}
    # 1. known-answer vector sets (module-level literals of the test file)
    for name in ("bfloat16_compat_per_tensor_4b_test_set", "bfloat16_compat_per_tensor_8b_test_set",
                 "per_tensor_4b_test_set", "per_tensor_8b_test_set", "per_channel_4b_test_set",
                 "per_channel_8b_test_set"):
        ts = getattr(T, name)
        for f in ("tensor", "tensor_q", "tensor_qdq", "mask", "delta", "offset"):
            out[f"set/{name}/{f}"] = getattr(ts, f).numpy()
        out[f"set/{name}/q"] = np.array([ts.qmin, ts.qmax])

    # 2. gradient comparisons, built exactly as the test file builds them (seed, helper functions, plain-autograd modules)
    def seeded():
        random.seed(19521)
        torch.random.manual_seed(19521)

    seeded()
    session_offset = torch.randint(-5, 5, []).to(torch.float32)   # the file's session fixture
    for kind in ("quantize", "dequantize", "qdq"):
        for qmin, qmax in ((0, 255), (-128, 127)):
            seeded()
            scale = torch.rand([])
            scale[scale == 0.0] = 0.1
            offset = session_offset.detach().clone()
            if kind == "dequantize":
                x = T.get_random_quantized_tensor((2, 3, 4, 5), qmin, qmax)
                module = T.AutogradDequantizationModule(scale, offset)
            else:
                x = T.get_round_safe_quantizable_tensor((2, 3, 4, 5), scale, qmin, qmax)
                module = (T.AutogradQuantizationModule if kind == "quantize" else T.AutogradQuantDequantModule)(
                    scale, offset, qmin, qmax)
            xa = x.detach().clone().requires_grad_(True)
            expected = module(xa)
            grad_in = torch.randn_like(x)
            expected.backward(grad_in)
            key = f"grad/{kind}/{qmin}_{qmax}"
            out[f"{key}/x"], out[f"{key}/scale"], out[f"{key}/offset"] = x.numpy(), scale.numpy(), offset.numpy()
            out[f"{key}/grad_in"], out[f"{key}/y"] = grad_in.numpy(), expected.detach().numpy()
            out[f"{key}/dx"] = xa.grad.numpy()
            out[f"{key}/dscale"], out[f"{key}/doffset"] = module.scale.grad.numpy(), module.offset.grad.numpy()

    # 3. block quantization: the parametrised cases of test_block_quant (inputs and expected codes are its literals)
    marks = [m for m in T.TestQuantizationBackends.test_block_quant.pytestmark if m.name == "parametrize"
             and m.args[0].startswith("scale")]
    inp = torch.tensor([[-1.2, 2.4], [-.6, -.18]])
    out["block/inp"] = inp.numpy()
    for i, (scale, offset, block_size, output) in enumerate(marks[0].args[1]):
        out[f"block/{i}/scale"], out[f"block/{i}/offset"] = scale.numpy(), offset.numpy()
        out[f"block/{i}/block_size"] = np.array(block_size if block_size is not None else [], dtype=np.int64)
        out[f"block/{i}/codes"] = output.numpy()
    out["block/count"] = np.array(len(marks[0].args[1]))
    # test_block_size and test_block_quant_2: shapes as in the file; expected values from torch_builtins on CPU
    for name, ishape, sshape, block_size in (("block_size", (8, 6, 8, 3), (4, 3, 8, 1), [-1, 2, 1, 3]),
                                             ("block_quant_2", (3, 5, 4, 6, 12, 9), (2, 1, 4, 9), [2, 6, 3, 1])):
        seeded()
        if name == "block_size":
            scale = torch.randn(*sshape)
            offset = torch.randint(low=-128, high=127, size=sshape).to(dtype=scale.dtype)
            x = torch.randn(*ishape)
        else:
            x = torch.randn(*ishape)
            scale = torch.randn(*sshape)
            offset = torch.randint(low=-128, high=127, size=sshape).to(dtype=scale.dtype)
        with torch.no_grad():
            q = tb.quantize(x, scale, offset, -128, 127, block_size)
            dq = tb.dequantize(q, scale, offset, block_size)
            qdq = tb.quantize_dequantize(x, scale, offset, -128, 127, block_size)
        out[f"blockcase/{name}/x"], out[f"blockcase/{name}/scale"] = x.numpy(), scale.numpy()
        out[f"blockcase/{name}/offset"] = offset.numpy()
        out[f"blockcase/{name}/block_size"] = np.array(block_size, dtype=np.int64)
        out[f"blockcase/{name}/q"], out[f"blockcase/{name}/dq"], out[f"blockcase/{name}/qdq"] = \
            q.numpy(), dq.numpy(), qdq.numpy()
    np.savez_compressed(os.path.join(HERE, "v2_backend_reference_tests.npz"), **out)


def sqnr_scenarios():
    """(name, observer shape, num_bins, analyzer kwargs, list of batches)."""
    g = torch.Generator().manual_seed(77)

    def relu(n, seed):
        gg = torch.Generator().manual_seed(seed)
        a = torch.relu(torch.randn(n, generator=gg))
        m = torch.rand(n, generator=gg) < 1e-3
        return torch.where(m, a * 20, a)

    sc = []
    sc.append(("relu_512", (1,), 512, {}, [relu(20000, 1000 + b) for b in range(4)]))
    sc.append(("relu_2048", (1,), 2048, {}, [relu(20000, 1000 + b) for b in range(3)]))
    sc.append(("normal_growing", (), 512, {}, [torch.randn(10000, generator=g) * (1 + b) + 0.3 * b for b in range(4)]))
    sc.append(("shrinking", (1,), 512, {}, [torch.randn(8000, generator=g) * s for s in (4.0, 1.0, 0.25)]))
    sc.append(("negative", (1,), 512, {}, [-torch.rand(8000, generator=g) * 3 - 1, -torch.rand(8000, generator=g) * 5 - 0.5]))
    sc.append(("with_inf_nan", (1,), 512, {}, [torch.cat([torch.randn(5000, generator=g), torch.tensor([float("inf"), -float("inf"), float("nan")])]),
                                               torch.cat([torch.randn(5000, generator=g) * 2, torch.tensor([float("inf"), float("inf")])])]))
    sc.append(("gamma1_uniform", (1,), 2048, {"gamma": 1}, [torch.arange(-100, 101) / 100]))
    # the tensors of the reference's own histogram tests (test_encoding_analyzer.py:286-362), 3 bins
    sc.append(("ref_resize", (), 3, {}, [torch.tensor([2.0, 3.5, 4.2, 5.0]), torch.tensor([5.3, 6.4, 7.0, 8.0]),
                                          torch.tensor([-4.2, 0, 2.3, 4.5])]))
    sc.append(("ref_no_resize", (), 3, {}, [torch.tensor([2.0, 3.5, 4.2, 5.0]), torch.tensor([2.0, 3.3, 4.8, 5]),
                                             torch.tensor([3.1, 3.3, 3.7, 3.9])]))
    sc.append(("ref_ambiguous", (), 3, {}, [torch.tensor([-4.2, 2.4, 7.0, 8.0]), torch.tensor([-6.7, -2.5, 7.2, 10.3])]))
    sc.append(("constant_then_wider", (1,), 16, {}, [torch.full((100,), 2.0), torch.tensor([2.0, 2.0, 2.0])]))
    sc.append(("per_channel", (4, 1), 64, {}, [torch.randn(4, 3000, generator=g) * torch.tensor([[0.5], [1.0], [2.0], [4.0]]),
                                                torch.randn(4, 3000, generator=g) * torch.tensor([[1.0], [1.0], [3.0], [2.0]])]))
    sc.append(("conv_weight_axis0", (6, 1, 1, 1), 128, {}, [torch.randn(6, 8, 3, 3, generator=g) * 0.2]))
    return sc


SQNR_GRIDS = ((255, False), (255, True), (15, False), (15, True), (65535, False), (256.0, False))


def gen_sqnr(ref_root: str):
    _, _, ea = load_reference_v2(ref_root)
    out = {}
    names = []
    for name, shape, bins, kw, batches in sqnr_scenarios():
        an = ea.SqnrEncodingAnalyzer(shape, bins, **kw)
        names.append(name)
        out[f"{name}/shape"] = np.array(shape, dtype=np.int64)
        out[f"{name}/bins"] = np.array(bins)
        out[f"{name}/gamma"] = np.array(float(kw.get("gamma", 3.0)))
        out[f"{name}/num_batches"] = np.array(len(batches))
        for b, x in enumerate(batches):
            out[f"{name}/x{b}"] = x.numpy()
            new = an.update_stats(x)
            for h, st in enumerate(new):
                out[f"{name}/b{b}/batch/{h}/hist"] = st.histogram.numpy()
                out[f"{name}/b{b}/batch/{h}/edges"] = st.bin_edges.numpy()
                out[f"{name}/b{b}/batch/{h}/minmax"] = np.array([st.min.item(), st.max.item()], np.float32)
            for h, st in enumerate(an.observer.get_stats()):
                out[f"{name}/b{b}/state/{h}/hist"] = st.histogram.numpy()
                out[f"{name}/b{b}/state/{h}/edges"] = st.bin_edges.numpy()
                out[f"{name}/b{b}/state/{h}/minmax"] = np.array([st.min.item(), st.max.item()], np.float32)
            for gi, (steps, sym) in enumerate(SQNR_GRIDS):
                mn, mx = an.compute_encodings_from_stats(new, steps, sym)
                out[f"{name}/b{b}/dynamic/{gi}"] = np.stack([mn.reshape(-1).numpy(), mx.reshape(-1).numpy()])
        for gi, (steps, sym) in enumerate(SQNR_GRIDS):
            mn, mx = an.compute_encodings(steps, sym)
            out[f"{name}/final/{gi}"] = np.stack([mn.reshape(-1).numpy(), mx.reshape(-1).numpy()])
    out["names"] = np.array(names)
    out["grids"] = np.array([[float(s), float(y)] for s, y in SQNR_GRIDS])
    np.savez_compressed(os.path.join(HERE, "v2_sqnr.npz"), **out)


def gen_histc_rule():
    """torch.histc (CPU) on boundary values: for random ranges and bin counts, every value that the float32 expression
    lo + k * (hi - lo) / bins produces, its two neighbours, the bounds themselves, and specials."""
    rng = np.random.default_rng(5)
    out = {}
    cases = 0
    for nb in (1, 3, 10, 64, 512, 2048):
        for rep in range(6):
            lo = np.float32(rng.standard_normal() * 10.0 ** rng.integers(-2, 3))
            hi = np.float32(lo + abs(rng.standard_normal()) * 10.0 ** rng.integers(-2, 3) + 1e-3)
            if rep == 0:
                lo, hi = np.float32(0.0), np.float32(abs(hi))     # post-ReLU ranges start at zero
            step = (hi - lo) / np.float32(nb)
            k = rng.integers(0, nb + 1, 600).astype(np.float32)
            e = (lo + k * step).astype(np.float32)
            x = np.concatenate([e, np.nextafter(e, np.float32(np.inf)), np.nextafter(e, np.float32(-np.inf)),
                                (rng.random(3000).astype(np.float32) * (hi - lo) * np.float32(1.2) + lo - np.float32(0.1) * (hi - lo)),
                                np.array([np.nan, np.inf, -np.inf, lo, hi, np.nextafter(hi, np.float32(np.inf)),
                                          np.nextafter(lo, np.float32(-np.inf)), 0.0, -0.0], np.float32)]).astype(np.float32)
            want = torch.histc(torch.from_numpy(x), bins=nb, min=float(lo), max=float(hi)).numpy()
            out[f"c{cases}/x"], out[f"c{cases}/range"], out[f"c{cases}/bins"] = x, np.array([lo, hi], np.float32), np.array(nb)
            out[f"c{cases}/counts"] = want
            cases += 1
    # equal bounds: constant data, and data around the bound
    for val in (2.0, 0.0, -3.5):
        x = np.full(50, val, np.float32)
        out[f"c{cases}/x"], out[f"c{cases}/range"], out[f"c{cases}/bins"] = x, np.array([val, val], np.float32), np.array(8)
        out[f"c{cases}/counts"] = torch.histc(torch.from_numpy(x), bins=8, min=val, max=val).numpy()
        cases += 1
    out["count"] = np.array(cases)
    np.savez_compressed(os.path.join(HERE, "histc_rule.npz"), **out)


def _load_v1_grad(ref_root: str):
    at = os.path.join(ref_root, "TrainingExtensions", "torch", "src", "python", "aimet_torch")
    for name in ("aimet_torch", "aimet_torch.v1"):
        if name not in sys.modules:
            m = types.ModuleType(name)
            m.__path__ = []
            sys.modules[name] = m

    def load(modname, relpath):
        spec = importlib.util.spec_from_file_location(modname, os.path.join(at, relpath))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[modname] = mod
        spec.loader.exec_module(mod)
        return mod

    load("aimet_torch.v1.tensor_factory_utils", "v1/tensor_factory_utils.py")
    return load("aimet_torch.v1.quantsim_straight_through_grad", "v1/quantsim_straight_through_grad.py")


def gen_ste_v1(ref_root: str):
    """compute_dloss_by_dx (aimet_torch/v1/quantsim_straight_through_grad.py:91-118) on seeded inputs."""
    gf = _load_v1_grad(ref_root)
    g = torch.Generator().manual_seed(321)
    out = {}

    def case(name, x, emin, emax, axis):
        grad = torch.randn(x.shape, generator=g)
        dx = gf.compute_dloss_by_dx(x, grad, emin, emax, axis)
        out[f"{name}/x"], out[f"{name}/grad"] = x.numpy(), grad.numpy()
        out[f"{name}/min"], out[f"{name}/max"] = emin.numpy(), emax.numpy()
        out[f"{name}/axis"], out[f"{name}/dx"] = np.array(axis), dx.numpy()

    x = torch.randn(4, 6, 5, 3, generator=g) * 2
    flat = x.view(-1)
    flat[:6] = torch.tensor([-1.5, 2.25, float("nan"), float("inf"), -float("inf"), 0.0])   # bounds, specials
    case("per_tensor", x, torch.tensor([-1.5]), torch.tensor([2.25]), 0)
    case("per_tensor_scalar", x, torch.tensor(-0.75), torch.tensor(0.5), 0)
    mins, maxs = -torch.linspace(0.2, 2.0, 4), torch.linspace(0.3, 2.5, 4)
    x0 = x.clone()
    x0[1, 0, 0, 0], x0[2, 0, 0, 0] = mins[1], maxs[2]
    case("per_channel_axis0", x0, mins, maxs, 0)
    mins, maxs = -torch.linspace(0.1, 3.0, 6), torch.linspace(0.5, 1.0, 6)
    case("per_channel_axis1", x, mins, maxs, 1)
    w = torch.randn(16, 9, generator=g) * 0.3
    case("linear_weight_axis0", w, -w.abs().amax(dim=1) * 0.5, w.abs().amax(dim=1) * 0.5, 0)
    np.savez_compressed(os.path.join(HERE, "v1_ste.npz"), **out)


def gen_libpymo():
    from _data import SPECIALS, conv_weight, normal, relu_activations
    from oracle import Reference, RefAnalyzer
    r = Reference()
    out = {}
    x = np.concatenate([normal(2000, seed=0, scale=2.0), SPECIALS])
    out["qdq/x"] = x
    for i, (mn, mx, bw) in enumerate([(-0.46, 0.72, 8), (-3.1, 4.2, 8), (-2.0, 2.0, 8), (0.0, 5.0, 4), (-7.0, 3.0, 16)]):
        out[f"qdq/{i}/enc"] = np.array([mn, mx, bw])
        out[f"qdq/{i}/y"] = r.qdq_per_tensor(x, mn, mx, bw)
        out[f"qdq/{i}/codes"] = r.quantize_per_tensor(x, mn, mx, bw, False)
        out[f"qdq/{i}/codes_signed"] = r.quantize_per_tensor(x, mn, mx, bw, True)
    # calibration scenarios: (kind, n) batches
    scen = {"relu": [relu_activations(6000, 1000 + b) for b in range(4)],
            "normal": [normal(6000, 50 + b, 2.0, 1.0) for b in range(3)],
            "zeros_then_relu": [np.zeros(3000, np.float32), relu_activations(3000, 7), relu_activations(3000, 8)],
            "negative": [normal(6000, 60 + b, 1.0, -2.0) for b in range(2)]}
    for name, batches in scen.items():
        tfe, tf = RefAnalyzer(r, "tfe"), RefAnalyzer(r, "tf")
        for b, xb in enumerate(batches):
            out[f"cal/{name}/batch{b}"] = xb
            tfe.update(xb)
            tf.update(xb)
        xl, pdf = tfe.histogram()
        out[f"cal/{name}/x_left"] = xl
        out[f"cal/{name}/pdf"] = pdf
        for b, xb in enumerate(batches):
            if xl is not None:
                out[f"cal/{name}/hist{b}"] = r.batch_hist(xb, xl)
        for bw in (8, 4):
            for sym, strict, uns in ((0, 0, 0), (1, 0, 0), (1, 1, 0), (1, 0, 1)):
                out[f"cal/{name}/tfe_b{bw}_{sym}{strict}{uns}"] = tfe.compute(bw, sym, strict, uns)
                out[f"cal/{name}/tf_b{bw}_{sym}{strict}{uns}"] = tf.compute(bw, sym, strict, uns)
    np.savez_compressed(os.path.join(HERE, "libpymo.npz"), **out)


if __name__ == "__main__":
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("AIMET_REFERENCE_ROOT")
    if not ref:
        raise SystemExit("usage: gen_golden.py /path/to/aimet   (a checkout of the reference; or set AIMET_REFERENCE_ROOT)")
    only = sys.argv[2:]   # optionally: names of the generators to run
    gens = {"v2": lambda: gen_v2(ref), "quantizer": lambda: gen_quantizer(ref),
            "range_learning": lambda: gen_range_learning(ref), "reference_backend_tests": lambda: gen_reference_backend_tests(ref),
            "ste_v1": lambda: gen_ste_v1(ref), "wire_format": lambda: gen_wire_format(ref), "sqnr": lambda: gen_sqnr(ref), "histc_rule": gen_histc_rule, "libpymo": gen_libpymo}
    for name, fn in gens.items():
        if not only or name in only:
            fn()
    for f in ("v2_backend.npz", "v2_minmax.npz", "v2_quantizer.npz", "v1_range_learning.npz", "v1_ste.npz", "v2_sqnr.npz", "histc_rule.npz", "v2_backend_reference_tests.npz",
              "libpymo.npz", "v2_wire_format.json"):
        print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")
