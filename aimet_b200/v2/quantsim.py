"""Quantization simulation of a whole model: which tensors get a quantizer, and the calibration driver.

Orchestration only, no arithmetic: every quantizer is a :class:`aimet_b200.v2.quantizer.QuantizeDequantize`.
Mirrors the user-facing surface of ``QuantizationSimModel`` (aimet_torch/v2/quantsim/quantsim.py:71-224: constructor
arguments ``model, dummy_input, quant_scheme, default_output_bw, default_param_bw``; ``sim.model``;
``sim.compute_encodings(forward_pass_callback, forward_pass_callback_args)``) and of the quantized layers
(aimet_torch/v2/nn/base.py:90-196: ``param_quantizers``, ``_compute_param_encodings``).

The reference decides quantizer placement from a JSON configuration and a connected graph of the model; here the
model is traced with ``torch.fx`` and the placement follows the reference's default configuration in its common
form: parameters of convolution / linear layers per output channel, symmetric; the model input, and the output of
every convolution, linear layer, element-wise addition, ReLU and pooling call, asymmetric, per tensor -- except that
a layer or addition whose only consumer is a ReLU is quantized after the ReLU (the "supergroup" rule).  Batch norms
directly after a convolution are folded into it first.
"""
from __future__ import annotations

import contextlib
import copy
import operator
from typing import Callable, Dict, List, Optional

import torch
import torch.nn.functional as F
from torch import fx, nn

from .encoding_analyzer import MinMaxEncodingAnalyzer, SqnrEncodingAnalyzer, TfEnhancedEncodingAnalyzer
from .quantizer import QuantizeDequantize

__all__ = ["QuantizationSimModel", "QuantizedLayer", "fold_batch_norms"]

_LAYERS = (nn.Conv1d, nn.Conv2d, nn.Conv3d, nn.Linear)
_RELUS = (nn.ReLU, nn.ReLU6)
_POOLS = (nn.MaxPool2d, nn.AvgPool2d, nn.AdaptiveAvgPool2d)
_ADDS = (operator.add, operator.iadd, torch.add)
_RELU_FUNCS = (F.relu, torch.relu, F.relu6)


class QuantizedLayer(nn.Module):
    """A convolution / linear layer whose weight passes through a quantizer on every call
    (the fake-quantized layers of aimet_torch/v2/nn/fake_quant.py; parameter handling of v2/nn/base.py:117-196)."""

    def __init__(self, layer: nn.Module, weight_quantizer: Optional[QuantizeDequantize]):
        super().__init__()
        self.layer = layer
        self.param_quantizers = nn.ModuleDict({"weight": weight_quantizer})

    def forward(self, x):
        wq = self.param_quantizers["weight"]
        if wq is None:
            return self.layer(x)
        return torch.func.functional_call(self.layer, {"weight": wq(self.layer.weight)}, (x,))

    @torch.no_grad()
    def compute_param_encodings(self):
        """Weights are calibrated from the weights themselves, once (base.py:128-150)."""
        wq = self.param_quantizers["weight"]
        if wq is not None:
            with wq.compute_encodings():
                wq(self.layer.weight)


@torch.no_grad()
def fold_batch_norms(gm: fx.GraphModule) -> int:
    """Folds every BatchNorm that directly follows a convolution (its only consumer) into that convolution:
    W' = W * g / sqrt(var + eps), b' = beta + (b - mean) * g / sqrt(var + eps).  Returns the number folded."""
    mods = dict(gm.named_modules())
    folded = 0
    for node in list(gm.graph.nodes):
        if node.op != "call_module" or not isinstance(mods.get(node.target), (nn.BatchNorm1d, nn.BatchNorm2d)):
            continue
        src = node.args[0]
        if not (isinstance(src, fx.Node) and src.op == "call_module" and isinstance(mods.get(src.target), _LAYERS[:3])
                and len(src.users) == 1):
            continue
        conv, bn = mods[src.target], mods[node.target]
        if bn.training or bn.running_var is None:
            continue
        inv = (bn.weight if bn.weight is not None else torch.ones_like(bn.running_var)) / torch.sqrt(bn.running_var + bn.eps)
        conv.weight.mul_(inv.reshape([-1] + [1] * (conv.weight.dim() - 1)))
        bias = conv.bias if conv.bias is not None else torch.zeros_like(bn.running_mean)
        new_bias = (bias - bn.running_mean) * inv + (bn.bias if bn.bias is not None else 0)
        conv.bias = nn.Parameter(new_bias)
        node.replace_all_uses_with(src)
        gm.graph.erase_node(node)
        folded += 1
    gm.graph.lint()
    gm.recompile()
    gm.delete_all_unused_submodules()
    return folded


def _is_relu(node: fx.Node, mods: Dict[str, nn.Module]) -> bool:
    if node.op == "call_module":
        return isinstance(mods.get(node.target), _RELUS)
    if node.op == "call_function":
        return node.target in _RELU_FUNCS
    return node.op == "call_method" and node.target in ("relu", "relu_")


class QuantizationSimModel:
    """``sim = QuantizationSimModel(model, dummy_input); sim.compute_encodings(callback, args); sim.model(x)``.

    quant_scheme, mapped to analyzers as the reference does (aimet_torch/quantsim_config/builder.py:294-309):

    * ``"post_training_tf"``: min/max for parameters and activations;
    * ``"post_training_tf_enhanced"``: the v2 ``SqnrEncodingAnalyzer`` (histogram + SQNR search) for parameters (one
      histogram per output channel) and activations;
    * ``"post_training_tf_enhanced_libpymo"``: not a reference scheme name -- activations get the v1 / libpymo
      TF-Enhanced analyzer (512-bucket PDF frozen by the first batch) behind the v2 interface, parameters min/max.
    """

    def __init__(self, model: nn.Module, dummy_input=None, quant_scheme: str = "post_training_tf_enhanced",
                 default_output_bw: int = 8, default_param_bw: int = 8, per_channel_quantization: bool = True,
                 fold_bn: bool = True):
        if quant_scheme not in ("post_training_tf_enhanced", "post_training_tf", "post_training_tf_enhanced_libpymo"):
            raise ValueError(f"unsupported quant_scheme {quant_scheme!r}")
        self._scheme = quant_scheme
        self._act_bw, self._param_bw = int(default_output_bw), int(default_param_bw)
        gm = fx.symbolic_trace(copy.deepcopy(model))
        if fold_bn:
            fold_batch_norms(gm)
        mods = dict(gm.named_modules())
        self.layers: Dict[str, QuantizedLayer] = {}
        self.activation_quantizers: Dict[str, QuantizeDequantize] = {}
        self._activation_keys: Dict[str, tuple] = {}
        # ---- parameters ----
        for node in gm.graph.nodes:
            if node.op == "call_module" and isinstance(mods.get(node.target), _LAYERS):
                layer = mods[node.target]
                shape = (layer.weight.shape[0],) + (1,) * (layer.weight.dim() - 1) if per_channel_quantization else ()
                wq = QuantizeDequantize(shape, self._param_bw, True, self._new_analyzer(shape, for_param=True))
                wq.plain_outputs = True
                wrapped = QuantizedLayer(layer, wq)
                self._set_submodule(gm, node.target, wrapped)
                self.layers[node.target] = wrapped
        mods = dict(gm.named_modules())
        # ---- activations ----
        for node in list(gm.graph.nodes):
            if not self._wants_output_quantizer(node, mods):
                continue
            name = "act_q_" + node.name
            q = QuantizeDequantize((), self._act_bw, False, self._new_analyzer(()))
            q.plain_outputs = True
            # where the exported files list this quantizer: a layer's output, or the model input
            self._activation_keys[name] = ((node.name, "input") if node.op == "placeholder" else
                                           (node.target if node.op == "call_module" else node.name, "output"))
            gm.add_submodule(name, q)
            with gm.graph.inserting_after(node):
                new = gm.graph.call_module(name, (node,))
            node.replace_all_uses_with(new)
            new.args = (node,)
            self.activation_quantizers[name] = q
        gm.graph.lint()
        gm.recompile()
        self.model = gm
        if dummy_input is not None:
            ref = dummy_input[0] if isinstance(dummy_input, (tuple, list)) else dummy_input
            self.model.to(ref.device)

    # ---- construction helpers ----------------------------------------------------------------------------------
    def _new_analyzer(self, shape, for_param: bool = False):
        if self._scheme == "post_training_tf_enhanced":
            return SqnrEncodingAnalyzer(shape)
        if self._scheme == "post_training_tf_enhanced_libpymo" and not for_param:
            return TfEnhancedEncodingAnalyzer(shape)
        return MinMaxEncodingAnalyzer(shape)

    @staticmethod
    def _set_submodule(root: nn.Module, target: str, new: nn.Module):
        parent_name, _, leaf = target.rpartition(".")
        parent = root.get_submodule(parent_name) if parent_name else root
        setattr(parent, leaf, new)

    @staticmethod
    def _wants_output_quantizer(node: fx.Node, mods: Dict[str, nn.Module]) -> bool:
        if node.op == "placeholder":
            return True
        only_user_is_relu = len(node.users) == 1 and _is_relu(next(iter(node.users)), mods)
        if node.op == "call_module":
            m = mods.get(node.target)
            if isinstance(m, QuantizedLayer):
                return not only_user_is_relu
            return isinstance(m, _RELUS + _POOLS)
        if node.op == "call_function":
            if node.target in _ADDS:
                return not only_user_is_relu
            return node.target in _RELU_FUNCS
        return _is_relu(node, mods)

    # ---- calibration -------------------------------------------------------------------------------------------
    def quantizers(self) -> List[QuantizeDequantize]:
        return [l.param_quantizers["weight"] for l in self.layers.values()] + list(self.activation_quantizers.values())

    def compute_encodings(self, forward_pass_callback: Callable, forward_pass_callback_args=None):
        """Calibrates every quantizer: weights from the weights, activations from what flows through the model while
        ``forward_pass_callback(sim.model, forward_pass_callback_args)`` runs (quantsim.py:205-224)."""
        for layer in self.layers.values():
            layer.compute_param_encodings()
        with contextlib.ExitStack() as stack:
            for q in self.activation_quantizers.values():
                stack.enter_context(q.compute_encodings())
            with torch.no_grad():
                forward_pass_callback(self.model, forward_pass_callback_args)

    # ---- encodings on disk -------------------------------------------------------------------------------------
    def get_encodings_dict(self) -> dict:
        """The calibrated encodings in the layout of the reference's ``<prefix>_torch.encodings`` file
        (aimet_torch/v1/quantsim.py:884-938, 1028-1040): ``param_encodings`` maps ``<layer>.weight`` to one dict per
        output channel, ``activation_encodings`` maps a layer name to ``{"input" | "output": {"0": dict}}``; every
        dict is what ``get_legacy_encodings`` returns.  Quantizers that were never calibrated are left out."""
        params, acts = {}, {}
        for name, layer in self.layers.items():
            wq = layer.param_quantizers["weight"]
            enc = wq.get_legacy_encodings() if wq is not None else None
            if enc is not None:
                params[name + ".weight"] = enc
        for name, q in self.activation_quantizers.items():
            enc = q.get_legacy_encodings()
            if enc is not None:
                key, kind = self._activation_keys[name]
                acts.setdefault(key, {}).setdefault(kind, {})["0"] = enc[0]
        return {"version": "0.6.1", "activation_encodings": acts, "param_encodings": params, "excluded_layers": []}

    def export_encodings(self, path: str, filename_prefix: str) -> str:
        """Writes ``<path>/<filename_prefix>_torch.encodings`` (JSON) and returns its name."""
        import json
        import os
        os.makedirs(path, exist_ok=True)
        target = os.path.join(path, filename_prefix + "_torch.encodings")
        with open(target, "w") as f:
            json.dump(self.get_encodings_dict(), f, sort_keys=True, indent=4)
        return target

    def load_encodings(self, encodings, strict: bool = True, partial: bool = True,
                       requires_grad: Optional[bool] = None, allow_overwrite: bool = True):
        """Sets quantizers from an encodings dictionary or file (aimet_torch/v1/quantsim.py:1695-1756 with the
        per-layer rules of aimet_torch/v2/nn/base.py:282-420).  ``strict``: unknown names raise; ``partial`` = False:
        quantizers the dictionary does not mention are removed; ``requires_grad``: trainability of the loaded
        ranges (None = unchanged); ``allow_overwrite`` = False freezes them against later calibration.  Quantizers
        that were frozen by an earlier load are skipped."""
        import json
        import os
        if isinstance(encodings, (str, os.PathLike)):
            with open(encodings) as f:
                encodings = json.load(f)
        if "param_encodings" not in encodings:
            params, acts = encodings, {}
        else:
            params, acts = encodings.get("param_encodings", {}), encodings.get("activation_encodings", {})
        if not params and not acts:
            raise RuntimeError("the encodings dictionary is empty")
        by_key = {self._activation_keys[name]: name for name in self.activation_quantizers}
        if strict:
            known = {n + ".weight" for n in self.layers} | {key for key, _ in by_key}
            missing = sorted((set(params) | set(acts)) - known)
            if missing:
                raise RuntimeError("Encoding dictionary contains modules/parameters that doesn't exist in the model: "
                                   + ", ".join(missing))

        def apply(q, enc):
            q.set_legacy_encodings([enc] if isinstance(enc, dict) else list(enc))
            if requires_grad is not None:
                q.requires_grad_(requires_grad)
            q.allow_overwrite(allow_overwrite)

        for name, layer in self.layers.items():
            wq = layer.param_quantizers["weight"]
            if wq is not None and not wq._allow_overwrite:   # pylint: disable=protected-access
                continue
            enc = params.get(name + ".weight")
            if not enc:
                if not partial:
                    layer.param_quantizers["weight"] = None
                continue
            if wq is None:
                if strict:
                    raise RuntimeError(f"Failed to import encoding of {name}.weight: no quantizer present.")
                continue
            apply(wq, enc)
        for (key, kind), name in by_key.items():
            q = self.activation_quantizers[name]
            if not q._allow_overwrite:   # pylint: disable=protected-access
                continue
            enc = acts.get(key, {}).get(kind, {})
            enc = enc.get("0", enc.get(0)) if isinstance(enc, dict) else None
            if not enc:
                if not partial:
                    self._remove_activation_quantizer(name)
                continue
            apply(q, enc)

    def _remove_activation_quantizer(self, name: str):
        """Takes a quantizer out of the traced graph: its consumers read the tensor it used to wrap."""
        for node in list(self.model.graph.nodes):
            if node.op == "call_module" and node.target == name:
                node.replace_all_uses_with(node.args[0])
                self.model.graph.erase_node(node)
        self.model.graph.lint()
        self.model.recompile()
        self.model.delete_submodule(name)
        del self.activation_quantizers[name]
        del self._activation_keys[name]

