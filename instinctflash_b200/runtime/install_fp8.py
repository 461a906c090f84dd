"""Install sites of the per-tensor FP8 projection (``SM100FP8Linear``) in loaded models.

Counterparts of the reference's explicit installers, which replace audited ``nn.Linear``
projections of a loaded model by ``ThorFP8Linear``:

* ``install_dreamzero_fp8``        instinctflash/runtime/dreamzero_fp8.py:14-70
* ``install_cosmos_fp8``           instinctflash/runtime/cosmos_fp8.py:18-57
* ``install_cosmos_dense_mlp_fp8`` instinctflash/runtime/cosmos_fp8.py:59-107
* ``install_groot_backbone_fp8``   instinctflash/runtime/groot_fp8.py:5-27 (the projection
  replacement; the CUDA-graph wrappers that file adds around the replaced modules belong to the
  reference's runtime, not to the FP8 linear path)

All four share one rule set, implemented once in :func:`install_projections`: only modules whose
class is EXACTLY an audited class are touched (subclasses, LoRA wrappers and look-alike names are
not), a projection with forward / backward hooks is refused, every replacement is packed before
the model is changed (a bad dtype, shape or an allocation failure leaves the model untouched), and
the caller gets a receipt listing what was replaced.  Same argument names, error conditions and
receipt keys as the reference's functions; call them after the last ``model.to()`` and before the
first prediction or graph capture.
"""
from __future__ import annotations

import importlib
import os
from typing import Callable, Iterable, Mapping, Sequence

from torch import nn

from .torch_fp8_linear import SM100FP8Linear


def _hooked(module: nn.Module) -> bool:
    return bool(module._forward_hooks or module._forward_pre_hooks or module._backward_hooks)


def _classes(module_name: str, *names: str):
    """The audited third-party classes; ImportError propagates (as in the reference, an installer
    is meaningless without the model code it audits)."""
    mod = importlib.import_module(module_name)
    return tuple(getattr(mod, n) for n in names)


def collect_projections(model: nn.Module, layouts: Mapping[type, Sequence[str]], *, family: str,
                        child: Callable[[nn.Module, str], tuple] | None = None) -> list:
    """[(path, parent, attribute, source)] for every named projection of every module whose class is
    exactly a key of ``layouts``.  ``child(module, name) -> (parent, attribute, source, path suffix)``
    resolves a name that is not a direct attribute (e.g. an index into a Sequential)."""
    found = []
    for path, module in model.named_modules():
        for name in layouts.get(type(module), ()):
            if child is not None:
                parent, attribute, source, suffix = child(module, name)
            else:
                parent, attribute, source, suffix = module, name, getattr(module, name), ""
            if _hooked(source):
                raise ValueError(f"Cannot replace hooked {family} projection {path}{suffix}.{attribute}")
            found.append((path + suffix, parent, attribute, source))
    return found


def install_projections(targets: Iterable[tuple], *, recipe: str, scope: str, linear_type=None, bias_in_receipt: bool = True,
                        extra: Mapping | None = None) -> dict:
    """Pack every target first, then swap them in; returns the receipt."""
    targets = list(targets)
    linear_type = linear_type or SM100FP8Linear
    packed = [linear_type(source) for _, _, _, source in targets]   # nothing is changed if any of these raises
    projections = []
    for path, _, name, source in targets:
        entry = {"path": f"{path}.{name}".lstrip("."), "in_features": source.in_features, "out_features": source.out_features}
        if bias_in_receipt:
            entry["bias"] = source.bias is not None
        projections.append(entry)
    receipt = {"recipe": recipe + linear_type.recipe, "projections": projections, "scope": scope}
    receipt.update(extra or {})
    for (_, parent, name, _), replacement in zip(targets, packed):
        setattr(parent, name, replacement)
    return receipt


# ------------------------------------------------------------------------------------------------
def install_dreamzero_fp8(action_head, *, include_ffn=False, linear_type=None):
    """DreamZero causal self-attention Q/K/V (and, on request, the block FFN's two Linears)."""
    if getattr(action_head, "cpu_offload", False):
        raise ValueError("Pack DreamZero FP8 only after selecting GPU-resident native components")
    if getattr(action_head, "trt_engine", None) is not None:
        raise ValueError("Native PyTorch FP8 projections cannot be installed behind a loaded TensorRT engine")
    if os.environ.get("ENABLE_TENSORRT", "false").lower() == "true":
        raise ValueError("Native PyTorch FP8 projections cannot be installed behind a TensorRT execution path")
    source_module = "groot.vla.model.dreamzero.modules.wan_video_dit_action_casual_chunk"
    (attention_cls,) = _classes(source_module, "CausalWanSelfAttention")
    model = action_head.model
    targets = collect_projections(model, {attention_cls: ("q", "k", "v")}, family="DreamZero")
    if not targets:
        raise ValueError("No audited DreamZero causal Q/K/V projections found")
    attention_layers = len(targets) // 3
    if include_ffn:
        (block_cls,) = _classes(source_module, "CausalWanAttentionBlock")

        def ffn_child(block, index):
            return block.ffn, index, block.ffn[int(index)], ".ffn"

        ffn = collect_projections(model, {block_cls: ("0", "2")}, family="DreamZero FFN", child=ffn_child)
        if len(ffn) != attention_layers * 2:
            raise ValueError("DreamZero FFN layout does not match causal attention blocks")
        targets += ffn
    extra = {
        "attention_layers": attention_layers,
        "scheduler_steps": int(action_head.num_inference_steps),
        "dit_step_mask": list(action_head.dit_step_mask),
        "dynamic_cache_schedule": bool(getattr(action_head, "dynamic_cache_schedule", False)),
        "quality_certificate": None if include_ffn else "checkpoint-specific; see evaluation receipts",
    }
    return install_projections(
        targets, recipe="dreamzero_causal_qkv_ffn_" if include_ffn else "dreamzero_causal_qkv_", linear_type=linear_type,
        scope="Causal self-attention Q/K/V" + (" and block FFN" if include_ffn else " only") +
              "; other computation and history remain native", extra=extra)


COSMOS_PROJECTIONS = ("q_proj", "k_proj", "v_proj", "q_proj_moe_gen", "k_proj_moe_gen", "v_proj_moe_gen")


def install_cosmos_fp8(model, *, linear_type=None):
    """Cosmos MoT attention Q/K/V of both towers."""
    (attention_cls,) = _classes("cosmos_framework.model.generator.mot.unified_mot", "PackedAttentionMoT")
    targets = collect_projections(model, {attention_cls: COSMOS_PROJECTIONS}, family="Cosmos")
    if not targets:
        raise ValueError("No audited PackedAttentionMoT projections found; FP8 was not installed")
    return install_projections(targets, recipe="cosmos_mot_qkv_", linear_type=linear_type,
                               scope="Q/K/V in both MoT towers only; native attention, output projections and MLP",
                               extra={"attention_layers": len(targets) // len(COSMOS_PROJECTIONS)})


def install_cosmos_dense_mlp_fp8(model, *, linear_type=None):
    """Experimental: the dense MoT MLPs of both towers (sparse experts, routers and the visual
    encoder are not converted)."""
    layer_cls, qwen_mlp, nemotron_mlp = _classes("cosmos_framework.model.generator.mot.unified_mot", "MoTDecoderLayer",
                                                 "Qwen3VLTextMLP", "Nemotron3DenseVLMLP")
    layouts = {qwen_mlp: ("gate_proj", "up_proj", "down_proj"), nemotron_mlp: ("up_proj", "down_proj")}
    targets, mlp_count = [], 0
    for path, layer in model.named_modules():
        if type(layer) is not layer_cls:
            continue
        for tower in ("mlp", "mlp_moe_gen"):
            module = getattr(layer, tower)
            names = layouts.get(type(module))
            where = f"{path}.{tower}"
            if names is None:
                raise ValueError(f"Unsupported Cosmos dense MLP type at {where}")
            if _hooked(module):
                raise ValueError(f"Cannot convert hooked Cosmos MLP {where}")
            mlp_count += 1
            for name in names:
                source = getattr(module, name)
                if _hooked(source):
                    raise ValueError(f"Cannot replace hooked Cosmos MLP projection {where}.{name}")
                targets.append((where.lstrip("."), module, name, source))
    if not targets:
        raise ValueError("No audited dense MoT MLPs found; FP8 MLP was not installed")
    return install_projections(targets, recipe="cosmos_mot_dense_mlp_", linear_type=linear_type,
                               scope="Experimental dense MoT MLP extension; native activation and routing preserved",
                               extra={"mlp_modules": mlp_count})


def install_groot_backbone_fp8(backbone, *, linear_type=None):
    """GR00T Qwen3 text attention and MLP projections (vision and processors stay native)."""
    attention_cls, mlp_cls = _classes("transformers.models.qwen3_vl.modeling_qwen3_vl", "Qwen3VLTextAttention",
                                      "Qwen3VLTextMLP")
    layouts = {attention_cls: ("q_proj", "k_proj", "v_proj", "o_proj"), mlp_cls: ("gate_proj", "up_proj", "down_proj")}
    targets = collect_projections(backbone, layouts, family="GR00T")
    if not targets:
        raise ValueError("No audited Qwen3 text projections found in GR00T backbone")
    return install_projections(targets, recipe="groot_qwen3_text_", linear_type=linear_type, bias_in_receipt=False,
                               scope="Qwen3 text attention and MLP; native vision",
                               extra={"quality_certificate": None, "graph_boundaries": 0})
