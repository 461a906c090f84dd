"""Rebind the reference's engine modules to the sm_100a operators.

The reference's engines call module-level names imported into each engine module
(``from ..kernels.fp8 import gemm`` ... at instinctflash/engines/pi05/engine.py:20-24 and the
same lines of the vla4, vla2, groot_n17 and wan_va engines), resolved from module globals at call
time.  ``install()`` replaces those names, in the kernel modules and in every engine module
already imported, with the operators of this package.  It must run before an engine captures
its CUDA graph (first ``infer``): a captured graph keeps the kernels it was captured with.
"""
from __future__ import annotations

import importlib
import sys

import functools

from .kernels import activation, fp8, norm, rope, wan

REPLACEMENTS = {
    "gemm": fp8.gemm,
    "quantize_weight": fp8.quantize_weight,
    "Fp8Weight": fp8.Fp8Weight,
    "row_quant": norm.row_quant,
    "dequant_rows": norm.dequant_rows,
    "residual_norm_quant": norm.residual_norm_quant,
    "gated_act_quant": activation.gated_act_quant,
    "qkv_split": rope.qkv_split,
    "rope_inv_freq": rope.rope_inv_freq,
    "wan_qkv": wan.wan_qkv,
}
KERNEL_MODULES = {"instinctflash.kernels.fp8": ("gemm", "quantize_weight", "Fp8Weight"),
                  "instinctflash.kernels.norm": ("row_quant", "dequant_rows", "residual_norm_quant"),
                  "instinctflash.kernels.activation": ("gated_act_quant",),
                  "instinctflash.kernels.rope": ("qkv_split", "rope_inv_freq"),
                  "instinctflash.kernels.wan": ("wan_qkv",)}
ENGINE_MODULES = tuple(f"instinctflash.engines.{fam}.engine" for fam in ("pi05", "vla4", "vla2", "groot_n17", "wan_va"))


def _keep_router_tail(original):
    """``residual_norm_quant`` for a module whose own version is ``original``.

    The reference's kernel also carries the mixture-of-experts router tail
    (instinctflash/kernels/norm.py:81-94), which the LingBot-VLA-V2 expert layers use
    (instinctflash/engines/vla2/engine.py:208).  That tail is outside the FP8 linear path, so a
    call that passes ``router=`` goes to the function the module had before the rebinding; every
    other call goes to this package's kernel."""
    if getattr(original, "_iflb200_router_tail", False):
        return original   # installed before
    if original is norm.residual_norm_quant or not callable(original):
        return norm.residual_norm_quant

    @functools.wraps(norm.residual_norm_quant)
    def residual_norm_quant(res, *args, router=None, **kwargs):
        if router is not None:
            return original(res, *args, router=router, **kwargs)
        return norm.residual_norm_quant(res, *args, **kwargs)

    residual_norm_quant._iflb200_router_tail = True
    residual_norm_quant._iflb200_original = original
    return residual_norm_quant


def install(modules=None, *, import_missing: bool = False) -> dict:
    """Rebind and return ``{module name: [names rebound]}``.

    ``modules`` may be an iterable of module objects (tests pass fakes); by default the
    reference's kernel and engine modules that are already imported (or all of them with
    ``import_missing``) are patched.  ``Fp8Weight`` is only rebound in kernel modules: engine
    weights built with the reference's dataclass have the same fields and are accepted as is.
    ``residual_norm_quant`` keeps the module's previous function for calls with ``router=``
    (the mixture-of-experts tail, not part of this path); installing twice is harmless.
    """
    report = {}
    if modules is None:
        modules = []
        for name in (*KERNEL_MODULES, *ENGINE_MODULES):
            mod = sys.modules.get(name)
            if mod is None and import_missing:
                try:
                    mod = importlib.import_module(name)
                except ImportError:
                    mod = None
            if mod is not None:
                modules.append(mod)
    for mod in modules:
        done = []
        for name, fn in REPLACEMENTS.items():
            if name == "Fp8Weight" and getattr(mod, "__name__", "") not in KERNEL_MODULES:
                continue
            if hasattr(mod, name):
                if name == "residual_norm_quant":
                    fn = _keep_router_tail(getattr(mod, name))
                setattr(mod, name, fn)
                done.append(name)
        report[getattr(mod, "__name__", repr(mod))] = done
    return report
