"""The drop-in seam against the reference's own modules (no GPU).

The unmodified reference, pip-installed into the git-ignored ``baseline/_ref`` by the build step,
is imported here; every test is skipped when that install is absent.  Checked: the operators of
this package have exactly the signatures of the functions they replace
(instinctflash/kernels/{fp8,norm,activation,rope,wan}.py), ``install()`` rebinds the names the
engine modules resolve at call time (instinctflash/engines/*/engine.py import blocks) and can be
undone, and a ``router=`` call still reaches the reference's own kernel.
"""
import importlib
import inspect
import sys
from pathlib import Path

import pytest
import torch

from instinctflash_b200 import install as inst

REF = Path(__file__).resolve().parents[1] / "baseline" / "_ref"


@pytest.fixture(scope="module")
def reference():
    if not (REF / "instinctflash").is_dir():
        pytest.skip("the reference is not installed under baseline/_ref")
    sys.path.insert(0, str(REF))
    try:
        mods = {name: importlib.import_module(name) for name in inst.KERNEL_MODULES}
    except Exception as exc:  # triton or another dependency of the reference missing
        sys.path.remove(str(REF))
        pytest.skip(f"the reference's kernel modules do not import here: {exc}")
    yield mods
    sys.path.remove(str(REF))


def test_every_replacement_has_the_reference_signature(reference):
    for module_name, names in inst.KERNEL_MODULES.items():
        for name in names:
            theirs = getattr(reference[module_name], name)
            ours = inst.REPLACEMENTS[name]
            if inspect.isclass(theirs):
                assert [f for f in theirs.__dataclass_fields__] == [f for f in ours.__dataclass_fields__], name
                continue
            a, b = inspect.signature(theirs), inspect.signature(ours)
            assert list(a.parameters) == list(b.parameters), f"{name}: {a} != {b}"
            for p in a.parameters.values():
                q = b.parameters[p.name]
                assert p.kind == q.kind, f"{name}.{p.name}: {p.kind} != {q.kind}"
                assert p.default == q.default, f"{name}.{p.name}: default {p.default!r} != {q.default!r}"


def test_activation_codes_match(reference):
    theirs = reference["instinctflash.kernels.activation"]
    from instinctflash_b200.kernels import activation
    assert (theirs.GELU_TANH, theirs.SILU) == (activation.GELU_TANH, activation.SILU)
    assert reference["instinctflash.kernels.fp8"].FP8_MAX == 448.0


def test_install_rebinds_the_real_engine_modules_and_can_be_undone(reference):
    """Every engine family's module is imported from the reference, patched, checked and restored."""
    saved = {}
    engines = []
    for name in inst.ENGINE_MODULES:
        try:
            engines.append(importlib.import_module(name))
        except Exception:
            continue                       # an engine whose own dependencies are absent here
    assert engines, "no reference engine module could be imported"
    targets = list(reference.values()) + engines
    for mod in targets:
        saved[mod.__name__] = {n: getattr(mod, n) for n in inst.REPLACEMENTS if hasattr(mod, n)}
    try:
        report = inst.install(targets)
        for mod in engines:
            expected = [n for n in saved[mod.__name__] if n != "Fp8Weight"]
            assert sorted(report[mod.__name__]) == sorted(expected)
            assert {"gemm", "residual_norm_quant"} <= set(expected), mod.__name__
            for n in expected:
                bound = getattr(mod, n)
                if n == "residual_norm_quant":
                    assert bound is not saved[mod.__name__][n]
                    assert inspect.signature(bound) == inspect.signature(inst.REPLACEMENTS[n])
                else:
                    assert bound is inst.REPLACEMENTS[n], f"{mod.__name__}.{n}"
            # what the engine's _forward will call is resolved from these globals at call time
            fwd = [v for k, v in vars(mod).items() if inspect.isclass(v) and hasattr(v, "_forward")]
            for cls in fwd:
                assert cls._forward.__globals__["gemm"] is inst.REPLACEMENTS["gemm"]
        again = inst.install(targets)      # idempotent
        assert again.keys() == report.keys()
    finally:
        for mod in targets:
            for n, fn in saved[mod.__name__].items():
                setattr(mod, n, fn)
    for mod in targets:
        for n, fn in saved[mod.__name__].items():
            assert getattr(mod, n) is fn


def test_router_calls_keep_the_reference_kernel():
    """The LingBot-VLA-V2 expert layers pass ``router=`` (instinctflash/engines/vla2/engine.py:208);
    after install() such a call must reach the function the module had before."""
    import types
    calls = []

    def original(res, *, router=None, **kw):
        calls.append(router)
        return "reference"

    engine = types.ModuleType("instinctflash.engines.vla2.engine")
    engine.residual_norm_quant = original
    inst.install([engine])
    res = torch.empty(2, 16, device="meta")
    assert engine.residual_norm_quant(res, router=(None, None, None, 2, 1.0)) == "reference"
    assert calls == [(None, None, None, 2, 1.0)]
    with pytest.raises(ValueError, match="CUDA"):          # no router: this package's kernel (which refuses meta/CPU tensors)
        engine.residual_norm_quant(res)
    first = engine.residual_norm_quant
    inst.install([engine])
    assert engine.residual_norm_quant is first             # installing twice does not stack wrappers
