"""Host-side behaviour of the operator wrappers: the reference's signatures, its error
behaviour (ValueError / RuntimeError before launch) and the install seam.  No GPU."""
import inspect
import types

import pytest
import torch

from instinctflash_b200 import install as inst
from instinctflash_b200.kernels import activation, fp8, norm
from instinctflash_b200.runtime import fp8_pack, torch_fp8_linear

E4M3 = torch.float8_e4m3fn


def params(fn):
    return list(inspect.signature(fn).parameters)


def test_signatures_match_the_reference_operators():
    # instinctflash/kernels/fp8.py:30,50; norm.py:97-99,150,178; activation.py:46
    assert params(fp8.gemm) == ["a", "w", "out"]
    assert params(fp8.quantize_weight) == ["w", "bias", "device"]
    assert params(norm.row_quant) == ["x", "q", "q_scale", "row", "col", "bias", "gelu", "num_warps"]
    assert params(norm.dequant_rows) == ["x", "y", "row", "col", "bias", "block", "num_warps"]
    assert params(activation.gated_act_quant) == ["gu", "q", "q_scale", "row", "col", "act", "num_warps"]
    assert params(norm.residual_norm_quant) == [
        "res", "delta", "delta_row", "delta_col", "bias", "gate", "write_res", "layernorm", "weight", "beta",
        "mod_scale", "mod_shift", "q", "q_scale", "y", "eps", "num_warps", "router", "mod_index"]
    assert (activation.GELU_TANH, activation.SILU) == (0, 1)
    assert [f for f in fp8.Fp8Weight.__dataclass_fields__] == ["w", "scale", "bias"]
    assert params(fp8_pack.dynamic_pack_bf16_e4m3) == ["x"]
    assert params(fp8_pack.pack_bf16_e4m3) == ["x", "scale"]


def test_quantize_weight_layout_and_values_on_cpu():
    w = torch.randn(48, 32) * 0.02
    fw = fp8.quantize_weight(w, torch.randn(48).to(torch.bfloat16))
    assert fw.w.dtype == E4M3 and fw.w.shape == (48, 32) and fw.w.is_contiguous()
    assert fw.scale.dtype == torch.float32 and fw.scale.shape == (48,)
    assert fw.bias.dtype == torch.float32 and fw.shape == (48, 32)
    deq = fw.w.float() * fw.scale[:, None]
    assert (deq - w).abs().max() <= w.abs().amax() * 2 ** -4
    assert torch.equal(fw.w.float().abs().amax(1), torch.full((48,), 448.0))


def test_operators_refuse_cpu_tensors_instead_of_falling_back():
    x = torch.randn(4, 32).to(torch.bfloat16)
    q = torch.empty(4, 32, dtype=E4M3)
    s = torch.empty(4)
    with pytest.raises(ValueError, match="no CPU implementation"):
        norm.row_quant(x, q, s)
    with pytest.raises(ValueError, match="CUDA"):
        fp8_pack.dynamic_pack_bf16_e4m3(x)
    w = fp8.quantize_weight(torch.randn(16, 32))
    with pytest.raises(ValueError):
        fp8.gemm(q, w, torch.empty(4, 16, dtype=torch.bfloat16))


def test_gated_act_quant_width_limit_message_matches_reference():
    class Fake:
        pass
    gu = torch.empty(2, 2 * 32768, dtype=torch.bfloat16, device="meta")
    q = torch.empty(2, 32768, dtype=E4M3, device="meta")
    with pytest.raises(ValueError):
        activation.gated_act_quant(gu, q, torch.empty(2, device="meta"))


def test_residual_norm_quant_rejects_the_router_tail():
    res = torch.empty(2, 16, device="meta")
    with pytest.raises(NotImplementedError):
        norm.residual_norm_quant(res, router=(None, None, None, 2, 1.0))


def test_sm100_linear_constructor_checks_follow_the_reference():
    lin = torch.nn.Linear(32, 16, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="capability"):
        torch_fp8_linear.SM100FP8Linear(lin)               # CPU weights, no CUDA target
    class Sub(torch.nn.Linear):
        pass
    with pytest.raises(TypeError):
        torch_fp8_linear.SM100FP8Linear(Sub(32, 16))


def test_install_rebinds_engine_and_kernel_modules():
    engine = types.ModuleType("instinctflash.engines.pi05.engine")
    sentinel = object()
    for name in ("gemm", "row_quant", "gated_act_quant", "residual_norm_quant", "attention", "Fp8Weight"):
        setattr(engine, name, sentinel)
    kernels_fp8 = types.ModuleType("instinctflash.kernels.fp8")
    kernels_fp8.gemm = kernels_fp8.quantize_weight = kernels_fp8.Fp8Weight = sentinel
    report = inst.install([engine, kernels_fp8])
    assert engine.gemm is fp8.gemm and engine.row_quant is norm.row_quant
    assert engine.gated_act_quant is activation.gated_act_quant
    assert engine.residual_norm_quant is norm.residual_norm_quant
    assert engine.attention is sentinel            # not part of this path: untouched
    assert engine.Fp8Weight is sentinel            # engines keep their weight class
    assert kernels_fp8.Fp8Weight is fp8.Fp8Weight and kernels_fp8.gemm is fp8.gemm
    assert sorted(report["instinctflash.engines.pi05.engine"]) == ["gated_act_quant", "gemm", "residual_norm_quant", "row_quant"]


def test_calls_run_with_the_tensor_device_current(monkeypatch):
    """The library keys its per-device state and the launch itself on the current device, so every
    call must be made with the operand's device current (and the previous one restored).  Checked on
    the host with a stand-in library that records the device at call time: nothing is launched."""
    from instinctflash_b200 import _lib
    from instinctflash_b200.kernels import _common

    state = {"current": 0, "seen": [], "sets": []}

    class FakeLib:
        def iflb200_probe(self, *args):
            state["seen"].append((state["current"], args))
            return 0

        def iflb200_status_string(self, status):
            return b"bad"

    def set_device(i):
        state["sets"].append(i)
        state["current"] = i

    monkeypatch.setattr(torch.cuda, "current_device", lambda: state["current"])
    monkeypatch.setattr(torch.cuda, "set_device", set_device)
    monkeypatch.setattr(_lib, "lib", lambda: FakeLib())
    monkeypatch.setattr(_lib, "stream_handle", lambda device=None: 1000 + device.index)
    on_gpu1 = types.SimpleNamespace(device=torch.device("cuda", 1))   # only .device is looked at
    _common.launch("iflb200_probe", on_gpu1, 7, 8)
    assert state["seen"] == [(1, (7, 8, 1001))]            # called with cuda:1 current, on cuda:1's stream
    assert state["sets"] == [1, 0] and state["current"] == 0  # and cuda:0 current again afterwards
    state["current"], state["sets"] = 1, []
    _common.launch("iflb200_probe", on_gpu1, 9)
    assert state["sets"] == []                              # already current: no switch
    other = types.SimpleNamespace(device=torch.device("cuda", 0))
    with pytest.raises(ValueError, match="expected"):
        _common.same_device(on_gpu1, q=other)                # operands on different devices are refused


def test_install_default_patches_only_imported_modules():
    assert isinstance(inst.install(), dict)


def test_qkv_consumers_reject_bad_arguments_before_launch():
    from instinctflash_b200.kernels import rope, wan
    x = torch.zeros(4, 3 * 64, dtype=torch.bfloat16)
    q = torch.zeros(4, 1, 64, dtype=torch.float16)
    kv = torch.zeros(8, 1, 64, dtype=torch.float16)
    with pytest.raises(ValueError, match="CUDA"):          # no CPU implementation
        rope.qkv_split(x, q, kv, kv.clone(), heads_q=1, heads_kv=1, head_dim=64)
    with pytest.raises(ValueError, match="share a dtype"):
        rope.qkv_split(x, q, kv, kv.float(), heads_q=1, heads_kv=1, head_dim=64)
    with pytest.raises(ValueError, match="position table"):
        rope.qkv_split(x, q, kv, kv.clone(), heads_q=1, heads_kv=1, head_dim=64, inv_freq=torch.ones(32))
    with pytest.raises(ValueError, match="CUDA"):
        wan.wan_qkv(x, torch.zeros(4, 64, dtype=torch.float16), heads=1, head_dim=64, tokens=4)
    assert rope.rope_inv_freq(8, 10000.0, "cpu").tolist() == pytest.approx([1.0, 0.1, 0.01, 0.001])
