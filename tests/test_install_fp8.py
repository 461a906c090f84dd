"""The per-tensor FP8 projection's install sites on toy models (no GPU): exact-class matching,
hook refusal, pack-before-mutate atomicity and the receipts, with stand-ins for the third-party
model classes the reference's installers audit (instinctflash/runtime/dreamzero_fp8.py:14-70,
cosmos_fp8.py:18-107, groot_fp8.py:5-27)."""
import sys
import types

import pytest
from torch import nn

from instinctflash_b200.runtime import install_fp8 as I


class FakeFP8Linear(nn.Module):
    """Stands in for SM100FP8Linear (which needs a CUDA device): records its source, refuses what the
    real one refuses."""
    recipe = "e4m3fn_weights_dynamic_per_tensor_activations_fp32_accum_bf16_output"

    def __init__(self, linear):
        super().__init__()
        if type(linear) is not nn.Linear:
            raise TypeError("FP8 packing requires a plain nn.Linear with no custom forward")
        if linear.in_features % 16 or linear.out_features % 16:
            raise ValueError("FP8 projection input/output dimensions must be multiples of 16")
        self.source = linear


def fake_module(monkeypatch, name, **classes):
    parts = name.split(".")
    for i in range(1, len(parts) + 1):
        key = ".".join(parts[:i])
        if key not in sys.modules:
            monkeypatch.setitem(sys.modules, key, types.ModuleType(key))
    mod = sys.modules[name]
    for k, v in classes.items():
        monkeypatch.setattr(mod, k, v, raising=False)
    return mod


def lin(i=32, o=48, bias=True):
    return nn.Linear(i, o, bias=bias)


# ------------------------------------------------------------------------------------- DreamZero
class CausalWanSelfAttention(nn.Module):
    def __init__(self):
        super().__init__()
        self.q, self.k, self.v, self.o = lin(), lin(), lin(), lin()


class CausalWanAttentionBlock(nn.Module):
    def __init__(self):
        super().__init__()
        self.self_attn = CausalWanSelfAttention()
        self.ffn = nn.Sequential(lin(32, 64), nn.GELU(), lin(64, 32))


class LookAlike(CausalWanSelfAttention):   # a subclass must not be touched
    pass


def dreamzero_head(blocks=2, extra=None):
    head = types.SimpleNamespace(model=nn.ModuleList([CausalWanAttentionBlock() for _ in range(blocks)]),
                                 num_inference_steps=16, dit_step_mask=[1, 0, 1], dynamic_cache_schedule=True)
    if extra is not None:
        head.model.append(extra)
    return head


@pytest.fixture
def dreamzero(monkeypatch):
    fake_module(monkeypatch, "groot.vla.model.dreamzero.modules.wan_video_dit_action_casual_chunk",
                CausalWanSelfAttention=CausalWanSelfAttention, CausalWanAttentionBlock=CausalWanAttentionBlock)
    monkeypatch.delenv("ENABLE_TENSORRT", raising=False)


def test_dreamzero_qkv_only(dreamzero):
    head = dreamzero_head(extra=LookAlike())
    receipt = I.install_dreamzero_fp8(head, linear_type=FakeFP8Linear)
    assert receipt["recipe"] == "dreamzero_causal_qkv_" + FakeFP8Linear.recipe
    assert receipt["attention_layers"] == 2 and len(receipt["projections"]) == 6
    assert receipt["projections"][0] == {"path": "0.self_attn.q", "in_features": 32, "out_features": 48, "bias": True}
    assert receipt["scheduler_steps"] == 16 and receipt["dit_step_mask"] == [1, 0, 1] and receipt["dynamic_cache_schedule"]
    assert receipt["quality_certificate"] is not None and "only" in receipt["scope"]
    for block in list(head.model)[:2]:
        assert all(isinstance(getattr(block.self_attn, n), FakeFP8Linear) for n in "qkv")
        assert type(block.self_attn.o) is nn.Linear and type(block.ffn[0]) is nn.Linear   # output projection and FFN stay
    assert type(head.model[2].q) is nn.Linear                                            # the subclass is untouched


def test_dreamzero_with_ffn_and_refusals(dreamzero, monkeypatch):
    head = dreamzero_head()
    receipt = I.install_dreamzero_fp8(head, include_ffn=True, linear_type=FakeFP8Linear)
    assert len(receipt["projections"]) == 10 and receipt["quality_certificate"] is None
    assert {p["path"] for p in receipt["projections"]} >= {"0.ffn.0", "0.ffn.2", "1.ffn.0"}
    assert isinstance(head.model[0].ffn[0], FakeFP8Linear) and isinstance(head.model[0].ffn[1], nn.GELU)
    with pytest.raises(ValueError, match="GPU-resident"):
        I.install_dreamzero_fp8(types.SimpleNamespace(cpu_offload=True), linear_type=FakeFP8Linear)
    with pytest.raises(ValueError, match="TensorRT engine"):
        I.install_dreamzero_fp8(types.SimpleNamespace(trt_engine=object()), linear_type=FakeFP8Linear)
    monkeypatch.setenv("ENABLE_TENSORRT", "TRUE")
    with pytest.raises(ValueError, match="TensorRT execution path"):
        I.install_dreamzero_fp8(dreamzero_head(), linear_type=FakeFP8Linear)
    monkeypatch.delenv("ENABLE_TENSORRT")
    with pytest.raises(ValueError, match="No audited"):
        I.install_dreamzero_fp8(types.SimpleNamespace(model=nn.ModuleList([nn.Linear(16, 16)])), linear_type=FakeFP8Linear)


def test_a_hooked_projection_or_a_bad_shape_leaves_the_model_untouched(dreamzero):
    head = dreamzero_head()
    head.model[1].self_attn.k.register_forward_hook(lambda m, i, o: None)
    with pytest.raises(ValueError, match="hooked DreamZero projection 1.self_attn.k"):
        I.install_dreamzero_fp8(head, linear_type=FakeFP8Linear)
    assert all(type(getattr(b.self_attn, n)) is nn.Linear for b in head.model for n in "qkv")
    head = dreamzero_head()
    head.model[1].self_attn.v = nn.Linear(32, 40)            # 40 is not a multiple of 16: packing fails late in the list
    with pytest.raises(ValueError, match="multiples of 16"):
        I.install_dreamzero_fp8(head, linear_type=FakeFP8Linear)
    assert all(type(getattr(b.self_attn, n)) is nn.Linear for b in head.model for n in "qkv")   # nothing half-converted


# ------------------------------------------------------------------------------------- Cosmos
class PackedAttentionMoT(nn.Module):
    def __init__(self):
        super().__init__()
        for n in I.COSMOS_PROJECTIONS + ("o_proj",):
            setattr(self, n, lin())


class Qwen3VLTextMLP(nn.Module):
    def __init__(self):
        super().__init__()
        self.gate_proj, self.up_proj, self.down_proj = lin(32, 64), lin(32, 64), lin(64, 32)


class Nemotron3DenseVLMLP(nn.Module):
    def __init__(self):
        super().__init__()
        self.up_proj, self.down_proj = lin(32, 64), lin(64, 32)


class MoTDecoderLayer(nn.Module):
    def __init__(self, second=Nemotron3DenseVLMLP):
        super().__init__()
        self.attn = PackedAttentionMoT()
        self.mlp, self.mlp_moe_gen = Qwen3VLTextMLP(), second()


@pytest.fixture
def cosmos(monkeypatch):
    fake_module(monkeypatch, "cosmos_framework.model.generator.mot.unified_mot", PackedAttentionMoT=PackedAttentionMoT,
                MoTDecoderLayer=MoTDecoderLayer, Qwen3VLTextMLP=Qwen3VLTextMLP, Nemotron3DenseVLMLP=Nemotron3DenseVLMLP)


def test_cosmos_attention_and_dense_mlp(cosmos):
    model = nn.ModuleList([MoTDecoderLayer(), MoTDecoderLayer()])
    receipt = I.install_cosmos_fp8(model, linear_type=FakeFP8Linear)
    assert receipt["attention_layers"] == 2 and len(receipt["projections"]) == 12
    assert receipt["recipe"].startswith("cosmos_mot_qkv_")
    assert isinstance(model[0].attn.q_proj_moe_gen, FakeFP8Linear) and type(model[0].attn.o_proj) is nn.Linear
    receipt = I.install_cosmos_dense_mlp_fp8(model, linear_type=FakeFP8Linear)
    assert receipt["mlp_modules"] == 4 and len(receipt["projections"]) == 2 * (3 + 2)
    assert receipt["projections"][0]["path"] == "0.mlp.gate_proj"
    assert isinstance(model[1].mlp_moe_gen.down_proj, FakeFP8Linear)
    with pytest.raises(ValueError, match="No audited PackedAttentionMoT"):
        I.install_cosmos_fp8(nn.ModuleList([nn.Linear(16, 16)]), linear_type=FakeFP8Linear)
    with pytest.raises(ValueError, match="Unsupported Cosmos dense MLP type"):
        I.install_cosmos_dense_mlp_fp8(nn.ModuleList([MoTDecoderLayer(second=nn.Identity)]), linear_type=FakeFP8Linear)


# ------------------------------------------------------------------------------------- GR00T
class Qwen3VLTextAttention(nn.Module):
    def __init__(self):
        super().__init__()
        self.q_proj, self.k_proj, self.v_proj, self.o_proj = lin(), lin(), lin(), lin(48, 32)


def test_groot_backbone(monkeypatch):
    fake_module(monkeypatch, "transformers.models.qwen3_vl.modeling_qwen3_vl", Qwen3VLTextAttention=Qwen3VLTextAttention,
                Qwen3VLTextMLP=Qwen3VLTextMLP)
    backbone = nn.ModuleDict({"layer": nn.ModuleList([Qwen3VLTextAttention(), Qwen3VLTextMLP()]), "vision": nn.Linear(32, 32)})
    receipt = I.install_groot_backbone_fp8(backbone, linear_type=FakeFP8Linear)
    assert len(receipt["projections"]) == 7 and "bias" not in receipt["projections"][0]
    assert receipt["recipe"].startswith("groot_qwen3_text_") and receipt["quality_certificate"] is None
    assert isinstance(backbone["layer"][0].o_proj, FakeFP8Linear) and type(backbone["vision"]) is nn.Linear


def test_default_linear_type_is_the_sm100_projection(dreamzero):
    """Without a stand-in the installers build SM100FP8Linear, which refuses CPU weights: the model
    stays as it was."""
    head = dreamzero_head()
    with pytest.raises(ValueError, match="capability"):
        I.install_dreamzero_fp8(head)
    assert type(head.model[0].self_attn.q) is nn.Linear
