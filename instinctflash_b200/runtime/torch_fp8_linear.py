"""Inference-only per-tensor FP8 projection for sm_100.

``SM100FP8Linear`` follows ``ThorFP8Linear`` of ``instinctflash/runtime/torch_fp8_linear.py``
(lines 10-79): same constructor checks and packed buffers (``weight_fp8`` [N, K] e4m3,
``weight_scale`` [1] float32, ``bias`` bf16 or None), same recipe string, same forward contract
(bf16 in, bf16 out, empty input -> empty output).  The forward is ``dynamic_pack_bf16_e4m3``
followed by the tcgen05 GEMM with both per-tensor scales and the bias applied to the fp32
accumulator in its epilogue (the place of ``torch._scaled_mm`` at lines 74-78).
"""
from __future__ import annotations

import torch
from torch import nn

from ..kernels.fp8 import Fp8Weight, fp8_linear
from .fp8_pack import dynamic_pack_bf16_e4m3


def _target_device(weight: torch.Tensor, device, storage_device, capabilities) -> torch.device:
    """Where the packed projection will live; raises for everything the recipe does not cover
    (same conditions and messages as the reference's constructor, minus its CPU-source branch)."""
    target = weight.device if device is None else torch.device(device)
    on_cuda = target.type == "cuda"
    if not on_cuda or torch.cuda.get_device_capability(target) not in capabilities:
        raise ValueError(f"FP8 projections require CUDA capability in {capabilities}")
    if storage_device is not None and torch.device(storage_device) != target:
        raise ValueError("Packed storage lives on the target device for this recipe")
    if weight.device != target:
        # "cuda" without an index and the current CUDA device are the same place
        resolved = torch.device("cuda", torch.cuda.current_device() if target.index is None else target.index)
        if weight.device != resolved:
            raise ValueError("Pack FP8 weights on their target device")
    return target


def pack_per_tensor(weight: torch.Tensor):
    """(codes [N, K] e4m3, scale [1] float32) with one scale for the whole matrix:
    scale = max(|w|, 1e-12) / 448 -- on CUDA torch divides a tensor by a Python scalar by
    multiplying with fp32(1/448), the arithmetic the reference pins
    (instinctflash/runtime/torch_fp8_linear.py:39-48, tests/test_sm89_fp8.py:48-56)."""
    wide = weight.float()
    scale = wide.abs().amax().clamp_min(1e-12).reshape(1) / 448.0
    codes = (wide / scale).clamp(-448, 448).to(torch.float8_e4m3fn).contiguous()
    return codes, scale


class SM100FP8Linear(nn.Module):
    recipe = "e4m3fn_weights_dynamic_per_tensor_activations_fp32_accum_bf16_output"
    supported_capabilities = ((10, 0), (10, 3))

    def __init__(self, linear: nn.Linear, *, device=None, storage_device=None):
        super().__init__()
        if type(linear) is not nn.Linear:
            raise TypeError("FP8 packing requires a plain nn.Linear with no custom forward")
        weight = linear.weight.detach()
        _target_device(weight, device, storage_device, self.supported_capabilities)
        bias = None if linear.bias is None else linear.bias.detach().clone()
        problems = (
            (weight.dtype != torch.bfloat16, "This FP8 recipe requires native BF16 projection weights"),
            (linear.in_features % 16 or linear.out_features % 16,
             "FP8 projection input/output dimensions must be multiples of 16"),
            (weight.dtype == torch.bfloat16 and not torch.isfinite(weight).all(), "Cannot quantize non-finite projection weights"),
            (bias is not None and (bias.dtype != torch.bfloat16 or not torch.isfinite(bias).all()),
             "This FP8 recipe requires finite BF16 bias"),
        )
        for bad, message in problems:
            if bad:
                raise ValueError(message)
        self.in_features, self.out_features = linear.in_features, linear.out_features
        codes, scale = pack_per_tensor(weight)
        self.register_buffer("weight_fp8", codes)
        self.register_buffer("weight_scale", scale)
        self.register_buffer("bias", bias)

    @torch.no_grad()
    def forward(self, x):
        if x.ndim < 1 or x.shape[-1] != self.in_features:
            raise ValueError("FP8 projection input has incompatible feature dimension")
        if x.dtype != torch.bfloat16 or x.device != self.weight_fp8.device:
            raise ValueError("FP8 projection input must be BF16 on the packed weight device")
        if self.weight_fp8.dtype != torch.float8_e4m3fn or self.weight_scale.dtype != torch.float32:
            raise RuntimeError("FP8 packed buffers were cast after construction; pack after model.to()")
        shape = (*x.shape[:-1], self.out_features)
        if x.numel() == 0:
            return x.new_empty(shape)     # a model may call a tower whose token partition is empty
        rows = x.reshape(-1, self.in_features).contiguous()
        packed, scale = dynamic_pack_bf16_e4m3(rows)
        out = torch.empty(rows.shape[0], self.out_features, device=x.device, dtype=torch.bfloat16)
        fp8_linear(packed, scale, Fp8Weight(self.weight_fp8, self.weight_scale, None), out,
                   bias=self.bias, use_weight_bias=False, exact=True)
        return out.reshape(shape)
