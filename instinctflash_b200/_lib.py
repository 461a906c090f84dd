"""ctypes binding of ``libiflb200.so`` (declared in ``include/iflb200.h``).

The library is looked up at ``$IFLB200_KERNEL_LIBRARY`` first, then next to this file (the
in-tree build output of :mod:`instinctflash_b200.build`).  There is no fallback: when the
library is missing or its ABI version differs, :func:`lib` raises, and so does every operator
of this package.  Same convention as the reference's raw-pointer loaders
(instinctflash/backends/sm120_residual.py:17-57,72-88).
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

LIBRARY_ENV = "IFLB200_KERNEL_LIBRARY"
LIBRARY_NAME = "libiflb200.so"
ABI_VERSION = 1

F32, BF16, F16 = 0, 1, 2
ERR_ARG, ERR_SHAPE, ERR_ALIGN, ERR_DTYPE = -1, -2, -3, -4   # IFLB200_ERR_* of include/iflb200.h
ROUND_ENGINE, ROUND_EXACT = 0, 1

_p = ctypes.c_void_p
_i = ctypes.c_int
_l = ctypes.c_int64
_f = ctypes.c_float
_z = ctypes.c_size_t

# name -> (restype, argtypes); one entry per declaration of include/iflb200.h
SIGNATURES = {
    "iflb200_abi_version": (_i, []),
    "iflb200_status_string": (ctypes.c_char_p, [_i]),
    "iflb200_row_quant": (_i, [_p, _i, _l, _i, _i, _p, _p, _p, _i, _p, _l, _p, _p]),
    "iflb200_row_quant_sharded": (_i, [_p, _i, _l, _i, _i, _p, _p, _p, _i, _i, _p, _p, _l, _p, _p]),
    "iflb200_row_max_sharded": (_i, [_p, _i, _l, _i, _i, _p, _p, _p, _i, _p, _p, _i, _p]),
    "iflb200_quant_from_amax": (_i, [_p, _l, _i, _i, _p, _p, _p, _l, _p, _p]),
    "iflb200_dequant_rows": (_i, [_p, _i, _l, _i, _i, _p, _p, _p, _p, _i, _l, _p]),
    "iflb200_gated_act_quant": (_i, [_p, _i, _l, _i, _i, _p, _p, _i, _p, _l, _p, _p]),
    "iflb200_residual_norm_quant": (_i, [_p, _i, _l, _i, _i, _p, _l, _p, _p, _p, _p, _i, _i, _p, _p,
                                         _p, _p, _p, _f, _p, _l, _p, _p, _i, _l, _p]),
    "iflb200_residual_norm_quant_partials": (_i, [_p, _i, _l, _i, _i, _p, _i, _l, _p, _p, _p, _p, _i, _i, _p, _p,
                                                  _p, _p, _p, _f, _p, _l, _p, _p, _i, _l, _p]),
    "iflb200_residual_norm_quant_peers": (_i, [_p, _i, _l, _i, _i, _p, _i, _l, _p, _p, _p, _p, _i, _i, _p, _p,
                                               _p, _p, _p, _f, _p, _l, _p, _p, _p, _i, _p]),
    "iflb200_qkv_split": (_i, [_p, _i, _l, _i, _i, _i, _i, _p, _p, _p, _p, _p, _f, _p, _p, _l, _p, _p, _i,
                               _p, _l, _l, _p, _l, _l, _p, _l, _l, _i, _p]),
    "iflb200_wan_qkv": (_i, [_p, _i, _l, _i, _i, _i, _i, _p, _p, _p, _p, _p, _f, _p, _p, _l, _p, _p,
                             _p, _l, _p, _l, _l, _p, _l, _l, _i, _p]),
    "iflb200_attn_combine_quant": (_i, [_p, _p, _p, _i, _i, _i, _i, _i, _i, _p, _i, _l, _l, _l, _p, _l, _p, _p]),
    "iflb200_gemm_fp8_raw": (_i, [_p, _l, _p, _l, _i, _i, _i, _p, _l, _p]),
    "iflb200_gemm_fp8_partials": (_i, [_p, _l, _p, _l, _i, _i, _i, _i, _p, _l, _p]),
    "iflb200_fp8_linear": (_i, [_p, _l, _p, _l, _i, _i, _i, _p, _i, _p, _i, _p, _i, _i, _p, _i, _l, _p]),
    "iflb200_fp8_linear_residual": (_i, [_p, _l, _p, _l, _i, _i, _i, _p, _p, _p, _p, _p, _p, _i, _l, _p]),
    "iflb200_fp8_linear_gated": (_i, [_p, _l, _p, _l, _i, _i, _i, _p, _p, _i, _p, _l, _p, _p]),
    "iflb200_pack_workspace_bytes": (_z, [_l]),
    "iflb200_dynamic_pack_bf16_e4m3": (_i, [_p, _l, _p, _p, _p, _z, _p]),
    "iflb200_dynamic_pack_bf16_e4m3_noalloc": (_i, [_p, _l, _p, _p, _p]),
    "iflb200_pack_bf16_e4m3": (_i, [_p, _l, _p, _p, _p]),
    "iflb200_encode_operand_map": (_i, [_p, _p, _i, _i, _l, _i]),
    "iflb200_encode_gated_weight_map": (_i, [_p, _p, _i, _i, _l]),
    "iflb200_stack_activation_box_rows": (_i, [_i]),
    "iflb200_stack_weight_box_rows": (_i, []),
    "iflb200_stack_run": (_i, [_p, _i, _p, _p, _i, _i, _p, _p]),
    "iflb200_gemm_take_timeout_record": (_i, [ctypes.POINTER(ctypes.c_uint32), _p]),
    "iflb200_encode_rowblock_map": (_i, [_p, _i, _i, _l, _p]),
    "iflb200_gemm_fp8_rowblocks": (_i, [_p, _l, _p, _l, _i, _i, _i, _i, _p, _p]),
    "iflb200_peer_barrier": (_i, [_p, _p, _p, _i, _i, _p, _p]),
    "iflb200_peer_exchange": (_i, [_p, _p, _p, _i, _i, _p, _p, _p, _i, _p]),
    "iflb200_set_wait_budget_us": (_i, [_l]),
    "iflb200_gemm_last_launch": (_i, [ctypes.POINTER(_i), ctypes.POINTER(_i), ctypes.POINTER(_i)]),
    "iflb200_gemm_set_config": (_i, [_i, _i, _i]),
    "iflb200_gemm_set_mode": (_i, [_i]),
    "iflb200_set_dependent_launch": (_i, [_i]),
    "iflb200_gemm_set_split_k": (_i, [_i]),
    "iflb200_row_set_group": (_i, [_i]),
}

_LIB = None


def library_candidates() -> tuple[Path, ...]:
    configured = os.environ.get(LIBRARY_ENV)
    packaged = Path(__file__).resolve().parent / LIBRARY_NAME
    return tuple([Path(configured)] if configured else []) + (packaged,)


def _open(path: Path):
    if not path.is_file():
        return None
    try:
        handle = ctypes.CDLL(str(path))
        version = handle.iflb200_abi_version
        version.argtypes, version.restype = [], ctypes.c_int
        return handle if int(version()) == ABI_VERSION else None
    except (OSError, AttributeError):
        return None


def available() -> bool:
    return any(_open(p) is not None for p in library_candidates())


def lib():
    """The loaded library with argument types set.  Raises when it cannot be loaded."""
    global _LIB
    if _LIB is None:
        for path in library_candidates():
            handle = _open(path)
            if handle is not None:
                for name, (restype, argtypes) in SIGNATURES.items():
                    fn = getattr(handle, name)
                    fn.restype, fn.argtypes = restype, argtypes
                handle.path = path
                _LIB = handle
                break
        else:
            searched = ", ".join(str(p) for p in library_candidates())
            raise RuntimeError(
                f"iflb200 ABI v{ABI_VERSION} is unavailable; searched {searched}. Build it with "
                f"`python -m instinctflash_b200.build` or point {LIBRARY_ENV} at {LIBRARY_NAME}. "
                "There is no CPU or PyTorch fallback for this path.")
    return _LIB


def check(status: int, what: str) -> None:
    if status != 0:
        message = lib().iflb200_status_string(int(status)).decode()
        raise RuntimeError(f"{what} failed with status {status}: {message}")


def dtype_code(dtype) -> int:
    import torch

    try:
        return {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}[dtype]
    except KeyError:
        raise ValueError(f"unsupported element type {dtype}; expected float32, bfloat16 or float16") from None


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def stream_handle(device=None) -> int:
    import torch

    return torch.cuda.current_stream(device).cuda_stream
