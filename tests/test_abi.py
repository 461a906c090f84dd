"""The C-ABI library loads without a GPU, exports every symbol the header declares, and
rejects bad arguments before it touches a device."""
import ctypes
import re
from pathlib import Path

import pytest

from instinctflash_b200 import _lib

HEADER = Path(__file__).resolve().parents[1] / "include" / "iflb200.h"


def declared_symbols():
    text = HEADER.read_text()
    return sorted(set(re.findall(r"IFLB200_API\s+[\w\s\*]+?\b(iflb200_\w+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_symbols()
    for required in ("iflb200_row_quant", "iflb200_dequant_rows", "iflb200_gated_act_quant",
                     "iflb200_residual_norm_quant", "iflb200_gemm_fp8_raw", "iflb200_fp8_linear",
                     "iflb200_fp8_linear_residual", "iflb200_dynamic_pack_bf16_e4m3", "iflb200_pack_bf16_e4m3",
                     "iflb200_abi_version"):
        assert required in names


def test_library_exports_every_declared_symbol():
    lib = _lib.lib()
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in include/iflb200.h but not exported"


def test_binding_table_matches_header():
    assert sorted(_lib.SIGNATURES) == declared_symbols()
    text = HEADER.read_text()
    for name, (_, argtypes) in _lib.SIGNATURES.items():
        decl = re.search(rf"{name}\s*\(([^;]*?)\)\s*;", text, re.S).group(1)
        n_args = 0 if decl.strip() == "void" else decl.count(",") + 1
        assert n_args == len(argtypes), f"{name}: header has {n_args} arguments, binding has {len(argtypes)}"


def test_abi_version_and_status_strings():
    lib = _lib.lib()
    assert lib.iflb200_abi_version() == _lib.ABI_VERSION
    m = re.search(r"#define IFLB200_ABI_VERSION (\d+)", HEADER.read_text())
    assert int(m.group(1)) == _lib.ABI_VERSION
    for code in range(-7, 1):
        assert lib.iflb200_status_string(code)


def test_argument_errors_are_reported_before_any_launch():
    lib = _lib.lib()
    one = ctypes.c_void_p(16)  # never dereferenced: the calls below are rejected on the host
    assert lib.iflb200_row_quant(None, 1, 16, 4, 16, None, None, None, 0, one, 16, one, None) == -1
    assert lib.iflb200_row_quant(one, 7, 16, 4, 16, None, None, None, 0, one, 16, one, None) == -4
    assert lib.iflb200_row_quant(one, 1, 1 << 20, 4, 1 << 20, None, None, None, 0, one, 1 << 20, one, None) == -2
    assert lib.iflb200_row_quant(one, 1, 8, 4, 16, None, None, None, 0, one, 16, one, None) == -1      # ld < K
    assert lib.iflb200_row_quant(one, 1, 16, 0, 16, None, None, None, 0, one, 16, one, None) == 0      # empty
    assert lib.iflb200_gated_act_quant(one, 1, 65536, 4, 32768, None, None, 0, one, 32768, one, None) == -2
    assert lib.iflb200_gated_act_quant(one, 1, 64, 4, 32, None, None, 9, one, 32, one, None) == -1
    assert lib.iflb200_gemm_fp8_raw(one, 24, one, 24, 4, 16, 24, one, 16, None) == -2                  # K % 16
    assert lib.iflb200_gemm_fp8_raw(one, 32, one, 32, 4, 24, 32, one, 24, None) == -2                  # N % 16
    assert lib.iflb200_gemm_fp8_raw(ctypes.c_void_p(8), 32, one, 32, 4, 16, 32, one, 16, None) == -3   # alignment
    assert lib.iflb200_gemm_fp8_raw(one, 32, one, 32, 0, 16, 32, one, 16, None) == 0                   # empty
    assert lib.iflb200_gemm_fp8_raw(None, 32, one, 32, 4, 16, 32, one, 16, None) == -1
    assert lib.iflb200_fp8_linear(one, 32, one, 32, 4, 16, 32, None, 1, None, 1, None, 0, 5, one, 1, 16, None) == -1
    assert lib.iflb200_fp8_linear(one, 32, one, 32, 4, 16, 32, None, 1, None, 1, None, 0, 0, one, 9, 16, None) == -4
    assert lib.iflb200_dynamic_pack_bf16_e4m3(one, 64, one, one, None, 0, None) == -7
    assert lib.iflb200_pack_workspace_bytes(1 << 20) >= 4
    assert lib.iflb200_gemm_set_config(100, 0, 0) == -1
    assert lib.iflb200_gemm_set_config(0, 0, 0) == 0


def test_missing_library_is_a_loud_error(monkeypatch, tmp_path):
    monkeypatch.setenv(_lib.LIBRARY_ENV, str(tmp_path / "nope.so"))
    monkeypatch.setattr(_lib, "_LIB", None)
    monkeypatch.setattr(_lib, "library_candidates", lambda: (tmp_path / "nope.so",))
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.lib()


def test_tuning_switches_validate_their_arguments():
    """The setters are host-only: they accept the documented values and nothing else, and the
    defaults are restored afterwards (no device is touched)."""
    lib = _lib.lib()
    try:
        for ok in (0, 1, 2, 3, 16, 128, 256, 256 + 512, 3 + 16, 1024, 2048, 4096):
            assert lib.iflb200_gemm_set_mode(ok) == 0, ok
        for bad in (-1, 4, 32, 64, 3 + 16 + 64, 128 + 256, 1024 + 2048, 8192):
            assert lib.iflb200_gemm_set_mode(bad) != 0, bad
        for ok in (0, 1, 2, 4):
            assert lib.iflb200_gemm_set_split_k(ok) == 0
        for bad in (-1, 3, 8, 16):
            assert lib.iflb200_gemm_set_split_k(bad) != 0
        for ok in (0, 1, 2):
            assert lib.iflb200_set_dependent_launch(ok) == 0
        for bad in (-1, 3):
            assert lib.iflb200_set_dependent_launch(bad) != 0
        for ok in ((0, 0, 0), (64, 0, 0), (128, 4, 2), (192, 0, 0), (224, 0, 0), (256, 3, 16)):
            assert lib.iflb200_gemm_set_config(*ok) == 0
        for bad in ((32, 0, 0), (100, 0, 0), (256, -1, 0), (256, 0, -2)):
            assert lib.iflb200_gemm_set_config(*bad) != 0
    finally:
        lib.iflb200_gemm_set_mode(0)
        lib.iflb200_gemm_set_split_k(0)
        lib.iflb200_set_dependent_launch(1)
        lib.iflb200_gemm_set_config(0, 0, 0)


def test_qkv_entry_points_reject_bad_arguments_before_any_launch():
    lib = _lib.lib()
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.addressof(buf)
    BF16, F16 = 1, 2
    # qkv_split: odd head width, head width above 512, rotary without positions, one norm vector only
    args = dict(qkv=p, dt=BF16, ld=1024, T=2, hq=1, hkv=1, hd=64)

    def split(**kw):
        a = {**args, **kw}
        return lib.iflb200_qkv_split(a["qkv"], a["dt"], a["ld"], a["T"], a["hq"], a["hkv"], a["hd"], None, None, None,
                                     kw.get("qn"), kw.get("kn"), 1e-6, kw.get("inv"), kw.get("pos"), 0, None, None, 0,
                                     p, 64, 64, p, 64, 64, p, 64, 64, F16, None)
    assert split(hd=63) != 0 and split(hd=1024) != 0
    assert split(inv=p) != 0                      # inv_freq without a position table
    assert split(qn=p) != 0                       # q_norm without k_norm
    assert split(dt=7) != 0 and split(ld=10) != 0
    assert split(T=0) == 0                        # empty input: nothing to do, no launch
    # wan_qkv: V without K, width above 8192, rotary without sections
    def wan(**kw):
        return lib.iflb200_wan_qkv(p, BF16, kw.get("ld", 3 * 256), kw.get("rows", 2), 2, kw.get("heads", 2),
                                   kw.get("hd", 128), None, None, None, None, None, 1e-6, kw.get("inv"), kw.get("pos"), 0,
                                   None, None, p, 256, kw.get("kp"), 0, 0, kw.get("vp"), 0, 0, F16, None)
    assert wan(vp=p) != 0
    assert wan(heads=80) != 0
    assert wan(inv=p, pos=p) != 0
    assert wan(ld=100) != 0
    assert wan(rows=0) == 0
