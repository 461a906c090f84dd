"""Parity of the split-KV attention merge + FP8 row quantiser (through the C ABI) with the
reference's ``_attn_combine`` kernel: bit-exact against vectors recorded from the unmodified
reference on a B200, and against the CPU oracle within what its exp2f / IEEE division allow."""
import pytest
import torch

import cases
from util import E4M3, GOLDEN, assert_quant_close_to_oracle, golden, i32, sha

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def B200():
    if not (GOLDEN / "golden_b200_attn.json").exists():
        pytest.skip("vectors of the reference's _attn_combine have not been recorded yet")
    return golden("golden_b200_attn.json")


def run(c, *, write_o=True, quant=True):
    from instinctflash_b200.kernels.attention import SplitWorkspace, attn_combine
    T, HQ, HKV, HD, SP = c["tokens"], c["heads_q"], c["heads_kv"], c["head_dim"], c["splits"]
    ws = SplitWorkspace(1, T, HQ, HKV, HD, SP, DEV)
    ws.po.copy_(c["po"].flatten().to(DEV))
    ws.pm.copy_(c["pm"].flatten().to(DEV))
    ws.pl.copy_(c["pl"].flatten().to(DEV))
    o = torch.full((1, T, HQ, HD), float("nan"), device=DEV, dtype=c["out_dtype"]) if write_o else None
    q8 = torch.full((T, HQ * HD), 0x7F, device=DEV, dtype=torch.uint8).view(E4M3) if quant else None
    qs = torch.full((T,), float("nan"), device=DEV) if quant else None
    attn_combine(ws, o, heads_q=HQ, heads_kv=HKV, head_dim=HD, tokens=T, q8=q8, q8_scale=qs)
    torch.cuda.synchronize()
    return o, q8, qs


@pytest.mark.parametrize("name", [n for n, _ in cases.attn_combine_cases()])
def test_attn_combine_quant_bit_exact(B200, name):
    c = dict(cases.attn_combine_cases())[name]
    g = B200[name]
    o, q8, qs = run(c, write_o=c["write_o"])
    assert i32(qs).tolist() == g["qs_bits"], "scales differ from the reference's _attn_combine on a B200"
    assert sha(q8) == g["q_sha"], "codes differ from the reference's _attn_combine on a B200"
    if c["write_o"]:
        assert sha(o) == g["o_sha"], "merged output differs from the reference's on a B200"


@pytest.mark.parametrize("name", [n for n, _ in cases.attn_combine_cases()])
def test_attn_combine_quant_against_oracle(name):
    from oracle import oracle as O
    c = dict(cases.attn_combine_cases())[name]
    o, q8, qs = run(c)
    oo, qo, so = O.attn_combine_quant(c["po"], c["pm"], c["pl"], splits=c["splits"], batch=1, tokens=c["tokens"],
                                      heads_q=c["heads_q"], heads_kv=c["heads_kv"], head_dim=c["head_dim"],
                                      out_dtype=c["out_dtype"])
    assert not torch.isnan(o.float()).any()
    tol = 2e-3 if c["out_dtype"] != torch.float32 else 1e-5
    assert ((o.float().cpu() - oo.float()).abs().max() <= tol * oo.float().abs().max())
    assert_quant_close_to_oracle(q8, qs, qo, so, name, max_scale_ulp=16, max_code_frac=2e-2)
    # the quantised row is the merged row: dequantised codes within one e4m3 step of it
    deq = q8.float().cpu() * qs.cpu()[:, None]
    full = o.float().cpu().reshape(c["tokens"], -1)
    assert ((deq - full).abs().amax(1) <= full.abs().amax(1) * 2.0 ** -3).all()


def test_attn_combine_merge_only_and_quant_only_agree():
    c = dict(cases.attn_combine_cases())["pi05_expert"]
    o, q8, qs = run(c)
    o2, _, _ = run(c, quant=False)
    _, q3, s3 = run(c, write_o=False)
    assert torch.equal(o, o2) and torch.equal(q8.view(torch.uint8), q3.view(torch.uint8)) and torch.equal(qs, s3)


def test_attn_combine_rejects_bad_arguments():
    from instinctflash_b200.kernels.attention import SplitWorkspace, attn_combine
    ws = SplitWorkspace(2, 4, 4, 2, 64, 2, DEV)
    q8 = torch.empty(4, 256, device=DEV, dtype=torch.uint8).view(E4M3)
    with pytest.raises(ValueError, match="batch 1"):
        attn_combine(ws, None, heads_q=4, heads_kv=2, head_dim=64, tokens=4, batch=2, q8=q8, q8_scale=torch.empty(4, device=DEV))
    with pytest.raises(ValueError, match="nothing to write"):
        attn_combine(ws, None, heads_q=4, heads_kv=2, head_dim=64, tokens=4)
    with pytest.raises(ValueError, match="multiple of 4"):
        attn_combine(ws, torch.empty(1, 4, 4, 6, device=DEV), heads_q=4, heads_kv=2, head_dim=6, tokens=4)
    with pytest.raises(ValueError, match="smaller"):
        attn_combine(ws, torch.empty(1, 64, 4, 64, device=DEV), heads_q=4, heads_kv=2, head_dim=64, tokens=64)
