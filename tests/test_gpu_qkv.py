"""Parity of the QKV consumers (``qkv_split``, ``wan_qkv``) through the C ABI.

Evidence per case: vectors recorded from the unmodified reference kernels on a B200
(``golden/golden_b200_qkv.json``) and the CPU oracle on the same seeded inputs.  Outputs that
pass through no RMS norm must equal the recording bit for bit (same dequantisation chain, same
rotation, same sine and cosine routines); normed outputs differ only in the order the squares
are summed, so they are held to the GEMM bar of this build (relative Frobenius error <= 1e-3,
max|delta| <= 2^-7 x row absmax) and in practice to a unit in the last place of the output type.
"""
import pytest
import torch

import cases
from util import golden, rel_frobenius, sha

pytestmark = pytest.mark.gpu

DEV = "cuda"


@pytest.fixture(scope="module")
def ops():
    from instinctflash_b200 import _lib
    from instinctflash_b200.kernels import rope, wan
    _lib.lib()   # raises if the CUDA library is missing: no fallback
    return dict(rope=rope, wan=wan)


@pytest.fixture(scope="module")
def oracle():
    from oracle import oracle as O
    return O


@pytest.fixture(scope="module")
def G():
    return golden("golden_b200_qkv.json")


def dev(t):
    return None if t is None else t.to(DEV)


def bits(t):
    return t.detach().contiguous().cpu().float().flatten().view(torch.int32)


def check(got, rec, want_oracle, exact, what, stride=97):
    """``rec``: the reference's recording; ``want_oracle``: the CPU oracle's tensor."""
    flat = got.detach().contiguous().cpu().float().flatten()
    ref_sample = torch.tensor(rec["sample"], dtype=torch.int32).view(torch.float32)
    ref_head = torch.tensor(rec["head"], dtype=torch.int32).view(torch.float32)
    if exact:
        assert torch.equal(flat[:64].view(torch.int32), ref_head.view(torch.int32)), f"{what}: first elements differ from the reference"
        assert sha(got) == rec["sha"], f"{what}: differs from the reference's recording"
    else:
        mine = flat[::stride]
        scale = ref_sample.abs().max().clamp_min(1e-30)
        assert ((mine - ref_sample).abs().max() / scale).item() <= 2.0 ** -7, f"{what}: sample too far from the reference"
        assert rel_frobenius(mine[None], ref_sample[None]) <= 1e-3, what
        assert rel_frobenius(flat[:64][None], ref_head[None]) <= 1e-3, what
    o = want_oracle.float().flatten()
    assert rel_frobenius(flat[None], o[None]) <= 1e-3, f"{what}: far from the CPU oracle"
    assert ((flat - o).abs().max() / o.abs().max().clamp_min(1e-30)).item() <= 2.0 ** -7, f"{what}: far from the CPU oracle"


@pytest.mark.parametrize("name,c", list(cases.qkv_split_cases()), ids=lambda v: v if isinstance(v, str) else "")
def test_qkv_split(ops, oracle, G, name, c):
    T, HQ, HKV, HD, odt = c["qkv"].shape[0], c["heads_q"], c["heads_kv"], c["head_dim"], c["out_dtype"]
    q = torch.zeros(T, HQ, HD, device=DEV, dtype=odt)
    k = torch.zeros(c["kv_rows"], HKV, HD, device=DEV, dtype=odt)
    v = torch.zeros_like(k)
    base = torch.tensor([c["kv_base"]], device=DEV, dtype=torch.int32) if c["dynamic_base"] else c["kv_base"]
    kw = dict(heads_q=HQ, heads_kv=HKV, head_dim=HD, row=c["row"], col=c["col"], bias=c["bias"], inv_freq=c["inv_freq"],
              pos=c["pos"], sections=c["sections"], q_norm=c["q_norm"], k_norm=c["k_norm"])
    ops["rope"].qkv_split(dev(c["qkv"]), q, k, v, kv_base=base, **{n: dev(t) if torch.is_tensor(t) else t for n, t in kw.items()})
    qo, ko, vo = oracle.qkv_split(c["qkv"], kv_rows=c["kv_rows"], kv_base=c["kv_base"], out_dtype=odt, **kw)
    rec = G[f"qkv_split/{name}"]
    normed = c["q_norm"] is not None
    check(q, rec["q"], qo, not normed, f"{name}/q")
    check(k, rec["k"], ko, not normed, f"{name}/k")
    check(v, rec["v"], vo, True, f"{name}/v")
    lo, hi = c["kv_base"], c["kv_base"] + T
    assert k[:lo].abs().max().item() == 0 if lo else True
    assert k[hi:].abs().max().item() == 0 if hi < c["kv_rows"] else True


@pytest.mark.parametrize("name,c", list(cases.wan_qkv_cases()), ids=lambda v: v if isinstance(v, str) else "")
def test_wan_qkv(ops, oracle, G, name, c):
    n_rows, D, odt, parts, S = c["raw"].shape[0], c["heads"] * c["head_dim"], c["out_dtype"], c["parts"], c["pool_rows"]
    B = n_rows // c["tokens"]
    q = torch.zeros(n_rows, D, device=DEV, dtype=odt)
    kp = torch.zeros(B, S, D, device=DEV, dtype=odt) if parts >= 2 else None
    vp = torch.zeros(B, S, D, device=DEV, dtype=odt) if parts >= 3 else None
    kw = dict(heads=c["heads"], head_dim=c["head_dim"], tokens=c["tokens"], slots=c["slots"], row=c["row"], col=c["col"],
              bias=c["bias"], q_norm=c["q_norm"], k_norm=c["k_norm"], pos=c["pos"], sections=c["sections"],
              inv_freq=c["inv_freq"])
    ops["wan"].wan_qkv(dev(c["raw"]), q, k_pool=kp, v_pool=vp, **{n: dev(t) if torch.is_tensor(t) else t for n, t in kw.items()})
    qo, ko, vo = oracle.wan_qkv(c["raw"], parts=parts, pool_rows=S, out_dtype=odt, **kw)
    rec = G[f"wan_qkv/{name}"]
    check(q, rec["q"], qo, c["q_norm"] is None, f"{name}/q")
    if kp is not None:
        check(kp, rec["k"], ko, c["k_norm"] is None, f"{name}/k")
    if vp is not None:
        check(vp, rec["v"], vo, True, f"{name}/v")


def test_qkv_split_under_graph_follows_device_base(ops):
    """K/V rows follow a device-resident base across replays of one captured graph
    (instinctflash/kernels/rope.py:11-12)."""
    c = dict(cases.qkv_split_cases())["pi05_expert"]
    T, HQ, HKV, HD = c["qkv"].shape[0], c["heads_q"], c["heads_kv"], c["head_dim"]
    x = dev(c["qkv"])
    q = torch.zeros(T, HQ, HD, device=DEV, dtype=torch.float16)
    k = torch.zeros(c["kv_rows"], HKV, HD, device=DEV, dtype=torch.float16)
    v = torch.zeros_like(k)
    base = torch.tensor([3], device=DEV, dtype=torch.int32)
    row, col, inv, pos = dev(c["row"]), dev(c["col"]), dev(c["inv_freq"]), dev(c["pos"])

    def run():
        ops["rope"].qkv_split(x, q, k, v, heads_q=HQ, heads_kv=HKV, head_dim=HD, row=row, col=col,
                              inv_freq=inv, pos=pos, kv_base=base)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        run()
    torch.cuda.current_stream().wait_stream(side)
    eager_k = k.clone()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        run()
    k.zero_()
    base.fill_(60)
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(k[60:60 + T], eager_k[3:3 + T])
    assert k[:60].abs().max().item() == 0
