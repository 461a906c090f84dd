"""The barrier / exchange kernel between tensor-parallel ranks, on ONE GPU: the peers' flag words and
buffers are local stand-ins that the test sets itself, so no kernel here waits for another kernel.
The two-process runs over NVLink are in test_multi_gpu.py."""
import ctypes

import pytest
import torch

from instinctflash_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


def _ptrs(*tensors):
    return torch.tensor([t.data_ptr() for t in tensors], dtype=torch.int64, device=DEV)


def _exchange(lib, flag_ptrs, my_flags, arrival, rank, p, status, max_in=None, max_out=None, max_n=0):
    st = lib.iflb200_peer_exchange(flag_ptrs.data_ptr(), my_flags.data_ptr(), arrival.data_ptr(), rank, p,
                                   status.data_ptr(), None if max_in is None else max_in.data_ptr(),
                                   None if max_out is None else max_out.data_ptr(), max_n,
                                   torch.cuda.current_stream().cuda_stream)
    assert st == 0, st


def test_exchange_signals_every_peer_and_reduces_the_maxima():
    """Rank 1 of 3 with both peers already arrived (their words preset): arrival number 1 is stored
    into word 1 of both peers' flags, the arrival counter advances, and the slots are reduced with
    max -- twice, the second time with arrival 2."""
    lib = _lib.lib()
    p, rank, n = 3, 1, 1000
    flags = [torch.zeros(p, dtype=torch.int32, device=DEV) for _ in range(p)]   # flags[r] = rank r's words
    arrival = torch.zeros(1, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    g = torch.Generator(device="cpu").manual_seed(5)
    slots = torch.rand(p, n, generator=g).to(DEV)                               # this rank's [p][n] maxima slots
    out = torch.zeros(n, device=DEV)
    flag_ptrs = _ptrs(*flags)
    for e in (1, 2):
        flags[rank][0] = e
        flags[rank][2] = e                                                      # "peers 0 and 2 have arrived"
        _exchange(lib, flag_ptrs, flags[rank], arrival, rank, p, status, max_in=slots, max_out=out, max_n=n)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert int(arrival.item()) == e
        for r in (0, 2):
            assert int(flags[r][rank].item()) == e
            assert int(flags[r][0].item()) == 0 and int(flags[r][2].item()) == 0   # only this rank's word
        assert torch.equal(out, slots.amax(0))
        slots.mul_(0.5)


def test_plain_barrier_is_the_exchange_without_a_reduction():
    lib = _lib.lib()
    flags = [torch.zeros(2, dtype=torch.int32, device=DEV) for _ in range(2)]
    flags[0][1] = 1
    arrival = torch.zeros(1, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    st = lib.iflb200_peer_barrier(_ptrs(*flags).data_ptr(), flags[0].data_ptr(), arrival.data_ptr(), 0, 2,
                                  status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert st == 0
    torch.cuda.synchronize()
    assert (int(status.item()), int(arrival.item()), int(flags[1][0].item())) == (0, 1, 1)


def test_a_peer_that_never_arrives_runs_the_wait_out_and_leaves_the_context_usable():
    """Nothing sets this rank's word for peer 1: after the (shortened) budget the kernel records
    0x50000000 | peer << 16 | arrival and returns; the next call on the same context works."""
    lib = _lib.lib()
    flags = [torch.zeros(2, dtype=torch.int32, device=DEV) for _ in range(2)]
    arrival = torch.zeros(1, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ptrs = _ptrs(*flags)
    try:
        assert lib.iflb200_set_wait_budget_us(3000) == 0
        _exchange(lib, ptrs, flags[0], arrival, 0, 2, status)
        torch.cuda.synchronize()                                               # returns: the wait is bounded
    finally:
        assert lib.iflb200_set_wait_budget_us(0) == 0
    assert int(status.item()) & 0xFFFFFFFF == 0x50000000 | (1 << 16) | 1
    assert int(flags[1][0].item()) == 1                                        # it did signal before waiting
    status.zero_()
    flags[0][1] = 2
    _exchange(lib, ptrs, flags[0], arrival, 0, 2, status)
    torch.cuda.synchronize()
    assert (int(status.item()), int(arrival.item())) == (0, 2)


def test_argument_checks():
    lib = _lib.lib()
    f = torch.zeros(4, dtype=torch.int32, device=DEV)
    ptrs = _ptrs(f, f)
    s = torch.cuda.current_stream().cuda_stream
    assert lib.iflb200_peer_barrier(None, f.data_ptr(), f.data_ptr(), 0, 2, f.data_ptr(), s) == _lib.ERR_ARG
    assert lib.iflb200_peer_barrier(ptrs.data_ptr(), f.data_ptr(), f.data_ptr(), 2, 2, f.data_ptr(), s) == _lib.ERR_ARG
    assert lib.iflb200_peer_exchange(ptrs.data_ptr(), f.data_ptr(), f.data_ptr(), 0, 2, f.data_ptr(), None, None, 8,
                                     s) == _lib.ERR_ARG
    assert lib.iflb200_peer_exchange(ptrs.data_ptr(), f.data_ptr() + 2, f.data_ptr(), 0, 2, f.data_ptr(), None, None, 0,
                                     s) == _lib.ERR_ALIGN


# ---- the fused kernels of the tensor-parallel row-split linear, with local stand-ins for the peers ----
E4M3 = torch.float8_e4m3fn


def _codes(rows, cols, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(rows, cols, generator=g) * 0.5).to(DEV).to(E4M3)


@pytest.mark.parametrize("groups,group_rows,N,K", [(2, 300, 512, 256), (3, 128, 256, 512), (2, 2340, 3072, 1536),
                                                   (4, 40, 64, 128)])
def test_rowblock_gemm_equals_one_call_per_block_and_stays_inside_each_destination(groups, group_rows, N, K):
    from instinctflash_b200.kernels import fp8
    a = _codes(groups * group_rows, K, 1)
    w = fp8.Fp8Weight(_codes(N, K, 2), None, None)
    guard = 8
    outs = [torch.full((group_rows + guard, N), -7.0, device=DEV) for _ in range(groups)]
    maps = fp8.encode_rowblock_maps([o[:group_rows] for o in outs])
    fp8.gemm_rowblocks(a, w, group_rows, maps)
    family = ctypes.c_int()
    _lib.lib().iflb200_gemm_last_launch(ctypes.byref(family), None, None)
    assert family.value == 1 + 32
    torch.cuda.synchronize()
    for g in range(groups):
        want = torch.empty(group_rows, N, device=DEV)
        fp8.fp8_linear(a[group_rows * g: group_rows * (g + 1)], None, w, want, use_weight_bias=False, exact=True)
        assert torch.equal(outs[g][:group_rows], want), g
        assert bool((outs[g][group_rows:] == -7.0).all()), g       # rows of the next block were loaded, never stored


def test_row_max_with_mirrors_is_phase_one_everywhere():
    from instinctflash_b200.kernels import norm
    g = torch.Generator(device="cpu").manual_seed(3)
    M, K = 333, 1536
    x = (torch.randn(M, K, generator=g) * 40).to(torch.bfloat16).to(DEV)
    row = torch.rand(M, generator=g).to(DEV)
    col = torch.rand(K, generator=g).to(DEV)
    want = torch.empty(M, device=DEV)
    norm.row_quant_sharded(x, None, None, want, 1, row=row, col=col, gelu=True)
    got = torch.zeros(M, device=DEV)
    mirrors = [torch.zeros(M, device=DEV) for _ in range(3)]
    norm.row_max_sharded(x, got, mirrors, row=row, col=col, gelu=True)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    for t in mirrors:
        assert torch.equal(t, want)


@pytest.mark.parametrize("D,planes", [(3072, 2), (5120, 2), (1024, 4), (8192, 3)])
def test_residual_kernel_writes_the_same_codes_and_scales_into_the_mirrors(D, planes):
    """The mirrored form against the partial-sum form without mirrors (same kernel, same bits), and
    its residual against the ordinary kernel fed the planes' sum rounded to bf16."""
    from instinctflash_b200.kernels import norm
    g = torch.Generator(device="cpu").manual_seed(11)
    M = 77
    res0 = torch.randn(M, D, generator=g).to(torch.bfloat16).to(DEV)
    part = (torch.randn(planes, M, D, generator=g) * 30).to(DEV)
    drow = torch.rand(M, generator=g).to(DEV) * 0.01
    dcol = torch.rand(D, generator=g).to(DEV) * 0.1
    bias = torch.randn(D, generator=g).to(DEV) * 0.1
    gate = torch.randn(D, generator=g).to(DEV)
    kw = dict(delta_row=drow, delta_col=dcol, bias=bias, gate=gate, layernorm=True)

    def buffers():
        return torch.zeros(M, D, dtype=torch.uint8, device=DEV).view(E4M3), torch.zeros(M, device=DEV)

    res_a, (q_a, s_a) = res0.clone(), buffers()
    norm.residual_norm_quant(res_a, delta=part, q=q_a, q_scale=s_a, **kw)
    res_b, (q_b, s_b) = res0.clone(), buffers()
    mirrors = [buffers() for _ in range(2)]
    norm.residual_norm_quant_peers(res_b, delta=part, q=q_b, q_scale=s_b, q_mirrors=[m[0] for m in mirrors],
                                   q_scale_mirrors=[m[1] for m in mirrors], **kw)
    torch.cuda.synchronize()
    assert torch.equal(res_a, res_b) and torch.equal(s_a, s_b) and torch.equal(q_a.view(torch.uint8), q_b.view(torch.uint8))
    for q_m, s_m in mirrors:
        assert torch.equal(q_m.view(torch.uint8), q_b.view(torch.uint8)) and torch.equal(s_m, s_b)
    total = part[0].clone()
    for k in range(1, planes):
        total = total + part[k]
    res_c, (q_c, s_c) = res0.clone(), buffers()
    norm.residual_norm_quant(res_c, delta=total.to(torch.bfloat16), q=q_c, q_scale=s_c, **kw)
    torch.cuda.synchronize()
    assert torch.equal(res_c, res_b)                                   # the residual update has no reduction in it
    torch.testing.assert_close(s_c, s_b, rtol=1e-5, atol=0)            # the norm's sums may run in another thread layout
    differing = (q_c.view(torch.uint8) != q_b.view(torch.uint8)).float().mean().item()
    assert differing < 2e-3, differing
