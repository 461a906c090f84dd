"""The no-allocation variant of the dynamic per-tensor pack, through the C ABI.

Some hosts cannot give the library scratch memory: they run from a memory plan fixed at
start-up, have no allocator of their own, or cannot afford the device-wide stall of cudaMalloc
in a control loop.  For them
``iflb200_dynamic_pack_bf16_e4m3_noalloc`` keeps its scratch in a device array that is part of
the library image.  This file checks that it produces exactly what the workspace-taking entry
point produces, twice in a row (the array is shared and keeps the previous call's contents), and
that it refuses inputs beyond its stated capacity.  Collected last on purpose.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"
E4M3 = torch.float8_e4m3fn


def _pack_with_workspace(lib, x):
    n = x.numel()
    nbytes = int(lib.iflb200_pack_workspace_bytes(n))
    ws = torch.empty((nbytes + 3) // 4, device=DEV, dtype=torch.int32)
    q = torch.empty(x.shape, device=DEV, dtype=E4M3)
    s = torch.empty(1, device=DEV, dtype=torch.float32)
    st = lib.iflb200_dynamic_pack_bf16_e4m3(x.data_ptr(), n, q.data_ptr(), s.data_ptr(), ws.data_ptr(), nbytes,
                                            torch.cuda.current_stream().cuda_stream)
    assert st == 0
    return q, s


def _pack_noalloc(lib, x, q, s):
    return lib.iflb200_dynamic_pack_bf16_e4m3_noalloc(x.data_ptr(), x.numel(), q.data_ptr(), s.data_ptr(),
                                                      torch.cuda.current_stream().cuda_stream)


def test_noalloc_pack_matches_workspace_pack_on_consecutive_calls():
    from instinctflash_b200 import _lib
    lib = _lib.lib()
    gen = torch.Generator().manual_seed(4242)
    # two different inputs back to back: a large one that uses many scratch words, then a small
    # one that must not be disturbed by what the first left behind
    first = (torch.randn(2048, 5120, generator=gen) * 3.0).to(torch.bfloat16).to(DEV)
    second = (torch.randn(40, 2048, generator=gen) * 1e-3).to(torch.bfloat16).to(DEV)
    for x in (first, second):
        want_q, want_s = _pack_with_workspace(lib, x)
        q = torch.empty(x.shape, device=DEV, dtype=E4M3)
        s = torch.empty(1, device=DEV, dtype=torch.float32)
        assert _pack_noalloc(lib, x, q, s) == 0
        torch.cuda.synchronize()
        assert torch.equal(s.view(torch.int32), want_s.view(torch.int32))   # bit-exact: same kernels
        assert torch.equal(q.view(torch.uint8), want_q.view(torch.uint8))
    # and the first input again, after the small one
    want_q, want_s = _pack_with_workspace(lib, first)
    q = torch.empty(first.shape, device=DEV, dtype=E4M3)
    s = torch.empty(1, device=DEV, dtype=torch.float32)
    assert _pack_noalloc(lib, first, q, s) == 0
    torch.cuda.synchronize()
    assert torch.equal(s.view(torch.int32), want_s.view(torch.int32))
    assert torch.equal(q.view(torch.uint8), want_q.view(torch.uint8))


def test_noalloc_pack_refuses_inputs_beyond_its_capacity():
    from instinctflash_b200 import _lib
    lib = _lib.lib()
    x = torch.zeros(16, device=DEV, dtype=torch.bfloat16)
    q = torch.empty(16, device=DEV, dtype=E4M3)
    s = torch.empty(1, device=DEV, dtype=torch.float32)
    too_many = (1 << 28) + 1          # IFLB200_PACK_NOALLOC_MAX_ELEMENTS + 1; rejected before any launch
    st = lib.iflb200_dynamic_pack_bf16_e4m3_noalloc(x.data_ptr(), too_many, q.data_ptr(), s.data_ptr(), None)
    assert st == -8
    assert b"capacity" in lib.iflb200_status_string(st)
    assert lib.iflb200_dynamic_pack_bf16_e4m3_noalloc(None, 16, q.data_ptr(), s.data_ptr(), None) == -1
