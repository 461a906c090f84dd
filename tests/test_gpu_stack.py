"""Layer stacks on the GPU: the per-operator driver against the CPU oracle driver, and the
persistent whole-stack kernel against the per-operator driver."""
import pytest
import torch

import oracle_ops
from instinctflash_b200.stack import LinearStack, StackSpec, make_inputs, make_weights

pytestmark = pytest.mark.gpu
DEV = "cuda"


def to_cpu_weights(weights):
    from types import SimpleNamespace
    out = []
    for lw in weights:
        w = {k: oracle_ops.CpuFp8Weight(v.w.cpu(), v.scale.cpu(), None if v.bias is None else v.bias.cpu())
             for k, v in lw.w.items()}
        out.append(SimpleNamespace(w=w, vec={k: v.cpu() for k, v in lw.vec.items()}))
    return out


@pytest.mark.parametrize("kind,M", [("gemma", 50), ("gemma", 200), ("wan", 96)])
def test_stack_matches_cpu_oracle_stack(kind, M):
    """Two layers end to end.  The CPU oracle divides in IEEE where the GPU uses div.full, so a few
    codes differ by one step per quantiser and the difference cascades: the residual stream must
    stay within quantisation-noise distance (the per-operator tests hold the bit-exact claims)."""
    spec = StackSpec("t", kind, 2, M, 512, 1024, 768, o_in=512, cross=kind == "wan", outlier_frac=0.02,
                     outlier_scale=10.0, seed=11)
    weights = make_weights(spec, DEV, cpu_seeded=True)
    x, attn = make_inputs(spec, DEV)
    gpu = LinearStack(spec, weights, DEV)
    gpu.load(x, attn)
    got = gpu.forward().float().cpu()
    cpu = LinearStack(spec, to_cpu_weights(weights), "cpu", ops=oracle_ops.ops())
    cpu.load(x.cpu(), attn.cpu())
    want = cpu.forward().float()
    rel = float((got - want).norm() / want.norm())
    assert rel < 2e-2, rel


@pytest.mark.parametrize("M,split", [(50, 1), (7, 1), (100, 1), (50, 8), (64, 3)])
def test_persistent_stack_against_per_operator_stack(M, split):
    from instinctflash_b200 import _lib
    from instinctflash_b200.stack_persistent import PersistentExpertStack
    spec = StackSpec("expert", "gemma", 3, M, 1024, 4096, 1536, steps=2, seed=2)
    weights = make_weights(spec, DEV)
    x, attn = make_inputs(spec, DEV)
    ref = LinearStack(spec, weights, DEV)
    ref.load(x, attn)
    _lib.lib().iflb200_gemm_set_split_k(1)   # the per-operator arm with the unsplit K loop
    try:
        ref.forward()
    finally:
        _lib.lib().iflb200_gemm_set_split_k(0)
    ps = PersistentExpertStack(spec, weights, DEV, down_split_k=split)
    ps.load(x)
    ps.forward()
    torch.cuda.synchronize()
    assert ps.timeout_record() == 0, f"a wait inside the persistent kernel timed out: {ps.timeout_record():#x}"
    if split == 1:
        # same kernels' arithmetic, same K order: bit-identical residual stream, codes and scales
        assert torch.equal(ps.res, ref.res)
        assert torch.equal(ps.q8.view(torch.uint8), ref._q8(spec.hidden).view(torch.uint8))
        assert torch.equal(ps.s0, ref.scale[0])
    else:
        # split-K partials are summed in split order before the bf16 rounding point
        rel = float((ps.res - ref.res).norm() / ref.res.norm())
        assert rel < 5e-3, rel
    # a second run on the same input gives the same bits (fixed-order reductions, no atomics on data)
    first = ps.res.clone()
    ps.load(x)
    ps.forward()
    torch.cuda.synchronize()
    assert torch.equal(ps.res, first)


def test_persistent_stack_is_graph_capturable():
    from instinctflash_b200.stack_persistent import PersistentExpertStack
    spec = StackSpec("expert", "gemma", 2, 50, 1024, 4096, 1536, steps=2, seed=3)
    weights = make_weights(spec, DEV)
    x, _ = make_inputs(spec, DEV)
    ps = PersistentExpertStack(spec, weights, DEV)
    ps.load(x)
    ps.forward()
    eager = ps.res.clone()
    torch.cuda.synchronize()
    ps.load(x)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ps.forward()
    ps.load(x)
    graph.replay()
    torch.cuda.synchronize()
    assert ps.timeout_record() == 0
    assert torch.equal(ps.res, eager)


def test_persistent_stack_rejects_unsupported_specs():
    from instinctflash_b200.stack_persistent import PersistentExpertStack
    w = []
    with pytest.raises(ValueError):
        PersistentExpertStack(StackSpec("x", "gemma", 1, 200, 1024, 4096, 1536), w, DEV)
    with pytest.raises(ValueError):
        PersistentExpertStack(StackSpec("x", "gemma", 1, 50, 1024, 4096, 1536, o_in=2048), w, DEV)
    with pytest.raises(ValueError):
        PersistentExpertStack(StackSpec("x", "wan", 1, 50, 1024, 4096, 1536), w, DEV)


@pytest.mark.parametrize("kind,M", [("gemma", 50), ("gemma", 816), ("wan", 300)])
def test_dependent_launch_modes_give_identical_results(kind, M):
    """Programmatic dependent launch only changes when a kernel may be scheduled: eager and
    CUDA-graph runs of a stack give the same bits with it off (0), automatic (1) and forced (2)."""
    from instinctflash_b200 import _lib
    lib = _lib.lib()
    spec = StackSpec("t", kind, 2, M, 1024, 2048, 1536, o_in=1024, cross=kind == "wan", seed=5)
    weights = make_weights(spec, DEV)
    x, attn = make_inputs(spec, DEV)
    results = []
    try:
        for mode in (0, 1, 2):
            assert lib.iflb200_set_dependent_launch(mode) == 0
            st = LinearStack(spec, weights, DEV)
            st.load(x, attn)
            g = st.capture()
            st.load(x, attn)          # back to the initial residual stream, then one replay
            g.replay()
            torch.cuda.synchronize()
            results.append((st.res.clone(), st._q8(spec.hidden).view(torch.uint8).clone()))
            st.load(x, attn)
            eager = st.forward().clone()
            torch.cuda.synchronize()
            assert torch.equal(eager, results[-1][0]), f"mode {mode}: eager and graph replay differ"
    finally:
        lib.iflb200_set_dependent_launch(1)
    assert lib.iflb200_set_dependent_launch(3) != 0
    for res, codes in results[1:]:
        assert torch.equal(res, results[0][0]) and torch.equal(codes, results[0][1])
