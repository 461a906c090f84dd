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


@pytest.mark.parametrize("M,hidden,ffn", [(50, 1024, 4096), (816, 512, 2048), (130, 256, 272)])
def test_fused_epilogues_give_the_bits_of_the_three_launch_structure(M, hidden, ffn):
    """The driver's default (gated activation in the gate_up GEMM's epilogue) and the optional fused
    residual epilogue against the reference's structure (gemm, then the consumer kernel): the same
    residual stream, codes and scales, bit for bit, eagerly and from a captured graph."""
    from instinctflash_b200 import _lib
    lib = _lib.lib()
    spec = StackSpec("t", "gemma", 3, M, hidden, ffn, 768, o_in=hidden, outlier_frac=0.02, outlier_scale=10.0, seed=21)
    weights = make_weights(spec, DEV)
    x, attn = make_inputs(spec, DEV)
    assert lib.iflb200_gemm_set_split_k(1) == 0      # same K loop in every arm
    try:
        plain = LinearStack(spec, weights, DEV, fused=False, split_partials=False)
        plain.load(x, attn)
        want = plain.forward().clone()
        want_q, want_s = plain._q8(hidden).view(torch.uint8).clone(), plain.scale[0].clone()
        for fuse_residual in (False, True):
            st = LinearStack(spec, weights, DEV, fused=True, fuse_residual=fuse_residual, split_partials=False)
            assert st.fused and st.fuse_residual == fuse_residual
            st.load(x, attn)
            got = st.forward()
            assert torch.equal(got, want), f"fuse_residual={fuse_residual}"
            assert torch.equal(st._q8(hidden).view(torch.uint8), want_q) and torch.equal(st.scale[0], want_s)
            g = st.capture()
            st.load(x, attn)
            g.replay()
            torch.cuda.synchronize()
            assert torch.equal(st.res, want) and bool((st.amax == 0).all())
    finally:
        lib.iflb200_gemm_set_split_k(0)


@pytest.mark.parametrize("cfg", ["c2", "c3", "c4", "c5"])
def test_benchmark_geometry_with_default_knobs(cfg):
    """Two layers of each benchmark configuration at its full widths and its full row count, every
    tuning knob at its default (so the kernels the heuristics pick for that configuration are the
    ones that run: CTA pairs for M = 16384, cluster split-K for the deep, few-tile down projections).
    Checked against (a) the same stack forced onto the single-CTA unsplit kernel, which the per-
    operator tests pin to the reference's recorded bits: identical where no split-K is chosen,
    within 5e-3 otherwise; (b) the CPU oracle stack on a sample of rows (rows are independent:
    per-token scales, per-row norms), within the distance the oracle's IEEE divisions allow."""
    from instinctflash_b200 import _lib
    from instinctflash_b200.stack import SPECS
    lib = _lib.lib()
    full = SPECS[cfg]
    spec = StackSpec(**{**full.__dict__, "layers": 2, "steps": 1, "name": cfg + "_two_layers"})
    weights = make_weights(spec, DEV)
    x, attn = make_inputs(spec, DEV)
    st = LinearStack(spec, weights, DEV)
    st.load(x, attn)
    got = st.forward().clone()
    torch.cuda.synchronize()
    assert torch.isfinite(got.float()).all()
    try:
        assert lib.iflb200_gemm_set_mode(1) == 0 and lib.iflb200_gemm_set_split_k(1) == 0
        st.load(x, attn)
        plain = st.forward().clone()
        torch.cuda.synchronize()
    finally:
        lib.iflb200_gemm_set_mode(0)
        lib.iflb200_gemm_set_split_k(0)
    if cfg in ("c4", "c5"):       # no split-K at these sizes: same K loop, same bits
        assert torch.equal(got, plain)
    else:
        rel = float((got.float() - plain.float()).norm() / plain.float().norm())
        assert rel < 5e-3, rel
    rows = torch.randperm(spec.M, generator=torch.Generator().manual_seed(7))[:16].sort().values
    sub = StackSpec(**{**spec.__dict__, "M": 16})
    cpu = LinearStack(sub, to_cpu_weights(weights), "cpu", ops=oracle_ops.ops())
    cpu.load(x.cpu()[rows], attn.cpu()[rows])
    want = cpu.forward().float()
    rel = float((got.float().cpu()[rows] - want).norm() / want.norm())
    assert rel < 2e-2, rel
    rec = __import__("ctypes").c_uint32(0)
    assert lib.iflb200_gemm_take_timeout_record(__import__("ctypes").byref(rec), None) == 0 and rec.value == 0


@pytest.mark.parametrize("gated_in_gemm", [True, False])
@pytest.mark.parametrize("M,split", [(50, 1), (7, 1), (100, 1), (50, 8), (64, 3)])
def test_persistent_stack_against_per_operator_stack(M, split, gated_in_gemm):
    from instinctflash_b200 import _lib
    from instinctflash_b200.stack_persistent import PersistentExpertStack
    spec = StackSpec("expert", "gemma", 3, M, 1024, 4096, 1536, steps=2, seed=2)
    weights = make_weights(spec, DEV)
    x, attn = make_inputs(spec, DEV)
    ref = LinearStack(spec, weights, DEV, split_partials=False)
    ref.load(x, attn)
    _lib.lib().iflb200_gemm_set_split_k(1)   # the per-operator arm with the unsplit K loop
    try:
        ref.forward()
    finally:
        _lib.lib().iflb200_gemm_set_split_k(0)
    ps = PersistentExpertStack(spec, weights, DEV, down_split_k=split, gated_in_gemm=gated_in_gemm)
    ps.load(x)
    ps.forward()
    torch.cuda.synchronize()
    assert ps.timeout_record() == 0, f"a wait inside the persistent kernel timed out: {ps.timeout_record():#x}"
    assert bool((ps.amax == 0).all())       # the row maxima of the gated GEMM are consumed and left at zero
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


def test_a_wait_that_nothing_satisfies_runs_out_and_leaves_the_context_usable():
    """Two operators; the second waits on a dependency counter that no operator arrives on.  With
    the wait budget set to a few milliseconds the launch returns, status2[0] names the wait that
    gave up (epilogue role 3, grid dependency 5, operator 1), and the next ordinary launch on the
    same context passes.  Nothing waits without a bound."""
    import numpy as np
    from instinctflash_b200 import _lib
    from instinctflash_b200.stack_persistent import ENCODE, GATED, GEMM, OP_DTYPE, PersistentExpertStack
    lib = _lib.lib()
    spec = StackSpec("expert", "gemma", 1, 50, 1024, 4096, 1536, steps=1, seed=9)
    weights = make_weights(spec, DEV)
    x, _ = make_inputs(spec, DEV)
    ps = PersistentExpertStack(spec, weights, DEV, down_split_k=1)
    ps.load(x)
    ps.forward()
    torch.cuda.synchronize()
    assert ps.timeout_record() == 0
    want = ps.res.clone()
    program = np.frombuffer(ps.d_ops.cpu().numpy().tobytes(), dtype=OP_DTYPE).copy()
    assert program["type"][0] == GEMM and program["type"][2] in (GATED, ENCODE)
    two = program[[0, 2]].copy()
    two["wait_bar"][0], two["arrive_bar"][0] = -1, -1      # the GEMM depends on nothing and signals nothing
    two["wait_bar"][1], two["arrive_bar"][1] = 0, -1       # counter 0: nobody arrives on it
    d_two = torch.from_numpy(two.view(np.uint8).copy()).to(DEV)
    bars = torch.zeros(1, dtype=torch.int32, device=DEV)
    status = torch.zeros(2, dtype=torch.int32, device=DEV)
    try:
        assert lib.iflb200_set_wait_budget_us(4000) == 0
        st = lib.iflb200_stack_run(d_two.data_ptr(), 2, ps.d_maps.data_ptr(), bars.data_ptr(), 1, spec.M,
                                   status.data_ptr(), torch.cuda.current_stream().cuda_stream)
        assert st == 0
        torch.cuda.synchronize()                            # returns: the wait is bounded
    finally:
        assert lib.iflb200_set_wait_budget_us(0) == 0
    code = int(status[0].item()) & 0xFFFFFFFF
    assert code == (3 << 24) | (5 << 16) | 1, hex(code)
    assert int(status[1].item()) == 1                       # the abort word every spinning CTA watches
    # the context is intact: the ordinary program runs and reproduces its earlier result
    ps.load(x)
    ps.forward()
    torch.cuda.synchronize()
    assert ps.timeout_record() == 0
    assert torch.equal(ps.res, want)


def test_episode_batch_branches_equal_separate_runs():
    """Independent episodes in flight as parallel branches of one CUDA graph: every episode's
    residual stream equals the one a lone stack computes from the same input."""
    from instinctflash_b200.stack import EpisodeBatch
    spec = StackSpec("expert", "gemma", 3, 50, 1024, 4096, 1536, steps=2, seed=4)
    weights = make_weights(spec, DEV)
    xs = []
    for e in range(4):
        x, attn = make_inputs(StackSpec(**{**spec.__dict__, "seed": 40 + e}), DEV)
        xs.append(x)
    want = []
    for x in xs:
        st = LinearStack(spec, weights, DEV)
        st.load(x, attn)
        want.append(st.forward().clone())
    batch = EpisodeBatch(spec, weights, DEV, 4)
    batch.load(xs, attn)
    g = batch.capture()
    batch.load(xs, attn)
    g.replay()
    torch.cuda.synchronize()
    for st, w in zip(batch.stacks, want):
        assert torch.equal(st.res, w)
    assert batch.launches_per_forward == 4 * batch.stacks[0].launches_per_forward


def test_results_do_not_depend_on_what_ran_before():
    """The reference's contract check (benchmarks/native/order_check.py:1-53): every record's result
    is bit-identical whatever ran before it.  Three different stacks (different shapes, different
    kernels: cluster split-K, gated epilogue, the persistent kernel, CTA pairs) are run in recorded,
    reversed and interleaved order on the same buffers-per-case; each case must reproduce its own
    bits every time."""
    from instinctflash_b200.kernels import fp8
    from instinctflash_b200.stack_persistent import PersistentExpertStack
    E4M3 = torch.float8_e4m3fn
    cases_ = {}
    a = StackSpec("a", "gemma", 2, 816, 512, 2048, 768, o_in=512, outlier_frac=0.02, outlier_scale=10.0, seed=31)
    b = StackSpec("b", "wan", 2, 300, 1024, 2048, 3072, o_in=1024, cross=True, seed=32)
    c = StackSpec("c", "gemma", 2, 50, 1024, 4096, 1536, steps=2, seed=33)
    for sp in (a, b, c):
        w = make_weights(sp, DEV)
        x, attn = make_inputs(sp, DEV)
        st = LinearStack(sp, w, DEV)
        cases_[sp.name] = (lambda st=st, x=x, attn=attn: (st.load(x, attn), st.forward().clone())[1])
    wc = make_weights(c, DEV)
    xc, _ = make_inputs(c, DEV)
    ps = PersistentExpertStack(c, wc, DEV)
    cases_["persistent"] = lambda: (ps.load(xc), ps.forward().clone())[1]
    g = torch.Generator().manual_seed(5)
    big_a = (torch.randn(4352, 1024, generator=g) * 60).clamp(-448, 448).to(E4M3).to(DEV)
    big_w = fp8.Fp8Weight((torch.randn(1024, 1024, generator=g) * 60).clamp(-448, 448).to(E4M3).to(DEV), torch.ones(1024, device=DEV), None)
    big_out = torch.empty(4352, 1024, device=DEV, dtype=torch.bfloat16)
    cases_["pair_gemm"] = lambda: fp8.gemm(big_a, big_w, big_out).clone()
    names = list(cases_)
    recorded = {n: cases_[n]() for n in names}
    torch.cuda.synchronize()
    orders = [list(reversed(names)), names[::2] + names[1::2], names + names]
    for order in orders:
        for n in order:
            got = cases_[n]()
            torch.cuda.synchronize()
            assert torch.equal(got, recorded[n]), f"{n} changed after {order}"


@pytest.mark.parametrize("M,N,K", [(50, 1024, 4096), (7, 1024, 2048), (128, 2048, 4096), (50, 1024, 1024), (33, 272, 512)])
def test_split_k_partials_feed_the_residual_kernel(M, N, K):
    """Skinny split-K: (tile, K range) pairs on independent CTAs write fp32 partial sums, the residual
    kernel adds the planes in split order and rounds the sum to bf16.  One plane reproduces
    gemm + residual_norm_quant bit for bit; several planes differ only in the summation order of the
    accumulator (GEMM bar) and are deterministic."""
    import cases
    from util import assert_gemm_parity
    from instinctflash_b200.kernels import fp8, norm
    E4M3 = torch.float8_e4m3fn
    x = cases.activations(M, K, 5000 + M, outlier_frac=0.01, outlier_scale=20.0).to(DEV)
    a = torch.empty(M, K, device=DEV, dtype=E4M3)
    s = torch.empty(M, device=DEV)
    norm.row_quant(x, a, s)
    wq, wscale = cases.pack_weight_cpu(cases.weights(N, K, 5100 + N))
    W = fp8.Fp8Weight(wq.to(DEV), wscale.to(DEV), None)
    res0 = cases.activations(M, N, 5200, dtype=torch.float32).to(DEV)
    raw = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    fp8.gemm(a, W, raw)
    want = res0.clone()
    q0 = torch.empty(M, N, device=DEV, dtype=E4M3)
    s0 = torch.empty(M, device=DEV)
    norm.residual_norm_quant(want, delta=raw, delta_row=s, delta_col=W.scale, q=q0, q_scale=s0)
    limit = max(1, min(8, (K // 128 + 3) // 4))
    suggested = fp8.partial_splits(M, N, K)
    assert 1 <= suggested <= limit
    for S in sorted({1, suggested, limit}):
        part = torch.full((S, M, N), float("nan"), device=DEV)
        fp8.gemm_partials(a, W, part)
        assert not torch.isnan(part).any()
        got = res0.clone()
        q1 = torch.empty(M, N, device=DEV, dtype=E4M3)
        s1 = torch.empty(M, device=DEV)
        norm.residual_norm_quant(got, delta=part, delta_row=s, delta_col=W.scale, q=q1, q_scale=s1)
        if S == 1:
            # one plane: the same accumulator bits, so the same residual stream; the norm + quantiser
            # tail sums the squares in this kernel's thread layout, which can differ from the ordinary
            # kernel's for the same width (tolerance class, as for the reference's own layouts)
            assert torch.equal(got, want)
            assert ((s1 - s0).abs() / s0).max().item() < 1e-5
            assert (q1.view(torch.uint8) != q0.view(torch.uint8)).float().mean().item() < 2e-3
        else:
            assert_gemm_parity(got - res0, want - res0, f"{S} planes")
            again = res0.clone()
            part2 = torch.empty_like(part)
            fp8.gemm_partials(a, W, part2)
            norm.residual_norm_quant(again, delta=part2, delta_row=s, delta_col=W.scale, q=q1, q_scale=s1)
            assert torch.equal(part, part2) and torch.equal(again, got)
    with pytest.raises(RuntimeError, match="unsupported shape"):
        fp8.gemm_partials(a, W, torch.empty(limit + 1, M, N, device=DEV))


def test_install_on_the_reference_engine_module_and_run_its_call_sequence_both_ways():
    """The reference's pi05 engine module (unmodified, from baseline/_ref) before and after
    install(): the names its _forward resolves (gemm, row_quant, gated_act_quant,
    residual_norm_quant) drive the layer sequence of instinctflash/engines/pi05/engine.py:199-216
    through the same driver.  After install() they are this package's operators (bit-identical to
    calling the package directly); against the reference's own kernels the residual stream agrees
    to quantisation noise and the first quantiser's codes are the same up to the norm's summation order."""
    import importlib
    import sys
    from pathlib import Path
    from types import SimpleNamespace
    ref = Path(__file__).resolve().parents[1] / "baseline" / "_ref"
    if not (ref / "instinctflash").is_dir():
        pytest.skip("the reference is not installed under baseline/_ref")
    sys.path.insert(0, str(ref))
    try:
        eng = importlib.import_module("instinctflash.engines.pi05.engine")
        fp8_mod = importlib.import_module("instinctflash.kernels.fp8")
    except Exception as exc:   # noqa: BLE001
        pytest.skip(f"the reference's engine module does not import here: {exc}")
    finally:
        sys.path.remove(str(ref))
    from instinctflash_b200 import install as inst

    def resolved():
        g = eng.Pi05Engine._forward.__globals__ if hasattr(eng, "Pi05Engine") else vars(eng)
        return SimpleNamespace(gemm=g["gemm"], row_quant=g["row_quant"], residual_norm_quant=g["residual_norm_quant"],
                               gated_act_quant=g["gated_act_quant"], dequant_rows=vars(importlib.import_module(
                                   "instinctflash.kernels.norm"))["dequant_rows"], GELU_TANH=0, Fp8Weight=fp8_mod.Fp8Weight)

    spec = StackSpec("t", "gemma", 2, 200, 512, 1024, 768, o_in=512, outlier_frac=0.02, outlier_scale=10.0, seed=41)
    weights = make_weights(spec, DEV)
    x, attn = make_inputs(spec, DEV)
    saved = {n: getattr(eng, n) for n in inst.REPLACEMENTS if hasattr(eng, n)}
    before = LinearStack(spec, weights, DEV, ops=resolved())
    before.load(x, attn)
    first_codes = before._q8(spec.hidden).view(torch.uint8).clone()
    ref_res = before.forward().clone()
    try:
        report = inst.install([eng])
        assert {"gemm", "row_quant", "gated_act_quant", "residual_norm_quant"} <= set(report[eng.__name__])
        after = LinearStack(spec, weights, DEV, ops=resolved())
        after.load(x, attn)
        # same norm + quantiser: the row sums of the norm run in another thread layout than Triton's,
        # so a code next to a rounding boundary may move by one step
        differing = (after._q8(spec.hidden).view(torch.uint8) != first_codes).float().mean().item()
        assert differing < 2e-3, differing
        got = after.forward().clone()
    finally:
        for n, fn in saved.items():
            setattr(eng, n, fn)
    native = LinearStack(spec, weights, DEV, fused=False, split_partials=False)
    native.load(x, attn)
    assert torch.equal(native.forward(), got)                       # the installed names ARE this package's operators
    rel = float((got - ref_res).norm() / ref_res.norm())
    assert rel < 2e-2, rel


def test_host_pipeline_returns_each_step_its_own_result():
    """Pinned host inputs through the overlapped serving loop: step i's output is the residual
    stream a lone run computes from step i's input, for more steps than staging buffers."""
    from instinctflash_b200.stack import HostPipeline
    spec = StackSpec("t", "gemma", 2, 200, 512, 1024, 768, o_in=512, outlier_frac=0.02, outlier_scale=10.0, seed=51)
    weights = make_weights(spec, DEV)
    xs, attn = [], None
    for e in range(5):
        x, attn = make_inputs(StackSpec(**{**spec.__dict__, "seed": 60 + e}), DEV)
        xs.append(x)
    st = LinearStack(spec, weights, DEV)
    want = []
    for x in xs:
        st.load(x, attn)
        want.append(st.forward().clone())
    st.load(xs[0], attn)
    graph = st.capture()
    pipe = HostPipeline(st, graph)
    x_hosts = [x.cpu().pin_memory() for x in xs]
    out_hosts = [torch.empty(spec.M, spec.hidden, dtype=st.res.dtype).pin_memory() for _ in xs]
    for xh, oh in zip(x_hosts, out_hosts):
        pipe.submit(xh, oh, attn)
    pipe.drain()
    torch.cuda.synchronize()
    for e, (oh, w) in enumerate(zip(out_hosts, want)):
        assert torch.equal(oh, w.cpu()), e
