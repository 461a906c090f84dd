"""One rank of the tensor-parallel parity check (launched by torch.distributed.run, or spawned
under gloo on CPU by test_stack_cpu.py).  Compares ``tp.WanTPStack`` on ``world`` ranks with the
single-device ``stack.LinearStack`` of the same build on identical seeded weights and inputs."""
from __future__ import annotations

import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parents[1]
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

from instinctflash_b200.stack import LinearStack, StackSpec, make_inputs, make_weights  # noqa: E402
from instinctflash_b200.tp import Comm, WanTPStack  # noqa: E402

TINY = StackSpec("tiny_wan", "wan", layers=2, M=32, hidden=64, ffn=128, qkv=192, o_in=64, cross=True,
                 outlier_frac=0.05, outlier_scale=10.0, seed=7)
SMALL = StackSpec("small_wan", "wan", layers=2, M=256, hidden=1024, ffn=2048, qkv=3072, o_in=1024, cross=True,
                  outlier_frac=0.01, outlier_scale=20.0, seed=8)


def run(spec, device, ops_single, ops_tp, comm, link=None):
    """Returns a dict of checks (all ranks compute it; rank 0 reports)."""
    weights = make_weights(spec, device, cpu_seeded=True)
    x, attn = make_inputs(spec, device)
    single = LinearStack(spec, weights, device, ops=ops_single)
    single.load(x, attn)
    first_codes = single._q8(spec.hidden).clone()
    first_scales = single.scale[0].clone()
    single.forward()
    tp = WanTPStack(spec, weights, device, comm, ops=ops_tp, link=link)
    tp.load(x, attn)
    out = {}
    # replicated input after load: per-row norm + quantiser on row shards, all-gathered
    out["input_codes_equal"] = bool(torch.equal(tp.q8.view(torch.uint8), first_codes.view(torch.uint8)))
    out["input_scales_equal"] = bool(torch.equal(tp.s0, first_scales))
    tp.forward()
    full = tp.gather_residual().float()
    ref = single.res.float()
    out["residual_rel_frobenius"] = float((full - ref).norm() / ref.norm())
    out["residual_row_max_fraction"] = float(((full - ref).abs().amax(1) / ref.abs().amax(1)).max())
    out["full"] = full
    if link is not None:
        if device.type == "cuda":
            torch.cuda.synchronize(device)
        link.check()
    return out


def sharded_quantiser_exact(device, ops_single, ops_tp, comm):
    """A row quantised in column shards around one all-reduce-max equals the unsharded row."""
    g = torch.Generator().manual_seed(99)
    M, K = 40, 512
    raw = (torch.randn(M, K, generator=g) * 300).to(torch.bfloat16).to(device)
    row = (torch.rand(M, generator=g) * 0.02).to(device)
    col = (torch.rand(K, generator=g) * 0.001).to(device)
    bias = (torch.randn(K, generator=g) * 0.1).to(device)
    E4M3 = torch.float8_e4m3fn
    q = torch.empty(M, K, dtype=torch.uint8, device=device).view(E4M3)
    s = torch.empty(M, device=device)
    ops_single.row_quant(raw, q, s, row=row, col=col, bias=bias, gelu=True)
    p, r = comm.size, comm.rank
    w = K // p
    sl = slice(w * r, w * (r + 1))
    xs = raw[:, sl].contiguous()
    ql = torch.empty(M, w, dtype=torch.uint8, device=device).view(E4M3)
    sl_s = torch.empty(M, device=device)
    amax = torch.empty(M, device=device)
    kw = dict(row=row, col=col[sl].contiguous(), bias=bias[sl].contiguous(), gelu=True)
    ops_tp.row_quant_sharded(xs, ql, sl_s, amax, 1, **kw)
    comm.all_reduce_max(amax)
    ops_tp.row_quant_sharded(xs, ql, sl_s, amax, 2, **kw)
    return bool(torch.equal(ql.view(torch.uint8), q[:, sl].contiguous().view(torch.uint8)) and torch.equal(sl_s, s))


def main():
    backend = os.environ.get("IFLB200_TP_BACKEND", "nccl")
    rank = int(os.environ["RANK"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    if backend == "nccl":
        torch.cuda.set_device(local)
        device = torch.device("cuda", local)
        dist.init_process_group("nccl", device_id=device)
        from instinctflash_b200 import stack as S, tp as T
        from instinctflash_b200.kernels import norm
        ops_single, ops_tp = S.native_ops(), T.native_ops()
        ops_single.row_quant = norm.row_quant
        spec = SMALL
    else:
        device = torch.device("cpu")
        dist.init_process_group("gloo")
        import oracle_ops
        ops_single = ops_tp = oracle_ops.ops()
        spec = TINY
    comm = Comm()
    ok_q = sharded_quantiser_exact(device, ops_single, ops_tp, comm)
    res = run(spec, device, ops_single, ops_tp, comm)
    res["sharded_quantiser_exact"] = ok_q
    # the same stack over the peer-memory transport: plane sums in rank order are the
    # reduce-scatter's sums (bit for bit between two ranks, where fp32 addition commutes)
    layout = WanTPStack.peer_layout(spec, comm.size)
    if backend == "nccl":
        from instinctflash_b200.tp import PeerLink
        link = PeerLink(layout, device)
    else:
        from fake_link import GlooLink
        link = GlooLink(layout)
    peer = run(spec, device, ops_single, ops_tp, comm, link=link)
    peer_ok = bool(peer["input_codes_equal"] and peer["input_scales_equal"] and peer["residual_rel_frobenius"] <= 2e-2)
    if comm.size == 2:
        peer_ok = peer_ok and bool(torch.equal(peer["full"], res["full"]))
    ok_q = ok_q and peer_ok
    flags = torch.tensor([float(ok_q), float(res["input_codes_equal"]), float(res["input_scales_equal"]),
                          res["residual_rel_frobenius"], res["residual_row_max_fraction"]], device=device)
    dist.all_reduce(flags, op=dist.ReduceOp.MAX)
    ok_all = torch.tensor([float(ok_q and res["input_codes_equal"] and res["input_scales_equal"])], device=device)
    dist.all_reduce(ok_all, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("TP_RESULT", dict(world=comm.size, exact_ok=bool(ok_all.item()), rel_frobenius=float(flags[3]),
                                row_max_fraction=float(flags[4]), peer_transport_ok=peer_ok,
                                peer_rel_frobenius=peer["residual_rel_frobenius"]), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    # the K-split sums differ from the single-device accumulator only by summation order; two
    # blocks later the residual stream must still be within quantisation-noise distance
    if not ok_all.item() or flags[3].item() > 2e-2:
        sys.exit(1)


if __name__ == "__main__":
    main()
