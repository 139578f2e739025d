"""One rank of the tensor-parallel GPU check (run in-process for one GPU, under torch.distributed.run for several).

Runs arcinferzero_b200.tp.Stack on a small configuration in both summation modes and checks every stage against the
oracle from the stage before it: column-parallel outputs, row-parallel partial outputs, the summed residual stream
(x += sum of partials in rank order, zero/kernels/tp.cl:5-11) and the quantised stream every rank must hold identically."""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(__file__), ".."))
from arcinferzero_b200 import synth as S  # noqa: E402
from arcinferzero_b200 import tp  # noqa: E402
from oracle import oracle as O  # noqa: E402

TOL = 1e-5


def relerr(a, b) -> float:
    return float(np.max(np.abs(a.astype(np.float64) - b.astype(np.float64))) / max(1e-30, np.max(np.abs(b))))


def silu_mul(g, u):
    g = g.astype(np.float32)
    return (u.astype(np.float32) * (g / (np.float32(1) + np.exp(-g, dtype=np.float32)))).astype(np.float32)


def gather(t, world):
    import torch
    import torch.distributed as dist
    if world == 1:
        return [t.cpu().numpy()]
    out = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(out, t.contiguous())
    return [o.cpu().numpy() for o in out]


def check_mode(mode: str, world: int, rank: int, device: int, chunks: int = 1, overlap: bool = False, balance: bool = False) -> None:
    import torch
    n = max(2, world)  # every rank gets at least one 256-wide unit of each split dimension
    # (with balance the Q rows do not divide evenly: the extra units must land on the last ranks and still add up)
    cfg = tp.StackConfig(layers=2, tokens=256, hidden=512, q_rows=256 * n + (256 if balance else 0), kv_rows=128 * n,
                         ffn=256 * max(4, world), seed=4242)
    QT, E, T = cfg.qtype, cfg.hidden, cfg.tokens
    st = tp.Stack(cfg, world, rank, device, mode=mode, chunks=chunks, overlap=overlap, balance=balance, comm_sms=8)
    x_in = (S.make_act(T, E, cfg.seed) * np.float32(0.1)).astype(np.float32)
    st.set_input(torch.from_numpy(x_in).cuda(device))
    trace = []
    st.forward(trace)
    torch.cuda.synchronize()
    plan = st.plan
    mine = st.owned_rows()
    nq = plan.q[1] - plan.q[0]
    for li, t in enumerate(trace):
        sh = tp.shard_rows(cfg, tp.layer_weights(cfg, li), plan)
        n = {k: v.cpu().numpy() for k, v in t.items()}
        # column-parallel QKV from the quantised stream all ranks share
        ref = O.matmul(QT, sh["qkv"][0], E, n["xq0"], n["xsc0"], T)
        assert relerr(n["qkv"], ref) <= TOL, (mode, li, "qkv", relerr(n["qkv"], ref))
        # row-parallel O from this rank's Q columns
        hq, hsc, _ = O.quantize_act(np.ascontiguousarray(n["qkv"][:, :nq]))
        rows, _, K, cr = sh["o"]
        ref = O.matmul(QT, tp.slice_cols(QT, rows, K, *cr), nq, hq, hsc, T)
        assert relerr(n["o_part"], ref) <= TOL, (mode, li, "o_part")
        # the sum over ranks, added to the residual stream
        parts = np.stack(gather(t["o_part"], world))
        x1_ref = O.tp_add(n["x0"], parts)
        assert relerr(n["x1"][mine], x1_ref[mine]) <= TOL, (mode, li, "x1", relerr(n["x1"][mine], x1_ref[mine]))
        # every rank holds the same quantised stream, and it is the quantiser applied to the summed rows
        for key in ("xq1", "xsc1"):
            g = gather(t[key], world)
            assert all(np.array_equal(g[0], gi) for gi in g[1:]), (mode, li, key, "differs between ranks")
        aq, asc, _ = O.quantize_act(np.ascontiguousarray(n["x1"][mine]))
        assert np.array_equal(n["xq1"][mine], aq), (mode, li, "xq1")
        assert np.array_equal(n["xsc1"][:, mine], asc), (mode, li, "xsc1")
        # FFN: gate / up (SwiGLU store mode) and down
        rows_g, _, K, _ = sh["gate"]
        h_ref = silu_mul(O.matmul(QT, rows_g, K, n["xq1"], n["xsc1"], T), O.matmul(QT, sh["up"][0], K, n["xq1"], n["xsc1"], T))
        assert relerr(n["h"], h_ref) <= TOL, (mode, li, "h", relerr(n["h"], h_ref))
        hq, hsc, _ = O.quantize_act(n["h"])
        rows, _, K, cr = sh["down"]
        ref = O.matmul(QT, tp.slice_cols(QT, rows, K, *cr), cr[1] - cr[0], hq, hsc, T)
        assert relerr(n["down_part"], ref) <= TOL, (mode, li, "down_part")
        parts = np.stack(gather(t["down_part"], world))
        x2_ref = O.tp_add(n["x1"], parts)
        assert relerr(n["x2"][mine], x2_ref[mine]) <= TOL, (mode, li, "x2")
        for key in ("xq2", "xsc2"):
            g = gather(t[key], world)
            assert all(np.array_equal(g[0], gi) for gi in g[1:]), (mode, li, key, "differs between ranks")
    # the same input once more without a trace (the pipelined order of the sums, no waits between the halves): same stream
    st.set_input(torch.from_numpy(x_in).cuda(device))
    st.forward()
    torch.cuda.synchronize()
    last = trace[-1]
    assert torch.equal(st.xq, last["xq2"]) and torch.equal(st.xsc, last["xsc2"]), (mode, "untraced pass differs (xq)")
    sel = torch.from_numpy(mine).to(st.x.device)
    assert torch.equal(st.x[sel], last["x2"][sel]), (mode, "untraced pass differs (x)")
    st.close()


def check_head_gather(world: int, rank: int, device: int) -> None:
    """The output head split by vocabulary rows (units of 16, the last rank also takes the remainder): every rank runs the
    few-row GEMV on its rows, izb_tp_gather_logits joins them in rank order; the result against the oracle on the whole head."""
    import torch
    import arcinferzero_b200 as izb
    K, T = 512, 2
    vocab = 16 * (3 * world + 1) + 5
    w = S.make_weight(8, vocab, K, 99)
    b, e = tp.tp_range(vocab, 16, world, rank)
    if rank == world - 1:
        e = vocab
    W = izb.Weight(8, w, vocab, K, device=device, row_range=(b, e))
    x = S.make_act(T, K, 98)
    aq, asc, _ = O.quantize_act(x, Mp=16)
    comm = izb.TpComm(world, rank, device)
    local = izb.gemv(W, torch.from_numpy(aq).cuda(device), torch.from_numpy(asc).cuda(device), T)
    full = torch.full((T, vocab + 3), float("nan"), dtype=torch.float32, device=f"cuda:{device}")
    comm.gather_logits(local, vocab, full=full)
    torch.cuda.synchronize()
    got = full.cpu().numpy()
    assert np.isnan(got[:, vocab:]).all()
    assert relerr(got[:, :vocab], O.matmul(8, w, K, aq, asc, T, "gemv")) <= TOL
    comm.close()
    W.close()


def main() -> int:
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    try:
        for mode in ("allreduce", "rs_quant_ag"):
            check_mode(mode, world, rank, local)
            print(f"TP_WORKER_OK mode={mode} rank={rank}/{world}", flush=True)
        # the pipelined form: two token chunks, sums on a second stream beside the next chunk's GEMMs, balanced Q split
        check_mode("rs_quant_ag", world, rank, local, chunks=2, overlap=True, balance=True)
        print(f"TP_WORKER_OK mode=rs_quant_ag/overlap rank={rank}/{world}", flush=True)
        if world == 2:
            # the sums moved by the copy engines (izb_p2p_push / izb_p2p_wait) instead of NCCL: same owners, same arithmetic
            check_mode("p2p", world, rank, local, chunks=2, balance=True)
        print(f"TP_WORKER_OK mode=p2p rank={rank}/{world}" + ("" if world == 2 else " (two-rank runs only)"), flush=True)
        check_head_gather(world, rank, local)
        print(f"TP_WORKER_OK head gather rank={rank}/{world}", flush=True)
    finally:
        if world > 1:
            dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
