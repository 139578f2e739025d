"""Tensor-parallel host logic on CPU: two `gloo` ranks run the split of zero/mgpu/engine_tp_shard.h (tp_range :68-72, T()
:243-279, tp_slice :202-234) with the oracle standing in for the device kernels, and sum the row-parallel partial outputs
like tp_out / tp_add (zero/mgpu/engine_tp_shard.h:318-325, zero/kernels/tp.cl:5-11).  No GPU, no CUDA library."""
import datetime
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

sys.path.insert(0, os.path.join(os.path.dirname(__file__), ".."))
from arcinferzero_b200 import synth as S  # noqa: E402
from arcinferzero_b200 import tp  # noqa: E402
from oracle import oracle as O  # noqa: E402

CFG = tp.StackConfig(layers=1, tokens=32, hidden=512, q_rows=512, kv_rows=256, ffn=1024, seed=77)
TOL = 1e-5


def free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def relerr(a, b) -> float:
    return float(np.max(np.abs(a.astype(np.float64) - b.astype(np.float64))) / max(1e-30, np.max(np.abs(b))))


def silu_mul(g, u):
    """SwiGLU store mode of the GEMM (zero/kernels/gemm.cl:562-565): h = up * (gate / (1 + exp(-gate))) in f32."""
    g = g.astype(np.float32)
    return (u.astype(np.float32) * (g / (np.float32(1) + np.exp(-g, dtype=np.float32)))).astype(np.float32)


def allreduce(a: np.ndarray) -> np.ndarray:
    t = torch.from_numpy(a.copy())
    dist.all_reduce(t)
    return t.numpy()


def worker_parity(rank: int, world: int, port: int, q):
    try:
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=60))
        cfg, QT = CFG, CFG.qtype
        E, T = cfg.hidden, cfg.tokens
        w = tp.layer_weights(cfg, 0)
        plan = tp.shard_plan(cfg, world, rank)
        sh = tp.shard_rows(cfg, w, plan)
        x = (S.make_act(T, E, cfg.seed) * np.float32(0.1)).astype(np.float32)

        # ---- the plans of all ranks tile every dimension exactly once
        plans = [None] * world
        dist.all_gather_object(plans, (plan.q, plan.kv, plan.ffn))
        for dim, total in ((0, cfg.q_rows), (1, cfg.kv_rows), (2, cfg.ffn)):
            edges = [p[dim] for p in plans]
            assert edges[0][0] == 0 and edges[-1][1] == total
            assert all(edges[i][1] == edges[i + 1][0] for i in range(world - 1))

        # ---- QKV, column parallel: this rank's columns are bit-identical to the unsplit product's
        aq, asc, _ = O.quantize_act(x)
        qkv_full = O.matmul(QT, w["qkv"], E, aq, asc, T)
        rows, N, K, _ = sh["qkv"]
        qkv = O.matmul(QT, rows, K, aq, asc, T)
        q0, q1 = plan.q
        k0, k1 = plan.kv
        assert np.array_equal(qkv[:, :q1 - q0], qkv_full[:, q0:q1])
        assert np.array_equal(qkv[:, q1 - q0:q1 - q0 + k1 - k0], qkv_full[:, cfg.q_rows + k0:cfg.q_rows + k1])
        assert np.array_equal(qkv[:, q1 - q0 + k1 - k0:], qkv_full[:, cfg.q_rows + cfg.kv_rows + k0:cfg.q_rows + cfg.kv_rows + k1])

        # ---- O, row parallel: the sum of the partial outputs equals the unsplit product (f32 order only)
        hq, hsc, _ = O.quantize_act(np.ascontiguousarray(qkv[:, :q1 - q0]))
        hq_full, hsc_full, _ = O.quantize_act(np.ascontiguousarray(qkv_full[:, :cfg.q_rows]))
        assert np.array_equal(hq, hq_full[:, q0:q1]) and np.array_equal(hsc, hsc_full[q0 // 32:q1 // 32])
        rows, N, K, cr = sh["o"]
        part = O.matmul(QT, tp.slice_cols(QT, rows, K, *cr), cr[1] - cr[0], hq, hsc, T)
        o_sum = allreduce(part)
        o_full = O.matmul(QT, w["o"], cfg.q_rows, hq_full, hsc_full, T)
        assert relerr(o_sum, o_full) <= TOL
        # tp_add in rank order (the reference's order) against the collective's order
        parts = [None] * world
        dist.all_gather_object(parts, part)
        x_ref = O.tp_add(x, np.stack(parts))
        x1 = x + o_sum
        assert relerr(x1, x_ref) <= TOL

        # ---- FFN with the summed stream as the common input (teacher forcing: both sides start from x1)
        aq, asc, _ = O.quantize_act(x1)
        rows_g, Nf, K, _ = sh["gate"]
        rows_u = sh["up"][0]
        h = silu_mul(O.matmul(QT, rows_g, K, aq, asc, T), O.matmul(QT, rows_u, K, aq, asc, T))
        h_full = silu_mul(O.matmul(QT, w["gate"], E, aq, asc, T), O.matmul(QT, w["up"], E, aq, asc, T))
        f0, f1 = plan.ffn
        assert np.array_equal(h, h_full[:, f0:f1])
        hq, hsc, _ = O.quantize_act(h)
        hq_full, hsc_full, _ = O.quantize_act(h_full)
        rows, N, K, cr = sh["down"]
        part = O.matmul(QT, tp.slice_cols(QT, rows, K, *cr), cr[1] - cr[0], hq, hsc, T)
        d_sum = allreduce(part)
        d_full = O.matmul(QT, w["down"], cfg.ffn, hq_full, hsc_full, T)
        assert relerr(d_sum, d_full) <= TOL

        # ---- reduce-scatter by token rows -> quantise own rows -> all-gather: identical int8 rows on every rank, equal to
        #      the quantiser applied to the whole summed stream
        x2 = x1 + d_sum
        own = T // world
        mine = np.ascontiguousarray(x2[rank * own:(rank + 1) * own])
        mq, msc, _ = O.quantize_act(mine)
        gathered = [None] * world
        dist.all_gather_object(gathered, (mq, msc))
        gq = np.concatenate([g[0] for g in gathered])
        gsc = np.concatenate([g[1] for g in gathered], axis=1)
        fq, fsc, _ = O.quantize_act(x2)
        assert np.array_equal(gq, fq) and np.array_equal(gsc, fsc)
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        q.put((rank, f"{type(e).__name__}: {e}"))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def worker_failure(rank: int, world: int, port: int, q):
    """Rank 1 leaves between steps 1 and 2 (no collective in flight); rank 0 learns of it on the host before its next
    launch.  A second guard shows the timeout when a rank never announces anything."""
    try:
        store = dist.TCPStore("127.0.0.1", port, world, rank == 0, timeout=datetime.timedelta(seconds=30))
        dist.init_process_group("gloo", store=store, rank=rank, world_size=world, timeout=datetime.timedelta(seconds=30))
        guard = tp.StepGuard(store, world, rank, timeout_s=3.0)
        done = []
        for k in range(3):
            if rank == 1 and k == 2:
                guard.leave("injected exit between steps")
                break
            guard.enter(k)
            t = torch.ones(4)
            dist.all_reduce(t)
            assert float(t[0]) == world
            done.append(k)
        q.put((rank, f"steps {done}"))
    except tp.PeerGone as e:
        q.put((rank, f"PeerGone after {done}: {e}"))
    except Exception as e:  # noqa: BLE001
        q.put((rank, f"{type(e).__name__}: {e}"))
    finally:
        # rank 0 hosts the store: keep it alive until rank 1 has reported
        if rank == 0:
            import time
            time.sleep(0.5)
        if dist.is_initialized():
            dist.destroy_process_group()


def run_ranks(fn, world: int = 2):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=fn, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=240) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
    return res


@pytest.fixture(scope="module", autouse=True)
def _oracle_built():
    O.lib()


def test_tp_range_matches_oracle():
    for total, unit in ((17408, 256), (5120, 256), (1024, 128), (151936, 1)):
        for n in (1, 2, 3, 4, 8):
            got = [tp.tp_range(total, unit, n, r) for r in range(n)]
            assert got == [tuple(O.tp_range(total, unit, n, r)) for r in range(n)]
            assert got[0][0] == 0 and got[-1][1] == total // unit * unit


def test_config5_plan_is_aligned_for_all_world_sizes():
    cfg = tp.StackConfig()
    for n in (1, 2, 4, 8):
        for r in range(n):
            p = tp.shard_plan(cfg, n, r)
            assert (p.q[1] - p.q[0]) % 256 == 0 and p.q[0] % 256 == 0      # K range of O: whole superblocks
            assert (p.ffn[1] - p.ffn[0]) % 256 == 0 and p.ffn[0] % 256 == 0
            assert p.qkv_rows % 128 == 0
    assert [tp.shard_plan(cfg, 8, r).ffn[1] - tp.shard_plan(cfg, 8, r).ffn[0] for r in range(8)] == [2304] * 4 + [2048] * 4


def test_balanced_plan_moves_the_extra_q_units_to_the_last_ranks():
    cfg = tp.StackConfig()
    for total, unit in ((5120, 256), (17408, 256), (1024, 128)):
        for n in (1, 2, 3, 4, 8):
            got = [tp.tp_range_tail(total, unit, n, r) for r in range(n)]
            assert got[0][0] == 0 and got[-1][1] == total // unit * unit
            assert all(got[i][1] == got[i + 1][0] for i in range(n - 1))
            sizes = [e - b for b, e in got]
            assert sorted(sizes) == sizes and max(sizes) - min(sizes) <= unit  # the larger shards come last
            assert sorted(sizes) == sorted(e - b for b, e in (tp.tp_range(total, unit, n, r) for r in range(n)))
    # config 5 at 8 ranks, work in units of 256 rows (2 per Q unit for QKV + O, 3 per FFN unit): 33 : 28 becomes 31 : 30
    def work(p):
        return 2 * (p.q[1] - p.q[0]) // 256 + 3 * (p.ffn[1] - p.ffn[0]) // 256
    plain = [work(tp.shard_plan(cfg, 8, r)) for r in range(8)]
    even = [work(tp.shard_plan(cfg, 8, r, balance=True)) for r in range(8)]
    assert (max(plain), min(plain)) == (33, 28) and (max(even), min(even)) == (31, 30) and sum(plain) == sum(even)


def test_slice_cols_rejects_partial_superblocks():
    w = S.make_weight(S.GGML_Q4_K, 4, 512, 1)
    assert tp.slice_cols(S.GGML_Q4_K, w, 512, 256, 512).shape == (4, 144)
    with pytest.raises(ValueError):
        tp.slice_cols(S.GGML_Q4_K, w, 512, 128, 512)


def test_split_stack_two_ranks_gloo():
    res = run_ranks(worker_parity)
    assert res == {0: "ok", 1: "ok"}, res


def test_peer_leaving_between_steps_is_seen_on_the_host():
    res = run_ranks(worker_failure)
    assert res[1] == "steps [0, 1]", res
    assert res[0].startswith("PeerGone after [0, 1]"), res


@pytest.mark.parametrize("chunks,lag", [(2, 1), (4, 1), (8, 1), (4, 2), (3, 0), (1, 1)])
def test_sum_pipeline_order(chunks, lag):
    """The order in which the copy-engine mode queues the owners' reduces (tp.SumPipeline, pure bookkeeping): every sum of
    every chunk is reduced exactly once, after its partials were sent and before its gathered rows are awaited; at most
    `lag` reduces are held back; and the sequence is the same on every rank, with every await depending only on
    operations earlier in it (what rules out a deadlock between ranks)."""
    p = tp.SumPipeline(chunks, lag)
    log = []
    seq = 0
    for half in range(7):
        seq += 1
        for c in range(chunks):
            reduces, s = p.needed(c)
            log += [("reduce", rc, rs) for rc, rs in reduces]
            log.append(("await", c, s))
            log.append(("send", c, seq))
            log += [("reduce", rc, rs) for rc, rs in p.sent(c, seq)]
            assert len(p.pending) <= lag
    for c in range(chunks):
        reduces, s = p.needed(c)
        log += [("reduce", rc, rs) for rc, rs in reduces]
        log.append(("await", c, s))
    assert not p.pending and not any(p.waiting)
    pos = {e: i for i, e in enumerate(log)}
    assert len(pos) == len([e for e in log if e[2] != 0]) + len({e for e in log if e[2] == 0})  # nothing queued twice
    for s in range(1, seq + 1):
        for c in range(chunks):
            assert pos[("send", c, s)] < pos[("reduce", c, s)] < pos[("await", c, s)], (c, s)
    # reduces leave in the order their partials were sent
    sends = [e[1:] for e in log if e[0] == "send"]
    reds = [e[1:] for e in log if e[0] == "reduce"]
    assert reds == sends
    # with a lag, a chunk's reduce is queued only after `lag` later sends (the copies run beside those chunks' GEMMs)
    if lag and chunks > lag:
        tail = set(sends[-lag:])   # (the last sends of the run: flushed at the end, nothing follows them)
        for s in range(1, seq + 1):
            for c in range(chunks):
                if (c, s) in tail:
                    continue
                between = [e for e in log[pos[("send", c, s)] + 1:pos[("reduce", c, s)]] if e[0] == "send"]
                assert len(between) >= min(lag, 1), (c, s, between)
