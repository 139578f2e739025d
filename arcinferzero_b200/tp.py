"""Tensor-parallel projection stack: the split the reference's multi-GPU mode performs (zero/mgpu/engine_tp_shard.h)
applied to a stack of dense layers, one process per GPU.

Per layer (BASELINE.json config 5; no attention, no norms: only the quantised projections and what lies between them):

    x [T, E] f32 --quantise--> QKV (column parallel: this rank's rows of the Q, K and V blocks)
      q = the rank's Q columns --quantise--> O (row parallel: the matching K range) --sum over ranks--> x += .
    x --quantise--> gate, up (column parallel; up stored with the fused SwiGLU mode: h = up * silu(gate))
      h --quantise--> down (row parallel) --sum over ranks--> x += .

Ranges follow tp_range (zero/mgpu/engine_tp_shard.h:68-72): whole units, the first `units % N` ranks one unit more.
FFN rows split in units of 256 (:128-144).  The Q rows also split in units of 256 here (= two 128-wide heads) rather than
by kv-head group: with 8 ranks a head-group split leaves the O projection 640 input columns per rank, which is not a
whole number of 256-element superblocks (the reference refuses such a split, :128, :216); K and V rows split evenly.

Two ways to sum the row-parallel partial outputs:
  "allreduce"  f32 all-reduce of the partials, added to the residual stream (tp_out / tp_reduce_at, tp_add);
  "rs_quant_ag"  reduce-scatter by token rows, add the residual rows, quantise them, all-gather int8 + scales:
               every element is summed on one rank only (all ranks end up with identical int8 rows) and fewer bytes
               cross NVLink; the next projection consumes the gathered int8 rows directly.
  "p2p"        the same arithmetic and the same owners as "rs_quant_ag", moved by the copy engines instead of NCCL
               (izb_p2p_push / izb_p2p_wait): every rank copies its partial rows into the owner's receive buffer and
               raises a flag there, the owner adds the parts in rank order (izb_tp_add), quantises and copies its rows
               into every rank's buffers.  No multiprocessor is taken by the transport, so the GEMMs keep all of them;
               the owner's small kernels run between the GEMMs of later chunks (the reduce of chunk c is queued one
               GEMM slot after its partials left, its result is needed a whole half layer later).  The buffers other
               ranks write into come from torch's symmetric-memory allocator (peer mappings are host plumbing).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import synth as S


@dataclass
class StackConfig:
    layers: int = 8
    tokens: int = 32768
    hidden: int = 5120
    q_rows: int = 5120      # 40 heads x 128
    kv_rows: int = 1024     # 8 kv heads x 128 (each of K and V)
    ffn: int = 17408
    qtype: int = S.GGML_Q4_K
    seed: int = 20261125

    @property
    def ops_per_pass(self) -> float:
        """2*M*N*K integer operations of one pass over all layers (all ranks together)."""
        per_tok = self.hidden * (self.q_rows + 2 * self.kv_rows) + self.q_rows * self.hidden + 2 * self.hidden * self.ffn + self.ffn * self.hidden
        return 2.0 * self.tokens * self.layers * per_tok


def tp_range(total: int, unit: int, n: int, r: int) -> tuple[int, int]:
    """zero/mgpu/engine_tp_shard.h:68-72 (host copy of izb_tp_range, usable without the CUDA library)."""
    units = total // unit
    base, extra = divmod(units, n)
    b = r * base + min(r, extra)
    e = b + base + (1 if r < extra else 0)
    return b * unit, e * unit


@dataclass
class ShardPlan:
    q: tuple[int, int]      # this rank's Q rows of the QKV matrix = its K range of O
    kv: tuple[int, int]     # its rows inside the K block (and inside the V block)
    ffn: tuple[int, int]    # its gate / up rows = its K range of down

    @property
    def qkv_rows(self) -> int:
        return (self.q[1] - self.q[0]) + 2 * (self.kv[1] - self.kv[0])


def tp_range_tail(total: int, unit: int, n: int, r: int) -> tuple[int, int]:
    """The same split with the extra units on the LAST `units % n` ranks instead of the first."""
    units = total // unit
    base, extra = divmod(units, n)
    b = r * base + max(0, r - (n - extra))
    e = b + base + (1 if r >= n - extra else 0)
    return b * unit, e * unit


def shard_plan(cfg: StackConfig, world: int, rank: int, balance: bool = False) -> ShardPlan:
    """tp_range for every split dimension.  balance=True puts the extra Q units on the last ranks: tp_range gives the
    first ranks the extra unit of EVERY dimension (at 8 ranks: 3 Q units + 9 FFN units against 2 + 8), so the same ranks
    are the slowest in both halves of a layer; moving the Q extras to the ranks with fewer FFN rows costs nothing and
    evens the work (33 : 28 units of 256 rows becomes 31 : 30)."""
    q = tp_range_tail(cfg.q_rows, 256, world, rank) if balance else tp_range(cfg.q_rows, 256, world, rank)
    return ShardPlan(q=q, kv=tp_range(cfg.kv_rows, 128, world, rank), ffn=tp_range(cfg.ffn, 256, world, rank))


def condition_weight(qtype: int, rows: np.ndarray, K: int) -> np.ndarray:
    """Rescale the fp16 super-scales of generated rows in place so that a stack without normalisation layers stays finite:
    zero-mean weights with a root-mean-square of 1/sqrt(K) (each projection then keeps the magnitude of its input).
    The generator's Q4_K weights d*sc*q - dmin*mn have mean ~1 and rms ~1.8; dmin is raised by 7.5 (= mean q) to centre
    them, then both scales shrink by 1/(1.77*sqrt(K)).  Bit layout and integer fields are untouched."""
    n = rows.shape[0]
    f = np.float32(1.0 / (1.77 * np.sqrt(K)))
    if qtype == S.GGML_Q4_K:
        v = rows.reshape(n, K // 256, 144)
        dd = np.ascontiguousarray(v[:, :, :4]).view(np.float16).astype(np.float32)
        dd[:, :, 0] *= f
        dd[:, :, 1] *= np.float32(7.5) * f
        v[:, :, :4] = dd.astype(np.float16).view(np.uint8).reshape(n, K // 256, 4)
    else:
        v = rows.reshape(n, K // 32, 34)
        d = np.ascontiguousarray(v[:, :, :2]).view(np.float16).astype(np.float32) * (f * np.float32(1.77 / 0.85))
        v[:, :, :2] = d.astype(np.float16).view(np.uint8).reshape(n, K // 32, 2)
    return rows


def layer_weights(cfg: StackConfig, layer: int) -> dict[str, np.ndarray]:
    """Full (unsplit) GGUF rows of one layer, seeded per tensor."""
    s = cfg.seed + 100 * layer
    E, qt = cfg.hidden, cfg.qtype
    return {
        "qkv": condition_weight(qt, S.make_weight(qt, cfg.q_rows + 2 * cfg.kv_rows, E, s + 1), E),
        "o": condition_weight(qt, S.make_weight(qt, E, cfg.q_rows, s + 2), cfg.q_rows),
        "gate": condition_weight(qt, S.make_weight(qt, cfg.ffn, E, s + 3), E),
        "up": condition_weight(qt, S.make_weight(qt, cfg.ffn, E, s + 4), E),
        "down": condition_weight(qt, S.make_weight(qt, E, cfg.ffn, s + 5), cfg.ffn),
    }


def shard_rows(cfg: StackConfig, w: dict[str, np.ndarray], plan: ShardPlan) -> dict[str, tuple[np.ndarray, int, int, tuple | None]]:
    """This rank's part of every tensor as (rows_bytes, N, K, col_range): QKV rows are gathered from the three blocks on
    the host (Engine::T(), zero/mgpu/engine_tp_shard.h:243-279); the K ranges of O / down are cut by the library."""
    E = cfg.hidden
    q0, q1 = plan.q
    k0, k1 = plan.kv
    qkv = np.concatenate([w["qkv"][q0:q1], w["qkv"][cfg.q_rows + k0:cfg.q_rows + k1],
                          w["qkv"][cfg.q_rows + cfg.kv_rows + k0:cfg.q_rows + cfg.kv_rows + k1]])
    f0, f1 = plan.ffn
    return {
        "qkv": (qkv, qkv.shape[0], E, None),
        "o": (w["o"], E, cfg.q_rows, (q0, q1)),
        "gate": (np.ascontiguousarray(w["gate"][f0:f1]), f1 - f0, E, None),
        "up": (np.ascontiguousarray(w["up"][f0:f1]), f1 - f0, E, None),
        "down": (w["down"], E, cfg.ffn, (f0, f1)),
    }


def slice_cols(qtype: int, rows: np.ndarray, K: int, k0: int, k1: int) -> np.ndarray:
    """Columns [k0, k1) of GGUF rows, cut at 256-element superblocks (tp_slice, zero/mgpu/engine_tp_shard.h:202-234)."""
    if k0 % 256 or k1 % 256 or not 0 <= k0 < k1 <= K:
        raise ValueError(f"column range [{k0}, {k1}) of {K} must be whole 256-element superblocks")
    sb = S.sb_bytes(qtype)
    n = rows.shape[0]
    return np.ascontiguousarray(rows.reshape(n, K // 256, sb)[:, k0 // 256:k1 // 256]).reshape(n, -1)


class PeerGone(RuntimeError):
    """Another rank announced that it left (or never confirmed a step) before this rank's next launch."""


class StepGuard:
    """Host-side liveness check between steps (the reference's barrier timeout, zero/mgpu/engine_tp.h:57-60,960-977, moved
    in front of the launch: no kernel or collective is started once a peer is known to be gone).

    Each rank adds 1 to the counter `step/<k>` of a torch.distributed store when it is about to start step k and sets the
    key `gone` when it leaves between steps.  `enter(k)` returns when all ranks have arrived, raises PeerGone when `gone`
    is set or when the others do not arrive within `timeout_s`."""

    def __init__(self, store, world: int, rank: int, timeout_s: float = 5.0):
        self.store, self.world, self.rank, self.timeout_s = store, world, rank, timeout_s

    def leave(self, why: str = "left") -> None:
        self.store.set("gone", f"rank {self.rank}: {why}")

    def enter(self, k: int) -> None:
        import time
        self.store.add(f"step/{k}", 1)
        t_end = time.monotonic() + self.timeout_s
        while True:
            if self.store.check(["gone"]):
                raise PeerGone(self.store.get("gone").decode())
            if self.store.add(f"step/{k}", 0) >= self.world:
                return
            if time.monotonic() > t_end:
                raise PeerGone(f"rank {self.rank}: peers did not reach step {k} within {self.timeout_s} s")
            time.sleep(0.01)


class SumPipeline:
    """Order of the owner's work in the "p2p" mode, as pure bookkeeping (no device): which reduce is queued when.

    A chunk's partial rows leave right after its GEMMs (`sent`); the owner's reduce of that chunk is queued `lag` GEMM
    slots later, so that the copies run beside the GEMMs of the chunks in between; a chunk's gathered rows are awaited
    just before its next GEMMs (`needed`), by which time its reduce must have been queued.  Every rank runs the same
    sequence, and every wait in it depends only on operations that come earlier in it: no rank can wait for something
    another rank has not been asked to do yet."""

    def __init__(self, chunks: int, lag: int = 1):
        assert chunks >= 1 and lag >= 0
        self.chunks, self.lag = chunks, lag
        self.pending: list[tuple[int, int]] = []   # (chunk, seq): partials sent, reduce not queued yet
        self.waiting = [0] * chunks                # seq of the sum whose gathered rows chunk c has not awaited yet (0: none)

    def sent(self, c: int, seq: int) -> list[tuple[int, int]]:
        """The partials of (c, seq) have been handed to the transport.  Returns the reduces to queue now, oldest first."""
        assert self.waiting[c] == 0, "a chunk hands in a new sum only after it has awaited the one before"
        self.pending.append((c, seq))
        self.waiting[c] = seq
        out = []
        while len(self.pending) > self.lag:
            out.append(self.pending.pop(0))
        return out

    def needed(self, c: int) -> tuple[list[tuple[int, int]], int]:
        """Chunk c is about to be read.  Returns (reduces to queue first, seq to await or 0)."""
        out = []
        if any(pc == c for pc, _ in self.pending):   # (its own reduce is still held back: everything up to it goes now)
            while self.pending:
                out.append(self.pending.pop(0))
                if out[-1][0] == c:
                    break
        seq, self.waiting[c] = self.waiting[c], 0
        return out, seq


class Stack:
    """The rank-local stack on one GPU (needs the CUDA library and torch.distributed when world > 1).

    distinct_layers=False uploads one generated layer `cfg.layers` times (separate device copies, same bytes): the
    benchmark's way to keep host-side generation short; timing and traffic are those of distinct layers.

    chunks > 1 splits the token rows into equal chunks that run through a layer one after the other; with overlap=True
    the sum of a chunk's row-parallel partials runs on a second stream while the next chunk's GEMMs run on the first
    (the reference hides its FFN sums behind the next chunk's GEMMs the same way: TpOverlap, zero/mgpu/engine_tp.h:126-151,
    tpo_out :629).  The persistent GEMM then leaves `comm_sms` multiprocessors free (izb_set_sm_limit) and the collectives
    are capped at as many CTAs, so that both are resident at once.  Every chunk owns its buffers; in "rs_quant_ag" mode a
    rank owns the rows [rank * own, (rank + 1) * own) of EACH chunk (own = chunk rows / world).

    fused_ffn=True loads the gate and up shards as one interleaved weight (izb_weight_create_gateup) and runs them as one
    GEMM whose epilogue stores up * silu(gate); False keeps the reference's two launches (gate, then up with store mode 2)."""

    def __init__(self, cfg: StackConfig, world: int, rank: int, device: int, mode: str = "allreduce", distinct_layers: bool = True,
                 chunks: int = 1, overlap: bool = False, balance: bool = False, comm_sms: int = 8, timeout_ms: int = 0,
                 fused_ffn: bool = True):
        import torch

        import arcinferzero_b200 as izb
        self.izb, self.torch = izb, torch
        self.cfg, self.world, self.rank, self.device, self.mode = cfg, world, rank, device, mode
        assert mode in ("allreduce", "rs_quant_ag", "p2p")
        if mode == "p2p" and world == 1:
            mode = self.mode = "rs_quant_ag"  # (one rank: nothing to move)
        if mode == "p2p":
            assert chunks >= 2, "the p2p pipeline hides a chunk's sum behind the next chunk's GEMMs: chunks >= 2"
            overlap = False  # (no second compute stream, no SM limit: the transport runs on the copy engines)
        T, E = cfg.tokens, cfg.hidden
        assert T % chunks == 0 and (T // chunks) % (16 * world) == 0, "chunk rows must be a multiple of 16 * world"
        self.chunks, self.Tc = chunks, T // chunks
        self.overlap = bool(overlap and world > 1)
        self.plan = shard_plan(cfg, world, rank, balance)
        self.layers = []
        sh = None
        for li in range(cfg.layers):
            if sh is None or distinct_layers:
                sh = shard_rows(cfg, layer_weights(cfg, li), self.plan)
            L = {k: izb.Weight(cfg.qtype, rows, N, K, device=device, col_range=cr) for k, (rows, N, K, cr) in sh.items()
                 if not (fused_ffn and k in ("gate", "up"))}
            if fused_ffn:  # gate | up rows interleaved in one weight: one GEMM, the SwiGLU product formed in its epilogue
                L["gateup"] = izb.gateup_weight(cfg.qtype, sh["gate"][0], sh["up"][0], sh["gate"][1], sh["gate"][2], device=device)
            self.layers.append(L)
        self.comm = None if mode == "p2p" else izb.TpComm(world, rank, device, timeout_ms=timeout_ms, max_ctas=comm_sms if self.overlap else 0)
        dev = torch.device("cuda", device)
        f32, i8 = torch.float32, torch.int8
        nf = self.plan.ffn[1] - self.plan.ffn[0]
        Tc = self.Tc
        self.x = torch.empty((T, E), dtype=f32, device=dev)
        self.part_a = torch.empty((T, E), dtype=f32, device=dev)   # partial outputs of O, per chunk rows
        self.part_f = torch.empty((T, E), dtype=f32, device=dev) if chunks > 1 else self.part_a  # ... of down
        self.qkv = torch.empty((T, self.plan.qkv_rows), dtype=f32, device=dev)
        self.h = torch.empty((T, nf), dtype=f32, device=dev)
        kmax = max(E, nf)
        self.aq = torch.empty((Tc * kmax,), dtype=i8, device=dev)
        self.asc = torch.empty((Tc * (kmax // 32),), dtype=f32, device=dev)
        if mode == "p2p":
            self._p2p_setup(dev)                                       # xq lives in memory the other ranks write into
        else:
            self.xq = torch.empty((T, E), dtype=i8, device=dev)        # quantised residual stream (input of QKV / gate / up)
        self.xsc_c = torch.empty((chunks, E // 32, Tc), dtype=f32, device=dev)  # its scales, [E/32][rows] per chunk
        self.compute = None
        self.side = torch.cuda.Stream(device=dev, priority=-1) if self.overlap else None
        if self.overlap:
            sms = torch.cuda.get_device_properties(device).multi_processor_count
            izb.set_sm_limit(device, sms - comm_sms)
        # every arena at its final size before the first step: no allocation, no device-wide wait inside the pipeline
        izb.reserve(device, Tc, kmax)
        self.ev_sum = [None] * chunks    # the last sum of chunk c (side stream)

    # ---- views
    def rows(self, c):
        return slice(c * self.Tc, (c + 1) * self.Tc)

    @property
    def part(self):
        return self.part_a

    @property
    def xsc(self):
        """Scales of the whole quantised stream as [E/32][T]."""
        E32 = self.cfg.hidden // 32
        return self.xsc_c[0] if self.chunks == 1 else self.xsc_c.permute(1, 0, 2).reshape(E32, self.cfg.tokens)

    def owned_rows(self) -> np.ndarray:
        """Token rows whose residual-stream values this rank holds after a sum ("rs_quant_ag": its rows of every chunk)."""
        if self.mode not in ("rs_quant_ag", "p2p"):
            return np.arange(self.cfg.tokens)
        own = self.Tc // self.world
        return np.concatenate([np.arange(c * self.Tc + self.rank * own, c * self.Tc + (self.rank + 1) * own) for c in range(self.chunks)])

    def _quant(self, src, K):
        Tc = self.Tc
        aq = self.aq[:Tc * K].view(Tc, K)
        asc = self.asc[:Tc * (K // 32)].view(K // 32, Tc)
        self.izb.quantize_act(src, Mp=Tc, out=(aq, asc, None))
        return aq, asc

    def _quant_matmul(self, w, src, K, out):
        """quant_rows + matmul of a chunk in one call (the quantiser writes the GEMM's operand images as well)."""
        Tc = self.Tc
        aq = self.aq[:Tc * K].view(Tc, K)
        asc = self.asc[:Tc * (K // 32)].view(K // 32, Tc)
        self.izb.quant_matmul(w, src, Tc, Tc, out=out, qout=(aq, asc))

    # ---- "p2p": copy-engine transport
    def _p2p_setup(self, dev):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        torch, cfg, R = self.torch, self.cfg, self.world
        T, E, Tc = cfg.tokens, cfg.hidden, self.Tc
        own = Tc // R
        self.own, self.n_own = own, own * E
        al = lambda n: (n + 255) // 256 * 256
        self.off_rx = 0                                                  # [chunks][R][own][E] f32: partial rows by source rank
        self.off_xq = al(self.off_rx + T * E * 4)                        # [T][E] int8: the gathered quantised stream
        self.off_stage = al(self.off_xq + T * E)                         # [chunks][R][E/32][own] f32: block scales by owner
        self.off_flag = al(self.off_stage + self.chunks * R * (E // 32) * own * 4)  # [2][chunks][R] u32, 4 bytes apart
        total = al(self.off_flag + 2 * self.chunks * R * 4)
        self.sym = symm.empty(total, dtype=torch.uint8, device=dev)
        self.sym.zero_()
        torch.cuda.synchronize()
        self.sym_hdl = symm.rendezvous(self.sym, dist.group.WORLD.group_name)
        self.peer = [int(p) for p in self.sym_hdl.buffer_ptrs]           # base address of every rank's buffer, as mapped here
        dist.barrier()
        me = self.sym
        self.rx = me[self.off_rx:self.off_rx + T * E * 4].view(torch.float32).view(self.chunks, R, own, E)
        self.xq = me[self.off_xq:self.off_xq + T * E].view(torch.int8).view(T, E)
        self.stage = me[self.off_stage:self.off_stage + self.chunks * R * (E // 32) * own * 4].view(torch.float32).view(self.chunks, R, E // 32, own)
        self.copy_st = torch.cuda.Stream(device=dev)
        self.seq = 0          # number of the sum in flight (flags carry it: they only grow)
        self.pipe = SumPipeline(self.chunks, lag=1)
        self.ev_local = [None] * self.chunks  # this rank's own part of chunk c has been copied (copy stream)

    def _flag(self, r, kind, c, src):
        """Address, in rank r's buffer, of the flag (kind 0: partials arrived, 1: gathered rows arrived) of chunk c raised by src."""
        return self.peer[r] + self.off_flag + ((kind * self.chunks + c) * self.world + src) * 4

    def _p2p_push_partials(self, c, part, seq):
        """This rank's partial rows of chunk c -> every owner's receive buffer (its own included), then the flag there."""
        torch, izb, R, me = self.torch, self.izb, self.world, self.rank
        ev = torch.cuda.Event()
        ev.record(self.compute)
        self.copy_st.wait_event(ev)
        nb = self.n_own * 4
        copies = [(self.peer[r] + self.off_rx + ((c * R + me) * self.n_own) * 4, part.data_ptr() + r * nb, nb) for r in range(R)]
        # Flags only on the OTHER ranks: a stream may wait for a value that another device writes, never for one that a
        # stream of its own device writes (CUDA does not see that order and may run the two streams the wrong way round).
        # This rank's own part is ordered with an event.
        flags = [self._flag(r, 0, c, me) for r in range(R) if r != me]
        izb.p2p_push(copies, flags, seq, stream=self.copy_st.cuda_stream)
        self.ev_local[c] = torch.cuda.Event()
        self.ev_local[c].record(self.copy_st)

    def _p2p_reduce(self, c, seq):
        """Owner's part of sum `seq` for chunk c, on the compute stream: wait for all partials, add them in rank order to this
        rank's residual rows, quantise, and send the rows + scales to every rank."""
        torch, izb, R, me, E = self.torch, self.izb, self.world, self.rank, self.cfg.hidden
        izb.p2p_wait([self._flag(me, 0, c, src) for src in range(R) if src != me], seq)
        self.compute.wait_event(self.ev_local[c])
        r0 = c * self.Tc + me * self.own
        xs = self.x[r0:r0 + self.own]
        izb.tp_add(xs, self.rx[c].view(R, self.n_own))
        izb.quantize_act(xs, Mp=self.own, out=(self.xq[r0:r0 + self.own], self.stage[c, me], None))
        ev = torch.cuda.Event()
        ev.record(self.compute)
        self.copy_st.wait_event(ev)
        sb = (E // 32) * self.own * 4
        copies = []
        for r in range(R):
            if r == me:
                continue
            copies.append((self.peer[r] + self.off_xq + r0 * E, self.xq.data_ptr() + r0 * E, self.n_own))
            copies.append((self.peer[r] + self.off_stage + ((c * R + me) * (E // 32) * self.own) * 4, self.stage[c, me].data_ptr(), sb))
        izb.p2p_push(copies, [self._flag(r, 1, c, me) for r in range(R) if r != me], seq, stream=self.copy_st.cuda_stream)

    def _p2p_await(self, c, seq):
        """Before the compute stream reads chunk c of the quantised stream: every owner's rows of sum `seq` have arrived."""
        if seq == 0:
            return
        izb = self.izb
        izb.p2p_wait([self._flag(self.rank, 1, c, src) for src in range(self.world) if src != self.rank], seq)
        izb.tp_scales_from_ranks(self.xsc_c[c], self.stage[c], self.world, self.own, self.cfg.hidden)

    def _sum(self, c, part):
        """Row-parallel partials of chunk c -> residual stream; leaves the chunk's quantised stream in xq / xsc_c[c]."""
        izb, r = self.izb, self.rows(c)
        x, xq, xsc = self.x[r], self.xq[r], self.xsc_c[c]
        if self.mode == "allreduce":
            self.comm.allreduce_rows(x, part)
            izb.quantize_act(x, Mp=self.Tc, out=(xq, xsc, None))
        else:
            own = self.Tc // self.world
            xs = x[self.rank * own:(self.rank + 1) * own]
            self.comm.reduce_quant_gather(x, part, xq, xsc, xsum=xs)

    def _sum_async(self, c, part):
        """The sum of chunk c: on the side stream, after what the compute stream has queued so far."""
        torch = self.torch
        if self.mode == "p2p":
            # the partials leave now; the owner's reduce of the chunk BEFORE this one is queued behind this chunk's GEMMs
            self._p2p_push_partials(c, part, self.seq)
            for rc, rseq in self.pipe.sent(c, self.seq):
                self._p2p_reduce(rc, rseq)
            return
        if not self.overlap:
            self._sum(c, part)
            return
        ev = torch.cuda.Event()
        ev.record(self.compute)
        self.side.wait_event(ev)
        with torch.cuda.stream(self.side):
            self._sum(c, part)
            done = torch.cuda.Event()
            done.record(self.side)
        self.ev_sum[c] = done

    def _await_sum(self, c):
        if self.mode == "p2p":
            reduces, seq = self.pipe.needed(c)
            for rc, rseq in reduces:
                self._p2p_reduce(rc, rseq)
            self._p2p_await(c, seq)
            return
        if self.overlap and self.ev_sum[c] is not None:
            self.compute.wait_event(self.ev_sum[c])

    def set_input(self, x):
        self.x.copy_(x)
        for c in range(self.chunks):
            r = self.rows(c)
            self.izb.quantize_act(self.x[r], Mp=self.Tc, out=(self.xq[r], self.xsc_c[c], None))

    def _attn_half(self, L, c):
        izb, Tc, r = self.izb, self.Tc, self.rows(c)
        nq = self.plan.q[1] - self.plan.q[0]
        izb.matmul(L["qkv"], self.xq[r], self.xsc_c[c], Tc, out=self.qkv[r])
        self._quant_matmul(L["o"], self.qkv[r][:, :nq], nq, self.part_a[r])

    def _ffn_half(self, L, c):
        izb, Tc, r = self.izb, self.Tc, self.rows(c)
        if "gateup" in L:
            izb.gemm(L["gateup"], self.xq[r], self.xsc_c[c], M=Tc, out=self.h[r], acc=3)
        else:
            izb.matmul(L["gate"], self.xq[r], self.xsc_c[c], Tc, out=self.h[r])
            izb.matmul(L["up"], self.xq[r], self.xsc_c[c], Tc, out=self.h[r], acc=2)
        self._quant_matmul(L["down"], self.h[r], self.h.shape[1], self.part_f[r])

    def forward(self, trace: list | None = None, layers: int | None = None):
        """One pass over all (or the first `layers`) layers.  `trace` (tests, parity fields of the benchmark) receives per
        layer a dict of copies of every stage's output, so that each stage can be checked against the oracle from the
        stage before it; with a trace the two halves of a layer are separated by device-wide waits."""
        torch = self.torch
        self.compute = torch.cuda.current_stream()
        sync = torch.cuda.synchronize
        for L in self.layers[:layers]:
            t = {} if trace is not None else None
            if t is not None:
                sync()
                t["xq0"], t["xsc0"], t["x0"] = self.xq.clone(), self.xsc.clone(), self.x.clone()
                t["o_part"], t["down_part"] = torch.empty_like(self.part_a), torch.empty_like(self.part_a)
            if self.mode == "p2p":
                self.seq += 1
            for c in range(self.chunks):
                self._await_sum(c)
                self._attn_half(L, c)
                if t is not None:  # (before the sum: the collectives work in place)
                    t["o_part"][self.rows(c)].copy_(self.part_a[self.rows(c)])
                self._sum_async(c, self.part_a[self.rows(c)])
            if t is not None:
                self._settle()
                sync()
                t["qkv"], t["x1"], t["xq1"], t["xsc1"] = self.qkv.clone(), self.x.clone(), self.xq.clone(), self.xsc.clone()
            if self.mode == "p2p":
                self.seq += 1
            for c in range(self.chunks):
                self._await_sum(c)
                self._ffn_half(L, c)
                if t is not None:
                    t["down_part"][self.rows(c)].copy_(self.part_f[self.rows(c)])
                self._sum_async(c, self.part_f[self.rows(c)])
            if t is not None:
                self._settle()
                sync()
                t["h"], t["x2"], t["xq2"], t["xsc2"] = self.h.clone(), self.x.clone(), self.xq.clone(), self.xsc.clone()
                trace.append(t)
        for c in range(self.chunks):
            self._await_sum(c)
        return self.x

    def _settle(self):
        """Everything that was handed to a sum has arrived (used where a trace looks at the stream between two halves)."""
        for c in range(self.chunks):
            self._await_sum(c)

    def close(self):
        if self.overlap:
            self.izb.set_sm_limit(self.device, 0)
        for L in self.layers:
            for w in L.values():
                w.close()
        if self.comm is not None:
            self.comm.close()
        if self.mode == "p2p":
            self.torch.cuda.synchronize()
            import torch.distributed as dist
            dist.barrier()  # (no rank frees memory another rank may still be writing)
            self.rx = self.xq = self.stage = self.sym = self.sym_hdl = None
