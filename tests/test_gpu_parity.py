"""GPU parity tests: every CUDA kernel, called through the C ABI, against the CPU oracle on the same seeded inputs.

Bars: int8 activations, scales and per-block int32 dots bit-exact; f32 outputs max|err| / max|ref| <= 1e-5 (the
reference's own error form, bench/gemv_bench.cpp:199-214) against both oracle orders and the f64 model.
"""
import os

import numpy as np
import pytest

from arcinferzero_b200 import synth as S
from oracle import oracle as O

pytestmark = pytest.mark.gpu
TOL = 1e-5


@pytest.fixture(scope="module")
def torch():
    import torch as t
    assert t.cuda.is_available(), "GPU tests need a CUDA device"
    return t


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def rel(got, ref):
    return float(np.abs(got.astype(np.float64) - ref.astype(np.float64)).max() / np.abs(ref).max())


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


# ------------------------------------------------------------------------------------------------ quantiser
def test_quantize_golden_bit_exact(izb, torch, golden_dir):
    g = np.load(os.path.join(golden_dir, "quantize.npz"))
    aq, asc, absum = izb.quantize_act(dev(torch, g["x"]), Mp=16, want_absum=True)
    aq, asc, absum = aq.cpu().numpy(), asc.cpu().numpy(), absum.cpu().numpy()
    bad = np.argwhere(aq[:9] != g["aq"])
    assert bad.size == 0, (bad[:5], aq[:9][tuple(bad[0])], g["aq"][tuple(bad[0])], g["x"][tuple(bad[0])])
    assert (aq[9:] == 0).all()
    assert (bits(asc[:, :9]) == bits(g["asc"])).all() and (asc[:, 9:] == 0).all()
    assert (absum[:, :9] == g["absum"]).all() and (absum[:, 9:] == 0).all()


@pytest.mark.parametrize("M,K,Mp,ldx", [(1, 256, 16, 256), (5, 512, 16, 516), (33, 1024, 48, 1024), (128, 5120, 128, 5120),
                                        (200, 768, 256, 772), (64, 17408, 64, 17408)])
def test_quantize_bit_exact_ragged(izb, torch, M, K, Mp, ldx):
    rng = np.random.default_rng(M * 7 + K)
    xs = np.zeros((M, ldx), np.float32)
    xs[:, :K] = rng.standard_normal((M, K), dtype=np.float32) * np.float32(10.0) ** rng.integers(-3, 3, (M, 1))
    xs[:, K:] = 777.0  # beyond the row: must not be read into the result
    xd = dev(torch, xs)[:, :K]
    # NaN / sentinel poison: every output byte the call owns must be overwritten, nothing else touched
    aq = torch.full((Mp + 1, K), 99, dtype=torch.int8, device="cuda")
    asc = torch.full((K // 32 + 1, Mp), float("nan"), dtype=torch.float32, device="cuda")
    absum = torch.full((K // 16 + 1, Mp), -7, dtype=torch.int16, device="cuda")
    izb.quantize_act(xd, Mp=Mp, out=(aq, asc, absum))
    raq, rasc, rab = O.quantize_act(xs[:, :K], Mp=Mp)
    assert (aq[:Mp].cpu().numpy() == raq).all() and (aq[Mp].cpu().numpy() == 99).all()
    assert (bits(asc[:-1].cpu().numpy()) == bits(rasc)).all() and torch.isnan(asc[-1]).all()
    assert (absum[:-1].cpu().numpy() == rab).all() and (absum[-1].cpu().numpy() == -7).all()


def test_swiglu_quant_stagewise(izb, torch):
    rng = np.random.default_rng(3)
    M, F = 40, 768
    gu = rng.standard_normal((M, 2 * F), dtype=np.float32) * 3
    aq, asc, h = izb.swiglu_quant(dev(torch, gu), F, want_h=True)
    h = h.cpu().numpy()
    want = gu[:, :F] / (1 + np.exp(-gu[:, :F].astype(np.float64))) * gu[:, F:]
    assert rel(h, want.astype(np.float32)) < 1e-6
    raq, rasc, _ = O.quantize_act(h, Mp=asc.shape[1])  # teacher forcing: the oracle quantises the GPU's own h
    assert (aq.cpu().numpy() == raq).all() and (bits(asc.cpu().numpy()) == bits(rasc)).all()


@pytest.mark.parametrize("M,K", [(37, 5120), (300, 1024), (1, 256)])
def test_rmsnorm_quant_bit_exact(izb, torch, M, K):
    """izb_rmsnorm_quant against the oracle: the sum of squares is taken in the same defined order, so the normalised
    rows, the int8 values and the scales are identical bit for bit; padding rows are zero."""
    rng = np.random.default_rng(M * 7 + K)
    x = rng.standard_normal((M, K), dtype=np.float32) * rng.uniform(0.01, 30.0, (M, 1)).astype(np.float32)
    if M > 2:
        x[2] = 0.0
    w = (1.0 + 0.2 * rng.standard_normal(K)).astype(np.float32)
    aq, asc, h = izb.rmsnorm_quant(dev(torch, x), dev(torch, w), 1e-6, want_h=True)
    Mp = asc.shape[1]
    ry, raq, rasc, _ = O.rmsnorm_quant(x, w, 1e-6, Mp=Mp)
    assert (bits(h.cpu().numpy()) == bits(ry)).all()
    assert (aq.cpu().numpy() == raq).all()
    assert (bits(asc.cpu().numpy()) == bits(rasc)).all()
    assert (aq.cpu().numpy()[M:] == 0).all()


@pytest.mark.parametrize("M,K,second", [(1, 5120, True), (5, 1024, False), (8, 16384, True)])
def test_add_norm_quant_bit_exact(izb, torch, M, K, second):
    """izb_add_norm_quant against the oracle (same defined summation orders): the updated residual rows, the int8 values
    and the scales are identical bit for bit."""
    rng = np.random.default_rng(M + K)
    x = rng.standard_normal((M, K), dtype=np.float32)
    t = rng.standard_normal((M, K), dtype=np.float32) * 3
    w = (1.0 + 0.2 * rng.standard_normal(K)).astype(np.float32)
    w2 = (1.0 + 0.2 * rng.standard_normal(K)).astype(np.float32) if second else None
    xd = dev(torch, x)
    aq, asc = izb.add_norm_quant(xd, dev(torch, t), dev(torch, w), 1e-6, 0.75, None if w2 is None else dev(torch, w2))
    rx, raq, rasc, _ = O.add_norm_quant(x, t, w, 1e-6, 0.75, w2, Mp=asc.shape[1])
    assert (bits(xd.cpu().numpy()) == bits(rx)).all()
    assert (aq.cpu().numpy() == raq).all()
    assert (bits(asc.cpu().numpy()) == bits(rasc)).all()


# ------------------------------------------------------------------------------------------------ GEMV
@pytest.mark.parametrize("qt", [12, 8])
@pytest.mark.parametrize("T", [1, 2, 3, 8])
@pytest.mark.parametrize("N,K", [(37, 256), (64, 1280), (130, 5120), (16, 17408)])
def test_gemv_matches_oracle(izb, torch, qt, T, N, K):
    w = S.make_weight(qt, N, K, 1000 + N + K + qt)
    x = S.make_act(T, K, 2000 + T + K)
    aq, asc, _ = O.quantize_act(x, Mp=16)
    W = izb.Weight(qt, w, N, K)
    out = torch.full((T, N + 8), float("nan"), dtype=torch.float32, device="cuda")
    izb.gemv(W, dev(torch, aq), dev(torch, asc), T, out=out, c_off=4)
    got = out.cpu().numpy()
    assert np.isnan(got[:, :4]).all() and np.isnan(got[:, N + 4:]).all()
    for order in ("gemv", "gemm", "f64"):
        assert rel(got[:, 4:N + 4], O.matmul(qt, w, K, aq, asc, T, order)) < TOL, order
    # accumulate mode
    base = np.random.default_rng(5).standard_normal((T, N)).astype(np.float32) * 50
    o2 = dev(torch, base)
    izb.gemv(W, dev(torch, aq), dev(torch, asc), T, out=o2, acc=1)
    assert rel(o2.cpu().numpy() - base, O.matmul(qt, w, K, aq, asc, T, "gemv")) < 1e-4  # (after cancellation with base)
    W.close()


@pytest.mark.parametrize("T", [1, 2, 3, 4])
@pytest.mark.parametrize("N,K", [(1030, 2048), (8195, 1024), (9001, 3072), (5120, 5120), (17408, 5120), (5120, 17408), (1501, 8192), (1100, 7168)])
def test_gemv_q4k_many_rows(izb, torch, T, N, K):
    """The Q4_K decode kernels taken from 1024 weight rows on (activations in registers for one row, staged per lane for
    2..4; two weight rows per warp pass): odd row counts, K with a half-empty last step, store offset and accumulate."""
    qt = 12
    w = S.make_weight(qt, N, K, 77 + N + K)
    x = S.make_act(T, K, 88 + T + K)
    aq, asc, _ = O.quantize_act(x, Mp=16)
    W = izb.Weight(qt, w, N, K)
    out = torch.full((T, N + 8), float("nan"), dtype=torch.float32, device="cuda")
    izb.gemv(W, dev(torch, aq), dev(torch, asc), T, out=out, c_off=4)
    got = out.cpu().numpy()
    assert np.isnan(got[:, :4]).all() and np.isnan(got[:, N + 4:]).all()
    ref = O.matmul(qt, w, K, aq, asc, T, "gemv")
    assert rel(got[:, 4:N + 4], ref) < TOL
    assert rel(got[:, 4:N + 4], O.matmul(qt, w, K, aq, asc, T, "f64")) < TOL
    base = np.random.default_rng(6).standard_normal((T, N)).astype(np.float32) * 50
    o2 = dev(torch, base)
    izb.gemv(W, dev(torch, aq), dev(torch, asc), T, out=o2, acc=1)
    assert rel(o2.cpu().numpy() - base, ref) < 1e-4
    assert izb.device_status(0) == 0
    W.close()


def test_matmul_dispatch_by_rows(izb, torch):
    K, N = 1024, 64
    for qt in (12, 8):
        w = S.make_weight(qt, N, K, 31 + qt)
        W = izb.Weight(qt, w, N, K)
        for T in (1, 2, 8, 9, 40):
            x = S.make_act(T, K, 77 + T)
            Mp = izb.pad_rows(T)
            aq, asc, _ = O.quantize_act(x, Mp=Mp)
            n0 = izb.launch_count()
            out = izb.matmul(W, dev(torch, aq), dev(torch, asc), T)
            assert izb.launch_count() > n0
            assert rel(out.cpu().numpy()[:T], O.matmul(qt, w, K, aq, asc, T, "f64")) < TOL
        with pytest.raises(izb.IzbError):
            izb.matmul(W, dev(torch, aq), dev(torch, asc), 2, acc=2)
        W.close()


# ------------------------------------------------------------------------------------------------ CUDA-core GEMM
@pytest.mark.parametrize("qt", [12, 8])
@pytest.mark.parametrize("M,N,K", [(16, 16, 256), (48, 80, 512), (130, 272, 1280), (64, 64, 5120)])
def test_gemm_core_is_bit_exact_with_the_reference_order(izb, torch, qt, M, N, K):
    w = S.make_weight(qt, N, K, 10 + M + N + K + qt)
    x = S.make_act(M, K, 20 + M + K)
    Mp = izb.pad_rows(M)
    aq, asc, _ = O.quantize_act(x, Mp=Mp)
    W = izb.Weight(qt, w, N, K)
    out = izb.gemm(W, dev(torch, aq), dev(torch, asc), impl=izb.GEMM_CORE).cpu().numpy()
    ref = O.matmul(qt, w, K, aq, asc, Mp, "gemm")
    assert (bits(out) == bits(ref)).all()
    assert rel(out[:M], O.matmul(qt, w, K, aq, asc, M, "f64")) < TOL
    dots = izb.block_dots(W, dev(torch, aq), M, impl=izb.GEMM_CORE).cpu().numpy()
    rd, _ = O.block_dots(qt, w, K, aq[:M])
    assert (dots == rd).all()
    W.close()


def test_gemm_core_store_modes_and_offsets(izb, torch):
    qt, M, N, K = 12, 32, 48, 512
    w = S.make_weight(qt, N, K, 1)
    aq, asc, _ = O.quantize_act(S.make_act(M, K, 2), Mp=M)
    W = izb.Weight(qt, w, N, K)
    c0 = np.random.default_rng(9).standard_normal((M, 64)).astype(np.float32)
    for acc in (0, 1, 2):
        out = dev(torch, c0)
        izb.gemm(W, dev(torch, aq), dev(torch, asc), out=out, c_off=8, acc=acc, impl=izb.GEMM_CORE)
        ref = O.matmul(qt, w, K, aq, asc, M, "gemm", C_in=c0, ldc=64, c_off=8, acc=acc)
        got = out.cpu().numpy()
        if acc < 2:
            assert (bits(got) == bits(ref)).all()
        else:
            assert (bits(got[:, :8]) == bits(ref[:, :8])).all() and (bits(got[:, 56:]) == bits(ref[:, 56:])).all()
            assert rel(got[:, 8:56], ref[:, 8:56]) < 1e-6
    # fewer valid rows than Mp: rows past M_rows are left alone
    out = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    izb.gemm(W, dev(torch, aq), dev(torch, asc), M=20, out=out, impl=izb.GEMM_CORE)
    got = out.cpu().numpy()
    assert not np.isnan(got[:20]).any() and np.isnan(got[20:]).all()
    W.close()


def test_config1_q8_0_gemm_full_size(izb, torch):
    """BASELINE config 1 in full: M=512, N=4096, K=4096, Q8_0."""
    M, N, K = 512, 4096, 4096
    w = S.make_weight(8, N, K, 20261125)
    x = S.make_act(M, K, 20261126)
    xd = dev(torch, x)
    aq, asc, _ = izb.quantize_act(xd, Mp=M)
    raq, rasc, _ = O.quantize_act(x, Mp=M)
    assert (aq.cpu().numpy() == raq).all() and (bits(asc.cpu().numpy()) == bits(rasc)).all()
    W = izb.Weight(8, w, N, K)
    core = izb.gemm(W, aq, asc, impl=izb.GEMM_CORE).cpu().numpy()
    assert (bits(core) == bits(O.matmul(8, w, K, raq, rasc, M, "gemm"))).all()
    auto = izb.matmul(W, aq, asc, M).cpu().numpy()
    assert rel(auto, core) < TOL
    rows = np.arange(0, M, 37)
    assert rel(auto[rows], O.matmul(8, w, K, raq[rows], np.ascontiguousarray(rasc[:, rows]), len(rows), "f64")) < TOL
    W.close()


# ------------------------------------------------------------------------------------------------ mixture of experts
def test_moe_route_and_sort(izb, torch):
    rng = np.random.default_rng(4)
    T, NE, NU = 300, 128, 8
    lg = rng.standard_normal((T, NE), dtype=np.float32)
    lg[3, :] = 0.25  # all ties: the lowest ids win
    lg[4, 10] = lg[4, 90] = 5.0
    ids, wts, counts = izb.moe_route(dev(torch, lg), NU)
    rid, rw, rc = O.moe_route(lg, NU)
    assert (ids.cpu().numpy() == rid).all() and (counts.cpu().numpy() == rc).all()
    assert np.abs(wts.cpu().numpy() - rw).max() < 1e-6
    assert (rid[3] == np.arange(8)).all()
    for TM in (8, 128):
        offs, tiles, max_tiles, stok, swt, inv = izb.moe_sort(ids, wts, counts, TM)
        roffs, rtiles, rstok, rswt, rinv = O.moe_sort(rid, wts.cpu().numpy(), rc, TM)
        assert (offs.cpu().numpy() == roffs).all()
        nt = int(tiles[0])
        assert nt == rtiles[0] and (tiles.cpu().numpy()[:1 + 3 * nt] == rtiles[:1 + 3 * nt]).all()
        assert (stok.cpu().numpy() == rstok).all() and (inv.cpu().numpy() == rinv).all()
        assert (bits(swt.cpu().numpy()) == bits(rswt)).all()


@pytest.mark.parametrize("qt", [12, 8])
def test_moe_expert_path_stagewise(izb, torch, qt):
    """gate/up -> SiLU*mul -> quantise -> down -> combine on a small MoE; each stage checked with teacher forcing."""
    rng = np.random.default_rng(11)
    T, E, F, NE, NU, TM = 48, 512, 256, 8, 2, 8
    wg, wu = S.make_weight(qt, NE * F, E, 1), S.make_weight(qt, NE * F, E, 2)
    wd = S.make_weight(qt, NE * E, F, 3)
    x = S.make_act(T, E, 4)
    lg = rng.standard_normal((T, NE), dtype=np.float32)
    Wg, Wu, Wd = izb.Weight(qt, wg, F, E, n_mats=NE), izb.Weight(qt, wu, F, E, n_mats=NE), izb.Weight(qt, wd, E, F, n_mats=NE)
    xd = dev(torch, x)
    aq, asc, _ = izb.quantize_act(xd, Mp=T)
    ids, wts, counts = izb.moe_route(dev(torch, lg), NU)
    offs, tiles, max_tiles, stok, swt, inv = izb.moe_sort(ids, wts, counts, TM)
    S_ = T * NU
    h = izb.moe_gateup(Wg, Wu, aq, asc, tiles, max_tiles, TM, stok, S_)
    se = O.slot_experts(offs.cpu().numpy())
    rh = O.moe_gateup(qt, wg, wu, F, E, aq.cpu().numpy(), asc.cpu().numpy(), se, stok.cpu().numpy())
    assert rel(h.cpu().numpy(), rh) < TOL
    hq, hsc, _ = izb.quantize_act(h, Mp=S_)
    rq, rs, _ = O.quantize_act(h.cpu().numpy(), Mp=S_)
    assert (hq.cpu().numpy() == rq).all() and (bits(hsc.cpu().numpy()) == bits(rs)).all()
    y = izb.moe_down(Wd, hq, hsc, tiles, max_tiles, TM, swt, S_)
    ry = O.moe_down(qt, wd, E, F, rq, rs, se, swt.cpu().numpy())
    assert rel(y.cpu().numpy(), ry) < TOL
    x0 = rng.standard_normal((T, E), dtype=np.float32)
    out = izb.moe_combine(dev(torch, x0), y, inv, NU)
    assert (bits(out.cpu().numpy()) == bits(O.moe_combine(x0, y.cpu().numpy(), inv.cpu().numpy(), NU))).all()
    for W in (Wg, Wu, Wd):
        W.close()


# ------------------------------------------------------------------------------------------------ tensor parallel pieces
def test_tp_add_rank_order(izb, torch):
    rng = np.random.default_rng(8)
    x = rng.standard_normal((40, 256), dtype=np.float32)
    parts = rng.standard_normal((4, 40, 256), dtype=np.float32) * 100
    got = izb.tp_add(dev(torch, x), dev(torch, parts)).cpu().numpy()
    assert (bits(got) == bits(O.tp_add(x, parts))).all()


@pytest.mark.parametrize("qt", [12, 8])
def test_sharded_matmul_equals_unsplit(izb, torch, qt):
    """Column-parallel rows concatenate; row-parallel K slices sum to the unsplit product (zero/mgpu/engine_tp_shard.h)."""
    M, N, K, R = 32, 96, 2048, 4
    w = S.make_weight(qt, N, K, 5)
    aq, asc, _ = O.quantize_act(S.make_act(M, K, 6), Mp=M)
    full = O.matmul(qt, w, K, aq, asc, M, "f64")
    aqd, ascd = dev(torch, aq), dev(torch, asc)
    cols = []
    for r in range(R):
        n0, n1 = izb.tp_range(N, 16, R, r)
        Wr = izb.Weight(qt, w, N, K, row_range=(n0, n1))
        cols.append(izb.gemm(Wr, aqd, ascd, impl=izb.GEMM_CORE).cpu().numpy())
        Wr.close()
    assert rel(np.concatenate(cols, 1), full) < TOL
    parts = []
    for r in range(R):
        k0, k1 = izb.tp_range(K, 256, R, r)
        Wr = izb.Weight(qt, w, N, K, col_range=(k0, k1))
        parts.append(izb.gemm(Wr, dev(torch, aq[:, k0:k1]), dev(torch, asc[k0 // 32:k1 // 32]), impl=izb.GEMM_CORE))
        Wr.close()
    x = torch.zeros((M, N), dtype=torch.float32, device="cuda")
    izb.tp_add(x, torch.stack(parts))
    assert rel(x.cpu().numpy(), full) < TOL


def test_matmul_host_round_trip(izb, torch):
    qt, M, N, K = 12, 100, 256, 1024
    w = S.make_weight(qt, N, K, 1)
    x = S.make_act(M, K, 2)
    W = izb.Weight(qt, w, N, K)
    xh = torch.from_numpy(x).pin_memory()
    oh = torch.empty((M, N), dtype=torch.float32).pin_memory()
    izb.matmul_host(W, xh, oh)
    aq, asc, _ = O.quantize_act(x, Mp=izb.pad_rows(M))
    assert rel(oh.numpy(), O.matmul(qt, w, K, aq, asc, M, "f64")) < TOL
    W.close()


@pytest.mark.parametrize("rows,ld,N,off,cap", [(1, 151936, 151936, 0, 30.0), (8, 1032, 1000, 4, 50.0), (3, 517, 501, 7, 30.0), (2, 64, 1, 3, 0.5)])
def test_softcap_rows_against_the_oracle(izb, torch, rows, ld, N, off, cap):
    """izb_softcap_rows (softcap_rows, zero/kernels/ops_attn_g.cl:724) against the oracle: within 1e-6 of the cap
    (tanhf of two math libraries), vectorised and scalar row starts, everything outside the capped region untouched."""
    rng = np.random.default_rng(N + off)
    c = (rng.standard_normal((rows + 1, ld)) * 2 * cap).astype(np.float32)
    c[0, off:off + min(N, 4)] = [0.0, 1e4, -1e4, 1e-20][:min(N, 4)]
    d = torch.from_numpy(c).cuda()
    izb.softcap_rows(d, rows, N, cap, off)
    out = d.cpu().numpy()
    ref = O.softcap_rows(c, rows, N, cap, off)
    assert np.abs(out - ref).max() <= 1e-6 * cap
    keep = np.ones_like(c, dtype=bool)
    keep[:rows, off:off + N] = False
    assert (out[keep] == c[keep]).all()
    assert np.abs(out[:rows, off:off + N]).max() <= cap


def test_softcap_after_the_head_gemv(izb, torch):
    """The output head as the reference runs it (zero/engine.h:1080-1111): Q8_0 GEMV of one row, then the soft-cap."""
    N, K, cap = 4096, 1024, 30.0
    w = S.make_weight(8, N, K, 31)
    W = izb.Weight(8, w, N, K)
    x = S.make_act(1, K, 32) * 40
    aq, asc, _ = izb.quantize_act(torch.from_numpy(x).cuda(), Mp=16)
    out = izb.matmul(W, aq, asc, 1)
    izb.softcap_rows(out, 1, N, cap)
    ref = O.matmul(8, w, K, aq.cpu().numpy(), asc.cpu().numpy(), 1, "f64")[:1].astype(np.float64)
    ref = cap * np.tanh(ref / cap)
    assert np.abs(out.cpu().numpy()[:1] - ref).max() / np.abs(ref).max() < 1e-5
    W.close()
