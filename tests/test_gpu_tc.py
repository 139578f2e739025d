"""GPU tests of the tcgen05 GEMM: its TMEM accumulators read back must equal the CPU's int32 block dots bit for bit, and
its f32 outputs must lie within 1e-5 of max|ref| of the oracle (both reference orders and the f64 model)."""
import numpy as np
import pytest

from arcinferzero_b200 import synth as S
from oracle import oracle as O

pytestmark = pytest.mark.gpu
TOL = 1e-5


@pytest.fixture(scope="module")
def torch():
    import torch as t
    assert t.cuda.is_available()
    return t


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def rel(got, ref):
    return float(np.abs(got.astype(np.float64) - ref.astype(np.float64)).max() / np.abs(ref).max())


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_selfcheck_passes_and_no_wait_gave_up(izb, torch):
    izb.selfcheck(0)
    assert izb.device_status(0) == 0


@pytest.mark.parametrize("qt", [12, 8])
@pytest.mark.parametrize("M,N,K", [(16, 128, 256), (130, 256, 512), (128, 128, 1280), (200, 384, 5120)])
def test_tc_block_dots_bit_exact(izb, torch, qt, M, N, K):
    w = S.make_weight(qt, N, K, 300 + M + N + K + qt)
    if qt == 12:
        w = w.copy().reshape(N, K // 256, 144)
        w[0, :, 16:] = 0xFF   # every quant 15
        w[1, :, 4:16] = 0xFF  # every scale / min 63
        w = w.reshape(N, -1)
    x = S.make_act(M, K, 400 + M + K)
    x[0, :] = 1.0   # every int8 = 127
    x[1, :] = -1.0  # every int8 = -127
    aq, _, _ = O.quantize_act(x, Mp=M)
    W = izb.Weight(qt, w, N, K)
    dots = izb.block_dots(W, dev(torch, aq), M, impl=izb.GEMM_TC).cpu().numpy()
    ref, _ = O.block_dots(qt, w, K, aq)
    assert (dots == ref).all(), np.argwhere(dots != ref)[:5]
    assert izb.device_status(0) == 0
    W.close()


@pytest.mark.parametrize("qt", [12, 8])
@pytest.mark.parametrize("M,N,K", [(16, 128, 256), (130, 256, 512), (300, 128, 1280), (128, 384, 5120), (64, 128, 17408)])
def test_tc_gemm_matches_oracle(izb, torch, qt, M, N, K):
    w = S.make_weight(qt, N, K, 500 + M + N + K + qt)
    x = S.make_act(M, K, 600 + M + K)
    Mp = izb.pad_rows(M)
    aq, asc, _ = O.quantize_act(x, Mp=Mp)
    W = izb.Weight(qt, w, N, K)
    out = torch.full((Mp, N + 8), float("nan"), dtype=torch.float32, device="cuda")
    izb.gemm(W, dev(torch, aq), dev(torch, asc), M=M, out=out, c_off=4, impl=izb.GEMM_TC)
    got = out.cpu().numpy()
    assert np.isnan(got[:, :4]).all() and np.isnan(got[:, N + 4:]).all() and np.isnan(got[M:]).all()
    for order in ("gemm", "gemv", "f64"):
        assert rel(got[:M, 4:N + 4], O.matmul(qt, w, K, aq, asc, M, order)) < TOL, order
    assert izb.device_status(0) == 0
    W.close()


@pytest.mark.parametrize("qt", [12, 8])
def test_tc_store_modes(izb, torch, qt):
    M, N, K = 144, 256, 1024
    w = S.make_weight(qt, N, K, 7 + qt)
    aq, asc, _ = O.quantize_act(S.make_act(M, K, 8), Mp=M)
    W = izb.Weight(qt, w, N, K)
    c0 = np.random.default_rng(9).standard_normal((M, N)).astype(np.float32)
    for acc in (1, 2):
        out = dev(torch, c0)
        izb.gemm(W, dev(torch, aq), dev(torch, asc), out=out, acc=acc, impl=izb.GEMM_TC)
        ref = O.matmul(qt, w, K, aq, asc, M, "gemm", C_in=c0, acc=acc)
        assert rel(out.cpu().numpy(), ref) < TOL
    W.close()


def test_config2_q4k_prefill_gemm_full_size(izb, torch):
    """BASELINE config 2 in full (M=8192, N=17408, K=5120, Q4_K): tensor-core kernel against the oracle on sampled
    token rows x all columns, against the CUDA-core kernel (bit-exact with the reference order) on everything, and the
    block dots of a sample."""
    M, N, K = 8192, 17408, 5120
    w = S.make_weight(12, N, K, 20261125)
    x = S.make_act(M, K, 20261126)
    aq, asc, _ = izb.quantize_act(dev(torch, x), Mp=M)
    W = izb.Weight(12, w, N, K)
    tc = izb.matmul(W, aq, asc, M)
    assert izb.device_status(0) == 0
    core = izb.gemm(W, aq, asc, impl=izb.GEMM_CORE)
    err = float((tc - core).abs().max() / core.abs().max())
    assert err < TOL, err
    rows = np.arange(5, M, 1021)
    raq, rasc = aq[rows].cpu().numpy(), asc[:, rows].cpu().numpy()
    sub = np.ascontiguousarray(w[::97])
    ref = O.matmul(12, sub, K, raq, np.ascontiguousarray(rasc), len(rows), "f64")
    assert rel(tc[rows][:, ::97].cpu().numpy(), ref) < TOL
    xq, xs, _ = O.quantize_act(x[rows], Mp=len(rows))
    assert (xq == raq).all() and (bits(xs) == bits(rasc)).all()
    W.close()


def test_moe_grouped_tensor_core_path(izb, torch):
    """The grouped GEMM (tiles of 128 slots per expert) against the per-tile kernels and the oracle, stage by stage."""
    rng = np.random.default_rng(12)
    T, E, F, NE, NU = 700, 512, 256, 8, 2
    qt = 12
    wg, wu = S.make_weight(qt, NE * F, E, 1), S.make_weight(qt, NE * F, E, 2)
    wd = S.make_weight(qt, NE * E, F, 3)
    Wg, Wu, Wd = izb.Weight(qt, wg, F, E, n_mats=NE), izb.Weight(qt, wu, F, E, n_mats=NE), izb.Weight(qt, wd, E, F, n_mats=NE)
    x = S.make_act(T, E, 4)
    lg = rng.standard_normal((T, NE), dtype=np.float32)
    lg[:, 0] += 2.0  # a hot expert: several full tiles; others ragged
    Tp = izb.pad_rows(T)
    aq, asc, _ = izb.quantize_act(dev(torch, x), Mp=Tp)
    ids, wts, counts = izb.moe_route(dev(torch, lg), NU)
    S_ = T * NU
    offs, tiles, max_tiles, stok, swt, inv = izb.moe_sort(ids, wts, counts, 128)
    h = izb.moe_gateup(Wg, Wu, aq, asc, tiles, max_tiles, 128, stok, S_)
    se = O.slot_experts(offs.cpu().numpy())
    rh = O.moe_gateup(qt, wg, wu, F, E, aq.cpu().numpy(), asc.cpu().numpy(), se, stok.cpu().numpy())
    assert rel(h.cpu().numpy(), rh) < TOL
    Sp = izb.pad_rows(S_)
    hq, hsc, _ = izb.quantize_act(h, Mp=Sp)
    y = izb.moe_down(Wd, hq, hsc, tiles, max_tiles, 128, swt, S_)
    ry = O.moe_down(qt, wd, E, F, hq.cpu().numpy()[:S_], np.ascontiguousarray(hsc.cpu().numpy()[:, :S_]), se, swt.cpu().numpy())
    assert rel(y.cpu().numpy(), ry) < TOL
    assert izb.device_status(0) == 0
    for W in (Wg, Wu, Wd):
        W.close()
