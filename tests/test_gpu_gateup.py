"""Gate and up projection as one interleaved weight (izb_weight_create_gateup) with the SwiGLU product in the GEMM's
epilogue (store mode 3): the same operations and roundings as the reference's two-launch form (gate GEMM, then the up
GEMM with store mode 2, zero/kernels/gemm.cl:562-565), so the two agree bit for bit; both within 1e-5 of the oracle."""
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


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def rel(got, ref):
    return float(np.abs(got.astype(np.float64) - ref.astype(np.float64)).max() / np.abs(ref).max())


@pytest.mark.parametrize("qt", [12, 8, 2])
@pytest.mark.parametrize("M,F,K", [(200, 256, 1024), (512, 704, 2048)])
def test_dense_fused_equals_two_launches_and_the_oracle(izb, torch, qt, M, F, K):
    wg, wu = S.make_weight(qt, F, K, 40 + qt + F), S.make_weight(qt, F, K, 41 + qt + F)
    Mp = izb.pad_rows(M)
    aq, asc, _ = O.quantize_act(S.make_act(M, K, 42 + M), Mp=Mp)
    daq, dasc = dev(torch, aq), dev(torch, asc)
    Wgu = izb.gateup_weight(qt, wg, wu, F, K)
    assert (Wgu.N, Wgu.K) == (2 * F, K)
    # the interleaved rows: groups of 32 alternate
    raw, per = Wgu.download(), Wgu.download().size // (2 * F)
    Wg = izb.Weight(qt, wg, F, K)
    Wu = izb.Weight(qt, wu, F, K)
    rg, ru = Wg.download().reshape(F, per), Wu.download().reshape(F, per)
    inter = np.stack([rg.reshape(F // 32, 32, per), ru.reshape(F // 32, 32, per)], axis=1).reshape(2 * F, per)
    assert (raw.reshape(2 * F, per) == inter).all()
    fused = torch.full((Mp, F + 8), float("nan"), dtype=torch.float32, device="cuda")
    izb.gemm(Wgu, daq, dasc, M=M, out=fused, c_off=4, acc=3)
    two = izb.gemm(Wg, daq, dasc, M=M)
    izb.gemm(Wu, daq, dasc, M=M, out=two, acc=2)
    got = fused.cpu().numpy()
    assert np.isnan(got[:, :4]).all() and np.isnan(got[:, F + 4:]).all() and np.isnan(got[M:]).all()
    if F % 128 == 0:  # (both forms on the tensor-core kernel: identical operations)
        assert (bits(got[:M, 4:F + 4]) == bits(two.cpu().numpy()[:M])).all()
    gate = O.matmul(qt, wg, K, aq, asc, M, "f64").astype(np.float64)
    ref = (O.matmul(qt, wu, K, aq, asc, M, "f64").astype(np.float64) * gate / (1.0 + np.exp(-gate))).astype(np.float32)
    assert rel(got[:M, 4:F + 4], ref) < TOL
    # the CUDA-core route of the same call
    core = izb.gemm(Wgu, daq, dasc, M=M, acc=3, impl=izb.GEMM_CORE).cpu().numpy()
    assert core.shape == (Mp, F) and rel(core[:M], ref) < TOL
    assert izb.device_status(0) == 0
    for W in (Wg, Wu, Wgu):
        W.close()


def test_moe_fused_stack_equals_the_two_stacks(izb, torch):
    rng = np.random.default_rng(5)
    T, E, F, NE, NU, TM, qt = 700, 512, 256, 12, 3, 128, 12
    wg, wu = S.make_weight(qt, NE * F, E, 51), S.make_weight(qt, NE * F, E, 52)
    Wg, Wu = izb.Weight(qt, wg, F, E, n_mats=NE), izb.Weight(qt, wu, F, E, n_mats=NE)
    Wgu = izb.gateup_weight(qt, wg, wu, F, E, n_mats=NE)
    x = S.make_act(T, E, 53)
    aq, asc, _ = izb.quantize_act(dev(torch, x), Mp=izb.pad_rows(T))
    ids, wts, counts = izb.moe_route(dev(torch, rng.standard_normal((T, NE)).astype(np.float32)), NU)
    offs, tiles, max_tiles, stok, swt, inv = izb.moe_sort(ids, wts, counts, TM)
    Sn = T * NU
    two = izb.moe_gateup(Wg, Wu, aq, asc, tiles, max_tiles, TM, stok, Sn).cpu().numpy()
    one = izb.moe_gateup(Wgu, None, aq, asc, tiles, max_tiles, TM, stok, Sn).cpu().numpy()
    assert one.shape == (Sn, F) and (bits(one) == bits(two)).all()
    se = O.slot_experts(offs.cpu().numpy())
    smp = np.unique(np.concatenate([[0, Sn - 1], rng.integers(0, Sn, 24)]))
    ref = O.moe_gateup(qt, wg, wu, F, E, aq.cpu().numpy(), asc.cpu().numpy(), se[smp], stok.cpu().numpy()[smp])
    assert rel(one[smp], ref) < TOL
    with pytest.raises(izb.IzbError):
        izb.moe_gateup(Wgu, None, aq, asc, tiles, max_tiles, 8, stok, Sn)
    assert izb.device_status(0) == 0
    for W in (Wg, Wu, Wgu):
        W.close()


def test_store_mode_3_needs_the_interleaved_weight(izb, torch):
    qt, F, K = 12, 128, 512
    w = S.make_weight(qt, F, K, 61)
    W = izb.Weight(qt, w, F, K)
    aq, asc, _ = O.quantize_act(S.make_act(16, K, 62), Mp=16)
    with pytest.raises(izb.IzbError):
        izb.gemm(W, dev(torch, aq), dev(torch, asc), acc=3)
    with pytest.raises(izb.IzbError):
        izb.gateup_weight(qt, w[:96], w[:96], 96, K)  # F % 64
    with pytest.raises(izb.IzbError):
        izb.gateup_weight(14, S.make_weight(14, F, K, 63), S.make_weight(14, F, K, 64), F, K)  # Q6_K: not a tensor-core type
    Wgu = izb.gateup_weight(qt, w, w, F, K)
    with pytest.raises(izb.IzbError):
        izb.matmul(Wgu, dev(torch, aq), dev(torch, asc), 2, acc=3)  # GEMV rows: no fused store
    W.close()
    Wgu.close()


@pytest.mark.parametrize("qt", [12, 8])
@pytest.mark.parametrize("T,N,K", [(200, 384, 1024), (40, 256, 512), (1024, 128, 2048), (5, 256, 512)])
def test_quant_matmul_is_the_two_calls_bit_for_bit(izb, torch, qt, T, N, K):
    """izb_quant_matmul (quantiser fused with the GEMM's pre-pass) against izb_quantize_act + izb_matmul: the int8 rows, the
    scales and the outputs are identical, for row counts that are not multiples of the tile and for the GEMV row counts
    (where it is the two calls)."""
    w = S.make_weight(qt, N, K, 70 + qt + N)
    W = izb.Weight(qt, w, N, K)
    x = S.make_act(T, K, 71 + T)
    x[0, :32] = 0.0                      # a zero block
    x[min(T - 1, 3), 32:64] = 1e-42      # denormals: 127 / amax overflows
    Mp = izb.pad_rows(T)
    dx = dev(torch, x)
    aq, asc, _ = izb.quantize_act(dx, Mp=Mp)
    ref = izb.matmul(W, aq, asc, T)
    out = torch.full((Mp, N + 16), float("nan"), dtype=torch.float32, device="cuda")
    _, aq2, asc2 = izb.quant_matmul(W, dx, T, Mp, out=out, c_off=8)
    assert (aq2.cpu().numpy() == aq.cpu().numpy()).all()
    assert (bits(asc2.cpu().numpy()) == bits(asc.cpu().numpy())).all()
    got, rows = out.cpu().numpy(), (Mp if T > 8 else T)
    assert (bits(got[:rows, 8:N + 8]) == bits(ref.cpu().numpy()[:rows])).all()
    assert np.isnan(got[:, :8]).all() and np.isnan(got[:, N + 8:]).all()
    oq, osc, _ = O.quantize_act(x, Mp=Mp)
    assert (aq2.cpu().numpy() == oq).all() and (bits(asc2.cpu().numpy()) == bits(osc)).all()
    assert rel(got[:T, 8:N + 8], O.matmul(qt, w, K, oq, osc, T, "f64")) < TOL
    # a padded row count far beyond the tiles the GEMM reads, and the store modes
    if T > 8:
        big = Mp + 256
        o2, aq3, asc3 = izb.quant_matmul(W, dx, T, big)
        assert (aq3.cpu().numpy()[:Mp] == oq).all() and not aq3.cpu().numpy()[Mp:].any()
        assert (bits(o2.cpu().numpy()[:T]) == bits(ref.cpu().numpy()[:T])).all()
        acc1 = ref.clone()
        izb.quant_matmul(W, dx, T, Mp, out=acc1, acc=1)
        two = ref.clone()
        izb.matmul(W, aq, asc, T, out=two, acc=1)
        assert (bits(acc1.cpu().numpy()[:T]) == bits(two.cpu().numpy()[:T])).all()
    assert izb.device_status(0) == 0
    W.close()
