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
