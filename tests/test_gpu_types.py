"""Further GGUF weight types on the GPU: Q4_0 (held as Q8_0), Q5_K, Q6_K, IQ4_XS (held in the reference's generic view with a
scale and a min per 16 elements).  Per-block integer dots bit-exact against the oracle, f32 outputs of the GEMV (1..8
rows) and the GEMM within 1e-5 of max|ref| against both summation orders and the f64 model (the oracle itself is pinned
to the reference's decode_sb / dequant_row / matmul through tests/golden/types.npz)."""
import numpy as np
import pytest

from arcinferzero_b200 import synth as S
from oracle import oracle as O

pytestmark = pytest.mark.gpu
TOL = 1e-5
TYPES = [2, 13, 14, 23]


@pytest.fixture(scope="module")
def torch():
    import torch as t
    assert t.cuda.is_available()
    return t


def rel(got, ref):
    return float(np.abs(got.astype(np.float64) - ref.astype(np.float64)).max() / np.abs(ref).max())


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def edge_rows(qt, w, K):
    """Plant the extreme field values of each format in the first rows."""
    w = w.copy()
    if qt == 14:
        w[0, 192:208] = 0x80                    # every scale -128
        w[0, 0:192] = 0                         # every quant -32: the largest |scale * quant| = 4096
        w[1, 0:192] = 0xFF                      # every quant 31
    if qt == 13:
        w[0, 4:176] = 0xFF                      # scales / mins 63, quants 31
    if qt == 23:
        w[0, 2:136] = 0xFF                      # scale 63 - 32 = 31, codebook value 113
        w[1, 2:8] = 0                           # scale -32
        w[1, 8:136] = 0                         # codebook value -127
    if qt == 2:
        w[0, 2:18] = 0                          # every quant -8
    return w


@pytest.mark.parametrize("qt", TYPES)
def test_block_dots_and_device_form(izb, torch, qt):
    N, K, M = 70, 768, 37
    w = edge_rows(qt, S.make_weight(qt, N, K, 500 + qt), K)
    x = S.make_act(M, K, 600 + qt)
    x[0, :] = 1.0
    x[1, :] = -1.0
    aq, _, _ = O.quantize_act(x, Mp=M)
    W = izb.Weight(qt, w, N, K)
    # the device form is the host decoder's output (Q4_0: regrouped like any Q8_0)
    if qt != 2:
        assert (W.download() == izb.weight_decode_host(qt, w, K).reshape(-1)).all()
    dots = izb.block_dots(W, dev(torch, aq), M, impl=izb.GEMM_CORE).cpu().numpy()
    ref, _ = O.block_dots(qt, w, K, aq)
    assert (dots == ref).all(), np.argwhere(dots != ref)[:5]
    W.close()


@pytest.mark.parametrize("qt", TYPES)
@pytest.mark.parametrize("K", [512, 5120])
def test_gemv_1_to_8_rows(izb, torch, qt, K):
    N = 203
    w = edge_rows(qt, S.make_weight(qt, N, K, 700 + qt + K), K)
    W = izb.Weight(qt, w, N, K)
    x = S.make_act(8, K, 800 + qt)
    aq, asc, _ = O.quantize_act(x, Mp=16)
    daq, dasc = dev(torch, aq), dev(torch, asc)
    for T in range(1, 9):
        out = torch.full((T + 1, N + 8), float("nan"), dtype=torch.float32, device="cuda")
        izb.matmul(W, daq, dasc, T, out=out, c_off=4)
        got = out.cpu().numpy()
        assert np.isnan(got[:, :4]).all() and np.isnan(got[:, N + 4:]).all() and np.isnan(got[T:]).all()
        for order in ("gemv", "f64"):
            assert rel(got[:T, 4:N + 4], O.matmul(qt, w, K, aq, asc, T, order)) < TOL, (T, order)
    # accumulate mode
    base = torch.ones((2, N), dtype=torch.float32, device="cuda")
    izb.gemv(W, daq, dasc, 2, out=base, acc=1)
    assert rel(base.cpu().numpy() - 1.0, O.matmul(qt, w, K, aq, asc, 2, "gemv")) < 1e-4
    assert izb.device_status(0) == 0
    W.close()


@pytest.mark.parametrize("qt", TYPES)
def test_gemm_and_store_modes(izb, torch, qt):
    M, N, K = 130, 208, 1024     # (the GEMM keeps the reference's shape rule: N % 16 == 0)
    w = edge_rows(qt, S.make_weight(qt, N, K, 900 + qt), K)
    W = izb.Weight(qt, w, N, K)
    Mp = izb.pad_rows(M)
    aq, asc, _ = O.quantize_act(S.make_act(M, K, 901), Mp=Mp)
    daq, dasc = dev(torch, aq), dev(torch, asc)
    out = torch.full((Mp, N + 8), float("nan"), dtype=torch.float32, device="cuda")
    izb.matmul(W, daq, dasc, M, out=out, c_off=4)     # T > 8: the GEMM over Mp rows
    got = out.cpu().numpy()
    assert np.isnan(got[:, :4]).all() and np.isnan(got[:, N + 4:]).all()
    for order in ("gemm", "gemv", "f64"):
        assert rel(got[:M, 4:N + 4], O.matmul(qt, w, K, aq, asc, M, order)) < TOL, order
    c0 = np.random.default_rng(9).standard_normal((Mp, N)).astype(np.float32)
    for acc in (1, 2):
        o2 = dev(torch, c0)
        izb.gemm(W, daq, dasc, M=M, out=o2, acc=acc)
        assert rel(o2.cpu().numpy()[:M], O.matmul(qt, w, K, aq, asc, M, "gemm", C_in=c0[:M], acc=acc)) < TOL
    assert izb.device_status(0) == 0
    W.close()


def test_q4_0_takes_the_tensor_core_gemm(izb, torch):
    M, N, K = 200, 256, 2048
    w = S.make_weight(2, N, K, 33)
    W = izb.Weight(2, w, N, K)
    aq, asc, _ = O.quantize_act(S.make_act(M, K, 34), Mp=256)
    out = izb.gemm(W, dev(torch, aq), dev(torch, asc), M=M, impl=izb.GEMM_TC).cpu().numpy()[:M]
    assert rel(out, O.matmul(2, w, K, aq, asc, M, "f64")) < TOL
    dots = izb.block_dots(W, dev(torch, aq), M, impl=izb.GEMM_TC).cpu().numpy()
    assert (dots == O.block_dots(2, w, K, aq[:M])[0]).all()
    assert izb.device_status(0) == 0
    W.close()


def test_entry_points_that_do_not_take_the_generic_form_say_so(izb, torch):
    N, K = 128, 512
    W = izb.Weight(14, S.make_weight(14, N, K, 3), N, K)
    aq = torch.zeros((128, K), dtype=torch.int8, device="cuda")
    asc = torch.zeros((K // 32, 128), dtype=torch.float32, device="cuda")
    for call in (lambda: izb.gemm(W, aq, asc, impl=izb.GEMM_TC), lambda: izb.gemm_noalloc(W, aq, asc),
                 lambda: izb.block_dots(W, aq, 128, impl=izb.GEMM_TC)):
        with pytest.raises(izb.IzbError) as e:
            call()
        assert e.value.status == -3
    with pytest.raises(izb.IzbError) as e:
        izb.Weight(10, np.zeros((4, 84), np.uint8), 4, 256)   # Q2_K: not taken
    assert e.value.status == -3
    W.close()


@pytest.mark.parametrize("qt", [8, 12, 2, 14])
def test_stacked_weight_is_the_parts_side_by_side(izb, torch, qt):
    """Several tensors loaded as one weight (the reference's load_w_stack for Q | K | V and gate | up): one GEMV / GEMM over
    the stack writes bit for bit what the separate launches write, side by side."""
    K, rows = 1024, [96, 208, 64]
    parts = [S.make_weight(qt, n, K, 900 + qt + n) for n in rows]
    Wst = izb.stacked_weight(qt, parts, K)
    assert (Wst.N, Wst.K) == (sum(rows), K)
    Ws = [izb.Weight(qt, p, n, K) for p, n in zip(parts, rows)]
    assert (Wst.download() == np.concatenate([W.download() for W in Ws])).all()
    x = S.make_act(48, K, 901)
    aq, asc, _ = O.quantize_act(x, Mp=48)
    daq, dasc = dev(torch, aq), dev(torch, asc)
    for T in (1, 2, 48):
        got = izb.matmul(Wst, daq, dasc, T).cpu().numpy()[:T]
        off = 0
        for W, p, n in zip(Ws, parts, rows):
            one = izb.matmul(W, daq, dasc, T).cpu().numpy()[:T]
            if T <= 8:
                assert (got[:, off:off + n] == one).all(), (T, off)
            assert rel(got[:, off:off + n], O.matmul(qt, p, K, aq, asc, T, "f64")) < TOL
            off += n
    with pytest.raises(ValueError):
        izb.stacked_weight(qt, [parts[0], parts[1][:, :-16]], K)
    assert izb.device_status(0) == 0
    for W in Ws + [Wst]:
        W.close()
