"""GPU parity at the stated sizes of the benchmark configurations that the other files only cover at reduced size, the
time-out path of the tensor-core GEMM's bounded waits, the device form of Q8_0 weights, and the library's per-device
state (two GPUs driven by two threads of one process; no allocation after izb_reserve).

Bars as everywhere: routing ids, counts, slots, int8 rows and scales exact; f32 outputs within 1e-5 of max|ref| (the
reference's error form, bench/gemv_bench.cpp:199-214), stage by stage with teacher forcing."""
import os
import threading

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


def rel(got, ref):
    return float(np.abs(got.astype(np.float64) - ref.astype(np.float64)).max() / np.abs(ref).max())


def dev(torch, a, device=0):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda(device)


def test_config4_moe_full_size(izb, torch):
    """BASELINE config 4 in full: 4096 tokens, 128 experts, top-8, hidden 2048, expert FFN 768, Q4_K.  The grouped
    tensor-core GEMM (tiles of 128 slots) against the per-tile kernels (tiles of 8 slots, the reference's structure,
    zero/kernels/decode_moe.cl:92-449) on EVERY slot, both against the oracle on sampled slots, and the routing / sort
    against the oracle on everything."""
    T, E, F, NE, NU, qt = 4096, 2048, 768, 128, 8, 12
    seed = 20261125
    wg, wu = S.make_weight(qt, NE * F, E, seed + 11), S.make_weight(qt, NE * F, E, seed + 12)
    wd = S.make_weight(qt, NE * E, F, seed + 13)
    Wg, Wu, Wd = izb.Weight(qt, wg, F, E, n_mats=NE), izb.Weight(qt, wu, F, E, n_mats=NE), izb.Weight(qt, wd, E, F, n_mats=NE)
    x = S.make_act(T, E, seed + 14)
    lg = np.random.default_rng(seed + 9).standard_normal((T, NE), dtype=np.float32)
    lg[7, 40:48] = 9.0  # an eight-way tie
    aq, asc, _ = izb.quantize_act(dev(torch, x), Mp=T)
    ids, wts, counts = izb.moe_route(dev(torch, lg), NU)
    rid, rwt, rcnt = O.moe_route(lg, NU)
    assert (ids.cpu().numpy() == rid).all() and (counts.cpu().numpy() == rcnt).all()
    assert np.abs(wts.cpu().numpy() - rwt).max() <= 1e-6
    Sn = T * NU
    sorted_ = {}
    for TM in (128, 8):
        offs, tiles, max_tiles, stok, swt, inv = izb.moe_sort(ids, wts, counts, TM)
        roffs, rtiles, rstok, rswt, rinv = O.moe_sort(rid, wts.cpu().numpy(), rcnt, TM)
        nt = int(tiles[0].item())
        assert nt == rtiles[0] and (tiles.cpu().numpy()[:1 + 3 * nt] == rtiles[:1 + 3 * nt]).all()
        assert (offs.cpu().numpy() == roffs).all() and (stok.cpu().numpy() == rstok).all() and (inv.cpu().numpy() == rinv).all()
        assert (swt.cpu().numpy().view(np.uint32) == rswt.view(np.uint32)).all()
        sorted_[TM] = (offs, tiles, max_tiles, stok, swt, inv)
    se = O.slot_experts(sorted_[128][0].cpu().numpy())
    stok_h, swt_h = sorted_[128][3].cpu().numpy(), sorted_[128][4].cpu().numpy()
    # ---- gate / up with the SwiGLU store
    h = {}
    for TM in (128, 8):
        _, tiles, max_tiles, stok, _, _ = sorted_[TM]
        h[TM] = izb.moe_gateup(Wg, Wu, aq, asc, tiles, max_tiles, TM, stok, Sn)
    assert izb.device_status(0) == 0
    err = float((h[128] - h[8]).abs().max() / h[8].abs().max())
    assert err < TOL, ("grouped vs per-tile gate/up", err)
    # sampled slots: first and last slot of several experts (tile edges), a few in the middle
    offs_h = sorted_[128][0].cpu().numpy()
    sample = sorted({int(s) for e in (0, 1, 63, 127) for s in (offs_h[e], offs_h[e + 1] - 1, (offs_h[e] + offs_h[e + 1]) // 2)}
                    | {int(v) for v in np.random.default_rng(5).integers(0, Sn, 52)})
    sample = np.array(sample, np.int64)
    aq_h, asc_h = aq.cpu().numpy(), asc.cpu().numpy()
    rh = O.moe_gateup(qt, wg, wu, F, E, aq_h, asc_h, se[sample], stok_h[sample])
    assert rel(h[128][sample].cpu().numpy(), rh) < TOL
    assert rel(h[8][sample].cpu().numpy(), rh) < TOL
    # ---- quantise h (teacher forcing: the oracle quantises the GPU's own h) and down, scaled by the router weight
    Sp = izb.pad_rows(Sn)
    hq, hsc, _ = izb.quantize_act(h[128], Mp=Sp)
    rq, rs, _ = O.quantize_act(h[128][sample].cpu().numpy())
    assert (hq[sample].cpu().numpy() == rq).all()
    assert (hsc[:, sample].cpu().numpy().view(np.uint32) == rs.view(np.uint32)).all()
    y = {}
    for TM in (128, 8):
        _, tiles, max_tiles, _, swt, _ = sorted_[TM]
        y[TM] = izb.moe_down(Wd, hq, hsc, tiles, max_tiles, TM, swt, Sn)
    assert izb.device_status(0) == 0
    err = float((y[128] - y[8]).abs().max() / y[8].abs().max())
    assert err < TOL, ("grouped vs per-tile down", err)
    ry = O.moe_down(qt, wd, E, F, rq, rs, se[sample], swt_h[sample])
    assert rel(y[128][sample].cpu().numpy(), ry) < TOL
    # ---- combine, in choice order: bit-exact against the oracle fed the GPU's y
    out = dev(torch, x).clone()
    izb.moe_combine(out, y[128], sorted_[128][5], NU)
    tok = np.arange(0, T, 97)
    ref = O.moe_combine(x, y[128].cpu().numpy(), sorted_[128][5].cpu().numpy(), NU)
    assert (out.cpu().numpy()[tok].view(np.uint32) == ref[tok].view(np.uint32)).all()
    for W in (Wg, Wu, Wd):
        W.close()


@pytest.mark.parametrize("T", [1, 2])
def test_config3_q8_0_output_head_full_size(izb, torch, T):
    """BASELINE config 3's Q8_0 head, 151936 x 5120, batch 1 and 2: ~2000 sampled weight rows (the first and last rows
    among them) against the f64 model and the reference's GEMV order; NaN-poisoned borders must stay NaN."""
    N, K, qt = 151936, 5120, 8
    w = S.make_weight(qt, N, K, 20261125 + N)
    W = izb.Weight(qt, w, N, K)
    x = S.make_act(T, K, 77 + T)
    aq, asc, _ = izb.quantize_act(dev(torch, x), Mp=16)
    out = torch.full((T + 1, N + 8), float("nan"), dtype=torch.float32, device="cuda")
    izb.gemv(W, aq, asc, T, out=out, c_off=4)
    assert izb.device_status(0) == 0
    got = out.cpu().numpy()
    assert np.isnan(got[:, :4]).all() and np.isnan(got[:, N + 4:]).all() and np.isnan(got[T:]).all()
    assert np.isfinite(got[:T, 4:N + 4]).all()
    rows = np.unique(np.concatenate([np.arange(0, 40), np.arange(N - 40, N), np.random.default_rng(3).integers(0, N, 1920)]))
    sub = np.ascontiguousarray(w[rows])
    aq_h, asc_h = aq.cpu().numpy(), asc.cpu().numpy()
    for order in ("f64", "gemv"):
        ref = O.matmul(qt, sub, K, aq_h, asc_h, T, order)
        assert rel(got[:T, 4:N + 4][:, rows], ref) < TOL, order
    W.close()


def test_bounded_wait_runs_out_and_the_next_gemm_is_correct(izb, torch):
    """The tensor-core GEMM's waits are bounded.  With the activation producer told to leave one operand stage out
    (izb_debug_wait_test) the MMA issuer's wait for that stage must give up: the kernel returns through its drain path,
    izb_device_status reports where it gave up, nothing hangs, and the very next GEMM is correct again."""
    M, N, K, qt = 256, 256, 1024, 12
    w = S.make_weight(qt, N, K, 91)
    aq, asc, _ = O.quantize_act(S.make_act(M, K, 92), Mp=M)
    W = izb.Weight(qt, w, N, K)
    daq, dasc = dev(torch, aq), dev(torch, asc)
    ref = O.matmul(qt, w, K, aq, asc, M, "gemm")
    good = izb.gemm(W, daq, dasc, impl=izb.GEMM_TC)
    assert rel(good.cpu().numpy(), ref) < TOL and izb.device_status(0) == 0
    out = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    izb.debug_wait_test(1 << 13, 7)   # stage 7 of the first tile of every CTA never arrives
    izb.gemm(W, daq, dasc, out=out, impl=izb.GEMM_TC)
    torch.cuda.synchronize()
    word = izb.device_status(0)
    E_MMA, E_EPI = 16, 32  # the MMA issuer's wait for the operand stage / the combine warps' wait for its accumulator
    assert word & (E_MMA | E_EPI), hex(word)
    assert izb.device_status(0) == 0          # read-and-clear
    assert torch.isnan(out).any()             # the tiles that gave up stored nothing
    again = izb.gemm(W, daq, dasc, impl=izb.GEMM_TC)
    assert rel(again.cpu().numpy(), ref) < TOL and izb.device_status(0) == 0
    W.close()


def test_q8_0_device_form_is_the_reference_raw_superblock(izb, torch, golden_dir):
    """The loader regroups GGUF Q8_0 blocks on the device; the result must be gpu_raw_sb's bytes (src/quants.h:728-751),
    as stored in tests/golden/rawsb.npz for the rows of decode.npz.  Q4_K superblocks are kept as they are."""
    g = np.load(os.path.join(golden_dir, "decode.npz"))
    raw = np.load(os.path.join(golden_dir, "rawsb.npz"))["raw8"]
    W8 = izb.Weight(8, g["w8"], 6, 512)
    got = W8.download().reshape(12, 272)
    assert (got == raw[:, :272]).all()
    W4 = izb.Weight(12, g["w4"], 6, 512)
    assert (W4.download() == g["w4"].reshape(-1)).all()
    W8.close()
    W4.close()


def test_reserve_then_calls_do_not_allocate(izb, torch):
    """After izb_reserve sized the arenas, GEMMs of growing size leave the device's free memory unchanged (no hidden
    cudaMalloc / cudaFree + device synchronisation inside izb_gemm)."""
    N, K, qt = 256, 2048, 12
    W = izb.Weight(qt, S.make_weight(qt, N, K, 5), N, K)
    izb.reserve(0, 2048, K)
    runs = []
    for M in (128, 640, 2048):
        aq = torch.zeros((M, K), dtype=torch.int8, device="cuda")
        asc = torch.ones((K // 32, M), dtype=torch.float32, device="cuda")
        out = torch.empty((M, N), dtype=torch.float32, device="cuda")
        runs.append((aq, asc, out))
    izb.gemm(W, runs[0][0], runs[0][1], out=runs[0][2], impl=izb.GEMM_TC)  # warm-up: the kernel's code is loaded
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    for aq, asc, out in runs:
        izb.gemm(W, aq, asc, out=out, impl=izb.GEMM_TC)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0
    assert izb.device_status(0) == 0
    W.close()


def test_two_devices_from_two_threads_of_one_process(izb, torch):
    """The reference drives its GPUs from one process, one thread per GPU (zero/mgpu/engine_tp.h:825).  Two threads, each
    bound to its own device, run the whole dispatch (GEMV, few-row GEMV, tensor-core GEMM, MoE tiles) at once; both must
    match the oracle, and a handle used with the wrong device current must be refused."""
    if torch.cuda.device_count() < 2:
        pytest.skip("one GPU visible")
    N, K, qt = 384, 2048, 12
    w = S.make_weight(qt, N, K, 11)
    x = S.make_act(200, K, 12)
    aq, asc, _ = O.quantize_act(x, Mp=256)
    refs = {T: O.matmul(qt, w, K, aq, asc, T, "f64") for T in (1, 3, 200)}
    errors = []

    def run(d):
        try:
            torch.cuda.set_device(d)
            W = izb.Weight(qt, w, N, K, device=d)
            daq, dasc = dev(torch, aq, d), dev(torch, asc, d)
            for _ in range(3):
                for T in (1, 3, 200):
                    got = izb.matmul(W, daq, dasc, T).cpu().numpy()[:T]
                    assert rel(got, refs[T]) < TOL, (d, T)
            assert izb.device_status(d) == 0
            W.close()
        except Exception as e:  # noqa: BLE001
            errors.append((d, repr(e)))

    th = [threading.Thread(target=run, args=(d,)) for d in (0, 1)]
    for t in th:
        t.start()
    for t in th:
        t.join()
    assert not errors, errors
    torch.cuda.set_device(1)
    W1 = izb.Weight(qt, w, N, K, device=1)
    torch.cuda.set_device(0)
    with pytest.raises(izb.IzbError) as e:
        izb.matmul(W1, dev(torch, aq, 0), dev(torch, asc, 0), 200)
    assert e.value.status == -1 and "device" in str(e.value)
    W1.close()


def test_measured_tensor_peaks_are_plausible(izb, torch):
    """The TMEM-resident tcgen05.mma loop behind the benchmark's "% of int8 tensor peak": kind::i8 must run about twice as
    fast as kind::f16, both far above anything CUDA cores reach, and no wait may give up."""
    f16, clk16 = izb.tensor_peak(0, 0, 2048, 2)
    i8, clk8 = izb.tensor_peak(0, 1, 2048, 2)
    assert izb.device_status(0) == 0
    assert 500.0 < f16 < 3000.0 and 1000.0 < i8 < 6000.0, (f16, i8)
    assert 1.5 < i8 / f16 < 2.5, (f16, i8)
    assert 50.0 < clk16 < 400.0 and 50.0 < clk8 < 400.0, (clk16, clk8)  # (128 clocks per 128 x 256 instruction at the full rate)
