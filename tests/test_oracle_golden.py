"""The CPU oracle (oracle/izb_oracle.c) against vectors produced by the reference's own code (tests/golden/, made by
tests/golden/make_golden.py) and, when oracle/_ref is present, against that code live."""
import os
import tempfile

import numpy as np
import pytest

from arcinferzero_b200 import synth as S
from oracle import oracle as O


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def test_quantize_matches_reference_vectors(golden_dir):
    g = np.load(os.path.join(golden_dir, "quantize.npz"))
    aq, asc, absum = O.quantize_act(g["x"])
    assert (aq == g["aq"]).all()
    assert (bits(asc) == bits(g["asc"])).all()
    assert (absum == g["absum"]).all()


def test_quantize_padding_rows_are_zero(golden_dir):
    g = np.load(os.path.join(golden_dir, "quantize.npz"))
    aq, asc, absum = O.quantize_act(g["x"], Mp=16)
    assert (aq[:9] == g["aq"]).all() and (aq[9:] == 0).all()
    assert (bits(asc[:, :9]) == bits(g["asc"])).all() and (asc[:, 9:] == 0).all()
    assert (absum[:, 9:] == 0).all()


def test_decode_and_dequant_match_reference_vectors(golden_dir):
    g = np.load(os.path.join(golden_dir, "decode.npz"))
    i = 0
    for n in range(6):
        for s in range(2):
            d, dmin, sc, mn, q = O.decode_q4k_sb(g["w4"][n, 144 * s:144 * (s + 1)])
            assert np.float32(d) == g["q4_d"][i] and np.float32(dmin) == g["q4_dmin"][i]
            assert (sc == g["q4_sc"][i]).all() and (mn == g["q4_mn"][i]).all() and (q == g["q4_q"][i]).all()
            d8, q8 = O.decode_q8_0_sb(g["w8"][n, 272 * s:272 * (s + 1)])
            assert (bits(d8) == bits(g["q8_d"][i])).all() and (q8 == g["q8_q"][i]).all()
            i += 1
    assert (bits(O.dequant_rows(12, g["w4"], 512)) == bits(g["deq4"])).all()
    assert (bits(O.dequant_rows(8, g["w8"], 512)) == bits(g["deq8"])).all()


def test_fp16_conversions_match_reference_vectors(golden_dir):
    g = np.load(os.path.join(golden_dir, "fp16.npz"))
    L = O.lib()
    got = np.array([L.orc_fp16_to_f32(h) for h in range(65536)], np.float32)
    same = bits(got) == g["to_f32"]
    nan = np.isnan(got)
    assert (same | nan).all() and (np.isnan(g["to_f32"].view(np.float32)) == nan).all()
    assert (np.array([L.orc_f32_to_fp16(float(v)) for v in g["xs"]], np.uint16) == g["to_f16"]).all()
    # numpy's float16 agrees with the reference's conversion (the generator relies on it)
    assert (g["xs"].astype(np.float16).view(np.uint16) == g["to_f16"]).all()
    assert (bits(np.arange(65536, dtype=np.uint32).astype(np.uint16).view(np.float16).astype(np.float32))[~nan]
            == g["to_f32"][~nan]).all()


def test_f64_order_is_ref_forward_matmul(golden_dir):
    """orc_matmul_f64 == tools/ref_forward.cpp matmul() bit for bit; the two kernel orders agree with it to ~1e-7."""
    g = np.load(os.path.join(golden_dir, "forward.npz"))
    d = np.load(os.path.join(golden_dir, "decode.npz"))
    aq, asc, _ = O.quantize_act(g["x"])
    for qt, w, y in ((12, d["w4"], g["y4"]), (8, d["w8"], g["y8"])):
        assert (bits(O.matmul(qt, w, 512, aq, asc, 5, "f64")) == bits(y)).all()
        for order in ("gemm", "gemv"):
            err = np.abs(O.matmul(qt, w, 512, aq, asc, 5, order) - y).max() / np.abs(y).max()
            assert err < 1e-6, (qt, order, err)


def test_pack_q4k_round_trip():
    rng = np.random.default_rng(7)
    R = 64
    d = rng.uniform(0, 0.01, R).astype(np.float16)
    dmin = rng.uniform(0, 0.01, R).astype(np.float16)
    sc = rng.integers(0, 64, (R, 8), dtype=np.uint8)
    mn = rng.integers(0, 64, (R, 8), dtype=np.uint8)
    q = rng.integers(0, 16, (R, 256), dtype=np.uint8)
    p = S.pack_q4k(d, dmin, sc, mn, q)
    for r in range(R):
        dd, dm, s2, m2, q2 = O.decode_q4k_sb(p[r])
        assert np.float32(dd) == np.float32(d[r]) and np.float32(dm) == np.float32(dmin[r])
        assert (s2 == sc[r]).all() and (m2 == mn[r]).all() and (q2 == q[r]).all()
        out = np.zeros(144, np.uint8)
        O.lib().orc_q4k_pack_sb(int(d[r:r + 1].view(np.uint16)[0]), int(dmin[r:r + 1].view(np.uint16)[0]),
                                sc[r].ctypes.data, mn[r].ctypes.data, q[r].ctypes.data, out.ctypes.data)
        assert (out == p[r]).all()


def test_block_dots_are_the_sum_of_products():
    x = S.make_act(3, 512, 21)
    aq, asc, absum = O.quantize_act(x)
    for qt in (12, 8):
        w = S.make_weight(qt, 5, 512, 22 + qt)
        dots, asum = O.block_dots(qt, w, 512, aq)
        for n in range(5):
            qs = []
            for s in range(2):
                qs.append(O.decode_q4k_sb(w[n, 144 * s:144 * s + 144])[4] if qt == 12 else O.decode_q8_0_sb(w[n, 272 * s:272 * s + 272])[1])
            qv = np.concatenate(qs).astype(np.int64)
            want = (aq.astype(np.int64) * qv[None, :]).reshape(3, 16, 32).sum(-1)
            assert (dots[:, n, :] == want).all()
        assert (asum == aq.astype(np.int64).reshape(3, 16, 32).sum(-1)).all()
        assert (absum.astype(np.int64).reshape(16, 2, 3).sum(1).T == asum).all()


@pytest.mark.skipif(O.ref() is None, reason="oracle/_ref not built (reference sources absent)")
def test_live_reference_agrees_on_fresh_inputs():
    x = S.make_act(11, 1024, 99)
    aq, asc, absum = O.quantize_act(x)
    raq, rasc, rab = O.ref_quantize_act(x)
    assert (aq == raq).all() and (bits(asc) == bits(rasc)).all() and (absum == rab).all()
    for qt in (12, 8):
        w = S.make_weight(qt, 17, 1024, 100 + qt)
        assert (bits(O.dequant_rows(qt, w, 1024)) == bits(O.ref_dequant_rows(qt, w, 1024))).all()
        with tempfile.TemporaryDirectory() as d:
            p = os.path.join(d, "t.gguf")
            S.write_gguf(p, {"w": (qt, w, 17, 1024)})
            y = O.ref_forward_matmul(p, "w", x, 17)
        assert (bits(O.matmul(qt, w, 1024, aq, asc, 11, "f64")) == bits(y)).all()


def test_store_modes():
    x = S.make_act(4, 256, 5)
    aq, asc, _ = O.quantize_act(x)
    w = S.make_weight(12, 8, 256, 6)
    base = O.matmul(12, w, 256, aq, asc, 4, "gemm")
    c0 = np.random.default_rng(1).standard_normal((4, 20)).astype(np.float32)
    add = O.matmul(12, w, 256, aq, asc, 4, "gemm", C_in=c0, ldc=20, c_off=3, acc=1)
    assert (bits(add[:, 3:11]) == bits(base + c0[:, 3:11])).all()
    assert (bits(add[:, :3]) == bits(c0[:, :3])).all() and (bits(add[:, 11:]) == bits(c0[:, 11:])).all()
    sw = O.matmul(12, w, 256, aq, asc, 4, "gemm", C_in=c0, ldc=20, c_off=3, acc=2)
    g = c0[:, 3:11]
    want = base * (g / (np.float32(1) + np.exp(-g, dtype=np.float32)))
    assert np.abs(sw[:, 3:11] - want).max() <= 1e-5 * np.abs(want).max()


def test_tp_range_properties():
    for total, unit in ((17408, 256), (8, 1), (151936, 16), (5120, 256)):
        for N in (1, 2, 3, 4, 8):
            rs = [O.tp_range(total, unit, N, r) for r in range(N)]
            assert rs[0][0] == 0 and rs[-1][1] == total // unit * unit
            for a, b in zip(rs, rs[1:]):
                assert a[1] == b[0]
            sizes = [e - b for b, e in rs]
            assert all(s % unit == 0 for s in sizes) and sizes == sorted(sizes, reverse=True)
            assert max(sizes) - min(sizes) <= unit


def test_rmsnorm_quant_matches_reference_rows(golden_dir):
    """The restated rmsnorm_quant (zero/kernels/ops.cl:104-141, f32 sum in a defined order) against
    tools/ref_forward.cpp's rmsnorm (double sum): the normalised rows agree to float rounding, the quantised rows are the
    quantiser applied to them."""
    g = np.load(os.path.join(golden_dir, "rmsnorm.npz"))
    y, aq, asc, absum = O.rmsnorm_quant(g["x"], g["w"], float(g["eps"]), Mp=16)
    err = np.max(np.abs(y.astype(np.float64) - g["y"].astype(np.float64))) / np.max(np.abs(g["y"]))
    assert err <= 2e-6, err
    assert (y[3] == 0).all()  # the all-zero row stays zero (r = 1/sqrt(eps) is finite)
    raq, rasc, rabsum = O.quantize_act(y, Mp=16)
    assert (aq == raq).all() and (bits(asc) == bits(rasc)).all() and (absum == rabsum).all()
    if O.ref() is not None:
        live = O.ref_rmsnorm(g["x"], g["w"], float(g["eps"]))
        assert (bits(live) == bits(g["y"])).all()


def test_add_norm_quant_composes_the_pinned_pieces(golden_dir):
    """add_norm_quant (zero/kernels/ops_attn_g.cl:617-680) restated: with x = 0 and s = 1 its first step is rmsnorm(t) * w,
    which must agree with tools/ref_forward.cpp's rmsnorm rows; its quantised output is the quantiser applied to the
    (optionally normalised) new row."""
    g = np.load(os.path.join(golden_dir, "rmsnorm.npz"))
    t, w, eps = g["x"], g["w"], float(g["eps"])
    xn, aq, asc, absum = O.add_norm_quant(np.zeros_like(t), t, w, eps, 1.0, None)
    err = np.max(np.abs(xn.astype(np.float64) - g["y"].astype(np.float64))) / np.max(np.abs(g["y"]))
    assert err <= 2e-6, err
    raq, rasc, rabsum = O.quantize_act(xn)
    assert (aq == raq).all() and (bits(asc) == bits(rasc)).all() and (absum == rabsum).all()
    # with the second norm the quantised row is rmsnorm_quant of the new x, up to the two kernels' different (both defined)
    # orders of the sum of squares: scales within float rounding, int8 values within one step
    xn2, aq2, asc2, _ = O.add_norm_quant(np.ones_like(t), t, w, eps, 0.5, w)
    y2, raq2, rasc2, _ = O.rmsnorm_quant(xn2, w, eps)
    assert np.max(np.abs(aq2.astype(np.int32) - raq2.astype(np.int32))) <= 1
    assert np.allclose(asc2, rasc2, rtol=1e-6, atol=0)


def test_softcap_rows_oracle_against_the_formula_in_double():
    """cap * tanh(v / cap) (tools/ref_forward.cpp:1479-1483 is the reference's CPU form, zero/kernels/ops_attn_g.cl:724 the
    device form): the oracle's f32 result against the same expression in f64; untouched outside the rows and columns."""
    rng = np.random.default_rng(3)
    c = (rng.standard_normal((5, 300)) * 40).astype(np.float32)
    c[0, :6] = [0.0, -0.0, 1e-30, -1e4, 1e4, 29.999]
    for cap, rows, N, off in ((30.0, 3, 256, 8), (50.0, 5, 300, 0), (0.5, 1, 7, 3)):
        out = O.softcap_rows(c, rows, N, cap, off)
        ref = c.astype(np.float64)
        ref[:rows, off:off + N] = cap * np.tanh(ref[:rows, off:off + N] / cap)
        assert np.abs(out - ref).max() <= 4e-7 * cap
        keep = np.ones_like(c, dtype=bool)
        keep[:rows, off:off + N] = False
        assert (out[keep] == c[keep]).all()


def test_moe_routing_matches_reference_rule_vectors(golden_dir):
    """moe.npz: ids and weights by the rule of tools/ref_forward.cpp:1668-1676 (stable descending sort, double exp,
    renormalised over the choice): the restated moe_route (zero/kernels/moe.cl:50-89) must choose the same experts in the
    same order (ties, +0 / -0 included) and weigh them within 1e-6."""
    g = np.load(os.path.join(golden_dir, "moe.npz"))
    ids, wts, counts = O.moe_route(g["logits"], g["ids"].shape[1])
    assert (ids == g["ids"]).all(), np.argwhere(ids != g["ids"])[:5]
    assert np.abs(wts.astype(np.float64) - g["wts"]).max() <= 1e-6
    assert (counts == np.bincount(g["ids"].ravel(), minlength=g["logits"].shape[1])).all()


def test_moe_expert_projections_match_reference_vectors(golden_dir):
    """moe.npz: gate / up / down of routed experts from the reference's expert_mv() (tools/ref_forward.cpp:333, inputs
    rounded to int8 per 32, dequantised weights, double sums) and its silu() (:321).  The restated integer path
    (decode_moe.cl moe_gateup_q / moe_down_q) must agree within 1e-5 of max|ref|, stage by stage: the down projection is
    fed the golden h, as the reference fed it."""
    g = np.load(os.path.join(golden_dir, "moe.npz"))
    E, F = g["x"].shape[1], g["g"].shape[1]
    pairs = g["pairs"]
    tok, exp_ = np.ascontiguousarray(pairs[:, 0]), np.ascontiguousarray(pairs[:, 1])
    aq, asc, _ = O.quantize_act(g["x"])
    h, gg, uu = O.moe_gateup(12, g["wg"], g["wu"], F, E, aq, asc, exp_, tok, want_gu=True)
    for got, ref, name in ((gg, g["g"], "gate"), (uu, g["u"], "up"), (h, g["h"], "h")):
        assert np.abs(got.astype(np.float64) - ref).max() <= 1e-5 * np.abs(ref).max(), name
    hq, hsc, _ = O.quantize_act(g["h"])
    one = np.ones(len(pairs), np.float32)
    y = O.moe_down(12, g["wd"], E, F, hq, hsc, exp_, one)
    assert np.abs(y.astype(np.float64) - g["dn"]).max() <= 1e-5 * np.abs(g["dn"]).max()


def test_moe_golden_is_what_the_live_reference_computes(golden_dir):
    if O.ref() is None:
        pytest.skip("oracle/_ref not built (needs the reference sources)")
    g = np.load(os.path.join(golden_dir, "moe.npz"))
    E, F = g["x"].shape[1], g["g"].shape[1]
    with tempfile.TemporaryDirectory() as d:
        p = os.path.join(d, "moe.gguf")
        S.write_gguf(p, {"blk.0.ffn_gate_exps.weight": (12, g["wg"], F, E, 3), "blk.0.ffn_down_exps.weight": (12, g["wd"], E, F, 3)})
        t, e = (int(v) for v in g["pairs"][1])
        assert (bits(O.ref_expert_mv(p, "blk.0.ffn_gate_exps", e, F, E, g["x"][t])) == bits(g["g"][1])).all()
        assert (bits(O.ref_expert_mv(p, "blk.0.ffn_down_exps", e, E, F, g["h"][1])) == bits(g["dn"][1])).all()
    assert (bits(O.ref_silu(g["g"][1]) * g["u"][1]) == bits(g["h"][1])).all()


def test_q8_0_regrouped_device_form_matches_reference_vectors(golden_dir):
    """rawsb.npz: gpu_raw_sb (src/quants.h:728-751) of the Q8_0 superblocks of decode.npz: eight fp16 scales, then the
    eight blocks' int8 values.  The restated regrouping (what the weight loader's kernel does on the device) in numpy."""
    g = np.load(os.path.join(golden_dir, "decode.npz"))
    raw = np.load(os.path.join(golden_dir, "rawsb.npz"))["raw8"]
    i = 0
    for n in range(6):
        for s in range(2):
            blocks = g["w8"][n, 272 * s:272 * (s + 1)].reshape(8, 34)
            want = np.concatenate([blocks[:, :2].reshape(-1), blocks[:, 2:].reshape(-1)])
            assert (raw[i][:272] == want).all()
            i += 1


TYPES = (("q4_0", 2), ("q5_k", 13), ("q6_k", 14), ("iq4_xs", 23))


@pytest.mark.parametrize("name,qt", TYPES)
def test_further_weight_types_match_reference_vectors(golden_dir, name, qt):
    """types.npz: decode_sb's generic view (wd, wdmin, a scale and a min per 16 elements, quants with their offset removed),
    dequant_row and tools/ref_forward.cpp's matmul() for Q4_0, Q5_K, Q6_K and IQ4_XS rows: the restated decoders bit for
    bit, the restated integer paths (both summation orders and the f64 model) within 1e-5 of max|ref|."""
    g = np.load(os.path.join(golden_dir, "types.npz"))
    w, K = g["w_" + name], 512
    assert (bits(O.dequant_rows(qt, w, K)) == bits(g["deq_" + name])).all()
    if qt != 2:
        sbb = S.sb_bytes(qt)
        i = 0
        for n in range(w.shape[0]):
            for s in range(K // 256):
                wd, wdmin, wsc, wmn, has_min, q = O.decode_generic_sb(qt, w[n, sbb * s:sbb * (s + 1)])
                assert np.float32(wd) == g["wd_" + name][i] and np.float32(wdmin) == g["wdmin_" + name][i]
                assert (wsc == g["wsc_" + name][i]).all() and (wmn == g["wmn_" + name][i]).all() and (q == g["q_" + name][i]).all()
                i += 1
    else:
        # Q4_0 rewritten as Q8_0 blocks dequantises to the same floats
        assert (bits(O.dequant_rows(8, O.q4_0_as_q8_0(w), K)) == bits(g["deq_" + name])).all()
    aq, asc, _ = O.quantize_act(g["x"])
    y = g["y_" + name]
    for order in ("f64", "gemv", "gemm"):
        got = O.matmul(qt, w, K, aq, asc, g["x"].shape[0], order)
        assert np.abs(got.astype(np.float64) - y).max() <= 1e-5 * np.abs(y).max(), (name, order)
    # the f64 model IS the reference's arithmetic
    assert (bits(O.matmul(qt, w, K, aq, asc, g["x"].shape[0], "f64")) == bits(y)).all()
    # block dots: the integer sums over 32 of a * (q - offset)
    dots, asum = O.block_dots(qt, w, K, aq)
    deq_int = None
    if qt != 2:
        qs = g["q_" + name].reshape(w.shape[0], K).astype(np.int64)
        deq_int = np.einsum("mbk,nbk->mnb", aq.astype(np.int64).reshape(-1, K // 32, 32), qs.reshape(-1, K // 32, 32))
        assert (dots == deq_int).all()
