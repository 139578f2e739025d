"""Generates tests/golden/*.npz from the REFERENCE's own code (oracle/_ref/libizb_ref.so, built by oracle/Makefile from
the reference sources in place).  Run where the reference sources exist:  python tests/golden/make_golden.py

What is stored (all inputs seeded; every array small):
  quantize.npz   x -> aq, asc, absum from quantize_act_cpu (src/quants.h:626), incl. zero blocks, ties and denormals
  decode.npz     random Q4_K / Q8_0 superblocks -> decode_sb fields (src/quants.h:89) and dequant_row (:519)
  fp16.npz       fp16_to_f32 over every 16-bit pattern, f32_to_fp16 over a seeded sample (src/quants.h:17-52)
  forward.npz    tools/ref_forward.cpp:251 matmul() outputs (REF_Q=all REF_QB=32) on small Q4_K / Q8_0 tensors
  rawsb.npz      gpu_raw_sb (src/quants.h:728) of Q8_0 superblocks: the regrouped form the weight loader must make
  rmsnorm.npz    tools/ref_forward.cpp:314 rmsnorm() rows (double-precision sum of squares)
  moe.npz        the reference's CPU mixture-of-experts block (tools/ref_forward.cpp:1660-1690): expert_mv() (:333) outputs of
                 the gate / up / down projections of routed experts, silu() (:321), and the routing of seeded logits.
                 expert_mv and silu are the reference's functions, called through oracle/_ref; the routing lines
                 (:1668-1676) sit inside its forward loop and cannot be called alone, so they are followed here step by
                 step in numpy: stable descending sort (ties keep the lower expert first), exp(l - l_max) in double,
                 normalised over the chosen NU, cast to float.

  types.npz      Q4_0, Q5_K, Q6_K, IQ4_XS rows: decode_sb in its generic view (src/quants.h:72-87), dequant_row, and
                 tools/ref_forward.cpp matmul() outputs on them

    python tests/golden/make_golden.py            # everything
    python tests/golden/make_golden.py moe        # only moe.npz (leaves the other files untouched)
    python tests/golden/make_golden.py types      # only types.npz
"""
import os
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from arcinferzero_b200 import synth as S  # noqa: E402
from oracle import oracle as O  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def make_moe():
    rng = np.random.default_rng(20261201)
    # ---- routing (tools/ref_forward.cpp:1668-1676): 128 experts, top 8, with planted ties
    T, NE, NU = 48, 128, 8
    lg = rng.standard_normal((T, NE), dtype=np.float32)
    lg[0, :] = 0.25                                   # every logit equal: experts 0..7 in order
    lg[1, 100:108] = lg[1].max() + np.float32(1.0)    # an eight-way tie at the top, high ids
    lg[2, [5, 90]] = lg[2].max() + np.float32(0.5)    # a two-way tie for the first place
    lg[3, 17] = np.float32(30.0)                      # one dominant expert: tiny weights for the rest
    lg[4, :] = np.round(lg[4] * 2) / 2                # many ties at all ranks
    lg[5, 7] = np.float32(-0.0)
    lg[5, 3] = np.float32(0.0)                        # +0 and -0 compare equal: a tie
    ids = np.empty((T, NU), np.int32)
    wts = np.empty((T, NU), np.float32)
    for t in range(T):
        order = np.argsort(-lg[t].astype(np.float64), kind="stable")  # std::stable_sort with l[a] > l[b]
        sel = order[:NU]
        p = np.exp(lg[t, sel].astype(np.float64) - np.float64(lg[t, sel[0]]))
        ids[t] = sel
        wts[t] = (p / p.sum()).astype(np.float32)
    # ---- expert projections: expert_mv on stacked Q4_K tensors, inputs rounded to int8 per 32 (REF_Q=all REF_QB=32)
    NEs, E, F = 3, 256, 256
    wg = S.make_weight(S.GGML_Q4_K, NEs * F, E, 31)
    wu = S.make_weight(S.GGML_Q4_K, NEs * F, E, 32)
    wd = S.make_weight(S.GGML_Q4_K, NEs * E, F, 33)
    x = rng.standard_normal((5, E), dtype=np.float32)
    pairs = np.array([(0, 0), (0, 2), (1, 1), (2, 0), (3, 2), (4, 1), (4, 2)], np.int32)  # (token, expert)
    g = np.empty((len(pairs), F), np.float32)
    u = np.empty_like(g)
    h = np.empty_like(g)
    dn = np.empty((len(pairs), E), np.float32)
    with tempfile.TemporaryDirectory() as d:
        p = os.path.join(d, "moe.gguf")
        S.write_gguf(p, {"blk.0.ffn_gate_exps.weight": (12, wg, F, E, NEs), "blk.0.ffn_up_exps.weight": (12, wu, F, E, NEs),
                         "blk.0.ffn_down_exps.weight": (12, wd, E, F, NEs)})
        for i, (t, e) in enumerate(pairs):
            g[i] = O.ref_expert_mv(p, "blk.0.ffn_gate_exps", int(e), F, E, x[t])
            u[i] = O.ref_expert_mv(p, "blk.0.ffn_up_exps", int(e), F, E, x[t])
            h[i] = O.ref_silu(g[i]) * u[i]
            dn[i] = O.ref_expert_mv(p, "blk.0.ffn_down_exps", int(e), E, F, h[i])
    np.savez_compressed(os.path.join(OUT, "moe.npz"), logits=lg, ids=ids, wts=wts, wg=wg, wu=wu, wd=wd, x=x, pairs=pairs,
                        g=g, u=u, h=h, dn=dn)


def make_types():
    rng = np.random.default_rng(20261202)
    K, N = 512, 5
    x = rng.standard_normal((4, K), dtype=np.float32)
    out = {"x": x}
    tensors = {}
    for name, qt in (("q4_0", 2), ("q5_k", 13), ("q6_k", 14), ("iq4_xs", 23)):
        w = S.make_weight(qt, N, K, 40 + qt)
        if qt == 13:
            w[0, 0:4] = 0                 # d = dmin = 0
            w[1, 4:16] = 0xFF             # every scale / min 63
        if qt == 14:
            w[0, 192:208] = 0x80          # every scale -128
            w[1, 0:192] = 0xFF            # every quant 63 - 32 = 31
            w[2, 0:192] = 0               # every quant -32
        out["w_" + name] = w
        out["deq_" + name] = O.ref_dequant_rows(qt, w, K)
        if qt != 2:
            sbb = S.sb_bytes(qt)
            dec = [O.ref_decode_generic_sb(qt, w[n, sbb * s:sbb * (s + 1)]) for n in range(N) for s in range(K // 256)]
            out["wd_" + name] = np.array([d[0] for d in dec], np.float32)
            out["wdmin_" + name] = np.array([d[1] for d in dec], np.float32)
            out["wsc_" + name] = np.stack([d[2] for d in dec])
            out["wmn_" + name] = np.stack([d[3] for d in dec])
            out["q_" + name] = np.stack([d[5] for d in dec])
        tensors[name] = (qt, w, N, K)
    with tempfile.TemporaryDirectory() as d:
        p = os.path.join(d, "t.gguf")
        S.write_gguf(p, tensors)
        for name in tensors:
            out["y_" + name] = O.ref_forward_matmul(p, name, x, N)
    np.savez_compressed(os.path.join(OUT, "types.npz"), **out)


def main():
    O.build(ref=True)
    assert O.ref() is not None, "oracle/_ref/libizb_ref.so missing: the reference sources are needed"
    if sys.argv[1:] == ["moe"]:
        make_moe()
        print("moe.npz written to", OUT)
        return
    if sys.argv[1:] == ["types"]:
        make_types()
        print("types.npz written to", OUT)
        return
    rng = np.random.default_rng(20261125)

    # ---- quantize
    x = rng.standard_normal((9, 768), dtype=np.float32)
    x[1, 32:64] = 0.0                      # an all-zero block: scale 0, inv 0
    x[2, 0:32] = 0.5                       # all equal: every value -> 127
    x[3, 64:96] = np.linspace(-1, 1, 32)   # symmetric ramp
    x[4, 0:32] = (np.arange(32) - 15.5) * (1.0 / 127.0) * 15.5  # products near .5 ties
    x[5, :] *= 1e-30                       # tiny values (scale near denormal range)
    x[6, :] *= 1e30                        # huge values
    x[7, 96:128] = np.float32(1e-42)       # denormal inputs
    x[8, 0:32] = np.where(np.arange(32) % 2 == 0, 1.0, -1.0) * 3.0
    aq, asc, absum = O.ref_quantize_act(x)
    np.savez_compressed(os.path.join(OUT, "quantize.npz"), x=x, aq=aq, asc=asc, absum=absum)

    # ---- decode / dequant
    w4 = S.make_weight(S.GGML_Q4_K, 6, 512, 11)
    w8 = S.make_weight(S.GGML_Q8_0, 6, 512, 12)
    w4[0, 0:4] = 0                         # d = dmin = 0
    w4[1, 0:2] = np.array([1, 0], np.uint8)  # fp16 subnormal d
    w4[2, 4:16] = 0xFF                     # every scale / min = 63
    w8[0, 0:2] = 0
    w8[1, 2:34] = np.array([-128] * 32, np.int8).view(np.uint8)
    d4 = [O.ref_decode_sb(12, w4[n, 144 * s:144 * (s + 1)]) for n in range(6) for s in range(2)]
    d8 = [O.ref_decode_sb(8, w8[n, 272 * s:272 * (s + 1)]) for n in range(6) for s in range(2)]
    np.savez_compressed(
        os.path.join(OUT, "decode.npz"), w4=w4, w8=w8,
        q4_d=np.array([t[0] for t in d4], np.float32), q4_dmin=np.array([t[1] for t in d4], np.float32),
        q4_sc=np.stack([t[2] for t in d4]), q4_mn=np.stack([t[3] for t in d4]), q4_q=np.stack([t[4] for t in d4]),
        q8_d=np.stack([t[5] for t in d8]), q8_q=np.stack([t[4] for t in d8]),
        deq4=O.ref_dequant_rows(12, w4, 512), deq8=O.ref_dequant_rows(8, w8, 512))

    # ---- fp16
    allh = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    f = np.array([O.ref().ref_fp16_to_f32(int(h)) for h in allh], np.float32)
    xs = np.concatenate([rng.standard_normal(2000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 6, 2000),
                         np.array([0, -0.0, 65504, 65520, 1e-8, 6e-8, 5.96e-8, 2.98e-8, np.inf, -np.inf], np.float32)])
    h = np.array([O.ref().ref_f32_to_fp16(float(v)) for v in xs], np.uint16)
    np.savez_compressed(os.path.join(OUT, "fp16.npz"), to_f32=f.view(np.uint32), xs=xs, to_f16=h)

    # ---- ref_forward matmul
    xa = rng.standard_normal((5, 512), dtype=np.float32)
    with tempfile.TemporaryDirectory() as d:
        p = os.path.join(d, "t.gguf")
        S.write_gguf(p, {"q4": (12, w4, 6, 512), "q8": (8, w8, 6, 512)})
        y4 = O.ref_forward_matmul(p, "q4", xa, 6)
        y8 = O.ref_forward_matmul(p, "q8", xa, 6)
    np.savez_compressed(os.path.join(OUT, "forward.npz"), x=xa, y4=y4, y8=y8)

    # ---- reference GPU raw form of Q8_0
    raw = np.stack([O.ref_gpu_raw_sb(8, w8[n, 272 * s:272 * (s + 1)]) for n in range(6) for s in range(2)])
    np.savez_compressed(os.path.join(OUT, "rawsb.npz"), raw8=raw)
    # ---- rmsnorm (tools/ref_forward.cpp:314) on rows of several magnitudes, one all-zero row
    r2 = np.random.default_rng(7)
    xn = r2.standard_normal((6, 1024), dtype=np.float32)
    xn[1] *= 1e-3
    xn[2] *= 300.0
    xn[3] = 0.0
    wn = (1.0 + 0.1 * r2.standard_normal(1024)).astype(np.float32)
    yn = O.ref_rmsnorm(xn, wn, 1e-6)
    np.savez_compressed(os.path.join(OUT, "rmsnorm.npz"), x=xn, w=wn, eps=np.float32(1e-6), y=yn)
    make_moe()
    make_types()
    print("golden vectors written to", OUT)


if __name__ == "__main__":
    main()
