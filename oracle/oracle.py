"""ctypes front end of the CPU oracle (oracle/izb_oracle.c) and of the reference's own CPU code (oracle/_ref).

TEST INFRASTRUCTURE ONLY.  Imported by tests/, by the smoke check and by the benchmark's cpu-baseline leg; the
shipped library (arcinferzero_b200) never imports it.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
Q8_0, Q4_K = 8, 12
Q4_0, Q5_K, Q6_K, IQ4_XS = 2, 13, 14, 23
GENERIC = (Q5_K, Q6_K, IQ4_XS)   # types decoded into the reference's generic view (scale and min per 16 elements)

_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C")
_i8p = np.ctypeslib.ndpointer(np.int8, flags="C")
_i16p = np.ctypeslib.ndpointer(np.int16, flags="C")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C")
_f32p = np.ctypeslib.ndpointer(np.float32, flags="C")


def build(ref: bool = True) -> None:
    """Compile the oracle (and, when the reference sources are present, oracle/_ref) with oracle/Makefile."""
    subprocess.run(["make", "-C", HERE, "libizb_oracle.so"] + (["ref"] if ref else []), check=True,
                   stdout=subprocess.DEVNULL)


_lib = None
_ref = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        p = os.path.join(HERE, "libizb_oracle.so")
        if not os.path.exists(p) or os.path.getmtime(p) < os.path.getmtime(os.path.join(HERE, "izb_oracle.c")):
            build(ref=False)
        _lib = C.CDLL(p)
        _lib.orc_fp16_to_f32.restype = C.c_float
        _lib.orc_fp16_to_f32.argtypes = [C.c_uint16]
        _lib.orc_f32_to_fp16.restype = C.c_uint16
        _lib.orc_f32_to_fp16.argtypes = [C.c_float]
    return _lib


def ref():
    """The reference's own code, or None when oracle/_ref was never built (it cannot be built without the sources)."""
    global _ref
    if _ref is None:
        p = os.path.join(HERE, "_ref", "libizb_ref.so")
        if not os.path.exists(p):
            return None
        _ref = C.CDLL(p)
        _ref.ref_fp16_to_f32.restype = C.c_float
        _ref.ref_fp16_to_f32.argtypes = [C.c_uint16]
        _ref.ref_f32_to_fp16.restype = C.c_uint16
        _ref.ref_f32_to_fp16.argtypes = [C.c_float]
    return _ref


def set_threads(n: int) -> int:
    """OpenMP threads of the restatement's loops (and of oracle/_ref's, which shares the process's OpenMP runtime when
    ref_forward_matmul is given no count of its own); returns the count now in force."""
    lib().orc_set_threads(int(n))
    return int(lib().orc_max_threads())


def _vp(a):
    return a.ctypes.data_as(C.c_void_p)


# ------------------------------------------------------------------ restatement
def quantize_act(x: np.ndarray, Mp: int | None = None, want_absum: bool = True):
    """x [M, K] f32 -> aq [Mp, K] int8, asc [K/32, Mp] f32, absum [K/16, Mp] int16."""
    x = np.ascontiguousarray(x, np.float32)
    M, K = x.shape
    Mp = Mp or M
    aq = np.empty((Mp, K), np.int8)
    asc = np.empty((K // 32, Mp), np.float32)
    absum = np.empty((K // 16, Mp), np.int16) if want_absum else None
    lib().orc_quantize_act(_vp(x), M, K, K, Mp, _vp(aq), _vp(asc), _vp(absum) if want_absum else None)
    return aq, asc, absum


def rmsnorm_quant(x: np.ndarray, w: np.ndarray, eps: float, Mp: int | None = None):
    """y = (x * r) * w, r = 1/sqrt(sum(x^2)/K + eps) per row in the CUDA kernel's summation order -> y, aq, asc, absum."""
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    M, K = x.shape
    Mp = Mp or M
    y = np.empty((M, K), np.float32)
    aq = np.empty((Mp, K), np.int8)
    asc = np.empty((K // 32, Mp), np.float32)
    absum = np.empty((K // 16, Mp), np.int16)
    lib().orc_rmsnorm_quant(_vp(x), M, K, K, _vp(w), C.c_float(eps), Mp, _vp(y), _vp(aq), _vp(asc), _vp(absum))
    return y, aq, asc, absum


def add_norm_quant(x: np.ndarray, t: np.ndarray, w: np.ndarray, eps: float, s: float, w2: np.ndarray | None, Mp: int | None = None):
    """x_new = (x + (t * r) * w) * s; y = (x_new * r2) * w2 (or x_new when w2 is None) quantised -> x_new, aq, asc, absum."""
    x = np.array(x, np.float32, copy=True, order="C")
    t = np.ascontiguousarray(t, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    w2c = None if w2 is None else np.ascontiguousarray(w2, np.float32)
    M, K = x.shape
    Mp = Mp or M
    aq = np.empty((Mp, K), np.int8)
    asc = np.empty((K // 32, Mp), np.float32)
    absum = np.empty((K // 16, Mp), np.int16)
    lib().orc_add_norm_quant(_vp(x), _vp(t), _vp(w), C.c_float(eps), C.c_float(s), None if w2c is None else _vp(w2c), M, K, Mp,
                             _vp(aq), _vp(asc), _vp(absum))
    return x, aq, asc, absum


def decode_q4k_sb(p: np.ndarray):
    d, dmin = C.c_float(), C.c_float()
    sc, mn, q = np.empty(8, np.uint8), np.empty(8, np.uint8), np.empty(256, np.uint8)
    lib().orc_q4k_decode_sb(_vp(np.ascontiguousarray(p, np.uint8)), C.byref(d), C.byref(dmin), _vp(sc), _vp(mn), _vp(q))
    return d.value, dmin.value, sc, mn, q


def decode_q8_0_sb(p: np.ndarray):
    d8, q = np.empty(8, np.float32), np.empty(256, np.int8)
    lib().orc_q8_0_decode_sb(_vp(np.ascontiguousarray(p, np.uint8)), _vp(d8), _vp(q))
    return d8, q


def dequant_rows(qtype: int, w: np.ndarray, K: int) -> np.ndarray:
    w = np.ascontiguousarray(w, np.uint8)
    out = np.empty((w.shape[0], K), np.float32)
    for n in range(w.shape[0]):
        lib().orc_dequant_row(qtype, _vp(w[n]), K, _vp(out[n]))
    return out


def q4_0_as_q8_0(w: np.ndarray) -> np.ndarray:
    """Q4_0 rows [N, K/32*18] rewritten as Q8_0 rows [N, K/32*34] (same scale, int8 quants q - 8): exact."""
    w = np.ascontiguousarray(w, np.uint8)
    nblk = w.shape[1] // 18
    out = np.empty((w.shape[0], nblk * 34), np.uint8)
    lib().orc_q4_0_to_q8_0(_vp(w), C.c_size_t(w.shape[0] * nblk), _vp(out))
    return out


def decode_generic_sb(qtype: int, p: np.ndarray):
    """One superblock of Q5_K / Q6_K / IQ4_XS in the generic view: wd, wdmin, wsc[16], wmn[16], has_min, q[256] (offset
    subtracted)."""
    wd, wdmin, hm = C.c_float(), C.c_float(), C.c_int()
    wsc, wmn, q = np.empty(16, np.int8), np.empty(16, np.uint8), np.empty(256, np.int16)
    rc = lib().orc_decode_generic_sb(qtype, _vp(np.ascontiguousarray(p, np.uint8)), C.byref(wd), C.byref(wdmin), _vp(wsc), _vp(wmn),
                                     C.byref(hm), _vp(q))
    assert rc == 0
    return wd.value, wdmin.value, wsc, wmn, bool(hm.value), q


def block_dots(qtype: int, w: np.ndarray, K: int, aq: np.ndarray):
    """dots [M, N, K/32] int32 and asum [M, K/32] int32 for the first M = aq.shape[0] rows."""
    if qtype == Q4_0:
        qtype, w = Q8_0, q4_0_as_q8_0(w)
    w = np.ascontiguousarray(w, np.uint8)
    aq = np.ascontiguousarray(aq, np.int8)
    N, M = w.shape[0], aq.shape[0]
    dots = np.empty((M, N, K // 32), np.int32)
    asum = np.empty((M, K // 32), np.int32)
    if qtype in GENERIC:
        lib().orc_block_dots_generic(qtype, _vp(w), N, K, _vp(aq), M, _vp(dots))
        asum[:] = aq.astype(np.int32).reshape(M, K // 32, 32).sum(axis=2)
        return dots, asum
    lib().orc_block_dots(qtype, _vp(w), N, K, _vp(aq), M, _vp(dots), _vp(asum))
    return dots, asum


def matmul(qtype: int, w: np.ndarray, K: int, aq: np.ndarray, asc: np.ndarray, T: int, order: str = "gemm",
           C_in: np.ndarray | None = None, ldc: int | None = None, c_off: int = 0, acc: int = 0) -> np.ndarray:
    """f32 outputs in one of the reference's two summation orders ("gemv": decode.cl, "gemm": gemm.cl) or "f64"
    (tools/ref_forward.cpp: dequantised weights, double accumulation)."""
    if qtype == Q4_0 and order != "f64":
        qtype, w = Q8_0, q4_0_as_q8_0(w)
    w = np.ascontiguousarray(w, np.uint8)
    aq = np.ascontiguousarray(aq, np.int8)
    asc = np.ascontiguousarray(asc, np.float32)
    N, Mp = w.shape[0], asc.shape[1]
    ldc = ldc or N
    out = np.zeros((T, ldc), np.float32) if C_in is None else np.array(C_in, np.float32, copy=True, order="C")
    if qtype in GENERIC and order != "f64":
        lib().orc_matmul_generic(qtype, _vp(w), N, K, _vp(aq), _vp(asc), Mp, T, _vp(out), ldc, c_off, acc, 0 if order == "gemv" else 1)
        return out
    if order == "f64":
        assert acc == 0 and c_off == 0
        lib().orc_matmul_f64(qtype, _vp(w), N, K, _vp(aq), _vp(asc), Mp, T, _vp(out), ldc)
    else:
        fn = lib().orc_matmul_gemv_order if order == "gemv" else lib().orc_matmul_gemm_order
        fn(qtype, _vp(w), N, K, _vp(aq), _vp(asc), Mp, T, _vp(out), ldc, c_off, acc)
    return out


def moe_route(logits: np.ndarray, NU: int):
    logits = np.ascontiguousarray(logits, np.float32)
    T, NE = logits.shape
    ids, wts = np.empty((T, NU), np.int32), np.empty((T, NU), np.float32)
    counts = np.empty(NE, np.int32)
    lib().orc_moe_route(_vp(logits), NE, T, NE, NU, _vp(ids), _vp(wts), _vp(counts))
    return ids, wts, counts


def moe_sort(ids: np.ndarray, wts: np.ndarray, counts: np.ndarray, TM: int):
    T, NU = ids.shape
    NE = counts.shape[0]
    offs = np.empty(NE + 1, np.int32)
    tiles = np.zeros(1 + 3 * (T * NU // TM + NE + 1), np.int32)
    stok, swt, inv = np.empty(T * NU, np.int32), np.empty(T * NU, np.float32), np.empty(T * NU, np.int32)
    lib().orc_moe_sort(_vp(np.ascontiguousarray(ids)), _vp(np.ascontiguousarray(wts)), T, NE, NU, TM, _vp(counts),
                       _vp(offs), _vp(tiles), _vp(stok), _vp(swt), _vp(inv))
    return offs, tiles, stok, swt, inv


def moe_sgate(logits: np.ndarray, NE: int) -> np.ndarray:
    logits = np.ascontiguousarray(logits, np.float32)
    T = logits.shape[0]
    out = np.empty(T, np.float32)
    lib().orc_moe_sgate(_vp(logits), logits.shape[1], T, NE, _vp(out))
    return out


def moe_sort_range(ids: np.ndarray, wts: np.ndarray, counts: np.ndarray, TM: int, e0: int, e1: int):
    T, NU = ids.shape
    NE = counts.shape[0]
    offs = np.empty(NE + 1, np.int32)
    tiles = np.zeros(1 + 3 * (T * NU // TM + NE + 1), np.int32)
    stok, swt, inv = np.zeros(T * NU, np.int32), np.zeros(T * NU, np.float32), np.empty(T * NU, np.int32)
    lib().orc_moe_sort_range(_vp(np.ascontiguousarray(ids)), _vp(np.ascontiguousarray(wts)), T, NE, NU, TM, _vp(counts), e0, e1,
                             _vp(offs), _vp(tiles), _vp(stok), _vp(swt), _vp(inv))
    return offs, tiles, stok, swt, inv


def moe_combine_ex(x: np.ndarray, y: np.ndarray, inv: np.ndarray, NU: int, sh=None, sgate=None, partial: bool = False) -> np.ndarray:
    out = np.array(x, np.float32, copy=True, order="C")
    T, E = out.shape
    lib().orc_moe_combine_ex(_vp(out), _vp(np.ascontiguousarray(y, np.float32)), _vp(np.ascontiguousarray(inv, np.int32)), T, NU, E,
                             None if sh is None else _vp(np.ascontiguousarray(sh, np.float32)),
                             None if sgate is None else _vp(np.ascontiguousarray(sgate, np.float32)), int(partial))
    return out


def slot_experts(offs: np.ndarray) -> np.ndarray:
    return np.repeat(np.arange(len(offs) - 1, dtype=np.int32), np.diff(offs)).astype(np.int32)


def moe_gateup(qtype, wg, wu, F, K, aq, asc, slot_expert, stok, want_gu=False):
    S, Mp = len(stok), asc.shape[1]
    h = np.empty((S, F), np.float32)
    g = np.empty((S, F), np.float32) if want_gu else None
    u = np.empty((S, F), np.float32) if want_gu else None
    lib().orc_moe_gateup(qtype, _vp(np.ascontiguousarray(wg)), _vp(np.ascontiguousarray(wu)), F, K,
                         _vp(np.ascontiguousarray(aq)), _vp(np.ascontiguousarray(asc)), Mp, S,
                         _vp(np.ascontiguousarray(slot_expert, np.int32)), _vp(np.ascontiguousarray(stok, np.int32)),
                         _vp(h), _vp(g) if want_gu else None, _vp(u) if want_gu else None)
    return (h, g, u) if want_gu else h


def moe_down(qtype, wd, E, F, hq, hsc, slot_expert, swt):
    S = hq.shape[0]
    y = np.empty((S, E), np.float32)
    lib().orc_moe_down(qtype, _vp(np.ascontiguousarray(wd)), E, F, _vp(np.ascontiguousarray(hq)),
                       _vp(np.ascontiguousarray(hsc)), S, _vp(np.ascontiguousarray(slot_expert, np.int32)),
                       _vp(np.ascontiguousarray(swt, np.float32)), _vp(y))
    return y


def moe_combine(x: np.ndarray, y: np.ndarray, inv: np.ndarray, NU: int) -> np.ndarray:
    out = np.array(x, np.float32, copy=True, order="C")
    T, E = out.shape
    lib().orc_moe_combine(_vp(out), _vp(np.ascontiguousarray(y, np.float32)), _vp(np.ascontiguousarray(inv, np.int32)),
                          T, NU, E)
    return out


def tp_range(total: int, unit: int, N: int, r: int):
    b, e = C.c_int64(), C.c_int64()
    lib().orc_tp_range(C.c_int64(total), C.c_int64(unit), N, r, C.byref(b), C.byref(e))
    return b.value, e.value


def softcap_rows(c: np.ndarray, rows: int, N: int, cap: float, off: int = 0) -> np.ndarray:
    """Copy of c [R, ld] f32 with c[r, off:off+N] = cap * tanh(c / cap) for r < rows."""
    out = np.ascontiguousarray(c, dtype=np.float32).copy()
    lib().orc_softcap_rows(_vp(out), rows, out.shape[1], off, N, C.c_float(cap))
    return out


def tp_add(x: np.ndarray, parts: np.ndarray) -> np.ndarray:
    out = np.array(x, np.float32, copy=True, order="C")
    parts = np.ascontiguousarray(parts, np.float32)
    n = out.size
    lib().orc_tp_add(_vp(out), _vp(parts), C.c_size_t(n), parts.shape[0], C.c_size_t(n))
    return out


# ------------------------------------------------------------------ the reference's own code (oracle/_ref)
def ref_quantize_act(x: np.ndarray):
    x = np.ascontiguousarray(x, np.float32)
    M, K = x.shape
    aq, asc, absum = np.empty((M, K), np.int8), np.empty((K // 32, M), np.float32), np.empty((K // 16, M), np.uint16)
    ref().ref_quantize_act(_vp(x), M, K, _vp(aq), _vp(asc), _vp(absum))
    return aq, asc, absum.view(np.int16)


def ref_rmsnorm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """tools/ref_forward.cpp rmsnorm() row by row."""
    y = np.array(x, np.float32, copy=True, order="C")
    w = np.ascontiguousarray(w, np.float32)
    for m in range(y.shape[0]):
        ref().ref_rmsnorm(_vp(y[m]), y.shape[1], _vp(w), C.c_float(eps))
    return y


def ref_decode_sb(qtype: int, p: np.ndarray):
    d, dmin = C.c_float(), C.c_float()
    sc, mn, q, d8 = np.empty(8, np.uint8), np.empty(8, np.uint8), np.empty(256, np.int16), np.empty(8, np.float32)
    ref().ref_decode_sb(qtype, _vp(np.ascontiguousarray(p, np.uint8)), C.byref(d), C.byref(dmin), _vp(sc), _vp(mn), _vp(q),
                        _vp(d8))
    return d.value, dmin.value, sc, mn, q, d8


def ref_dequant_rows(qtype: int, w: np.ndarray, K: int) -> np.ndarray:
    w = np.ascontiguousarray(w, np.uint8)
    out = np.empty((w.shape[0], K), np.float32)
    for n in range(w.shape[0]):
        ref().ref_dequant_row(qtype, _vp(w[n]), K, _vp(out[n]))
    return out


def ref_gpu_raw_sb(qtype: int, p: np.ndarray) -> np.ndarray:
    out = np.zeros(ref().ref_raw_padded_sb_bytes(qtype), np.uint8)
    ref().ref_gpu_raw_sb(qtype, _vp(np.ascontiguousarray(p, np.uint8)), _vp(out))
    return out


def ref_forward_matmul(gguf_path: str, name: str, x: np.ndarray, N: int, quant32: bool = True, threads: int = 0):
    """tools/ref_forward.cpp matmul() on a tensor of a GGUF file; x [T, K] f32 (rounded per 32 inside when quant32)."""
    x = np.ascontiguousarray(x, np.float32)
    y = np.empty((x.shape[0], N), np.float32)
    rc = ref().ref_forward_matmul(gguf_path.encode(), name.encode(), _vp(x), x.shape[0], int(quant32), _vp(y), threads)
    if rc != 0:
        raise RuntimeError("ref_forward_matmul failed")
    return y


def ref_expert_mv(gguf_path: str, name: str, e: int, N: int, K: int, x: np.ndarray, quant32: bool = True) -> np.ndarray:
    """tools/ref_forward.cpp expert_mv() (:333) on expert e of the stacked tensor `name`.weight; x [K] f32 -> y [N] f32."""
    x = np.ascontiguousarray(x, np.float32)
    y = np.empty(N, np.float32)
    if ref().ref_expert_mv(gguf_path.encode(), name.encode(), e, N, K, _vp(x), _vp(y), int(quant32)) != 0:
        raise RuntimeError("ref_expert_mv failed")
    return y


def ref_silu(x: np.ndarray) -> np.ndarray:
    """tools/ref_forward.cpp silu() (:321) element by element."""
    f = ref().ref_silu
    f.restype, f.argtypes = C.c_float, [C.c_float]
    return np.array([f(float(v)) for v in np.asarray(x, np.float32).ravel()], np.float32).reshape(np.shape(x))


def ref_decode_generic_sb(qtype: int, p: np.ndarray):
    """The reference's decode_sb (src/quants.h:89) in its generic view: wd, wdmin, wsc[16], wmn[16], has_min, q - qoff."""
    wd, wdmin, hm = C.c_float(), C.c_float(), C.c_int()
    wsc, wmn, q = np.empty(16, np.int8), np.empty(16, np.uint8), np.empty(256, np.int16)
    ref().ref_decode_generic_sb(qtype, _vp(np.ascontiguousarray(p, np.uint8)), C.byref(wd), C.byref(wdmin), _vp(wsc), _vp(wmn),
                                C.byref(hm), _vp(q))
    return wd.value, wdmin.value, wsc, wmn, bool(hm.value), q
