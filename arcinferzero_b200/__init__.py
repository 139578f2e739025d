"""arcinferzero_b200: the B200 (sm_100a) implementation of inferzero's quantised matrix product.

The product is the CUDA library `libizb200.so` behind the C ABI of include/izb200.h (built in-tree by
arcinferzero_b200/build.py).  This module is the thin ctypes binding the tests and the benchmark use: it passes raw
device pointers of torch tensors (torch is only the owner of device memory and streams here) and raises on any non-zero
status.  There is no CPU path: importing works without a GPU, every call needs one.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("IZB200_LIB") or os.path.join(HERE, "libizb200.so")  # IZB200_LIB: another build of the library

Q8_0, Q4_K = 8, 12
Q4_0, Q5_K, Q6_K, IQ4_XS = 2, 13, 14, 23
GEMM_AUTO, GEMM_CORE, GEMM_TC = 0, 1, 2

# every symbol include/izb200.h declares (tests check the library exports each of them)
SYMBOLS = [
    "izb_status_string", "izb_last_error", "izb_launch_count", "izb_device_status", "izb_profile_start", "izb_profile_stop",
    "izb_reserve", "izb_set_sm_limit", "izb_debug_wait_test", "izb_tensor_peak",
    "izb_weight_create", "izb_weight_create_slice", "izb_weight_create_stack", "izb_weight_create_gateup", "izb_gateup_interleave_host", "izb_weight_destroy", "izb_weight_info", "izb_weight_download", "izb_weight_decode_host",
    "izb_quantize_act", "izb_swiglu_quant", "izb_rmsnorm_quant", "izb_add_norm_quant", "izb_softcap_rows",
    "izb_matmul", "izb_quant_matmul", "izb_gemv", "izb_gemm", "izb_gemm_noalloc", "izb_block_dots", "izb_selfcheck", "izb_matmul_host",
    "izb_moe_route", "izb_moe_route_ex", "izb_moe_sort", "izb_moe_sort_ex", "izb_moe_gateup", "izb_moe_down", "izb_moe_combine",
    "izb_moe_combine_ex",
    "izb_tp_range", "izb_tp_add", "izb_tp_unique_id", "izb_tp_create", "izb_tp_create_ex", "izb_tp_wait", "izb_tp_abort", "izb_tp_destroy", "izb_tp_allreduce_rows",
    "izb_tp_reduce_quant_gather", "izb_tp_gather_logits", "izb_p2p_push", "izb_p2p_wait", "izb_p2p_wait_host", "izb_tp_scales_from_ranks",
]


class IzbError(RuntimeError):
    def __init__(self, status: int, detail: str):
        super().__init__(f"izb200 status {status}: {detail}")
        self.status = status


_lib = None


def lib() -> C.CDLL:
    """The loaded library.  Raises if it was never built: there is nothing to fall back to."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -m arcinferzero_b200.build` "
                              "(this package has no CPU or PyTorch fallback)")
        _lib = C.CDLL(LIB_PATH)
        _lib.izb_status_string.restype = C.c_char_p
        _lib.izb_last_error.restype = C.c_char_p
        _lib.izb_launch_count.restype = C.c_uint64
    return _lib


def _check(rc: int) -> None:
    if rc != 0:
        L = lib()
        raise IzbError(rc, f"{L.izb_status_string(rc).decode()}: {L.izb_last_error().decode()}")


def _p(t) -> C.c_void_p:
    """Device (or pinned host) pointer of a torch tensor / numpy array, or NULL."""
    if t is None:
        return C.c_void_p(0)
    if isinstance(t, np.ndarray):
        return C.c_void_p(t.ctypes.data)
    return C.c_void_p(t.data_ptr())


def _stream() -> C.c_void_p:
    import torch
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def launch_count() -> int:
    return int(lib().izb_launch_count())


def profile_start() -> None:
    _check(lib().izb_profile_start())


def profile_stop() -> dict:
    """Per-kernel {"launches", "ms"} of every library launch since profile_start (synchronises)."""
    import json
    buf = C.create_string_buffer(8192)
    _check(lib().izb_profile_stop(buf, C.c_size_t(8192)))
    return json.loads(buf.value.decode())


def pad_rows(M: int) -> int:
    """Row padding of the reference engine (zero/engine.h:521-522): multiples of 128 from 128 rows on, else of 16."""
    return (M + 127) // 128 * 128 if M >= 128 else (M + 15) // 16 * 16


class Weight:
    """Device weight handle (izb_weight): a matrix or a stack of n_mats matrices in GGUF block form."""

    def __init__(self, qtype: int, rows: np.ndarray, N: int, K: int, n_mats: int = 1, device: int = 0,
                 row_range: tuple[int, int] | None = None, col_range: tuple[int, int] | None = None):
        rows = np.ascontiguousarray(rows, np.uint8)
        self.handle = C.c_void_p(0)
        n0, n1 = row_range or (0, N)
        k0, k1 = col_range or (0, K)
        _check(lib().izb_weight_create_slice(qtype, _p(rows), n_mats, N, K, n0, n1, k0, k1, device, C.byref(self.handle)))
        self.qtype, self.N, self.K, self.n_mats, self.device = qtype, n1 - n0, k1 - k0, n_mats, device

    @property
    def nbytes(self) -> int:
        b = C.c_size_t(0)
        _check(lib().izb_weight_info(self.handle, None, None, None, None, C.byref(b)))
        return b.value

    def download(self, offset: int = 0, nbytes: int | None = None) -> np.ndarray:
        """The device form of the weight (without the slack) as bytes."""
        n = self.nbytes - 1024 - offset if nbytes is None else nbytes
        out = np.empty(n, np.uint8)
        _check(lib().izb_weight_download(self.handle, C.c_size_t(offset), C.c_size_t(n), _p(out)))
        return out

    def close(self):
        if self.handle:
            lib().izb_weight_destroy(self.handle)
            self.handle = C.c_void_p(0)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def stacked_weight(qtype: int, parts: list, K: int, device: int = 0) -> "Weight":
    """Several tensors (GGUF rows [N_i, row bytes]) of one type and K as one weight of sum(N_i) rows: one launch for Q | K | V
    or gate | up (izb_weight_create_stack)."""
    arrs = [np.ascontiguousarray(a, np.uint8) for a in parts]
    if any(a.ndim != 2 or a.shape[1] != arrs[0].shape[1] for a in arrs):
        raise ValueError("stacked_weight: every part is [rows, K/256 * superblock bytes] of the same K")
    ptrs = (C.c_void_p * len(arrs))(*[a.ctypes.data for a in arrs])
    rows = (C.c_int * len(arrs))(*[a.shape[0] for a in arrs])
    w = Weight.__new__(Weight)
    w.handle = C.c_void_p(0)
    _check(lib().izb_weight_create_stack(qtype, ptrs, rows, len(arrs), K, device, C.byref(w.handle)))
    w.qtype, w.N, w.K, w.n_mats, w.device = qtype, sum(a.shape[0] for a in arrs), K, 1, device
    return w


def gateup_weight(qtype: int, gate_rows: np.ndarray, up_rows: np.ndarray, F: int, K: int, n_mats: int = 1, device: int = 0) -> "Weight":
    """Gate and up projection ([n_mats * F, row bytes] each) as one weight of 2F rows per matrix, rows alternating in groups of
    32 (izb_weight_create_gateup): gemm(..., acc=3) and moe_gateup(W, None, ...) store up * silu(gate) from one GEMM."""
    g, u = np.ascontiguousarray(gate_rows, np.uint8), np.ascontiguousarray(up_rows, np.uint8)
    if g.shape != u.shape or g.size % (n_mats * F):
        raise ValueError("gateup_weight: gate and up are [n_mats * F, K/256 * superblock bytes] each")
    w = Weight.__new__(Weight)
    w.handle = C.c_void_p(0)
    _check(lib().izb_weight_create_gateup(qtype, _p(g), _p(u), n_mats, F, K, device, C.byref(w.handle)))
    w.qtype, w.N, w.K, w.n_mats, w.device = qtype, 2 * F, K, n_mats, device
    return w


def gateup_interleave_host(qtype: int, gate_rows: np.ndarray, up_rows: np.ndarray, F: int, K: int, n_mats: int = 1) -> np.ndarray:
    """The host-side row order of gateup_weight (no GPU): [n_mats * 2F, row bytes]."""
    g, u = np.ascontiguousarray(gate_rows, np.uint8), np.ascontiguousarray(up_rows, np.uint8)
    out = np.empty((2 * g.shape[0], g.shape[1]), np.uint8)
    _check(lib().izb_gateup_interleave_host(qtype, _p(g), _p(u), n_mats, F, K, _p(out), C.c_size_t(out.size)))
    return out


def weight_decode_host(qtype: int, rows: np.ndarray, K: int) -> np.ndarray:
    """The loader's host-side decoder (no GPU): rows [N, K/256 * file bytes] of Q4_0 / Q5_K / Q6_K / IQ4_XS -> the uploaded
    form [N, K/256 * (272 | 304 | 224)] (Q4_0 as Q8_0 blocks; Q5_K / IQ4_XS in the generic per-16-scale form; Q6_K packed)."""
    rows = np.ascontiguousarray(rows, np.uint8)
    per = 272 if qtype == Q4_0 else 224 if qtype == Q6_K else 304
    out = np.empty((rows.shape[0], K // 256 * per), np.uint8)
    _check(lib().izb_weight_decode_host(qtype, _p(rows), C.c_size_t(rows.shape[0] * (K // 256)), _p(out), C.c_size_t(out.size)))
    return out


def quantize_act(x, Mp: int | None = None, want_absum: bool = False, out=None):
    """x: [M, K] f32 cuda tensor (row stride may exceed K) -> aq [Mp, K] int8, asc [K/32, Mp] f32, absum or None."""
    import torch
    M, K = x.shape
    Mp = Mp or pad_rows(M)
    if out is None:
        aq = torch.empty((Mp, K), dtype=torch.int8, device=x.device)
        asc = torch.empty((K // 32, Mp), dtype=torch.float32, device=x.device)
        absum = torch.empty((K // 16, Mp), dtype=torch.int16, device=x.device) if want_absum else None
    else:
        aq, asc, absum = out
    _check(lib().izb_quantize_act(_p(x), x.stride(0), M, Mp, K, _p(aq), _p(asc), _p(absum), _stream()))
    return aq, asc, absum


def swiglu_quant(gu, F: int, Mp: int | None = None, want_h: bool = False):
    """gu: [M, 2F] f32 (gate | up) -> quantised h = silu(gate) * up; optionally h itself."""
    import torch
    M = gu.shape[0]
    Mp = Mp or pad_rows(M)
    aq = torch.empty((Mp, F), dtype=torch.int8, device=gu.device)
    asc = torch.empty((F // 32, Mp), dtype=torch.float32, device=gu.device)
    h = torch.empty((M, F), dtype=torch.float32, device=gu.device) if want_h else None
    _check(lib().izb_swiglu_quant(_p(gu), gu.stride(0), 1, M, Mp, F, _p(h), _p(aq), _p(asc), None, _stream()))
    return aq, asc, h


def rmsnorm_quant(x, w, eps: float, Mp: int | None = None, want_h: bool = False):
    """x: [M, K] f32, w: [K] f32 -> quantised y = (x * r) * w, r = 1/sqrt(mean(x^2) + eps) per row; optionally y itself."""
    import torch
    M, K = x.shape
    Mp = Mp or pad_rows(M)
    aq = torch.empty((Mp, K), dtype=torch.int8, device=x.device)
    asc = torch.empty((K // 32, Mp), dtype=torch.float32, device=x.device)
    h = torch.empty((M, K), dtype=torch.float32, device=x.device) if want_h else None
    _check(lib().izb_rmsnorm_quant(_p(x), x.stride(0), _p(w), C.c_float(eps), M, Mp, K, _p(h), _p(aq), _p(asc), None, _stream()))
    return aq, asc, h


def add_norm_quant(x, t, w, eps: float, s: float = 1.0, w2=None, Mp: int | None = None):
    """In place x = (x + rmsnorm(t) * w) * s on [M, K] f32 rows, then the quantised next-GEMV input rmsnorm(x) * w2 (or x)."""
    import torch
    M, K = x.shape
    Mp = Mp or pad_rows(M)
    aq = torch.empty((Mp, K), dtype=torch.int8, device=x.device)
    asc = torch.empty((K // 32, Mp), dtype=torch.float32, device=x.device)
    _check(lib().izb_add_norm_quant(_p(x), _p(t), _p(w), C.c_float(eps), C.c_float(s), _p(w2), M, Mp, K, _p(aq), _p(asc), None, _stream()))
    return aq, asc


def softcap_rows(c, rows: int, N: int, cap: float, off: int = 0):
    """In place c[r, off:off+N] = cap * tanh(c[r, off:off+N] / cap) for r < rows (the output head's logit soft-cap)."""
    _check(lib().izb_softcap_rows(_p(c), rows, c.stride(0), off, N, C.c_float(cap), _stream()))
    return c


def matmul(w: Weight, aq, asc, T: int, out=None, c_off: int = 0, acc: int = 0, mat: int = 0):
    """Engine::matmul dispatch: T == 1 GEMV, 2..8 few-row GEMV, else GEMM.  out: [rows, ldc] f32 (default [Mp, N])."""
    import torch
    Mp = asc.shape[1]
    if out is None:
        out = torch.empty((Mp, w.N), dtype=torch.float32, device=aq.device)
    _check(lib().izb_matmul(w.handle, mat, _p(aq), _p(asc), None, T, Mp, _p(out), out.stride(0), c_off, acc, _stream()))
    return out


def quant_matmul(w: Weight, x, T: int, Mp: int | None = None, out=None, c_off: int = 0, acc: int = 0, mat: int = 0, qout=None):
    """izb_quant_matmul: quantise x [T, K] f32 and multiply in one call.  Returns (out, aq, asc); qout = (aq, asc) to reuse
    buffers."""
    import torch
    Mp = Mp or pad_rows(T)
    K = w.K
    if qout is None:
        aq = torch.empty((Mp, K), dtype=torch.int8, device=x.device)
        asc = torch.empty((K // 32, Mp), dtype=torch.float32, device=x.device)
    else:
        aq, asc = qout
    if out is None:
        out = torch.empty((Mp, w.N // 2 if acc == 3 else w.N), dtype=torch.float32, device=x.device)
    _check(lib().izb_quant_matmul(w.handle, mat, _p(x), x.stride(0), T, Mp, _p(aq), _p(asc), _p(out), out.stride(0), c_off, acc, _stream()))
    return out, aq, asc


def gemv(w: Weight, aq, asc, T: int, out=None, c_off: int = 0, acc: int = 0, mat: int = 0):
    import torch
    Mp = asc.shape[1]
    if out is None:
        out = torch.empty((T, w.N), dtype=torch.float32, device=aq.device)
    _check(lib().izb_gemv(w.handle, mat, _p(aq), _p(asc), T, Mp, _p(out), out.stride(0), c_off, acc, _stream()))
    return out


def gemm(w: Weight, aq, asc, M: int | None = None, out=None, c_off: int = 0, acc: int = 0, impl: int = GEMM_AUTO,
         mat: int = 0):
    import torch
    Mp = asc.shape[1]
    M = M or Mp
    if out is None:
        out = torch.empty((Mp, w.N // 2 if acc == 3 else w.N), dtype=torch.float32, device=aq.device)
    _check(lib().izb_gemm(w.handle, mat, _p(aq), _p(asc), M, Mp, _p(out), out.stride(0), c_off, acc, impl, _stream()))
    return out


NOALLOC_SCRATCH_BYTES = 24 << 20


def gemm_noalloc(w: Weight, aq, asc, M: int | None = None, out=None, c_off: int = 0, acc: int = 0, mat: int = 0, status=None):
    """izb_gemm_noalloc: the tensor-core GEMM with its scratch in the library's fixed device array (no allocation inside
    the call).  `out` must be given by callers that really cannot allocate; it is created here only for convenience."""
    import torch
    Mp = asc.shape[1]
    M = M or Mp
    if out is None:
        out = torch.empty((Mp, w.N // 2 if acc == 3 else w.N), dtype=torch.float32, device=aq.device)
    _check(lib().izb_gemm_noalloc(w.handle, mat, _p(aq), _p(asc), M, Mp, _p(out), out.stride(0), c_off, acc, _p(status), _stream()))
    return out


def block_dots(w: Weight, aq, M: int, impl: int = GEMM_CORE, mat: int = 0):
    import torch
    dots = torch.empty((M, w.N, w.K // 32), dtype=torch.int32, device=aq.device)
    _check(lib().izb_block_dots(w.handle, mat, _p(aq), M, _p(dots), impl, _stream()))
    return dots


def selfcheck(device: int = 0) -> None:
    _check(lib().izb_selfcheck(device))


def device_status(device: int = 0) -> int:
    w = C.c_uint32(0)
    rc = lib().izb_device_status(device, C.byref(w))
    if rc not in (0, -7):
        _check(rc)
    return w.value


def reserve(device: int, max_rows: int, max_K: int) -> None:
    """Size the per-device scratch arenas once, so that later GEMM / MoE / TP calls neither allocate nor synchronise."""
    _check(lib().izb_reserve(device, max_rows, max_K))


def tensor_peak(device: int, kind: int, iters: int = 4096, launches: int = 1) -> tuple[float, float]:
    """(Tops/s, SM clocks per MMA) of a TMEM-resident tcgen05.mma loop; kind 0 = kind::f16, 1 = kind::i8."""
    tops, clk = C.c_double(0), C.c_double(0)
    _check(lib().izb_tensor_peak(device, kind, iters, launches, C.byref(tops), C.byref(clk)))
    return tops.value, clk.value


def set_sm_limit(device: int, sms: int) -> None:
    """Cap the persistent GEMM's grid at `sms` multiprocessors (0 = all), so that a collective can run beside it."""
    _check(lib().izb_set_sm_limit(device, sms))


def debug_wait_test(spin_limit: int, skip_stage: int) -> None:
    """Diagnostics: the next tensor-core GEMM launch gives up its waits early and leaves one operand stage out."""
    _check(lib().izb_debug_wait_test(C.c_uint32(spin_limit), skip_stage))


def matmul_host(w: Weight, x_host, out_host, mat: int = 0) -> None:
    """The host-buffer call: x_host [M, K] f32 and out_host [M, N] f32 live in (ideally pinned) host memory."""
    M = x_host.shape[0]
    _check(lib().izb_matmul_host(w.handle, mat, _p(x_host), M, _p(out_host), _stream()))


# ---------------------------------------------------------------------------------------------- mixture of experts
def moe_route(logits, NU: int, shared_gate: bool = False):
    """logits [T, NE] (or [T, NE + 1] with the shared expert's gate logit last) -> ids, wts, counts (, sgate [T])."""
    import torch
    T = logits.shape[0]
    NE = logits.shape[1] - (1 if shared_gate else 0)
    ids = torch.empty((T, NU), dtype=torch.int32, device=logits.device)
    wts = torch.empty((T, NU), dtype=torch.float32, device=logits.device)
    counts = torch.empty((NE,), dtype=torch.int32, device=logits.device)
    sgate = torch.empty((T,), dtype=torch.float32, device=logits.device) if shared_gate else None
    _check(lib().izb_moe_route_ex(_p(logits), logits.stride(0), T, NE, NU, _p(ids), _p(wts), _p(counts), _p(sgate), _stream()))
    return (ids, wts, counts, sgate) if shared_gate else (ids, wts, counts)


def moe_sort(ids, wts, counts, TM: int, expert_range: tuple[int, int] | None = None):
    import torch
    T, NU = ids.shape
    NE = counts.shape[0]
    e0, e1 = expert_range or (0, NE)
    dev = ids.device
    max_tiles = (T * NU + TM - 1) // TM + NE
    offs = torch.empty((NE + 1,), dtype=torch.int32, device=dev)
    tiles = torch.zeros((1 + 3 * max_tiles,), dtype=torch.int32, device=dev)
    stok = torch.empty((T * NU,), dtype=torch.int32, device=dev)
    swt = torch.empty((T * NU,), dtype=torch.float32, device=dev)
    inv = torch.empty((T * NU,), dtype=torch.int32, device=dev)
    _check(lib().izb_moe_sort_ex(_p(ids), _p(wts), _p(counts), T, NE, NU, TM, e0, e1, _p(offs), _p(tiles), max_tiles, _p(stok),
                                 _p(swt), _p(inv), _stream()))
    return offs, tiles, max_tiles, stok, swt, inv


def moe_gateup(wg: Weight, wu: Weight | None, aq, asc, tiles, max_tiles: int, TM: int, stok, S: int):
    """wu = None: wg is an interleaved gate | up stack (gateup_weight) and one grouped GEMM computes both."""
    import torch
    h = torch.empty((S, wg.N if wu is not None else wg.N // 2), dtype=torch.float32, device=aq.device)
    _check(lib().izb_moe_gateup(wg.handle, wu.handle if wu is not None else None, _p(aq), _p(asc), asc.shape[1], _p(tiles), max_tiles, TM, _p(stok), _p(h),
                                _stream()))
    return h


def moe_down(wd: Weight, hq, hsc, tiles, max_tiles: int, TM: int, swt, S: int):
    import torch
    y = torch.empty((S, wd.N), dtype=torch.float32, device=hq.device)
    _check(lib().izb_moe_down(wd.handle, _p(hq), _p(hsc), hsc.shape[1], _p(tiles), max_tiles, TM, _p(swt), _p(y), _stream()))
    return y


def moe_combine(x, y, inv, NU: int, sh=None, sgate=None, partial: bool = False):
    T, E = x.shape
    _check(lib().izb_moe_combine_ex(_p(x), _p(y), _p(inv), T, NU, E, _p(sh), _p(sgate), int(partial), _stream()))
    return x


# ---------------------------------------------------------------------------------------------- tensor parallel
def tp_range(total: int, unit: int, nranks: int, rank: int) -> tuple[int, int]:
    b, e = C.c_int64(0), C.c_int64(0)
    _check(lib().izb_tp_range(C.c_int64(total), C.c_int64(unit), nranks, rank, C.byref(b), C.byref(e)))
    return b.value, e.value


def tp_add(x, parts):
    n = x.numel()
    _check(lib().izb_tp_add(_p(x), _p(parts), C.c_size_t(n), parts.shape[0], C.c_size_t(n), _stream()))
    return x


def p2p_push(copies, flags, value: int, stream=None) -> None:
    """copies: [(dst_ptr, src_ptr, nbytes)], flags: [ptr] -- raw device addresses (izb_p2p_push)."""
    n, m = len(copies), len(flags)
    dst = (C.c_void_p * max(n, 1))(*[c[0] for c in copies])
    src = (C.c_void_p * max(n, 1))(*[c[1] for c in copies])
    nb = (C.c_size_t * max(n, 1))(*[c[2] for c in copies])
    fl = (C.c_void_p * max(m, 1))(*flags)
    _check(lib().izb_p2p_push(n, dst, src, nb, m, fl, C.c_uint32(value), C.c_void_p(stream) if stream is not None else _stream()))


def p2p_wait(flags, value: int, stream=None) -> None:
    fl = (C.c_void_p * max(len(flags), 1))(*flags)
    _check(lib().izb_p2p_wait(len(flags), fl, C.c_uint32(value), C.c_void_p(stream) if stream is not None else _stream()))


def p2p_wait_host(timeout_ms: int, stream=None) -> None:
    """Bounded host wait for the stream (IzbError with status -7 on time-out; the stream's own waits stay queued)."""
    _check(lib().izb_p2p_wait_host(C.c_void_p(stream) if stream is not None else _stream(), timeout_ms))


def tp_scales_from_ranks(asc, stage, nranks: int, own: int, E: int) -> None:
    _check(lib().izb_tp_scales_from_ranks(_p(asc), _p(stage), nranks, own, E, _stream()))


class TpComm:
    """NCCL communicator of the library (izb_tp); the 128-byte id travels through torch.distributed."""

    def __init__(self, nranks: int, rank: int, device: int, timeout_ms: int = 0, max_ctas: int = 0):
        import torch
        import torch.distributed as dist
        idbuf = (C.c_char * 128)()
        if nranks > 1:
            if rank == 0:
                _check(lib().izb_tp_unique_id(idbuf))
            t = torch.frombuffer(bytearray(idbuf.raw), dtype=torch.uint8).clone()
            if dist.get_backend() == "nccl":
                t = t.cuda(device)
            dist.broadcast(t, src=0)
            idbuf = (C.c_char * 128).from_buffer_copy(bytes(t.cpu().numpy().tobytes()))
        self.handle = C.c_void_p(0)
        _check(lib().izb_tp_create_ex(nranks, rank, idbuf, device, timeout_ms, max_ctas, C.byref(self.handle)))
        self.nranks, self.rank, self.device = nranks, rank, device

    def allreduce_rows(self, x, part):
        rows, E = part.shape
        _check(lib().izb_tp_allreduce_rows(self.handle, _p(x), _p(part), rows, E, _stream()))
        return x

    def reduce_quant_gather(self, x, part, aq, asc, xsum=None):
        rows, E = part.shape
        _check(lib().izb_tp_reduce_quant_gather(self.handle, _p(x), _p(part), rows, E, _p(xsum), _p(aq), _p(asc), _stream()))
        return aq, asc

    def gather_logits(self, local, vocab: int, full=None):
        """local [rows, >= this rank's vocabulary rows] f32 -> full [rows, vocab] on every rank (rank order)."""
        import torch
        rows = local.shape[0]
        if full is None:
            full = torch.empty((rows, vocab), dtype=torch.float32, device=local.device)
        _check(lib().izb_tp_gather_logits(self.handle, _p(local), local.stride(0), rows, vocab, _p(full), full.stride(0), _stream()))
        return full

    def wait(self, timeout_ms: int) -> None:
        """Bounded wait for the current stream's work; raises IzbError (status -7) and aborts the communicator on time-out."""
        _check(lib().izb_tp_wait(self.handle, _stream(), timeout_ms))

    def abort(self) -> None:
        _check(lib().izb_tp_abort(self.handle))

    def close(self):
        if self.handle:
            lib().izb_tp_destroy(self.handle)
            self.handle = C.c_void_p(0)
