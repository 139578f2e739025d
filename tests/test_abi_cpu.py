"""CPU-side checks of the C ABI: the library loads, exports every declared symbol, validates arguments before touching
a device, and fails loudly (no fallback) when there is no GPU."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import arcinferzero_b200 as izb
from oracle import oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    hdr = open(os.path.join(ROOT, "include", "izb200.h")).read()
    declared = set(re.findall(r"\b(izb_[a-z0-9_]+)\s*\(", hdr))
    assert declared == set(izb.SYMBOLS), declared ^ set(izb.SYMBOLS)
    L = izb.lib()
    for s in declared:
        assert hasattr(L, s), s


def test_status_strings():
    L = izb.lib()
    assert L.izb_status_string(0) == b"ok"
    for code in range(-10, 0):
        assert L.izb_status_string(code) not in (b"ok", b"unknown status")


def test_tp_range_matches_oracle_and_reference_rule():
    for total, unit in ((17408, 256), (8, 1), (151936, 16), (5120, 256), (40, 1)):
        for n in (1, 2, 3, 4, 8):
            for r in range(n):
                assert izb.tp_range(total, unit, n, r) == O.tp_range(total, unit, n, r)
    with pytest.raises(izb.IzbError):
        izb.tp_range(10, 0, 2, 0)
    with pytest.raises(izb.IzbError):
        izb.tp_range(10, 1, 2, 2)


def test_arguments_are_validated_before_any_launch():
    L = izb.lib()
    x = np.zeros((16, 256), np.float32)
    aq = np.zeros((16, 256), np.int8)
    asc = np.zeros((8, 16), np.float32)
    p = lambda a: C.c_void_p(a.ctypes.data)
    assert L.izb_quantize_act(None, 256, 16, 16, 256, p(aq), p(asc), None, None) == -1       # null
    assert L.izb_quantize_act(p(x), 256, 16, 16, 200, p(aq), p(asc), None, None) == -2       # K % 256
    assert L.izb_quantize_act(p(x), 256, 16, 24, 256, p(aq), p(asc), None, None) == -2       # Mp % 16
    assert L.izb_quantize_act(p(x), 256, 17, 16, 256, p(aq), p(asc), None, None) == -2       # M > Mp
    assert L.izb_quantize_act(p(x), 255, 16, 16, 256, p(aq), p(asc), None, None) == -2       # ldx < K
    assert L.izb_quantize_act(p(x), 258, 16, 16, 256, p(aq), p(asc), None, None) == -4       # ldx % 4
    assert b"multiple of 256" in L.izb_last_error() or b"aligned" in L.izb_last_error()
    h = C.c_void_p(0)
    assert L.izb_weight_create(7, p(x), 1, 16, 256, 0, C.byref(h)) == -3                       # type
    assert L.izb_weight_create(12, p(x), 1, 16, 100, 0, C.byref(h)) == -2                      # K
    assert L.izb_weight_create_slice(12, p(x), 1, 16, 512, 0, 16, 128, 512, 0, C.byref(h)) == -2  # k0 % 256
    assert L.izb_gemv(None, 0, p(aq), p(asc), 1, 16, p(x), 16, 0, 0, None) == -1
    assert L.izb_moe_route(p(x), 8, 4, 600, 8, p(x), p(x), p(x), None) == -2                  # NE > 512


def test_no_gpu_means_an_error_not_a_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    L = izb.lib()
    rows = np.zeros((16, 144), np.uint8)
    h = C.c_void_p(0)
    rc = L.izb_weight_create(12, C.c_void_p(rows.ctypes.data), 1, 16, 256, 0, C.byref(h))
    assert rc == -5 and not h.value
    assert b"no CPU path" in L.izb_last_error() or b"sm_100a" in L.izb_last_error()
    with pytest.raises(izb.IzbError):
        izb.Weight(12, rows, 16, 256)


def test_host_decoder_of_further_weight_types_matches_the_oracle():
    """izb_weight_decode_host (the loader's decoder, no device needed) against the oracle's restatement of the reference's
    decode_sb generic view, field by field; Q6_K, which stays packed on the device, as the file's bytes in 224; Q4_0
    against its Q8_0 rewrite."""
    import numpy as np
    import arcinferzero_b200 as izb
    from arcinferzero_b200 import synth as S
    from oracle import oracle as O
    K, N = 768, 7
    w = S.make_weight(14, N, K, 84)
    dev = izb.weight_decode_host(14, w, K).reshape(N, K // 256, 224)
    assert (dev[:, :, :210] == w.reshape(N, K // 256, 210)).all() and (dev[:, :, 210:] == 0).all()
    for qt in (13, 23):
        w = S.make_weight(qt, N, K, 70 + qt)
        dev = izb.weight_decode_host(qt, w, K).reshape(N, K // 256, 304)
        sbb = S.sb_bytes(qt)
        for n in range(N):
            for s in range(K // 256):
                wd, wdmin, wsc, wmn, has_min, q = O.decode_generic_sb(qt, w[n, sbb * s:sbb * (s + 1)])
                b = dev[n, s]
                assert b[0:4].view(np.float32)[0] == np.float32(wd) and b[4:8].view(np.float32)[0] == np.float32(wdmin)
                assert (b[8:24].view(np.int8) == wsc).all() and (b[24:40] == wmn).all() and (b[40:48] == 0).all()
                assert (b[48:304].view(np.int8) == q).all()
    w = S.make_weight(2, N, K, 72)
    assert (izb.weight_decode_host(2, w, K) == O.q4_0_as_q8_0(w)).all()


def test_gateup_interleave_on_the_host():
    """izb_gateup_interleave_host (the row order izb_weight_create_gateup uploads): per matrix, 32 gate rows then the 32 up
    rows of the same FFN channels, and so on; shapes it cannot take are refused."""
    import numpy as np
    import pytest
    import arcinferzero_b200 as izb
    from arcinferzero_b200 import synth as S
    for qt in (12, 8, 2):
        n_mats, F, K = 3, 128, 512
        g, u = S.make_weight(qt, n_mats * F, K, 90 + qt), S.make_weight(qt, n_mats * F, K, 91 + qt)
        out = izb.gateup_interleave_host(qt, g, u, F, K, n_mats=n_mats)
        per = g.shape[1]
        ref = np.stack([g.reshape(n_mats, F // 32, 32, per), u.reshape(n_mats, F // 32, 32, per)], axis=2).reshape(n_mats * 2 * F, per)
        assert out.shape == ref.shape and (out == ref).all()
    with pytest.raises(izb.IzbError):
        izb.gateup_interleave_host(12, g[:96], u[:96], 96, K)          # F % 64
    with pytest.raises(izb.IzbError):
        izb.gateup_interleave_host(99, g, u, F, K, n_mats=n_mats)       # unknown type
