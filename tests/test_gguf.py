"""The GGUF reader (arcinferzero_b200/gguf.py) on files written by the seeded generator: the same files the reference's
own reader accepts (tools/ref_forward.cpp reads them in tests/golden/make_golden.py and in the benchmark's CPU baseline)."""
import os
import struct

import numpy as np
import pytest

from arcinferzero_b200 import gguf as G
from arcinferzero_b200 import synth as S


@pytest.fixture
def model(tmp_path):
    w4 = S.make_weight(12, 6, 512, 1)
    w8 = S.make_weight(8, 5, 256, 2)
    ex = S.make_weight(12, 3 * 4, 256, 3)  # three experts of 4 rows
    p = str(tmp_path / "m.gguf")
    S.write_gguf(p, {"blk.0.ffn_up.weight": (12, w4, 6, 512), "output.weight": (8, w8, 5, 256), "blk.0.ffn_up_exps.weight": (12, ex, 4, 256, 3)},
                 meta={"general.architecture": "qwen3", "general.alignment": 64, "qwen3.block_count": 1, "f": 0.5, "flag": True,
                       "tokenizer.ggml.tokens": ["a", "bc", ""], "ints": [1, -2, 3]})
    return p, w4, w8, ex


def test_reads_back_tensors_and_metadata(model):
    p, w4, w8, ex = model
    with G.GGUFFile(p) as g:
        assert g.kv["general.architecture"] == "qwen3" and g.kv["qwen3.block_count"] == 1 and g.kv["flag"] is True
        assert abs(g.kv["f"] - 0.5) < 1e-7 and g.kv["tokenizer.ggml.tokens"] == ["a", "bc", ""] and list(g.kv["ints"]) == [1, -2, 3]
        assert g.data_start % 64 == 0
        typ, rows, N, K, nm = g.weight_rows("blk.0.ffn_up.weight")
        assert (typ, N, K, nm) == (12, 6, 512, 1) and np.array_equal(rows, w4)
        typ, rows, N, K, nm = g.weight_rows("output.weight")
        assert (typ, N, K, nm) == (8, 5, 256, 1) and np.array_equal(rows, w8)
        typ, rows, N, K, nm = g.weight_rows("blk.0.ffn_up_exps.weight")
        assert (typ, N, K, nm) == (12, 4, 256, 3) and np.array_equal(rows, ex)
        with pytest.raises(KeyError):
            g.tensor("missing")


def test_rejects_malformed_files(model, tmp_path):
    p, *_ = model
    raw = open(p, "rb").read()
    bad = str(tmp_path / "bad.gguf")

    def write(b):
        with open(bad, "wb") as f:
            f.write(b)

    write(b"XXXX" + raw[4:])
    with pytest.raises(G.GGUFError, match="not a GGUF"):
        G.GGUFFile(bad)
    write(raw[:4] + struct.pack("<I", 1) + raw[8:])
    with pytest.raises(G.GGUFError, match="version"):
        G.GGUFFile(bad)
    write(raw[:60])  # cut inside the metadata
    with pytest.raises(G.GGUFError):
        G.GGUFFile(bad)
    write(raw[:-100])  # the last tensor's payload runs past the end
    with pytest.raises(G.GGUFError, match="out of range"):
        G.GGUFFile(bad)
    write(raw[:8] + struct.pack("<QQ", 1 << 40, 0) + raw[24:])  # a tensor count the file cannot hold
    with pytest.raises(G.GGUFError):
        G.GGUFFile(bad)
    write(b"")
    with pytest.raises(G.GGUFError):
        G.GGUFFile(bad)


@pytest.mark.gpu
def test_load_weight_from_file_matches_direct_upload(izb, model):
    import torch
    from oracle import oracle as O
    p, w4, _, _ = model
    x = S.make_act(3, 512, 5)
    aq, asc, _ = O.quantize_act(x, Mp=16)
    W = G.load_weight(p, "blk.0.ffn_up.weight")
    y = izb.gemv(W, torch.from_numpy(aq).cuda(), torch.from_numpy(asc).cuda(), 3).cpu().numpy()
    ref = O.matmul(12, w4, 512, aq, asc, 3, "gemv")
    assert np.max(np.abs(y - ref)) / np.max(np.abs(ref)) < 1e-5
    W.close()


def test_reference_reader_accepts_the_same_file(model):
    """When the reference's own code is compiled (oracle/_ref), its GGUF reader (src/gguf.h:306-359) parses the file with
    metadata, 64-byte alignment and a 3-D tensor, and multiplies with the tensor this reader returns."""
    from oracle import oracle as O
    if O.ref() is None:
        pytest.skip("oracle/_ref not built here")
    p, w4, _, _ = model
    x = S.make_act(2, 512, 9)
    y = O.ref_forward_matmul(p, "blk.0.ffn_up.weight", x, 6)
    aq, asc, _ = O.quantize_act(x)
    mine = O.matmul(12, w4, 512, aq, asc, 2, "f64")
    assert np.max(np.abs(y - mine)) / np.max(np.abs(mine)) < 1e-6


def test_further_weight_types_and_stacked_parts(tmp_path):
    """The reader sizes and returns the further block types (Q4_0, Q5_K, Q6_K, IQ4_XS) as izb_weight_create takes them, and
    collects the parts of a stacked weight (Q | K | V) with their type and K checked."""
    K = 512
    ws = {qt: S.make_weight(qt, 7 + qt % 3, K, 30 + qt) for qt in (2, 13, 14, 23)}
    q, k, v = S.make_weight(12, 8, K, 41), S.make_weight(12, 4, K, 42), S.make_weight(12, 4, K, 43)
    p = str(tmp_path / "t.gguf")
    tensors = {f"t{qt}.weight": (qt, w, w.shape[0], K) for qt, w in ws.items()}
    tensors.update({"attn_q.weight": (12, q, 8, K), "attn_k.weight": (12, k, 4, K), "attn_v.weight": (12, v, 4, K),
                    "other_k.weight": (12, S.make_weight(12, 4, 256, 44), 4, 256)})
    S.write_gguf(p, tensors)
    with G.GGUFFile(p) as g:
        for qt, w in ws.items():
            typ, rows, N, Kk, nm = g.weight_rows(f"t{qt}.weight")
            assert (typ, N, Kk, nm) == (qt, w.shape[0], K, 1) and np.array_equal(rows, w)
        typ, parts, Kk = G.stacked_rows(g, ["attn_q.weight", "attn_k.weight", "attn_v.weight"])
        assert (typ, Kk) == (12, K) and [a.shape[0] for a in parts] == [8, 4, 4]
        assert np.array_equal(np.concatenate(parts), np.concatenate([q, k, v]))
        with pytest.raises(G.GGUFError):
            G.stacked_rows(g, ["attn_q.weight", "other_k.weight"])     # another K
        with pytest.raises(G.GGUFError):
            G.stacked_rows(g, ["attn_q.weight", "t14.weight"])         # another type
        with pytest.raises(G.GGUFError):
            G.stacked_rows(g, [])
    # the reference's own reader multiplies with the Q6_K tensor of the same file
    from oracle import oracle as O
    if O.ref() is not None:
        x = S.make_act(2, K, 9)
        y = O.ref_forward_matmul(p, "t14.weight", x, ws[14].shape[0])
        aq, asc, _ = O.quantize_act(x)
        mine = O.matmul(14, ws[14], K, aq, asc, 2, "f64")
        assert np.max(np.abs(y - mine)) / np.max(np.abs(mine)) < 1e-6
