"""Child process of test_gpu_tc_fold.py: runs with IZB_GEMM_FOLD=1 (the library reads the variable once per process) and
compares the folded-scale Q4_K tensor-core GEMM with the CUDA-core GEMM and, on a small case, with the CPU oracle."""
import itertools
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import arcinferzero_b200 as izb  # noqa: E402
from arcinferzero_b200 import synth as S  # noqa: E402
from oracle import oracle as O  # noqa: E402


def main():
    assert os.environ.get("IZB_GEMM_FOLD") == "1"
    qt = izb.Q4_K
    # store modes, column offset, ragged rows, one to nine superblocks, 1..5 column tiles of 256
    for M, N, K in itertools.product((1, 17, 129, 1000), (256, 512, 1280), (256, 1024, 2304)):
        w = S.make_weight(qt, N, K, N + K)
        W = izb.Weight(qt, w, N, K)
        Mp = izb.pad_rows(M)
        aq, asc, _ = izb.quantize_act(torch.from_numpy(S.make_act(M, K, M + K)).cuda(), Mp=Mp)
        for acc in (0, 1, 2):
            base = torch.from_numpy(np.random.default_rng(acc).standard_normal((Mp, N + 8)).astype(np.float32)).cuda()
            a, b = base.clone(), base.clone()
            izb.profile_start()
            izb.gemm(W, aq, asc, M=M, out=a, c_off=4, acc=acc, impl=izb.GEMM_TC)
            assert "gemm_tc_fold" in izb.profile_stop(), "the folded kernel did not run"
            izb.gemm(W, aq, asc, M=M, out=b, c_off=4, acc=acc, impl=izb.GEMM_CORE)
            ra, rb = a[:M].cpu().numpy(), b[:M].cpu().numpy()
            err = np.max(np.abs(ra - rb)) / max(1e-30, np.max(np.abs(rb)))
            assert err < 1e-5, (M, N, K, acc, err)
            assert torch.equal(a[:, :4], base[:, :4]) and torch.equal(a[:, N + 4:], base[:, N + 4:]) and torch.equal(a[M:], base[M:])
        W.close()
    # scales spread over 30 binary orders inside a row, a zero row, a zero block: against the oracle in f64
    M, N, K = 96, 256, 2048
    rng = np.random.default_rng(5)
    x = S.make_act(M, K, 9) * np.exp2(rng.integers(-15, 15, size=(M, K // 32))).repeat(32, axis=1).astype(np.float32)
    x[3] = 0.0
    x[5, 64:96] = 0.0
    w = S.make_weight(qt, N, K, 11)
    W = izb.Weight(qt, w, N, K)
    Mp = izb.pad_rows(M)
    aq, asc, _ = izb.quantize_act(torch.from_numpy(x).cuda(), Mp=Mp)
    out = izb.gemm(W, aq, asc, M=M, impl=izb.GEMM_TC).cpu().numpy()[:M]
    ref = O.matmul(qt, w, K, aq.cpu().numpy(), asc.cpu().numpy(), M, "f64")
    err = float(np.abs(out - ref).max() / np.abs(ref).max())
    assert err < 1e-5, err
    rowerr = np.abs(out - ref).max(axis=1) / np.maximum(np.abs(ref).max(axis=1), 1e-30)
    assert rowerr.max() < 1e-5, rowerr.max()  # per row too: the row factor keeps small rows exact
    assert (out[3] == 0).all()
    W.close()
    # superblock scales d that are zero (with dmin != 0), denormal, negative: the min term travels through the accumulator
    # that is multiplied by d, so these are the cases that could go wrong
    M, N, K = 64, 256, 1024
    w = S.make_weight(qt, N, K, 21).reshape(N, K // 256, 144).copy()
    w[0, :, 0:2] = 0                       # d = 0 in every superblock of row 0
    w[1, 1, 0:2] = 0                       # ... and in one superblock of row 1
    w[2, :, 0] = 1; w[2, :, 1] = 0         # d = 2^-24 (smallest denormal)
    w[3, :, 1] |= 0x80                     # d negative
    w[130, 2, 0:2] = 0                     # (second half of the tile)
    w = w.reshape(N, -1)
    W = izb.Weight(qt, w, N, K)
    Mp = izb.pad_rows(M)
    aq, asc, _ = izb.quantize_act(torch.from_numpy(S.make_act(M, K, 22)).cuda(), Mp=Mp)
    out = izb.gemm(W, aq, asc, M=M, impl=izb.GEMM_TC).cpu().numpy()[:M]
    ref = O.matmul(qt, w, K, aq.cpu().numpy(), asc.cpu().numpy(), M, "f64")
    for col in (0, 1, 2, 3, 130):
        e = float(np.abs(out[:, col] - ref[:, col]).max() / max(np.abs(ref[:, col]).max(), 1e-30))
        assert e < 1e-5, (col, e)
    err = float(np.abs(out - ref).max() / np.abs(ref).max())
    assert err < 1e-5, err
    W.close()
    # several tiles per CTA (persistent walk), K = 5120
    M, N, K = 2048, 10240, 5120
    w = S.make_weight(qt, N, K, 1)
    W = izb.Weight(qt, w, N, K)
    aq, asc, _ = izb.quantize_act(torch.from_numpy(S.make_act(M, K, 2)).cuda(), Mp=M)
    a = izb.gemm(W, aq, asc, impl=izb.GEMM_TC)
    b = izb.gemm(W, aq, asc, impl=izb.GEMM_CORE)
    err = float((a - b).abs().max() / b.abs().max())
    assert err < 1e-5, err
    W.close()
    assert izb.device_status(0) == 0
    print("fold ok")


if __name__ == "__main__":
    main()
