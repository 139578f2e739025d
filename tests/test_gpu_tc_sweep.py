"""The tcgen05 GEMM against the CUDA-core GEMM (itself bit-exact with the oracle's reference order) over a grid of shapes:
ragged row counts, one to nine superblocks of K, one to nine column tiles, both weight types, every store mode, with a
column offset; everything outside the written region must stay untouched."""
import itertools

import numpy as np
import pytest

from arcinferzero_b200 import synth as S

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("qt", [12, 8])
def test_tensor_core_gemm_equals_core_gemm_over_shapes(izb, qt):
    import torch
    for M, N, K in itertools.product((1, 17, 128, 129, 1000), (128, 256, 1152), (256, 512, 2304)):
        w = S.make_weight(qt, N, K, N + K + qt)
        W = izb.Weight(qt, w, N, K)
        x = torch.from_numpy(S.make_act(M, K, M + K)).cuda()
        Mp = izb.pad_rows(M)
        aq, asc, _ = izb.quantize_act(x, Mp=Mp)
        for acc in (0, 1, 2):
            base = torch.from_numpy(np.random.default_rng(acc).standard_normal((Mp, N + 8)).astype(np.float32)).cuda()
            a, b = base.clone(), base.clone()
            izb.gemm(W, aq, asc, M=M, out=a, c_off=4, acc=acc, impl=izb.GEMM_TC)
            izb.gemm(W, aq, asc, M=M, out=b, c_off=4, acc=acc, impl=izb.GEMM_CORE)
            ra, rb = a[:M].cpu().numpy(), b[:M].cpu().numpy()
            err = np.max(np.abs(ra - rb)) / max(1e-30, np.max(np.abs(rb)))
            assert err < 1e-5, (qt, M, N, K, acc, err)
            assert torch.equal(a[:, :4], base[:, :4]) and torch.equal(a[:, N + 4:], base[:, N + 4:]) and torch.equal(a[M:], base[M:]), (qt, M, N, K, acc)
        W.close()
    assert izb.device_status(0) == 0
