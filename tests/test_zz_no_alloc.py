"""izb_gemm_noalloc, the GEMM entry point that allocates nothing (its scratch is a fixed array inside the library's device
image), against izb_gemm on the same inputs.  Collected last on purpose: with `-x` every other test has already run if
this one fails.  The calls go through the C ABI; outputs are pre-allocated by the test, as a caller that cannot allocate
would do."""
import ctypes as C

import numpy as np
import pytest

from arcinferzero_b200 import synth as S
from oracle import oracle as O

pytestmark = pytest.mark.gpu
TOL = 1e-5


def rel(got, ref):
    return float(np.abs(got.astype(np.float64) - ref.astype(np.float64)).max() / np.abs(ref).max())


@pytest.mark.parametrize("qt", [12, 8])
def test_noalloc_gemm_matches_gemm_on_two_calls_in_a_row(izb, qt):
    import torch
    assert torch.cuda.is_available()
    N, K = 256, 1280
    w = S.make_weight(qt, N, K, 40 + qt)
    W = izb.Weight(qt, w, N, K)
    status = torch.full((1,), 123, dtype=torch.int32, device="cuda")  # garbage: the call must clear it
    free_after_warmup = None
    # two calls in a row on different shapes and data: the second must not see anything of the first in the shared array
    for call, (M, seed) in enumerate(((300, 1), (130, 2))):
        Mp = izb.pad_rows(M)
        x = S.make_act(M, K, seed)
        aq, asc, _ = izb.quantize_act(torch.from_numpy(x).cuda(), Mp=Mp)
        want = izb.gemm(W, aq, asc, M=M, impl=izb.GEMM_TC)
        out = torch.full((Mp, N), float("nan"), dtype=torch.float32, device="cuda")
        izb.gemm_noalloc(W, aq, asc, M=M, out=out, status=status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        got, ref = out.cpu().numpy(), want.cpu().numpy()
        assert np.isnan(got[M:]).all()
        assert rel(got[:M], ref[:M]) < TOL, (call, rel(got[:M], ref[:M]))
        # and against the CPU oracle
        assert rel(got[:M], O.matmul(qt, w, K, aq.cpu().numpy(), asc.cpu().numpy(), M, "f64")) < TOL
        # store mode 1 (add) through the same entry point, library-owned status word
        base = torch.ones((Mp, N), dtype=torch.float32, device="cuda")
        izb.gemm_noalloc(W, aq, asc, M=M, out=base, acc=1)
        assert rel(base.cpu().numpy()[:M] - 1.0, ref[:M]) < 1e-4
        assert izb.device_status(0) == 0  # (covers the library-owned status word of the call above)
        # The first iteration was the warm-up (the CUDA runtime loads a kernel's code at its first launch); from then on the
        # entry point must leave the device's free memory exactly as it found it.
        torch.cuda.synchronize()
        if free_after_warmup is None:
            free_after_warmup = torch.cuda.mem_get_info()[0]
        else:
            out2 = torch.empty((Mp, N), dtype=torch.float32, device="cuda")
            torch.cuda.synchronize()
            before = torch.cuda.mem_get_info()[0]
            for _ in range(3):
                izb.gemm_noalloc(W, aq, asc, M=M, out=out2, status=status)
            torch.cuda.synchronize()
            assert torch.cuda.mem_get_info()[0] == before
    W.close()


def test_noalloc_gemm_rejects_what_does_not_fit(izb):
    import torch
    N, K = 128, 5120
    W = izb.Weight(12, S.make_weight(12, N, K, 3), N, K)
    M = 4096  # 32 tiles x (20 x 5 x 16 KiB + 160 x 0.5 KiB) = 52 MiB > 24 MiB
    aq = torch.zeros((M, K), dtype=torch.int8, device="cuda")
    asc = torch.zeros((K // 32, M), dtype=torch.float32, device="cuda")
    out = torch.zeros((M, N), dtype=torch.float32, device="cuda")
    n0 = izb.launch_count()
    with pytest.raises(izb.IzbError) as e:
        izb.gemm_noalloc(W, aq, asc, out=out)
    assert e.value.status == -10 and "scratch bytes" in str(e.value)
    assert izb.launch_count() == n0  # nothing was launched
    W.close()
