"""Tensor-parallel stack on GPUs: one rank in-process, and all visible GPUs (2..8) as torch.distributed.run children with
NCCL.  Every stage is checked against the oracle inside tests/tp_gpu_worker.py."""
import os
import socket
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
pytestmark = pytest.mark.gpu


def test_stack_one_rank(izb):
    sys.path.insert(0, HERE)
    import tp_gpu_worker as W
    for mode in ("allreduce", "rs_quant_ag"):
        W.check_mode(mode, 1, 0, 0)
    W.check_mode("rs_quant_ag", 1, 0, 0, chunks=2, balance=True)
    W.check_head_gather(1, 0, 0)


def test_stack_all_visible_gpus(izb):
    import torch
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("one GPU visible: the multi-rank run needs at least two")
    n = 1 << (n.bit_length() - 1)
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "tp_gpu_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("TP_WORKER_OK") == 5 * n, r.stdout[-3000:]


def test_collective_with_a_missing_peer_times_out_and_aborts(izb):
    """Failure detection in the C ABI (izb_tp_create_ex with a time-out, izb_tp_wait, izb_tp_abort): two ranks, the second
    stays away from a collective between steps; the first rank's bounded wait must end with IZB_ERR_TIMEOUT, not hang."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("one GPU visible: the time-out check needs two ranks")
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "tp_timeout_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("TP_TIMEOUT_OK") == 2, r.stdout[-3000:]


def test_peer_transport_calls_on_one_gpu(izb):
    """izb_p2p_push / izb_p2p_wait / izb_p2p_wait_host with both ends on one GPU (the pointers are plain device addresses):
    copies and flag writes in stream order, a wait on a flag that is ALREADY raised, the host wait on a stream that
    drains.  A wait for a flag that a stream of the same device raises later is not a valid use (CUDA may order the two
    streams the wrong way round) and is not exercised; the two-rank run covers waits that another GPU satisfies."""
    import torch
    dev = torch.device("cuda", 0)
    src = torch.arange(1 << 20, dtype=torch.float32, device=dev)
    dst = torch.zeros_like(src)
    flags = torch.zeros(8, dtype=torch.int32, device=dev)
    fp = flags.data_ptr()
    side = torch.cuda.Stream(device=dev)
    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        izb.p2p_push([(dst.data_ptr(), src.data_ptr(), src.numel() * 4)], [fp, fp + 8], 3)
    izb.p2p_wait_host(5000, stream=side.cuda_stream)
    assert flags.tolist() == [3, 0, 3, 0, 0, 0, 0, 0] and torch.equal(dst, src)
    with torch.cuda.stream(side):
        izb.p2p_wait([fp, fp + 8], 2)      # already satisfied (the flags only grow: >=)
        dst.mul_(2.0)
    izb.p2p_wait_host(5000, stream=side.cuda_stream)
    assert torch.equal(dst, src * 2)
    with pytest.raises(izb.IzbError):
        izb.p2p_wait([fp + 1], 1)           # not 4-byte aligned
    with pytest.raises(izb.IzbError):
        izb.p2p_wait_host(0)
    assert izb.device_status(0) == 0
