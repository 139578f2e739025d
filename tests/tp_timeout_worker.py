"""One rank of the collective time-out check (two GPUs, launched by torch.distributed.run; rendezvous and the hand-shake
between the ranks go over gloo on the host).

Step 1: both ranks sum a small tensor through the library's communicator, created with a time-out (non-blocking NCCL).
Step 2: rank 1 stays away from the next collective -- it leaves BETWEEN steps, with nothing of its own in flight, and only
waits on the host.  Rank 0 enqueues the collective, and its bounded wait (izb_tp_wait) must give up, abort the communicator
(which ends the collective that is waiting for the missing peer) and report IZB_ERR_TIMEOUT; the CUDA context must still
work afterwards and the aborted communicator must refuse further collectives."""
import datetime
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(__file__), ".."))


def main() -> int:
    import torch
    import torch.distributed as dist

    import arcinferzero_b200 as izb
    world, rank, local = int(os.environ["WORLD_SIZE"]), int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    assert world == 2
    torch.cuda.set_device(local)
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=120))
    comm = izb.TpComm(world, rank, local, timeout_ms=20000)
    rows, E = 64, 256
    x = torch.zeros((rows, E), dtype=torch.float32, device="cuda")
    part = torch.full((rows, E), float(rank + 1), dtype=torch.float32, device="cuda")
    comm.allreduce_rows(x, part)
    comm.wait(20000)
    assert float(x[0, 0].item()) == 3.0 and float(x[-1, -1].item()) == 3.0
    dist.barrier()
    if rank == 1:
        dist.barrier()        # rank 0 is done with its time-out
        comm.abort()          # nothing of this rank was in flight
        comm.close()
        print("TP_TIMEOUT_OK rank=1", flush=True)
    else:
        part.fill_(1.0)
        comm.allreduce_rows(x, part)   # the peer never joins this one
        try:
            comm.wait(1500)
            raise AssertionError("the wait returned although the peer never joined")
        except izb.IzbError as e:
            assert e.status == -7, e
        # the context is alive: a kernel of the library runs and gives the right answer
        y = torch.ones((16, 256), dtype=torch.float32, device="cuda")
        aq, asc, _ = izb.quantize_act(y, Mp=16)
        torch.cuda.synchronize()
        assert int(aq[0, 0].item()) == 127 and abs(float(asc[0, 0].item()) - 1.0 / 127.0) < 1e-9
        try:
            comm.allreduce_rows(x, part)
            raise AssertionError("an aborted communicator accepted a collective")
        except izb.IzbError as e:
            assert e.status == -6, e
        dist.barrier()
        comm.close()
        print("TP_TIMEOUT_OK rank=0", flush=True)
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
