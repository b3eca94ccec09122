"""Multi-GPU tests (skipped with fewer than two devices): context parallelism through the C
entry point moba_cp_forward (means exchanged, K/V rows of earlier ranks received over NCCL while
the gating runs) gives the rows and the selection of the single-device run, bit for bit.
NVLS is switched off in NCCL for these short-lived child processes."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, total, chunk, topk, result):
    from baselinebenchmark_b200 import parallel, sharding
    from oracle import moba_oracle as O
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        q, k, v, cu = O.make_inputs([total], 8, 2, 128, chunk, seed=31)
        dev = torch.device("cuda", rank)
        qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
        full, _, full_sel = parallel.moba_forward(qd, kd, vd, torch.from_numpy(cu).to(dev), total, chunk, topk,
                                                  return_selected=True)
        lo, hi = sharding.context_window(total, chunk, world, rank)
        # the function interface (agreement step, then the C entry point moba_cp_forward) ...
        out = sharding.moba_context_parallel(qd[lo:hi].contiguous(), kd[lo:hi].contiguous(),
                                             vd[lo:hi].contiguous(), total, chunk, topk)
        # ... and the object a training or serving loop keeps, twice in a row on the same buffers
        cp = sharding.ContextParallel(total, 2, 128, chunk, torch.bfloat16, dev)
        cp.k_rows.copy_(kd[lo:hi])
        cp.v_rows.copy_(vd[lo:hi])
        ok = True
        for _ in range(2):
            out2, sel2 = cp.forward(qd[lo:hi].contiguous(), topk, return_selected=True)
            cp.finish(timeout_s=60.0)
            ok = ok and bool(torch.equal(out2, full[lo:hi])) and bool(torch.equal(sel2, full_sel[:, :, lo:hi]))
        # rows of the earlier ranks arrived in place; later ranks' rows were never sent
        ok = ok and bool(torch.equal(cp.k_full[:hi], kd[:hi])) and bool(torch.equal(cp.v_full[:hi], vd[:hi]))
        torch.cuda.synchronize()
        result[rank] = bool(torch.equal(out, full[lo:hi])) and ok
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("total,chunk,topk", [(8192, 512, 4), (5000, 256, 8)])
def test_context_parallel_nccl(total, chunk, topk):
    world = min(torch.cuda.device_count(), 4)
    with mp.Manager() as mgr:
        result = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), total, chunk, topk, result), nprocs=world, join=True)
        assert all(result[r] for r in range(world))
