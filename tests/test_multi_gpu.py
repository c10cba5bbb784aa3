"""Multi-GPU parity (needs >= 2 GPUs; skipped otherwise): expert-parallel MoE, column-parallel and
row-parallel W4A16 and row-parallel W8A8 against the single-GPU path, one process per GPU.  The checks
themselves live in ``mindpipe_b200.verify`` (``bench.py`` runs them too, inside its multi-rank job); here
the row-parallel W8A8 result is additionally pinned to the CPU oracle's arithmetic."""
import datetime
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


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    # a short collective timeout: if one rank fails, the others error out instead of waiting for it
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=120))
    try:
        from mindpipe_b200.verify import verify_multi_gpu
        from oracle import pseudo_quant as O
        ret[rank] = verify_multi_gpu(rank, world, torch.device("cuda", rank), oracle=O)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_expert_parallel_column_parallel_and_row_parallel_match_single_gpu():
    world = min(torch.cuda.device_count(), 4)
    while 8 % world:
        world -= 1
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert all(all(v.values()) for v in dict(ret).values()), dict(ret)
