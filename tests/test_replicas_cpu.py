"""Multi-GPU path = independent replicas; its only cross-rank logic (sum of tokens, max
of times) is exercised here with two gloo ranks on CPU."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out):
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, os.path.join(root, "cpm.cu_b200"))
    from cpmcu.replicas import combine_ranks, replica_seed
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    tokens, dev_s, wall = (100 + 10 * rank), (1.0 + rank), (2.0 - 0.5 * rank)
    total, dmax, wmax = combine_ranks(tokens, dev_s, wall, dist, "cpu")
    dist.barrier()
    out[rank] = (total, dmax, wmax, replica_seed(100, rank))
    dist.destroy_process_group()


def test_two_replicas_aggregate_tokens_and_slowest_time():
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    for rank in range(world):
        total, dmax, wmax, seed = out[rank]
        assert total == 210.0 and dmax == 2.0 and wmax == 2.0
        assert seed == 100 + rank


def test_single_process_passthrough():
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, os.path.join(root, "cpm.cu_b200"))
    from cpmcu.replicas import combine_ranks
    assert combine_ranks(7, 0.5, 0.75, None) == (7.0, 0.5, 0.75)
