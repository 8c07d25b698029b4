"""The data-parallel gradient sum on two gloo ranks, and its bucket plan."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from dism_b200.data_parallel import bucket_plan, sum_gradients


def test_bucket_plan_keeps_order_and_limit():
    sizes = [10, 10, 10, 50, 5, 5, 100, 1]
    plan = bucket_plan(sizes, 30)
    assert plan == [(0, 3), (3, 4), (4, 6), (6, 7), (7, 8)]
    assert bucket_plan([], 30) == [] and bucket_plan([7], 1) == [(0, 1)]
    covered = [i for first, end in plan for i in range(first, end)]
    assert covered == list(range(len(sizes)))


def _rank(rank, world, port, results):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    torch.manual_seed(0)
    shapes = [(64, 64), (3,), (1000, 40), (17,), (5, 5)]
    parameters = [torch.nn.Parameter(torch.zeros(s, dtype=torch.float32 if i != 3 else torch.float64)) for i, s in enumerate(shapes)]
    for index, parameter in enumerate(parameters):
        if index == 1 and rank == 0:
            continue      # used on rank 1 only: rank 0 contributes zeros
        if index == 4:
            continue      # used nowhere: stays None
        parameter.grad = torch.full_like(parameter, float(rank + 1) * (index + 1))
    sum_gradients(parameters, bucket_bytes=64 * 64 * 4 + 16)  # forces several buckets
    expected = {0: 3., 1: 4., 2: 9., 3: 12.}
    ok = all(torch.equal(parameters[i].grad, torch.full_like(parameters[i], value)) for i, value in expected.items())
    results[rank] = ok and parameters[4].grad is None
    dist.destroy_process_group()


def test_gradient_sum_two_ranks():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        port = s.getsockname()[1]
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_rank, args=(2, port, results), nprocs=2, join=True)
    assert results[0] and results[1]


def test_model_of_the_benchmark_has_the_stated_size():
    """The model workload's architecture (depth 20, width 1280, 10 heads of 128, vocabulary 65536), built on the meta
    device: parameter count as `bench.py --workload model` reports it, and the DISM layer's own parameters."""
    import torch
    from dism_b200.model import DismLM
    with torch.device('meta'):
        model = DismLM(depth=20, width=1280, heads=10, head_dim=128, vocab=65536)
    assert sum(p.numel() for p in model.parameters()) == 603586760
    mixer = model.blocks[0].mixer
    assert mixer.q_vocab.shape == (10, 512, 128) and mixer.k_vocab.shape == (10, 512, 128)
    assert mixer.sq_proj.weight.shape == (10 * 32, 1280) and mixer.log_sel_tau.shape == (10,)
