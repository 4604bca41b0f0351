"""Batch sharding and the logits all-gather, rehearsed on CPU ranks (gloo, world size 2)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from convnn_b200.sharded import gather_logits, shard_bounds, shared_candidates, sharded_forward


def test_shard_bounds_cover_and_balance():
    for n in (1, 7, 8, 256, 257):
        for w in (1, 2, 4, 8):
            spans = [shard_bounds(n, w, r) for r in range(w)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(w - 1))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, total, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        images = torch.randn(total, 6)
        model = torch.nn.Linear(6, 5)
        torch.manual_seed(1)
        with torch.no_grad():
            model.weight.copy_(torch.randn(5, 6))
            model.bias.zero_()
        out = sharded_forward(model, images)
        cand = shared_candidates(65, 16, torch.device("cpu"), seed=3)
        q.put((rank, out, cand))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("total", [8, 7])
def test_two_ranks_reproduce_single_process(total):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, total, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    torch.manual_seed(0)
    images = torch.randn(total, 6)
    torch.manual_seed(1)
    w = torch.randn(5, 6)
    want = images @ w.t()
    for rank, out, cand in got:
        assert out.shape == want.shape
        assert torch.allclose(out, want, atol=1e-6)
    assert torch.equal(got[0][2], got[1][2])            # every rank selects from the same candidates


def test_gather_is_identity_without_process_group():
    x = torch.randn(3, 4)
    assert gather_logits(x, 3) is x


@pytest.mark.skipif(torch.cuda.is_available(), reason="on a GPU box the call does bind the process")
def test_host_binding_is_a_no_op_without_a_gpu():
    """bind_host_to_device only narrows the process's CPU affinity when NVML knows the device;
    on a machine without one it reports False and leaves the affinity alone."""
    import os
    from convnn_b200.sharded import bind_host_to_device
    before = os.sched_getaffinity(0)
    assert bind_host_to_device("cuda:0") is False
    assert os.sched_getaffinity(0) == before
