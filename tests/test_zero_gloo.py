"""The sharding logic of ShardedAdafactor8Bit on two CPU ranks over gloo: partition,
flat-buffer views, in-place all-gather.  The per-rank optimizer is replaced by a stock
torch optimizer (the CUDA kernels need a GPU); the sharded run must equal a
single-process run bit for bit."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


SHAPES = [(37, 64), (128,), (300, 20), (5,), (64, 64), (1000,)]


def _make_params(seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.nn.Parameter(torch.randn(s, generator=g)) for s in SHAPES]


def _grads(step):
    g = torch.Generator().manual_seed(100 + step)
    return [torch.randn(s, generator=g) for s in SHAPES]


def _worker(rank, world, port, out):
    sys.path.insert(0, os.path.join(ROOT, "adafactor-8bit_b200"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from adafactor8bit.zero import ShardedAdafactor8Bit
        params = _make_params(1)
        opt = ShardedAdafactor8Bit(params, inner_factory=torch.optim.SGD, lr=0.1, momentum=0.9)
        owned = [i for i, o in enumerate(opt.owner) if o == rank]
        assert owned, "every rank owns something"
        assert all(p.data.data_ptr() >= opt.flat.data_ptr() for p in params)
        for step in range(3):
            for p, g in zip(params, _grads(step)):
                p.grad = g
            opt.step()
        states = sum(len(opt.state[p]) > 0 for p in params if p in opt.state)
        out[rank] = ([p.detach().clone() for p in params], list(opt.owner), states)
    finally:
        dist.destroy_process_group()


def test_two_rank_sharded_step_equals_single_process():
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
    ref = _make_params(1)
    sgd = torch.optim.SGD(ref, lr=0.1, momentum=0.9)
    for step in range(3):
        for p, g in zip(ref, _grads(step)):
            p.grad = g
        sgd.step()
    for rank in range(world):
        got, owner, states = out[rank]
        assert owner == out[0][1]
        assert states == sum(o == rank for o in owner)          # states exist only for owned tensors
        for a, b in zip(got, ref):
            assert torch.equal(a, b.detach())


def test_partition_is_balanced_and_deterministic():
    sys.path.insert(0, os.path.join(ROOT, "adafactor-8bit_b200"))
    from adafactor8bit.zero import partition_tensors
    numels = [65536000, 65536000] + [4194304, 524288, 524288, 4194304, 11534336, 11534336, 11534336, 2048, 2048] * 22 + [2048]
    for world in (1, 2, 4, 8):
        owner = partition_tensors(numels, world)
        loads = [sum(n for n, o in zip(numels, owner) if o == r) for r in range(world)]
        assert owner == partition_tensors(numels, world)
        assert max(loads) <= 1.02 * sum(numels) / world + 1


def test_split_parts_and_partition():
    sys.path.insert(0, os.path.join(ROOT, "adafactor-8bit_b200"))
    from adafactor8bit.zero import partition_tensors, split_parts
    assert split_parts([], 4) == []
    assert split_parts([10], 4) == [0]
    parts = split_parts([5, 5, 5, 5, 5, 5, 5, 5], 4)
    assert parts == [0, 0, 1, 1, 2, 2, 3, 3]
    parts = split_parts([100, 1, 1, 1], 2)
    assert parts[0] == 0 and parts[-1] == 1 and parts == sorted(parts)
    owner = partition_tensors([8, 7, 6, 5, 4, 3, 2, 1], 2)
    loads = [sum(n for n, o in zip([8, 7, 6, 5, 4, 3, 2, 1], owner) if o == r) for r in range(2)]
    assert loads == [18, 18]


def _ckpt_worker(rank, world, port, out, single_sd):
    sys.path.insert(0, os.path.join(ROOT, "adafactor-8bit_b200"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from adafactor8bit.zero import ShardedAdafactor8Bit
        params = _make_params(1)
        groups = [{"params": params[:2], "lr": 0.05}, {"params": params[2:]}]
        opt = ShardedAdafactor8Bit(groups, inner_factory=torch.optim.SGD, lr=0.1, momentum=0.9)
        for step in range(2):
            for p, g in zip(params, _grads(step)):
                p.grad = g
            opt.step()
        full = opt.full_state_dict(dst=0)
        assert (full is None) == (rank != 0)
        # a second sharded optimizer, started from the single-process checkpoint, continues like it
        params2 = _make_params(1)
        for p, q in zip(params2, single_sd["params"]):
            p.data.copy_(q)
        groups2 = [{"params": params2[:2], "lr": 0.05}, {"params": params2[2:]}]
        opt2 = ShardedAdafactor8Bit(groups2, inner_factory=torch.optim.SGD, lr=0.1, momentum=0.9)
        import copy
        opt2.load_full_state_dict(copy.deepcopy(single_sd["sd"]))    # (the spawned processes share the parent's tensors)
        for p, g in zip(params2, _grads(2)):
            p.grad = g
        opt2.step()
        out[rank] = (full, [p.detach().clone() for p in params2])
    finally:
        dist.destroy_process_group()


def test_full_state_dict_matches_single_process_layout():
    """The merged checkpoint of two ranks equals what one process saves (indices, options, momentum
    buffers), and a sharded optimizer loaded from a one-process checkpoint continues like it."""
    def single(steps):
        ref = _make_params(1)
        sgd = torch.optim.SGD([{"params": ref[:2], "lr": 0.05}, {"params": ref[2:]}], lr=0.1, momentum=0.9)
        for step in range(steps):
            for p, g in zip(ref, _grads(step)):
                p.grad = g
            sgd.step()
        return ref, sgd
    ref2, sgd2 = single(2)
    single_sd = {"sd": sgd2.state_dict(), "params": [p.detach().clone() for p in ref2]}
    world, port = 2, _free_port()
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_ckpt_worker, args=(world, port, out, single_sd), nprocs=world, join=True)
    full = out[0][0]
    want = single_sd["sd"]
    assert sorted(full["state"]) == sorted(want["state"])
    for idx, st in want["state"].items():
        assert torch.equal(full["state"][idx]["momentum_buffer"], st["momentum_buffer"])
    assert [g["params"] for g in full["param_groups"]] == [g["params"] for g in want["param_groups"]]
    assert [g["lr"] for g in full["param_groups"]] == [0.05, 0.1]
    ref3, _ = single(3)
    for rank in range(world):
        for a, b in zip(out[rank][1], ref3):
            assert torch.equal(a, b.detach())
