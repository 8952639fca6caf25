"""The sharding logic of ShardedAdafactor8Bit without a GPU: the layout of the flat parameter space
(cells, legal cuts, whole tensors), the order of the collectives, the round schedule of the launch
plans, and, on two CPU ranks over gloo, a sharded run with cut tensors that must equal a
single-process run bit for bit.  The per-rank optimizer of the gloo runs is a stock torch optimizer
(the CUDA kernels need a GPU); it sees the pieces as ordinary parameters."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "adafactor-8bit_b200"))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


SHAPES = [(37, 64), (128,), (300, 20), (5,), (64, 64), (10000,), (3, 4, 5), (9000, 2), (1000,)]


def _make_params(seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.nn.Parameter(torch.randn(s, generator=g)) for s in SHAPES]


def _grads(step):
    g = torch.Generator().manual_seed(100 + step)
    return [torch.randn(s, generator=g) for s in SHAPES]


def _worker(rank, world, port, out, parts):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from adafactor8bit.zero import ShardedAdafactor8Bit
        params = _make_params(1)
        opt = ShardedAdafactor8Bit(params, inner_factory=torch.optim.SGD, parts=parts, min_piece=1, lr=0.1, momentum=0.9)
        lo, hi = opt.flat.data_ptr(), opt.flat.data_ptr() + opt.flat.numel() * 4
        assert all(lo <= p.data.data_ptr() < hi and p.data.is_contiguous() for p in params)
        for step in range(3):
            for p, g in zip(params, _grads(step)):
                p.grad = g
            opt.step()
            assert opt.gather_log == list(range(opt.parts))
        n_states = sum(len(st) > 0 for st in opt.state.values())
        out[rank] = ([p.detach().clone() for p in params], [list(x) for x in opt.pieces_of], opt.cell, n_states,
                     len(opt._local), opt.owned_numel)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("parts", [1, 3])
def test_two_rank_sharded_step_equals_single_process(parts):
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, port, out, parts), nprocs=world, join=True)
    ref = _make_params(1)
    sgd = torch.optim.SGD(ref, lr=0.1, momentum=0.9)
    for step in range(3):
        for p, g in zip(ref, _grads(step)):
            p.grad = g
        sgd.step()
    pieces = out[0][1]
    assert pieces == out[1][1] and out[0][2] == out[1][2]            # every rank derives the same layout
    assert any(len(lst) > 1 for lst in pieces), "the case must cut a tensor"
    total = sum(p.numel() for p in ref)
    assert out[0][5] + out[1][5] == total                              # every element has exactly one owner
    for rank in range(world):
        got, _, _, n_states, n_local, _ = out[rank]
        assert n_states == n_local                                     # states exist for the rank's pieces only
        for a, b in zip(got, ref):
            assert torch.equal(a, b.detach())


def _tinyllama():
    per_layer = [(2048, 2048), (256, 2048), (256, 2048), (2048, 2048), (5632, 2048), (5632, 2048), (2048, 5632), (2048,), (2048,)]
    return [(32000, 2048)] + per_layer * 22 + [(2048,), (32000, 2048)]


def _llama3_8b():
    per_layer = [(4096, 4096), (1024, 4096), (1024, 4096), (4096, 4096), (14336, 4096), (14336, 4096), (4096, 14336), (4096,), (4096,)]
    return [(128256, 4096)] + per_layer * 32 + [(4096,), (128256, 4096)]


def _check_layout(shapes, rules, n_cells):
    from adafactor8bit.zero import UNIT, plan_layout
    import math
    numels = [math.prod(s) for s in shapes]
    cell, offsets = plan_layout([(n, k, g) for n, (k, g) in zip(numels, rules)], n_cells)
    assert (cell, offsets) == plan_layout([(n, k, g) for n, (k, g) in zip(numels, rules)], n_cells)    # deterministic
    spans = sorted((o, o + n) for o, n in zip(offsets, numels))
    assert all(a[1] <= b[0] for a, b in zip(spans, spans[1:])), "tensors overlap"
    assert all(o % UNIT == 0 for o in offsets)
    assert spans[-1][1] <= n_cells * cell
    for o, n, (kind, grain) in zip(offsets, numels, rules):
        first, last = o // cell, (o + n - 1) // cell
        if kind == "whole":
            assert first == last, "a whole tensor crosses a cell boundary"
        for j in range(first + 1, last + 1):
            assert (j * cell - o) % grain == 0, "a cell boundary is not a legal cut"
    return cell, offsets, sum(numels)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_layout_of_the_benchmark_models(world):
    from adafactor8bit.zero import cut_rule
    adamw = dict(beta1=0.9, beta2=0.999, factored=False, block_size=2048, m_block_size=256)
    came = dict(beta1=0.9, beta2=0.999, beta3=0.9999, factored=True, block_size=2048, m_block_size=256)
    apollo = dict(adamw, apollo_rank=256)
    for shapes, opts, parts in ((_tinyllama(), adamw, 4), (_tinyllama(), dict(factored=True, beta2_decay=-0.8, block_size=256), 2),
                                (_tinyllama(), came, 4), (_llama3_8b(), None, 4)):
        if opts is None:        # APOLLO on the matrices of the layers, AdamW on embedding, head and vectors
            rules = [cut_rule(apollo if (len(s) == 2 and s[0] != 128256) else adamw, s, 1 << 20) for s in shapes]
            assert rules[0] == ("flat", 2048) and rules[1] == ("whole", 0)
        else:
            rules = [cut_rule(opts, s, 1 << 20) for s in shapes]
        n_cells = world * (parts if world > 1 else 1)
        cell, offsets, total = _check_layout(shapes, rules, n_cells)
        assert n_cells * cell <= 1.02 * total + n_cells * 2048 * 64, (world, cell, total)      # padding stays small


def test_cut_rules():
    from adafactor8bit.zero import cut_rule, exchange_count
    adamw = dict(beta1=0.9, beta2=0.999, factored=False, scale_parameter=False, d=0.0)
    assert cut_rule(adamw, (32000, 2048), 1 << 20) == ("flat", 2048)
    assert cut_rule(dict(adamw, block_size=1024, m_block_size=96), (1 << 22,), 1) == ("flat", 6144)
    assert cut_rule(adamw, (2048,), 1) == ("whole", 0)
    assert cut_rule(dict(adamw, lag_norm=True), (32000, 2048), 1) == ("whole", 0)
    assert cut_rule(dict(adamw, apollo_rank=8), (32000, 2048), 1) == ("whole", 0)
    assert cut_rule(dict(adamw, apollo_rank=8), (1 << 22,), 1) == ("flat", 2048)
    fact = dict(factored=True, beta2_decay=-0.8)
    assert cut_rule(fact, (4, 32000, 2048), 1) == ("whole", 0)
    assert cut_rule(fact, (4096, 11008), 1) == ("rows", 8 * 11008)
    assert cut_rule(fact, (5632, 2048), 1) == ("rows", 2048)
    assert cut_rule(fact, (64, 131), 1) == ("whole", 0)                 # 2048 rows per cut unit
    assert cut_rule(dict(factored=True, beta2=None, beta2_decay=None), (4096, 2048), 1) == ("flat", 2048)   # SGD mode
    assert exchange_count(adamw, (32000, 2048)) == 0
    assert exchange_count(dict(adamw, enable_fira_for_adafactor=True), (32000, 2048)) == 1
    assert exchange_count(dict(fact, scale_parameter=True, d=1.0), (4096, 2048)) == 2
    assert exchange_count(dict(fact, scale_parameter=True, d=1.0), (2048,)) == 1
    assert exchange_count(dict(beta1=0.9, beta2=0.999, beta3=0.9999, factored=True, d=1.0), (4096, 2048)) == 3
    assert exchange_count(dict(adamw, apollo_rank=8), (4096, 2048)) == 0


def test_layout_keeps_whole_tensors_whole_and_fills_gaps():
    rules = [("whole", 0), ("flat", 2048), ("whole", 0), ("whole", 0), ("rows", 4096), ("whole", 0)]
    shapes = [(30000,), (100000,), (50000,), (3000,), (64, 2048), (70000,)]
    for n_cells in (1, 2, 3, 5, 8):
        _check_layout(shapes, rules, n_cells)


class _FakeShard:
    def __init__(self, rounds, parts, part_of_group, log):
        self.rounds, self.parts, self.part_of_group, self.log = rounds, parts, part_of_group, log

    def exchange(self, r):
        self.log.append(("exchange", r))

    def after_part(self, k):
        self.log.append(("after_part", k))


def test_round_schedule_of_the_launch_plans():
    """Plans with different numbers of exchange points: segment j of a plan with e points runs in round
    rounds - e + j, the parameter-writing segments run last, part by part, and the collectives come in
    one fixed order."""
    from adafactor8bit import Adafactor8Bit
    opt = Adafactor8Bit([torch.nn.Parameter(torch.zeros(4))])
    log = []

    def plan(name, e):
        for j in range(e):
            log.append((name, j))
            yield
        log.append((name, "write"))

    pending = [(0, 1, "cpu", plan("a", 1)), (1, 3, "cpu", plan("b", 3)), (2, 0, "cpu", plan("c", 0)), (3, 1, "cpu", plan("d", 1))]
    opt._shard = _FakeShard(3, 2, [0, 0, 1, 1], log)

    class _NoDevice:
        def __enter__(self):
            return self

        def __exit__(self, *a):
            return False
    import adafactor8bit.optimizer as mod
    saved = mod.torch.cuda.device
    mod.torch.cuda.device = lambda dev: _NoDevice()
    try:
        opt._step_sharded(pending)
    finally:
        mod.torch.cuda.device = saved
    assert log == [("b", 0), ("exchange", 0), ("b", 1), ("exchange", 1), ("a", 0), ("b", 2), ("d", 0), ("exchange", 2),
                   ("a", "write"), ("b", "write"), ("after_part", 0), ("c", "write"), ("d", "write"), ("after_part", 1)]
    with pytest.raises(RuntimeError):
        opt._step_sharded([(0, 4, "cpu", plan("x", 4))])


def _order_worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from adafactor8bit.zero import ShardedAdafactor8Bit
        # sizes for which a rank's middle parts are empty under a whole-tensor assignment
        numels = [n * 4096 for n in (1000, 1000, 900, 300, 300, 300, 100)]
        params = [torch.nn.Parameter(torch.zeros(n)) for n in numels]
        opt = ShardedAdafactor8Bit(params, inner_factory=torch.optim.SGD, parts=4, min_piece=1 << 30, lr=0.1)
        for p in params:
            p.grad = torch.ones_like(p)
        opt.step()
        out[rank] = list(opt.gather_log)
    finally:
        dist.destroy_process_group()


def test_every_rank_gathers_the_units_in_the_same_order():
    world, port = 2, _free_port()
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_order_worker, args=(world, port, out), nprocs=world, join=True)
    assert out[0] == out[1] == [0, 1, 2, 3]


def _ckpt_worker(rank, world, port, out, single_sd):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from adafactor8bit.zero import ShardedAdafactor8Bit
        params = _make_params(1)
        groups = [{"params": params[:2], "lr": 0.05}, {"params": params[2:]}]
        opt = ShardedAdafactor8Bit(groups, inner_factory=torch.optim.SGD, parts=2, min_piece=1, lr=0.1, momentum=0.9)
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
        opt2 = ShardedAdafactor8Bit(groups2, inner_factory=torch.optim.SGD, parts=2, min_piece=1, lr=0.1, momentum=0.9)
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
    buffers put together from the pieces), and a sharded optimizer loaded from a one-process checkpoint
    continues like it."""
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


def test_merging_and_cutting_of_native_state_entries():
    """full_state_dict / load_full_state_dict on the optimizer's own state layout, without a GPU: the states
    of the pieces of a cut tensor (code arrays padded to the block, per-block ranges, packed 4-bit momentum,
    row / column states kept by every owner) put together give the whole tensor's state, and cutting that
    again gives the pieces back."""
    from adafactor8bit.zero import ShardedAdafactor8Bit

    class Fake(ShardedAdafactor8Bit):
        def __init__(self, shape):
            self.all_params = [torch.zeros(shape)]

    block, m_block = 256, 64
    # a full-rank tensor of 1000 elements cut at 512 (both multiples of the blocks), packed uf4 momentum
    whole = {"step": 3, "block_size": block, "m_block_size": m_block, "m_quant_type": "uf4", "v_quant_type": "al8",
             "variance_q": torch.arange(1024, dtype=torch.int32).to(torch.uint8), "variance_scale": torch.arange(4.0),
             "variance_min_log": -torch.arange(4.0), "variance_shape": torch.Size([1000]), "variance_pad": 24,
             "m_q": torch.arange(512, dtype=torch.int32).to(torch.uint8), "m_scale": torch.arange(16.0),
             "fira_prev_norm": torch.tensor(0.5)}
    z = Fake((1000,))
    a = z._slice(0, 0, 512, (512,), whole)
    b = z._slice(0, 512, 1000, (488,), whole)
    assert a["variance_q"].numel() == 512 and b["variance_q"].numel() == 512 and b["variance_pad"] == 24 and a["variance_pad"] == 0
    assert a["m_q"].numel() == 256 and b["m_q"].numel() == 256 and a["m_scale"].numel() == 8 and b["m_scale"].numel() == 8
    assert tuple(b["variance_shape"]) == (488,) and float(b["fira_prev_norm"]) == 0.5
    merged = z._merge(0, [(512, 1000, (488,), b), (0, 512, (512,), a)])
    assert sorted(merged) == sorted(whole)
    for k, v in whole.items():
        assert torch.equal(merged[k], v) if isinstance(v, torch.Tensor) else merged[k] == v, k
    # a factored tensor cut by rows: fp32 momentum follows the rows, the row / column states are shared
    shape = (8, 64)
    whole = {"step": 1, "block_size": block, "m_block_size": m_block, "m": torch.arange(512.0).reshape(shape),
             "row_var_q": torch.arange(256, dtype=torch.int32).to(torch.uint8), "row_var_scale": torch.ones(1),
             "col_var": torch.arange(64.0).reshape(1, 64)}
    z = Fake(shape)
    a = z._slice(0, 0, 128, (2, 64), whole)
    b = z._slice(0, 128, 512, (6, 64), whole)
    assert tuple(a["m"].shape) == (2, 64) and tuple(b["m"].shape) == (6, 64) and torch.equal(b["row_var_q"], whole["row_var_q"])
    merged = z._merge(0, [(0, 128, (2, 64), a), (128, 512, (6, 64), b)])
    for k, v in whole.items():
        assert torch.equal(merged[k], v) if isinstance(v, torch.Tensor) else merged[k] == v, k
