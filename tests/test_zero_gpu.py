"""ShardedAdafactor8Bit on two GPUs over NCCL: the sharded step must equal the single-GPU step.
Tensors are cut across the two ranks and across two parts per rank; block-local arithmetic is
identical by construction, and the statistics of cut tensors (update norms, RMS(p), row / column
sums) are all-reduced in binary64, which reproduces the single-GPU values (a different rounding of
a binary64 sum would have to fall on a binary32 rounding boundary to show).
Skipped on machines with fewer than two GPUs."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu

SHAPES = [(300, 200), (4096,), (2048,), (128, 256), (64, 2048), (512, 384), (20000,)]


def _inputs(variant="f32"):
    """variant "f32": fp32 parameters; "bf16_sr": bf16 parameters written with stochastic rounding
    (the seeds must be those of the unsharded run); "adafactor" / "came": the factored paths."""
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    import cases
    hp = dict(cases.CASES["adamw_fira_bf16"]["hp"])
    if variant == "bf16_sr":
        hp["stochastic_round_writeback"] = True
    if variant == "adamw_noclip":       # no whole-tensor statistic at all
        hp = dict(cases.CASES["adamw_uf8_al8"]["hp"])
    if variant == "adafactor":          # factored second moments, relative step, parameter scaling, clip
        hp = dict(cases.CASES["adafactor_factored"]["hp"])
    if variant == "came":
        hp = dict(cases.CASES["came_al16"]["hp"])
    if variant == "apollo":             # projection seeds must be those of the unsharded run
        hp = dict(cases.CASES["apollo_r32"]["hp"], apollo_rank=16)
    p0 = [cases.make_param(s, 7000 + i, dtype="bf16" if variant == "bf16_sr" else "f32") for i, s in enumerate(SHAPES)]
    grads = {t: [cases.make_grad(s, 7100 + i, t, cases.CASES["adamw_fira_bf16"]["grad"]) for i, s in enumerate(SHAPES)]
             for t in (1, 2, 3)}
    return hp, p0, grads


def _bf16(g, shape, dev):
    return torch.from_numpy(g.view(np.int16).copy()).view(torch.bfloat16).reshape(shape).to(dev)


def _pdt(variant):
    return torch.bfloat16 if variant == "bf16_sr" else torch.float32


def _plain(x, path="state_dict"):
    """A checkpoint as plain Python / numpy objects (what travels between the processes of this test);
    every tensor must already be on the CPU."""
    if isinstance(x, torch.Tensor):
        assert x.device.type == "cpu", f"{path} is on {x.device}"
        a = x.detach().contiguous()
        return ["tensor", str(a.dtype), tuple(a.shape), a.view(torch.int16).numpy().copy() if a.dtype == torch.bfloat16 else a.numpy().copy()]
    if isinstance(x, torch.Size):
        return ["size"] + list(x)
    if isinstance(x, dict):
        return {k: _plain(v, f"{path}[{k!r}]") for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return [_plain(v, f"{path}[{i}]") for i, v in enumerate(x)]
    assert x is None or isinstance(x, (bool, int, float, str)), f"{path} holds a {type(x).__name__}"
    return x


def _same(a, b, path="state_dict"):
    if isinstance(a, dict):
        assert isinstance(b, dict) and sorted(a) == sorted(b), (path, sorted(a), sorted(b) if isinstance(b, dict) else b)
        for k in a:
            _same(a[k], b[k], f"{path}[{k!r}]")
    elif isinstance(a, list) and len(a) == 4 and a[0] == "tensor":
        assert isinstance(b, list) and b[:3] == a[:3], (path, a[:3], b[:3] if isinstance(b, list) else b)
        assert np.array_equal(a[3], b[3]), path
    elif isinstance(a, list):
        assert isinstance(b, list) and len(a) == len(b), path
        for i, (x, y) in enumerate(zip(a, b)):
            _same(x, y, f"{path}[{i}]")
    else:
        assert a == b, (path, a, b)


def _worker(rank, world, port, out, variant):
    sys.path.insert(0, os.path.join(ROOT, "adafactor-8bit_b200"))
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from adafactor8bit import ShardedAdafactor8Bit
        nccl = variant.endswith("_nccl")          # parameters by NCCL all-gather instead of peer copies
        variant = variant.replace("_nccl", "")
        hp, p0, grads = _inputs(variant)
        params = [torch.nn.Parameter(torch.from_numpy(p.copy()).to(dev).to(_pdt(variant))) for p in p0]
        for p in params:
            p.grad_dtype = None
        copy = variant == "bf16_copy"
        opt = ShardedAdafactor8Bit(params, parts=2, min_piece=1, compute_dtype=torch.bfloat16 if copy else None,
                                   exchange="nccl" if nccl else "auto", **hp)
        assert opt.exchange == ("nccl" if nccl else "push"), getattr(opt, "_symm_error", None)
        assert any(len(lst) > 1 for lst in opt.pieces_of) or variant == "apollo", "the case must cut a tensor"
        for t in (1, 2, 3):
            for p, g in zip(params, grads[t]):
                p.grad = _bf16(g, p.shape, dev)
            opt.step()
        torch.cuda.synchronize()
        assert opt.gather_log == [0, 1]
        out[rank] = [p.detach().float().cpu().numpy().copy() for p in params]
        if copy:                                    # the model's view is bf16; the fp32 masters stay sharded
            assert all(p.dtype == torch.bfloat16 for p in params)
            masters = opt.master_params(dst=0)
            if rank == 0:
                out["masters"] = [m.numpy().copy() for m in masters]
        full = opt.full_state_dict(dst=0)          # the merged checkpoint, in the unsharded layout
        if rank == 0:
            out["full"] = _plain(full)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("variant", ["f32", "f32_nccl", "adamw_noclip", "bf16_sr", "adafactor", "came", "apollo", "bf16_copy",
                                     "bf16_copy_nccl"])
def test_two_gpu_sharded_step_is_bit_identical_to_one_gpu(variant):
    import torch.multiprocessing as mp
    sys.path.insert(0, os.path.join(ROOT, "adafactor-8bit_b200"))
    from adafactor8bit import Adafactor8Bit
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(2, port, out, variant), nprocs=2, join=True)
    variant = variant.replace("_nccl", "")
    hp, p0, grads = _inputs(variant)
    params = [torch.nn.Parameter(torch.from_numpy(p.copy()).cuda().to(_pdt(variant))) for p in p0]
    for p in params:
        p.grad_dtype = None
    opt = Adafactor8Bit(params, **hp)
    for t in (1, 2, 3):
        for p, g in zip(params, grads[t]):
            p.grad = _bf16(g, p.shape, "cuda")
        opt.step()
    torch.cuda.synchronize()
    for rank in (0, 1):
        for a, p in zip(out[rank], params):
            want = p.detach()
            if variant == "bf16_copy":               # every rank reads the rounded copy of the masters
                want = want.to(torch.bfloat16)
            assert np.array_equal(a, want.float().cpu().numpy())
    if variant == "bf16_copy":
        for a, p in zip(out["masters"], params):
            assert np.array_equal(a, p.detach().cpu().numpy())
    # the merged checkpoint equals the one-GPU optimizer's, entry by entry
    full = out["full"]
    want = opt.state_dict()
    want = _plain({k: ({i: {kk: (vv.cpu() if isinstance(vv, torch.Tensor) else vv) for kk, vv in st.items()} for i, st in v.items()}
                       if k == "state" else v) for k, v in want.items()})
    assert sorted(full["state"]) == sorted(want["state"])
    assert full["_sr_seed_counter"] == want["_sr_seed_counter"]
    assert [g["params"] for g in full["param_groups"]] == [g["params"] for g in want["param_groups"]]
    _same(want["state"], full["state"], "state")
