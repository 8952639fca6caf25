"""ZeRO-1 style sharding of the optimizer step over the GPUs of one node.

The reference has no distributed code; this module is an addition around the
unchanged `Adafactor8Bit`.  Every rank holds the full fp32 parameters and the full
gradients (as after a data-parallel backward with gradient all-reduce), but
optimizer states exist only on the rank that owns a tensor, and only that rank
updates it.  After the step one in-place NCCL all-gather distributes the updated
parameters.

Partition.  Whole tensors are assigned to ranks (longest-processing-time greedy
on the element count), so every statistic of a step (update norms, row / column
sums, projections) is local to one rank and the only data exchange of the step
is the parameter all-gather.  All parameters live in ONE flat buffer laid out
[rank 0's tensors | rank 1's tensors | ...] with equal-sized rank regions, and
`param.data` of every parameter is a view into it: the kernels write updated
values straight into the all-gather buffer and `all_gather_into_tensor` runs in
place, without a staging copy.
"""
import torch
import torch.distributed as dist

from .optimizer import Adafactor8Bit

_ALIGN = 128   # elements: keeps every tensor of the flat buffer 512-byte aligned


def partition_tensors(numels, world):
    """Greedy longest-first assignment of tensors to ranks -> owner index per tensor."""
    loads = [0] * world
    owner = [0] * len(numels)
    for i in sorted(range(len(numels)), key=lambda k: (-numels[k], k)):
        r = min(range(world), key=lambda k: (loads[k], k))
        owner[i] = r
        loads[r] += numels[i]
    return owner


class ShardedAdafactor8Bit:
    """Adafactor8Bit whose states and step are partitioned over a process group.

    params: an iterable of tensors or of param-group dicts, as for Adafactor8Bit.
    inner_factory: class of the per-rank optimizer (the default is Adafactor8Bit; the
    CPU tests of the sharding logic plug in a stock torch optimizer).
    """

    def __init__(self, params, process_group=None, inner_factory=Adafactor8Bit, **kwargs):
        self.group = process_group
        self.world = dist.get_world_size(process_group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(process_group) if dist.is_initialized() else 0
        groups = list(params)
        if groups and not isinstance(groups[0], dict):
            groups = [{"params": groups}]
        groups = [dict(g, params=list(g["params"])) for g in groups]
        all_params = [p for g in groups for p in g["params"]]
        if not all_params:
            raise ValueError("optimizer got an empty parameter list")
        dev, dt = all_params[0].device, all_params[0].dtype
        for p in all_params:
            if p.device != dev or p.dtype != dt:
                raise ValueError("all parameters of a sharded optimizer must share device and dtype")
        numels = [p.numel() for p in all_params]
        self.owner = partition_tensors(numels, self.world)
        padded = [(n + _ALIGN - 1) // _ALIGN * _ALIGN for n in numels]
        fill = [0] * self.world
        offset = [0] * len(all_params)
        for i, r in enumerate(self.owner):
            offset[i] = fill[r]
            fill[r] += padded[i]
        self.region = max(max(fill), _ALIGN)
        self.flat = torch.zeros(self.world * self.region, dtype=dt, device=dev)
        with torch.no_grad():
            for i, p in enumerate(all_params):
                start = self.owner[i] * self.region + offset[i]
                view = self.flat[start:start + numels[i]].view(p.shape)
                view.copy_(p.data)
                p.data = view
        self.all_params = all_params
        owned = {id(p) for i, p in enumerate(all_params) if self.owner[i] == self.rank}
        self.owned_numel = sum(n for i, n in enumerate(numels) if self.owner[i] == self.rank)
        self.total_numel = sum(numels)
        inner_groups = []
        for g in groups:
            mine = [p for p in g["params"] if id(p) in owned]
            if mine:
                inner_groups.append(dict(g, params=mine))
        self.inner = inner_factory(inner_groups, **kwargs) if inner_groups else None
        self.gather_stream = None

    @property
    def param_groups(self):
        return self.inner.param_groups if self.inner is not None else []

    @property
    def state(self):
        return self.inner.state if self.inner is not None else {}

    def zero_grad(self, set_to_none=True):
        for p in self.all_params:
            if set_to_none:
                p.grad = None
            elif p.grad is not None:
                p.grad.zero_()

    def local_step(self, closure=None):
        """Update the tensors this rank owns (no communication)."""
        return self.inner.step(closure) if self.inner is not None else None

    def gather(self):
        """In-place all-gather of the rank regions of the flat parameter buffer."""
        if self.world > 1:
            mine = self.flat[self.rank * self.region:(self.rank + 1) * self.region]
            dist.all_gather_into_tensor(self.flat, mine, group=self.group)

    def step(self, closure=None):
        loss = self.local_step(closure)
        self.gather()
        return loss

    def state_dict(self):
        """State of the tensors this rank owns (a per-rank shard, not the reference's full layout)."""
        return {"rank": self.rank, "world": self.world, "owner": list(self.owner),
                "inner": self.inner.state_dict() if self.inner is not None else None}

    def load_state_dict(self, sd):
        if sd["world"] != self.world or list(sd["owner"]) != list(self.owner):
            raise ValueError("sharded state was saved with a different partition")
        if self.inner is not None and sd["inner"] is not None:
            self.inner.load_state_dict(sd["inner"])
