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
is the parameter all-gather.  All parameters live in ONE flat buffer made of a few
gather units, each laid out [rank 0's part | rank 1's part | ...] with equal slots,
and `param.data` of every parameter is a view into it: the kernels write updated
values straight into the all-gather buffer, `all_gather_into_tensor` runs in place,
without a staging copy, and the gather of one unit overlaps the update of the next.
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


def split_parts(sizes, k):
    """Cut a sequence of sizes into k consecutive parts of roughly equal total -> part index per item."""
    total = sum(sizes)
    part, acc, out = 0, 0, []
    for n in sizes:
        # move on when the running total has passed this part's share (never beyond the last part)
        while part < k - 1 and acc >= total * (part + 1) / k:
            part += 1
        out.append(part)
        acc += n
    return out


class ShardedAdafactor8Bit:
    """Adafactor8Bit whose states and step are partitioned over a process group.

    params: an iterable of tensors or of param-group dicts, as for Adafactor8Bit.
    gather_chunks: the tensors of every rank are cut into this many consecutive parts; the
    all-gather of part k runs on a second stream while part k + 1 is being updated.
    inner_factory: class of the per-rank optimizer (the default is Adafactor8Bit; the
    CPU tests of the sharding logic plug in a stock torch optimizer).
    """

    def __init__(self, params, process_group=None, inner_factory=Adafactor8Bit, gather_chunks=4, **kwargs):
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
        # every rank's tensors, in order, cut into parts; part k of all ranks forms gather unit k:
        # [rank 0's part k | rank 1's part k | ...] with equal slots, the units one after another
        k_parts = max(1, int(gather_chunks)) if self.world > 1 else 1
        part = [0] * len(all_params)
        for r in range(self.world):
            mine = [i for i in range(len(all_params)) if self.owner[i] == r]
            for i, pk in zip(mine, split_parts([padded[i] for i in mine], k_parts)):
                part[i] = pk
        fill = [[0] * k_parts for _ in range(self.world)]
        offset = [0] * len(all_params)
        for i, r in enumerate(self.owner):
            offset[i] = fill[r][part[i]]
            fill[r][part[i]] += padded[i]
        self.unit_slot = [max(max(fill[r][k] for r in range(self.world)), 0) for k in range(k_parts)]
        if sum(self.unit_slot) == 0:
            self.unit_slot[0] = _ALIGN
        self.unit_start = [0] * k_parts
        for k in range(1, k_parts):
            self.unit_start[k] = self.unit_start[k - 1] + self.world * self.unit_slot[k - 1]
        self.flat = torch.zeros(self.unit_start[-1] + self.world * self.unit_slot[-1], dtype=dt, device=dev)
        with torch.no_grad():
            for i, p in enumerate(all_params):
                start = self.unit_start[part[i]] + self.owner[i] * self.unit_slot[part[i]] + offset[i]
                view = self.flat[start:start + numels[i]].view(p.shape)
                view.copy_(p.data)
                p.data = view
        self.all_params = all_params
        self.part = part
        owned = {id(p) for i, p in enumerate(all_params) if self.owner[i] == self.rank}
        part_of = {id(p): part[i] for i, p in enumerate(all_params)}
        self.owned_numel = sum(n for i, n in enumerate(numels) if self.owner[i] == self.rank)
        self.total_numel = sum(numels)
        # inner groups: part-major, so that a part's launches are complete before the next part starts
        inner_groups, self._last_group_of_part = [], {}
        self._origin = []                  # inner group -> index of the group it was cut from
        for k in range(k_parts):
            for gi, g in enumerate(groups):
                mine = [p for p in g["params"] if id(p) in owned and part_of[id(p)] == k]
                if mine:
                    inner_groups.append(dict(g, params=mine))
                    self._origin.append(gi)
                    self._last_group_of_part[k] = len(inner_groups) - 1
        self._groups = groups
        self._global_index = {id(p): i for i, p in enumerate(all_params)}
        self.inner = inner_factory(inner_groups, **kwargs) if inner_groups else None
        if self.inner is not None and hasattr(self.inner, "_sr_seed_map"):
            # stochastic-rounding seeds as the unsharded optimizer would hand them out: one per
            # 16-bit parameter of a group that rounds stochastically, in parameter order
            seeds, nxt = {}, 1
            for g in groups:
                sr = g.get("stochastic_round_writeback", kwargs.get("stochastic_round_writeback", False))
                for p in g["params"]:
                    if sr and p.dtype in (torch.bfloat16, torch.float16):
                        seeds[id(p)] = nxt
                        nxt += 1
            self.inner._sr_seed_map = seeds
            self.inner._sr_seed_counter = nxt
        if self.inner is not None and hasattr(self.inner, "_apollo_seed_map"):
            # the same for the projection seeds of APOLLO (one per tensor of two or more dimensions in a group
            # with a rank, in parameter order: optimizer.py:1726-1728)
            seeds, nxt = {}, 1
            for g in groups:
                rank = g.get("apollo_rank", kwargs.get("apollo_rank", 0))
                for p in g["params"]:
                    if rank and rank > 0 and p.dim() >= 2:
                        seeds[id(p)] = nxt
                        nxt += 1
            self.inner._apollo_seed_map = seeds
            self.inner._apollo_seed_counter = nxt
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

    def _gather_unit(self, k):
        slot = self.unit_slot[k]
        if slot == 0:
            return
        unit = self.flat[self.unit_start[k]:self.unit_start[k] + self.world * slot]
        dist.all_gather_into_tensor(unit, unit[self.rank * slot:(self.rank + 1) * slot], group=self.group)

    def gather(self):
        """In-place all-gather of every unit of the flat parameter buffer."""
        if self.world > 1:
            for k in range(len(self.unit_slot)):
                self._gather_unit(k)

    def step(self, closure=None):
        """Local update and parameter all-gather.  On CUDA with the native optimizer the gather of a
        part starts, on a second stream, as soon as the launches of that part have been enqueued."""
        pipelined = (self.world > 1 and self.flat.is_cuda and self.inner is not None and hasattr(self.inner, "_after_group"))
        if not pipelined:
            loss = self.local_step(closure)
            self.gather()
            return loss
        if self.gather_stream is None:
            self.gather_stream = torch.cuda.Stream(device=self.flat.device)
        main = torch.cuda.current_stream(self.flat.device)
        done = set()

        def after_group(gi, group):
            for k, last in self._last_group_of_part.items():
                if last == gi and k not in done:
                    done.add(k)
                    ev = torch.cuda.Event()
                    ev.record(main)
                    with torch.cuda.stream(self.gather_stream):
                        self.gather_stream.wait_event(ev)
                        self._gather_unit(k)

        self.inner._after_group = after_group
        try:
            loss = self.inner.step(closure)
        finally:
            self.inner._after_group = None
        with torch.cuda.stream(self.gather_stream):          # parts this rank owns nothing of
            for k in range(len(self.unit_slot)):
                if k not in done:
                    self._gather_unit(k)
        main.wait_stream(self.gather_stream)
        return loss

    # -- checkpoints in the unsharded optimizer's layout ------------------------------------------
    def full_state_dict(self, dst=0):
        """The state of all ranks merged into the layout an unsharded optimizer saves (and the
        reference's class loads): {"state": {parameter index: state}, "param_groups": [...]} plus
        the optimizer-level counters.  Tensors are moved to the CPU.  Collective: every rank calls
        it; rank `dst` gets the dictionary, the others None."""
        inner_sd = self.inner.state_dict() if self.inner is not None else {"state": {}, "param_groups": []}
        inner_params = [p for g in self.inner.param_groups for p in g["params"]] if self.inner is not None else []
        mine = {}
        for idx, st in inner_sd["state"].items():
            mine[self._global_index[id(inner_params[idx])]] = {
                k: (v.detach().cpu() if isinstance(v, torch.Tensor) else v) for k, v in st.items()}
        extras = {k: v for k, v in inner_sd.items() if k not in ("state", "param_groups")}
        options = {self._origin[j]: {k: v for k, v in g.items() if k != "params"}
                   for j, g in enumerate(inner_sd["param_groups"])}
        payload = (mine, extras, options)
        if self.world > 1:
            gathered = [None] * self.world if self.rank == dst else None
            dist.gather_object(payload, gathered, dst=dst, group=self.group)
            if self.rank != dst:
                return None
        else:
            gathered = [payload]
        state, extras, options = {}, {}, {}
        for m, e, o in gathered:
            state.update(m)
            for k, v in e.items():
                extras[k] = max(extras[k], v) if (k in extras and isinstance(v, (int, float))) else v
            for gi, opts in o.items():
                options.setdefault(gi, opts)
        groups, first = [], 0
        for gi, g in enumerate(self._groups):
            opts = options.get(gi, {k: v for k, v in g.items() if k != "params"})
            groups.append(dict(opts, params=list(range(first, first + len(g["params"])))))
            first += len(g["params"])
        return dict(extras, state=dict(sorted(state.items())), param_groups=groups)

    def load_full_state_dict(self, sd):
        """Load a state dictionary in the unsharded layout (from full_state_dict, from an unsharded
        optimizer of this package or from the reference): every rank keeps the states of the
        tensors it owns."""
        if self.inner is None:
            return
        inner_sd = self.inner.state_dict()
        inner_params = [p for g in self.inner.param_groups for p in g["params"]]
        state = {}
        for idx, p in enumerate(inner_params):
            st = sd["state"].get(self._global_index[id(p)])
            if st is not None:
                state[idx] = st
        groups = []
        for j, g in enumerate(inner_sd["param_groups"]):
            saved = sd["param_groups"][self._origin[j]]
            groups.append(dict({k: v for k, v in saved.items() if k != "params"}, params=g["params"]))
        extras = {k: v for k, v in sd.items() if k not in ("state", "param_groups")}
        self.inner.load_state_dict(dict(extras, state=state, param_groups=groups))

    def state_dict(self):
        """State of the tensors this rank owns (a per-rank shard; full_state_dict gives the
        unsharded layout)."""
        return {"rank": self.rank, "world": self.world, "owner": list(self.owner),
                "inner": self.inner.state_dict() if self.inner is not None else None}

    def load_state_dict(self, sd):
        if sd["world"] != self.world or list(sd["owner"]) != list(self.owner):
            raise ValueError("sharded state was saved with a different partition")
        if self.inner is not None and sd["inner"] is not None:
            self.inner.load_state_dict(sd["inner"])
