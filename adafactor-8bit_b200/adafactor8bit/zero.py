"""ZeRO-1 style sharding of the optimizer step over the GPUs of one node.

The reference has no distributed code; this module is an addition around the unchanged
`Adafactor8Bit`.  Every rank holds the full gradients (as after a data-parallel backward with
gradient all-reduce); optimizer states exist only on the rank that owns a stretch of the
parameter space, and only that rank updates it.  After the step an in-place NCCL all-gather
publishes the updated parameters.

Partition.  All tensors are laid out one after another in ONE flat space, each padded to a multiple
of 2048 elements (a multiple of every quantisation block size, so no block is shared by two
tensors).  The space is divided into `parts * world` consecutive cells of equal size; cell j belongs
to rank j % world and to part j // world.  A tensor that crosses a cell boundary is cut there:
  * tensors on the full-rank path (AdamW, RMSprop, SGD, unfactored Adafactor) at a multiple of
    lcm(2048, block_size, m_block_size) elements: every quantisation block lies in one piece;
  * factored 2-D tensors (Adafactor, CAME) at a row boundary where the flat offset is such a
    multiple: momentum blocks stay whole, the row / column states are kept by every owner;
  * APOLLO tensors, tensors of more than two dimensions, tensors of a `lag_norm` group and small
    tensors stay whole (the projection side of APOLLO follows the tensor's shape, and a projection
    from the left contracts over the rows); they are packed into the cells first-fit.
The offset of a tensor is shifted by less than one cut unit where that makes a cell boundary fall on
a legal cut, so the flat space doubles as the all-gather buffer: every tensor is one contiguous
view of it, part k of all ranks is one contiguous unit, and `all_gather_into_tensor` runs in place
on the unit while the kernels write the next part.

Statistics of cut tensors.  What the reference computes over a whole tensor -- the update norm of
the clip and of the limiter, RMS(p) of `scale_parameter`, the row and column sums of the factored
paths and of CAME's residual -- is summed locally, all-reduced in one small float64 buffer per
round (at most four rounds per step, only tensors that are cut take part) and finished identically
on every owner.  Tensors that are not cut need no exchange.

Exchange of the parameters.  On CUDA the flat space is allocated as symmetric memory
(torch.distributed._symmetric_memory: every rank maps the other ranks' buffers), and a rank
publishes a finished cell by copying it into the same place of every peer's buffer with plain
asynchronous device copies, one stream per peer.  Those run on the copy engines: they take no SM
away from the update kernels of the next part, which the kernels of an NCCL all-gather do (the
update kernels are persistent grids sized to fill the GPU).  One small NCCL all-reduce per step,
enqueued behind the copies, tells every rank that all cells have arrived.  Where symmetric memory
is not available (or with `exchange="nccl"`) the cells travel by in-place `all_gather_into_tensor`.

Mixed precision.  With `compute_dtype=torch.bfloat16` the flat space holds the bf16 compute copy of
the parameters (what the model reads); the fp32 master values exist only for a rank's own cells, and
the update kernels write the rounded copy straight into the gather buffer next to the master.  The
all-gather then moves 2 bytes per parameter instead of 4.
"""
import math
import os

import torch
import torch.distributed as dist

from .optimizer import Adafactor8Bit

UNIT = 2048            # elements: alignment of every tensor and every cut in the flat space


def _pad(n, m):
    return (n + m - 1) // m * m


def cut_rule(options, shape, min_piece):
    """How a tensor of `shape` in a group with `options` may be cut -> (kind, grain):
    kind 'flat' (grain elements), 'rows' (grain elements = whole rows) or 'whole'."""
    numel = int(math.prod(shape)) if len(shape) else 1
    if numel < max(min_piece, 2 * UNIT) or len(shape) >= 3 or options.get("lag_norm", False):
        return "whole", 0
    if options.get("apollo_rank", 0) > 0 and len(shape) >= 2:
        return "whole", 0
    unit = UNIT
    for b in (options.get("block_size", 2048), options.get("m_block_size", 256)):
        unit = unit * int(b) // math.gcd(unit, int(b))
    sgd = options.get("beta2") is None and options.get("beta2_decay") is None
    if len(shape) == 2 and options.get("factored", True) and not sgd:
        cols = int(shape[1])
        k = unit // math.gcd(unit, cols)              # fewest rows whose elements fill whole units
        if 2 * k > shape[0]:
            return "whole", 0
        return "rows", k * cols
    if numel < 2 * unit:
        return "whole", 0
    return "flat", unit


def exchange_count(options, shape):
    """Exchange points of the launch plan that steps a tensor of `shape` in a group with `options`
    (the pass structure of Adafactor8Bit._run_fullrank / _run_factored / _run_apollo)."""
    from ._engine import factored_exchanges, fullrank_exchanges
    sgd = options.get("beta2") is None and options.get("beta2_decay") is None
    d = float(options.get("d", 1.0))
    fira = bool(options.get("enable_fira_for_adafactor", False))
    lag = bool(options.get("lag_norm", False))
    beta1, beta3 = options.get("beta1"), options.get("beta3")
    if not sgd and options.get("apollo_rank", 0) > 0 and len(shape) >= 2:
        return 0
    if not sgd and len(shape) >= 2 and options.get("factored", True):
        return factored_exchanges(beta3 is not None and beta1 is not None, d, fira, lag)
    adam = (not options.get("factored", True)) and options.get("beta2") is not None and beta3 is None
    momentum_only = options.get("momentum_only_1d")
    if momentum_only is None:
        momentum_only = not adam
    momentum_only = bool(momentum_only) and beta1 is not None and not sgd
    return fullrank_exchanges(bool(options.get("scale_parameter", True)), d, fira, momentum_only, lag)


def plan_layout(tensors, n_cells):
    """Place tensors in the flat space.  tensors: list of (numel, kind, grain).
    -> (cell, offsets): the cell size and each tensor's first flat element.  Cell boundaries fall on
    legal cuts of 'flat' / 'rows' tensors and never inside a 'whole' tensor."""
    total = sum(_pad(n, UNIT) for n, _, _ in tensors)
    cell = _pad(max(1, -(-total // n_cells)), UNIT)
    while True:
        # a tensor longer than a cell meets several boundaries: they must all be legal cuts
        step = UNIT
        for n, kind, grain in tensors:
            if kind != "whole" and n > cell:
                step = step * grain // math.gcd(step, grain)
        cell = _pad(cell, step)
        offsets = _place(tensors, cell)
        if offsets is not None and max(o + _pad(t[0], UNIT) for o, t in zip(offsets, tensors)) <= n_cells * cell:
            return cell, offsets
        cell += max(step, _pad(cell // 64, step))


def _place(tensors, cell):
    offsets = [None] * len(tensors)
    waiting = []                                  # whole tensors that did not fit where their turn came
    pos = 0

    def room():
        return cell - pos % cell

    def put_waiting():
        nonlocal pos
        for i in list(waiting):
            ln = _pad(tensors[i][0], UNIT)
            if ln <= room():
                offsets[i] = pos
                pos += ln
                waiting.remove(i)

    for i, (n, kind, grain) in enumerate(tensors):
        ln = _pad(n, UNIT)
        put_waiting()
        if kind == "whole":
            if ln > cell:
                return None
            if ln <= room():
                offsets[i] = pos
                pos += ln
            else:
                waiting.append(i)
            continue
        b = pos + room()                          # the next cell boundary
        if b < pos + ln:                          # it falls inside: shift so that it is a legal cut
            pos += (b - pos) % grain
        offsets[i] = pos
        pos += ln
    while waiting:                                # nothing left to fill the gaps with: open new cells
        before = len(waiting)
        put_waiting()
        if waiting and len(waiting) == before:
            pos += room()
    return offsets


class _Schedule:
    """What Adafactor8Bit._step_sharded needs: rounds, parts, part_of_group, exchange, after_part."""

    def __init__(self, owner):
        self.owner = owner
        self.rounds = owner.rounds
        self.parts = owner.parts
        self.part_of_group = owner._part_of_group

    def exchange(self, r):
        self.owner._exchange(r)

    def after_part(self, k):
        self.owner._after_part(k)


class ShardedAdafactor8Bit:
    """Adafactor8Bit whose states and step are partitioned over a process group.

    params: an iterable of tensors or of param-group dicts, as for Adafactor8Bit.
    parts: the parameter space of every rank is cut into this many cells; the all-gather of part k
        runs on a second stream while part k + 1 is being updated.  None: as many (1 to 4) as keep a
        cell above 32 M elements.
    compute_dtype: None, or torch.bfloat16 for a bf16 compute copy with sharded fp32 masters (see the
        module text).  The parameters passed in supply the initial master values; afterwards they are
        bf16 views of the gather buffer.
    min_piece: tensors with fewer elements are never cut.
    exchange: "auto" (peer copies over symmetric memory when it can be set up, else NCCL), "push" or "nccl".
    inner_factory: class of the per-rank optimizer (the default is Adafactor8Bit; the CPU tests of the
        sharding logic plug in a stock torch optimizer, which sees the pieces as ordinary parameters).
    """

    def __init__(self, params, process_group=None, inner_factory=Adafactor8Bit, parts=None, compute_dtype=None,
                 min_piece=1 << 20, exchange="auto", **kwargs):
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
        if compute_dtype is not None and compute_dtype != torch.bfloat16:
            raise ValueError("compute_dtype must be None or torch.bfloat16")
        if compute_dtype is not None and inner_factory is not Adafactor8Bit:
            raise ValueError("the compute copy is written by the kernels of Adafactor8Bit")
        self.compute_dtype = compute_dtype
        self.master_dtype = torch.float32 if compute_dtype is not None else dt
        self.all_params = all_params
        self._groups = groups
        self._global_index = {id(p): i for i, p in enumerate(all_params)}
        # group options as the inner optimizer will see them (constructor defaults filled in)
        self._options = []
        for g in groups:
            opts = {k: v for k, v in kwargs.items()}
            opts.update({k: v for k, v in g.items() if k != "params"})
            self._options.append(opts)
        native = inner_factory is Adafactor8Bit
        if native:
            import inspect
            defaults = {k: v.default for k, v in inspect.signature(Adafactor8Bit.__init__).parameters.items()
                        if v.default is not inspect.Parameter.empty}
            self._options = [dict(defaults, **o) for o in self._options]
        group_of = [gi for gi, g in enumerate(groups) for _ in g["params"]]
        shapes = [tuple(p.shape) for p in all_params]
        numels = [p.numel() for p in all_params]
        rules = [cut_rule(self._options[group_of[i]], shapes[i], min_piece) if native
                 else (("flat", UNIT) if numels[i] >= max(min_piece, 2 * UNIT) else ("whole", 0))
                 for i in range(len(all_params))]
        total = sum(_pad(n, UNIT) for n in numels)
        if parts is None:
            # a part should keep a GPU busy for longer than its launches take to issue (about half a millisecond of
            # host time per part): 256 M parameters per rank and part, at most 4 parts
            parts = max(1, min(4, total // max(1, self.world) // (256 << 20))) if self.world > 1 else 1
        self.parts = parts = max(1, int(parts))
        n_cells = self.parts * self.world
        self.cell, offsets = plan_layout([(numels[i], rules[i][0], rules[i][1]) for i in range(len(numels))], n_cells)
        self.offsets = offsets
        cell = self.cell
        # pieces: (tensor, first element, end element, cell) for every stretch of a tensor inside one cell
        self.pieces_of = []
        for i, off in enumerate(offsets):
            n, lst, lo = numels[i], [], 0
            if n == 0:
                self.pieces_of.append(lst)
                continue
            while lo < n:
                j = (off + lo) // cell
                hi = min(n, (j + 1) * cell - off)
                lst.append((lo, hi, j))
                lo = hi
            self.pieces_of.append(lst)
        # exchange rounds: the most any launch plan needs (all ranks agree: it follows from the options)
        self._e = [exchange_count(self._options[group_of[i]], shapes[i]) if native else 0 for i in range(len(all_params))]
        self.rounds = max(self._e) if self._e else 0
        cut = [i for i in range(len(all_params)) if len(self.pieces_of[i]) > 1]
        # exchange buffer: per round, for every cut tensor that has an exchange in that round, 8 scalars and
        # (factored tensors) its row and column sums
        self._slot_of, sizes = {}, [0] * self.rounds
        for i in cut:
            rows_kind = rules[i][0] == "rows"
            ln = 8 + ((_pad(shapes[i][0], 4) + _pad(shapes[i][1], 4)) if rows_kind else 0)
            for r in range(self.rounds - self._e[i], self.rounds):
                self._slot_of[(i, r)] = (sizes[r], ln)
                sizes[r] += ln
        self._round_start = [sum(sizes[:r]) for r in range(self.rounds)]
        self._round_size = sizes
        self.xbuf = torch.zeros(max(1, sum(sizes)), dtype=torch.float64, device=dev) if native else None
        # the flat space = the gather buffer
        gather_dtype = compute_dtype if compute_dtype is not None else dt
        if exchange not in ("auto", "push", "nccl"):
            raise ValueError("exchange must be 'auto', 'push' or 'nccl'")
        self.flat, self.peer_flat = None, None
        if exchange != "nccl" and self.world > 1 and dev.type == "cuda":
            self.flat, self.peer_flat = self._symmetric_buffer(n_cells * cell, gather_dtype, dev, exchange == "push")
        if self.flat is None:
            self.flat = torch.zeros(n_cells * cell, dtype=gather_dtype, device=dev)
        self.exchange = "push" if self.peer_flat is not None else "nccl"
        # order of a rank's peer copies: "shift" (one at a time, to rank + 1, rank + 2, ...) or "concurrent" (one stream per peer)
        self.push_order = os.environ.get("AF8_PUSH_ORDER", "shift" if self.world > 2 else "concurrent")
        if self.push_order not in ("shift", "concurrent"):
            raise ValueError("AF8_PUSH_ORDER must be 'shift' or 'concurrent'")
        self.master = (torch.zeros(self.parts * cell, dtype=torch.float32, device=dev) if compute_dtype is not None else None)
        owned_numel = 0
        local = []                       # (tensor, lo, hi, part, piece parameter)
        from ._engine import Piece
        pieces_info = {}
        with torch.no_grad():
            for i, p in enumerate(all_params):
                off, n = offsets[i], numels[i]
                src = p.data.reshape(-1)
                view = self.flat[off:off + n]
                view.copy_(src)
                for lo, hi, j in self.pieces_of[i]:
                    if j % self.world != self.rank:
                        continue
                    k = j // self.world
                    kind = rules[i][0]
                    if (lo, hi) == (0, n):
                        pshape = shapes[i]
                    elif kind == "rows":
                        pshape = ((hi - lo) // shapes[i][1], shapes[i][1])
                    else:
                        pshape = (hi - lo,)
                    if self.master is not None:
                        m_off = k * cell + (off + lo - j * cell)
                        store = self.master[m_off:m_off + (hi - lo)]
                        store.copy_(src[lo:hi])
                    else:
                        store = self.flat[off + lo:off + hi]
                    piece = torch.nn.Parameter(store.view(pshape), requires_grad=False)
                    piece.grad_dtype = None
                    local.append((i, lo, hi, k, piece))
                    owned_numel += hi - lo
                    if native:
                        whole = (lo, hi) == (0, n)
                        slots = None
                        if not whole:
                            slots = []
                            for r in range(self.rounds - self._e[i], self.rounds):
                                a, ln = self._slot_of[(i, r)]
                                a += self._round_start[r]
                                slots.append(self.xbuf[a:a + ln])
                        cols = shapes[i][1] if kind == "rows" else 0
                        pieces_info[id(piece)] = Piece(
                            full_numel=n, full_rows=shapes[i][0] if kind == "rows" else 0, elem0=lo,
                            row0=lo // cols if cols else 0, slots=slots,
                            copy=self.flat[off + lo:off + hi] if self.master is not None else None)
                p.data = view.view(shapes[i])
        self.owned_numel = owned_numel
        self.total_numel = sum(numels)
        self._local = local
        # inner groups: part-major, so that a part's parameters are complete before the next part's
        inner_groups, self._part_of_group, self._origin = [], [], []
        for k in range(self.parts):
            for gi, g in enumerate(groups):
                ids = {id(p) for p in g["params"]}
                mine = [pc for (i, lo, hi, kk, pc) in local if kk == k and id(all_params[i]) in ids]
                if mine:
                    inner_groups.append(dict({kk: v for kk, v in g.items() if kk != "params"}, params=mine))
                    self._part_of_group.append(k)
                    self._origin.append(gi)
        self.inner = inner_factory(inner_groups, **kwargs) if inner_groups else None
        if self.inner is not None and native:
            self.inner._pieces = pieces_info
            self.inner._shard = _Schedule(self)
            # stochastic-rounding seeds as the unsharded optimizer would hand them out: one per 16-bit
            # parameter of a group that rounds stochastically, in parameter order; every piece of a
            # tensor takes its tensor's seed
            seeds, nxt = {}, 1
            for gi, g in enumerate(groups):
                sr = self._options[gi].get("stochastic_round_writeback", False)
                for p in g["params"]:
                    if sr and p.dtype in (torch.bfloat16, torch.float16) and compute_dtype is None:
                        seeds[id(p)] = nxt
                        nxt += 1
            self.inner._sr_seed_map = {id(pc): seeds[id(all_params[i])] for (i, lo, hi, k, pc) in local
                                       if id(all_params[i]) in seeds}
            self.inner._sr_seed_counter = nxt
            # the same for the projection seeds of APOLLO (one per tensor of two or more dimensions in a
            # group with a rank, in parameter order: optimizer.py:1726-1728)
            seeds, nxt = {}, 1
            for gi, g in enumerate(groups):
                rank = self._options[gi].get("apollo_rank", 0)
                for p in g["params"]:
                    if rank and rank > 0 and p.dim() >= 2:
                        seeds[id(p)] = nxt
                        nxt += 1
            self.inner._apollo_seed_map = {id(pc): seeds[id(all_params[i])] for (i, lo, hi, k, pc) in local
                                           if id(all_params[i]) in seeds}
            self.inner._apollo_seed_counter = nxt
        self._bound = {}
        self._local_by_tensor = {}
        for (i, lo, hi, k, pc) in local:
            self._local_by_tensor.setdefault(i, []).append((lo, hi, pc))
        self.gather_stream = None
        self._push_streams, self._pushed = None, False
        self._fence = torch.zeros(1, dtype=torch.float32, device=dev) if self.peer_flat is not None else None
        self._start = torch.zeros(1, dtype=torch.float32, device=dev) if self.peer_flat is not None else None
        self.push_sync = self.push_order == "shift" and os.environ.get("AF8_PUSH_SYNC", "1") != "0"
        self._pipelined = self._in_step = False
        self.gather_log = []          # units in the order this rank gathered them during the last step

    # -- views of the inner optimizer ---------------------------------------------------------------
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
        for (_, _, _, _, pc) in self._local:
            pc.grad = None
        self._bound = {}

    # -- the step -------------------------------------------------------------------------------------
    def _bind_grads(self):
        """Every piece takes the matching stretch of its tensor's gradient (a view, no copy).  Pieces of
        a tensor whose gradient is the same tensor at the same address as at the last step keep theirs."""
        bound = self._bound
        for i, pcs in self._local_by_tensor.items():
            g = self.all_params[i].grad
            if g is None:
                if bound.get(i) is not None:
                    for (lo, hi, pc) in pcs:
                        pc.grad = None
                    bound[i] = None
                continue
            was = bound.get(i)
            if was is not None and was[0] is g and was[1] == g.data_ptr():
                continue
            fg = (g if g.is_contiguous() else g.contiguous()).view(-1)
            for (lo, hi, pc) in pcs:
                pc.grad = fg[lo:hi].view(pc.shape)
            bound[i] = (g, g.data_ptr()) if g.is_contiguous() else None

    def local_step(self, closure=None):
        """Update the pieces this rank owns.  With the native optimizer and cut tensors this includes
        the exchange of their statistics, so every rank must call it."""
        if not self._in_step:
            self._pipelined = False           # called on its own: no gather
        self._bind_grads()
        if self.xbuf is not None and self.rounds:
            self.xbuf.zero_()
        if self.inner is not None:
            return self.inner.step(closure)
        # a rank that owns nothing still takes part in the collectives
        for r in range(self.rounds):
            self._exchange(r)
        for k in range(self.parts):
            self._after_part(k)
        return None

    def _exchange(self, r):
        n = self._round_size[r]
        if n and self.world > 1:
            a = self._round_start[r]
            dist.all_reduce(self.xbuf[a:a + n], group=self.group)

    def _symmetric_buffer(self, numel, dtype, dev, required):
        """-> (buffer, [every rank's buffer as a tensor of this process]) in symmetric memory, or
        (None, None) when it cannot be set up on every rank."""
        ok, buf, peers = 1, None, None
        try:
            import torch.distributed._symmetric_memory as symm
            buf = symm.empty(numel, dtype=dtype, device=dev)
            group = self.group if self.group is not None else dist.group.WORLD
            handle = symm.rendezvous(buf, group)
            peers = [handle.get_buffer(r, (numel,), dtype) for r in range(self.world)]
            buf.zero_()
            self._symm_handle = handle
        except Exception as e:          # no fabric / file-descriptor passing, old driver, ...
            ok, self._symm_error = 0, repr(e)
        flag = torch.tensor([ok], device=dev, dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        if int(flag.item()) == 1:
            return buf, peers
        if required:
            raise RuntimeError("symmetric memory could not be set up on every rank: " + getattr(self, "_symm_error", "another rank failed"))
        return None, None

    def _unit(self, k):
        n = self.world * self.cell
        return self.flat[k * n:(k + 1) * n]

    def _gather_unit(self, k):
        """Publish this rank's cell of unit k (on the current stream's order)."""
        self.gather_log.append(k)
        if self.world == 1:
            return
        a = (k * self.world + self.rank) * self.cell
        if self.peer_flat is None:
            unit = self._unit(k)
            dist.all_gather_into_tensor(unit, unit[self.rank * self.cell:(self.rank + 1) * self.cell], group=self.group)
            return
        cur = torch.cuda.current_stream(self.flat.device)
        if self._push_streams is None:
            self._push_streams = [torch.cuda.Stream(device=self.flat.device) for _ in range(self.world)]
        ev = torch.cuda.Event()
        ev.record(cur)
        mine = self.flat[a:a + self.cell]
        if self.push_order == "shift":
            # one copy at a time, to rank + 1, rank + 2, ...: while the ranks move in step every rank sends to one
            # peer and receives from one, each pair at the full rate of a single peer copy (several copies running
            # at once from one GPU were measured at half that in total on 4 GPUs)
            st = self._push_streams[0]
            with torch.cuda.stream(st):
                st.wait_event(ev)
                if self.push_sync:
                    # the shifted order only avoids two senders at one receiver while the ranks move in step; ranks
                    # whose parts take different times (whole tensors of unequal cost) drift apart, and a drifted
                    # sender halves the rate of the receiver it shares.  A tiny all-reduce lines the ranks up
                    # before every unit; every rank issues it at the same place of its sequence of collectives.
                    dist.all_reduce(self._start, group=self.group)
                for j in range(1, self.world):
                    r = (self.rank + j) % self.world
                    self.peer_flat[r][a:a + self.cell].copy_(mine, non_blocking=True)     # a copy-engine transfer over NVLink
        else:
            for r in range(self.world):
                if r == self.rank:
                    continue
                st = self._push_streams[r]
                with torch.cuda.stream(st):
                    st.wait_event(ev)
                    self.peer_flat[r][a:a + self.cell].copy_(mine, non_blocking=True)
        self._pushed = True

    def _gather_fence(self):
        """After the last unit: when this returns (in stream order), every rank's cells have arrived here."""
        if self.peer_flat is None or self.world == 1 or not self._pushed:
            return
        cur = torch.cuda.current_stream(self.flat.device)
        for r in range(self.world):
            if r != self.rank:
                cur.wait_stream(self._push_streams[r])
        dist.all_reduce(self._fence, group=self.group)       # behind this rank's copies; complete only when all ranks got there
        self._pushed = False

    def gather(self):
        """Publish every unit of the flat parameter buffer, in unit order, and wait (in stream order)
        for the other ranks' cells."""
        for k in range(self.parts):
            self._gather_unit(k)
        self._gather_fence()

    def _after_part(self, k):
        if not self._pipelined:
            return
        ev = torch.cuda.Event()
        ev.record(self._main)
        with torch.cuda.stream(self.gather_stream):
            self.gather_stream.wait_event(ev)
            self._gather_unit(k)

    def step(self, closure=None):
        """Local update and parameter all-gather.  On CUDA with the native optimizer the gather of a
        part starts, on a second stream, as soon as the launches that write that part have been
        enqueued; every rank gathers the units in the same order, 0 .. parts - 1."""
        self.gather_log = []
        native = self.inner is None or hasattr(self.inner, "_shard")
        self._pipelined = bool(self.world > 1 and self.flat.is_cuda and native and self.xbuf is not None)
        if not self._pipelined:
            loss = self.local_step(closure)
            self.gather()
            return loss
        if self.gather_stream is None:
            self.gather_stream = torch.cuda.Stream(device=self.flat.device)
        self._main = torch.cuda.current_stream(self.flat.device)
        self._in_step = True
        try:
            loss = self.local_step(closure)
        finally:
            self._in_step = False
        with torch.cuda.stream(self.gather_stream):
            self._gather_fence()
        self._main.wait_stream(self.gather_stream)
        return loss

    # -- checkpoints in the unsharded optimizer's layout ------------------------------------------
    _CONCAT = ("variance_q", "variance_scale", "variance_min_log", "m_q", "m_scale")

    def _piece_states(self):
        """-> {tensor index: [(lo, hi, piece shape, state on the CPU)]} of this rank."""
        out = {}
        if self.inner is None:
            return out
        for (i, lo, hi, k, pc) in self._local:
            st = self.inner.state.get(pc)
            if st:
                out.setdefault(i, []).append((lo, hi, tuple(pc.shape), {
                    key: (v.detach().cpu() if isinstance(v, torch.Tensor) else v) for key, v in st.items()}))
        return out

    def _merge(self, i, parts):
        """States of the pieces of tensor i (sorted by position) -> the state of the whole tensor."""
        parts = sorted(parts, key=lambda t: t[0])
        if len(parts) == 1 and (parts[0][0], parts[0][1]) == (0, self.all_params[i].numel()):
            return parts[0][3]
        shape = tuple(self.all_params[i].shape)
        first = parts[0][3]
        out = {}
        for key, v in first.items():
            vals = [st[key] for (_, _, _, st) in parts]
            if not isinstance(v, torch.Tensor):
                out[key] = v
            elif key in self._CONCAT:
                out[key] = torch.cat([x.reshape(-1) for x in vals])
            elif tuple(v.shape) == parts[0][2] and v.dim() > 0:
                out[key] = torch.cat([x.reshape(-1) for x in vals]).reshape(shape)
            else:
                out[key] = v                           # kept by every owner (row / column states, scalars)
        if "variance_shape" in out:
            out["variance_shape"] = torch.Size(shape)
            out["variance_pad"] = parts[-1][3].get("variance_pad", 0)
        return out

    def full_state_dict(self, dst=0):
        """The state of all ranks merged into the layout an unsharded optimizer saves (and the
        reference's class loads): {"state": {parameter index: state}, "param_groups": [...]} plus
        the optimizer-level counters.  Tensors are moved to the CPU.  Collective: every rank calls
        it; rank `dst` gets the dictionary, the others None."""
        inner_sd = self.inner.state_dict() if self.inner is not None else {"state": {}, "param_groups": []}
        extras = {k: v for k, v in inner_sd.items() if k not in ("state", "param_groups")}
        options = {self._origin[j]: {k: v for k, v in g.items() if k != "params"}
                   for j, g in enumerate(inner_sd["param_groups"])}
        payload = (self._piece_states(), extras, options)
        if self.world > 1:
            gathered = [None] * self.world if self.rank == dst else None
            dist.gather_object(payload, gathered, dst=dst, group=self.group)
            if self.rank != dst:
                return None
        else:
            gathered = [payload]
        pieces, extras, options = {}, {}, {}
        for m, e, o in gathered:
            for i, lst in m.items():
                pieces.setdefault(i, []).extend(lst)
            for k, v in e.items():
                extras[k] = max(extras[k], v) if (k in extras and isinstance(v, (int, float))) else v
            for gi, opts in o.items():
                options.setdefault(gi, opts)
        state = {i: self._merge(i, lst) for i, lst in pieces.items()}
        groups, first = [], 0
        for gi, g in enumerate(self._groups):
            opts = options.get(gi, {k: v for k, v in g.items() if k != "params"})
            groups.append(dict(opts, params=list(range(first, first + len(g["params"])))))
            first += len(g["params"])
        return dict(extras, state=dict(sorted(state.items())), param_groups=groups)

    def _slice(self, i, lo, hi, pshape, st):
        """The part of the whole tensor's state `st` that belongs to elements lo .. hi of tensor i."""
        n = self.all_params[i].numel()
        if (lo, hi) == (0, n):
            return st
        shape = tuple(self.all_params[i].shape)
        out = {}
        block = st.get("block_size")
        m_block = st.get("m_block_size")
        packed = st.get("m_quant_type") in ("uf4", "d4")
        for key, v in st.items():
            if not isinstance(v, torch.Tensor):
                out[key] = v
            elif key in ("variance_q",):
                out[key] = v.reshape(-1)[lo:_pad(hi, block)].clone()
            elif key in ("variance_scale", "variance_min_log"):
                out[key] = v.reshape(-1)[lo // block:-(-hi // block)].clone()
            elif key == "m_q":
                a, b = lo, _pad(hi, m_block)
                out[key] = v.reshape(-1)[(a // 2 if packed else a):(b // 2 if packed else b)].clone()
            elif key == "m_scale":
                out[key] = v.reshape(-1)[lo // m_block:-(-hi // m_block)].clone()
            elif tuple(v.shape) == shape and v.dim() > 0:
                out[key] = v.reshape(-1)[lo:hi].reshape(pshape).clone()
            else:
                out[key] = v
        if "variance_shape" in out:
            out["variance_shape"] = torch.Size(pshape)
            out["variance_pad"] = _pad(hi - lo, block) - (hi - lo)
        return out

    def load_full_state_dict(self, sd):
        """Load a state dictionary in the unsharded layout (from full_state_dict, from an unsharded
        optimizer of this package or from the reference): every rank keeps the states of its pieces."""
        if self.inner is None:
            return
        inner_sd = self.inner.state_dict()
        index_of = {id(pc): (i, lo, hi) for (i, lo, hi, k, pc) in self._local}
        inner_params = [p for g in self.inner.param_groups for p in g["params"]]
        state = {}
        for idx, pc in enumerate(inner_params):
            i, lo, hi = index_of[id(pc)]
            st = sd["state"].get(i)
            if st is not None:
                state[idx] = self._slice(i, lo, hi, tuple(pc.shape), st)
        groups = []
        for j, g in enumerate(inner_sd["param_groups"]):
            saved = sd["param_groups"][self._origin[j]]
            groups.append(dict({k: v for k, v in saved.items() if k != "params"}, params=g["params"]))
        extras = {k: v for k, v in sd.items() if k not in ("state", "param_groups")}
        self.inner.load_state_dict(dict(extras, state=state, param_groups=groups))

    def state_dict(self):
        """State of the pieces this rank owns (a per-rank shard; full_state_dict gives the unsharded
        layout).  With a compute copy the shard also holds the rank's fp32 master values."""
        return {"rank": self.rank, "world": self.world, "parts": self.parts, "cell": self.cell,
                "offsets": list(self.offsets), "inner": self.inner.state_dict() if self.inner is not None else None,
                "master": self.master.detach().cpu() if self.master is not None else None}

    def load_state_dict(self, sd):
        if (sd["world"] != self.world or sd.get("parts") != self.parts or sd.get("cell") != self.cell
                or list(sd["offsets"]) != list(self.offsets)):
            raise ValueError("sharded state was saved with a different partition")
        if self.inner is not None and sd["inner"] is not None:
            self.inner.load_state_dict(sd["inner"])
        if self.master is not None and sd.get("master") is not None:
            self.master.copy_(sd["master"])

    def master_params(self, dst=0):
        """fp32 values of all parameters gathered on rank `dst` (None elsewhere): the masters with a
        compute copy, else the parameters themselves.  Collective."""
        mine = {}
        for (i, lo, hi, k, pc) in self._local:
            mine.setdefault(i, []).append((lo, pc.detach().reshape(-1).float().cpu()))
        if self.world > 1:
            gathered = [None] * self.world if self.rank == dst else None
            dist.gather_object(mine, gathered, dst=dst, group=self.group)
            if self.rank != dst:
                return None
        else:
            gathered = [mine]
        merged = {}
        for m in gathered:
            for i, lst in m.items():
                merged.setdefault(i, []).extend(lst)
        out = []
        for i, p in enumerate(self.all_params):
            lst = sorted(merged.get(i, []), key=lambda t: t[0])
            out.append(torch.cat([v for _, v in lst]).reshape(p.shape) if lst else torch.zeros(p.shape))
        return out
