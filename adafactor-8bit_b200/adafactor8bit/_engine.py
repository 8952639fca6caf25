"""Launch plans: the layer between the optimizer class and the C ABI.

A plan owns the device-side tables of one multi-tensor launch (tensor
descriptors, per-tensor dynamic scalars, per-block partial sums) and their
pinned host mirrors.  Each step the optimizer refreshes the host mirror
(gradient pointers and the step's scalars change) and the plan enqueues the
passes on the current CUDA stream.
"""
import ctypes
import math

import numpy as np
import torch

from . import _native as N

_GRAD_DT = {torch.float32: N.F32, torch.bfloat16: N.BF16, torch.float16: N.F16}
_SR_K1, _SR_K2, _M64 = 0x9E3779B97F4A7C15, 0xD1B54A32D192ED03, (1 << 64) - 1


def sr_base(seed, step):
    """Counter origin of a parameter's stochastic rounding at one step: the seed / step mix of
    the reference's seeded stream (optimizer.py:205; kernels.cu:56-61); element i draws from
    counter sr_base + i."""
    return (int(seed) * _SR_K1 + int(step) * _SR_K2) & _M64



def _ptr(t):
    return 0 if t is None else t.data_ptr()


class Piece:
    """Describes a launch-table entry that holds only part of a tensor: a run of flat elements
    (full-rank path) or a run of rows (factored path) of a tensor whose other parts sit in other
    launch tables, possibly on other GPUs (the sharded optimizer).  Everything that the
    reference derives from the whole tensor -- its element count in the clip and RMS divisors, its
    norms, its row and column statistics -- then comes from `full_*` and, for the sums, from the
    exchange slots.

    full_numel, full_rows: size of the whole tensor.
    elem0: flat index, in the whole tensor, of the entry's first element (origin of the stochastic
           rounding counters); row0: its first row (factored path).
    slots: None when the entry holds the whole tensor.  Otherwise one float64 tensor per exchange
           point of the plan's pass sequence: layout [8 scalars | full_rows row sums (padded to a
           multiple of 4) | column sums].  The plan ADDS its local sums there; between two passes
           the caller all-reduces the slots, after which they hold the whole tensor's sums.
    copy:  optional bf16 tensor of the entry's size that receives the updated parameter rounded to
           nearest (the compute copy of a mixed-precision run)."""
    __slots__ = ("full_numel", "full_rows", "elem0", "row0", "slots", "copy")

    def __init__(self, full_numel, full_rows=0, elem0=0, row0=0, slots=None, copy=None):
        self.full_numel, self.full_rows, self.elem0, self.row0 = int(full_numel), int(full_rows), int(elem0), int(row0)
        self.slots, self.copy = slots, copy


def fullrank_exchanges(scale, d, fira, momentum_only, lag):
    """Number of exchange points of FullrankPlan.stages for these options."""
    need_stat = bool(fira) or d > 0
    if not momentum_only:
        if lag and need_stat:
            return 0
        return 1 if (scale or need_stat) else 0
    return (1 if (scale or d > 0) else 0) + (1 if fira else 0)


def factored_exchanges(came, d, fira, lag):
    """Number of exchange points of FactoredPlan.stages for these options."""
    if came:
        return 3 + (1 if fira else 0)
    return 1 + (1 if ((fira or d > 0) and not lag) else 0)


def _add_to_slot(slot, k, values):
    """slot[k] += sum(values) in binary64."""
    slot[k].add_(values.sum(dtype=torch.float64))


def dynamic_map(total_bits):
    """The signed dynamic-map codebook of the d8 / d4 momentum formats, built
    with the same torch float32 operations as the reference so that both produce
    identical tables on the same host (_create_dynamic_map, optimizer.py:416-441;
    8 bits use 7 exponent bits, 4 bits use 3, optimizer.py:122-123)."""
    exp_bits = 7 if total_bits == 8 else 3
    mantissa_bits = total_bits - 1
    values = []
    for i in range(exp_bits):
        edges = torch.linspace(0.1, 1, int(2 ** (i + mantissa_bits - exp_bits) + 1), dtype=torch.float32)
        centres = (edges[:-1] + edges[1:]) / 2.0
        magnitude = 10 ** (-(exp_bits - 1) + i)
        values += (magnitude * centres).tolist() + (-magnitude * centres).tolist()
    extra = 2 ** (mantissa_bits - exp_bits) - 1
    if extra > 0:
        edges = torch.linspace(0.1, 1, extra + 1, dtype=torch.float32)
        centres = (edges[:-1] + edges[1:]) / 2.0
        values += centres.tolist() + (-centres).tolist()
    values += [0, 1.0]
    if len(values) != 2 ** total_bits:
        raise AssertionError("dynamic map has the wrong number of entries")
    return np.asarray(sorted(values), dtype=np.float32)


_QMAP_DEVICES = set()

# When set to a list, every kernel launch appends (name, parameters covered,
# start event, end event), recorded on the launch stream.  Used by bench.py to
# time individual kernels inside its timed region; None disables it.
LAUNCH_LOG = None
_MODE_NAMES = {N.MODE_NOCLIP: "noclip", N.MODE_SUMSQ: "sumsq", N.MODE_APPLY: "apply", N.MODE_SUMSQ_M: "sumsq_m",
               N.MODE_LAG: "lag"}


def lag_table(h_ring, d_table, states, device, first_block, n_blocks, numel, table_alpha, alpha_dev, d, fira,
              fira_margin, partials_f64, stream):
    """Fill and upload the af8_lag_tensor rows of a plan.  The three scalars are the reference's
    state entries (optimizer.py:1056-1071); entries that do not exist yet are created here."""
    n = len(states)
    buf = h_ring.next()
    lt = buf.numpy()[: n * N.LAG_TENSOR.itemsize].view(N.LAG_TENSOR)
    lt[:] = np.zeros(n, dtype=N.LAG_TENSOR)
    lt["first_block"], lt["n_blocks"] = first_block, n_blocks
    lt["alpha"] = table_alpha
    lt["alpha_dev"] = alpha_dev
    sqrt_n = np.sqrt(numel.astype(np.float64))
    lt["clip_div"] = (sqrt_n * d).astype(np.float32) if d > 0 else np.float32(0.0)
    lt["fira_margin1"] = np.float32(1.0 + fira_margin)
    lt["partials_f64"] = int(partials_f64)
    for i, st in enumerate(states):
        pun = st.get("prev_update_norm")
        if pun is None:
            pun = torch.zeros(1, dtype=torch.float32, device=device)
            st["prev_update_norm"] = pun
        lt["prev_update_norm"][i] = pun.data_ptr()
        if fira:
            fs = st.get("lag_fira_scale")
            lt["has_lag_fira"][i] = int(fs is not None)
            if fs is None:
                fs = torch.ones((), dtype=torch.float32, device=device)
                st["lag_fira_scale"] = fs
            prev = st.get("fira_prev_norm")
            lt["fira_has_prev"][i] = int(prev is not None)
            if prev is None:
                prev = torch.zeros((), dtype=torch.float32, device=device)
                st["fira_prev_norm"] = prev
            lt["lag_fira_scale"][i] = fs.data_ptr()
            lt["fira_prev"][i] = prev.data_ptr()
    d_table.copy_(buf[: d_table.numel()], non_blocking=True)
    h_ring.mark(stream)


def ensure_qmap(device):
    """Upload both codebooks to `device` once (optimizer.py:109-133)."""
    device = torch.device(device)
    if device in _QMAP_DEVICES:
        return
    m8 = np.ascontiguousarray(dynamic_map(8))
    m4 = np.ascontiguousarray(dynamic_map(4))
    with torch.cuda.device(device):
        rc = N.lib().af8_set_qmap(m8.ctypes.data, m4.ctypes.data, torch.cuda.current_stream().cuda_stream)
        N.check(rc, "af8_set_qmap")
        torch.cuda.current_stream().synchronize()   # the host arrays die with this frame
    _QMAP_DEVICES.add(device)


class _PinnedRing:
    """A small ring of pinned host buffers.  A buffer is reused only after the
    copy that read it has completed on the device."""

    def __init__(self, nbytes, depth=3):
        self.bufs = [torch.empty(max(nbytes, 16), dtype=torch.uint8, pin_memory=True) for _ in range(depth)]
        self.events = [None] * depth
        self.i = 0

    def next(self):
        self.i = (self.i + 1) % len(self.bufs)
        ev = self.events[self.i]
        if ev is not None:
            ev.synchronize()
        return self.bufs[self.i]

    def mark(self, stream):
        ev = self.events[self.i]
        if ev is None:
            ev = torch.cuda.Event()
            self.events[self.i] = ev
        ev.record(stream)


class FullrankKey(tuple):
    """(grad_dtype, v_fmt, m_fmt, block, m_block, use_adam_denom, momentum_only, negate)"""


class FullrankPlan:
    """One multi-tensor launch group of the full-rank path: all tensors share
    the kernel configuration `key`; per-tensor scalars live in the table.

    pieces: optional list with a Piece (or None) per entry, for entries that are parts of larger
    tensors."""

    def __init__(self, device, grad_dtype, v_fmt, m_fmt, block, m_block, use_adam_denom,
                 momentum_only, negate, params, states, stochastic_round=False, pieces=None):
        self.device = torch.device(device)
        self.params = list(params)
        self.states = list(states)
        n = len(self.params)
        self.n = n
        self.pieces = list(pieces) if pieces is not None else [None] * n
        self.cut = [i for i, pc in enumerate(self.pieces) if pc is not None and pc.slots is not None]
        self.cfg = N.FullrankCfg()
        pdt = self.params[0].dtype
        if pdt not in _GRAD_DT or any(p.dtype != pdt for p in self.params):
            raise RuntimeError("the full-rank kernels update fp32, bf16 or fp16 parameters, one dtype per launch group")
        self.cfg.param_dtype = _GRAD_DT[pdt]
        self.cfg.stochastic_round = int(bool(stochastic_round) and pdt != torch.float32)   # optimizer.py:2032
        self.cfg.grad_dtype = _GRAD_DT[grad_dtype]
        self.cfg.v_fmt = N.V_FMT[v_fmt]
        self.cfg.m_fmt = N.M_FMT[m_fmt]
        self.cfg.block = int(block)
        self.cfg.m_block = int(m_block) if m_block else 0
        # the momentum-only rule exists only with momentum and always normalises
        # with rsqrt(max(v, eps_sq)) (optimizer.py:893-896)
        momentum_only = bool(momentum_only) and m_fmt is not None
        self.cfg.use_adam_denom = int(bool(use_adam_denom) and not momentum_only)
        self.cfg.momentum_only = int(momentum_only)
        self.cfg.negate_grad = int(bool(negate))
        self.cfg.v_floor = -126.0     # optimizer.py:299 (default min_log_floor)
        if m_fmt in ("d8", "d4"):
            ensure_qmap(self.device)
        self.numel = np.array([p.numel() for p in self.params], dtype=np.int64)
        # element count of the tensor an entry belongs to: what the clip and RMS divisors use
        self.full_numel = np.array([pc.full_numel if pc is not None else p.numel()
                                    for p, pc in zip(self.params, self.pieces)], dtype=np.int64)
        self.nblocks = (self.numel + block - 1) // block
        self.first_block = np.concatenate([[0], np.cumsum(self.nblocks)[:-1]]).astype(np.int64)
        self.total_blocks = int(self.nblocks.sum())
        self.total_numel = int(self.numel.sum())

        self.d_table = torch.empty(n * N.FULLRANK_TENSOR.itemsize, dtype=torch.uint8, device=self.device)
        self.d_dyn = torch.zeros(n * N.DYN_SCALARS.itemsize, dtype=torch.uint8, device=self.device)
        self.d_norm = torch.empty(n * N.NORM_TENSOR.itemsize, dtype=torch.uint8, device=self.device)
        self.d_sumsq = None
        self.h_table = _PinnedRing(n * N.FULLRANK_TENSOR.itemsize)
        self.h_norm = _PinnedRing(n * N.NORM_TENSOR.itemsize)
        self.h_scale = None
        self.d_scale = None
        self.d_chunks = None
        self.h_lag = self.d_lag = None
        self._static = None
        self._ptr_sig = None
        self._alpha_on_device = False
        for p in self.params:
            if not p.is_contiguous():
                raise RuntimeError("parameters must be contiguous")

    # -- table ---------------------------------------------------------------
    def _pointer_signature(self):
        """Addresses of the parameters.  A parameter whose storage was replaced (p.data = ...,
        module.to(...)) keeps its Python identity, so the cached table is checked against the
        addresses at every step.  (State tensors are replaced only by the optimizer itself, which
        then drops its launch plans.)"""
        return [p.data_ptr() for p in self.params]

    def _static_fields(self):
        """Pointers and sizes that only change when a parameter's or a state's storage is replaced."""
        t = np.zeros(self.n, dtype=N.FULLRANK_TENSOR)
        for i, (p, st) in enumerate(zip(self.params, self.states)):
            t["param"][i] = p.data_ptr()
            t["v_q"][i] = _ptr(st.get("variance_q"))
            t["v_scale"][i] = _ptr(st.get("variance_scale"))
            t["v_min_log"][i] = _ptr(st.get("variance_min_log"))
            t["v_f32"][i] = _ptr(st.get("variance"))
            t["m_q"][i] = _ptr(st.get("m_q"))
            t["m_scale"][i] = _ptr(st.get("m_scale"))
            t["m_f32"][i] = _ptr(st.get("m"))
            pc = self.pieces[i]
            if pc is not None and pc.copy is not None:
                if pc.copy.numel() != p.numel() or pc.copy.dtype != torch.bfloat16:
                    raise RuntimeError("the compute copy of a parameter must be a bf16 tensor of its size")
                t["param_copy"][i] = pc.copy.data_ptr()
        t["numel"] = self.numel
        t["first_block"] = self.first_block
        return t

    def invalidate(self):
        self._static = None

    def fill_table(self, grads, scalars):
        """scalars: dict of per-tensor float32 arrays (or python floats) named as
        the table fields."""
        sig = self._pointer_signature()
        if self._static is None or sig != self._ptr_sig:
            self._static = self._static_fields()
            self._ptr_sig = sig
        buf = self.h_table.next()
        table = buf.numpy()[: self.n * N.FULLRANK_TENSOR.itemsize].view(N.FULLRANK_TENSOR)
        table[:] = self._static
        table["grad"] = [g.data_ptr() for g in grads]
        for k in ("decay", "alpha", "v_w", "v_keep", "v_eps_add", "m_w", "eps_gradsq", "eps_denom", "eps_sq"):
            table[k] = scalars[k]
        table["sr_base"] = scalars.get("sr_base", 0)
        return buf, table

    # -- launches ------------------------------------------------------------
    def kernel_name(self, mode):
        c = self.cfg
        fast = (c.v_fmt == N.V_AL8 and c.m_fmt == N.M_UF8 and c.block == 2048 and c.m_block == 256
                and c.use_adam_denom and not c.momentum_only and mode != N.MODE_SUMSQ_M
                and ((c.param_dtype == N.F32 and c.grad_dtype in (N.F32, N.BF16))
                     or (c.param_dtype == N.BF16 and c.grad_dtype == N.BF16)))
        if fast and mode == N.MODE_SUMSQ:
            return "fullrank_stat"
        return ("fullrank_fast_" if fast else "fullrank_generic_") + _MODE_NAMES[mode]

    def _step(self, mode, host_buf, stream):
        self.cfg.mode = mode
        log = LAUNCH_LOG
        if log is not None:
            e0 = torch.cuda.Event(enable_timing=True)
            e1 = torch.cuda.Event(enable_timing=True)
            e0.record(stream)
        rc = N.lib().af8_fullrank_step(
            ctypes.byref(self.cfg), host_buf.data_ptr() if host_buf is not None else None,
            self.d_table.data_ptr(), self.n, self.total_blocks, self.d_dyn.data_ptr(),
            self.d_sumsq.data_ptr() if self.d_sumsq is not None else None, stream.cuda_stream)
        N.check(rc, "af8_fullrank_step")
        if log is not None:
            e1.record(stream)
            log.append((self.kernel_name(mode), self.total_numel, e0, e1))
        if host_buf is not None:
            self.h_table.mark(stream)

    def _sums_to_slots(self, x, k, partials, first, count):
        """Add the local sum of every cut entry's partial sums into scalar k of its slot of exchange x."""
        for i in self.cut:
            a = int(first[i])
            _add_to_slot(self.pieces[i].slots[x], k, partials[a:a + int(count[i])])

    def _finalize(self, table, pre_div_mode, d, fira, fira_margin, stream, x=None, k=1):
        """x, k: exchange index and scalar index where the whole sums of the cut entries are."""
        buf = self.h_norm.next()
        nt = buf.numpy()[: self.n * N.NORM_TENSOR.itemsize].view(N.NORM_TENSOR)
        nt["first_block"] = self.first_block
        nt["n_blocks"] = self.nblocks
        if x is not None:
            for i in self.cut:
                nt["n_blocks"][i] = -1
                nt["first_block"][i] = self.pieces[i].slots[x].data_ptr() + 8 * k
        nt["pre_div_mode"] = pre_div_mode
        nt["partials_f64"] = 0
        nt["alpha"] = table["alpha"]
        if self._alpha_on_device:
            nt["alpha_dev"] = (self.d_table.data_ptr() + np.arange(self.n, dtype=np.uint64) * np.uint64(N.FULLRANK_TENSOR.itemsize)
                               + np.uint64(N.FULLRANK_TENSOR.fields["alpha"][1]))
        else:
            nt["alpha_dev"] = 0
        sqrt_n = np.sqrt(self.full_numel.astype(np.float64))
        nt["sqrt_n"] = sqrt_n.astype(np.float32)
        nt["d"] = np.float32(d)
        use_clip = d > 0 and pre_div_mode == 0
        nt["clip_div"] = (sqrt_n * d).astype(np.float32) if use_clip else np.float32(0.0)
        nt["fira_margin1"] = np.float32(1.0 + fira_margin)
        if fira and pre_div_mode != 1:
            nt["fira_prev"], nt["fira_has_prev"] = fira_state_pointers(self)
        else:
            nt["fira_prev"] = 0
            nt["fira_has_prev"] = 0
        self.d_norm.copy_(buf[: self.d_norm.numel()], non_blocking=True)
        self.h_norm.mark(stream)
        rc = N.lib().af8_norm_finalize(self.d_norm.data_ptr(), self.n, self.d_sumsq.data_ptr(),
                                       self.d_dyn.data_ptr(), stream.cuda_stream)
        N.check(rc, "af8_norm_finalize")

    def _scale_table(self, buf, scale, stream):
        """Upload the launch table and fill the host table of the parameter-RMS passes
        (scale_parameter=True, optimizer.py:850-853)."""
        chunk = N.lib().af8_scale_chunk()
        nchunks = (self.numel + chunk - 1) // chunk
        if self.h_scale is None:
            self.h_scale = _PinnedRing(self.n * N.SCALE_TENSOR.itemsize)
            self.d_scale = torch.empty(self.n * N.SCALE_TENSOR.itemsize, dtype=torch.uint8, device=self.device)
            self.d_chunks = torch.empty(int(nchunks.sum()), dtype=torch.float32, device=self.device)
        rc = N.lib().af8_fullrank_upload(ctypes.byref(self.cfg), buf.data_ptr(), self.d_table.data_ptr(), self.n,
                                         self.total_blocks, stream.cuda_stream)
        N.check(rc, "af8_fullrank_upload")
        self.h_table.mark(stream)
        hb = self.h_scale.next()
        t = hb.numpy()[: self.n * N.SCALE_TENSOR.itemsize].view(N.SCALE_TENSOR)
        fill_scale_table(t, self.params, self.numel, self.full_numel, nchunks, self.cfg.param_dtype, scale)
        self._scale_first, self._scale_count = t["first_chunk"].copy(), nchunks
        return hb, t

    def _param_scale(self, buf, scale, stream, x=None):
        """First half of alpha / decay from the parameters' RMS: partial sums of squares; the cut
        entries' local sums go to scalar 0 of their slots of exchange x.  _param_finish evaluates."""
        hb, t = self._scale_table(buf, scale, stream)
        if self.cut and x is not None:
            for i in self.cut:
                t["total"][i] = self.pieces[i].slots[x].data_ptr()         # scalar 0 of the slot
        N.check(N.lib().af8_param_sumsq(hb.data_ptr(), self.d_scale.data_ptr(), self.n, self.d_chunks.data_ptr(),
                                        stream.cuda_stream), "af8_param_sumsq")
        self.h_scale.mark(stream)
        if x is not None:
            self._sums_to_slots(x, 0, self.d_chunks, self._scale_first, self._scale_count)

    def _param_finish(self, stream):
        N.check(N.lib().af8_param_scale_finish(self.d_scale.data_ptr(), self.n, self.d_chunks.data_ptr(),
                                               self.d_table.data_ptr(), N.FULLRANK_TENSOR.itemsize,
                                               N.FULLRANK_TENSOR.fields["alpha"][1], N.FULLRANK_TENSOR.fields["decay"][1],
                                               stream.cuda_stream), "af8_param_scale_finish")

    def _alpha_dev_ptrs(self):
        if not self._alpha_on_device:
            return 0
        return (self.d_table.data_ptr() + np.arange(self.n, dtype=np.uint64) * np.uint64(N.FULLRANK_TENSOR.itemsize)
                + np.uint64(N.FULLRANK_TENSOR.fields["alpha"][1]))

    def _run_lag(self, buf, table, d, fira, fira_margin, stream):
        """lag_norm=True: one pass that clips and limits with the previous step's norm and leaves
        this step's norm for the next one (optimizer.py:1056-1071)."""
        if self.cut:
            raise RuntimeError("lag_norm needs whole tensors: a tensor that is split over launch tables cannot lag")
        if self.h_lag is None:
            self.h_lag = _PinnedRing(self.n * N.LAG_TENSOR.itemsize)
            self.d_lag = torch.empty(self.n * N.LAG_TENSOR.itemsize, dtype=torch.uint8, device=self.device)
        lag_table(self.h_lag, self.d_lag, self.states, self.device, self.first_block, self.nblocks, self.full_numel,
                  table["alpha"], self._alpha_dev_ptrs(), d, fira, fira_margin, False, stream)
        lib = N.lib()
        if buf is not None:
            N.check(lib.af8_fullrank_upload(ctypes.byref(self.cfg), buf.data_ptr(), self.d_table.data_ptr(), self.n,
                                            self.total_blocks, stream.cuda_stream), "af8_fullrank_upload")
            self.h_table.mark(stream)
        N.check(lib.af8_lag_scalars(self.d_lag.data_ptr(), self.n, 0, None, self.d_dyn.data_ptr(), stream.cuda_stream),
                "af8_lag_scalars")
        self._step(N.MODE_LAG, None, stream)
        N.check(lib.af8_lag_scalars(self.d_lag.data_ptr(), self.n, 1, self.d_sumsq.data_ptr(), self.d_dyn.data_ptr(),
                                    stream.cuda_stream), "af8_lag_scalars")

    def run(self, grads, scalars, d=0.0, fira=False, fira_margin=0.01, scale=None, stream=None, lag=False):
        """One optimizer step for every tensor of the plan, start to end."""
        for _ in self.stages(grads, scalars, d=d, fira=fira, fira_margin=fira_margin, scale=scale, stream=stream, lag=lag):
            pass

    def stages(self, grads, scalars, d=0.0, fira=False, fira_margin=0.01, scale=None, stream=None, lag=False):
        """The step as a generator (_dispatch_cuda_clip's pass structure, optimizer.py:1048-1077).
        It yields at every exchange point (fullrank_exchanges of them): the passes before a yield
        have added the local sums of the cut entries to their slots, the passes after it expect
        the slots to hold the whole tensors' sums.  Without cut entries the yields mean nothing.
        The last segment is the pass that writes the parameters.
        scale: per-tensor inputs of af8_param_scale when alpha depends on the
        parameter RMS; the table's alpha / decay are then produced on the device.
        lag: lag_norm=True; the momentum-only rule keeps its exact passes."""
        stream = stream or torch.cuda.current_stream(self.device)
        buf, table = self.fill_table(grads, scalars)
        self._alpha_on_device = scale is not None
        mom_only = bool(self.cfg.momentum_only)
        clip_first = d > 0                      # a statistic of the raw update is needed
        need_stat = fira or clip_first
        if need_stat and self.d_sumsq is None:
            self.d_sumsq = torch.empty(self.total_blocks, dtype=torch.float32, device=self.device)
        if need_stat and lag and not mom_only:
            if scale is not None:
                self._param_scale(buf, scale, stream)
                self._param_finish(stream)
                buf = None
            self._run_lag(buf, table, d, fira, fira_margin, stream)
            return
        x = 0
        if not mom_only:
            if scale is not None:
                self._param_scale(buf, scale, stream, x)
                buf = None
            if need_stat:
                self._step(N.MODE_SUMSQ, buf, stream)
                buf = None
                self._sums_to_slots(x, 1, self.d_sumsq, self.first_block, self.nblocks)
            if scale is not None or need_stat:
                yield
            if scale is not None:
                self._param_finish(stream)
            if need_stat:
                self._finalize(table, 0, d, fira, fira_margin, stream, x, 1)
                self._step(N.MODE_APPLY, None, stream)
            else:
                self._step(N.MODE_NOCLIP, buf, stream)
            return
        # momentum-only rule (optimizer.py:894-901): clip the normalised gradient
        # first, then limit the norm of the momentum that is applied with d = 0
        pending = buf
        if scale is not None:
            self._param_scale(pending, scale, stream, x)
            pending = None
        if clip_first:
            self._step(N.MODE_SUMSQ, pending, stream)
            pending = None
            self._sums_to_slots(x, 1, self.d_sumsq, self.first_block, self.nblocks)
        if scale is not None or clip_first:
            yield
            if scale is not None:
                self._param_finish(stream)
            if clip_first:
                self._finalize(table, 1, d, False, fira_margin, stream, x, 1)
            x += 1
        if not clip_first:
            self.d_dyn.view(torch.float32).view(self.n, 8)[:, 2] = 1.0   # pre_div
        if fira:
            self._step(N.MODE_SUMSQ_M, pending, stream)
            pending = None
            self._sums_to_slots(x, 1, self.d_sumsq, self.first_block, self.nblocks)
            yield
            self._finalize(table, 2, 0.0, True, fira_margin, stream, x, 1)
        self._step(N.MODE_APPLY, pending, stream)

    def norms(self):
        """Update norms measured by the last two-pass step (one per tensor)."""
        dyn = self.d_dyn.cpu().numpy().view(N.DYN_SCALARS)
        return dyn["norm"].copy()


def fira_state_pointers(plan):
    """-> (addresses of the tensors' "fira_prev_norm" scalars, flags: the scalar holds a value).  The
    state entry is created on a tensor's first limited step (optimizer.py:780-781); once every tensor
    of the plan has one, the addresses are reused while the entries stay the same objects."""
    cached = getattr(plan, "_fira_cache", None)
    if cached is not None and all(st.get("fira_prev_norm") is t for st, t in zip(plan.states, cached[0])):
        return cached[1], 1
    ptrs = np.zeros(plan.n, dtype=np.uint64)
    has = np.zeros(plan.n, dtype=np.int32)
    tensors = []
    for i, st in enumerate(plan.states):
        prev = st.get("fira_prev_norm")
        if prev is None:
            prev = torch.zeros((), dtype=torch.float32, device=plan.device)
            st["fira_prev_norm"] = prev
        else:
            has[i] = 1
        tensors.append(prev)
        ptrs[i] = prev.data_ptr()
    plan._fira_cache = (tensors, ptrs) if bool(has.all()) else None
    return ptrs, has


def fill_scale_table(t, params, numel, full_numel, nchunks, param_dtype, scale):
    """Fill an af8_scale_tensor table (host view `t`)."""
    t["param"] = [p.data_ptr() for p in params]
    t["numel"] = numel
    t["first_chunk"] = np.concatenate([[0], np.cumsum(nchunks)[:-1]])
    t["sqrt_n"] = np.sqrt(full_numel.astype(np.float64)).astype(np.float32)
    t["param_dtype"] = param_dtype
    t["total"] = 0
    for k in ("rho", "eps2", "bc", "weight_decay", "bc_mode", "scale_weight_decay"):
        t[k] = scale[k]


def _small_state_fields(row, st, prefix, fmt, block):
    """Fill one af8_small_state of a table row from the optimizer state dict."""
    row["fmt"] = N.V_FMT[fmt]
    row["block"] = int(block)
    if fmt == "fp32":
        row["f32"] = st[prefix].data_ptr()
    else:
        row["q"] = st[prefix + "_q"].data_ptr()
        row["scale"] = st[prefix + "_scale"].data_ptr()
        row["min_log"] = st[prefix + "_min_log"].data_ptr()


class FactoredPlan:
    """One multi-tensor launch group of the factored path (2-D tensors with row /
    column second moments; optionally momentum; optionally CAME confidence).

    pieces: optional list with a Piece (or None) per entry.  An entry with a Piece holds the rows
    row0 .. row0 + p.shape[0] of a tensor of full_rows rows; its row / column states describe the
    whole tensor."""

    def __init__(self, device, grad_dtype, m_fmt, m_block, came, negate, params, states, v_fmts, c_fmts,
                 stochastic_round=False, pieces=None):
        self.device = torch.device(device)
        self.params, self.states = list(params), list(states)
        self.n = n = len(self.params)
        self.pieces = list(pieces) if pieces is not None else [None] * n
        self.cut = [i for i, pc in enumerate(self.pieces) if pc is not None and pc.slots is not None]
        self.came = bool(came)
        self.cfg = N.FactoredCfg()
        pdt = self.params[0].dtype
        if pdt not in _GRAD_DT or any(p.dtype != pdt for p in self.params):
            raise RuntimeError("the factored kernels update fp32, bf16 or fp16 parameters, one dtype per launch group")
        self.cfg.param_dtype = _GRAD_DT[pdt]
        self.cfg.stochastic_round = int(bool(stochastic_round) and pdt != torch.float32)   # optimizer.py:2032
        self.cfg.grad_dtype = _GRAD_DT[grad_dtype]
        self.cfg.m_fmt = N.M_FMT[m_fmt]
        self.cfg.m_block = int(m_block) if m_block else 0
        self.cfg.came = int(self.came)
        self.cfg.negate_grad = int(bool(negate))
        self.cfg.v_floor = -126.0
        if m_fmt in ("d8", "d4"):
            ensure_qmap(self.device)
        for p, pc in zip(self.params, self.pieces):
            if not p.is_contiguous() or p.dim() < 2:
                raise RuntimeError("the factored kernels update contiguous parameters of two or more dimensions")
            if p.dim() > 2 and pc is not None and pc.slots is not None:
                raise RuntimeError("a tensor of more than two dimensions is not cut")
        # a tensor of more than two dimensions is a batch of matrices over its last two (optimizer.py:2203-2207):
        # rows counts the rows of all of them, mat_rows those of one, the column vectors hold batch * cols values
        self.cols = np.array([p.shape[-1] for p in self.params], dtype=np.int64)
        self.rows = np.array([p.numel() // p.shape[-1] for p in self.params], dtype=np.int64)
        self.mat_rows = np.array([p.shape[-2] for p in self.params], dtype=np.int64)
        self.batch = self.rows // self.mat_rows
        self.full_rows = np.array([(pc.full_rows or r) if pc is not None else r
                                   for r, pc in zip(self.rows.tolist(), self.pieces)], dtype=np.int64)
        self.row0 = np.array([pc.row0 if pc is not None else 0 for pc in self.pieces], dtype=np.int64)
        self.numel = self.rows * self.cols
        self.full_numel = self.full_rows * self.cols
        self.total_numel = int(self.numel.sum())
        # (batches of matrices take the general kernels; the optimizer keeps them in plans of their own)
        self.cfg.aligned8 = int(bool((self.cols % 8 == 0).all()) and not bool((self.batch > 1).any()))
        lib = N.lib()
        m_quant = m_fmt not in (None, "fp32")
        self.chunk = lib.af8_factored_chunk(self.cfg.m_block if m_quant else 0)
        self.tile = (lib.af8_factored_tile_rows(), lib.af8_factored_tile_cols())
        self.nchunks = (self.numel + self.chunk - 1) // self.chunk
        self.first_chunk = np.concatenate([[0], np.cumsum(self.nchunks)[:-1]]).astype(np.int64)
        self.total_chunks = int(self.nchunks.sum())
        # row sums (of the whole tensor's rows) then column sums of every tensor, each vector on a 16-byte boundary
        self._vec_len = ((self.full_rows + 3) // 4 * 4) + ((self.batch * self.cols + 3) // 4 * 4)
        rc = int(self._vec_len.sum())
        self.d_sums = torch.zeros(rc, dtype=torch.float64, device=self.device)
        self.d_inv = torch.empty(rc * (2 if self.came else 1), dtype=torch.float32, device=self.device)
        # one table for the passes over the elements (the entries as they are) and, when an entry holds
        # only some rows of its tensor, two for the row / column states (whole tensors; sums from the slots)
        self.n_tables = 3 if self.cut else 1
        tb = n * N.FACTORED_TENSOR.itemsize
        self.d_tables = torch.empty(self.n_tables * tb, dtype=torch.uint8, device=self.device)
        self.d_table = self.d_tables[:tb]
        self.d_dyn = torch.zeros(n * N.DYN_SCALARS.itemsize, dtype=torch.uint8, device=self.device)
        self.d_norm = torch.empty(n * N.NORM_TENSOR.itemsize, dtype=torch.uint8, device=self.device)
        self.d_sumsq = torch.empty(self.total_chunks, dtype=torch.float64, device=self.device)
        self.h_table = _PinnedRing(self.n_tables * tb)
        self.h_norm = _PinnedRing(n * N.NORM_TENSOR.itemsize)
        self.h_scale = self.d_scale = self.d_chunks = None
        self.h_lag = self.d_lag = None
        self.v_fmts, self.c_fmts = list(v_fmts), list(c_fmts)
        self._static = None
        self._ptr_sig = None
        self._alpha_on_device = False

    def _pointer_signature(self):
        return [p.data_ptr() for p in self.params]

    @staticmethod
    def _running(counts):
        return np.concatenate([[0], np.cumsum(counts)[:-1]]).astype(np.int64)

    def _static_fields(self):
        """-> the static part of the tables, shape (n_tables, n): [0] the entries as they are; with cut
        entries [1] / [2] describe the whole tensors for the second-moment / confidence state passes."""
        n = self.n
        t = np.zeros((self.n_tables, n), dtype=N.FACTORED_TENSOR)
        off = 0
        sums, inv = self.d_sums.data_ptr(), self.d_inv.data_ptr()
        half = int(self._vec_len.sum())
        tr, tc = self.tile
        for i, (p, st) in enumerate(zip(self.params, self.states)):
            C = int(self.cols[i])
            Rp = (int(self.full_rows[i]) + 3) // 4 * 4
            r0 = int(self.row0[i])
            e = t[0]
            e["param"][i] = p.data_ptr()
            e["m_q"][i] = _ptr(st.get("m_q"))
            e["m_scale"][i] = _ptr(st.get("m_scale"))
            e["m_f32"][i] = _ptr(st.get("m"))
            pc = self.pieces[i]
            if pc is not None and pc.copy is not None:
                if pc.copy.numel() != p.numel() or pc.copy.dtype != torch.bfloat16:
                    raise RuntimeError("the compute copy of a parameter must be a bf16 tensor of its size")
                e["param_copy"][i] = pc.copy.data_ptr()
            block = st.get("block_size", 2048)
            _small_state_fields(e["row_var"][i:i + 1], st, "row_var", self.v_fmts[i], block)
            _small_state_fields(e["col_var"][i:i + 1], st, "col_var", self.v_fmts[i], block)
            if self.came:
                _small_state_fields(e["conf_row"][i:i + 1], st, "conf_row", self.c_fmts[i], block)
                _small_state_fields(e["conf_col"][i:i + 1], st, "conf_col", self.c_fmts[i], block)
            for k in range(1, self.n_tables):
                t[k][i] = e[i]
            # the entry's own rows inside the whole tensor's vectors
            e["row_sum"][i] = sums + 8 * (off + r0)
            e["col_sum"][i] = sums + 8 * (off + Rp)
            e["inv_row"][i] = inv + 4 * (off + r0)
            e["inv_col"][i] = inv + 4 * (off + Rp)
            if self.came:
                e["inv_row_conf"][i] = inv + 4 * (half + off + r0)
                e["inv_col_conf"][i] = inv + 4 * (half + off + Rp)
            for k in range(1, self.n_tables):
                f = t[k]
                for name in ("inv_col", "inv_col_conf", "col_sum"):
                    f[name][i] = e[name][i]
                f["row_sum"][i] = sums + 8 * off
                f["inv_row"][i] = inv + 4 * off
                if self.came:
                    f["inv_row_conf"][i] = inv + 4 * (half + off)
                if i in self.cut:               # whole sums: exchange 0 (second moment), exchange 2 (confidence)
                    base = pc.slots[0 if k == 1 else 2].data_ptr() if (k == 1 or self.came) else 0
                    if base:
                        f["row_sum"][i] = base + 8 * 8
                        f["col_sum"][i] = base + 8 * (8 + Rp)
            off += int(self._vec_len[i])
        sb = t[0]["row_var"]["block"].astype(np.int64)
        for k in range(self.n_tables):
            rows = self.rows if k == 0 else self.full_rows
            t[k]["rows"], t[k]["cols"] = rows, self.cols
            t[k]["batch_rows"] = np.where(self.batch > 1, self.mat_rows, 0)
            mat_rows = np.where(self.batch > 1, self.mat_rows, rows)
            t[k]["first_chunk"] = self._running((rows * self.cols + self.chunk - 1) // self.chunk)
            tiles = self.batch * ((mat_rows + tr - 1) // tr) * ((self.cols + tc - 1) // tc)
            t[k]["first_tile"] = self._running(tiles)
            if k == 0:
                self.cfg.total_tiles = int(tiles.sum())
                self.cfg.cols_mult256 = int(bool((self.cols % 256 == 0).all()))
            # units of the small-state launch: the quantisation blocks of the row state, then of the column state
            units = (rows + sb - 1) // sb + (self.batch * self.cols + sb - 1) // sb
            t[k]["first_small"] = self._running(units)
            if k == self.n_tables - 1:
                self.small_units = int(units.sum())
        self._sums_off = self._running(self._vec_len)
        return t

    def kernel_name(self, what):
        return "factored_" + what

    def _log(self, name, fn, stream):
        log = LAUNCH_LOG
        if log is None:
            fn()
            return
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        fn()
        e1.record(stream)
        log.append((self.kernel_name(name), self.total_numel, e0, e1))

    def _table_ptr(self, k):
        return self.d_tables.data_ptr() + k * self.n * N.FACTORED_TENSOR.itemsize

    def _stats(self, mode, host_buf, stream, x=None):
        self.cfg.mode = mode
        lib = N.lib()
        if mode == N.FSTAT_RESIDUAL:
            # room for two tensor maps (128 bytes each) per entry: with them the library brings the rows in as boxes
            if getattr(self, "h_maps", None) is None:
                self.h_maps = _PinnedRing(self.n * 256)
                self.d_maps = torch.empty(self.n * 256, dtype=torch.uint8, device=self.device)
            hm = self.h_maps.next()
            self._log("stats_residual", lambda: N.check(
                lib.af8_factored_stats_boxes(ctypes.byref(self.cfg), self.d_table.data_ptr(), host_buf.data_ptr(), self.n,
                                             self.d_dyn.data_ptr(), hm.data_ptr(), self.d_maps.data_ptr(), stream.cuda_stream),
                "af8_factored_stats_boxes"), stream)
            self.h_maps.mark(stream)
        else:
            self._log("stats_gradsq", lambda: N.check(
                lib.af8_factored_stats(ctypes.byref(self.cfg), self.d_table.data_ptr(), host_buf.data_ptr(), self.n,
                                       self.d_dyn.data_ptr(), stream.cuda_stream), "af8_factored_stats"), stream)
        if x is not None:
            for i in self.cut:                  # the entry's rows and its column partial sums join the whole tensor's
                a, ln = int(self._sums_off[i]), int(self._vec_len[i])
                self.pieces[i].slots[x][8:8 + ln].add_(self.d_sums[a:a + ln])

    def _small(self, conf, stream):
        lib = N.lib()
        table = self._table_ptr((2 if conf else 1) if self.cut else 0)
        self._log("small_conf" if conf else "small_var", lambda: N.check(
            lib.af8_factored_small(ctypes.byref(self.cfg), table, self.n, int(conf), self.small_units,
                                   stream.cuda_stream), "af8_factored_small"), stream)

    def _update(self, mode, use_dyn, stream, x=None):
        self.cfg.mode = mode
        lib = N.lib()
        name = {N.FUPD_SUMSQ_U: "sumsq_u", N.FUPD_SUMSQ: "sumsq", N.FUPD_APPLY: "apply", N.FUPD_LAG: "lag"}[mode]
        self._log(name, lambda: N.check(
            lib.af8_factored_update(ctypes.byref(self.cfg), self.d_table.data_ptr(), self.n, self.total_chunks,
                                    self.d_dyn.data_ptr() if use_dyn else None, self.d_sumsq.data_ptr(),
                                    stream.cuda_stream), "af8_factored_update"), stream)
        if x is not None:
            for i in self.cut:
                a = int(self.first_chunk[i])
                _add_to_slot(self.pieces[i].slots[x], 1, self.d_sumsq[a:a + int(self.nchunks[i])])

    def _finalize(self, table, pre_div_mode, d, fira, fira_margin, stream, x=None):
        buf = self.h_norm.next()
        nt = buf.numpy()[: self.n * N.NORM_TENSOR.itemsize].view(N.NORM_TENSOR)
        nt["first_block"] = self.first_chunk
        nt["n_blocks"] = self.nchunks
        if x is not None:
            for i in self.cut:
                nt["n_blocks"][i] = -1
                nt["first_block"][i] = self.pieces[i].slots[x].data_ptr() + 8
        nt["pre_div_mode"] = pre_div_mode
        nt["partials_f64"] = 1
        nt["alpha"] = table["alpha"]
        if self._alpha_on_device:
            nt["alpha_dev"] = (self.d_table.data_ptr() + np.arange(self.n, dtype=np.uint64) * np.uint64(N.FACTORED_TENSOR.itemsize)
                               + np.uint64(N.FACTORED_TENSOR.fields["alpha"][1]))
        else:
            nt["alpha_dev"] = 0
        sqrt_n = np.sqrt(self.full_numel.astype(np.float64))
        nt["sqrt_n"] = sqrt_n.astype(np.float32)
        nt["d"] = np.float32(d)
        nt["clip_div"] = (sqrt_n * d).astype(np.float32) if (d > 0 and pre_div_mode == 0) else np.float32(0.0)
        nt["fira_margin1"] = np.float32(1.0 + fira_margin)
        if fira and pre_div_mode != 1:
            nt["fira_prev"], nt["fira_has_prev"] = fira_state_pointers(self)
        else:
            nt["fira_prev"] = 0
            nt["fira_has_prev"] = 0
        self.d_norm.copy_(buf[: self.d_norm.numel()], non_blocking=True)
        self.h_norm.mark(stream)
        N.check(N.lib().af8_norm_finalize(self.d_norm.data_ptr(), self.n, self.d_sumsq.data_ptr(),
                                          self.d_dyn.data_ptr(), stream.cuda_stream), "af8_norm_finalize")

    def run(self, grads, scalars, d=0.0, fira=False, fira_margin=0.01, scale=None, stream=None, lag=False):
        """One optimizer step for every tensor of the plan, start to end."""
        for _ in self.stages(grads, scalars, d=d, fira=fira, fira_margin=fira_margin, scale=scale, stream=stream, lag=lag):
            pass

    def stages(self, grads, scalars, d=0.0, fira=False, fira_margin=0.01, scale=None, stream=None, lag=False):
        """The step as a generator (optimizer.py:2202-2552) that yields at its factored_exchanges(...)
        exchange points, like FullrankPlan.stages; the last segment writes the parameters."""
        stream = stream or torch.cuda.current_stream(self.device)
        sig = self._pointer_signature()
        if self._static is None or sig != self._ptr_sig:
            self._static = self._static_fields()
            self._ptr_sig = sig
        buf = self.h_table.next()
        tables = buf.numpy()[: self.n_tables * self.n * N.FACTORED_TENSOR.itemsize].view(N.FACTORED_TENSOR).reshape(self.n_tables, self.n)
        tables[:] = self._static
        table = tables[0]
        table["grad"] = [g.data_ptr() for g in grads]
        for k in ("decay", "alpha", "v_w", "m_w", "c_w", "eps1", "eps_came"):
            table[k] = scalars[k]
        table["sr_base"] = scalars.get("sr_base", 0)
        for k in range(1, self.n_tables):
            for name in ("grad", "decay", "alpha", "v_w", "m_w", "c_w", "eps1", "eps_came"):
                tables[k][name] = table[name]
        lib = N.lib()
        for k in range(self.n_tables):
            N.check(lib.af8_factored_upload(ctypes.byref(self.cfg), buf.data_ptr() + k * self.n * N.FACTORED_TENSOR.itemsize,
                                            self._table_ptr(k), self.n, stream.cuda_stream), "af8_factored_upload")
        self.h_table.mark(stream)
        self._alpha_on_device = scale is not None
        need_stat = fira or d > 0
        if self.cut and not self.came and need_stat and lag:
            raise RuntimeError("lag_norm needs whole tensors: a tensor that is split over launch tables cannot lag")
        if scale is not None:
            self._param_scale(scale, stream, 0)
        self._stats(N.FSTAT_GRADSQ, buf, stream, 0)
        yield
        if scale is not None:
            self._param_finish(stream)
        self._small(False, stream)
        if self.came:
            # clip of U (optimizer.py:826-828); d == 0 means no clip: an infinite threshold gives divisor 1
            self._update(N.FUPD_SUMSQ_U, False, stream, 1)
            yield
            self._finalize(table, 1, d if d > 0 else float("inf"), False, fira_margin, stream, 1)
            self._stats(N.FSTAT_RESIDUAL, buf, stream, 2)
            yield
            self._small(True, stream)
            if fira:                                    # the final update is applied with d = 0 (optimizer.py:953)
                self._update(N.FUPD_SUMSQ, True, stream, 3)
                yield
                self._finalize(table, 2, 0.0, True, fira_margin, stream, 3)
            self._update(N.FUPD_APPLY, True, stream)
        elif need_stat and lag:
            # lag_norm=True: one pass with the previous step's norm (optimizer.py:1056-1071)
            if self.h_lag is None:
                self.h_lag = _PinnedRing(self.n * N.LAG_TENSOR.itemsize)
                self.d_lag = torch.empty(self.n * N.LAG_TENSOR.itemsize, dtype=torch.uint8, device=self.device)
            alpha_dev = 0
            if self._alpha_on_device:
                alpha_dev = (self.d_table.data_ptr() + np.arange(self.n, dtype=np.uint64) * np.uint64(N.FACTORED_TENSOR.itemsize)
                             + np.uint64(N.FACTORED_TENSOR.fields["alpha"][1]))
            lag_table(self.h_lag, self.d_lag, self.states, self.device, self.first_chunk, self.nchunks, self.full_numel,
                      table["alpha"], alpha_dev, d, fira, fira_margin, True, stream)
            N.check(lib.af8_lag_scalars(self.d_lag.data_ptr(), self.n, 0, None, self.d_dyn.data_ptr(), stream.cuda_stream),
                    "af8_lag_scalars")
            self._update(N.FUPD_LAG, True, stream)
            N.check(lib.af8_lag_scalars(self.d_lag.data_ptr(), self.n, 1, self.d_sumsq.data_ptr(), self.d_dyn.data_ptr(),
                                        stream.cuda_stream), "af8_lag_scalars")
        elif need_stat:
            self._update(N.FUPD_SUMSQ, False, stream, 1)
            yield
            self._finalize(table, 0, d, fira, fira_margin, stream, 1)
            self._update(N.FUPD_APPLY, True, stream)
        else:
            self._update(N.FUPD_APPLY, False, stream)

    def _param_scale(self, scale, stream, x=None):
        chunk = N.lib().af8_scale_chunk()
        nchunks = (self.numel + chunk - 1) // chunk
        if self.h_scale is None:
            self.h_scale = _PinnedRing(self.n * N.SCALE_TENSOR.itemsize)
            self.d_scale = torch.empty(self.n * N.SCALE_TENSOR.itemsize, dtype=torch.uint8, device=self.device)
            self.d_chunks = torch.empty(int(nchunks.sum()), dtype=torch.float32, device=self.device)
        hb = self.h_scale.next()
        t = hb.numpy()[: self.n * N.SCALE_TENSOR.itemsize].view(N.SCALE_TENSOR)
        fill_scale_table(t, self.params, self.numel, self.full_numel, nchunks, self.cfg.param_dtype, scale)
        if x is not None:
            for i in self.cut:
                t["total"][i] = self.pieces[i].slots[x].data_ptr()
        self._log("param_scale", lambda: N.check(N.lib().af8_param_sumsq(
            hb.data_ptr(), self.d_scale.data_ptr(), self.n, self.d_chunks.data_ptr(), stream.cuda_stream), "af8_param_sumsq"),
            stream)
        self.h_scale.mark(stream)
        if x is not None:
            first = t["first_chunk"]
            for i in self.cut:
                _add_to_slot(self.pieces[i].slots[x], 0, self.d_chunks[int(first[i]):int(first[i]) + int(nchunks[i])])

    def _param_finish(self, stream):
        N.check(N.lib().af8_param_scale_finish(
            self.d_scale.data_ptr(), self.n, self.d_chunks.data_ptr(), self.d_table.data_ptr(),
            N.FACTORED_TENSOR.itemsize, N.FACTORED_TENSOR.fields["alpha"][1], N.FACTORED_TENSOR.fields["decay"][1],
            stream.cuda_stream), "af8_param_scale_finish")

    def norms(self):
        dyn = self.d_dyn.cpu().numpy().view(N.DYN_SCALARS)
        return dyn["norm"].copy()


# True: APOLLO projections as correctly rounded dot products (binary64 accumulation, SIMT);
# False: bf16 gradients go through the tensor cores with a three-plane split of the projection
EXACT_PROJECTION = False


class ApolloPlan:
    """APOLLO tensors of one parameter group (optimizer.py:2587-3084): per-tensor
    projection, one batched low-rank state update (the full-rank kernel run on the
    projected gradients), per-tensor scaling and write-back."""

    def __init__(self, device, grad_dtype, v_fmt, m_fmt, block, m_block, negate, params, states, rank, copies=None,
                 rule=None, c_fmt="fp32"):
        """copies: optional list with a bf16 tensor (or None) per parameter that receives the updated
        parameter rounded to nearest (the compute copy of a mixed-precision run).
        rule: None for the plain Adam rule over the projected gradient, or dict(factorize=, came=) for
        apollo_factorize and / or CAME (optimizer.py:2688-2760, 2801-2903); c_fmt: format of their
        confidence / instability states."""
        self.device = torch.device(device)
        self.params, self.states = list(params), list(states)
        self.n = len(self.params)
        self.copies = list(copies) if copies is not None else [None] * self.n
        self.grad_dtype = _GRAD_DT[grad_dtype]
        self.v_fmt, self.m_fmt, self.block, self.m_block = v_fmt, m_fmt, int(block), int(m_block) if m_block else 0
        self.negate = int(bool(negate))
        self.rank = int(rank)
        self.rule, self.c_fmt = rule, c_fmt
        for p in self.params:
            if p.dtype not in _GRAD_DT or p.dtype != self.params[0].dtype or not p.is_contiguous() or p.dim() != 2:
                raise RuntimeError("the APOLLO kernels update contiguous 2-D fp32, bf16 or fp16 parameters, one dtype per group")
        self.param_dtype = _GRAD_DT[self.params[0].dtype]
        self.rows = [int(p.shape[0]) for p in self.params]
        self.cols = [int(p.shape[1]) for p in self.params]
        self.nch = [max(r, c) for r, c in zip(self.rows, self.cols)]
        self.nl = [n * self.rank for n in self.nch]
        self.total_numel = int(sum(r * c for r, c in zip(self.rows, self.cols)))
        dev = self.device
        self.g_low = [torch.empty(n, dtype=torch.float32, device=dev) for n in self.nl]
        # update_low of every tensor in one buffer (cleared with one memset per step), 512-byte aligned slices
        offs = np.concatenate([[0], np.cumsum([(n + 127) // 128 * 128 for n in self.nl])]).astype(np.int64)
        self.upd_all = torch.zeros(int(offs[-1]), dtype=torch.float32, device=dev)
        self.upd = [self.upd_all[int(offs[i]):int(offs[i]) + self.nl[i]] for i in range(self.n)]
        self.chan_g2 = [torch.empty(n, dtype=torch.float64, device=dev) for n in self.nch]
        # tensor-core projection: per-tensor workspaces (flag + bf16 planes of the projection)
        # cut from one buffer, and the task table of the multi-tensor launch
        lib = N.lib()
        need = [(int(lib.af8_apollo_project_workspace(r, c, self.rank)) + 255) // 256 * 256
                for r, c in zip(self.rows, self.cols)]
        self.ws_bytes = need
        self.workspace = torch.empty(sum(need) + 256, dtype=torch.uint8, device=dev)
        base = (self.workspace.data_ptr() + 255) // 256 * 256
        self.ws_ptr = [base + sum(need[:i]) for i in range(self.n)]
        task_bytes = int(lib.af8_apollo_project_task_bytes()) * self.n
        self.h_tasks = _PinnedRing(task_bytes)
        self.d_tasks = torch.empty(task_bytes, dtype=torch.uint8, device=dev)
        self.descs = np.zeros(self.n, dtype=N.APOLLO_PROJ_DESC)
        # room for transposed gradients of left-case tensors (rows < cols): the largest one, or
        # 256 MB when several fit, so that they reach the tcgen05 kernel a few at a time
        left = [r * c * 2 for r, c in zip(self.rows, self.cols) if r < c]
        self.t_bytes = 0 if (not left or grad_dtype != torch.bfloat16) else (max(max(left), min(sum(left), 256 << 20)) + 255) // 256 * 256 + 256 * len(left)
        self.t_scratch = torch.empty(self.t_bytes + 256, dtype=torch.uint8, device=dev) if self.t_bytes else None
        self.t_ptr = (self.t_scratch.data_ptr() + 255) // 256 * 256 if self.t_bytes else 0
        self.sf = [torch.empty(n, dtype=torch.float32, device=dev) for n in self.nch]
        self.sums = torch.zeros(3 * self.n, dtype=torch.float64, device=dev)
        self.out = torch.zeros(4 * self.n, dtype=torch.float32, device=dev)
        self._low_plans = {}
        self._plane_version = [None] * self.n
        if rule is not None:          # one work area, sized for the largest tensor (stream order makes its reuse safe)
            shapes = [((r, self.rank) if r >= c else (self.rank, c)) for r, c in zip(self.rows, self.cols)]
            self.low_shapes = shapes
            self.rule_bytes = max(int(lib.af8_apollo_rule_workspace(a, b)) for a, b in shapes)
            self.rule_work = torch.empty(self.rule_bytes + 256, dtype=torch.uint8, device=dev)
            self.rule_ptr = (self.rule_work.data_ptr() + 255) // 256 * 256
        # table of the batched scaling-factor / scalar-chain launches (static part)
        fs = np.zeros(self.n, dtype=N.APOLLO_FINISH_TENSOR)
        units = [(n + 7) // 8 for n in self.nch]
        for i in range(self.n):
            fs["upd"][i], fs["g_low"][i], fs["chan_g2"][i] = self.upd[i].data_ptr(), self.g_low[i].data_ptr(), self.chan_g2[i].data_ptr()
            fs["sf"][i], fs["sums"][i], fs["out"][i] = self.sf[i].data_ptr(), self.sums.data_ptr() + 24 * i, self.out.data_ptr() + 16 * i
            fs["rows"][i], fs["cols"][i], fs["rank"][i] = self.rows[i], self.cols[i], self.rank
            fs["first_unit"][i] = sum(units[:i])
        self._finish_static = fs
        self.finish_units = int(sum(units))
        # table of the batched write-back (static part): 2048-element chunks numbered across the tensors
        ap = np.zeros(self.n, dtype=N.APOLLO_APPLY_TENSOR)
        chunks = [(r * c + 2047) // 2048 for r, c in zip(self.rows, self.cols)]
        for i in range(self.n):
            ap["sf"][i], ap["scalars"][i] = self.sf[i].data_ptr(), self.out.data_ptr() + 16 * i
            ap["param_copy"][i] = self.copies[i].data_ptr() if self.copies[i] is not None else 0
            ap["rows"][i], ap["cols"][i], ap["first_chunk"][i] = self.rows[i], self.cols[i], sum(chunks[:i])
        self._apply_static = ap
        self.apply_chunks = int(sum(chunks))
        self.h_apply = _PinnedRing(self.n * N.APOLLO_APPLY_TENSOR.itemsize)
        self.d_apply = torch.empty(self.n * N.APOLLO_APPLY_TENSOR.itemsize, dtype=torch.uint8, device=dev)
        self.h_finish = _PinnedRing(self.n * N.APOLLO_FINISH_TENSOR.itemsize)
        self.d_finish = torch.empty(self.n * N.APOLLO_FINISH_TENSOR.itemsize, dtype=torch.uint8, device=dev)

    def _low_plan(self, idx):
        """Full-rank plan over the projected space for the tensors `idx` (they share the
        first-step status, which selects the min_log floor)."""
        key = tuple(idx)
        plan = self._low_plans.get(key)
        if plan is None:
            fake_states = []
            for i in idx:
                st = self.states[i]
                fs = {}
                for src, dst in (("v_low_q", "variance_q"), ("v_low_scale", "variance_scale"),
                                 ("v_low_min_log", "variance_min_log"), ("v_low", "variance"),
                                 ("m_low_q", "m_q"), ("m_low_scale", "m_scale"), ("m_low", "m")):
                    if st.get(src) is not None:
                        fs[dst] = st[src]
                fake_states.append(fs)
            plan = FullrankPlan(self.device, torch.float32, self.v_fmt, self.m_fmt, self.block, self.m_block,
                                True, False, False, [self.upd[i] for i in idx], fake_states)
            self._low_plans[key] = plan
        return plan

    def _alpha_decay(self, scale, stream):
        """scale_parameter=True: alpha_t = max(RMS(p), eps2) * rho and the decay factor of every tensor, computed on
        the device from the parameters as they are before the update (optimizer.py:850-853, 3007-3013), into
        self.alpha_decay ([n][2] floats) for the finaliser and the write-back."""
        lib = N.lib()
        chunk = lib.af8_scale_chunk()
        numel = np.array([r * c for r, c in zip(self.rows, self.cols)], dtype=np.int64)
        nchunks = (numel + chunk - 1) // chunk
        if getattr(self, "alpha_decay", None) is None:
            self.alpha_decay = torch.zeros(self.n, 2, dtype=torch.float32, device=self.device)
            self.h_scale = _PinnedRing(self.n * N.SCALE_TENSOR.itemsize)
            self.d_scale = torch.empty(self.n * N.SCALE_TENSOR.itemsize, dtype=torch.uint8, device=self.device)
            self.d_chunks = torch.empty(int(nchunks.sum()), dtype=torch.float32, device=self.device)
        hb = self.h_scale.next()
        t = hb.numpy()[: self.n * N.SCALE_TENSOR.itemsize].view(N.SCALE_TENSOR)
        fill_scale_table(t, self.params, numel, numel, nchunks, self.param_dtype, scale)
        N.check(lib.af8_param_scale(hb.data_ptr(), self.d_scale.data_ptr(), self.n, self.d_chunks.data_ptr(),
                                    self.alpha_decay.data_ptr(), 8, 0, 4, stream.cuda_stream), "af8_param_scale")
        self.h_scale.mark(stream)

    def run(self, grads, pts, per_tensor, lowrank_scalars, first_flags, floor_later, stream=None, params=None, scale=None,
            versions=None):
        """per_tensor: list of dicts with the ApolloScalarsIn fields, decay, has_decay and the
        device scalar `fira_prev` (or None).  lowrank_scalars: v_w, m_w, apollo_eps.
        params: this step's 2-D views of the parameters (their storage may have been replaced).
        scale: per-tensor inputs of af8_param_scale when the step size follows the parameters' RMS
        (scale_parameter=True); alpha and the decay factor then come from the device.
        versions: one hashable per tensor that changes whenever its projection matrix does; while it stays
        the same the bf16 planes of the matrix are kept in the workspace instead of being rebuilt."""
        stream = stream or torch.cuda.current_stream(self.device)
        if params is not None:
            self.params = list(params)
        lib = N.lib()
        s = stream.cuda_stream
        if scale is not None:
            self._alpha_decay(scale, stream)
        log = LAUNCH_LOG
        ev = None
        if log is not None:
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            ev[0].record(stream)
        d = self.descs
        for i in range(self.n):
            d["grad"][i], d["pt"][i] = grads[i].data_ptr(), pts[i].data_ptr()
            d["g_low"][i], d["chan_g2"][i] = self.g_low[i].data_ptr(), self.chan_g2[i].data_ptr()
            d["workspace"][i] = 0 if EXACT_PROJECTION else self.ws_ptr[i]
            d["workspace_bytes"][i] = 0 if EXACT_PROJECTION else self.ws_bytes[i]
            d["rows"][i], d["cols"][i], d["rank"][i], d["negate"][i] = self.rows[i], self.cols[i], self.rank, self.negate
            ver = (versions[i], pts[i].data_ptr()) if versions is not None and not EXACT_PROJECTION else None
            d["planes_valid"][i] = int(ver is not None and self._plane_version[i] == ver)
            self._plane_version[i] = ver
        h_tasks = self.h_tasks.next()
        N.check(lib.af8_apollo_project_batch(d.ctypes.data, self.n, self.grad_dtype, h_tasks.data_ptr(),
                                             self.d_tasks.data_ptr(), self.t_ptr, self.t_bytes, s), "af8_apollo_project_batch")
        self.h_tasks.mark(stream)
        if log is not None:
            ev[1].record(stream)
        self.upd_all.zero_()        # the low-rank step writes p*0 + u into it; stale NaNs must not survive
        if self.rule is not None:
            self._run_rule(lowrank_scalars, first_flags, floor_later, s)
        for first in ((True, False) if self.rule is None else ()):
            idx = [i for i in range(self.n) if bool(first_flags[i]) == first]
            if not idx:
                continue
            plan = self._low_plan(idx)
            plan.cfg.v_floor = -126.0 if first else float(floor_later)
            k = len(idx)
            cols = dict(decay=np.zeros(k, np.float32), alpha=np.full(k, -1.0, np.float32),
                        v_w=np.full(k, lowrank_scalars["v_w"], np.float32),
                        v_keep=np.full(k, -1.0 if self.v_fmt == "fp32" else lowrank_scalars["v_keep"], np.float32),   # fp32 V: lerp_
                        v_eps_add=np.zeros(k, np.float32),
                        m_w=np.full(k, lowrank_scalars["m_w"], np.float32), eps_gradsq=np.zeros(k, np.float32),
                        eps_denom=np.full(k, lowrank_scalars["apollo_eps"], np.float32),
                        eps_sq=np.full(k, 1.17549435e-38, np.float32))
            plan.run([self.g_low[i] for i in idx], cols, d=0.0, fira=False)
        if log is not None:
            ev[2].record(stream)
        sins = []
        for i in range(self.n):
            t = per_tensor[i]
            sin = N.ApolloScalarsIn()
            for k in ("alpha", "bc", "d", "clip_div", "fira_margin1", "sqrt_scale"):
                setattr(sin, k, float(t[k]))
            for k in ("bc_mode", "fira", "fira_has_prev", "scale_tensor", "scale_front"):
                setattr(sin, k, int(t[k]))
            sins.append(sin)
        if any(sin.scale_tensor for sin in sins):
            for i, sin in enumerate(sins):          # tensor-wise scaling: one tensor at a time
                prev = per_tensor[i].get("fira_prev")
                N.check(lib.af8_apollo_scales(self.upd[i].data_ptr(), self.g_low[i].data_ptr(), self.chan_g2[i].data_ptr(),
                                              self.rows[i], self.cols[i], self.rank, ctypes.byref(sin), self.sf[i].data_ptr(),
                                              self.sums.data_ptr() + 24 * i, prev.data_ptr() if prev is not None else None,
                                              self.out.data_ptr() + 16 * i,
                                              self.alpha_decay.data_ptr() + 8 * i if scale is not None else None, s), "af8_apollo_scales")
        else:                                       # channel-wise scaling: all tensors in two launches
            h = self.h_finish.next()
            ft = np.frombuffer(h.numpy(), dtype=N.APOLLO_FINISH_TENSOR, count=self.n)
            ft[:] = self._finish_static
            for i, sin in enumerate(sins):
                prev = per_tensor[i].get("fira_prev")
                ft["fira_prev"][i] = prev.data_ptr() if prev is not None else 0
                ft["alpha_decay"][i] = self.alpha_decay.data_ptr() + 8 * i if scale is not None else 0
                for k in ("alpha", "bc", "d", "clip_div", "fira_margin1", "sqrt_scale", "bc_mode", "fira", "fira_has_prev",
                          "scale_tensor", "scale_front"):
                    ft[k][i] = getattr(sin, k)
            N.check(lib.af8_apollo_scales_batch(h.data_ptr(), self.d_finish.data_ptr(), self.n, self.finish_units, s),
                    "af8_apollo_scales_batch")
            self.h_finish.mark(stream)
        h = self.h_apply.next()                     # the write-back of all tensors: one launch
        at = np.frombuffer(h.numpy(), dtype=N.APOLLO_APPLY_TENSOR, count=self.n)
        at[:] = self._apply_static
        for i, sin in enumerate(sins):
            t = per_tensor[i]
            at["param"][i], at["grad"][i] = self.params[i].data_ptr(), grads[i].data_ptr()   # (this step's storage)
            at["sr_base"][i], at["stochastic_round"][i] = int(t.get("sr_base", 0)), int(t.get("sr", False))
            at["decay"][i], at["has_decay"][i] = float(t["decay"]), 2 if scale is not None else int(t["has_decay"])
            at["sqrt_scale"][i], at["scale_tensor"][i] = sin.sqrt_scale, sin.scale_tensor
            at["fira"][i], at["scale_front"][i] = sin.fira, sin.scale_front
        N.check(lib.af8_apollo_apply_batch(h.data_ptr(), self.d_apply.data_ptr(), self.n, self.apply_chunks, self.param_dtype,
                                           self.grad_dtype, self.negate, s), "af8_apollo_apply_batch")
        self.h_apply.mark(stream)
        if log is not None:
            ev[3].record(stream)
            log.append(("apollo_project", self.total_numel, ev[0], ev[1]))
            log.append(("apollo_scales_apply", self.total_numel, ev[2], ev[3]))

    def _run_rule(self, sc, first_flags, floor_later, s):
        """update_low of every tensor under apollo_factorize and / or CAME: one af8_apollo_rule_step each."""
        lib = N.lib()

        def ptr(t):
            return t.data_ptr() if t is not None else None

        def rule_state(st, prefix, n, fmt):
            rs = N.ApolloRuleState()
            rs.n, rs.fmt = n, N.V_FMT[fmt]
            if fmt == "fp32":
                rs.f32 = ptr(st[prefix])
            else:
                rs.q, rs.scale, rs.min_log = ptr(st[prefix + "_q"]), ptr(st[prefix + "_scale"]), ptr(st[prefix + "_min_log"])
            return rs

        for i in range(self.n):
            st = self.states[i]
            lr, lc = self.low_shapes[i]
            r = N.ApolloRule()
            r.g_low, r.upd, r.work, r.work_bytes = self.g_low[i].data_ptr(), self.upd[i].data_ptr(), self.rule_ptr, self.rule_bytes
            r.lr_rows, r.lr_cols = lr, lc
            r.factorize, r.came = int(self.rule["factorize"]), int(self.rule["came"])
            r.m_fmt, r.m_block, r.block = N.M_FMT[self.m_fmt], self.m_block, self.block
            r.first_factor = int(bool(first_flags[i]) and self.rule["factorize"])
            r.first_v = int(bool(first_flags[i]) and not self.rule["factorize"])
            for k in ("v_w", "v_keep", "m_w", "c_w", "eps_came", "eps_sq", "apollo_eps", "d"):
                setattr(r, k, float(sc[k]))
            r.v_floor_later = float(floor_later)
            if self.m_fmt is not None:
                if self.m_fmt == "fp32":
                    r.m_f32 = ptr(st["m_low"])
                else:
                    r.m_q, r.m_scale = ptr(st["m_low_q"]), ptr(st["m_low_scale"])
            if self.rule["factorize"]:
                r.row_var_low, r.col_var_low = ptr(st["row_var_low"]), ptr(st["col_var_low"])
                if self.rule["came"]:
                    r.conf_row = rule_state(st, "conf_row_low", lr, self.c_fmt)
                    r.conf_col = rule_state(st, "conf_col_low", lc, self.c_fmt)
            else:
                r.v = rule_state(st, "v_low", lr * lc, self.v_fmt)
                r.res = rule_state(st, "res_low", lr * lc, self.c_fmt)
            N.check(lib.af8_apollo_rule_step(ctypes.byref(r), s), "af8_apollo_rule_step")

    def norms(self):
        return self.out.cpu().numpy().reshape(self.n, 4)[:, 2].copy()
