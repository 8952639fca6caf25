"""`Adafactor8Bit`: the reference's optimizer class, served by libaf8.

The constructor signature, the argument checks, `param_groups`, the per-
parameter state keys / dtypes and the two extra `state_dict` entries are those
of the reference (adafactor8bit/optimizer.py:1313-1467), so code written for
the reference runs unchanged.  What differs is how a step executes: the
reference walks the parameters one by one and issues 1-8 kernels (or ~25 torch
ops) per tensor; here the parameters of a group are sorted into launch plans
and every plan runs one multi-tensor kernel per pass.

There is no PyTorch or CPU path in this class: parameters must live on a CUDA
device and libaf8.so must be loadable.  `use_cuda_kernel` is accepted for
compatibility and ignored.
"""
import logging
import math
from typing import Any, Dict, Iterable, Optional, Tuple, Union

import numpy as np
import torch
from torch import Tensor
from torch.optim import Optimizer

from . import _native as N
from ._engine import ApolloPlan, FactoredPlan, FullrankPlan, factored_exchanges, fullrank_exchanges, sr_base

_FULLRANK_COLS = ("decay", "alpha", "v_w", "v_keep", "v_eps_add", "m_w", "eps_gradsq", "eps_denom", "eps_sq")

__all__ = ["Adafactor8Bit"]

# Device on which APOLLO's random projections are drawn.  None follows the reference
# (the gradient's device, optimizer.py:139-149, so the values depend on the device type);
# "cpu" draws the CPU generator's values, which is what CPU-side checkers reproduce.
APOLLO_RNG_DEVICE = None

logger = logging.getLogger(__name__)

_FLOOR = 1.17549435e-38                                   # optimizer.py:23
_M_TYPES = ("uf4", "uf8", "d4", "d8", "fp32")              # optimizer.py:24
_V_TYPES = ("al8", "al16", "fp32")                         # optimizer.py:25
f32 = np.float32


def _pad_to(n, block):
    return (block - n % block) % block


def _new_al_state(state, prefix, shape, block, device, fmt):
    """Zero-initialised AL state (optimizer.py:389-401): codes 0, scale 1, min_log 0."""
    numel = int(math.prod(shape)) if not isinstance(shape, int) else shape
    if fmt == "fp32":
        state[prefix] = torch.zeros(shape, dtype=torch.float32, device=device)
        return
    pad = _pad_to(numel, block)
    nblocks = (numel + pad) // block
    state[prefix + "_q"] = torch.zeros(numel + pad, dtype=torch.uint8 if fmt == "al8" else torch.int16, device=device)
    state[prefix + "_scale"] = torch.ones(nblocks, dtype=torch.float32, device=device)
    state[prefix + "_min_log"] = torch.zeros(nblocks, dtype=torch.float32, device=device)
    state[prefix + "_shape"] = shape
    state[prefix + "_pad"] = pad


def _new_m_state(state, numel, m_block, fmt, device, shape, prefix="m"):
    """Zero momentum (optimizer.py:574-590): the code of 0.0 with scale 1."""
    if fmt == "fp32":
        state[prefix] = torch.zeros(shape, dtype=torch.float32, device=device)
    else:
        padded = ((numel + m_block - 1) // m_block) * m_block
        if fmt in ("uf4", "d4"):
            fill, count = (0x88 if fmt == "uf4" else 0x77), padded // 2
        else:
            fill, count = (128 if fmt == "uf8" else 127), padded
        state[prefix + "_q"] = torch.full((count,), fill, dtype=torch.uint8, device=device)
        state[prefix + "_scale"] = torch.ones(padded // m_block, dtype=torch.float32, device=device)
        state["m_block_size"] = m_block
    state["m_quant_type"] = fmt


class Adafactor8Bit(Optimizer):
    """Memory-efficient optimizer family (Adafactor, AdamW, RMSprop, CAME, APOLLO)
    over block-quantised states.  See the reference's class docstring
    (optimizer.py:1177-1311) for the meaning of every argument; names, defaults
    and validation are identical."""

    def __init__(
        self,
        params: Iterable[Union[Tensor, Dict[str, Any]]],
        lr: float = 1e-2,
        beta1: Optional[float] = None,
        beta2: Optional[float] = None,
        beta2_decay: Optional[float] = -0.8,
        beta3: Optional[float] = None,
        eps_came: float = 1e-16,
        eps: Tuple[Optional[float], float] = (1e-30, 1e-3),
        weight_decay: float = 0.0,
        d: float = 1.0,
        maximize: bool = False,
        relative_step: bool = True,
        scale_parameter: bool = True,
        factored: bool = True,
        quantize: bool = True,
        block_size: int = 2048,
        m_block_size: int = 256,
        m_quant_type: str = "uf8",
        v_quant_type: str = "al8",
        c_quant_type: Optional[str] = None,
        min_8bit_size: int = 4096,
        use_cuda_kernel: bool = True,
        stochastic_round_writeback: bool = False,
        apollo_rank: int = 0,
        apollo_update_proj_gap: int = 200,
        apollo_scale_type: str = "channel",
        apollo_scale: float = 1.0,
        apollo_scale_front: bool = False,
        apollo_eps: float = 1e-6,
        apollo_factorize: bool = False,
        apollo_cache_proj: bool = False,
        enable_fira_for_apollo: bool = True,
        scale_weight_decay: bool = True,
        enable_fira_for_adafactor: bool = False,
        fira_margin: float = 0.01,
        lag_norm: bool = False,
        momentum_only_1d: Optional[bool] = None,
        bias_correction: Optional[bool] = None,
        warmup_multiplier: float = 0.0,
    ):
        # argument checks, in the reference's order (optimizer.py:1362-1432)
        if lr < 0.0:
            raise ValueError(f"Invalid lr: {lr}, must be >= 0.0")
        if beta1 is not None and not (0.0 <= beta1 < 1.0):
            raise ValueError(f"Invalid beta1: {beta1}, must be in [0.0, 1.0)")
        if beta2_decay is not None and beta2_decay > 0.0:
            raise ValueError(f"Invalid beta2_decay: {beta2_decay}, must be <= 0.0")
        if beta2 is None and beta2_decay is None:
            if relative_step:
                raise ValueError("When `beta2` and `beta2_decay` are both None, `relative_step` must be False. "
                                 "Please set `relative_step=False` for standard SGD, or specify "
                                 "`beta2`/`beta2_decay` to use adaptive optimizers.")
            if apollo_rank > 0:
                raise ValueError("APOLLO requires a second-moment estimate (`beta2` or `beta2_decay`), "
                                 "but both are currently None.")
            if beta3 is not None:
                raise ValueError("CAME (`beta3`) requires both `beta1` and `beta2`, but `beta2` is currently None.")
        eps1, eps2 = eps
        if eps1 is None:
            eps1 = 1e-30
        if eps1 < 0.0:
            raise ValueError(f"Invalid eps1: {eps1}, must be >= 0.0")
        if eps2 < 0.0:
            raise ValueError(f"Invalid eps2: {eps2}, must be >= 0.0")
        if d < 0.0:
            raise ValueError(f"Invalid d: {d}, must be >= 0.0. d=0 disables RMS clipping.")
        if weight_decay < 0.0:
            raise ValueError(f"Invalid weight_decay: {weight_decay}, must be >= 0.0")
        if beta2 is not None and not (0.0 <= beta2 < 1.0):
            raise ValueError(f"Invalid beta2: {beta2}, must be in [0.0, 1.0)")
        if quantize and (block_size < 128 or block_size % 128 != 0):
            raise ValueError(f"block_size must be >= 128 and a multiple of 128, but got {block_size}.")
        if m_block_size < 32 or m_block_size % 4 != 0:
            raise ValueError(f"m_block_size must be a multiple of 4 and >= 32, but got {m_block_size}.")
        if m_quant_type not in _M_TYPES:
            raise ValueError(f"m_quant_type must be one of {_M_TYPES}, got '{m_quant_type}'.")
        if v_quant_type not in _V_TYPES:
            raise ValueError(f"v_quant_type must be one of {_V_TYPES}, got '{v_quant_type}'.")
        if c_quant_type is not None and c_quant_type not in _V_TYPES:
            raise ValueError(f"c_quant_type must be one of {_V_TYPES} or None, got '{c_quant_type}'.")
        if quantize and beta1 is not None and m_quant_type != "fp32" and block_size % m_block_size != 0:
            raise ValueError("For the fused 1D kernel, block_size must be a multiple of m_block_size "
                             f"(got block_size={block_size}, m_block_size={m_block_size}).")
        if apollo_rank > 0 and apollo_scale_type not in ("channel", "tensor"):
            raise ValueError(f"apollo_scale_type must be 'channel' or 'tensor', got {apollo_scale_type}.")
        if apollo_scale < 0.0:
            raise ValueError(f"Invalid apollo_scale: {apollo_scale}, must be >= 0.0")
        if fira_margin < 0.0:
            raise ValueError(f"Invalid fira_margin: {fira_margin}, must be >= 0.0")
        if beta3 is not None:
            if not (0.0 <= beta3 < 1.0):
                raise ValueError(f"Invalid beta3: {beta3}, must be in [0.0, 1.0)")
            if beta1 is None:
                raise ValueError("CAME (beta3) strictly requires momentum (beta1) to compute update instability.")
            if apollo_rank == 0 and not factored:
                raise ValueError("CAME (beta3) requires factored=True (2D row/col factorization). "
                                 "It is not supported for 1D full-rank paths.")

        defaults = dict(
            lr=lr, beta1=beta1, beta2=beta2, beta2_decay=beta2_decay, beta3=beta3, eps_came=eps_came,
            eps=eps, weight_decay=weight_decay, d=d, maximize=maximize,
            relative_step=relative_step, scale_parameter=scale_parameter, factored=factored,
            quantize=quantize, block_size=block_size, m_block_size=m_block_size,
            m_quant_type=m_quant_type, v_quant_type=v_quant_type, c_quant_type=c_quant_type,
            min_8bit_size=min_8bit_size, use_cuda_kernel=use_cuda_kernel,
            stochastic_round_writeback=stochastic_round_writeback,
            apollo_rank=apollo_rank, apollo_update_proj_gap=apollo_update_proj_gap,
            apollo_scale_type=apollo_scale_type, apollo_scale=apollo_scale,
            apollo_scale_front=apollo_scale_front, apollo_eps=apollo_eps,
            apollo_factorize=apollo_factorize, apollo_cache_proj=apollo_cache_proj,
            enable_fira_for_apollo=enable_fira_for_apollo,
            scale_weight_decay=scale_weight_decay,
            enable_fira_for_adafactor=enable_fira_for_adafactor, fira_margin=fira_margin,
            lag_norm=lag_norm, momentum_only_1d=momentum_only_1d, bias_correction=bias_correction,
            warmup_multiplier=warmup_multiplier,
        )
        super().__init__(params, defaults)
        self._apollo_seed_counter = 1          # optimizer.py:1460-1461
        self._sr_seed_counter = 1
        self._sr_seed_map = None
        self._apollo_seed_map = None
        self._cfg_seen = {}       # id(param) -> option signature its state was last checked against
        self._plans = {}
        self._group_cache = {}    # group index -> how its parameters were sorted into launch groups at the last step
        self._after_group = None               # optional hook(gi, group), called when a group's launches are enqueued
        # Set by a sharding wrapper (zero.py): `_pieces` maps id(parameter) to the _engine.Piece that says which
        # part of which tensor the parameter is; `_shard` schedules the passes of all launch plans in
        # rounds with an exchange of partial sums between them (see _step_sharded).
        self._pieces = {}
        self._shard = None

    # ------------------------------------------------------------------
    # checkpointing (optimizer.py:1463-1553)
    # ------------------------------------------------------------------
    def state_dict(self):
        if torch.cuda.is_available() and any(p.is_cuda for g in self.param_groups for p in g["params"]):
            self.check_device()
        sd = super().state_dict()
        sd["_apollo_seed_counter"] = self._apollo_seed_counter
        sd["_sr_seed_counter"] = self._sr_seed_counter
        return sd

    def load_state_dict(self, state_dict):
        state_dict = dict(state_dict)
        self._cfg_seen.clear()       # loaded states are checked against the group options at the next step
        self._plans.clear()
        self._group_cache.clear()
        # APOLLO keeps its momentum in the projected space: full-size momentum left in an APOLLO state is
        # dropped before the base loader would move it to the device (optimizer.py:1472-1480)
        state_dict["state"] = {
            idx: ({k: v for k, v in st.items() if k not in ("m", "m_q", "m_scale")}
                  if isinstance(st, dict) and "apollo_seed" in st else st)
            for idx, st in state_dict.get("state", {}).items()}
        # counters a checkpoint does not carry start from 0 (optimizer.py:1502-1503)
        self._apollo_seed_counter = state_dict.pop("_apollo_seed_counter", 0)
        self._sr_seed_counter = state_dict.pop("_sr_seed_counter", 0)
        # groups saved without a stochastic-rounding policy keep the current one (optimizer.py:1505-1520)
        current_sr = [g.get("stochastic_round_writeback", False) for g in self.param_groups]
        sr_missing = [("stochastic_round_writeback" not in sg) if isinstance(sg, dict) else True
                      for sg in state_dict.get("param_groups", [])]
        # torch's loader casts floating-point state to the parameter's dtype and
        # moves everything to its device; remember the saved dtypes and restore
        # them afterwards (the reference does the same, optimizer.py:1482-1539)
        saved = {idx: {k: v.dtype for k, v in st.items() if isinstance(v, Tensor)}
                 for idx, st in state_dict["state"].items()}
        saved_vals = {idx: {k: v for k, v in st.items() if isinstance(v, Tensor)}
                      for idx, st in state_dict["state"].items()}
        # ... and it rebuilds every iterable value element by element, which turns the format
        # names (strings) and shapes into garbage: keep the saved non-tensor values as they are
        saved_plain = {idx: {k: v for k, v in st.items() if not isinstance(v, Tensor)}
                       for idx, st in state_dict["state"].items()}
        super().load_state_dict(state_dict)
        if len(self.param_groups) == len(sr_missing):
            for group, missing, policy in zip(self.param_groups, sr_missing, current_sr):
                if missing:
                    group["stochastic_round_writeback"] = policy
        idx_of = {}
        i = 0
        for g in self.param_groups:
            for p in g["params"]:
                idx_of[p] = i
                i += 1
        keys = list(saved.keys())
        for p, st in self.state.items():
            idx = idx_of.get(p)
            src = saved.get(idx, saved.get(str(idx)))
            if src is None:
                continue
            vals = saved_vals.get(idx, saved_vals.get(str(idx)))
            for k, dt in src.items():
                if k in st and isinstance(st[k], Tensor) and st[k].dtype != dt:
                    st[k] = vals[k].to(device=p.device, dtype=dt).clone()
            plain = saved_plain.get(idx, saved_plain.get(str(idx))) or {}
            for k, v in plain.items():
                st[k] = v
            if "step" in st and isinstance(st["step"], Tensor):
                st["step"] = int(st["step"].item())
        del keys
        self._plans.clear()

    def update_norms(self):
        """Norms of the updates measured by the last step's statistic passes, one
        per tensor of every launch plan (zeros where no norm was needed).  Reads
        them back from the device, so it synchronises."""
        out = [plan.norms() for plan in self._plans.values()]
        self.check_device()
        return np.concatenate(out) if out else np.zeros(0, dtype=np.float32)

    def check_device(self):
        """Raise if a kernel of this library gave up a bounded wait on any device this optimizer steps on
        (an asynchronous copy that never completed: the launch skipped its stores, so parameters and
        states of that step are incomplete).  Synchronises; called where the host synchronises anyway
        (update_norms, state_dict)."""
        devices = {p.device for g in self.param_groups for p in g["params"] if p.is_cuda}
        for dev in devices:
            with torch.cuda.device(dev):
                code = N.device_status(torch.cuda.current_stream(dev).cuda_stream)
            if code != 0:
                raise RuntimeError(f"libaf8 reported device error {code} on {dev}: a kernel gave up waiting for an "
                                   f"asynchronous copy; the step that ran then is incomplete")

    # ------------------------------------------------------------------
    # lazy state creation (first-step branch of _init_group, optimizer.py:1711-1773)
    # ------------------------------------------------------------------
    def _create_state(self, p, grad, group):
        state = self.state[p]
        numel = p.numel()
        piece = self._pieces.get(id(p))
        full_numel = piece.full_numel if piece is not None else numel      # the whole tensor decides the formats
        use_quant = group.get("quantize", True) and not (full_numel < group.get("min_8bit_size", 4096))
        block = group.get("block_size", 2048)
        m_block = group.get("m_block_size", 256)
        vqt = group.get("v_quant_type", "al8")
        cqt = group.get("c_quant_type") or vqt
        mqt = group.get("m_quant_type", "uf8")
        beta1, beta3 = group.get("beta1"), group.get("beta3")
        sgd = group.get("beta2") is None and group.get("beta2_decay") is None
        if "step" not in state:
            state["step"] = 0
        state["is_quantized"] = use_quant
        state["block_size"] = block
        state["v_quant_type"] = vqt
        state["c_quant_type"] = cqt
        dev = p.device
        v_fmt = vqt if use_quant else "fp32"
        c_fmt = cqt if use_quant else "fp32"
        m_fmt = mqt if use_quant else "fp32"
        if sgd:
            if beta1 is not None:
                _new_m_state(state, numel, m_block, m_fmt, dev, p.shape)
        elif group.get("apollo_rank", 0) > 0 and grad.dim() >= 2:
            seed = self._apollo_seed_map.get(id(p)) if self._apollo_seed_map is not None else None
            if seed is None:                                  # (a sharding wrapper presets the seeds of the unsharded run)
                seed = self._apollo_seed_counter
                self._apollo_seed_counter += 1
            gap = group.get("apollo_update_proj_gap", 200)
            state.update(apollo_seed=seed, apollo_rank=group["apollo_rank"],
                         apollo_factorize=group.get("apollo_factorize", False), beta3=beta3,
                         apollo_update_proj_gap=gap, last_proj_step=-gap,
                         apollo_proj_matrix_T=None, m_quant_type=mqt)
            for k in ("v_low_q", "v_low_scale", "v_low_min_log", "v_low_shape", "v_low_pad", "v_low"):
                state[k] = None
        elif grad.dim() >= 2 and group.get("factored", True):
            shape = grad.shape
            if piece is not None and piece.full_rows:          # some rows of a tensor: its row state covers all rows
                shape = (piece.full_rows, shape[-1])
            r_shape = list(shape[:-2]) + [shape[-2], 1]
            c_shape = list(shape[:-2]) + [1, shape[-1]]
            _new_al_state(state, "row_var", r_shape, block, dev, v_fmt)
            _new_al_state(state, "col_var", c_shape, block, dev, v_fmt)
            if beta1 is not None:
                _new_m_state(state, numel, m_block, m_fmt, dev, p.shape)
            if beta3 is not None:
                _new_al_state(state, "conf_row", r_shape, block, dev, c_fmt)
                _new_al_state(state, "conf_col", c_shape, block, dev, c_fmt)
        else:
            _new_al_state(state, "variance", grad.shape, block, dev, v_fmt)
            if beta1 is not None:
                _new_m_state(state, numel, m_block, m_fmt, dev, p.shape)
        return state

    # ------------------------------------------------------------------
    # state migration when a group option changed between steps (optimizer.py:1650-1860, 976-1045)
    # ------------------------------------------------------------------
    @staticmethod
    def _group_signature(group):
        """The group options that decide which states a parameter has and which kernels step it."""
        return (bool(group.get("quantize", True)), group.get("block_size", 2048), group.get("m_block_size", 256),
                group.get("m_quant_type", "uf8"), group.get("v_quant_type", "al8"), group.get("c_quant_type"),
                group.get("min_8bit_size", 4096), group.get("apollo_rank", 0), bool(group.get("apollo_factorize", False)),
                bool(group.get("factored", True)), group.get("beta1") is None, group.get("beta2") is None,
                group.get("beta2_decay") is None, group.get("beta3") is None)

    @classmethod
    def _config_signature(cls, group, grad):
        return cls._group_signature(group) + (grad.dim(),)

    @staticmethod
    def _reset_keep_step(state):
        """optimizer.py:380-386"""
        step, seed = state.get("step", 0), state.get("sr_seed")
        state.clear()
        state["step"] = step
        if seed is not None:
            state["sr_seed"] = seed

    @staticmethod
    def _al_to_fp32(state, prefix):
        """_deq_v(..., pop=True) (optimizer.py:358-365) through af8_al_dequant."""
        q = state.pop(prefix + "_q")
        scale, min_log = state.pop(prefix + "_scale"), state.pop(prefix + "_min_log")
        shape, pad = state.pop(prefix + "_shape"), state.pop(prefix + "_pad")
        numel = q.numel() - pad
        out = torch.empty(numel, dtype=torch.float32, device=q.device)
        with torch.cuda.device(q.device):
            N.check(N.lib().af8_al_dequant(q.data_ptr(), scale.data_ptr(), min_log.data_ptr(), numel, q.numel() // scale.numel(),
                                           8 if q.dtype == torch.uint8 else 16, out.data_ptr(),
                                           torch.cuda.current_stream(q.device).cuda_stream), "af8_al_dequant")
        return out.view(list(shape))

    @staticmethod
    def _fp32_to_al(state, prefix, tensor, block, fmt):
        """_quant_v (optimizer.py:373-377) through af8_al_quant."""
        x = tensor.contiguous().float()
        numel = x.numel()
        pad = _pad_to(numel, block)
        q = torch.empty(numel + pad, dtype=torch.uint8 if fmt == "al8" else torch.int16, device=x.device)
        scale = torch.empty((numel + pad) // block, dtype=torch.float32, device=x.device)
        min_log = torch.empty_like(scale)
        with torch.cuda.device(x.device):
            N.check(N.lib().af8_al_quant(x.data_ptr(), numel, block, 8 if fmt == "al8" else 16, -126.0, q.data_ptr(),
                                         scale.data_ptr(), min_log.data_ptr(),
                                         torch.cuda.current_stream(x.device).cuda_stream), "af8_al_quant")
        state[prefix + "_q"], state[prefix + "_scale"], state[prefix + "_min_log"] = q, scale, min_log
        state[prefix + "_shape"], state[prefix + "_pad"] = tensor.shape, pad

    @staticmethod
    def _m_to_fp32(state, p, m_block):
        """_m_dequantize of the stored momentum (optimizer.py:1029-1039)."""
        fmt = state.get("m_quant_type", "uf8")
        if fmt in ("d8", "d4"):
            from ._engine import ensure_qmap
            ensure_qmap(p.device)
        q, scale = state["m_q"], state["m_scale"]
        out = torch.empty(p.numel(), dtype=torch.float32, device=p.device)
        with torch.cuda.device(p.device):
            N.check(N.lib().af8_m_dequant(q.data_ptr(), scale.data_ptr(), p.numel(), m_block, N.M_FMT[fmt], out.data_ptr(),
                                          torch.cuda.current_stream(p.device).cuda_stream), "af8_m_dequant")
        return out.view(p.shape)

    @staticmethod
    def _fp32_to_m(state, m, fmt, m_block):
        """_m_quantize (optimizer.py:547-552) through af8_m_quant."""
        if fmt in ("d8", "d4"):
            from ._engine import ensure_qmap
            ensure_qmap(m.device)
        x = m.contiguous().float()
        numel = x.numel()
        padded = ((numel + m_block - 1) // m_block) * m_block
        q = torch.empty(padded // 2 if fmt in ("uf4", "d4") else padded, dtype=torch.uint8, device=x.device)
        scale = torch.empty(padded // m_block, dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            N.check(N.lib().af8_m_quant(x.data_ptr(), numel, m_block, N.M_FMT[fmt], q.data_ptr(), scale.data_ptr(),
                                        torch.cuda.current_stream(x.device).cuda_stream), "af8_m_quant")
        state["m_q"], state["m_scale"] = q, scale

    def _sync_state(self, p, grad, group, state):
        """Bring an existing state in line with the group's current options, as _init_group does at
        every step (optimizer.py:1650-1860): a changed momentum format resets the momentum, a changed
        V / C format or block size and a changed mode (APOLLO, factored) re-initialise the state and
        keep the step count, the quantize flag converts the states in place, CAME's confidence states
        come and go with beta3.  Returns the state to step with."""
        numel = p.numel()
        piece = self._pieces.get(id(p))
        full_numel = piece.full_numel if piece is not None else numel
        use_quant = group.get("quantize", True) and not (full_numel < group.get("min_8bit_size", 4096))
        block, m_block = group.get("block_size", 2048), group.get("m_block_size", 256)
        mqt, vqt = group.get("m_quant_type", "uf8"), group.get("v_quant_type", "al8")
        cqt = group.get("c_quant_type") or vqt
        beta1, beta3 = group.get("beta1"), group.get("beta3")
        sgd = group.get("beta2") is None and group.get("beta2_decay") is None
        use_apollo = group.get("apollo_rank", 0) > 0 and grad.dim() >= 2
        expect_factored = grad.dim() >= 2 and group.get("factored", True)
        shape = tuple(p.shape)
        if piece is not None and piece.full_rows and expect_factored:
            shape = (piece.full_rows, shape[-1])
        needs_init = False

        old_mqt = state.get("m_quant_type", "uf8")
        if old_mqt not in _M_TYPES:
            state["m_quant_type"] = old_mqt = "uf8"
        old_mbs = state.get("m_block_size", m_block)
        if not isinstance(old_mbs, int):
            state["m_block_size"] = old_mbs = m_block
        if (old_mqt != mqt or old_mbs != m_block) and use_quant:
            logger.warning(f"Adafactor8Bit: M config changed (type: '{old_mqt}'->'{mqt}', block: {old_mbs}->{m_block}) "
                           f"for param shape {p.shape}. Momentum history will be reset to zero.")
            for k in ("m_q", "m_scale", "m_block_size", "m", "m_low_q", "m_low_scale", "m_low"):
                state.pop(k, None)
            state["m_quant_type"] = mqt
        old_vqt = state.get("v_quant_type", "al8")
        old_cqt = state.get("c_quant_type", old_vqt)
        old_bs = state.get("block_size", block)
        if (old_vqt != vqt or old_cqt != cqt or old_bs != block) and use_quant:
            logger.warning(f"Adafactor8Bit: V/C/Block config changed (V: '{old_vqt}'->'{vqt}', C: '{old_cqt}'->'{cqt}', "
                           f"BS: {old_bs}->{block}) for param shape {p.shape}. Re-initializing state.")
            self._reset_keep_step(state)
            needs_init = True
        is_apollo_state = "apollo_seed" in state
        if use_apollo != is_apollo_state:
            logger.warning(f"Adafactor8Bit: Apollo/Adafactor mode changed for param shape {p.shape}. Re-initializing state.")
            self._reset_keep_step(state)
            needs_init = True
        elif use_apollo:
            came_toggled = (state.get("beta3") is None) != (beta3 is None)
            if (state.get("apollo_rank") != group.get("apollo_rank", 0)
                    or state.get("apollo_factorize", False) != group.get("apollo_factorize", False) or came_toggled):
                logger.warning(f"Adafactor8Bit: Apollo/CAME config changed for param shape {p.shape}. Re-initializing state.")
                self._reset_keep_step(state)
                needs_init = True
            else:
                state["beta3"] = beta3
        elif not sgd:
            if ("row_var" in state or "row_var_q" in state) != expect_factored:
                logger.warning(f"Adafactor8Bit: factored mode mismatch for param shape {p.shape}. Re-initializing state.")
                self._reset_keep_step(state)
                needs_init = True
        if needs_init:
            return self._create_state(p, grad, group)

        cur_block = state.get("block_size", block)
        cur_m_block = state.get("m_block_size", m_block) if beta1 is not None else 0
        was_quant = state.get("is_quantized", False)
        if use_apollo and use_quant != was_quant:
            raise NotImplementedError("changing `quantize` on APOLLO states is not available in this build")
        if use_quant and not was_quant:                      # optimizer.py:978-1019
            if vqt != "fp32":
                for k in ("row_var", "col_var", "variance"):
                    if k in state and k + "_q" not in state:
                        self._fp32_to_al(state, k, state.pop(k), cur_block, vqt)
            if cqt != "fp32" and beta3 is not None:
                for k in ("conf_row", "conf_col"):
                    if k in state and k + "_q" not in state:
                        self._fp32_to_al(state, k, state.pop(k), cur_block, cqt)
            if beta1 is not None and "m_q" not in state and mqt != "fp32":
                mb = state.get("m_block_size", cur_m_block)
                if "m" in state:
                    self._fp32_to_m(state, state.pop("m"), mqt, mb)
                    state["m_quant_type"] = mqt
                else:
                    _new_m_state(state, numel, mb, mqt, p.device, p.shape)
                state["m_block_size"] = mb
            state["is_quantized"] = True
        elif not use_quant and was_quant:                    # optimizer.py:1021-1045
            for k in ("row_var", "col_var", "conf_row", "conf_col", "variance"):
                if k + "_q" in state:
                    state[k] = self._al_to_fp32(state, k)
            if "m_q" in state:
                state["m"] = self._m_to_fp32(state, p, state.get("m_block_size", cur_m_block))
                for k in ("m_q", "m_scale", "m_block_size", "m_quant_type"):
                    state.pop(k, None)
            state["is_quantized"] = False

        if not use_apollo:
            if beta3 is None:                                # optimizer.py:1799-1806
                for prefix in ("conf_row", "conf_col"):
                    state.pop(prefix, None)
                    for suffix in ("q", "scale", "min_log", "shape", "pad"):
                        state.pop(f"{prefix}_{suffix}", None)
            elif expect_factored:                            # optimizer.py:1808-1836
                r_shape = list(shape[:-2]) + [shape[-2], 1]
                c_shape = list(shape[:-2]) + [1, shape[-1]]
                c_fmt = cqt if use_quant else "fp32"
                if "conf_row" not in state and "conf_row_q" not in state:
                    _new_al_state(state, "conf_row", r_shape, cur_block, p.device, c_fmt)
                if "conf_col" not in state and "conf_col_q" not in state:
                    _new_al_state(state, "conf_col", c_shape, cur_block, p.device, c_fmt)
        if beta1 is not None and "m_q" not in state and not use_apollo:     # optimizer.py:1838-1849
            mb = state.get("m_block_size", m_block)
            if use_quant and mqt != "fp32":
                if "m" in state:
                    self._fp32_to_m(state, state.pop("m"), mqt, mb)
                    state["m_quant_type"] = mqt
                else:
                    _new_m_state(state, numel, mb, mqt, p.device, p.shape)
                state["m_block_size"] = mb
            elif "m" not in state and mqt == "fp32":
                state["m"] = torch.zeros(p.shape, dtype=torch.float32, device=p.device)
                state["m_quant_type"] = "fp32"
        if "block_size" not in state:
            state["block_size"] = block
        if beta1 is None:
            for k in ("m_q", "m_scale", "m_block_size", "m_quant_type", "m"):
                state.pop(k, None)
        return state

    # ------------------------------------------------------------------
    # per-step host scalars (optimizer.py:1957-2040, 832-856)
    # ------------------------------------------------------------------
    @staticmethod
    def _step_scalars(group, step):
        """Scalars of one parameter at step `step` that do not depend on tensor
        contents, rounded to binary32 where the reference's 0-d tensors round."""
        eps1, eps2 = group["eps"]
        if eps1 is None:
            eps1 = 1e-30
        beta1, beta2, beta3 = group.get("beta1"), group["beta2"], group.get("beta3")
        factored = group.get("factored", True)
        adam = (not factored) and beta2 is not None and beta3 is None
        eps_denom = eps1 if adam else 0.0
        eps_gradsq = 0.0 if adam else eps1
        relative = group["relative_step"]
        if beta2 is not None:
            beta_val = 1.0 - beta2
        elif group["beta2_decay"] is not None:
            beta_val = math.pow(step, group["beta2_decay"])
        else:
            beta_val = 0.0
        lr = float(group["lr"])
        rho = f32(min(lr, 1.0 / math.sqrt(step)) if relative else lr)
        bc_mul = None      # multiplies alpha
        bc_div = None      # divides alpha
        if beta1 is not None and not relative and not (beta2 is None and group["beta2_decay"] is None):
            apply_bc = adam if group.get("bias_correction") is None else group["bias_correction"]
            if apply_bc:
                bc1 = 1.0 - beta1 ** step
                if beta2 is not None:
                    bc2 = 1.0 - beta2 ** step
                    bc_mul = f32(math.sqrt(bc2) / bc1)
                    if adam:
                        eps_denom = eps1 * math.sqrt(bc2)
                else:
                    bc_div = f32(bc1)
        return dict(eps1=eps1, eps2=eps2, adam=adam, beta_val=beta_val, rho=rho,
                    bc_mul=bc_mul, bc_div=bc_div, eps_denom=eps_denom, eps_gradsq=eps_gradsq,
                    eps_sq=max(eps1 * eps1, _FLOOR))

    @staticmethod
    def _alpha_decay(group, sc):
        """alpha and the weight-decay factor when alpha does not depend on the
        parameter's RMS (scale_parameter=False)."""
        alpha = sc["rho"]
        if sc["bc_mul"] is not None:
            alpha = f32(alpha * sc["bc_mul"])
        elif sc["bc_div"] is not None:
            alpha = f32(alpha / sc["bc_div"])
        wd = group["weight_decay"]
        if wd != 0:
            mult = alpha if group.get("scale_weight_decay", True) else sc["rho"]
            decay = f32(f32(1.0) - f32(mult * f32(wd)))
        else:
            decay = f32(1.0)
        return alpha, decay

    # ------------------------------------------------------------------
    # step
    # ------------------------------------------------------------------
    @torch.no_grad()
    def step(self, closure=None, *, grad_ready=None):
        """One optimization step (optimizer.py:1866-1938).

        grad_ready (not in the reference): an optional sequence with one CUDA event (or None) per
        parameter group.  The launches of a group wait for its event on the current stream, so a
        caller that brings gradients in on another stream (host-to-device copies, a reduce-scatter)
        group by group overlaps that transfer with the update of the groups already there."""
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        N.lib()   # fail loudly when the CUDA library is missing
        if grad_ready is not None and len(grad_ready) != len(self.param_groups):
            raise ValueError("grad_ready needs one entry per parameter group")
        pending = []                  # sharded step: (group index, exchange count, device, generator) of every launch plan
        for gi, group in enumerate(self.param_groups):
            if grad_ready is not None and grad_ready[gi] is not None:
                torch.cuda.current_stream().wait_event(grad_ready[gi])
            runs, copy_back = self._group_runs(gi, group)
            for e, dev, gen in runs:
                if self._shard is not None:
                    pending.append((gi, e, dev, gen))
                    continue
                with torch.cuda.device(dev):             # the whole pass sequence of the plan, now
                    for _ in gen:
                        pass
            for p, work in copy_back:
                p.copy_(work)
            if self._after_group is not None:
                self._after_group(gi, group)
        if self._shard is not None:
            self._step_sharded(pending)
        return loss

    def _step_sharded(self, pending):
        """The passes of all launch plans, scheduled for a sharding wrapper.  `self._shard` provides
          rounds            the largest exchange count of any plan on any rank;
          exchange(r)       sums the exchange slots of round r over the ranks (r = 0 .. rounds - 1);
          part_of_group[gi] the part of the parameter space a parameter group lies in; parts are numbered
                            in the order their parameters may be published;
          parts             their number;
          after_part(k)     called when every parameter-writing pass of part k has been enqueued.
        A plan with e exchange points consists of e + 1 segments; they run in rounds
        rounds - e .. rounds, so that the last segment of every plan, the one that writes parameters,
        falls into the last round, where the plans run part by part.  Every rank calls exchange and
        after_part in the same order, whatever it owns."""
        sh = self._shard
        S = int(sh.rounds)

        def advance(item, last):
            gi, e, dev, gen = item
            with torch.cuda.device(dev):
                try:
                    next(gen)
                    if last:
                        raise RuntimeError("a launch plan has more exchange points than it announced")
                except StopIteration:
                    if not last:
                        raise RuntimeError("a launch plan has fewer exchange points than it announced") from None

        for gi, e, dev, gen in pending:
            if e > S:
                raise RuntimeError("a launch plan needs more exchange rounds than the sharding wrapper provides")
        for r in range(S):
            for item in pending:
                if r >= S - item[1]:
                    advance(item, False)
            sh.exchange(r)
        for k in range(int(sh.parts)):
            for item in pending:
                if sh.part_of_group[item[0]] == k:
                    advance(item, True)
            sh.after_part(k)

    def _sr_seed(self, state, p=None):
        """The parameter's stochastic-rounding seed, taken from the optimizer-level counter the
        first time the parameter is rounded (optimizer.py:1889-1892).  A wrapper that steps only a
        subset of the parameters (the sharded optimizer) presets `_sr_seed_map` (id(param) -> seed)
        so that the seeds are those of the unsharded run."""
        if "sr_seed" not in state:
            preset = self._sr_seed_map.get(id(p)) if (self._sr_seed_map is not None and p is not None) else None
            if preset is not None:
                state["sr_seed"] = preset
            else:
                state["sr_seed"] = self._sr_seed_counter
                self._sr_seed_counter += 1
        return state["sr_seed"]

    def _group_runs(self, gi, group):
        """-> ([(exchange count, device, generator)] for the launch plans of the group's parameters that
        have gradients, [(parameter, contiguous copy)] to copy back).

        The slow path looks at every parameter: creates its state on its first step, re-checks the
        state against the group's options when they changed (or after a load), hands out
        stochastic-rounding seeds, sorts the tensors into launch groups.  Its result is remembered;
        while the same parameters carry gradients of the same kind and the options that matter are
        unchanged, the next steps reuse the sorting and only collect the gradients."""
        params = group["params"]
        gsig = self._group_signature(group) + (bool(group.get("stochastic_round_writeback", False)),)
        c = self._group_cache.get(gi)
        if c is not None and c["gsig"] == gsig and len(c["params"]) == len(params):
            grads = []
            for p, q, kind in zip(params, c["params"], c["kinds"]):
                g = p.grad
                if p is not q or ((None if g is None else (g.dim(), g.dtype)) != kind):
                    grads = None
                    break
                grads.append(g)
            if grads is not None:
                states = c["states"]
                return [fn(gi, group, key, [(params[j], grads[j], states[j]) for j in idx])
                        for fn, key, idx in c["launches"]], ()
        entries, copy_back, kinds, states, cacheable = [], [], [], [], True
        for j, p in enumerate(params):
            g = p.grad
            kinds.append(None if g is None else (g.dim(), g.dtype))
            states.append(None)
            if g is None:
                continue
            if not p.is_cuda:
                raise RuntimeError("Adafactor8Bit (B200 build) only updates CUDA parameters; "
                                   "there is no CPU path")
            state = self.state[p]
            if len(state) == 0 or "is_quantized" not in state:
                state = self._create_state(p, g, group)
                self._cfg_seen[id(p)] = self._config_signature(group, g)
            else:
                sig = self._config_signature(group, g)
                if self._cfg_seen.get(id(p)) != sig:     # first step after a load, or an option was edited
                    state = self._sync_state(p, g, group, state)
                    self._cfg_seen[id(p)] = sig
                    self._plans.clear()                  # launch plans cache state pointers and formats
            states[j] = state
            if group.get("stochastic_round_writeback", False) and p.dtype in (torch.bfloat16, torch.float16):
                self._sr_seed(state, p)     # seeds follow the parameter order of the step (optimizer.py:1889-1892)
            if p.numel() == 0:              # an empty parameter has a state and a step count, nothing to launch
                state["step"] = state.get("step", 0) + 1
                cacheable = False
                continue
            work = p
            if not p.is_contiguous():       # stepped on a contiguous copy, copied back (optimizer.py:2000-2005, 3081-3084)
                work = p.detach().contiguous()
                copy_back.append((p, work))
                cacheable = False
            entries.append((j, work, g, state))
        launches = self._sort_group(group, entries)
        self._group_cache.pop(gi, None)
        if cacheable:
            self._group_cache[gi] = dict(gsig=gsig, params=list(params), kinds=kinds, states=states,
                                         launches=[(fn, key, [e[0] for e in items]) for fn, key, items in launches])
        return [fn(gi, group, key, [(p, g, st) for _, p, g, st in items]) for fn, key, items in launches], copy_back

    def _sort_group(self, group, entries):
        """Sort (index, parameter, gradient, state) entries into launch groups ->
        [(method that runs one, its key, entries)]."""
        apollo_rank = group.get("apollo_rank", 0)
        factored = group.get("factored", True)
        sgd = group["beta2"] is None and group["beta2_decay"] is None
        fullrank, factored_items, apollo_items = {}, {}, []
        for ent in entries:
            _, p, g, st = ent
            if sgd:                 # optimizer.py:2045-2071: no second moment, every shape takes the flat path
                if group.get("beta1") is not None:
                    m_fmt = "fp32" if "m" in st else st.get("m_quant_type", "uf8")
                    m_block = st.get("m_block_size", group.get("m_block_size", 256))
                else:
                    m_fmt, m_block = None, 0
                key = (p.device, g.dtype, "none", m_fmt, st.get("block_size", group.get("block_size", 2048)), m_block, p.dtype)
                fullrank.setdefault(key, []).append(ent)
                continue
            if apollo_rank > 0 and "apollo_seed" in st:
                apollo_items.append(ent)        # more than two dimensions: stepped as (shape[0], -1), optimizer.py:2634-2639
                continue
            quant = st.get("is_quantized", False)
            if group.get("beta1") is not None:
                m_fmt = "fp32" if "m" in st else st.get("m_quant_type", "uf8")
                m_block = st.get("m_block_size", group.get("m_block_size", 256))
            else:
                m_fmt, m_block = None, 0
            if g.dim() >= 2 and factored:
                came = group.get("beta3") is not None and group.get("beta1") is not None
                key = (p.device, g.dtype, m_fmt, m_block, came, p.dtype, g.dim() > 2)    # batches of matrices: a plan of their own
                factored_items.setdefault(key, []).append(ent)
                continue
            v_fmt = st.get("v_quant_type", "al8") if quant else "fp32"
            key = (p.device, g.dtype, v_fmt, m_fmt, st.get("block_size", group.get("block_size", 2048)), m_block, p.dtype)
            fullrank.setdefault(key, []).append(ent)
        out = [(self._run_fullrank, key, items) for key, items in fullrank.items()]
        out += [(self._run_factored, key, items) for key, items in factored_items.items()]
        if apollo_items:
            out.append((self._run_apollo, None, apollo_items))
        return out

    # ------------------------------------------------------------------
    # APOLLO (optimizer.py:2557-3084)
    # ------------------------------------------------------------------
    @staticmethod
    def _stable_randn(shape, seed, device):
        gen = torch.Generator(device=device).manual_seed(int(seed))           # optimizer.py:139-149
        return torch.randn(shape, generator=gen, device=device, dtype=torch.float32)

    @staticmethod
    def _next_seed(seed, adv=0xF):
        gen = torch.Generator().manual_seed(int(seed))                         # optimizer.py:152-155
        return torch.randint(0, torch.iinfo(torch.int64).max, (adv,), generator=gen).tolist()[-1]

    def _projection(self, state, shape, step, device, cache_proj):
        """Transposed projection matrix of this step (_get_apollo_proj_matrix, optimizer.py:2557-2584)."""
        rank = int(state["apollo_rank"])
        gap = int(state["apollo_update_proj_gap"])
        refresh = (step - int(state.get("last_proj_step", -gap))) >= gap
        cached = state.get("apollo_proj_matrix_T") if cache_proj else state.get("_proj_T")
        if not refresh and cached is not None:
            return cached
        if refresh:
            state["current_proj_seed"] = int(state["apollo_seed"])
            state["apollo_seed"] = self._next_seed(state["current_proj_seed"])
            state["last_proj_step"] = step
        R, C = shape
        m_shape = (rank, C) if R >= C else (R, rank)
        seed = state.get("current_proj_seed", state["apollo_seed"])
        rng_dev = APOLLO_RNG_DEVICE if APOLLO_RNG_DEVICE is not None else device
        proj = self._stable_randn(m_shape, seed, rng_dev) / math.sqrt(rank)
        proj_t = proj.T.contiguous().to(device)
        if cache_proj:
            state["apollo_proj_matrix_T"] = proj_t
        else:
            state["_proj_T"] = proj_t      # same values the reference would regenerate each step
        return proj_t

    def _run_apollo(self, gi, group, key, items):
        rank = int(group["apollo_rank"])
        beta1, beta2 = group.get("beta1"), group["beta2"]
        beta3 = group.get("beta3")
        factorize = bool(group.get("apollo_factorize", False))
        came = beta3 is not None and beta1 is not None
        rule = dict(factorize=factorize, came=came) if (factorize or came) else None
        block = group.get("block_size", 2048)
        m_block = group.get("m_block_size", 256)
        device = items[0][0].device
        quant0 = items[0][2].get("is_quantized", False)
        v_fmt = items[0][2].get("v_quant_type", "al8") if quant0 else "fp32"
        m_fmt = ((items[0][2].get("m_quant_type", "uf8") if quant0 else "fp32") if beta1 is not None else None)
        # tensors of more than two dimensions are stepped as (shape[0], -1) matrices (optimizer.py:2634-2639);
        # fp16 gradients are widened first, as the reference widens every gradient (optimizer.py:2601)
        pcs = [self._pieces.get(id(p)) for p, _, _ in items]
        items = [(p if p.dim() == 2 else p.view(p.shape[0], -1),
                  (g.float() if g.dtype == torch.float16 else g).reshape(g.shape[0], -1), st) for p, g, st in items]
        ids = tuple(p.data_ptr() for p, _, _ in items)     # (also follows a parameter whose storage was replaced)
        c_fmt = items[0][2].get("c_quant_type", items[0][2].get("v_quant_type", "al8")) if quant0 else "fp32"
        pkey = (gi, "apollo", items[0][1].dtype, items[0][0].dtype, v_fmt, m_fmt, rank, bool(group["maximize"]), factorize, came, c_fmt)
        sr = bool(group.get("stochastic_round_writeback", False)) and items[0][0].dtype in (torch.bfloat16, torch.float16)
        plan = self._plans.get(pkey)
        first_flags, pts, per_tensor, grads = [], [], [], []
        apollo_eps = group.get("apollo_eps", 1e-6)
        # low-rank states are created on the tensor's first step (optimizer.py:2763-2779, 2916-2917)
        for p, g, st in items:
            quant = st.get("is_quantized", False)
            if quant != quant0:
                raise NotImplementedError("APOLLO tensors of one group must share the quantisation setting")
            R, C = p.shape
            nl = max(R, C) * rank
            first = st.get("v_low_q") is None and st.get("v_low") is None
            low_shape = (R, rank) if R >= C else (rank, C)
            if factorize:                               # fp32 factors instead of v_low (optimizer.py:2688-2700)
                first = "row_var_low" not in st
                if first:
                    st["row_var_low"] = torch.zeros((low_shape[0], 1), dtype=torch.float32, device=p.device)
                    st["col_var_low"] = torch.zeros((1, low_shape[1]), dtype=torch.float32, device=p.device)
                if came and st.get("conf_row_low_q") is None and st.get("conf_row_low") is None:      # optimizer.py:2729-2744
                    for prefix, shp in (("conf_row_low", (low_shape[0], 1)), ("conf_col_low", (1, low_shape[1]))):
                        tmp = {}
                        _new_al_state(tmp, prefix, shp, st.get("block_size", block), p.device, c_fmt)
                        st.update(tmp)
            elif came and st.get("res_low_q") is None and st.get("res_low") is None:                   # optimizer.py:2806-2810
                tmp = {}
                _new_al_state(tmp, "res_low", low_shape, st.get("block_size", block), p.device, c_fmt)
                st.update(tmp)
            first_flags.append(first)
            if first and not factorize:
                tmp = {}
                _new_al_state(tmp, "v_low", (nl,), st.get("block_size", block), p.device, v_fmt)
                for k in ("v_low_q", "v_low_scale", "v_low_min_log", "v_low_shape", "v_low_pad", "v_low"):
                    if k in tmp:
                        st[k] = tmp[k]
                if v_fmt != "fp32":
                    st["v_low_shape"] = torch.Size([nl])
            if beta1 is not None and st.get("m_low_q") is None and st.get("m_low") is None:
                tmp = {}
                low_shape = (R, rank) if R >= C else (rank, C)             # an fp32 momentum has the projected gradient's shape
                _new_m_state(tmp, nl, st.get("m_block_size", m_block), m_fmt, p.device, low_shape, prefix="m_low")
                tmp.pop("m_quant_type", None)
                st.update(tmp)
        if plan is None or plan.ids != ids:
            plan = ApolloPlan(device, items[0][1].dtype, v_fmt, m_fmt, block, m_block, group["maximize"],
                              [p for p, _, _ in items], [s for _, _, s in items], rank,
                              copies=[pc.copy if pc is not None else None for pc in pcs], rule=rule, c_fmt=c_fmt)
            plan.ids = ids
            self._plans[pkey] = plan
        step_any = None
        for p, g, st in items:
            step = st["step"] + 1
            st["step"] = step
            step_any = step
            sc = self._step_scalars(group, step)
            R, C = p.shape
            pts.append(self._projection(st, (R, C), step, p.device, group.get("apollo_cache_proj", False)))
            alpha = sc["rho"]
            wd = group["weight_decay"]
            decay = f32(f32(1.0) - f32(alpha * f32(wd))) if wd != 0 else f32(1.0)      # optimizer.py:3007-3009
            t = dict(alpha=alpha, bc=1.0, bc_mode=0, d=f32(group["d"]), clip_div=f32(math.sqrt(R * C) * group["d"]),
                     fira_margin1=f32(1.0 + group.get("fira_margin", 0.01)),
                     sqrt_scale=f32(math.sqrt(group.get("apollo_scale", 1.0))),
                     fira=bool(group.get("enable_fira_for_apollo", True)),
                     scale_tensor=group.get("apollo_scale_type", "channel") == "tensor",
                     scale_front=bool(group.get("apollo_scale_front", False)), decay=decay, has_decay=wd != 0,
                     sr=sr, sr_base=sr_base(self._sr_seed(st, p), step) if sr else 0)      # optimizer.py:3050-3051
            if beta1 is not None and not group["relative_step"]:                       # optimizer.py:3015-3023
                apply_bc = True if group.get("bias_correction") is None else group["bias_correction"]
                if apply_bc:
                    bc1 = 1.0 - beta1 ** step
                    if beta2 is not None:
                        t["bc"], t["bc_mode"] = f32(math.sqrt(1.0 - beta2 ** step) / bc1), 1
                    else:
                        t["bc"], t["bc_mode"] = f32(bc1), 2
            if t["fira"]:
                prev = st.get("scaled_grad_norm_prev")
                t["fira_has_prev"] = prev is not None
                if prev is None:
                    prev = torch.zeros((), dtype=torch.float32, device=p.device)
                    st["scaled_grad_norm_prev"] = prev
                t["fira_prev"] = prev
            else:
                t["fira_has_prev"] = False
            per_tensor.append(t)
            grads.append(g if g.is_contiguous() else g.contiguous())
        sc = self._step_scalars(group, step_any)
        bv = sc["beta_val"]
        low = dict(v_w=f32(bv), v_keep=f32(1.0 - bv), m_w=f32(1.0 - beta1) if beta1 is not None else f32(0.0),
                   apollo_eps=f32(apollo_eps), c_w=f32(1.0 - beta3) if beta3 is not None else f32(0.0),
                   eps_came=f32(group.get("eps_came", 1e-16)), eps_sq=f32(max(apollo_eps * apollo_eps, _FLOOR)), d=f32(group["d"]))
        floor_later = math.log2(max(apollo_eps * apollo_eps, _FLOOR))                  # optimizer.py:2766-2767
        # the projection matrix of a tensor changes every apollo_update_proj_gap steps only (optimizer.py:2557-2584)
        versions = [(st.get("last_proj_step"), st.get("current_proj_seed")) for _, _, st in items]
        scale = None
        if group["scale_parameter"]:                     # alpha_t from the parameters' RMS, on the device (optimizer.py:850-853)
            scale = self._scale_inputs(group, len(items))
            for i, (p, g, st) in enumerate(items):
                self._fill_scale(scale, i, group, self._step_scalars(group, st["step"]))
            scale["bc_mode"][:] = 0                      # the bias correction enters the update scale (optimizer.py:3015-3023)

        def passes():
            plan.run(grads, pts, per_tensor, low, first_flags, floor_later, params=[p for p, _, _ in items], scale=scale,
                     versions=versions)
            return
            yield                                                                       # (no exchange points)
        return 0, device, passes()

    def _scale_inputs(self, group, n):
        scale = {k: np.zeros(n, dtype=f32) for k in ("rho", "eps2", "bc", "weight_decay")}
        scale["bc_mode"] = np.zeros(n, dtype=np.int32)
        scale["scale_weight_decay"] = np.full(n, int(bool(group.get("scale_weight_decay", True))), dtype=np.int32)
        return scale

    def _fill_scale(self, scale, i, group, sc):
        scale["rho"][i] = sc["rho"]
        scale["eps2"][i] = f32(sc["eps2"])
        scale["weight_decay"][i] = f32(group["weight_decay"])
        if sc["bc_mul"] is not None:
            scale["bc"][i], scale["bc_mode"][i] = sc["bc_mul"], 1
        elif sc["bc_div"] is not None:
            scale["bc"][i], scale["bc_mode"][i] = sc["bc_div"], 2

    def _run_factored(self, gi, group, key, items):
        device, gdtype, m_fmt, m_block, came, pdtype = key[:6]
        sr = bool(group.get("stochastic_round_writeback", False)) and pdtype in (torch.bfloat16, torch.float16)
        ids = tuple(id(p) for p, _, _ in items)
        pkey = (gi, "factored", key, bool(group["maximize"]), sr)
        plan = self._plans.get(pkey)
        pcs = [self._pieces.get(id(p)) for p, _, _ in items]
        if plan is None or plan.ids != ids:
            v_fmts = [(st.get("v_quant_type", "al8") if st.get("is_quantized", False) else "fp32") for _, _, st in items]
            c_fmts = [(st.get("c_quant_type", st.get("v_quant_type", "al8")) if st.get("is_quantized", False) else "fp32")
                      for _, _, st in items]
            plan = FactoredPlan(device, gdtype, m_fmt, m_block, came, group["maximize"],
                                [p for p, _, _ in items], [s for _, _, s in items], v_fmts, c_fmts, stochastic_round=sr,
                                pieces=pcs)
            plan.ids = ids
            self._plans[pkey] = plan
        n = len(items)
        scale = self._scale_inputs(group, n) if group["scale_parameter"] else None
        cols = {k: np.empty(n, dtype=f32) for k in ("decay", "alpha", "v_w", "m_w", "c_w", "eps1", "eps_came")}
        if sr:
            cols["sr_base"] = np.zeros(n, dtype=np.uint64)
        steps = []
        for _, _, st in items:
            step = st["step"] + 1
            st["step"] = step
            steps.append(step)
        grads = [g if g.is_contiguous() else g.contiguous() for _, g, _ in items]
        if sr:                      # a part of a tensor draws the counters of its elements in the whole tensor
            for i, (_, _, st) in enumerate(items):
                first = pcs[i].elem0 if pcs[i] is not None else 0
                cols["sr_base"][i] = (sr_base(self._sr_seed(st), steps[i]) + first) & 0xFFFFFFFFFFFFFFFF
        uniform = steps.count(steps[0]) == n          # the usual case: every tensor of the group is at the same step
        for i in ([0] if uniform else range(n)):
            where = slice(None) if uniform else i
            sc = self._step_scalars(group, steps[i])
            alpha, decay = self._alpha_decay(group, sc)
            cols["decay"][where], cols["alpha"][where] = decay, alpha
            cols["v_w"][where] = f32(sc["beta_val"])
            cols["m_w"][where] = f32(1.0 - group["beta1"]) if group.get("beta1") is not None else f32(0.0)
            cols["c_w"][where] = f32(1.0 - group["beta3"]) if group.get("beta3") is not None else f32(0.0)
            cols["eps1"][where] = f32(sc["eps1"])
            cols["eps_came"][where] = f32(group.get("eps_came", 1e-16))
            if scale is not None:
                self._fill_scale(scale, where, group, sc)
        d, fira, lag = float(group["d"]), bool(group.get("enable_fira_for_adafactor", False)), bool(group.get("lag_norm", False))
        return (factored_exchanges(came, d, fira, lag), device,
                plan.stages(grads, cols, d=d, fira=fira, fira_margin=float(group.get("fira_margin", 0.01)), scale=scale, lag=lag))

    def _run_fullrank(self, gi, group, key, items):
        device, gdtype, v_fmt, m_fmt, block, m_block, pdtype = key
        sr = bool(group.get("stochastic_round_writeback", False)) and pdtype in (torch.bfloat16, torch.float16)
        sc0 = self._step_scalars(group, 1)
        momentum_only = group.get("momentum_only_1d")
        if momentum_only is None:
            momentum_only = not sc0["adam"]
        sgd = v_fmt == "none"
        if sgd:
            momentum_only = False
        ids = tuple(id(p) for p, _, _ in items)
        pkey = (gi, "fullrank", key, bool(momentum_only), bool(group["maximize"]), sr)
        plan = self._plans.get(pkey)
        pcs = [self._pieces.get(id(p)) for p, _, _ in items]
        if plan is None or plan.ids != ids:
            plan = FullrankPlan(device, gdtype, v_fmt, m_fmt, block, m_block, sc0["adam"], momentum_only,
                                group["maximize"], [p for p, _, _ in items], [s for _, _, s in items],
                                stochastic_round=sr, pieces=pcs)
            plan.ids = ids
            self._plans[pkey] = plan
        n = len(items)
        scale = None
        if group["scale_parameter"]:
            scale = {k: np.zeros(n, dtype=f32) for k in ("rho", "eps2", "bc", "weight_decay")}
            scale["bc_mode"] = np.zeros(n, dtype=np.int32)
            scale["scale_weight_decay"] = np.full(n, int(bool(group.get("scale_weight_decay", True))), dtype=np.int32)
        cols = {k: np.empty(n, dtype=f32) for k in _FULLRANK_COLS}
        if sr:
            cols["sr_base"] = np.zeros(n, dtype=np.uint64)
        def row_values(step):
            sc = self._step_scalars(group, step)
            alpha, decay = self._alpha_decay(group, sc)
            bv = sc["beta_val"]
            keep = f32(1.0 - group["beta1"]) if (sgd and group.get("beta1") is not None) else f32(1.0 - bv)
            return sc, (decay, alpha, f32(bv), keep, f32(bv * sc["eps_gradsq"]),
                        f32(1.0 - group["beta1"]) if group.get("beta1") is not None else f32(0.0),
                        f32(sc["eps_gradsq"]), f32(sc["eps_denom"]), f32(sc["eps_sq"]))

        steps = []
        for _, _, st in items:
            step = st["step"] + 1
            st["step"] = step
            steps.append(step)
        grads = [g if g.is_contiguous() else g.contiguous() for _, g, _ in items]
        if sr:                      # a part of a tensor draws the counters of its elements in the whole tensor
            for i, (_, _, st) in enumerate(items):
                first = pcs[i].elem0 if pcs[i] is not None else 0
                cols["sr_base"][i] = (sr_base(self._sr_seed(st), steps[i]) + first) & 0xFFFFFFFFFFFFFFFF
        cache = {}
        uniform = steps.count(steps[0]) == n          # the usual case: every tensor of the group is at the same step
        for i in ([0] if uniform else range(n)):
            step = steps[i]
            got = cache.get(step)
            if got is None:
                got = cache[step] = row_values(step)
            sc, vals = got
            where = slice(None) if uniform else i
            for k, v in zip(_FULLRANK_COLS, vals):
                cols[k][where] = v
            if scale is not None:
                scale["rho"][where] = sc["rho"]
                scale["eps2"][where] = f32(sc["eps2"])
                scale["weight_decay"][where] = f32(group["weight_decay"])
                if sc["bc_mul"] is not None:
                    scale["bc"][where], scale["bc_mode"][where] = sc["bc_mul"], 1
                elif sc["bc_div"] is not None:
                    scale["bc"][where], scale["bc_mode"][where] = sc["bc_div"], 2
        d, fira, lag = float(group["d"]), bool(group.get("enable_fira_for_adafactor", False)), bool(group.get("lag_norm", False))
        return (fullrank_exchanges(scale is not None, d, fira, bool(plan.cfg.momentum_only), lag), device,
                plan.stages(grads, cols, d=d, fira=fira, fira_margin=float(group.get("fira_margin", 0.01)), scale=scale, lag=lag))
