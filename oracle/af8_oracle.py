"""ctypes front end of the CPU oracle (af8_oracle.c) plus the host-side scalar
logic of the reference's per-parameter update, restated with numpy float32.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
benchmark's CPU-baseline leg.  The shipped package never imports this module.

The state of one parameter is a plain dict that uses the reference's own key
names (optimizer.py:1711-1773): ``step``, ``variance_q`` / ``variance_scale`` /
``variance_min_log`` or ``variance``; ``m_q`` / ``m_scale`` or ``m``;
``row_var_*`` / ``col_var_*`` / ``conf_row_*`` / ``conf_col_*``;
``fira_prev_norm``.  Arrays are numpy; AL16 codes are uint16 (the reference
stores the same bit pattern in int16, optimizer.py:323-324).
"""
import ctypes
import math
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_BUILD = os.path.join(_HERE, "_build")
_LIB_PATH = os.path.join(_BUILD, "libaf8_oracle.so")
_SRC = os.path.join(_HERE, "af8_oracle.c")

LOG_QUANT_FLOOR = 1.17549435e-38  # optimizer.py:23

V_FMT = {"fp32": 0, "al8": 8, "al16": 16, "none": 1}
M_FMT = {None: 0, "uf8": 1, "uf4": 2, "d8": 3, "d4": 4, "fp32": 5}
G_F32, G_BF16, G_F16 = 0, 1, 2
P_FMT = {"f32": G_F32, "bf16": G_BF16, "f16": G_F16}

f32 = np.float32
c_f = ctypes.c_float
c_i = ctypes.c_int32
c_l = ctypes.c_int64
c_p = ctypes.c_void_p


def build(force=False):
    """Compile af8_oracle.c into oracle/_build/libaf8_oracle.so with gcc."""
    os.makedirs(_BUILD, exist_ok=True)
    if (not force and os.path.exists(_LIB_PATH)
            and os.path.getmtime(_LIB_PATH) >= os.path.getmtime(_SRC)):
        return _LIB_PATH
    cmd = ["gcc", "-O2", "-fopenmp", "-ffp-contract=off", "-fno-fast-math",
           "-fvisibility=hidden", "-shared", "-fPIC", "-o", _LIB_PATH, _SRC, "-lm"]
    subprocess.run(cmd, check=True)
    return _LIB_PATH


class FullrankCfg(ctypes.Structure):
    _fields_ = [
        ("numel", c_l), ("block", c_l), ("m_block", c_l),
        ("grad_dtype", c_i), ("v_fmt", c_i), ("m_fmt", c_i), ("negate_grad", c_i),
        ("use_adam_denom", c_i), ("momentum_only", c_i), ("fira", c_i), ("has_decay", c_i),
        ("decay", c_f), ("alpha", c_f), ("v_w", c_f), ("v_keep", c_f), ("v_eps_add", c_f),
        ("m_w", c_f), ("eps_gradsq", c_f), ("eps_denom", c_f), ("eps_sq", c_f),
        ("d", c_f), ("sqrt_n", c_f), ("clip_div", c_f), ("fira_margin1", c_f),
        ("v_floor", c_f),
    ]


_lib = None


def lib():
    global _lib
    if _lib is None:
        path = build() if os.path.exists(_SRC) else _LIB_PATH
        _lib = ctypes.CDLL(path)
        _lib.af8o_fira_scale.restype = c_f
        _lib.af8o_fira_scale.argtypes = [c_f, c_f, ctypes.POINTER(c_i), ctypes.POINTER(c_f)]
        _lib.af8o_norm2.restype = c_f
        _lib.af8o_norm2.argtypes = [c_p, c_l]
        _lib.af8o_al_quantize.argtypes = [c_p, c_l, c_l, c_f, c_i, c_p, c_p, c_p]
        _lib.af8o_al_dequantize.argtypes = [c_p, c_p, c_p, c_l, c_l, c_i, c_p]
        _lib.af8o_m_quantize.argtypes = [c_p, c_l, c_l, c_i, c_p, c_p, c_p]
        _lib.af8o_m_dequantize.argtypes = [c_p, c_p, c_l, c_l, c_i, c_p, c_p]
        _lib.af8o_fullrank_step.argtypes = [ctypes.POINTER(FullrankCfg)] + [c_p] * 10 + [
            ctypes.POINTER(c_i), ctypes.POINTER(c_f), ctypes.POINTER(c_f)]
        _lib.af8o_set_param_format.argtypes = [c_i, c_i, ctypes.c_uint64, ctypes.c_uint64]
        _lib.af8o_set_lag.argtypes = [c_i, c_f, c_f]
        _lib.af8o_sr_uniform.restype = c_f
        _lib.af8o_sr_uniform.argtypes = [ctypes.c_uint64] * 3
        for fn in (_lib.af8o_sr_bf16, _lib.af8o_sr_f16):
            fn.restype = ctypes.c_uint16
            fn.argtypes = [c_f, c_f]
    return _lib


def _ptr(a):
    return None if a is None else a.ctypes.data_as(c_p)


def num_threads():
    return lib().af8o_num_threads()


def set_num_threads(n):
    lib().af8o_set_num_threads(int(n))


# ---------------------------------------------------------------------------
# codecs
# ---------------------------------------------------------------------------
def al_quantize(x, block, bits=8, floor_log=-126.0):
    """_log_quantize_nonneg (optimizer.py:299-325) -> (q, scale, min_log, pad)."""
    x = np.ascontiguousarray(x, dtype=f32).reshape(-1)
    n = x.size
    nblocks = (n + block - 1) // block
    q = np.zeros(nblocks * block, dtype=np.uint16 if bits == 16 else np.uint8)
    scale = np.zeros(nblocks, dtype=f32)
    min_log = np.zeros(nblocks, dtype=f32)
    rc = lib().af8o_al_quantize(_ptr(x), n, block, floor_log, bits, _ptr(q), _ptr(scale), _ptr(min_log))
    assert rc == 0
    return q, scale, min_log, nblocks * block - n


def al_dequantize(q, scale, min_log, n, bits=8):
    """_log_dequantize_nonneg (optimizer.py:328-353)."""
    q = np.ascontiguousarray(q).reshape(-1)
    block = q.size // scale.size
    out = np.empty(n, dtype=f32)
    rc = lib().af8o_al_dequantize(_ptr(q), _ptr(scale), _ptr(min_log), n, block, bits, _ptr(out))
    assert rc == 0
    return out


def dynamic_map(total_bits):
    """_create_dynamic_map(signed=True, ...) (optimizer.py:416-441) for the two
    codebooks the reference uses (optimizer.py:122-123): 8 bits with 7 exponent
    bits, 4 bits with 3 exponent bits."""
    max_exponent_bits = 7 if total_bits == 8 else 3
    non_sign_bits = total_bits - 1
    additional_items = 2 ** (non_sign_bits - max_exponent_bits) - 1
    data = []

    def linspace32(n):
        # torch.linspace(0.1, 1, n, dtype=float32): symmetric evaluation from
        # both ends with a float32 step.
        start, end = f32(0.1), f32(1.0)
        step = f32((end - start) / f32(n - 1))
        out = np.empty(n, dtype=f32)
        half = n // 2
        for i in range(n):
            out[i] = start + step * f32(i) if i < half else end - step * f32(n - i - 1)
        return out

    for i in range(max_exponent_bits):
        fraction_items = int(2 ** (i + non_sign_bits - max_exponent_bits) + 1)
        b = linspace32(fraction_items)
        means = (b[:-1] + b[1:]) / f32(2.0)
        mult = f32(10 ** (-(max_exponent_bits - 1) + i))
        data += [float(v) for v in (mult * means)]
        data += [float(v) for v in (-mult * means)]
    if additional_items > 0:
        b = linspace32(additional_items + 1)
        means = (b[:-1] + b[1:]) / f32(2.0)
        data += [float(v) for v in means]
        data += [float(v) for v in (-means)]
    data.append(0.0)
    data.append(1.0)
    assert len(data) == 2 ** total_bits
    data.sort()
    return np.asarray(data, dtype=f32)


_MAPS = {}


def set_dynamic_map(bits, values):
    """Use `values` (the codebook a caller built on this host) instead of the
    numpy restatement above, which can differ from torch.linspace by an ulp."""
    arr = np.ascontiguousarray(values, dtype=f32)
    assert arr.size == 2 ** bits
    _MAPS[bits] = arr


def _map_for(fmt):
    if fmt in ("d8", "d4"):
        bits = 8 if fmt == "d8" else 4
        if bits not in _MAPS:
            _MAPS[bits] = dynamic_map(bits)
        return _MAPS[bits]
    return None


def m_quantize(m, block, fmt="uf8"):
    """_m_quantize (optimizer.py:547-552) -> (q, scale)."""
    m = np.ascontiguousarray(m, dtype=f32).reshape(-1)
    n = m.size
    nblocks = (n + block - 1) // block
    nbytes = nblocks * block // (2 if fmt in ("uf4", "d4") else 1)
    q = np.zeros(nbytes, dtype=np.uint8)
    scale = np.zeros(nblocks, dtype=f32)
    mp = _map_for(fmt)
    rc = lib().af8o_m_quantize(_ptr(m), n, block, M_FMT[fmt], _ptr(mp), _ptr(q), _ptr(scale))
    assert rc == 0
    return q, scale


def m_dequantize(q, scale, n, block, fmt="uf8"):
    """_m_dequantize (optimizer.py:555-560)."""
    out = np.empty(n, dtype=f32)
    mp = _map_for(fmt)
    rc = lib().af8o_m_dequantize(_ptr(q), _ptr(scale), n, block, M_FMT[fmt], _ptr(mp), _ptr(out))
    assert rc == 0
    return out


def fira_scale(norm, margin, prev):
    """_compute_fira_scale (optimizer.py:760-782) -> (scale, new_prev)."""
    has = c_i(0 if prev is None else 1)
    pv = c_f(0.0 if prev is None else float(prev))
    fs = lib().af8o_fira_scale(float(f32(norm)), float(f32(1.0 + margin)), ctypes.byref(has), ctypes.byref(pv))
    return f32(fs), f32(pv.value)


# ---------------------------------------------------------------------------
# hyper-parameters and state initialisation
# ---------------------------------------------------------------------------
# constructor defaults (optimizer.py:1313-1360)
DEFAULTS = dict(
    lr=1e-2, beta1=None, beta2=None, beta2_decay=-0.8, beta3=None, eps_came=1e-16,
    eps=(1e-30, 1e-3), weight_decay=0.0, d=1.0, maximize=False,
    relative_step=True, scale_parameter=True, factored=True,
    quantize=True, block_size=2048, m_block_size=256, m_quant_type="uf8",
    v_quant_type="al8", c_quant_type=None, min_8bit_size=4096,
    apollo_rank=0, apollo_update_proj_gap=200, apollo_scale_type="channel",
    apollo_scale=1.0, apollo_scale_front=False, apollo_eps=1e-6,
    apollo_factorize=False, apollo_cache_proj=False, enable_fira_for_apollo=True,
    scale_weight_decay=True, enable_fira_for_adafactor=False, fira_margin=0.01,
    lag_norm=False, momentum_only_1d=None, bias_correction=None,
    stochastic_round_writeback=False,
    param_dtype="f32",      # not a constructor option: the dtype of the parameter tensors of the run
)


def hyper(**kw):
    hp = dict(DEFAULTS)
    hp.update(kw)
    return hp


def _init_al(state, prefix, numel, block, fmt):
    """_init_v_state (optimizer.py:389-401)."""
    if fmt == "fp32":
        state[prefix] = np.zeros(numel, dtype=f32)
        return
    pad = (block - numel % block) % block
    nblocks = (numel + pad) // block
    state[prefix + "_q"] = np.zeros(numel + pad, dtype=np.uint8 if fmt == "al8" else np.uint16)
    state[prefix + "_scale"] = np.ones(nblocks, dtype=f32)
    state[prefix + "_min_log"] = np.zeros(nblocks, dtype=f32)
    state[prefix + "_pad"] = pad


def _init_m(state, numel, m_block, fmt, prefix="m"):
    """_m_init_state (optimizer.py:574-590)."""
    if fmt == "fp32":
        state[prefix] = np.zeros(numel, dtype=f32)
    else:
        padded = ((numel + m_block - 1) // m_block) * m_block
        if fmt in ("uf4", "d4"):
            state[prefix + "_q"] = np.full(padded // 2, 0x88 if fmt == "uf4" else 0x77, dtype=np.uint8)
        else:
            state[prefix + "_q"] = np.full(padded, 128 if fmt == "uf8" else 127, dtype=np.uint8)
        state[prefix + "_scale"] = np.ones(padded // m_block, dtype=f32)
        state["m_block_size"] = m_block
    state["m_quant_type"] = fmt


def init_state(shape, hp):
    """First-step branch of _init_group (optimizer.py:1711-1773) for the
    non-SGD paths."""
    shape = tuple(shape)
    numel = int(np.prod(shape)) if shape else 1
    use_quant = hp["quantize"] and not (numel < hp["min_8bit_size"])
    vqt = hp["v_quant_type"]
    cqt = hp["c_quant_type"] or vqt
    st = {"step": 0, "is_quantized": use_quant, "block_size": hp["block_size"],
          "v_quant_type": vqt, "c_quant_type": cqt, "shape": shape}
    use_apollo = hp["apollo_rank"] > 0 and len(shape) >= 2
    factored = len(shape) >= 2 and hp["factored"]
    if is_sgd(hp):
        # optimizer.py:1719-1725: only the momentum, quantised or fp32
        if hp["beta1"] is not None:
            _init_m(st, numel, hp["m_block_size"], hp["m_quant_type"] if use_quant else "fp32")
        return st
    v_fmt = vqt if use_quant else "fp32"
    c_fmt = cqt if use_quant else "fp32"
    m_fmt = hp["m_quant_type"] if use_quant else "fp32"
    if use_apollo:
        # optimizer.py:1726-1739; the seed is assigned by the caller in first-step order
        gap = hp["apollo_update_proj_gap"]
        st.update(apollo_seed=None, apollo_rank=hp["apollo_rank"], apollo_update_proj_gap=gap,
                  last_proj_step=-gap, apollo_proj_matrix_T=None, m_quant_type=hp["m_quant_type"])
        return st
    if factored:
        R, C = shape[-2], shape[-1]
        batch = numel // (R * C)           # more than two dimensions: a batch of matrices (optimizer.py:1750-1760)
        _init_al(st, "row_var", batch * R, hp["block_size"], v_fmt)
        _init_al(st, "col_var", batch * C, hp["block_size"], v_fmt)
        if hp["beta1"] is not None:
            _init_m(st, numel, hp["m_block_size"], m_fmt)
        if hp["beta3"] is not None:
            _init_al(st, "conf_row", batch * R, hp["block_size"], c_fmt)
            _init_al(st, "conf_col", batch * C, hp["block_size"], c_fmt)
    else:
        _init_al(st, "variance", numel, hp["block_size"], v_fmt)
        if hp["beta1"] is not None:
            _init_m(st, numel, hp["m_block_size"], m_fmt)
    return st


def is_sgd(hp):
    """SGD mode: neither beta2 nor beta2_decay (optimizer.py:1957)."""
    return hp["beta2"] is None and hp["beta2_decay"] is None


class param_format:
    """Context: the parameter array of the step calls inside holds the exact values of a bf16 /
    fp16 parameter; writes round to that format, to nearest or stochastically with the
    per-parameter seed (state["sr_seed"], optimizer.py:1889-1892) and the step number."""

    def __init__(self, hp, state, step):
        self.args = (P_FMT[hp.get("param_dtype", "f32")], int(bool(hp.get("stochastic_round_writeback", False))),
                     int(state.get("sr_seed", 0)), int(step))

    def __enter__(self):
        lib().af8o_set_param_format(*self.args)

    def __exit__(self, *exc):
        lib().af8o_set_param_format(G_F32, 0, 0, 0)


class lag_mode:
    """Context for lag_norm=True as the reference's CUDA dispatcher defines it (optimizer.py:1056-1071;
    the pure-PyTorch path ignores the flag, so this part of the oracle restates the dispatcher and the
    kernels' step-size rule, kernels.cu:651-656, and has no fixture behind it).  Inside, a step call
    clips with state["prev_update_norm"] and scales alpha by state["lag_fira_scale"]; `finish`
    stores this step's norm and advances the limiter."""

    def __init__(self, state, hp, active):
        self.state, self.hp, self.active = state, hp, active

    def __enter__(self):
        if self.active:
            lib().af8o_set_lag(1, float(self.state.get("prev_update_norm", 0.0)), float(self.state.get("lag_fira_scale", 1.0)))
        return self

    def __exit__(self, *exc):
        lib().af8o_set_lag(0, 0.0, 1.0)

    def finish(self, norm, fira):
        if not self.active:
            return
        self.state["prev_update_norm"] = f32(norm)
        if fira:
            n = f32(norm) if np.isfinite(norm) else f32(0.0)
            fs, new_prev = fira_scale(n, self.hp["fira_margin"], self.state.get("fira_prev_norm"))
            self.state["lag_fira_scale"] = fs
            self.state["fira_prev_norm"] = new_prev


def sr_round(x, rnd, fmt):
    """Stochastic rounding of binary32 values with given uniform numbers -> uint16 bit patterns."""
    fn = lib().af8o_sr_bf16 if fmt == "bf16" else lib().af8o_sr_f16
    return np.array([fn(float(a), float(b)) for a, b in zip(np.asarray(x, f32).reshape(-1), np.asarray(rnd, f32).reshape(-1))],
                    dtype=np.uint16)


def sr_uniform(seed, step, idx):
    return f32(lib().af8o_sr_uniform(int(seed), int(step), int(idx)))


def _grad_args(g):
    g = np.ascontiguousarray(g)
    if g.dtype == np.uint16:
        return g, G_BF16
    if g.dtype == np.float16:
        return g, G_F16
    assert g.dtype == f32
    return g, G_F32


def prologue(p, state, hp):
    """Per-step host scalars of _update_param_8bit (optimizer.py:1957-2040) and
    _compute_alpha (optimizer.py:832-856), rounded to float32 where the
    reference's 0-d float32 tensors round."""
    eps1, eps2 = hp["eps"]
    if eps1 is None:
        eps1 = 1e-30
    beta1, beta2, beta3 = hp["beta1"], hp["beta2"], hp["beta3"]
    factored = hp["factored"]
    eps_sq = max(eps1 * eps1, LOG_QUANT_FLOOR)
    use_adam_denom = (not factored) and (beta2 is not None) and (beta3 is None)
    eps_for_denom = eps1 if use_adam_denom else 0.0
    eps_for_grad_sq = eps1 if not use_adam_denom else 0.0
    momentum_only = hp["momentum_only_1d"]
    if momentum_only is None:
        momentum_only = not use_adam_denom
    step = state["step"] + 1
    state["step"] = step
    sgd = is_sgd(hp)
    if sgd:
        beta_val = 0.0
    else:
        beta_val = 1.0 - beta2 if beta2 is not None else math.pow(step, hp["beta2_decay"])
    lr = hp["lr"]
    rho = f32(min(lr, 1.0 / math.sqrt(step)) if hp["relative_step"] else lr)
    if hp["scale_parameter"]:
        n = p.size
        rms = f32(lib().af8o_norm2(_ptr(p), n)) / f32(math.sqrt(n))
        alpha = f32(max(rms, f32(eps2))) * rho
    else:
        alpha = rho
    if beta1 is not None and not hp["relative_step"] and not sgd:
        apply_bc = use_adam_denom if hp["bias_correction"] is None else hp["bias_correction"]
        if apply_bc:
            bc1 = 1.0 - beta1 ** step
            if beta2 is not None:
                bc2 = 1.0 - beta2 ** step
                alpha = f32(alpha * f32(math.sqrt(bc2) / bc1))
                if use_adam_denom:
                    eps_for_denom = eps1 * math.sqrt(bc2)
            else:
                alpha = f32(alpha / f32(bc1))
    decay = None
    if hp["weight_decay"] != 0:
        wd_mult = alpha if hp["scale_weight_decay"] else rho
        decay = f32(f32(1.0) - f32(wd_mult * f32(hp["weight_decay"])))
    return dict(step=step, beta_val=beta_val, alpha=f32(alpha), rho=rho, decay=decay,
                eps1=eps1, eps_sq=eps_sq, use_adam_denom=use_adam_denom,
                eps_for_denom=eps_for_denom, eps_for_grad_sq=eps_for_grad_sq,
                momentum_only=momentum_only)


def fullrank_step(p, g, state, hp, sc=None):
    """Full-rank branch of _update_param_8bit (optimizer.py:2076-2194).
    p: float32 array updated in place; g: float32, or uint16 holding bf16 bits."""
    assert p.dtype == f32 and p.flags.c_contiguous
    if sc is None:
        sc = prologue(p, state, hp)
    n = p.size
    g, gdt = _grad_args(g)
    quant = state["is_quantized"]
    vqt = state["v_quant_type"] if quant else "fp32"
    sgd = is_sgd(hp)
    if sgd:
        vqt = "none"
    has_m = hp["beta1"] is not None
    mqt = (("fp32" if "m" in state else state.get("m_quant_type", "uf8")) if has_m else None)
    cfg = FullrankCfg()
    cfg.numel = n
    cfg.block = state["block_size"]
    cfg.m_block = state.get("m_block_size", hp["m_block_size"])
    cfg.grad_dtype = gdt
    cfg.v_fmt = V_FMT[vqt]
    cfg.m_fmt = M_FMT[mqt]
    cfg.negate_grad = int(bool(hp["maximize"]))
    cfg.use_adam_denom = int(sc["use_adam_denom"])
    cfg.momentum_only = int(sc["momentum_only"])
    cfg.fira = int(bool(hp["enable_fira_for_adafactor"]))
    cfg.has_decay = int(sc["decay"] is not None)
    cfg.decay = float(sc["decay"]) if sc["decay"] is not None else 1.0
    cfg.alpha = float(sc["alpha"])
    cfg.v_w = float(f32(sc["beta_val"]))
    cfg.v_keep = float(f32(1.0 - hp["beta1"])) if (sgd and has_m) else float(f32(1.0 - sc["beta_val"]))
    cfg.v_eps_add = float(f32(sc["beta_val"] * sc["eps_for_grad_sq"]))
    cfg.m_w = float(f32(1.0 - hp["beta1"])) if has_m else 0.0
    cfg.eps_gradsq = float(f32(sc["eps_for_grad_sq"]))
    cfg.eps_denom = float(f32(sc["eps_for_denom"]))
    cfg.eps_sq = float(f32(sc["eps_sq"]))
    cfg.d = float(f32(hp["d"]))
    cfg.sqrt_n = float(f32(math.sqrt(n)))
    cfg.clip_div = float(f32(math.sqrt(n) * hp["d"]))
    cfg.fira_margin1 = float(f32(1.0 + hp["fira_margin"]))
    cfg.v_floor = -126.0
    has_prev = c_i(1 if "fira_prev_norm" in state else 0)
    prev = c_f(float(state.get("fira_prev_norm", 0.0)))
    norm = c_f(-1.0)
    lag = lag_mode(state, hp, bool(hp["lag_norm"]) and (cfg.fira or hp["d"] > 0) and not (cfg.momentum_only and has_m))
    with param_format(hp, state, sc["step"]), lag:
        rc = lib().af8o_fullrank_step(
            ctypes.byref(cfg), _ptr(p.reshape(-1)), _ptr(g.reshape(-1)),
            _ptr(state.get("variance_q")), _ptr(state.get("variance_scale")),
            _ptr(state.get("variance_min_log")), _ptr(state.get("variance")),
            _ptr(state.get("m_q")), _ptr(state.get("m_scale")), _ptr(state.get("m")),
            _ptr(_map_for(mqt)), ctypes.byref(has_prev), ctypes.byref(prev), ctypes.byref(norm))
    if rc != 0:
        raise RuntimeError(f"af8o_fullrank_step failed with {rc}")
    if lag.active:
        lag.finish(norm.value, bool(cfg.fira))
    elif has_prev.value:
        state["fira_prev_norm"] = f32(prev.value)
    return float(norm.value)


# ---------------------------------------------------------------------------
# factored path
# ---------------------------------------------------------------------------
class SmallState(ctypes.Structure):
    _fields_ = [("q", c_p), ("scale", c_p), ("min_log", c_p), ("f32", c_p), ("n", c_l),
                ("fmt", c_i), ("pad_", c_i)]


class FactoredCfg(ctypes.Structure):
    _fields_ = [
        ("rows", c_l), ("cols", c_l), ("block", c_l), ("m_block", c_l),
        ("grad_dtype", c_i), ("m_fmt", c_i), ("came", c_i), ("negate_grad", c_i),
        ("fira", c_i), ("has_decay", c_i),
        ("decay", c_f), ("alpha", c_f), ("v_w", c_f), ("m_w", c_f), ("c_w", c_f),
        ("eps1", c_f), ("eps_came", c_f), ("d", c_f), ("sqrt_n", c_f), ("clip_div", c_f),
        ("fira_margin1", c_f), ("v_floor", c_f),
    ]


def _small(state, prefix, n, fmt):
    s = SmallState()
    s.n = n
    s.fmt = V_FMT[fmt]
    if fmt == "fp32":
        s.f32 = _ptr(state[prefix])
    else:
        s.q = _ptr(state[prefix + "_q"])
        s.scale = _ptr(state[prefix + "_scale"])
        s.min_log = _ptr(state[prefix + "_min_log"])
    return s


def factored_step(p, g, state, hp, sc=None):
    """Factored branch of _update_param_8bit (optimizer.py:2202-2552, pure route); a tensor of more
    than two dimensions is a batch of matrices over its last two."""
    assert p.dtype == f32 and p.ndim >= 2 and p.flags.c_contiguous
    lib_ = lib()
    if not hasattr(lib_, "_factored_ready"):
        lib_.af8o_factored_step.argtypes = [ctypes.POINTER(FactoredCfg), c_p, c_p] + \
            [ctypes.POINTER(SmallState)] * 4 + [c_p, c_p, c_p, c_p, ctypes.POINTER(c_i),
                                                ctypes.POINTER(c_f), ctypes.POINTER(c_f)]
        lib_._factored_ready = True
    if sc is None:
        sc = prologue(p, state, hp)
    R, C = p.shape[-2:]
    n = p.size
    B = n // (R * C)
    g, gdt = _grad_args(g)
    quant = state["is_quantized"]
    vqt = state["v_quant_type"] if quant else "fp32"
    cqt = state["c_quant_type"] if quant else "fp32"
    has_m = hp["beta1"] is not None
    mqt = ("fp32" if "m" in state else state.get("m_quant_type", "uf8")) if has_m else None
    came = hp["beta3"] is not None and has_m
    cfg = FactoredCfg()
    cfg.rows, cfg.cols = R, C
    cfg.block = state["block_size"]
    cfg.m_block = state.get("m_block_size", hp["m_block_size"])
    cfg.grad_dtype = gdt
    cfg.m_fmt = M_FMT[mqt]
    cfg.came = int(came)
    cfg.negate_grad = int(bool(hp["maximize"]))
    cfg.fira = int(bool(hp["enable_fira_for_adafactor"]))
    cfg.has_decay = int(sc["decay"] is not None)
    cfg.decay = float(sc["decay"]) if sc["decay"] is not None else 1.0
    cfg.alpha = float(sc["alpha"])
    cfg.v_w = float(f32(sc["beta_val"]))
    cfg.m_w = float(f32(1.0 - hp["beta1"])) if has_m else 0.0
    cfg.c_w = float(f32(1.0 - hp["beta3"])) if came else 0.0
    cfg.eps1 = float(f32(sc["eps1"]))
    cfg.eps_came = float(f32(hp["eps_came"]))
    cfg.d = float(f32(hp["d"]))
    cfg.sqrt_n = float(f32(math.sqrt(n)))
    cfg.clip_div = float(f32(math.sqrt(n) * hp["d"]))
    cfg.fira_margin1 = float(f32(1.0 + hp["fira_margin"]))
    cfg.v_floor = -126.0
    row = _small(state, "row_var", B * R, vqt)
    col = _small(state, "col_var", B * C, vqt)
    crow = _small(state, "conf_row", B * R, cqt) if came else SmallState()
    ccol = _small(state, "conf_col", B * C, cqt) if came else SmallState()
    has_prev = c_i(1 if "fira_prev_norm" in state else 0)
    prev = c_f(float(state.get("fira_prev_norm", 0.0)))
    norm = c_f(-1.0)
    lag = lag_mode(state, hp, bool(hp["lag_norm"]) and (cfg.fira or hp["d"] > 0) and not came)
    lib_.af8o_factored_set_batch.argtypes = [c_l]
    lib_.af8o_factored_set_batch(B)
    with param_format(hp, state, sc["step"]), lag:
        rc = lib_.af8o_factored_step(
            ctypes.byref(cfg), _ptr(p), _ptr(g.reshape(-1)), ctypes.byref(row), ctypes.byref(col),
            ctypes.byref(crow), ctypes.byref(ccol), _ptr(state.get("m_q")), _ptr(state.get("m_scale")),
            _ptr(state.get("m")), _ptr(_map_for(mqt)), ctypes.byref(has_prev), ctypes.byref(prev),
            ctypes.byref(norm))
    if rc != 0:
        raise RuntimeError(f"af8o_factored_step failed with {rc}")
    if lag.active:
        lag.finish(norm.value, bool(cfg.fira))
    elif has_prev.value:
        state["fira_prev_norm"] = f32(prev.value)
    return float(norm.value)


# ---------------------------------------------------------------------------
# APOLLO
# ---------------------------------------------------------------------------
class ApolloCfg(ctypes.Structure):
    _fields_ = [
        ("rows", c_l), ("cols", c_l), ("rank", c_l), ("block", c_l), ("m_block", c_l),
        ("grad_dtype", c_i), ("v_fmt", c_i), ("m_fmt", c_i), ("negate_grad", c_i), ("first_step", c_i),
        ("scale_tensor", c_i), ("scale_front", c_i), ("fira", c_i), ("has_decay", c_i),
        ("decay", c_f), ("alpha", c_f), ("bc", c_f), ("bc_mode", c_i), ("v_w", c_f), ("m_w", c_f),
        ("apollo_eps", c_f), ("sqrt_scale", c_f), ("d", c_f), ("clip_div", c_f), ("fira_margin1", c_f),
        ("v_floor_first", c_f), ("v_floor_later", c_f),
    ]


def stable_randn(shape, seed):
    """stable_randn on the CPU generator (optimizer.py:139-149)."""
    import torch
    gen = torch.Generator(device="cpu").manual_seed(int(seed))
    return torch.randn(tuple(shape), generator=gen, device="cpu", dtype=torch.float32)


def next_seed(seed, adv=0xF):
    """next_seed (optimizer.py:152-155)."""
    import torch
    gen = torch.Generator().manual_seed(int(seed))
    return torch.randint(0, torch.iinfo(torch.int64).max, (adv,), generator=gen).tolist()[-1]


def apollo_projection(state, shape, step, rank, gap):
    """_get_apollo_proj_matrix (optimizer.py:2557-2584) -> proj_matrix_T as a numpy array."""
    last = int(state.get("last_proj_step", -gap))
    refresh = (step - last) >= gap
    if not refresh and state.get("apollo_proj_matrix_T") is not None:
        return state["apollo_proj_matrix_T"]
    if refresh:
        state["current_proj_seed"] = int(state["apollo_seed"])
        state["apollo_seed"] = next_seed(state["current_proj_seed"])
        state["last_proj_step"] = step
    R, C = shape
    m_shape = (rank, C) if R >= C else (R, rank)
    seed = state.get("current_proj_seed", state["apollo_seed"])
    proj = stable_randn(m_shape, seed) / math.sqrt(rank)
    pt = proj.T.contiguous().numpy().copy()
    state["apollo_proj_matrix_T"] = pt
    return pt


class ApolloExtra(ctypes.Structure):
    _fields_ = [("factorize", c_i), ("came", c_i), ("c_fmt", c_i), ("first_factor", c_i),
                ("v_keep", c_f), ("c_w", c_f), ("eps_came", c_f), ("eps_sq", c_f), ("d", c_f), ("reserved", c_f),
                ("row_var_low", c_p), ("col_var_low", c_p),
                ("conf_row", SmallState), ("conf_col", SmallState), ("res", SmallState)]


def apollo_step(p, g, state, hp, g_low=None):
    """_update_param_apollo (optimizer.py:2587-3084) for 2-D fp32 parameters: the plain rule,
    apollo_factorize (2688-2760) and CAME over the projected gradient (2801-2903, the
    pure-PyTorch branch).  g_low: a projected gradient (float32, rows x rank or
    rank x cols) to use instead of computing G @ Pt: everything after the contraction then
    starts from the same values as a device run whose projection was copied here."""
    assert p.dtype == f32 and p.ndim == 2 and p.flags.c_contiguous
    lib_ = lib()
    if not hasattr(lib_, "_apollo_ready"):
        lib_.af8o_apollo_step.argtypes = [ctypes.POINTER(ApolloCfg)] + [c_p] * 11 + [
            ctypes.POINTER(c_i), ctypes.POINTER(c_f), ctypes.POINTER(c_f)]
        lib_._apollo_ready = True
    R, C = p.shape
    n = R * C
    rank = int(hp["apollo_rank"])
    step = state["step"] + 1
    state["step"] = step
    beta1, beta2 = hp["beta1"], hp["beta2"]
    beta_val = 1.0 - beta2 if beta2 is not None else math.pow(step, hp["beta2_decay"])
    lr = hp["lr"]
    rho = f32(min(lr, 1.0 / math.sqrt(step)) if hp["relative_step"] else lr)
    if hp["scale_parameter"]:
        rms = f32(lib_.af8o_norm2(_ptr(p), n)) / f32(math.sqrt(n))
        alpha = f32(max(rms, f32(hp["eps"][1]))) * rho
    else:
        alpha = rho
    pt = apollo_projection(state, (R, C), step, rank, int(hp["apollo_update_proj_gap"]))
    g, gdt = _grad_args(g)
    quant = state["is_quantized"]
    vqt = state["v_quant_type"] if quant else "fp32"
    has_m = beta1 is not None
    mqt = (state.get("m_quant_type", "uf8") if quant else "fp32") if has_m else None
    nl = max(R, C) * rank
    block = state["block_size"]
    m_block = state.get("m_block_size", hp["m_block_size"])
    factorize = bool(hp.get("apollo_factorize", False))
    beta3 = hp.get("beta3")
    first = state.get("v_low_q") is None and state.get("v_low") is None
    extra = None
    if factorize or beta3 is not None:
        LR, LC = (R, rank) if R >= C else (rank, C)
        cqt = (state.get("c_quant_type", state["v_quant_type"]) if quant else "fp32")
        extra = ApolloExtra()
        extra.factorize, extra.came = int(factorize), int(beta3 is not None)
        extra.c_fmt = V_FMT[cqt]
        extra.v_keep = float(f32(1.0 - beta_val))
        extra.c_w = float(f32(1.0 - beta3)) if beta3 is not None else 0.0
        extra.eps_came = float(f32(hp["eps_came"]))
        extra.eps_sq = float(f32(max(hp["apollo_eps"] * hp["apollo_eps"], LOG_QUANT_FLOOR)))
        extra.d = float(f32(hp["d"]))
        if factorize:
            extra.first_factor = int("row_var_low" not in state)
            if extra.first_factor:
                state["row_var_low"] = np.zeros(LR, dtype=f32)
                state["col_var_low"] = np.zeros(LC, dtype=f32)
            extra.row_var_low, extra.col_var_low = _ptr(state["row_var_low"]), _ptr(state["col_var_low"])
            if has_m and beta3 is not None:
                if state.get("conf_row_low_q") is None and state.get("conf_row_low") is None:
                    _init_al(state, "conf_row_low", LR, block, cqt)
                    _init_al(state, "conf_col_low", LC, block, cqt)
                extra.conf_row = _small(state, "conf_row_low", LR, cqt)
                extra.conf_col = _small(state, "conf_col_low", LC, cqt)
        elif has_m:
            if state.get("res_low_q") is None and state.get("res_low") is None:
                _init_al(state, "res_low", nl, block, cqt)
            extra.res = _small(state, "res_low", nl, cqt)
    if factorize:
        first = False                 # no v_low state in this mode
    elif first:
        if vqt == "fp32":
            state["v_low"] = np.zeros(nl, dtype=f32)
        else:
            _init_al(state, "v_low", nl, block, vqt)
    if has_m and state.get("m_low_q") is None and state.get("m_low") is None:
        _init_m(state, nl, m_block, mqt, prefix="m_low")
    cfg = ApolloCfg()
    cfg.rows, cfg.cols, cfg.rank, cfg.block, cfg.m_block = R, C, rank, block, m_block
    cfg.grad_dtype, cfg.v_fmt, cfg.m_fmt = gdt, V_FMT[vqt], M_FMT[mqt]
    cfg.negate_grad = int(bool(hp["maximize"]))
    cfg.first_step = int(first)
    cfg.scale_tensor = int(hp["apollo_scale_type"] == "tensor")
    cfg.scale_front = int(bool(hp["apollo_scale_front"]))
    cfg.fira = int(bool(hp["enable_fira_for_apollo"]))
    wd = hp["weight_decay"]
    cfg.has_decay = int(wd != 0)
    mult = alpha if hp["scale_weight_decay"] else rho
    cfg.decay = float(f32(f32(1.0) - f32(mult * f32(wd)))) if wd != 0 else 1.0
    cfg.alpha = float(alpha)
    cfg.bc_mode, cfg.bc = 0, 1.0
    if has_m and not hp["relative_step"]:
        apply_bc = True if hp["bias_correction"] is None else hp["bias_correction"]
        if apply_bc:
            bc1 = 1.0 - beta1 ** step
            if beta2 is not None:
                cfg.bc_mode, cfg.bc = 1, float(f32(math.sqrt(1.0 - beta2 ** step) / bc1))
            else:
                cfg.bc_mode, cfg.bc = 2, float(f32(bc1))
    cfg.v_w = float(f32(beta_val))
    cfg.m_w = float(f32(1.0 - beta1)) if has_m else 0.0
    cfg.apollo_eps = float(f32(hp["apollo_eps"]))
    cfg.sqrt_scale = float(f32(math.sqrt(hp["apollo_scale"])))
    cfg.d = float(f32(hp["d"]))
    cfg.clip_div = float(f32(math.sqrt(n) * hp["d"]))
    cfg.fira_margin1 = float(f32(1.0 + hp["fira_margin"]))
    cfg.v_floor_first = -126.0
    cfg.v_floor_later = float(f32(math.log2(max(hp["apollo_eps"] * hp["apollo_eps"], LOG_QUANT_FLOOR))))
    has_prev = c_i(1 if "scaled_grad_norm_prev" in state else 0)
    prev = c_f(float(state.get("scaled_grad_norm_prev", 0.0)))
    norm = c_f(-1.0)
    if g_low is not None:
        g_low = np.ascontiguousarray(g_low, dtype=f32).reshape(-1)
        assert g_low.size == nl
        lib_.af8o_apollo_override_g_low.argtypes = [c_p]
        lib_.af8o_apollo_override_g_low(_ptr(g_low))
    if extra is not None:
        lib_.af8o_apollo_set_extra.argtypes = [ctypes.POINTER(ApolloExtra)]
        lib_.af8o_apollo_set_extra(ctypes.byref(extra))
    with param_format(hp, state, state["step"]):
        rc = lib_.af8o_apollo_step(
            ctypes.byref(cfg), _ptr(p), _ptr(g.reshape(-1)), _ptr(pt),
            _ptr(state.get("v_low_q")), _ptr(state.get("v_low_scale")), _ptr(state.get("v_low_min_log")),
            _ptr(state.get("v_low")), _ptr(state.get("m_low_q")), _ptr(state.get("m_low_scale")), _ptr(state.get("m_low")),
            _ptr(_map_for(mqt)), ctypes.byref(has_prev), ctypes.byref(prev), ctypes.byref(norm))
    if rc != 0:
        raise RuntimeError(f"af8o_apollo_step failed with {rc}")
    if has_prev.value:
        state["scaled_grad_norm_prev"] = f32(prev.value)
    return float(norm.value)


# ---------------------------------------------------------------------------
# state migration when a group option changes between steps
# ---------------------------------------------------------------------------
def _al_keys(prefix):
    return [prefix + s for s in ("_q", "_scale", "_min_log", "_pad")]


def _to_al(state, prefix, x, block, fmt):
    """_quant_v (optimizer.py:373-377)."""
    q, s, ml, pad = al_quantize(np.ascontiguousarray(x, dtype=f32).reshape(-1), block, bits=8 if fmt == "al8" else 16)
    state[prefix + "_q"], state[prefix + "_scale"], state[prefix + "_min_log"], state[prefix + "_pad"] = q, s, ml, pad


def _from_al(state, prefix):
    """_deq_v(..., pop=True) (optimizer.py:358-365)."""
    q = state.pop(prefix + "_q")
    s, ml, pad = state.pop(prefix + "_scale"), state.pop(prefix + "_min_log"), state.pop(prefix + "_pad")
    return al_dequantize(q, s, ml, q.size - pad, bits=8 if q.dtype == np.uint8 else 16)


def migrate_state(state, hp, shape):
    """What _init_group does to an existing state at the start of a step (optimizer.py:1650-1860,
    976-1045) for the full-rank and factored paths: momentum reset on a momentum-format change,
    re-initialisation (step kept) on a V / C / block change or a factored-mode change, in-place
    conversion on a `quantize` change, CAME's confidence states dropped or created with beta3.
    Returns the state to use (a new dict after a re-initialisation)."""
    shape = tuple(shape)
    numel = int(np.prod(shape)) if shape else 1
    use_quant = hp["quantize"] and not (numel < hp["min_8bit_size"])
    block, m_block = hp["block_size"], hp["m_block_size"]
    mqt, vqt = hp["m_quant_type"], hp["v_quant_type"]
    cqt = hp["c_quant_type"] or vqt
    beta1, beta3 = hp["beta1"], hp["beta3"]
    expect_factored = len(shape) >= 2 and hp["factored"]

    def reinit():
        new = init_state(shape, hp)
        new["step"] = state.get("step", 0)
        if "sr_seed" in state:
            new["sr_seed"] = state["sr_seed"]
        return new

    old_mqt = state.get("m_quant_type", "uf8")
    old_mbs = state.get("m_block_size", m_block)
    if (old_mqt != mqt or old_mbs != m_block) and use_quant:
        for k in ("m_q", "m_scale", "m_block_size", "m"):
            state.pop(k, None)
        state["m_quant_type"] = mqt
    old_vqt = state.get("v_quant_type", "al8")
    old_cqt = state.get("c_quant_type", old_vqt)
    if (old_vqt != vqt or old_cqt != cqt or state.get("block_size", block) != block) and use_quant:
        return reinit()
    if not is_sgd(hp) and (("row_var" in state or "row_var_q" in state) != expect_factored):
        return reinit()

    cur_block = state.get("block_size", block)
    was_quant = state.get("is_quantized", False)
    if use_quant and not was_quant:
        if vqt != "fp32":
            for k in ("row_var", "col_var", "variance"):
                if k in state and k + "_q" not in state:
                    _to_al(state, k, state.pop(k), cur_block, vqt)
        if cqt != "fp32" and beta3 is not None:
            for k in ("conf_row", "conf_col"):
                if k in state and k + "_q" not in state:
                    _to_al(state, k, state.pop(k), cur_block, cqt)
        if beta1 is not None and "m_q" not in state and mqt != "fp32":
            mb = state.get("m_block_size", m_block)
            if "m" in state:
                state["m_q"], state["m_scale"] = m_quantize(state.pop("m"), mb, mqt)
                state["m_quant_type"] = mqt
            else:
                _init_m(state, numel, mb, mqt)
            state["m_block_size"] = mb
        state["is_quantized"] = True
    elif not use_quant and was_quant:
        for k in ("row_var", "col_var", "conf_row", "conf_col", "variance"):
            if k + "_q" in state:
                state[k] = _from_al(state, k)
        if "m_q" in state:
            mb = state.get("m_block_size", m_block)
            state["m"] = m_dequantize(state["m_q"], state["m_scale"], numel, mb, state.get("m_quant_type", "uf8"))
            for k in ("m_q", "m_scale", "m_block_size", "m_quant_type"):
                state.pop(k, None)
        state["is_quantized"] = False

    if beta3 is None:
        for prefix in ("conf_row", "conf_col"):
            state.pop(prefix, None)
            for k in _al_keys(prefix):
                state.pop(k, None)
    elif expect_factored:
        c_fmt = cqt if use_quant else "fp32"
        if "conf_row" not in state and "conf_row_q" not in state:
            _init_al(state, "conf_row", shape[-2], cur_block, c_fmt)
        if "conf_col" not in state and "conf_col_q" not in state:
            _init_al(state, "conf_col", shape[-1], cur_block, c_fmt)
    if beta1 is not None and "m_q" not in state:
        mb = state.get("m_block_size", m_block)
        if use_quant and mqt != "fp32":
            if "m" in state:
                state["m_q"], state["m_scale"] = m_quantize(state.pop("m"), mb, mqt)
                state["m_quant_type"] = mqt
            else:
                _init_m(state, numel, mb, mqt)
            state["m_block_size"] = mb
        elif "m" not in state and mqt == "fp32":
            _init_m(state, numel, mb, "fp32")
    if beta1 is None:
        for k in ("m_q", "m_scale", "m_block_size", "m_quant_type", "m"):
            state.pop(k, None)
    return state
