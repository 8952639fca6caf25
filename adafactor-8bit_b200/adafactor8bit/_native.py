"""ctypes binding of libaf8 (include/af8.h): the only way this package reaches
the GPU.  There is no fallback: if the library is missing or a call fails, a
RuntimeError is raised.

The table structs of the C ABI are mirrored as numpy structured dtypes so that
a whole table can be filled with vectorised assignments.
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_DEFAULT_LIB = os.path.join(os.path.dirname(_HERE), "lib", "libaf8.so")

OK, ERR_INVALID, ERR_UNSUPPORTED, ERR_CUDA = 0, 1, 2, 3
F32, BF16, F16 = 0, 1, 2
V_FP32, V_AL8, V_AL16 = 0, 8, 16
M_NONE, M_UF8, M_UF4, M_D8, M_D4, M_FP32 = 0, 1, 2, 3, 4, 5
MODE_NOCLIP, MODE_SUMSQ, MODE_APPLY, MODE_SUMSQ_M, MODE_LAG = 0, 1, 2, 3, 4

V_NONE = 1
V_FMT = {"fp32": V_FP32, "al8": V_AL8, "al16": V_AL16, "none": V_NONE}
M_FMT = {None: M_NONE, "uf8": M_UF8, "uf4": M_UF4, "d8": M_D8, "d4": M_D4, "fp32": M_FP32}

_P = np.uint64   # device / host pointers inside tables

FULLRANK_TENSOR = np.dtype([
    ("param", _P), ("grad", _P), ("v_q", _P), ("v_scale", _P), ("v_min_log", _P), ("v_f32", _P),
    ("m_q", _P), ("m_scale", _P), ("m_f32", _P),
    ("numel", np.int64), ("first_block", np.int64),
    ("decay", np.float32), ("alpha", np.float32), ("v_w", np.float32), ("v_keep", np.float32),
    ("v_eps_add", np.float32), ("m_w", np.float32), ("eps_gradsq", np.float32),
    ("eps_denom", np.float32), ("eps_sq", np.float32), ("reserved", np.float32),
    ("sr_base", np.uint64), ("param_copy", _P),
], align=True)
assert FULLRANK_TENSOR.itemsize == 144

DYN_SCALARS = np.dtype([
    ("step", np.float32), ("fira", np.float32), ("pre_div", np.float32), ("zero", np.float32),
    ("norm", np.float32), ("reserved", np.float32, (3,)),
], align=True)
assert DYN_SCALARS.itemsize == 32

NORM_TENSOR = np.dtype([
    ("first_block", np.int64), ("n_blocks", np.int64), ("fira_prev", _P),
    ("fira_has_prev", np.int32), ("pre_div_mode", np.int32),
    ("alpha", np.float32), ("clip_div", np.float32), ("sqrt_n", np.float32), ("d", np.float32),
    ("fira_margin1", np.float32), ("partials_f64", np.int32), ("alpha_dev", _P),
], align=True)
assert NORM_TENSOR.itemsize == 64

LAG_TENSOR = np.dtype([
    ("first_block", np.int64), ("n_blocks", np.int64), ("prev_update_norm", _P), ("lag_fira_scale", _P),
    ("fira_prev", _P), ("alpha_dev", _P), ("alpha", np.float32), ("clip_div", np.float32), ("fira_margin1", np.float32),
    ("has_lag_fira", np.int32), ("fira_has_prev", np.int32), ("partials_f64", np.int32), ("reserved", np.int32, (2,)),
], align=True)      # af8_lag_tensor
assert LAG_TENSOR.itemsize == 80

APOLLO_PROJ_DESC = np.dtype([(n, np.uint64) for n in ("grad", "pt", "g_low", "chan_g2", "workspace")] +
                            [(n, np.int64) for n in ("workspace_bytes", "rows", "cols", "rank")] +
                            [("negate", np.int32), ("planes_valid", np.int32)], align=True)     # af8_apollo_proj_desc, 80 B

APOLLO_FINISH_TENSOR = np.dtype(
    [(n, np.uint64) for n in ("upd", "g_low", "chan_g2", "sf", "sums", "fira_prev", "out")] +
    [(n, np.int64) for n in ("rows", "cols", "rank", "first_unit")] +
    [(n, np.float32) for n in ("alpha", "bc", "d", "clip_div", "fira_margin1", "sqrt_scale")] +
    [(n, np.int32) for n in ("bc_mode", "fira", "fira_has_prev", "scale_tensor", "scale_front", "in_reserved")] +
    [("alpha_decay", np.uint64)], align=True)     # af8_apollo_finish_tensor, 144 B

APOLLO_APPLY_TENSOR = np.dtype(
    [(n, np.uint64) for n in ("param", "grad", "sf", "scalars", "param_copy")] +
    [(n, np.int64) for n in ("rows", "cols", "first_chunk")] + [("sr_base", np.uint64)] +
    [(n, np.float32) for n in ("sqrt_scale", "decay")] +
    [(n, np.int32) for n in ("scale_tensor", "fira", "scale_front", "has_decay", "stochastic_round", "reserved")],
    align=True)     # af8_apollo_apply_tensor, 104 B

SMALL_STATE = np.dtype([
    ("q", _P), ("scale", _P), ("min_log", _P), ("f32", _P), ("fmt", np.int32), ("block", np.int32),
], align=True)
assert SMALL_STATE.itemsize == 40

FACTORED_TENSOR = np.dtype([
    ("param", _P), ("grad", _P), ("m_q", _P), ("m_scale", _P), ("m_f32", _P),
    ("row_sum", _P), ("col_sum", _P), ("inv_row", _P), ("inv_col", _P),
    ("inv_row_conf", _P), ("inv_col_conf", _P),
    ("row_var", SMALL_STATE), ("col_var", SMALL_STATE), ("conf_row", SMALL_STATE), ("conf_col", SMALL_STATE),
    ("rows", np.int64), ("cols", np.int64), ("first_chunk", np.int64), ("first_tile", np.int64),
    ("decay", np.float32), ("alpha", np.float32), ("v_w", np.float32), ("m_w", np.float32),
    ("c_w", np.float32), ("eps1", np.float32), ("eps_came", np.float32), ("first_small", np.int32),
    ("sr_base", np.uint64), ("param_copy", _P), ("batch_rows", np.int64),
], align=True)
assert FACTORED_TENSOR.itemsize == 336

SCALE_TENSOR = np.dtype([
    ("param", _P), ("numel", np.int64), ("first_chunk", np.int64),
    ("sqrt_n", np.float32), ("rho", np.float32), ("eps2", np.float32), ("bc", np.float32),
    ("weight_decay", np.float32), ("bc_mode", np.int32), ("scale_weight_decay", np.int32),
    ("param_dtype", np.int32), ("total", _P),
], align=True)
assert SCALE_TENSOR.itemsize == 64


class FullrankCfg(ctypes.Structure):
    _fields_ = [
        ("param_dtype", ctypes.c_int32), ("grad_dtype", ctypes.c_int32),
        ("v_fmt", ctypes.c_int32), ("m_fmt", ctypes.c_int32),
        ("block", ctypes.c_int32), ("m_block", ctypes.c_int32),
        ("use_adam_denom", ctypes.c_int32), ("momentum_only", ctypes.c_int32),
        ("negate_grad", ctypes.c_int32), ("mode", ctypes.c_int32),
        ("v_floor", ctypes.c_float), ("stochastic_round", ctypes.c_int32),
    ]


class FactoredCfg(ctypes.Structure):
    _fields_ = [
        ("param_dtype", ctypes.c_int32), ("grad_dtype", ctypes.c_int32), ("m_fmt", ctypes.c_int32),
        ("m_block", ctypes.c_int32), ("came", ctypes.c_int32), ("negate_grad", ctypes.c_int32),
        ("mode", ctypes.c_int32), ("v_floor", ctypes.c_float),
        ("aligned8", ctypes.c_int32), ("stochastic_round", ctypes.c_int32), ("total_tiles", ctypes.c_int64),
        ("cols_mult256", ctypes.c_int32), ("reserved", ctypes.c_int32),
    ]


class ApolloScalarsIn(ctypes.Structure):
    _fields_ = [
        ("alpha", ctypes.c_float), ("bc", ctypes.c_float), ("d", ctypes.c_float), ("clip_div", ctypes.c_float),
        ("fira_margin1", ctypes.c_float), ("sqrt_scale", ctypes.c_float),
        ("bc_mode", ctypes.c_int32), ("fira", ctypes.c_int32), ("fira_has_prev", ctypes.c_int32),
        ("scale_tensor", ctypes.c_int32), ("scale_front", ctypes.c_int32), ("reserved", ctypes.c_int32),
    ]


class ApolloRuleState(ctypes.Structure):
    _fields_ = [("q", ctypes.c_void_p), ("scale", ctypes.c_void_p), ("min_log", ctypes.c_void_p), ("f32", ctypes.c_void_p),
                ("n", ctypes.c_int64), ("fmt", ctypes.c_int32), ("reserved", ctypes.c_int32)]


class ApolloRule(ctypes.Structure):
    _fields_ = [
        ("g_low", ctypes.c_void_p), ("upd", ctypes.c_void_p), ("work", ctypes.c_void_p), ("work_bytes", ctypes.c_int64),
        ("lr_rows", ctypes.c_int64), ("lr_cols", ctypes.c_int64),
        ("factorize", ctypes.c_int32), ("came", ctypes.c_int32), ("m_fmt", ctypes.c_int32), ("m_block", ctypes.c_int32),
        ("block", ctypes.c_int32), ("first_factor", ctypes.c_int32), ("first_v", ctypes.c_int32), ("reserved", ctypes.c_int32),
        ("v_w", ctypes.c_float), ("v_keep", ctypes.c_float), ("m_w", ctypes.c_float), ("c_w", ctypes.c_float),
        ("eps_came", ctypes.c_float), ("eps_sq", ctypes.c_float), ("apollo_eps", ctypes.c_float), ("d", ctypes.c_float),
        ("v_floor_later", ctypes.c_float), ("reserved2", ctypes.c_float),
        ("row_var_low", ctypes.c_void_p), ("col_var_low", ctypes.c_void_p),
        ("m_q", ctypes.c_void_p), ("m_scale", ctypes.c_void_p), ("m_f32", ctypes.c_void_p),
        ("v", ApolloRuleState), ("res", ApolloRuleState), ("conf_row", ApolloRuleState), ("conf_col", ApolloRuleState),
    ]


FSTAT_GRADSQ, FSTAT_RESIDUAL = 0, 1
FUPD_SUMSQ_U, FUPD_SUMSQ, FUPD_APPLY, FUPD_LAG = 0, 1, 2, 3

_c_p = ctypes.c_void_p
_c_i = ctypes.c_int32
_c_l = ctypes.c_int64
_c_f = ctypes.c_float

# name -> (restype, argtypes); every symbol that include/af8.h declares
PROTOTYPES = {
    "af8_version": (_c_i, []),
    "af8_last_error": (ctypes.c_char_p, []),
    "af8_struct_size": (ctypes.c_int32, [ctypes.c_int32]),
    "af8_device_status": (_c_i, [ctypes.POINTER(ctypes.c_int32), _c_p]),
    "af8_device_status_clear": (_c_i, [_c_p]),
    "af8_selftest_bounded_wait": (_c_i, [_c_p, _c_l, _c_p, _c_p]),
    "af8_set_qmap": (_c_i, [_c_p, _c_p, _c_p]),
    "af8_fullrank_step": (_c_i, [ctypes.POINTER(FullrankCfg), _c_p, _c_p, _c_i, _c_l, _c_p, _c_p, _c_p]),
    "af8_fullrank_upload": (_c_i, [ctypes.POINTER(FullrankCfg), _c_p, _c_p, _c_i, _c_l, _c_p]),
    "af8_factored_chunk": (_c_i, [_c_i]),
    "af8_factored_tile_rows": (_c_i, []),
    "af8_factored_tile_cols": (_c_i, []),
    "af8_factored_upload": (_c_i, [ctypes.POINTER(FactoredCfg), _c_p, _c_p, _c_i, _c_p]),
    "af8_factored_stats": (_c_i, [ctypes.POINTER(FactoredCfg), _c_p, _c_p, _c_i, _c_p, _c_p]),
    "af8_factored_stats_boxes": (_c_i, [ctypes.POINTER(FactoredCfg), _c_p, _c_p, _c_i, _c_p, _c_p, _c_p, _c_p]),
    "af8_factored_small": (_c_i, [ctypes.POINTER(FactoredCfg), _c_p, _c_i, _c_i, _c_i, _c_p]),
    "af8_factored_update": (_c_i, [ctypes.POINTER(FactoredCfg), _c_p, _c_i, _c_l, _c_p, _c_p, _c_p]),
    "af8_apollo_project": (_c_i, [_c_p, _c_i, _c_i, _c_p, _c_l, _c_l, _c_l, _c_p, _c_p, _c_p]),
    "af8_apollo_project_workspace": (ctypes.c_int64, [_c_l, _c_l, _c_l]),
    "af8_apollo_project_ws": (_c_i, [_c_p, _c_i, _c_i, _c_p, _c_l, _c_l, _c_l, _c_p, _c_p, _c_p, _c_l, _c_p]),
    "af8_apollo_project_task_bytes": (ctypes.c_int32, []),
    "af8_apollo_project_batch": (_c_i, [_c_p, _c_i, _c_i, _c_p, _c_p, _c_p, _c_l, _c_p]),
    "af8_apollo_scales_batch": (_c_i, [_c_p, _c_p, _c_i, _c_l, _c_p]),
    "af8_apollo_scales": (_c_i, [_c_p, _c_p, _c_p, _c_l, _c_l, _c_l, ctypes.POINTER(ApolloScalarsIn), _c_p, _c_p, _c_p,
                                 _c_p, _c_p, _c_p]),
    "af8_apollo_apply": (_c_i, [_c_p, _c_i, _c_i, ctypes.c_uint64, _c_p, _c_i, _c_i, _c_p, _c_p, _c_l, _c_l,
                                ctypes.POINTER(ApolloScalarsIn), _c_f, _c_i, _c_p, _c_p]),
    "af8_apollo_apply_batch": (_c_i, [_c_p, _c_p, _c_i, _c_l, _c_i, _c_i, _c_i, _c_p]),
    "af8_apollo_rule_workspace": (ctypes.c_int64, [_c_l, _c_l]),
    "af8_apollo_rule_step": (_c_i, [ctypes.POINTER(ApolloRule), _c_p]),
    "af8_norm_finalize": (_c_i, [_c_p, _c_i, _c_p, _c_p, _c_p]),
    "af8_lag_scalars": (_c_i, [_c_p, _c_i, _c_i, _c_p, _c_p, _c_p]),
    "af8_fullrank_limited_step_noalloc": (_c_i, [ctypes.POINTER(FullrankCfg), _c_p, _c_f, _c_i, _c_f, _c_p, _c_i, _c_p, _c_p]),
    "af8_noalloc_max_numel": (_c_l, [_c_i]),
    "af8_param_scale": (_c_i, [_c_p, _c_p, _c_i, _c_p, _c_p, _c_l, _c_l, _c_l, _c_p]),
    "af8_param_sumsq": (_c_i, [_c_p, _c_p, _c_i, _c_p, _c_p]),
    "af8_param_scale_finish": (_c_i, [_c_p, _c_i, _c_p, _c_p, _c_l, _c_l, _c_l, _c_p]),
    "af8_scale_chunk": (_c_i, []),
    "af8_al_dequant": (_c_i, [_c_p, _c_p, _c_p, _c_l, _c_i, _c_i, _c_p, _c_p]),
    "af8_al_quant": (_c_i, [_c_p, _c_l, _c_i, _c_i, _c_f, _c_p, _c_p, _c_p, _c_p]),
    "af8_m_dequant": (_c_i, [_c_p, _c_p, _c_l, _c_i, _c_i, _c_p, _c_p]),
    "af8_m_quant": (_c_i, [_c_p, _c_l, _c_i, _c_i, _c_p, _c_p, _c_p]),
}

_lib = None


def library_path():
    return os.environ.get("AF8_LIBRARY", _DEFAULT_LIB)


def lib():
    """Load libaf8.so once.  Raises RuntimeError when it cannot be loaded."""
    global _lib
    if _lib is None:
        path = library_path()
        if not os.path.exists(path):
            raise RuntimeError(
                f"libaf8.so not found at {path}; build it with "
                f"`python adafactor-8bit_b200/build.py` (this package has no CPU or PyTorch fallback)")
        try:
            handle = ctypes.CDLL(path)
        except OSError as e:  # missing libcudart and the like
            raise RuntimeError(f"cannot load {path}: {e}") from e
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        # the mirrors of this module against the structures the library was compiled with
        mirrors = [FULLRANK_TENSOR.itemsize, DYN_SCALARS.itemsize, ctypes.sizeof(FullrankCfg), NORM_TENSOR.itemsize,
                   SCALE_TENSOR.itemsize, SMALL_STATE.itemsize, FACTORED_TENSOR.itemsize, ctypes.sizeof(FactoredCfg),
                   ctypes.sizeof(ApolloScalarsIn), 16, APOLLO_PROJ_DESC.itemsize, APOLLO_FINISH_TENSOR.itemsize,
                   LAG_TENSOR.itemsize, ctypes.sizeof(ApolloRule), APOLLO_APPLY_TENSOR.itemsize]
        for i, mine in enumerate(mirrors):
            theirs = handle.af8_struct_size(i)
            if theirs != mine:
                raise RuntimeError(f"{path}: structure {i} is {theirs} bytes in the library, {mine} in this binding; "
                                   f"rebuild the library")
        _lib = handle
    return _lib


def check(rc, what):
    if rc != OK:
        msg = lib().af8_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"{what} failed (code {rc}): {msg}")


def device_status(stream=None):
    """Synchronise `stream` (a raw cudaStream_t or None) and return the sticky device error flag."""
    out = ctypes.c_int32(0)
    check(lib().af8_device_status(ctypes.byref(out), stream), "af8_device_status")
    return out.value


def clear_device_status(stream=None):
    check(lib().af8_device_status_clear(stream), "af8_device_status_clear")


def version():
    return lib().af8_version()
