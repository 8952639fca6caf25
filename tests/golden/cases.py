"""Case definitions and seeded input generators shared by the golden-vector
generator (gen_golden.py, which runs the reference) and by the parity tests.

Everything here is plain numpy so that the same inputs can be rebuilt on a
machine that has neither the reference nor a GPU.  Each fixture stores a digest
of the inputs it was generated from; a test that rebuilds different bytes
fails instead of comparing against the wrong vectors.
"""
import hashlib

import numpy as np

f32 = np.float32


def f32_to_bf16_bits(x):
    """Round-to-nearest-even float32 -> bfloat16, returned as uint16 bit patterns."""
    u = np.ascontiguousarray(x, dtype=f32).view(np.uint32).astype(np.uint64)
    rounded = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return rounded.astype(np.uint16)


def bf16_bits_to_f32(h):
    return (h.astype(np.uint32) << 16).view(f32)


def make_param(shape, seed, std=0.02, dtype="f32"):
    """Initial parameter values as float32; for a bf16 / f16 parameter they are rounded to that
    format first, so the float32 array holds the parameter exactly."""
    rng = np.random.Generator(np.random.PCG64(seed))
    p = (rng.standard_normal(shape, dtype=np.float64) * std).astype(f32)
    if dtype == "bf16":
        p = bf16_bits_to_f32(f32_to_bf16_bits(p)).reshape(shape)
    elif dtype == "f16":
        p = p.astype(np.float16).astype(f32)
    return p


def sr_uniform(seed, step, n):
    """The n uniform numbers that stochastic rounding draws for the elements of one parameter at
    one step: SplitMix64 finaliser of a counter made of the parameter's seed, the step and the
    element index; the top 24 of its upper 32 bits scaled to [0, 1)."""
    m64 = (1 << 64) - 1
    base = (int(seed) * 0x9E3779B97F4A7C15 + int(step) * 0xD1B54A32D192ED03 + 0x9E3779B97F4A7C15) & m64
    with np.errstate(over="ignore"):
        z = np.arange(n, dtype=np.uint64) + np.uint64(base)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    return ((z >> np.uint64(40)).astype(f32) * f32(1.0 / 16777216.0)).astype(f32)


def make_grad(shape, seed, step, spec):
    """spec keys: dist ('normal' | 'rowscale'), std, zero_frac, dtype ('f32' | 'bf16'),
    spike_step / spike_mult (optional)."""
    rng = np.random.Generator(np.random.PCG64([seed, step]))
    g = rng.standard_normal(shape, dtype=np.float64) * spec["std"]
    if spec.get("dist") == "rowscale" and len(shape) >= 2:
        rows = rng.standard_normal(shape[:-1] + (1,), dtype=np.float64)
        g = g * np.exp(rows)
    elif spec.get("dist") == "rowscale":
        g = g * np.exp(rng.standard_normal((), dtype=np.float64))
    zf = spec.get("zero_frac", 0.0)
    if zf > 0:
        g = np.where(rng.random(shape) < zf, 0.0, g)
    if spec.get("spike_step") == step:
        g = g * spec.get("spike_mult", 100.0)
    g = g.astype(f32)
    if spec.get("dtype", "f32") == "bf16":
        return f32_to_bf16_bits(g)
    if spec.get("dtype") == "f16":
        return g.astype(np.float16)
    return g


def sr_edge_inputs():
    """-> (x, rnd): every edge value paired with every uniform number."""
    vals = np.array([0.0, -0.0, 1.0, 1.0 + 2.0 ** -9, -1.0 - 2.0 ** -9, 1.0 + 2.0 ** -8, 1.0 + 2.0 ** -11, 1.0 + 3 * 2.0 ** -12,
                     3.3895313892515355e38, 3.39e38, 3.4028234663852886e38, -3.4e38, np.inf, -np.inf, np.nan, -np.nan,
                     65504.0, 65505.0, 65519.0, 65520.0, 1e5, -1e5, 6e-8, -6e-8, 2.0 ** -25, 1e-10, -1e-10, 1e-45, 0.1, -0.3,
                     6.1e-5, 6.097e-5], dtype=f32)
    u = np.array([0.0, 0.1, 0.25, 0.5, 0.75, 0.9, 0.99999994], dtype=f32)
    return np.repeat(vals, u.size).copy(), np.tile(u, vals.size).copy()


def digest(arrays):
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


_ADAMW = dict(beta1=0.9, beta2=0.999, beta2_decay=None, beta3=None, factored=False,
              relative_step=False, scale_parameter=False, scale_weight_decay=False,
              d=0.0, eps=(1e-8, 1e-3))
_CAME = dict(beta1=0.9, beta2=0.999, beta2_decay=None, beta3=0.9999, factored=True,
             relative_step=False, scale_parameter=False, scale_weight_decay=False,
             d=1.0, eps_came=1e-16)
_SGD = dict(beta1=None, beta2=None, beta2_decay=None, beta3=None, factored=False, relative_step=False,
            scale_parameter=False, scale_weight_decay=False, d=0.0)
_RMSPROP = dict(beta1=None, beta2=0.99, beta2_decay=None, beta3=None, factored=False,
                relative_step=False, scale_parameter=False, scale_weight_decay=False,
                d=0.0, eps=(1e-8, 1e-3))
_APOLLO = dict(beta1=0.9, beta2=0.999, beta2_decay=None, beta3=None, factored=False,
               relative_step=False, scale_parameter=False, scale_weight_decay=False,
               d=0.0, eps=(1e-6, 1e-3), apollo_eps=1e-6, apollo_factorize=False,
               apollo_scale_type="channel", apollo_scale=1.0, apollo_scale_front=False,
               apollo_cache_proj=True, enable_fira_for_apollo=True)

_G_CFG0 = dict(dist="normal", std=1e-2, zero_frac=0.01, dtype="f32")
_G_HEAVY = dict(dist="rowscale", std=1e-3, zero_frac=0.005, dtype="bf16")
_G_BF16 = dict(dist="rowscale", std=1e-3, zero_frac=0.0, dtype="bf16")

# name -> dict(shapes, hp, grad, steps, seed)
CASES = {
    # AdamW UF8 (block 256) / AL8 (block 2048), fp32 grads with 1 % exact zeros.
    "adamw_uf8_al8": dict(shapes=[(64, 200), (4096,)], steps=10, seed=11, grad=_G_CFG0,
                          hp=dict(_ADAMW, lr=1e-3, weight_decay=0.01, block_size=2048,
                                  m_block_size=256, m_quant_type="uf8", v_quant_type="al8")),
    # same optimizer + Fira limiter, bf16 heavy-tailed grads, x100 spike on step 5.
    "adamw_fira_bf16": dict(shapes=[(96, 200), (2048,)], steps=10, seed=12,
                            grad=dict(_G_HEAVY, spike_step=5, spike_mult=100.0),
                            hp=dict(_ADAMW, lr=1e-3, weight_decay=0.01, block_size=2048,
                                    m_block_size=256, m_quant_type="uf8", v_quant_type="al8",
                                    enable_fira_for_adafactor=True, fira_margin=0.01)),
    # other state formats on the full-rank path.
    "adamw_uf4_al16": dict(shapes=[(40, 130)], steps=4, seed=13, grad=_G_CFG0,
                           hp=dict(_ADAMW, lr=1e-3, weight_decay=0.01, block_size=1024,
                                   m_block_size=128, m_quant_type="uf4", v_quant_type="al16")),
    "adamw_d8_al8": dict(shapes=[(40, 130)], steps=4, seed=14, grad=_G_CFG0,
                         hp=dict(_ADAMW, lr=1e-3, block_size=2048, m_block_size=256,
                                 m_quant_type="d8", v_quant_type="al8")),
    "adamw_d4_al8": dict(shapes=[(40, 130)], steps=4, seed=15, grad=_G_CFG0,
                         hp=dict(_ADAMW, lr=1e-3, block_size=2048, m_block_size=256,
                                 m_quant_type="d4", v_quant_type="al8")),
    "adamw_fp32m_al8": dict(shapes=[(40, 130)], steps=4, seed=16, grad=_G_CFG0,
                            hp=dict(_ADAMW, lr=1e-3, block_size=2048, m_block_size=256,
                                    m_quant_type="fp32", v_quant_type="al8")),
    "rmsprop_al8": dict(shapes=[(40, 130)], steps=4, seed=17, grad=_G_CFG0,
                        hp=dict(_RMSPROP, lr=1e-3, block_size=256)),
    # SGD mode (neither beta2 nor beta2_decay): quantised momentum, clipping and the limiter
    "sgd_momentum_uf8": dict(shapes=[(40, 130), (4096,)], steps=4, seed=23, grad=_G_CFG0,
                             hp=dict(_SGD, beta1=0.9, lr=1e-2, weight_decay=0.01, d=1.0, block_size=256,
                                     enable_fira_for_adafactor=True, min_8bit_size=1024)),
    # plain SGD, bf16 gradients, no momentum, no clipping
    "sgd_plain_bf16": dict(shapes=[(40, 130)], steps=3, seed=24, grad=_G_BF16, hp=dict(_SGD, lr=1e-2, block_size=256)),
    # unfactored Adafactor (relative step, parameter scaling, clip d=1).
    "adafactor_unfactored": dict(shapes=[(40, 130), (300,)], steps=4, seed=18, grad=_G_HEAVY,
                                 hp=dict(factored=False, block_size=256)),
    # factored Adafactor, constructor defaults, AL8 block 256, no momentum.
    "adafactor_factored": dict(shapes=[(320, 192), (64, 384), (2048,)], steps=10, seed=19,
                               grad=_G_HEAVY, hp=dict(block_size=256)),
    # factored Adafactor with quantised momentum.
    "adafactor_factored_m": dict(shapes=[(128, 256)], steps=4, seed=20, grad=_G_HEAVY,
                                 hp=dict(block_size=256, beta1=0.9, relative_step=False,
                                         lr=1e-3)),
    # CAME: UF8 momentum, AL16 second moment and confidence, block 2048.
    "came_al16": dict(shapes=[(320, 192), (64, 384), (4096,)], steps=10, seed=21, grad=_G_BF16,
                      hp=dict(_CAME, lr=1e-4, m_quant_type="uf8", v_quant_type="al16",
                              c_quant_type="al16", block_size=2048)),
    # APOLLO rank 32, projection refreshed every 3 steps, UF8/AL8 low-rank states.
    "apollo_r32": dict(shapes=[(256, 128), (64, 384), (4096,)], steps=8, seed=22,
                       grad=dict(dist="normal", std=1e-3, zero_frac=0.0, dtype="bf16"),
                       hp=dict(_APOLLO, lr=1e-3, weight_decay=0.01, apollo_rank=32,
                               apollo_update_proj_gap=3, m_quant_type="uf8",
                               v_quant_type="al8", block_size=2048)),
    # ---- bf16 / fp16 parameters (case key param_dtype): nearest rounding on every write, or
    #      stochastic rounding fed by the counter generator of sr_uniform ----
    "adamw_bf16p": dict(shapes=[(64, 200), (4096,)], steps=6, seed=31, param_dtype="bf16",
                        grad=dict(_G_HEAVY, spike_step=4, spike_mult=100.0),
                        hp=dict(_ADAMW, lr=1e-3, weight_decay=0.01, block_size=2048, m_block_size=256,
                                enable_fira_for_adafactor=True, fira_margin=0.01)),
    "adamw_f16p": dict(shapes=[(40, 130)], steps=4, seed=32, param_dtype="f16",
                       grad=dict(dist="normal", std=1e-2, zero_frac=0.01, dtype="f16"),
                       hp=dict(_ADAMW, lr=1e-3, weight_decay=0.01, block_size=2048, m_block_size=256)),
    "adamw_sr_bf16p": dict(shapes=[(64, 200), (4096,)], steps=6, seed=33, param_dtype="bf16",
                           grad=dict(_G_HEAVY, spike_step=4, spike_mult=100.0),
                           hp=dict(_ADAMW, lr=1e-3, weight_decay=0.01, block_size=2048, m_block_size=256,
                                   enable_fira_for_adafactor=True, fira_margin=0.01, stochastic_round_writeback=True)),
    "adamw_sr_f16p": dict(shapes=[(40, 130)], steps=4, seed=34, param_dtype="f16",
                          grad=dict(dist="normal", std=1e-2, zero_frac=0.01, dtype="f16"),
                          hp=dict(_ADAMW, lr=1e-3, weight_decay=0.01, block_size=2048, m_block_size=256,
                                  stochastic_round_writeback=True)),
    "adafactor_bf16p": dict(shapes=[(320, 192), (2048,)], steps=4, seed=35, param_dtype="bf16", grad=_G_HEAVY,
                            hp=dict(block_size=256, weight_decay=0.01)),
    "came_sr_bf16p": dict(shapes=[(64, 384)], steps=4, seed=36, param_dtype="bf16", grad=_G_BF16,
                          hp=dict(_CAME, lr=1e-4, weight_decay=0.01, m_quant_type="uf8", v_quant_type="al16", c_quant_type="al16",
                                  block_size=2048, stochastic_round_writeback=True)),
}

# ---- group options edited between steps (case key `changes`: {step: {option: value}}, applied to the
#      parameter group before that step): the state migrations of _init_group (optimizer.py:1650-1860) ----
CASES.update({
    "migrate_quantize_off_on": dict(shapes=[(40, 130), (4096,)], steps=6, seed=41, grad=_G_CFG0,
                                    changes={3: {"quantize": False}, 5: {"quantize": True}},
                                    hp=dict(_ADAMW, lr=1e-3, weight_decay=0.01, block_size=2048, m_block_size=256)),
    "migrate_formats": dict(shapes=[(40, 130)], steps=6, seed=42, grad=_G_CFG0,
                            changes={3: {"m_quant_type": "uf4"}, 5: {"v_quant_type": "al16"}},
                            hp=dict(_ADAMW, lr=1e-3, weight_decay=0.01, block_size=2048, m_block_size=256)),
    "migrate_came_toggle": dict(shapes=[(64, 384)], steps=6, seed=43, grad=_G_BF16,
                                changes={3: {"beta3": None}, 5: {"beta3": 0.9999}},
                                hp=dict(_CAME, lr=1e-4, m_quant_type="uf8", v_quant_type="al8", block_size=256)),
    "migrate_factored_off": dict(shapes=[(128, 256)], steps=5, seed=44, grad=_G_HEAVY,
                                 changes={3: {"factored": False}, 5: {"quantize": False}},
                                 hp=dict(block_size=256, beta1=0.9, relative_step=False, lr=1e-3)),
})
# APOLLO with one scaling factor per tensor (apollo_scale_type="tensor") and a larger apollo_scale, rank 8
CASES["apollo_r8_tensor"] = dict(shapes=[(256, 128), (64, 384)], steps=5, seed=45,
                                 grad=dict(dist="normal", std=1e-3, zero_frac=0.0, dtype="bf16"),
                                 hp=dict(_APOLLO, lr=1e-3, weight_decay=0.01, apollo_rank=8, apollo_update_proj_gap=3,
                                         apollo_scale_type="tensor", apollo_scale=128.0, m_quant_type="uf8",
                                         v_quant_type="al8", block_size=2048))
# ragged sizes with quantised states from one element up (min_8bit_size=1): single elements, sizes one below
# and one above the M block (256) and the V block (2048), a matrix whose rows straddle blocks
CASES["adamw_ragged"] = dict(shapes=[(1,), (255,), (257,), (2047,), (2049,), (3, 700), (4097,)], steps=4, seed=46,
                             grad=dict(_G_HEAVY, spike_step=3, spike_mult=100.0),
                             hp=dict(_ADAMW, lr=1e-3, weight_decay=0.01, block_size=2048, m_block_size=256, min_8bit_size=1,
                                     enable_fira_for_adafactor=True, fira_margin=0.01))
# APOLLO on bf16 parameters: nearest rounding (mul_ / addcmul_ in place) and stochastic rounding
CASES["apollo_bf16p"] = dict(shapes=[(256, 128), (64, 384), (4096,)], steps=5, seed=47, param_dtype="bf16",
                             grad=dict(dist="normal", std=1e-3, zero_frac=0.0, dtype="bf16"),
                             hp=dict(_APOLLO, lr=1e-3, weight_decay=0.01, apollo_rank=16, apollo_update_proj_gap=3,
                                     m_quant_type="uf8", v_quant_type="al8", block_size=2048))
CASES["apollo_sr_bf16p"] = dict(CASES["apollo_bf16p"], seed=48, hp=dict(CASES["apollo_bf16p"]["hp"], stochastic_round_writeback=True))
# APOLLO with fp32 low-rank states (quantize=False: Tensor.lerp_ on both moments, momentum kept in the projected
# gradient's shape), and on a tensor of three dimensions (stepped as (shape[0], -1)) with fp16 gradients
CASES["apollo_fp32_states"] = dict(shapes=[(96, 64), (32, 160)], steps=5, seed=49,
                                   grad=dict(dist="normal", std=1e-3, zero_frac=0.0, dtype="bf16"),
                                   hp=dict(_APOLLO, lr=1e-3, weight_decay=0.01, apollo_rank=8, apollo_update_proj_gap=3,
                                           quantize=False))
CASES["apollo_3d_f16g"] = dict(shapes=[(12, 8, 16), (40, 4, 6)], steps=5, seed=50,
                               grad=dict(dist="normal", std=1e-3, zero_frac=0.0, dtype="f16"),
                               hp=dict(_APOLLO, lr=1e-3, weight_decay=0.01, apollo_rank=8, apollo_update_proj_gap=3,
                                       m_quant_type="uf8", v_quant_type="al8", block_size=256, min_8bit_size=64))
# APOLLO's further low-rank rules: factored second moment of the projected gradient (apollo_factorize), the same
# with CAME's confidence vectors, CAME over the projected gradient with its instability state shaped like it
# (quantised AL8 and fp32), and the momentum-free factorised form (beta3 without beta1 is refused by the constructor)
_APOLLO_X = dict(_APOLLO, lr=1e-3, weight_decay=0.01, apollo_rank=8, apollo_update_proj_gap=3, m_quant_type="uf8",
                 v_quant_type="al8", block_size=256, m_block_size=256, min_8bit_size=64, eps_came=1e-16)
_G_APX = dict(dist="normal", std=1e-3, zero_frac=0.0, dtype="bf16")
CASES["apollo_factorize"] = dict(shapes=[(96, 64), (32, 160)], steps=5, seed=51, grad=_G_APX,
                                 hp=dict(_APOLLO_X, apollo_factorize=True))
CASES["apollo_factorize_came"] = dict(shapes=[(96, 64), (32, 160)], steps=5, seed=52, grad=_G_APX,
                                      hp=dict(_APOLLO_X, apollo_factorize=True, beta3=0.9999, d=1.0))
CASES["apollo_came"] = dict(shapes=[(96, 64), (32, 160)], steps=5, seed=53, grad=_G_APX,
                            hp=dict(_APOLLO_X, beta3=0.9999, d=1.0))
CASES["apollo_came_fp32"] = dict(shapes=[(96, 64), (32, 160)], steps=5, seed=54, grad=_G_APX,
                                 hp=dict(_APOLLO_X, beta3=0.9999, d=1.0, quantize=False))
CASES["apollo_factorize_nomom"] = dict(shapes=[(96, 64), (32, 160)], steps=4, seed=55, grad=_G_APX,
                                       hp=dict(_APOLLO_X, apollo_factorize=True, beta1=None))
# the step size follows the parameters' RMS (scale_parameter=True), weight decay scaled with it
CASES["apollo_scale_param"] = dict(shapes=[(96, 64), (32, 160)], steps=5, seed=57, grad=_G_APX,
                                   hp=dict(_APOLLO_X, lr=1e-2, scale_parameter=True, scale_weight_decay=True))
CASES["apollo_scale_param_tensor"] = dict(shapes=[(96, 64), (32, 160)], steps=4, seed=59, grad=_G_APX,
                                          hp=dict(_APOLLO_X, lr=1e-2, scale_parameter=True, scale_weight_decay=False,
                                                  relative_step=True, apollo_scale_type="tensor"))
APOLLO_RULE_CASES = ["apollo_factorize", "apollo_factorize_came", "apollo_came", "apollo_came_fp32",
                     "apollo_factorize_nomom", "apollo_scale_param", "apollo_scale_param_tensor"]
# factored tensors of more than two dimensions: a batch of matrices over the last two dimensions, with row / column
# states whose quantisation blocks run across the batch entries (3 x 40 x 72: 120 row values, 216 column values in
# blocks of 128) -- Adafactor without and CAME with momentum
CASES["adafactor_3d"] = dict(shapes=[(3, 40, 72), (2, 2, 24, 16)], steps=5, seed=60, grad=_G_BF16,
                             hp=dict(lr=1e-3, block_size=128, min_8bit_size=64, relative_step=False, scale_parameter=True,
                                     weight_decay=0.01))
CASES["came_3d"] = dict(shapes=[(3, 40, 72), (2, 2, 24, 16)], steps=5, seed=61, grad=_G_BF16,
                        hp=dict(_CAME, lr=1e-4, m_quant_type="uf8", v_quant_type="al8", block_size=128, m_block_size=64,
                                min_8bit_size=64, enable_fira_for_adafactor=True))
# odd sizes: columns that are no multiple of 8, rows and matrices that straddle the state blocks, a momentum
CASES["adafactor_3d_odd"] = dict(shapes=[(2, 5, 12), (3, 33, 7)], steps=4, seed=62, grad=_G_CFG0,
                                 hp=dict(lr=1e-3, beta1=0.9, block_size=128, m_block_size=64, min_8bit_size=16, relative_step=False,
                                         weight_decay=0.01, d=1.0))
FACTORED_3D_CASES = ["adafactor_3d", "came_3d", "adafactor_3d_odd"]
MIGRATION_CASES = ["migrate_quantize_off_on", "migrate_formats", "migrate_came_toggle", "migrate_factored_off"]

LOWP_FULLRANK_CASES = ["adamw_bf16p", "adamw_f16p", "adamw_sr_bf16p", "adamw_sr_f16p"]
LOWP_FACTORED_CASES = ["adafactor_bf16p", "came_sr_bf16p"]


def case_inputs(name):
    """-> (params0, grads[step][i]) for a case (its name, or a dict of the same form), steps numbered from 1."""
    c = name if isinstance(name, dict) else CASES[name]
    params = [make_param(s, c["seed"] * 1000 + i, dtype=c.get("param_dtype", "f32")) for i, s in enumerate(c["shapes"])]
    grads = {}
    for t in range(1, c["steps"] + 1):
        grads[t] = [make_grad(s, c["seed"] * 1000 + 500 + i, t, c["grad"])
                    for i, s in enumerate(c["shapes"])]
    return params, grads


def inputs_digest(params, grads):
    arrays = list(params)
    for t in sorted(grads):
        arrays += grads[t]
    return digest(arrays)
