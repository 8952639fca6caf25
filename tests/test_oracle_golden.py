"""The CPU oracle against the golden vectors produced by the reference itself
(tests/golden/gen_golden.py).  This is what pins the oracle; it needs neither
the reference nor a GPU."""
import numpy as np
import pytest

import cases
import parity
from oracle_runner import FULLRANK_CASES, OracleRun, golden_entries, load_golden

CODE_KEYS = ("variance_q", "m_q", "row_var_q", "col_var_q", "conf_row_q", "conf_col_q", "v_low_q", "m_low_q")
RANGE_SUFFIXES = ("_scale", "_min_log")


def test_known_answers(oracle):
    # anchors observed on the reference's pure-PyTorch codecs (optimizer.py:299-353, 504-532)
    q, s, ml, pad = oracle.al_quantize(np.zeros(256, np.float32), 256)
    assert not q.any() and s[0] == 1.0 and abs(ml[0] + 127.23327) < 1e-5
    q, s, ml, pad = oracle.al_quantize(np.full(256, 3e-5, np.float32), 256)
    assert (q == 255).all() and abs(s[0] - 0.99999905) < 1e-7 and abs(ml[0] + 16.024677) < 1e-5
    x = np.zeros(256, np.float32); x[0] = 2.0 ** -20; x[1] = 2.0 ** -10
    q, s, ml, pad = oracle.al_quantize(x, 256)
    assert list(q[:3]) == [1, 255, 0] and s[0] == 10.0 and ml[0] == -20.0
    x = np.zeros(256, np.float32); x[0] = 1e-40; x[1] = 1.0
    q, s, ml, pad = oracle.al_quantize(x, 256)
    assert s[0] == 126.0 and ml[0] == -126.0
    q, s, ml, pad = oracle.al_quantize(np.ones(130, np.float32), 128)
    assert pad == 126 and s.size == 2
    q, s, ml, pad = oracle.al_quantize(np.ones(256, np.float32), 256, bits=16)
    assert q.dtype == np.uint16 and (q == 65535).all()      # int16 -1 in the reference
    q, s = oracle.m_quantize(np.array([0, 1, -1, 0.5, 127.4 / 128] + [0] * 251, np.float32), 256)
    assert list(q[:5]) == [128, 255, 0, 192, 255] and s[0] == 1.0
    q, s = oracle.m_quantize(np.zeros(256, np.float32), 256)
    assert (q == 128).all() and abs(s[0] - 1e-12) < 1e-18
    q, s = oracle.m_quantize(np.array([0, 1, -1, 0.5] + [0] * 28, np.float32), 32, "uf4")
    assert list(q[:2]) == [143, 12]
    m4 = oracle.dynamic_map(4)
    assert np.allclose(m4, [-0.8875, -0.6625, -0.4375, -0.2125, -0.0775, -0.0325, -0.0055, 0, 0.0055,
                            0.0325, 0.0775, 0.2125, 0.4375, 0.6625, 0.8875, 1.0], rtol=1e-6)
    m8 = oracle.dynamic_map(8)
    assert m8[127] == 0.0 and m8[-1] == 1.0 and (np.diff(m8) > 0).all()


def test_codec_round_trip(oracle):
    rng = np.random.default_rng(5)
    v = (rng.standard_normal(5000) ** 2 * 1e-6).astype(np.float32)
    v[::97] = 0.0
    for bits, rel in ((8, 0.06), (16, 3e-4)):
        q, s, ml, pad = oracle.al_quantize(v, 1024, bits=bits)
        back = oracle.al_dequantize(q, s, ml, v.size, bits=bits)
        assert ((back == 0) == (v == 0)).all()
        nz = v != 0
        assert np.max(np.abs(np.log2(back[nz]) - np.log2(v[nz]))) <= np.max(s) / (2 ** bits - 2) * 0.5 + 1e-3
        # re-encoding decoded values is idempotent on the codes
        q2, s2, ml2, _ = oracle.al_quantize(back, 1024, bits=bits)
        assert parity.code_stats(q, q2)["max"] <= 1
    m = (rng.standard_normal(4000) * 1e-3).astype(np.float32)
    for fmt in ("uf8", "uf4", "d8", "d4"):
        q, s = oracle.m_quantize(m, 256, fmt)
        back = oracle.m_dequantize(q, s, m.size, 256, fmt)
        # (not idempotent by design: +absmax saturates one level below full scale)
        assert np.max(np.abs(back - m)) <= np.max(s) * (0.13 if fmt in ("uf4", "d4") else 0.02)


@pytest.mark.parametrize("name", FULLRANK_CASES)
def test_oracle_matches_reference_golden(name, oracle):
    run = OracleRun(name)
    gold = load_golden(name)
    assert str(gold["digest"]) == cases.inputs_digest(run.params0, run.grads), \
        "seeded inputs differ from the ones the fixture was generated from"
    steps = run.case["steps"]
    for t in range(1, steps + 1):
        run.step()
        for i, (p, st) in enumerate(zip(run.params, run.states)):
            ref = golden_entries(gold, t, i)
            for key, want in ref.items():
                what = f"{name} step {t} param {i} {key}"
                if key == "param":
                    parity.assert_params(p, want, what)
                    continue
                got = st[key]
                if key in CODE_KEYS:
                    al16 = want.dtype == np.uint16
                    fmt = st.get("m_quant_type") if key.startswith("m") else None
                    if fmt in ("uf4", "d4"):
                        got, want = parity.unpack_nibbles(got), parity.unpack_nibbles(want)
                    parity.assert_codes(got, want, what, al16=al16, zero_reserved=not key.startswith("m"))
                elif key.endswith(RANGE_SUFFIXES):
                    # free-running comparison: a range may move once a code of its
                    # extreme element differs; bounded instead of exact
                    parity.assert_ranges(got, want, what, max_ulp=4)
                elif key in ("fira_prev_norm", "scaled_grad_norm_prev"):
                    # the reference measures norms with torch.linalg.vector_norm, whose
                    # float32 accumulation is off by 1e-6..1e-4 at these sizes (and by
                    # up to 5e-3 on 65 M elements); the oracle accumulates in binary64
                    assert parity.rel_l2(got, want) <= 1e-4, what
                else:
                    assert parity.rel_l2(got, want) <= 1e-6, what


# ---------------------------------------------------------------------------
# factored paths (Adafactor, CAME)
# ---------------------------------------------------------------------------
from oracle_runner import FACTORED_CASES, state_from_golden  # noqa: E402

FACTORED_CODE_KEYS = ("row_var_q", "col_var_q", "conf_row_q", "conf_col_q", "variance_q", "m_q")


def _check_step(name, t, i, p, st, ref, param_tol, al16_frac=None, range_ulp=4):
    for key, want in ref.items():
        what = f"{name} step {t} param {i} {key}"
        if key == "param":
            parity.assert_params(p, want, what, tol=param_tol)
        elif key in FACTORED_CODE_KEYS:
            al16 = want.dtype == np.uint16
            if al16 and al16_frac is not None:
                s = parity.code_stats(st[key], want)
                assert s["zero_mismatch"] == 0 and s["max"] <= parity.CODE_SLACK_AL16, (what, s)
                assert s["neq"] <= max(2, al16_frac * s["n"]), (what, s)
            else:
                parity.assert_codes(st[key], want, what, al16=al16, zero_reserved=not key.startswith("m"))
        elif key.endswith(("_scale", "_min_log")):
            parity.assert_ranges(st[key], want, what, max_ulp=range_ulp)


@pytest.mark.parametrize("name", ["adafactor_factored", "adafactor_factored_m"])
@pytest.mark.parametrize("suffix", ["", "__accnorm"])
def test_factored_adafactor_free_running(name, suffix, oracle):
    """10 free-running steps against the reference (as it is, and with its float32 norm
    routine replaced by an accurate one): row/col codes and ranges, parameters."""
    run = OracleRun(name)
    gold = load_golden(name + suffix)
    assert str(gold["digest"]) == cases.inputs_digest(run.params0, run.grads)
    for t in range(1, run.case["steps"] + 1):
        run.step()
        for i, (p, st) in enumerate(zip(run.params, run.states)):
            _check_step(name + suffix, t, i, p, st, golden_entries(gold, t, i), param_tol=1e-6, range_ulp=128)


@pytest.mark.parametrize("suffix", ["", "__accnorm"])
def test_came_teacher_forced_steps(suffix, oracle):
    """CAME, one step at a time from the reference's own state.  AL16 codes resolve 1.6e-4
    relative, so the one-ulp difference between torch's float32 `mean` and an exactly
    rounded mean moves about one code in a hundred by one step: the bound on differing AL16
    codes is 3e-2 here, all other bounds are the standard ones."""
    name = "came_al16"
    run = OracleRun(name)
    gold = load_golden(name + suffix)
    steps = run.case["steps"]
    checked = 0
    for i, p0 in enumerate(run.params0):
        for t in range(1, steps):
            before, after = golden_entries(gold, t, i), golden_entries(gold, t + 1, i)
            if "param" not in before or "param" not in after or ("m_q" not in before):
                continue     # large arrays are stored for steps 1, 2 and the last one only
            st = state_from_golden(before, run.hp, p0.shape, t)
            p = before["param"].reshape(p0.shape).copy()
            run.step_param(i, p, run.grads[t + 1][i], st)
            # the clip factor carries the reference's norm error (1e-6 at this size) into m_scale
            _check_step(name + suffix, t + 1, i, p, st, after, param_tol=2e-6, al16_frac=3e-2,
                        range_ulp=128 if suffix == "" else 8)
            checked += 1
    assert checked >= 10


def test_came_free_running_states(oracle):
    """Free-running CAME for 10 steps.  A flipped AL16 column code changes that column's
    normaliser by 1e-4, which can flip a UF8 momentum code (1/128 of the block range), and
    each such element then carries a large parameter difference: the parameter bound that
    holds here is 5e-5, not 1e-5; the states stay inside their code bounds."""
    name = "came_al16"
    run = OracleRun(name)
    gold = load_golden(name)
    for t in range(1, run.case["steps"] + 1):
        run.step()
    t = run.case["steps"]
    for i, (p, st) in enumerate(zip(run.params, run.states)):
        _check_step(name, t, i, p, st, golden_entries(gold, t, i), param_tol=5e-5, al16_frac=3e-2, range_ulp=4096)


@pytest.mark.parametrize("name", ["apollo_r32", "apollo_r8_tensor"])
def test_apollo_oracle_against_reference(oracle, name):
    """APOLLO, 8 free-running steps with a refresh of the projection every 3.  The projected
    gradient comes out of a float32 GEMM in the reference and out of exactly rounded dot products
    in the oracle; outputs that nearly cancel differ in many ulps, they sit at the minimum of
    their AL block and move that block's range.  Hence: momentum codes and seeds exact, V codes
    only bounded statistically, the limiter state to 1e-4, parameters to 5e-5.  The second case
    scales per tensor (apollo_scale_type="tensor") with apollo_scale=128."""
    run = OracleRun(name)
    gold = load_golden(name)
    assert str(gold["digest"]) == cases.inputs_digest(run.params0, run.grads)
    steps = run.case["steps"]
    for t in range(1, steps + 1):
        run.step()
        for i, (p, st) in enumerate(zip(run.params, run.states)):
            ref = golden_entries(gold, t, i)
            what = f"{name} step {t} param {i}"
            if "param" in ref:
                parity.assert_params(p, ref["param"], what, tol=5e-5)
            if "apollo_proj_matrix_T" in ref:
                assert np.array_equal(st["apollo_proj_matrix_T"].reshape(-1), ref["apollo_proj_matrix_T"]), what
            if "m_low_q" in ref:
                s = parity.code_stats(st["m_low_q"], ref["m_low_q"])
                assert s["max"] <= 1 and s["neq"] <= max(2, 1e-4 * s["n"]), (what, s)
                s = parity.code_stats(st["v_low_q"], ref["v_low_q"])
                assert s["zero_mismatch"] == 0 and s["neq"] <= 0.06 * s["n"] and s["gt1"] <= 0.01 * s["n"], (what, s)
                assert parity.rel_l2(st["scaled_grad_norm_prev"], ref["scaled_grad_norm_prev"]) <= 1e-4, what
            elif "variance_q" in ref:
                parity.assert_codes(st["variance_q"], ref["variance_q"], what + " variance_q")
                parity.assert_codes(st["m_q"], ref["m_q"], what + " m_q", zero_reserved=False)


@pytest.mark.parametrize("name", ["apollo_fp32_states", "apollo_3d_f16g"])
def test_apollo_variants_against_reference(oracle, name):
    """APOLLO with fp32 low-rank states (quantize=False: both moments by Tensor.lerp_, no codes), and on
    tensors of three dimensions (stepped as (shape[0], -1) matrices) with fp16 gradients.  Bounds as in the
    test above: the reference's float32 GEMM rounds the projected gradient differently."""
    run = OracleRun(name)
    gold = load_golden(name)
    assert str(gold["digest"]) == cases.inputs_digest(run.params0, run.grads)
    for t in range(1, run.case["steps"] + 1):
        run.step()
        for i, (p, st) in enumerate(zip(run.params, run.states)):
            ref = golden_entries(gold, t, i)
            what = f"{name} step {t} param {i}"
            parity.assert_params(p, ref["param"], what, tol=5e-5)
            if "apollo_proj_matrix_T" in ref:
                assert np.array_equal(st["apollo_proj_matrix_T"].reshape(-1), ref["apollo_proj_matrix_T"]), what
            for key in ("v_low", "m_low"):
                if key in ref:
                    assert st[key].size == ref[key].size, what
                    assert parity.rel_l2(st[key], ref[key]) <= 2e-5, (what, key, parity.rel_l2(st[key], ref[key]))
            if "m_low_q" in ref:
                s = parity.code_stats(st["m_low_q"], ref["m_low_q"])
                assert s["max"] <= 1 and s["neq"] <= max(2, 2e-3 * s["n"]), (what, s)
            assert parity.rel_l2(st["scaled_grad_norm_prev"], ref["scaled_grad_norm_prev"]) <= 1e-4, what


@pytest.mark.parametrize("name", cases.FACTORED_3D_CASES)
def test_factored_batches_against_reference(oracle, name):
    """Factored tensors of more than two dimensions (batches of matrices over the last two dimensions,
    optimizer.py:2203-2253): Adafactor with a parameter-scaled step and CAME with momentum and the limiter,
    free-running against the reference.  The row / column states are flat over the batch, so their
    quantisation blocks run across the matrices; codes must agree exactly up to two single steps."""
    run = OracleRun(name)
    gold = load_golden(name)
    assert str(gold["digest"]) == cases.inputs_digest(run.params0, run.grads)
    for t in range(1, run.case["steps"] + 1):
        run.step()
        for i, (p, st) in enumerate(zip(run.params, run.states)):
            ref = golden_entries(gold, t, i)
            what = f"{name} step {t} param {i}"
            parity.assert_params(p, ref["param"], what, tol=2e-5)
            seen = 0
            for key, want in ref.items():
                if key == "param":
                    continue
                assert st.get(key) is not None, (what, key)
                have = np.asarray(st[key]).reshape(-1)
                seen += 1
                if have.dtype in (np.uint8, np.uint16):
                    s = parity.code_stats(have[:want.size], want)
                    assert s["max"] <= 1 and s["neq"] <= 2, (what, key, s)
                else:
                    assert parity.rel_l2(have[:want.size], want) <= 1e-4, (what, key)
            assert seen >= 6, (what, sorted(ref))


@pytest.mark.parametrize("name", cases.APOLLO_RULE_CASES)
def test_apollo_lowrank_rules_against_reference(oracle, name):
    """APOLLO's other low-rank rules, free-running against the reference: apollo_factorize (fp32 row / column
    factors of the projected gradient's squares, optimizer.py:2688-2760), the same with CAME's confidence
    vectors (2708-2750), CAME over the projected gradient with its instability state res_low, AL8-coded and
    fp32 (2801-2903, pure-PyTorch branch), factorisation without momentum, and a step size that follows the
    parameters' RMS (scale_parameter=True, channel-wise and tensor-wise scaling).  Codes agree to one step on a
    few elements (the float32 GEMM of the reference rounds the projected gradient differently), fp32 states
    and block ranges to 1e-4 relative."""
    run = OracleRun(name)
    gold = load_golden(name)
    assert str(gold["digest"]) == cases.inputs_digest(run.params0, run.grads)
    for t in range(1, run.case["steps"] + 1):
        run.step()
        for i, (p, st) in enumerate(zip(run.params, run.states)):
            ref = golden_entries(gold, t, i)
            what = f"{name} step {t} param {i}"
            parity.assert_params(p, ref["param"], what, tol=5e-5)
            seen = 0
            for key, want in ref.items():
                if key in ("param", "apollo_proj_matrix_T"):
                    continue
                assert st.get(key) is not None, (what, key)
                have = np.asarray(st[key]).reshape(-1)
                seen += 1
                if have.dtype in (np.uint8, np.uint16):
                    # (an element of the projected gradient that cancels to almost nothing is a different small
                    # number in the reference's float32 GEMM: at most two such codes may be further off)
                    s = parity.code_stats(have[:want.size], want)
                    assert s["gt1"] <= 2 and s["neq"] <= max(2, 2e-3 * s["n"]), (what, key, s)
                else:
                    assert have.size >= want.size, (what, key)
                    assert parity.rel_l2(have[:want.size], want) <= 1e-4, (what, key, parity.rel_l2(have[:want.size], want))
            assert seen >= 3, (what, sorted(ref))


# ---------------------------------------------------------------------------
# bf16 / fp16 parameters, nearest and stochastic rounding (optimizer.py:162-292, 866-881)
# ---------------------------------------------------------------------------
def test_stochastic_rounding_known_answers(oracle):
    """The two rounding routines on edge values (zeros, exact values, the largest finite numbers,
    overflow, infinities, NaNs, subnormals), bit for bit against the reference's routines."""
    gold = load_golden("sr_edges")
    x, rnd = cases.sr_edge_inputs()
    assert str(gold["digest"]) == cases.digest([x, rnd])
    for fmt in ("bf16", "f16"):
        assert np.array_equal(oracle.sr_round(x, rnd, fmt), gold[fmt]), fmt
    # the counter generator: the C routine and the numpy restatement that fed the reference
    u = cases.sr_uniform(3, 7, 1000)
    assert u.min() >= 0.0 and u.max() < 1.0 and abs(float(u.mean()) - 0.5) < 0.03
    for idx in (0, 1, 17, 999):
        assert oracle.sr_uniform(3, 7, idx) == u[idx]


@pytest.mark.parametrize("name", cases.LOWP_FULLRANK_CASES + cases.LOWP_FACTORED_CASES)
def test_low_precision_parameters_free_running(name, oracle):
    """Free-running steps on bf16 / fp16 parameters.  The full-rank cases agree with the reference
    in every parameter bit and every code, stochastic rounding included (same uniform numbers);
    in the factored cases torch's float32 means move a parameter in ten thousand to the
    neighbouring number of its format and an occasional small-state code by one."""
    run = OracleRun(name)
    gold = load_golden(name)
    assert str(gold["digest"]) == cases.inputs_digest(run.params0, run.grads)
    fmt = run.case["param_dtype"]
    exact = name in cases.LOWP_FULLRANK_CASES
    for t in range(1, run.case["steps"] + 1):
        run.step()
        for i, (p, st) in enumerate(zip(run.params, run.states)):
            ref = golden_entries(gold, t, i)
            for key, want in ref.items():
                what = f"{name} step {t} param {i} {key}"
                if key == "param":
                    parity.assert_lowp_params(p, want, fmt, what, frac=0.0 if exact else 2e-4)
                    if exact:
                        assert np.array_equal(p.reshape(-1), want), what
                elif key in CODE_KEYS:
                    if exact:
                        assert np.array_equal(st[key], want), what
                    else:
                        s = parity.code_stats(st[key], want)
                        al16 = want.dtype == np.uint16
                        assert s["zero_mismatch"] == 0 and s["max"] <= (parity.CODE_SLACK_AL16 if al16 else 1), (what, s)
                        assert s["neq"] <= max(2, (3e-2 if al16 else 1e-4) * s["n"]), (what, s)
                elif key.endswith(RANGE_SUFFIXES):
                    parity.assert_ranges(st[key], want, what, max_ulp=0 if exact else 128)


# ---------------------------------------------------------------------------
# group options edited between steps: the state migrations of _init_group (optimizer.py:1650-1860)
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("name", cases.MIGRATION_CASES)
def test_state_migration_against_reference(name, oracle):
    """`quantize` off and on again, a new momentum format (momentum reset), a new V format
    (re-initialisation, step kept), CAME switched off and on (confidence states dropped and
    recreated), factored mode switched off: after every step the oracle holds the same state
    entries as the reference, with codes, ranges and parameters inside the usual bounds."""
    run = OracleRun(name)
    gold = load_golden(name)
    assert str(gold["digest"]) == cases.inputs_digest(run.params0, run.grads)
    for t in range(1, run.case["steps"] + 1):
        run.step()
        for i, (p, st) in enumerate(zip(run.params, run.states)):
            ref = golden_entries(gold, t, i)
            mine = {k for k, v in st.items() if isinstance(v, np.ndarray)}
            theirs = {k for k in ref if k not in ("param", "fira_prev_norm")}
            assert mine == theirs, f"{name} step {t} param {i}: state entries {sorted(mine ^ theirs)} differ"
            for key, want in ref.items():
                what = f"{name} step {t} param {i} {key}"
                if key == "param":
                    parity.assert_params(p, want, what)
                elif key in CODE_KEYS:
                    fmt = st.get("m_quant_type") if key.startswith("m") else None
                    got = st[key]
                    if fmt in ("uf4", "d4"):
                        got, want = parity.unpack_nibbles(got), parity.unpack_nibbles(want)
                    parity.assert_codes(got, want, what, al16=want.dtype == np.uint16, zero_reserved=not key.startswith("m"))
                elif key.endswith(RANGE_SUFFIXES):
                    parity.assert_ranges(st[key], want, what, max_ulp=128)
                elif key in st:
                    assert parity.rel_l2(st[key], want) <= 2e-4, what


@pytest.mark.parametrize("name", ["apollo_bf16p", "apollo_sr_bf16p"])
def test_apollo_low_precision_parameters(name, oracle):
    """APOLLO on bf16 parameters (optimizer.py:3043-3079): in-place ops rounded to bf16, or one
    stochastic rounding of p*decay + (g*scale)*update_scale.  The first step agrees with the reference
    in every parameter bit; afterwards the reference's float32 GEMM moves a scaling factor now and then
    (see test_apollo_oracle_against_reference), which shows as a few parameters per thousand on a
    neighbouring bf16 number."""
    run = OracleRun(name)
    gold = load_golden(name)
    assert str(gold["digest"]) == cases.inputs_digest(run.params0, run.grads)
    for t in range(1, run.case["steps"] + 1):
        run.step()
        for i, (p, st) in enumerate(zip(run.params, run.states)):
            ref = golden_entries(gold, t, i)
            what = f"{name} step {t} param {i}"
            if "param" in ref:
                s = parity.lowp_stats(p, ref["param"], "bf16")
                if t == 1:
                    assert s["neq"] == 0, (what, s)
                assert s["neq"] <= 2e-3 * s["n"] and parity.rel_l2(p, ref["param"]) <= 5e-4, (what, s)
            if "m_low_q" in ref:
                sm = parity.code_stats(st["m_low_q"], ref["m_low_q"])
                assert sm["max"] <= 1 and sm["neq"] <= max(2, 1e-4 * sm["n"]), (what, sm)
