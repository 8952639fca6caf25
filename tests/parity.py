"""Comparison helpers for the parity tests.

Tolerances (the contract this build is held to, per quantity):
  * exact-zero codes: positions identical;
  * other codes: differ by at most one code on at most 1e-4 of the elements
    (AL8, UF8, UF4, d8, d4).  AL16 has 257 times finer code steps, so one ulp of
    log2 already moves a code; there the bound is |diff| <= CODE_SLACK_AL16 on at
    most 1e-3 of the elements;
  * per-block ranges (scale, min_log, m_scale): within 1 ulp when both sides
    start the step from identical state;
  * fp32 parameters: relative L2 error per tensor <= 1e-5 after the last step.
"""
import math

import numpy as np

CODE_FRAC = 1e-4
CODE_FRAC_AL16 = 1e-3
CODE_SLACK_AL16 = 8
PARAM_REL = 1e-5


def ulp_diff(a, b):
    a = np.ascontiguousarray(a, dtype=np.float32).reshape(-1)
    b = np.ascontiguousarray(b, dtype=np.float32).reshape(-1)
    ia = a.view(np.int32).astype(np.int64)
    ib = b.view(np.int32).astype(np.int64)
    ia = np.where(ia < 0, -(ia & 0x7FFFFFFF), ia)
    ib = np.where(ib < 0, -(ib & 0x7FFFFFFF), ib)
    return np.abs(ia - ib)


def rel_l2(a, b):
    a = np.asarray(a, dtype=np.float64).reshape(-1)
    b = np.asarray(b, dtype=np.float64).reshape(-1)
    den = np.linalg.norm(b)
    return float(np.linalg.norm(a - b) / den) if den > 0 else float(np.linalg.norm(a - b))


def unpack_nibbles(q):
    q = np.asarray(q, dtype=np.uint8).reshape(-1)
    out = np.empty(q.size * 2, dtype=np.uint8)
    out[0::2] = q >> 4
    out[1::2] = q & 0xF
    return out


def code_stats(a, b):
    a = np.asarray(a).reshape(-1).astype(np.int64)
    b = np.asarray(b).reshape(-1).astype(np.int64)
    d = np.abs(a - b)
    return dict(n=a.size, neq=int((d > 0).sum()), gt1=int((d > 1).sum()), max=int(d.max()) if d.size else 0,
                zero_mismatch=int(((a == 0) != (b == 0)).sum()))


def assert_codes(a, b, what, al16=False, zero_reserved=True):
    s = code_stats(a, b)
    frac = CODE_FRAC_AL16 if al16 else CODE_FRAC
    allowed = max(2, math.ceil(frac * s["n"]))
    slack = CODE_SLACK_AL16 if al16 else 1
    if zero_reserved:
        assert s["zero_mismatch"] == 0, f"{what}: exact-zero codes differ at {s['zero_mismatch']} positions"
    assert s["max"] <= slack, f"{what}: a code differs by {s['max']} (> {slack}); stats {s}"
    assert s["neq"] <= allowed, f"{what}: {s['neq']} of {s['n']} codes differ (allowed {allowed})"
    return s


def assert_ranges(a, b, what, max_ulp=1):
    u = ulp_diff(a, b)
    assert u.size == 0 or int(u.max()) <= max_ulp, f"{what}: block range differs by {int(u.max())} ulp"
    return int(u.max()) if u.size else 0


def assert_params(a, b, what, tol=PARAM_REL):
    r = rel_l2(a, b)
    assert r <= tol, f"{what}: parameter relative L2 error {r:.3e} > {tol}"
    return r


def lowp_ordinal(x, fmt):
    """Position of each value (exactly representable in bf16 / f16) on that format's number line."""
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    if fmt == "bf16":
        bits = (x.view(np.uint32) >> 16).astype(np.int64)
    else:
        bits = x.astype(np.float16).view(np.uint16).astype(np.int64)
    return np.where(bits & 0x8000, -(bits & 0x7FFF), bits)


def lowp_stats(a, b, fmt):
    d = np.abs(lowp_ordinal(a, fmt) - lowp_ordinal(b, fmt))
    return dict(n=d.size, neq=int((d > 0).sum()), max=int(d.max()) if d.size else 0)


def assert_lowp_params(a, b, fmt, what, frac, max_units=1):
    """bf16 / f16 parameters: equal except on a fraction `frac` of the elements, which may sit
    on the neighbouring number of the format."""
    s = lowp_stats(a, b, fmt)
    assert s["max"] <= max_units, f"{what}: a parameter is {s['max']} units of the format away; {s}"
    assert s["neq"] <= max(1, math.ceil(frac * s["n"])), f"{what}: {s['neq']} of {s['n']} parameters differ (allowed fraction {frac})"
    return s
