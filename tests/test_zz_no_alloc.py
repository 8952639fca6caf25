"""af8_fullrank_limited_step_noalloc against the regular three-call sequence
(af8_fullrank_step SUMSQ -> af8_norm_finalize -> af8_fullrank_step APPLY).

The no-allocation entry point serves callers that cannot hand the library any
working buffers (a pointer-forwarding binding without a device allocator, or a
process whose framework allocator owns the whole GPU); its scratch is a fixed
array inside the library.  Both routes run the same arithmetic, so states and
parameters must come out identical, on two consecutive steps: the second step
reuses the array with the first step's leftovers in it and takes the limiter's
"previous norm" branch.  The results are also held against the CPU oracle at the
usual tolerances, a second format (AL16 / UF8 at block 1024, the general kernels)
and the clip-only configuration without a norm output are covered, and the calls
are checked to leave the amount of free device memory unchanged.

This file sorts last so that a run stopping at the first failure has already
executed every other test.  It does not depend on them: it also passes alone in
a fresh process.
"""
import ctypes

import numpy as np
import pytest
import torch

import cases
import parity

pytestmark = pytest.mark.gpu


def _bf16(g, shape):
    return torch.from_numpy(g.view(np.int16).copy()).view(torch.bfloat16).reshape(shape).cuda()


class _Tensor:
    """Parameter, gradient and quantised AdamW states of one tensor on the GPU."""

    def __init__(self, p0, numel, v_bits=8, block=2048, m_block=256):
        nvb = -(-numel // block)
        nmb = -(-numel // m_block)
        self.numel, self.block, self.m_block = numel, block, m_block
        self.param = torch.from_numpy(p0.copy()).cuda()
        self.v_q = torch.zeros(nvb * block, dtype=torch.uint8 if v_bits == 8 else torch.int16, device="cuda")
        self.v_scale = torch.ones(nvb, dtype=torch.float32, device="cuda")
        self.v_min_log = torch.zeros(nvb, dtype=torch.float32, device="cuda")
        self.m_q = torch.full((nmb * m_block,), 128, dtype=torch.uint8, device="cuda")
        self.m_scale = torch.ones(nmb, dtype=torch.float32, device="cuda")
        self.fira_prev = torch.zeros((), dtype=torch.float32, device="cuda")
        self.grad = None

    def row(self, N, step):
        r = np.zeros(1, dtype=N.FULLRANK_TENSOR)
        r["param"], r["grad"] = self.param.data_ptr(), self.grad.data_ptr()
        r["v_q"], r["v_scale"], r["v_min_log"] = self.v_q.data_ptr(), self.v_scale.data_ptr(), self.v_min_log.data_ptr()
        r["m_q"], r["m_scale"] = self.m_q.data_ptr(), self.m_scale.data_ptr()
        r["numel"] = self.numel
        bc1, bc2 = 1.0 - 0.9 ** step, 1.0 - 0.999 ** step
        r["alpha"] = np.float32(np.float32(1e-3) * np.float32(np.sqrt(bc2) / bc1))
        r["decay"] = np.float32(np.float32(1.0) - np.float32(np.float32(1e-3) * np.float32(0.01)))
        r["v_w"], r["v_keep"], r["m_w"] = np.float32(1.0 - 0.999), np.float32(0.999), np.float32(1.0 - 0.9)
        r["eps_denom"] = np.float32(1e-8 * np.sqrt(bc2))
        r["eps_sq"] = np.float32(1.17549435e-38)
        return r

    def snapshot(self):
        torch.cuda.synchronize()
        out = {k: getattr(self, k).detach().cpu().numpy().copy()
               for k in ("param", "v_q", "v_scale", "v_min_log", "m_q", "m_scale", "fira_prev")}
        if out["v_q"].dtype == np.int16:
            out["v_q"] = out["v_q"].view(np.uint16)
        return out


def _cfg(N, bf16, v_bits=8, block=2048, m_block=256):
    cfg = N.FullrankCfg()
    cfg.param_dtype, cfg.grad_dtype = N.F32, (N.BF16 if bf16 else N.F32)
    cfg.v_fmt, cfg.m_fmt, cfg.block, cfg.m_block = (N.V_AL8 if v_bits == 8 else N.V_AL16), N.M_UF8, block, m_block
    cfg.use_adam_denom, cfg.momentum_only, cfg.negate_grad = 1, 0, 0
    cfg.v_floor = -126.0
    return cfg


def _regular_step(N, t, cfg, step, d, margin, has_prev, fira=True):
    """The existing route with caller-allocated scratch."""
    lib = N.lib()
    stream = torch.cuda.current_stream().cuda_stream
    row = t.row(N, step)
    nblocks = -(-t.numel // t.block)
    d_table = torch.empty(N.FULLRANK_TENSOR.itemsize, dtype=torch.uint8, device="cuda")
    d_dyn = torch.zeros(N.DYN_SCALARS.itemsize, dtype=torch.uint8, device="cuda")
    d_sumsq = torch.empty(nblocks, dtype=torch.float32, device="cuda")
    cfg.mode = N.MODE_SUMSQ
    N.check(lib.af8_fullrank_step(ctypes.byref(cfg), row.ctypes.data, d_table.data_ptr(), 1, nblocks,
                                  d_dyn.data_ptr(), d_sumsq.data_ptr(), stream), "sumsq")
    torch.cuda.synchronize()
    nt = np.zeros(1, dtype=N.NORM_TENSOR)
    nt["n_blocks"], nt["fira_has_prev"] = nblocks, int(has_prev and fira)
    nt["fira_prev"] = t.fira_prev.data_ptr() if fira else 0
    nt["alpha"] = row["alpha"]
    nt["sqrt_n"] = np.float32(np.sqrt(float(t.numel)))
    nt["d"] = np.float32(d)
    nt["clip_div"] = np.float32(np.sqrt(float(t.numel)) * d) if d > 0 else np.float32(0)
    nt["fira_margin1"] = np.float32(1.0 + margin)
    d_norm = torch.from_numpy(nt.view(np.uint8).copy()).cuda()
    N.check(lib.af8_norm_finalize(d_norm.data_ptr(), 1, d_sumsq.data_ptr(), d_dyn.data_ptr(), stream), "finalize")
    cfg.mode = N.MODE_APPLY
    N.check(lib.af8_fullrank_step(ctypes.byref(cfg), None, d_table.data_ptr(), 1, nblocks,
                                  d_dyn.data_ptr(), d_sumsq.data_ptr(), stream), "apply")
    torch.cuda.synchronize()
    return float(d_dyn.cpu().numpy().view(N.DYN_SCALARS)["norm"][0])


def _noalloc_step(N, t, cfg, step, d, margin, has_prev, norm_out, fira=True):
    row = t.row(N, step)
    torch.cuda.synchronize()
    free_before, allocated_before = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
    rc = N.lib().af8_fullrank_limited_step_noalloc(
        ctypes.byref(cfg), row.ctypes.data, d, int(fira), float(np.float32(1.0 + margin)),
        t.fira_prev.data_ptr() if fira else None, int(has_prev and fira),
        norm_out.data_ptr() if norm_out is not None else None, torch.cuda.current_stream().cuda_stream)
    N.check(rc, "af8_fullrank_limited_step_noalloc")
    torch.cuda.synchronize()
    # the call took no device memory, neither from the driver nor from torch's allocator
    assert torch.cuda.mem_get_info()[0] == free_before and torch.cuda.memory_allocated() == allocated_before
    return float(norm_out.item()) if norm_out is not None else None


def _oracle_hp(oracle, d, fira, v_bits, block, m_block):
    return oracle.hyper(**dict(cases.CASES["adamw_fira_bf16"]["hp"], d=d, enable_fira_for_adafactor=fira,
                               v_quant_type="al8" if v_bits == 8 else "al16", block_size=block, m_block_size=m_block))


# (bf16 gradients, elements, clip d, limiter, V bits, V block, M block): the two specialised-kernel cases,
# the general kernels (AL16 at block 1024), and clip without the limiter and without a norm output
CASES = [(True, 300 * 200, 0.0, True, 8, 2048, 256), (False, 5 * 2048 + 77, 1.0, True, 8, 2048, 256),
         (False, 7 * 1024 + 300, 0.0, True, 16, 1024, 128), (True, 3 * 2048 + 5, 0.05, False, 8, 2048, 256)]


@pytest.mark.parametrize("bf16,numel,d,fira,v_bits,block,m_block", CASES)
def test_noalloc_matches_regular_route_and_oracle_on_two_steps(bf16, numel, d, fira, v_bits, block, m_block, oracle):
    from adafactor8bit import _native as N
    spec = dict(cases.CASES["adamw_fira_bf16"]["grad"], dtype="bf16" if bf16 else "f32")
    p0 = cases.make_param((numel,), 4242)
    a, b = _Tensor(p0, numel, v_bits, block, m_block), _Tensor(p0, numel, v_bits, block, m_block)
    cfg_a, cfg_b = _cfg(N, bf16, v_bits, block, m_block), _cfg(N, bf16, v_bits, block, m_block)
    # allocated by the test, not the library; the clip-only case passes no norm output at all
    norm_out = torch.zeros((), dtype=torch.float32, device="cuda") if fira else None
    ohp = _oracle_hp(oracle, d, fira, v_bits, block, m_block)
    ost = oracle.init_state((numel,), ohp)
    op = p0.copy()
    for step in (1, 2):
        g = cases.make_grad((numel,), 4300, step, spec)
        for t in (a, b):
            t.grad = _bf16(g, (numel,)) if bf16 else torch.from_numpy(g.copy()).cuda()
        n_ref = _regular_step(N, a, cfg_a, step, d, 0.01, has_prev=(step > 1), fira=fira)
        n_new = _noalloc_step(N, b, cfg_b, step, d, 0.01, has_prev=(step > 1), norm_out=norm_out, fira=fira)
        oracle.fullrank_step(op, g, ost, ohp)
        sa, sb = a.snapshot(), b.snapshot()
        what = f"noalloc bf16={bf16} AL{v_bits}/{block} step {step}"
        if norm_out is not None:
            assert n_new == n_ref, f"{what}: norm {n_new} vs {n_ref}"
        al16 = v_bits == 16
        parity.assert_codes(sb["v_q"], sa["v_q"], what + " v_q", al16=al16)
        parity.assert_codes(sb["m_q"], sa["m_q"], what + " m_q", zero_reserved=False)
        for k in ("v_scale", "v_min_log", "m_scale") + (("fira_prev",) if fira else ()):
            parity.assert_ranges(sb[k], sa[k], what + " " + k, max_ulp=1)
        parity.assert_params(sb["param"], sa["param"], what + " param")
        # same kernels, same inputs: in fact bit-identical
        assert np.array_equal(sb["param"], sa["param"]) and np.array_equal(sb["v_q"], sa["v_q"])
        # and against the CPU oracle of the reference's step
        parity.assert_codes(sb["v_q"], ost["variance_q"], what + " v_q vs oracle", al16=al16)
        parity.assert_codes(sb["m_q"], ost["m_q"], what + " m_q vs oracle", zero_reserved=False)
        for k, ok in (("v_scale", "variance_scale"), ("v_min_log", "variance_min_log"), ("m_scale", "m_scale")):
            parity.assert_ranges(sb[k], ost[ok], what + " " + k + " vs oracle", max_ulp=4)
        parity.assert_params(sb["param"], op, what + " param vs oracle")
        if fira:
            want = float(ost["fira_prev_norm"])
            assert abs(float(sb["fira_prev"]) - want) <= 2e-6 * abs(want), what
    if fira:
        assert float(b.fira_prev.item()) > 0.0


def test_noalloc_rejects_stochastic_rounding():
    from adafactor8bit import _native as N
    lib = N.lib()
    cfg = _cfg(N, True)
    cfg.stochastic_round = 1
    row = np.zeros(1, dtype=N.FULLRANK_TENSOR)
    row["numel"] = 4096
    prev = torch.zeros((), dtype=torch.float32, device="cuda")
    rc = lib.af8_fullrank_limited_step_noalloc(ctypes.byref(cfg), row.ctypes.data, 0.0, 1, 1.01, prev.data_ptr(), 0,
                                               None, torch.cuda.current_stream().cuda_stream)
    assert rc == N.ERR_INVALID


def test_noalloc_rejects_oversized_tensor():
    from adafactor8bit import _native as N
    lib = N.lib()
    limit = lib.af8_noalloc_max_numel(2048)
    assert limit == 262080 * 2048
    assert lib.af8_noalloc_max_numel(100) == 0
    cfg = _cfg(N, True)
    row = np.zeros(1, dtype=N.FULLRANK_TENSOR)
    row["numel"] = limit + 1
    prev = torch.zeros((), dtype=torch.float32, device="cuda")
    rc = lib.af8_fullrank_limited_step_noalloc(ctypes.byref(cfg), row.ctypes.data, 0.0, 1, 1.01, prev.data_ptr(), 0,
                                               None, torch.cuda.current_stream().cuda_stream)
    assert rc == N.ERR_UNSUPPORTED
    msg = lib.af8_last_error().decode()
    assert "built-in scratch" in msg and str(limit) in msg
