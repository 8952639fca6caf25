"""Drive the CPU oracle through a case of tests/golden/cases.py."""
import numpy as np

import af8_oracle as o
import cases

FULLRANK_CASES = ["adamw_uf8_al8", "adamw_fira_bf16", "adamw_uf4_al16", "adamw_d8_al8", "adamw_d4_al8",
                  "adamw_fp32m_al8", "rmsprop_al8", "adafactor_unfactored", "sgd_momentum_uf8", "sgd_plain_bf16", "adamw_ragged"]


def load_golden(name):
    import os
    path = os.path.join(os.path.dirname(os.path.abspath(cases.__file__)), name + ".npz")
    return np.load(path)


class OracleRun:
    def __init__(self, name, case=None):
        """`case`: a dict of the same form as the entries of cases.CASES, for cases without fixtures."""
        self.name = name
        self.case = case if case is not None else cases.CASES[name]
        self.hp = o.hyper(**self.case["hp"], param_dtype=self.case.get("param_dtype", "f32"))
        self.params0, self.grads = cases.case_inputs(self.case)
        self.params = [p.copy() for p in self.params0]
        # an APOLLO tensor of more than two dimensions is stepped as a (shape[0], -1) matrix (optimizer.py:2634-2639)
        self.states = [o.init_state(self._matrix_shape(p.shape), self.hp) for p in self.params]
        seed = 1                                 # optimizer-level counter (optimizer.py:1460, 1727-1728)
        for st in self.states:
            if "apollo_seed" in st:
                st["apollo_seed"] = seed
                seed += 1
        if self.hp["stochastic_round_writeback"] and self.hp["param_dtype"] != "f32":
            for k, st in enumerate(self.states):     # optimizer-level counter from 1, in parameter order (optimizer.py:1461, 1889-1892)
                st["sr_seed"] = k + 1
        self.t = 0

    def _matrix_shape(self, shape):
        if self.hp["apollo_rank"] > 0 and len(shape) > 2:
            return (shape[0], int(np.prod(shape[1:])))
        return tuple(shape)

    def step_param(self, i, p, g, st):
        shape = p.shape
        if self.hp["apollo_rank"] > 0 and len(shape) >= 2:
            m = self._matrix_shape(shape)
            return o.apollo_step(p.reshape(m), g.reshape(m), st, self.hp)      # (views: the update lands in p)
        if len(shape) >= 2 and self.hp["factored"] and not o.is_sgd(self.hp):
            return o.factored_step(p, g, st, self.hp)
        return o.fullrank_step(p.reshape(-1), g.reshape(-1), st, self.hp)

    def step(self):
        self.t += 1
        edits = self.case.get("changes", {}).get(self.t)
        if edits:                                # a group option edited before this step
            self.hp.update(edits)
            self.states = [o.migrate_state(st, self.hp, p.shape) for st, p in zip(self.states, self.params)]
        norms = []
        for i, (p, st) in enumerate(zip(self.params, self.states)):
            norms.append(self.step_param(i, p, self.grads[self.t][i], st))
        return norms


def golden_entries(gold, t, i):
    pre = f"t{t}_p{i}_"
    return {k[len(pre):]: gold[k] for k in gold.files if k.startswith(pre)}


FACTORED_CASES = ["adafactor_factored", "adafactor_factored_m", "came_al16"]
STATE_ARRAY_KEYS = ("variance_q", "variance_scale", "variance_min_log", "variance", "m_q", "m_scale", "m",
                    "row_var_q", "row_var_scale", "row_var_min_log", "row_var", "col_var_q", "col_var_scale",
                    "col_var_min_log", "col_var", "conf_row_q", "conf_row_scale", "conf_row_min_log", "conf_row",
                    "conf_col_q", "conf_col_scale", "conf_col_min_log", "conf_col")


def state_from_golden(entries, hp, shape, step):
    """Oracle state of one parameter rebuilt from a fixture snapshot (after `step` steps)."""
    st = o.init_state(shape, hp)
    st["step"] = step
    for k in STATE_ARRAY_KEYS:
        if k in entries and k in st:
            st[k] = np.ascontiguousarray(entries[k]).astype(st[k].dtype).reshape(st[k].shape).copy()
    if "fira_prev_norm" in entries:
        st["fira_prev_norm"] = np.float32(entries["fira_prev_norm"].reshape(-1)[0])
    return st
