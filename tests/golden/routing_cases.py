"""Toy models and scenarios for the parameter-group builder.  Shared by the script that
records what the reference package returns (gen_routing_golden.py) and by the test that
replays the scenarios against this repository's builder."""
import torch
from torch import nn


class _Attn(nn.Module):
    def __init__(self, h, kv, bias=False):
        super().__init__()
        self.q_proj = nn.Linear(h, h, bias=bias)
        self.k_proj = nn.Linear(h, kv, bias=bias)
        self.v_proj = nn.Linear(h, kv, bias=bias)
        self.o_proj = nn.Linear(h, h, bias=bias)


class _Mlp(nn.Module):
    def __init__(self, h, f):
        super().__init__()
        self.gate_proj = nn.Linear(h, f, bias=False)
        self.up_proj = nn.Linear(h, f, bias=False)
        self.down_proj = nn.Linear(f, h, bias=False)


class _Layer(nn.Module):
    def __init__(self, h, kv, f, bias=False):
        super().__init__()
        self.self_attn = _Attn(h, kv, bias)
        self.mlp = _Mlp(h, f)
        self.input_layernorm = nn.LayerNorm(h)
        self.post_attention_layernorm = nn.LayerNorm(h)


class _Body(nn.Module):
    def __init__(self, vocab, h, kv, f, layers, bias=False):
        super().__init__()
        self.embed_tokens = nn.Embedding(vocab, h)
        self.layers = nn.ModuleList([_Layer(h, kv, f, bias) for _ in range(layers)])
        self.norm = nn.LayerNorm(h)


class LlamaLike(nn.Module):
    """Decoder with Hugging-Face-style Llama module names."""
    def __init__(self, vocab=96, h=64, kv=32, f=128, layers=2, tied=False, bias=False):
        super().__init__()
        self.model = _Body(vocab, h, kv, f, layers, bias)
        self.lm_head = nn.Linear(h, vocab, bias=False)
        if tied:
            self.lm_head.weight = self.model.embed_tokens.weight


class GptLike(nn.Module):
    """GPT-2-style names, a positional table, a frozen tensor, a conv weight and a
    parameter whose name alone says "embed"."""
    def __init__(self, vocab=80, h=48):
        super().__init__()
        self.wte = nn.Embedding(vocab, h)
        self.wpe = nn.Embedding(32, h)
        self.time_embed = nn.Linear(h, h)
        self.patch_embed_proj = nn.Parameter(torch.zeros(h, h))
        self.h = nn.ModuleList([nn.ModuleDict(dict(attn=nn.Linear(h, 3 * h), mlp_fc=nn.Linear(h, 4 * h),
                                                   ln_1=nn.LayerNorm(h))) for _ in range(2)])
        self.conv = nn.Conv2d(4, 8, 3)
        self.frozen = nn.Linear(h, h)
        for p in self.frozen.parameters():
            p.requires_grad_(False)
        self.lm_head = nn.Linear(h, vocab, bias=False)


MODELS = {
    "llama": lambda: LlamaLike(),
    "llama_tied": lambda: LlamaLike(tied=True),
    "llama_bias": lambda: LlamaLike(bias=True),
    "gpt": lambda: GptLike(),
    "empty": lambda: nn.Module(),
}

_POLICY = {
    "defaults": {"lr": 3e-4, "weight_decay": 0.05},
    "presets": {"slow_adam": {"preset": "adamw", "lr": 1e-5}, "slower": {"preset": "slow_adam", "beta1": 0.8}},
    "mapping": {"embedding": {"preset": "slower", "quantize": False}, "other": {"block_size": 256},
                "nd": {"preset": "sgd"}},
}

# (scenario name, model, kwargs of build_param_groups)
SCENARIOS = []
for _m in ("llama", "llama_tied", "gpt"):
    for _p in ("sgd", "adafactor", "adamw", "rmsprop", "came", "apollo"):
        for _g in ("auto", "G0", "G1", "G2"):
            SCENARIOS.append((f"{_m}-{_p}-{_g}", _m, dict(preset=_p, grouping=_g)))
SCENARIOS += [
    ("bias-adamw", "llama_bias", dict(preset="adamw")),
    ("empty", "empty", dict(preset="adamw")),
    ("aliases", "llama", dict(preset="AdamW", grouping="protected")),
    ("alias-bare", "llama", dict(preset="came", grouping="bare")),
    ("alias-topology", "gpt", dict(preset="came", grouping="topology", nd_factored=True)),
    ("nd-factored-false", "gpt", dict(preset="adafactor", grouping="G2", nd_factored=False)),
    ("apollo-rank32", "llama", dict(preset="apollo", apollo_rank=32)),
    ("apollo-rank0", "llama", dict(preset="apollo", apollo_rank=0, apollo_targets=["attn"])),
    ("apollo-targets-q", "llama", dict(preset="apollo", apollo_rank=16, apollo_targets=["q_proj", "down"])),
    ("apollo-targets-head", "llama", dict(preset="apollo", apollo_rank=16, apollo_targets=["lm_head"])),
    ("apollo-targets-head-tied", "llama_tied", dict(preset="apollo", apollo_rank=16, apollo_targets=["lm_head"])),
    ("apollo-targets-embed-tied", "llama_tied", dict(preset="apollo", apollo_rank=16, apollo_targets=["embed"])),
    ("apollo-mult", "llama", dict(preset="apollo", apollo_rank=16, apollo_min_dim_multiplier=4)),
    ("apollo-g2-gpt", "gpt", dict(preset="apollo", apollo_rank=16, grouping="G2", apollo_targets=["attn", "mlp"])),
    ("apollo-empty-targets", "llama", dict(preset="apollo", apollo_rank=16, apollo_targets=[])),
    ("rule-overrides", "llama", dict(preset="apollo", apollo_rank=16, beta1=0.8, beta3=0.99, eps=(1e-7, 1e-3),
                                      apollo_update_proj_gap=50)),
    ("route-overrides", "llama", dict(preset="adamw", other_lr=1e-4, other_m_quant_type="uf4", other_block_size=512,
                                       one_d_quantize=True, embedding_v_quant_type="al16", lm_head_m_block_size=64,
                                       lm_head_min_8bit_size=0)),
    ("route-overrides-inactive", "llama", dict(preset="adafactor", embedding_block_size=256, other_m_quant_type="uf8",
                                                other_c_quant_type="al8")),
    ("route-override-unmatched", "llama", dict(preset="adamw", matrix_lr=1e-3)),
    ("route-override-tied", "llama_tied", dict(preset="adamw", lm_head_lr=1e-3)),
    ("route-quantize-auto", "llama", dict(preset="adamw", embedding_quantize="auto", other_quantize=False)),
    ("policy", "llama", dict(preset="adamw", policy=_POLICY)),
    ("policy-g2", "gpt", dict(preset="came", grouping="G2", policy=_POLICY)),
    ("policy-empty-model", "empty", dict(preset="adamw", policy=_POLICY)),
    # errors
    ("err-preset", "llama", dict(preset="lion")),
    ("err-grouping", "llama", dict(preset="adamw", grouping="G3")),
    ("err-grouping-none", "llama", dict(preset="adamw", grouping=None)),
    ("err-nd-type", "llama", dict(preset="adafactor", grouping="G2", nd_factored=1)),
    ("err-nd-grouping", "llama", dict(preset="adafactor", grouping="G1", nd_factored=True)),
    ("err-nd-preset", "llama", dict(preset="adamw", grouping="G2", nd_factored=True)),
    ("err-rank-preset", "llama", dict(preset="adamw", apollo_rank=8)),
    ("err-targets-preset", "llama", dict(preset="adamw", apollo_targets=["attn"])),
    ("err-mult-preset", "llama", dict(preset="adamw", apollo_min_dim_multiplier=2)),
    ("err-rank-type", "llama", dict(preset="apollo", apollo_rank=8.0)),
    ("err-rank-bool", "llama", dict(preset="apollo", apollo_rank=True)),
    ("err-rank-neg", "llama", dict(preset="apollo", apollo_rank=-1)),
    ("err-targets-str", "llama", dict(preset="apollo", apollo_targets="attn")),
    ("err-targets-none", "llama", dict(preset="apollo", apollo_targets=None)),
    ("err-targets-entry", "llama", dict(preset="apollo", apollo_targets=["attn", ""])),
    ("err-mult", "llama", dict(preset="apollo", apollo_min_dim_multiplier=0)),
    ("err-override-unknown", "llama", dict(preset="adamw", momentum=0.9)),
    ("err-override-factored", "llama", dict(preset="adamw", factored=True)),
    ("err-override-route", "llama", dict(preset="adamw", attention_lr=1e-3)),
    ("err-opt-mtype", "llama", dict(preset="adamw", other_m_quant_type="int8")),
    ("err-opt-vtype", "llama", dict(preset="adamw", other_v_quant_type="uf8")),
    ("err-opt-ctype", "llama", dict(preset="came", other_c_quant_type="al4")),
    ("err-opt-lr", "llama", dict(preset="adamw", other_lr=-1.0)),
    ("err-opt-lr-none", "llama", dict(preset="adamw", other_lr=None)),
    ("err-opt-quantize", "llama", dict(preset="adamw", other_quantize="yes")),
    ("err-opt-block", "llama", dict(preset="adamw", other_block_size=100)),
    ("err-opt-mblock", "llama", dict(preset="adamw", other_m_block_size=30)),
    ("err-opt-min8", "llama", dict(preset="adamw", other_min_8bit_size=-1)),
    ("err-opt-sr", "llama", dict(preset="adamw", other_stochastic_round_writeback=1)),
    ("err-policy-type", "llama", dict(preset="adamw", policy=[1])),
    ("err-policy-section", "llama", dict(preset="adamw", policy={"routes": {}})),
    ("err-policy-option", "llama", dict(preset="adamw", policy={"defaults": {"momentum": 0.9}})),
    ("err-policy-shadow", "llama", dict(preset="adamw", policy={"presets": {"adamw": {"preset": "sgd"}}})),
    ("err-policy-noparent", "llama", dict(preset="adamw", policy={"presets": {"mine": {"lr": 1.0}}})),
    ("err-policy-cycle", "llama", dict(preset="adamw", policy={"presets": {"a": {"preset": "b"}, "b": {"preset": "a"}}})),
    ("err-policy-route", "llama", dict(preset="adamw", policy={"mapping": {"attention": {"lr": 1.0}}})),
    ("err-policy-unknown-preset", "llama", dict(preset="adamw", policy={"mapping": {"other": {"preset": "nope"}}})),
    ("err-policy-rank", "llama", dict(preset="adamw", policy={"mapping": {"one_d": {"apollo_rank": 4}}})),
    ("err-policy-cycle3", "llama", dict(preset="adamw", policy={"presets": {"a": {"preset": "b"}, "b": {"preset": "c"}, "c": {"preset": "a"}}})),
    ("err-policy-parent-type", "llama", dict(preset="adamw", policy={"presets": {"a": {"preset": 5}}})),
    ("err-policy-parent-list", "llama", dict(preset="adamw", policy={"presets": {"a": {"preset": ["x"]}}})),
    ("err-policy-empty-name", "llama", dict(preset="adamw", policy={"presets": {"": {"preset": "adamw"}}})),
    ("err-policy-entry-type", "llama", dict(preset="adamw", policy={"mapping": {"other": 3}})),
    ("err-policy-definition-type", "llama", dict(preset="adamw", policy={"presets": {"a": 3}})),
    ("err-policy-unknown-parent", "llama", dict(preset="adamw", policy={"presets": {"a": {"preset": "zzz"}}})),
    ("policy-chain", "llama", dict(preset="adamw", policy={"presets": {"a": {"preset": "adamw", "lr": 1e-4}, "b": {"preset": "a", "beta1": 0.8}},
                                                            "mapping": {"other": {"preset": "b", "weight_decay": 0.1}}})),
    ("err-model", None, dict(preset="adamw")),
]


def param_names(model):
    """id(param) -> first name under which named_parameters reports it."""
    names = {}
    for name, p in model.named_parameters(remove_duplicate=False):
        names.setdefault(id(p), name)
    return names


def normalise(value):
    """JSON-comparable form of a group option."""
    if isinstance(value, (tuple, list)):
        return [normalise(v) for v in value]
    if isinstance(value, dict):
        return {k: normalise(v) for k, v in value.items()}
    return value


def run_scenario(build_param_groups, model_key, kwargs):
    """-> {"error": type name} or {"groups": [...], "warnings": n}."""
    import warnings
    if model_key is None:
        model, names = [torch.nn.Parameter(torch.zeros(2, 2))], {}
    else:
        torch.manual_seed(0)
        model = MODELS[model_key]()
        names = param_names(model)
    kwargs = dict(kwargs)
    preset = kwargs.pop("preset")
    with warnings.catch_warnings(record=True) as caught:
        warnings.simplefilter("always")
        try:
            groups = build_param_groups(model, preset, **kwargs)
        except (TypeError, ValueError) as e:
            return {"error": type(e).__name__}
    out = []
    for g in groups:
        rec = {k: normalise(v) for k, v in g.items() if k != "params"}
        rec["params"] = [names[id(p)] for p in g["params"]]
        out.append(rec)
    return {"groups": out, "warnings": sum(1 for w in caught if issubclass(w.category, UserWarning))}
