"""Constructor scenarios for Adafactor8Bit: keyword sets that must be accepted or refused
exactly as the reference refuses them.  Shared by gen_ctor_golden.py (records the reference's
behaviour) and tests/test_ctor.py."""
import inspect

_OK = dict(lr=1e-3)

SCENARIOS = [
    ("defaults", {}),
    ("adamw", dict(beta1=0.9, beta2=0.999, beta2_decay=None, factored=False, relative_step=False, scale_parameter=False)),
    ("came", dict(beta1=0.9, beta2=0.999, beta2_decay=None, beta3=0.9999, relative_step=False)),
    ("sgd", dict(beta2=None, beta2_decay=None, relative_step=False)),
    ("sgd-momentum", dict(beta1=0.9, beta2=None, beta2_decay=None, relative_step=False)),
    ("apollo", dict(beta1=0.9, beta2=0.999, beta2_decay=None, factored=False, relative_step=False, apollo_rank=8)),
    ("eps-none", dict(eps=(None, 1e-3))),
    ("neg-lr", dict(lr=-1.0)),
    ("beta1-high", dict(beta1=1.0)),
    ("beta1-neg", dict(beta1=-0.1)),
    ("beta2-high", dict(beta2=1.0, beta2_decay=None)),
    ("beta2-decay-pos", dict(beta2_decay=0.5)),
    ("sgd-relative", dict(beta2=None, beta2_decay=None, relative_step=True)),
    ("sgd-apollo", dict(beta2=None, beta2_decay=None, relative_step=False, apollo_rank=4)),
    ("sgd-beta3", dict(beta1=0.9, beta2=None, beta2_decay=None, relative_step=False, beta3=0.99)),
    ("eps1-neg", dict(eps=(-1e-8, 1e-3))),
    ("eps2-neg", dict(eps=(1e-8, -1e-3))),
    ("d-neg", dict(d=-1.0)),
    ("wd-neg", dict(weight_decay=-0.1)),
    ("block-small", dict(block_size=64)),
    ("block-odd", dict(block_size=200)),
    ("block-odd-unquantized", dict(block_size=200, quantize=False)),
    ("mblock-small", dict(m_block_size=16)),
    ("mblock-odd", dict(m_block_size=34)),
    ("m-type", dict(m_quant_type="int8")),
    ("v-type", dict(v_quant_type="uf8")),
    ("c-type", dict(c_quant_type="al4")),
    ("c-type-none", dict(c_quant_type=None)),
    ("block-vs-mblock", dict(beta1=0.9, block_size=256, m_block_size=96)),
    ("block-vs-mblock-no-momentum", dict(beta1=None, block_size=256, m_block_size=96)),
    ("block-vs-mblock-fp32m", dict(beta1=0.9, block_size=256, m_block_size=96, m_quant_type="fp32")),
    ("apollo-scale-type", dict(beta1=0.9, beta2=0.999, beta2_decay=None, factored=False, relative_step=False, apollo_rank=4,
                               apollo_scale_type="row")),
    ("apollo-scale-type-ignored", dict(apollo_scale_type="row")),
    ("apollo-scale-neg", dict(apollo_scale=-1.0)),
    ("fira-margin-neg", dict(fira_margin=-0.1)),
    ("beta3-high", dict(beta1=0.9, beta2=0.999, beta2_decay=None, beta3=1.0, relative_step=False)),
    ("beta3-no-momentum", dict(beta1=None, beta3=0.99)),
    ("beta3-unfactored", dict(beta1=0.9, beta2=0.999, beta2_decay=None, beta3=0.99, factored=False, relative_step=False)),
    ("beta3-unfactored-apollo", dict(beta1=0.9, beta2=0.999, beta2_decay=None, beta3=0.99, factored=False, relative_step=False,
                                     apollo_rank=4)),
]


def run_scenario(cls, kwargs):
    """-> {"ok": defaults of the created optimizer (JSON-comparable)} or {"error": type name}."""
    import warnings
    import torch
    p = torch.nn.Parameter(torch.zeros(4, 4))
    kw = dict(_OK)
    kw.update(kwargs)
    if "use_cuda_kernel" in inspect.signature(cls.__init__).parameters:
        kw.setdefault("use_cuda_kernel", False)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        try:
            opt = cls([p], **kw)
        except (ValueError, TypeError) as e:
            return {"error": type(e).__name__}
    d = {k: (list(v) if isinstance(v, tuple) else v) for k, v in opt.defaults.items()
         if isinstance(v, (int, float, str, bool, tuple, type(None)))}
    d.pop("use_cuda_kernel", None)
    return {"ok": d}


def signature_of(cls):
    """Keyword names and defaults of the constructor, JSON-comparable."""
    out = []
    for name, prm in inspect.signature(cls.__init__).parameters.items():
        if name in ("self", "params"):
            continue
        dv = prm.default
        out.append([name, list(dv) if isinstance(dv, tuple) else dv])
    return out
