"""Named optimizer semantics ("presets") consumed by build_param_groups.

Mirrors the preset table of the reference package (adafactor8bit/presets.py:33-164):
the same preset names, the same option values and the same PresetSpec fields, so that
`PRESETS["adamw"].primary` can be splatted into the constructor exactly as there.  A
preset fixes which update rule a route runs; learning rate, weight decay and the state
formats stay constructor or route options.
"""
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

__all__ = ["PRESETS", "PresetSpec"]


@dataclass(frozen=True)
class PresetSpec:
    """One preset: the options of its primary route and, for presets that split the
    model (APOLLO), the options of every parameter the primary route does not take."""
    name: str
    default_grouping: str
    primary: Dict[str, Any]
    fallback: Optional[Dict[str, Any]] = None
    default_apollo_rank: int = 0
    default_apollo_targets: Optional[Tuple[str, ...]] = None
    default_apollo_min_dim_multiplier: int = 1
    default_nd_factored: bool = False


def _plain(**changes):
    """Options shared by every non-factored, fixed-step rule, with `changes` on top."""
    base = dict(beta1=None, beta2=None, beta2_decay=None, beta3=None, factored=False,
                relative_step=False, scale_parameter=False, scale_weight_decay=False, d=0.0)
    base.update(changes)
    return base


_ADAM_EPS = (1e-8, 1e-3)
_APOLLO_EPS = (1e-6, 1e-3)        # the APOLLO routes, target and fallback alike, use the larger eps1

_TABLE = {
    # plain SGD: no moments at all
    "sgd": dict(primary=_plain()),
    # factored second moment with the decaying beta2 schedule, no momentum; the remaining
    # Adafactor switches (parameter scaling, clipping) keep their constructor defaults
    "adafactor": dict(primary=dict(beta1=None, beta2=None, beta2_decay=-0.8, beta3=None,
                                   factored=True, relative_step=False)),
    "adamw": dict(primary=_plain(beta1=0.9, beta2=0.999, eps=_ADAM_EPS)),
    "rmsprop": dict(primary=_plain(beta2=0.99, eps=_ADAM_EPS)),
    # confidence-guided factored rule
    "came": dict(primary=_plain(beta1=0.9, beta2=0.999, beta3=0.9999, factored=True, d=1.0, eps_came=1e-16)),
    # low-rank scaling on the target matrices, Adam-style everywhere else
    "apollo": dict(
        primary=_plain(beta1=0.9, beta2=0.999, eps=_APOLLO_EPS, apollo_eps=1e-6, apollo_factorize=False,
                       apollo_update_proj_gap=200, apollo_scale_type="channel", apollo_scale=1.0,
                       apollo_scale_front=False, apollo_cache_proj=True, enable_fira_for_apollo=True),
        fallback=_plain(beta1=0.9, beta2=0.999, eps=_APOLLO_EPS),
        default_apollo_rank=256,
        default_apollo_targets=("attn", "mlp"),
        default_apollo_min_dim_multiplier=1),
}

PRESETS: Dict[str, PresetSpec] = {
    name: PresetSpec(name=name, default_grouping="G1", **fields) for name, fields in _TABLE.items()
}


def _preset_names():
    return tuple(PRESETS)
