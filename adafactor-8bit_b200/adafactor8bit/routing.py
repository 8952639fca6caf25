"""build_param_groups: turn a model into optimizer parameter groups by parameter role.

Host-side mirror of the reference's guided API (adafactor8bit/routing.py:534-789): the
same signature, route names, grouping profiles, override keys, error types and warnings,
so that group lists built for the reference optimizer can be built for this one
unchanged.  Nothing here touches a device; the groups are ordinary dicts.

How a group list comes about:

1. census   every trainable Parameter once, with all the names it is reachable under
            (tied weights have several) and the modules that own it;
2. role     one_d (vectors, norm weights, biases) > embedding (token embeddings, also a
            tied embedding/LM-head weight) > lm_head > matrix (2-D) > nd;
3. APOLLO   on APOLLO-capable presets a parameter moves to the "apollo" route when its
            name matches a target, its shape admits the rank and its role is not
            protected (embedding / lm_head only on explicit request);
4. layout   the grouping profile (G0 bare, G1 protected, G2 topology) maps roles to
            routes and gives each route its options; route overrides
            (`<route>_<option>=...`) and an optional policy are laid on top.
"""
from __future__ import annotations

import warnings
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Mapping, Optional, Sequence, Tuple, Union

from torch import nn

from .presets import PRESETS, PresetSpec, _preset_names

__all__ = ["build_param_groups"]

ROUTES = ("all", "fallback", "other", "one_d", "embedding", "lm_head", "apollo", "matrix", "nd")
_ROUTE_NAMES = frozenset(ROUTES)
_PROTECTED = ("one_d", "embedding", "lm_head")
_GROUPINGS = {"G0": "G0", "g0": "G0", "bare": "G0", "G1": "G1", "g1": "G1", "protected": "G1",
              "G2": "G2", "g2": "G2", "topology": "G2"}

M_FORMATS = ("fp32", "uf4", "uf8", "d4", "d8")
VC_FORMATS = ("fp32", "al8", "al16")

# `<route>_<option>` keys; an option that is a suffix of another one comes after it
ROUTE_OPTIONS = ("m_quant_type", "v_quant_type", "c_quant_type", "stochastic_round_writeback",
                 "min_8bit_size", "m_block_size", "block_size", "quantize", "lr")
# rule options that reach both the primary route and its fallback ...
SHARED_RULE_KEYS = frozenset((
    "beta1", "beta2", "beta2_decay", "bias_correction", "relative_step", "scale_parameter",
    "scale_weight_decay", "d", "eps", "fira_margin", "lag_norm", "momentum_only_1d",
    "enable_fira_for_adafactor", "stochastic_round_writeback"))
# ... and those that only make sense on the primary one (confidence and APOLLO controls)
PRIMARY_RULE_KEYS = frozenset((
    "beta3", "eps_came", "apollo_factorize", "apollo_update_proj_gap", "apollo_scale_type",
    "apollo_scale", "apollo_scale_front", "apollo_eps", "apollo_cache_proj", "enable_fira_for_apollo"))
_PRECISION_KEYS = ("m_quant_type", "v_quant_type", "c_quant_type", "min_8bit_size", "m_block_size", "block_size")


# ----------------------------------------------------------------------------
# option validation (shared with the policy module)
# ----------------------------------------------------------------------------
def _is_int(v):
    return isinstance(v, int) and not isinstance(v, bool)


# option -> (exception type, predicate, what is expected)
_OPTION_RULES: Dict[str, Tuple[type, Callable[[Any], bool], str]] = {
    "stochastic_round_writeback": (TypeError, lambda v: isinstance(v, bool), "must be bool"),
    "m_quant_type": (ValueError, lambda v: v in M_FORMATS, f"must be one of {sorted(M_FORMATS)}"),
    "v_quant_type": (ValueError, lambda v: v in VC_FORMATS, f"must be one of {sorted(VC_FORMATS)}"),
    "c_quant_type": (ValueError, lambda v: v is None or v in VC_FORMATS, f"must be None or one of {sorted(VC_FORMATS)}"),
    "lr": (ValueError, lambda v: isinstance(v, (int, float)) and not isinstance(v, bool) and v >= 0, "must be a number >= 0"),
    "quantize": (TypeError, lambda v: isinstance(v, bool) or (isinstance(v, str) and v.lower() == "auto"),
                 "must be True, False or 'auto'"),
    "block_size": (ValueError, lambda v: _is_int(v) and v >= 128 and v % 128 == 0, "must be >= 128 and a multiple of 128"),
    "m_block_size": (ValueError, lambda v: _is_int(v) and v >= 32 and v % 4 == 0, "must be >= 32 and a multiple of 4"),
    "min_8bit_size": (ValueError, lambda v: _is_int(v) and v >= 0, "must be an integer >= 0"),
}


def _validate_route_options(route: str, opts: Mapping[str, Any]) -> None:
    """Type / range check of the per-route options present in `opts` (routing.py:238-293)."""
    for key, (exc, accepts, expected) in _OPTION_RULES.items():
        if key in opts and not accepts(opts[key]):
            raise exc(f"{route}_{key}={opts[key]!r} {expected}")


def _split_overrides(overrides: Mapping[str, Any]):
    """**overrides of build_param_groups -> (rule options, {route: {option: value}})."""
    rule: Dict[str, Any] = {}
    per_route: Dict[str, Dict[str, Any]] = {}
    for key, value in overrides.items():
        if key in SHARED_RULE_KEYS or key in PRIMARY_RULE_KEYS:
            rule[key] = value
            continue
        option = next((o for o in ROUTE_OPTIONS if key.endswith("_" + o)), None)
        if option is None:
            if key == "factored":
                raise TypeError("'factored' is decided per route by build_param_groups(); edit the returned group "
                                "dict to override it")
            raise TypeError(f"Unknown build_param_groups() override: {key!r}")
        route = key[:-(len(option) + 1)]
        if route not in _ROUTE_NAMES:
            raise TypeError(f"Unknown route prefix {route!r} in {key!r}. Known routes: {sorted(_ROUTE_NAMES)}")
        per_route.setdefault(route, {})[option] = value
    for route, opts in per_route.items():
        _validate_route_options(route, opts)
    return rule, per_route


# ----------------------------------------------------------------------------
# census and roles
# ----------------------------------------------------------------------------
_NORM_TYPES = tuple(getattr(nn, n) for n in (
    "BatchNorm1d", "BatchNorm2d", "BatchNorm3d", "SyncBatchNorm", "InstanceNorm1d", "InstanceNorm2d",
    "InstanceNorm3d", "LayerNorm", "GroupNorm", "LocalResponseNorm", "RMSNorm") if hasattr(nn, n))
_NOT_TOKEN_EMBEDDING = ("position", "pos_embed", "wpe", "time")


def _may_be_token_embedding(name: str) -> bool:
    low = name.lower()
    return not any(tag in low for tag in _NOT_TOKEN_EMBEDDING)


@dataclass
class _Entry:
    """One trainable Parameter and every (name, owning module, attribute name) it has."""
    param: nn.Parameter
    names: List[str] = field(default_factory=list)
    owners: List[nn.Module] = field(default_factory=list)
    attrs: List[str] = field(default_factory=list)

    @property
    def embedding_names(self) -> Tuple[str, ...]:
        out = []
        for name, owner in zip(self.names, self.owners):
            low = name.lower()
            by_type = isinstance(owner, nn.Embedding) and _may_be_token_embedding(name)
            by_name = _may_be_token_embedding(name) and ("embed" in low or "wte" in low)
            if by_type or by_name:
                out.append(name)
        return tuple(out)

    @property
    def lm_head_names(self) -> Tuple[str, ...]:
        return tuple(n for n in self.names if "lm_head" in n.lower())

    @property
    def role(self) -> str:
        p = self.param
        if p.ndim <= 1 or any(isinstance(m, _NORM_TYPES) for m in self.owners) or any(a.lower() == "bias" for a in self.attrs):
            return "one_d"
        if self.embedding_names:          # a weight tied to the LM head keeps the embedding role
            return "embedding"
        if self.lm_head_names:
            return "lm_head"
        return "matrix" if p.ndim == 2 else "nd"


def _census(model: nn.Module) -> List[_Entry]:
    entries: Dict[int, _Entry] = {}
    try:
        modules = list(model.named_modules(remove_duplicate=False))
    except TypeError:
        modules = list(model.named_modules())
    for mod_name, module in modules:
        for attr, p in module.named_parameters(recurse=False):
            if not p.requires_grad:
                continue
            e = entries.setdefault(id(p), _Entry(p))
            e.names.append(f"{mod_name}.{attr}" if mod_name else attr)
            e.owners.append(module)
            e.attrs.append(attr)
    # parameters that only the recursive listing reports
    for name, p in model.named_parameters():
        if p.requires_grad and id(p) not in entries:
            entries[id(p)] = _Entry(p, [name], [model], [name.rsplit(".", 1)[-1]])
    return list(entries.values())


def _names_hit(names: Sequence[str], targets: Sequence[str]) -> bool:
    lows = [n.lower() for n in names]
    return any(t.lower() in n for t in targets for n in lows)


# ----------------------------------------------------------------------------
# groups
# ----------------------------------------------------------------------------
def _fullrank(sem: Mapping[str, Any], drop_momentum: bool = False) -> Dict[str, Any]:
    """The full-rank variant of a rule, used by G2 for embeddings, LM heads and N-D tensors."""
    out = dict(sem, factored=False, scale_parameter=False, d=0.0, beta3=None)
    if drop_momentum:
        out["beta1"] = None
    return out


def _default_quantize(preset: str, grouping: str, route: str, auto_profile: bool) -> Optional[bool]:
    """The builder's own `quantize` for a route; None = inherit the optimizer's setting
    (routing.py:358-391)."""
    if grouping == "G1":
        if route == "one_d":
            return False
        if route in ("embedding", "lm_head"):
            if not auto_profile:                       # an explicit G1 protects both for every preset
                return False
            return False if preset in ("adafactor", "rmsprop") else None
    if grouping == "G2" and route in ("one_d", "embedding"):
        return False
    return None


@dataclass
class _Slot:
    route: str
    semantics: Mapping[str, Any]
    no_weight_decay: bool = False
    rank: Optional[int] = None


def _layout(grouping: str, apollo_preset: bool, primary, fallback, rank: int, nd_factored: bool) -> List[_Slot]:
    rest = fallback if apollo_preset else primary
    apollo = [_Slot("apollo", primary, rank=rank)] if apollo_preset else []
    if grouping == "G0":
        return apollo + [_Slot("fallback", fallback)] if apollo_preset else [_Slot("all", primary)]
    if grouping == "G1":
        return [_Slot(r, rest, no_weight_decay=True) for r in _PROTECTED] + apollo + [_Slot("other", rest)]
    return ([_Slot("one_d", rest, no_weight_decay=True),
             _Slot("embedding", _fullrank(rest, drop_momentum=True), no_weight_decay=True),
             _Slot("lm_head", _fullrank(rest), no_weight_decay=True)]
            + apollo
            + [_Slot("matrix", rest), _Slot("nd", dict(rest) if nd_factored else _fullrank(rest))])


def _route_of(grouping: str, apollo_preset: bool, role: str, use_apollo: bool) -> str:
    if use_apollo:
        return "apollo"
    if grouping == "G0":
        return "fallback" if apollo_preset else "all"
    if grouping == "G1":
        return role if role in _PROTECTED else "other"
    return role


def _make_group(slot: _Slot, params: List[nn.Parameter], route_opts: Mapping[str, Mapping[str, Any]],
                preset: str, grouping: str, auto_profile: bool) -> Dict[str, Any]:
    group: Dict[str, Any] = dict(params=list(params), group_name=slot.route)
    group.update(slot.semantics)
    group["apollo_rank"] = int(slot.rank) if slot.rank is not None else 0
    if slot.no_weight_decay:
        group["weight_decay"] = 0.0
    given = dict(route_opts.get(slot.route, {}))
    asked = given.pop("quantize", "auto")
    quantize = asked if isinstance(asked, bool) else _default_quantize(preset, grouping, slot.route, auto_profile)
    if quantize is not None:
        group["quantize"] = quantize
    if quantize is False and not isinstance(asked, bool) and any(k in given for k in _PRECISION_KEYS):
        warnings.warn(f"Route {slot.route!r} is unquantized by its auto policy, so its explicit precision / block "
                      f"options stay inactive unless {slot.route}_quantize=True is set as well.", UserWarning, stacklevel=3)
    group.update(given)
    if group.get("quantize", True):
        if group.get("beta1") is None and ("m_quant_type" in given or "m_block_size" in given):
            warnings.warn(f"Route {slot.route!r} has beta1=None, so its explicit M-state options are inactive.",
                          UserWarning, stacklevel=3)
        if group.get("beta3") is None and "c_quant_type" in given:
            warnings.warn(f"Route {slot.route!r} has beta3=None, so its explicit C-state option is inactive.",
                          UserWarning, stacklevel=3)
    return group


# ----------------------------------------------------------------------------
# argument resolution
# ----------------------------------------------------------------------------
def _resolve_grouping(spec: PresetSpec, grouping) -> Tuple[str, bool]:
    if grouping is None:
        raise TypeError("grouping=None is ambiguous; use 'auto' or G0/G1/G2")
    if isinstance(grouping, str) and grouping.lower() == "auto":
        return spec.default_grouping, True
    key = _GROUPINGS.get(str(grouping))
    if key is None:
        raise ValueError(f"Unknown grouping {grouping!r}; use 'auto', G0/bare, G1/protected or G2/topology.")
    return key, False


def _resolve_targets(spec: PresetSpec, value) -> Tuple[Optional[Tuple[str, ...]], bool]:
    """-> (targets or None for "any name", whether the caller listed them)."""
    if isinstance(value, str):
        if value.lower() != "auto":
            raise TypeError("apollo_targets must be 'auto' or a sequence such as ['attn', 'mlp']")
        return (None if spec.default_apollo_targets is None else tuple(spec.default_apollo_targets)), False
    if value is None:
        raise TypeError("apollo_targets=None is ambiguous; use 'auto' or an explicit sequence")
    targets = tuple(value)
    if any(not isinstance(t, str) or not t for t in targets):
        raise TypeError("apollo_targets entries must be non-empty strings")
    return targets, True


def _resolve_apollo(spec: PresetSpec, preset: str, apollo_rank, apollo_targets, apollo_min_dim_multiplier):
    """-> (rank, targets, explicit_targets, min_dim_multiplier)."""
    if spec.default_apollo_rank <= 0:
        for label, given in (("apollo_rank", apollo_rank is not None), ("apollo_targets", apollo_targets != "auto"),
                             ("apollo_min_dim_multiplier", apollo_min_dim_multiplier != "auto")):
            if given:
                raise ValueError(f"{label} requires an APOLLO-capable preset; got {preset!r}")
        return 0, (), False, 1
    rank = spec.default_apollo_rank
    if apollo_rank is not None:
        if not _is_int(apollo_rank):
            raise TypeError("apollo_rank must be an integer >= 0 or None")
        rank = apollo_rank
    if rank < 0:
        raise ValueError("apollo_rank must be >= 0")
    targets, explicit = _resolve_targets(spec, apollo_targets)
    mult = apollo_min_dim_multiplier
    if isinstance(mult, str) and mult.lower() == "auto":
        mult = spec.default_apollo_min_dim_multiplier
    elif not _is_int(mult) or mult < 1:
        raise ValueError("apollo_min_dim_multiplier must be 'auto' or an integer >= 1")
    if rank == 0:
        if explicit and targets:
            warnings.warn("apollo_rank=0 disables APOLLO; explicit apollo_targets are ignored.", UserWarning, stacklevel=3)
        targets = ()
    return rank, targets, explicit, mult


# ----------------------------------------------------------------------------
# the builder
# ----------------------------------------------------------------------------
def build_param_groups(
    model: nn.Module,
    preset: str,
    grouping: str = "auto",
    *,
    apollo_rank: Optional[int] = None,
    apollo_targets: Union[str, Sequence[str]] = "auto",
    apollo_min_dim_multiplier: Union[str, int] = "auto",
    nd_factored: Optional[bool] = None,
    policy: Optional[Mapping[str, Any]] = None,
    **overrides: Any,
) -> List[Dict[str, Any]]:
    """Parameter groups (plain, mutable dicts) for Adafactor8Bit.

    preset        one of sgd / adafactor / adamw / rmsprop / came / apollo.
    grouping      "auto" (the preset's default topology with preset-aware quantisation
                  defaults), "G0"/"bare", "G1"/"protected", "G2"/"topology".
    apollo_*      only with an APOLLO-capable preset: rank (None = preset default, 0 = off),
                  name targets ("auto" or a sequence of substrings) and the factor by which
                  the smaller dimension must exceed the rank.
    nd_factored   G2 only: keep the factored rule for tensors of more than two dimensions.
    policy        optional {"defaults", "presets", "mapping"} overlay (see config.apply_policy).
    **overrides   rule options (beta1, eps, d, ...) and `<route>_<option>` route options.

    Parameter values and dtypes are never changed.  Reference: routing.py:534-789.
    """
    if not isinstance(model, nn.Module):
        raise TypeError("build_param_groups() expects an nn.Module, not model.parameters()")
    preset_key = str(preset).lower()
    if preset_key not in PRESETS:
        raise ValueError(f"Unknown preset {preset!r}. Available presets: {', '.join(_preset_names())}")
    spec = PRESETS[preset_key]
    grouping_key, auto_profile = _resolve_grouping(spec, grouping)

    if nd_factored is not None:
        if not isinstance(nd_factored, bool):
            raise TypeError("nd_factored must be bool or None")
        if grouping_key != "G2":
            raise ValueError("nd_factored is only meaningful with G2/topology grouping")
        if nd_factored and preset_key not in ("adafactor", "came"):
            raise ValueError(f"nd_factored=True is not part of the {preset_key!r} preset semantics; use adafactor/came "
                             "or edit the returned nd group explicitly.")

    rule_overrides, route_opts = _split_overrides(overrides)
    primary = dict(spec.primary)
    fallback = dict(spec.fallback if spec.fallback is not None else spec.primary)
    for key, value in rule_overrides.items():
        primary[key] = value
        if key in SHARED_RULE_KEYS:
            fallback[key] = value

    apollo_preset = spec.default_apollo_rank > 0
    rank, targets, explicit_targets, mult = _resolve_apollo(spec, preset_key, apollo_rank, apollo_targets,
                                                            apollo_min_dim_multiplier)
    if policy is not None:
        from .config import apply_policy

    entries = _census(model)
    if not entries:
        return apply_policy([], policy) if policy is not None else []

    tied = any(e.embedding_names and e.lm_head_names for e in entries)
    tied_override_warned = False
    if "lm_head" in route_opts and tied:
        warnings.warn("A token embedding and lm_head share one Parameter. The shared tensor is routed as 'embedding', "
                      "so lm_head_* overrides do not reach it; untied lm_head parameters still use the lm_head route.",
                      UserWarning, stacklevel=2)
        tied_override_warned = True

    buckets: Dict[str, List[nn.Parameter]] = {}
    warned_tied_target = False
    for e in entries:
        role = e.role
        if targets is None:
            hit = True
        else:
            hit = bool(targets) and _names_hit(e.names, targets)
            # an explicit target that names only the LM-head alias of a tied weight must not
            # drag the shared embedding into APOLLO
            if hit and explicit_targets and role == "embedding" and e.lm_head_names and not _names_hit(e.embedding_names, targets):
                hit = False
                if not warned_tied_target:
                    warnings.warn("apollo_targets matched only the lm_head alias of a tied embedding/lm_head Parameter. "
                                  "The shared tensor stays on the embedding route unless an embedding alias is targeted.",
                                  UserWarning, stacklevel=2)
                    warned_tied_target = True
        p = e.param
        shape_ok = rank > 0 and p.ndim == 2 and min(p.shape) >= rank * mult
        allowed = role not in _PROTECTED or (explicit_targets and role in ("embedding", "lm_head"))
        use_apollo = apollo_preset and hit and shape_ok and allowed
        buckets.setdefault(_route_of(grouping_key, apollo_preset, role, use_apollo), []).append(p)

    use_nd_factored = spec.default_nd_factored if nd_factored is None else nd_factored
    groups = [
        _make_group(slot, buckets[slot.route], route_opts, preset_key, grouping_key, auto_profile)
        for slot in _layout(grouping_key, apollo_preset, primary, fallback, rank, use_nd_factored)
        if buckets.get(slot.route)
    ]

    placed = [id(p) for g in groups for p in g["params"]]
    if len(placed) != len(set(placed)) or set(placed) != {id(e.param) for e in entries}:
        raise RuntimeError("Internal routing error: parameters were duplicated or omitted")

    made = {g["group_name"] for g in groups}
    for route in route_opts:
        if route in made or (route == "lm_head" and tied_override_warned):
            continue
        warnings.warn(f"Route override for {route!r} did not match a generated group.", UserWarning, stacklevel=2)

    if policy is not None:
        groups = apply_policy(groups, policy)
    return groups
