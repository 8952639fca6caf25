"""Dictionary policies laid over the groups that build_param_groups generates.

Host-side mirror of the reference's policy module (adafactor8bit/config.py:19-108): a
policy is a mapping with up to three sections,

    defaults   constructor options applied to every group,
    presets    named option sets, each derived from a built-in preset or from another
               custom one through its "preset" entry,
    mapping    route name -> {"preset": <name>, <option>: <value>, ...},

and it is applied in the order: generated group < defaults < mapped preset < mapped
options.  Routes that a model does not have may stay in the mapping.
"""
from copy import deepcopy
from inspect import signature
from typing import Any, Dict, List, Mapping

from .optimizer import Adafactor8Bit
from .presets import PRESETS
from .routing import _ROUTE_NAMES, _validate_route_options

__all__ = ["validate_policy", "apply_policy"]

_CTOR = signature(Adafactor8Bit.__init__).parameters
_OPTION_NAMES = frozenset(_CTOR) - {"self", "params"}
# every option a built-in preset decides; resolving a preset resets all of them
_RULE_OPTIONS = {"apollo_rank"}
for _spec in PRESETS.values():
    _RULE_OPTIONS.update(_spec.primary)
    _RULE_OPTIONS.update(_spec.fallback or {})


def _check_options(options, where: str) -> None:
    if not isinstance(options, Mapping):
        raise TypeError(f"{where} must be a mapping")
    unknown = sorted(set(options) - _OPTION_NAMES)
    if unknown:
        raise TypeError(f"Unknown optimizer options in {where}: {unknown}")
    _validate_route_options(where, options)


def _without_parent(definition: Mapping[str, Any]) -> Dict[str, Any]:
    return {k: v for k, v in definition.items() if k != "preset"}


def _resolve(name, custom: Mapping[str, Any], seen=()) -> Dict[str, Any]:
    """Options of a built-in or custom preset, parents first."""
    if not isinstance(name, str):
        raise TypeError("Policy preset names must be strings")
    if name in PRESETS:
        spec = PRESETS[name]
        options = {k: deepcopy(_CTOR[k].default) for k in _RULE_OPTIONS}
        options.update(deepcopy(spec.primary))
        options["apollo_rank"] = spec.default_apollo_rank
        return options
    if name not in custom:
        raise ValueError(f"Unknown policy preset {name!r}")
    if name in seen:
        raise ValueError(f"Cyclic policy preset inheritance: {' -> '.join((*seen, name))}")
    definition = dict(custom[name])
    parent = definition.pop("preset", None)
    if parent is None:
        raise ValueError(f"Custom preset {name!r} requires a base 'preset'")
    options = _resolve(parent, custom, (*seen, name))
    options.update(deepcopy(definition))
    return options


def validate_policy(policy: Mapping[str, Any]) -> None:
    """Check a (possibly partial) policy; no model is inspected or changed."""
    if not isinstance(policy, Mapping):
        raise TypeError("policy must be a mapping")
    extra = sorted(set(policy) - {"defaults", "presets", "mapping"})
    if extra:
        raise TypeError(f"Unknown policy sections: {extra}")
    _check_options(policy.get("defaults", {}), "policy.defaults")
    custom, mapping = policy.get("presets", {}), policy.get("mapping", {})
    if not isinstance(custom, Mapping) or not isinstance(mapping, Mapping):
        raise TypeError("policy.presets and policy.mapping must be mappings")
    for name, definition in custom.items():
        if not isinstance(name, str) or not name:
            raise TypeError("Custom preset names must be non-empty strings")
        if name in PRESETS:
            raise ValueError(f"Custom preset {name!r} shadows a built-in; choose a distinct name")
        if not isinstance(definition, Mapping):
            raise TypeError(f"Custom preset {name!r} must be a mapping")
        _check_options(_without_parent(definition), f"presets.{name}")
    for name in custom:
        _resolve(name, custom)
    for route, entry in mapping.items():
        if route not in _ROUTE_NAMES:
            raise ValueError(f"Unknown policy route {route!r}; expected one of {sorted(_ROUTE_NAMES)}")
        if not isinstance(entry, Mapping):
            raise TypeError(f"mapping.{route} must be a mapping")
        _check_options(_without_parent(entry), f"mapping.{route}")
        if "preset" in entry:
            _resolve(entry["preset"], custom)


def apply_policy(groups: List[Dict[str, Any]], policy: Mapping[str, Any]) -> List[Dict[str, Any]]:
    """New group dicts with the policy applied; parameter identity and order are kept."""
    validate_policy(policy)
    defaults = dict(policy.get("defaults", {}))
    custom = policy.get("presets", {})
    out = []
    for group in groups:
        merged = dict(group)
        merged.update(deepcopy(defaults))
        entry = dict(policy.get("mapping", {}).get(group["group_name"], {}))
        chosen = entry.pop("preset", None)
        if chosen is not None:
            merged.update(_resolve(chosen, custom))
        merged.update(deepcopy(entry))
        rank = merged.get("apollo_rank", 0)
        if not isinstance(rank, int) or isinstance(rank, bool) or rank < 0:
            raise ValueError("apollo_rank must be an integer >= 0")
        if rank and any(p.ndim != 2 or min(p.shape) < rank for p in merged["params"]):
            raise ValueError(f"Route {group['group_name']!r} contains parameters ineligible for APOLLO rank {rank}")
        out.append(merged)
    return out
