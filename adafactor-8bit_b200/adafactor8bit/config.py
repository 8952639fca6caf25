"""Dictionary policies laid over the groups that build_param_groups generates.

Host-side mirror of the reference's policy module (adafactor8bit/config.py:19-108): a
policy is a mapping with up to three sections,

    defaults   constructor options applied to every group,
    presets    named option sets, each derived from a built-in preset or from another
               custom one through its "preset" entry,
    mapping    route name -> {"preset": <name>, <option>: <value>, ...},

and it is applied in the order: generated group < defaults < mapped preset < mapped
options.  Routes that a model does not have may stay in the mapping.

The two public functions keep the reference's names, argument meaning, exception types and
messages; the work is done by one object, `_Policy`, that parses the three sections once,
checks them, and resolves preset chains with a memo.
"""
from copy import deepcopy
from inspect import signature
from typing import Any, Dict, List, Mapping

from .optimizer import Adafactor8Bit
from .presets import PRESETS
from .routing import _ROUTE_NAMES, _validate_route_options

__all__ = ["validate_policy", "apply_policy"]

_SECTIONS = ("defaults", "presets", "mapping")
_CTOR = signature(Adafactor8Bit.__init__).parameters
_OPTION_NAMES = frozenset(_CTOR) - {"self", "params"}


def _rule_options():
    """Every option that some built-in preset decides; resolving a preset resets all of them
    to the constructor defaults before the preset's own values go on top."""
    names = {"apollo_rank"}
    for spec in PRESETS.values():
        for part in (spec.primary, spec.fallback or {}):
            names.update(part)
    return frozenset(names)


_RULE_OPTIONS = _rule_options()


class _Policy:
    def __init__(self, policy):
        if not isinstance(policy, Mapping):
            raise TypeError("policy must be a mapping")
        stray = sorted(k for k in policy if k not in _SECTIONS)
        if stray:
            raise TypeError(f"Unknown policy sections: {stray}")
        self.defaults = policy.get("defaults", {})
        self.custom = policy.get("presets", {})
        self.mapping = policy.get("mapping", {})
        self._memo: Dict[str, Dict[str, Any]] = {}

    # -- checks ------------------------------------------------------------------------------
    @staticmethod
    def _options(options, where, drop_parent=False):
        if not isinstance(options, Mapping):
            raise TypeError(f"{where} must be a mapping")
        if drop_parent:
            options = {k: v for k, v in options.items() if k != "preset"}
        unknown = sorted(k for k in options if k not in _OPTION_NAMES)
        if unknown:
            raise TypeError(f"Unknown optimizer options in {where}: {unknown}")
        _validate_route_options(where, options)

    def check(self):
        self._options(self.defaults, "policy.defaults")
        if not (isinstance(self.custom, Mapping) and isinstance(self.mapping, Mapping)):
            raise TypeError("policy.presets and policy.mapping must be mappings")
        for name, definition in self.custom.items():
            if not (isinstance(name, str) and name):
                raise TypeError("Custom preset names must be non-empty strings")
            if name in PRESETS:
                raise ValueError(f"Custom preset {name!r} shadows a built-in; choose a distinct name")
            if not isinstance(definition, Mapping):
                raise TypeError(f"Custom preset {name!r} must be a mapping")
            self._options(definition, f"presets.{name}", drop_parent=True)
        for name in self.custom:
            self.options_of(name)
        for route, entry in self.mapping.items():
            if route not in _ROUTE_NAMES:
                raise ValueError(f"Unknown policy route {route!r}; expected one of {sorted(_ROUTE_NAMES)}")
            if not isinstance(entry, Mapping):
                raise TypeError(f"mapping.{route} must be a mapping")
            self._options(entry, f"mapping.{route}", drop_parent=True)
            if "preset" in entry:
                self.options_of(entry["preset"])
        return self

    # -- preset chains ------------------------------------------------------------------------
    def options_of(self, name) -> Dict[str, Any]:
        """Options of a built-in or custom preset: walk up to the built-in ancestor, then lay the
        custom definitions on top, oldest first."""
        if not isinstance(name, str):
            raise TypeError("Policy preset names must be strings")
        if name in self._memo:
            return deepcopy(self._memo[name])
        chain = []                                   # custom presets from `name` up to the built-in one
        cursor = name
        while True:
            if not isinstance(cursor, str):
                raise TypeError("Policy preset names must be strings")
            if cursor in PRESETS:
                break
            if cursor not in self.custom:
                raise ValueError(f"Unknown policy preset {cursor!r}")
            if cursor in chain:
                raise ValueError(f"Cyclic policy preset inheritance: {' -> '.join((*chain, cursor))}")
            chain.append(cursor)
            cursor = dict(self.custom[cursor]).get("preset")
            if cursor is None:
                raise ValueError(f"Custom preset {chain[-1]!r} requires a base 'preset'")
        spec = PRESETS[cursor]
        options = {k: deepcopy(_CTOR[k].default) for k in _RULE_OPTIONS}
        options.update(deepcopy(spec.primary))
        options["apollo_rank"] = spec.default_apollo_rank
        for link in reversed(chain):
            options.update(deepcopy({k: v for k, v in self.custom[link].items() if k != "preset"}))
        self._memo[name] = deepcopy(options)
        return options

    # -- application ---------------------------------------------------------------------------
    def overlay(self, group: Dict[str, Any]) -> Dict[str, Any]:
        merged = dict(group)
        merged.update(deepcopy(dict(self.defaults)))
        entry = dict(self.mapping.get(group["group_name"], {}))
        parent = entry.pop("preset", None)
        if parent is not None:
            merged.update(self.options_of(parent))
        merged.update(deepcopy(entry))
        rank = merged.get("apollo_rank", 0)
        if isinstance(rank, bool) or not isinstance(rank, int) or rank < 0:
            raise ValueError("apollo_rank must be an integer >= 0")
        if rank and any(p.ndim != 2 or min(p.shape) < rank for p in merged["params"]):
            raise ValueError(f"Route {group['group_name']!r} contains parameters ineligible for APOLLO rank {rank}")
        return merged


def validate_policy(policy: Mapping[str, Any]) -> None:
    """Check a (possibly partial) policy; no model is inspected or changed."""
    _Policy(policy).check()


def apply_policy(groups: List[Dict[str, Any]], policy: Mapping[str, Any]) -> List[Dict[str, Any]]:
    """New group dicts with the policy applied; parameter identity and order are kept."""
    checked = _Policy(policy).check()
    return [checked.overlay(group) for group in groups]
