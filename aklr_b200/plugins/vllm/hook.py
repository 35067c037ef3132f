"""``@vllm_route``: how a vLLM call reaches the ops.

vLLM compiles most models' forward, so Python there runs once while tracing; a route therefore
replaces a function that a vLLM function looks up *when it runs* (inside one of vLLM's opaque
custom ops), as the reference's does (aklr/plugins/vllm/hook.py:48-193).  Routes are declared per
(caller, callee) and per tested vLLM release; routes of one ``group`` install together or not at
all; the route must take the callee's parameters; ``restore`` puts every original back.
"""

from __future__ import annotations

import inspect
import logging
import pkgutil
from collections.abc import Callable
from dataclasses import dataclass
from importlib.metadata import version

import torch
from packaging.version import Version

from aklr_b200.core import dispatch
from aklr_b200.core.dispatch import FallbackReason

__all__ = ["install", "original", "restore", "vllm_route"]

_LOGGER = logging.getLogger(__name__)


@dataclass(frozen=True)
class _Route:
    caller: str
    versions: tuple[str, ...]
    group: str | None


_ROUTES: dict[Callable, dict[str, _Route]] = {}
_INSTALLED: dict[str, tuple[object, str, Callable]] = {}  # callee -> (owner, attribute, original)


def vllm_route(caller: str, *callees: str, versions: tuple[str, ...], group: str | None = None):
    """Declare that vLLM's ``caller`` reaches the ops through this function where it calls
    ``callees`` (dotted names it looks up at run time), on the releases ``versions``."""

    def declare(route: Callable) -> Callable:
        declaration = _Route(caller, versions, group)
        targets = _ROUTES.setdefault(route, {})
        for callee in callees:
            if callee in targets and targets[callee] != declaration:
                raise ValueError(f"{callee}: conflicting declaration for route {route.__qualname__}")
            targets[callee] = declaration
        return route

    return declare


def vllm_version() -> str:
    return Version(version("vllm")).public


def _parameters(fn: Callable) -> list[tuple[str, object]]:
    return [(p.name, p.kind) for p in inspect.signature(fn).parameters.values()]


def install() -> list[str]:
    """Validate the routes tested on the installed vLLM, then bind them all; returns the callees."""
    installed = vllm_version()
    blocked_groups = {
        d.group for targets in _ROUTES.values() for d in targets.values()
        if d.group is not None and installed not in d.versions
    }
    plan, untested, blocked = [], [], []
    for route, targets in _ROUTES.items():
        for callee, declaration in targets.items():
            if installed not in declaration.versions:
                untested.append(declaration.caller)
                continue
            if declaration.group in blocked_groups:
                blocked.append(f"{declaration.caller} (group={declaration.group})")
                continue
            caller_fn = pkgutil.resolve_name(declaration.caller)
            attribute = callee.rsplit(".", 1)[-1]
            if f"{attribute}(" not in inspect.getsource(caller_fn):
                raise RuntimeError(f"{declaration.caller} does not call {callee}")
            owner_name, _, _ = callee.rpartition(".")
            owner = pkgutil.resolve_name(owner_name)
            orig = getattr(owner, attribute)
            if _parameters(route) != _parameters(orig):
                raise RuntimeError(f"{callee}: route {route.__qualname__} has incompatible parameters")
            plan.append((callee, owner, attribute, orig, route))
    # everything validated: bind the batch
    for callee, owner, attribute, orig, route in plan:
        if callee in _INSTALLED:
            continue
        setattr(owner, attribute, _around(route, orig, callee))
        _INSTALLED[callee] = (owner, attribute, orig)
    notes = []
    if untested:
        notes.append(f"untested callers: {', '.join(dict.fromkeys(untested))}")
    if blocked:
        notes.append(f"blocked by untested group members: {', '.join(dict.fromkeys(blocked))}")
    _LOGGER.warning("aklr_b200 hooks %d calls of vLLM %s%s", len(plan), installed, f"; {'; '.join(notes)}" if notes else "")
    return [p[0] for p in plan]


def restore() -> None:
    """Put every original callable back."""
    for owner, attribute, orig in _INSTALLED.values():
        setattr(owner, attribute, orig)
    _INSTALLED.clear()


def original(callee: str) -> Callable:
    """The callable ``callee`` named before its route was installed."""
    return _INSTALLED[callee][2]


def _around(route: Callable, orig: Callable, callee: str) -> Callable:
    route_name = f"{route.__module__}.{route.__qualname__}"

    def hooked(*args, **kwargs):
        # Dynamo would trace the dispatch lookup and recompile per shape: compiled regions keep vLLM's code
        if not torch.compiler.is_compiling():
            result = route(*args, **kwargs)
            fallback = result if isinstance(result, FallbackReason) else None
            if (tracer := dispatch.trace()) is not None and tracer.is_plugin:
                tracer.plugin("vllm", callee, route_name, fallback)
            if fallback is None:
                return result
        return orig(*args, **kwargs)

    hooked.__wrapped__ = orig
    hooked.__name__ = getattr(orig, "__name__", "hooked")
    return hooked
