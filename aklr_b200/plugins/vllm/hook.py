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


def _calling_convention(fn: Callable) -> list[tuple[str, object]]:
    """Parameter names and kinds: what a replacement must share with the function it replaces."""
    return [(p.name, p.kind) for p in inspect.signature(fn).parameters.values()]


@dataclass(frozen=True)
class _Binding:
    """One validated replacement, ready to be set: ``owner.attribute`` is ``callee``."""

    callee: str
    owner: object
    attribute: str
    replaced: Callable
    route: Callable

    @classmethod
    def check(cls, route: Callable, callee: str, caller: str) -> "_Binding":
        """Resolve ``callee`` and make sure replacing it can take effect and cannot break the caller:
        ``caller``'s source must mention the callee's name followed by "(", and the route must take
        the callee's parameters."""
        owner_path, _, attribute = callee.rpartition(".")
        if f"{attribute}(" not in inspect.getsource(pkgutil.resolve_name(caller)):
            raise RuntimeError(f"{caller} does not call {callee}")
        owner = pkgutil.resolve_name(owner_path)
        replaced = getattr(owner, attribute)
        if _calling_convention(route) != _calling_convention(replaced):
            raise RuntimeError(f"{callee}: route {route.__qualname__} has incompatible parameters")
        return cls(callee, owner, attribute, replaced, route)

    def apply(self) -> None:
        if self.callee not in _INSTALLED:
            setattr(self.owner, self.attribute, _around(self.route, self.replaced, self.callee))
            _INSTALLED[self.callee] = (self.owner, self.attribute, self.replaced)


def _declarations():
    for route, targets in _ROUTES.items():
        for callee, declaration in targets.items():
            yield route, callee, declaration


def install() -> list[str]:
    """Bind every route that stands on the installed vLLM; returns the callees replaced.

    Two passes, so that a failed check leaves vLLM untouched: first every declaration is sorted into
    untested (its versions do not name the installed release), held back (a member of its group is
    untested: a group replaces cooperating functions and half of one is worse than none) or checked
    into a ``_Binding``; then the bindings are applied."""
    release = vllm_version()
    partial_groups = {
        declaration.group
        for _, _, declaration in _declarations()
        if declaration.group is not None and release not in declaration.versions
    }
    bindings: list[_Binding] = []
    skipped: dict[str, list[str]] = {"untested callers": [], "blocked by untested group members": []}
    for route, callee, declaration in _declarations():
        if release not in declaration.versions:
            skipped["untested callers"].append(declaration.caller)
        elif declaration.group in partial_groups:
            skipped["blocked by untested group members"].append(f"{declaration.caller} (group={declaration.group})")
        else:
            bindings.append(_Binding.check(route, callee, declaration.caller))
    for binding in bindings:
        binding.apply()
    notes = "".join(f"; {what}: {', '.join(dict.fromkeys(who))}" for what, who in skipped.items() if who)
    _LOGGER.warning("aklr_b200: %d vLLM calls hooked on vLLM %s%s", len(bindings), release, notes)
    return [binding.callee for binding in bindings]


def restore() -> None:
    """Undo ``install``: every replaced attribute gets its original value back."""
    while _INSTALLED:
        _, (owner, attribute, replaced) = _INSTALLED.popitem()
        setattr(owner, attribute, replaced)


def original(callee: str) -> Callable:
    """What ``callee`` named before ``install`` replaced it."""
    return _INSTALLED[callee][2]


def _around(route: Callable, orig: Callable, callee: str) -> Callable:
    """``orig`` with ``route`` tried first.  Inside a ``torch.compile`` trace the route is not tried:
    dynamo would trace the dispatch lookup and recompile per shape, so compiled regions keep vLLM's
    own function."""
    label = f"{route.__module__}.{route.__qualname__}"

    def hooked(*args, **kwargs):
        if torch.compiler.is_compiling():
            return orig(*args, **kwargs)
        answer = route(*args, **kwargs)
        declined = isinstance(answer, FallbackReason)
        tracer = dispatch.trace()
        if tracer is not None and tracer.is_plugin:
            tracer.plugin("vllm", callee, label, answer if declined else None)
        return orig(*args, **kwargs) if declined else answer

    hooked.__wrapped__ = orig
    hooked.__name__ = getattr(orig, "__name__", "hooked")
    return hooked
