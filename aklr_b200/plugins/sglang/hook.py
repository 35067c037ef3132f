"""Routes from sglang functions to the ops.

A route is declared beside the op call it makes::

    @sglang_route("sglang.srt.models.x.Block.forward_normal", versions=("0.5.23",))
    def _forward_normal(self, hidden_states): ...

and carries the same meaning as the reference's decorator of that name
(aklr/plugins/sglang/hook.py:29-103): the target is the sglang function stood in for, ``versions`` the
sglang releases the route was checked against, a returned ``FallbackReason`` hands the call back to
sglang, and inside a ``torch.compile`` trace only routes declared ``eager`` run.  ``install`` registers
an AROUND hook with sglang's ``HookRegistry`` for every declared route whose ``versions`` name the
installed release.
"""

from __future__ import annotations

import dataclasses
import importlib.util
import logging
import pkgutil
from collections.abc import Callable
from importlib.metadata import version

import torch
from packaging.version import Version

from aklr_b200.core import dispatch
from aklr_b200.core.dispatch import FallbackReason

__all__ = ["Route", "around", "install", "routes", "sglang_route", "sglang_version"]

_LOGGER = logging.getLogger(__name__)


@dataclasses.dataclass(frozen=True)
class Route:
    """One declared route: ``serve`` stands in for the sglang function at ``target``."""

    target: str
    versions: tuple[str, ...]
    serve: Callable
    eager: bool = False

    @property
    def name(self) -> str:
        return f"{self.serve.__module__}.{self.serve.__qualname__}"

    def standing(self, release: str) -> str:
        """"hook" when the route applies to sglang ``release`` and its target imports; "untested" when
        ``release`` is not among its versions; otherwise why the target is out of reach.  A target that
        vanished from a package that IS installed raises: that is a rename, and starting without the
        route would silently serve nothing."""
        if release not in self.versions:
            return "untested"
        try:
            pkgutil.resolve_name(self.target)
        except ModuleNotFoundError as missing:
            top = (missing.name or "").split(".")[0]
            if top and importlib.util.find_spec(top) is None:
                return f"{top} is not installed"
            raise
        return "hook"

    def hook(self) -> Callable:
        """The AROUND hook sglang calls as ``hook(original, *args, **kwargs)``."""

        def attempt(original, args, kwargs):
            answer = self.serve(*args, **kwargs)
            declined = isinstance(answer, FallbackReason)
            tracer = dispatch.trace()
            if tracer is not None and tracer.is_plugin:
                tracer.plugin("sglang", self.target, self.name, answer if declined else None)
            return original(*args, **kwargs) if declined else answer

        # a compiled region may only call what dynamo is told to leave alone
        while_compiling = torch.compiler.disable(attempt) if self.eager else None

        def around_hook(original, *args, **kwargs):
            if torch.compiler.is_compiling():
                if while_compiling is None:
                    return original(*args, **kwargs)
                return while_compiling(original, args, kwargs)
            return attempt(original, args, kwargs)

        return around_hook


# by target: declaring a target again (a module reload) replaces the route instead of hooking twice
_DECLARED: dict[str, Route] = {}


def sglang_route(target: str, *, versions: tuple[str, ...], eager: bool = False) -> Callable[[Callable], Callable]:
    """Declare the decorated function as the route for ``target``; the function itself is returned."""

    def declare(serve: Callable) -> Callable:
        _DECLARED[target] = Route(target, tuple(versions), serve, eager)
        return serve

    return declare


def routes() -> list[Route]:
    return list(_DECLARED.values())


def around(serve: Callable, target: str, *, eager: bool = False) -> Callable:
    """The AROUND hook of an undeclared route (what ``install`` registers for a declared one)."""
    return Route(target, (), serve, eager).hook()


def sglang_version() -> str:
    """The installed sglang release, local build label dropped ("0.5.23+cu128" -> "0.5.23")."""
    return Version(version("sglang")).public


def install() -> int:
    """Register the hooks of every route that stands on the installed sglang; returns their number."""
    from sglang.srt.plugins.hook_registry import HookRegistry, HookType

    release = sglang_version()
    left_out: dict[str, list[str]] = {}
    hooked = 0
    for route in routes():
        standing = route.standing(release)
        if standing != "hook":
            left_out.setdefault(standing, []).append(route.target)
            continue
        HookRegistry.register(route.target, route.hook(), HookType.AROUND)
        hooked += 1
    summary = "".join(f"; {why}: {', '.join(targets)}" for why, targets in sorted(left_out.items()))
    _LOGGER.warning("aklr_b200: %d sglang functions hooked on sglang %s%s", hooked, release, summary)
    return hooked
