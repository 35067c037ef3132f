"""``@sglang_route``: how a sglang function reaches the ops, declared beside them.

Same contract as the reference's decorator (aklr/plugins/sglang/hook.py:29-103): a route names the
sglang function it stands in for and the sglang releases it was tested on; ``install`` wraps the
targets of the routes tested on the installed release as AROUND hooks; a route that returns a
``FallbackReason`` hands the call to sglang's own code; inside a torch.compile trace the route is
skipped unless declared ``eager``.
"""

from __future__ import annotations

import importlib.util
import logging
import pkgutil
from collections.abc import Callable
from importlib.metadata import version

import torch
from packaging.version import Version

from aklr_b200.core import dispatch
from aklr_b200.core.dispatch import FallbackReason

__all__ = ["install", "routes", "sglang_route", "sglang_version"]

_LOGGER = logging.getLogger(__name__)
_ROUTES: list[tuple[str, tuple[str, ...], Callable]] = []
_EAGER: set[Callable] = set()


def sglang_route(target: str, *, versions: tuple[str, ...], eager: bool = False) -> Callable[[Callable], Callable]:
    def declare(route: Callable) -> Callable:
        _ROUTES.append((target, versions, route))
        if eager:
            _EAGER.add(route)
        return route

    return declare


def routes() -> list[tuple[str, tuple[str, ...], Callable]]:
    return list(_ROUTES)


def sglang_version() -> str:
    """The installed sglang's release without a local label."""
    return Version(version("sglang")).public


def install() -> int:
    """Wrap the targets of the routes tested on the installed sglang; returns how many."""
    from sglang.srt.plugins.hook_registry import HookRegistry, HookType

    installed = sglang_version()
    untested, absent, hooked = [], [], 0
    for target, versions, route in _ROUTES:
        if installed not in versions:
            untested.append(target)
            continue
        try:
            pkgutil.resolve_name(target)
        except ModuleNotFoundError as e:
            # a target inside a package this environment lacks is never called; a target missing
            # from a package that is present was renamed, which must stop the start
            package = (e.name or "").partition(".")[0]
            if not package or importlib.util.find_spec(package) is not None:
                raise
            absent.append(f"{target} ({package} is not installed)")
            continue
        HookRegistry.register(target, around(route, target), HookType.AROUND)
        hooked += 1
    _LOGGER.warning(
        "aklr_b200 hooks %d sglang functions on sglang %s%s%s",
        hooked,
        installed,
        f"; not {', '.join(untested)}, untested on it" if untested else "",
        f"; not {', '.join(absent)}" if absent else "",
    )
    return hooked


def around(route: Callable, target: str) -> Callable:
    """The AROUND hook of ``route``: serve, trace, or call sglang's original."""
    route_name = f"{route.__module__}.{route.__qualname__}"

    def serve(orig, args, kwargs):
        result = route(*args, **kwargs)
        fallback = result if isinstance(result, FallbackReason) else None
        if (tracer := dispatch.trace()) is not None and tracer.is_plugin:
            tracer.plugin("sglang", target, route_name, fallback)
        return orig(*args, **kwargs) if fallback is not None else result

    serve_eagerly = torch.compiler.disable(serve) if route in _EAGER else None

    def hook(orig, *args, **kwargs):
        if not torch.compiler.is_compiling():
            return serve(orig, args, kwargs)
        if serve_eagerly is not None:
            return serve_eagerly(orig, args, kwargs)
        return orig(*args, **kwargs)

    return hook
