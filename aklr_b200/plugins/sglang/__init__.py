"""sglang plugin, loaded through the ``sglang.srt.plugins`` entry point
(the reference's: aklr/plugins/sglang/__init__.py:18-44, pyproject.toml:26-27)."""

from __future__ import annotations

import importlib

from aklr_b200.core.dispatch import DispatcherRegistry
from aklr_b200.core.env import RuntimeEnv
from aklr_b200.plugins.sglang import hook

__all__ = ["SGLANG_HOOKED_METHOD", "register"]

# the runtime starts after this sglang method: the rank's device is set by then
SGLANG_HOOKED_METHOD = "sglang.srt.model_executor.model_runner.ModelRunner.init_torch_distributed"
ROUTE_MODULES = ("deepseek_v2", "qwen3_moe", "minimax_m2", "qwen2_moe")


def _start_runtime(_result, *_args, **_kwargs) -> None:
    DispatcherRegistry.default().init_once()


def _hook_up() -> None:
    from sglang.srt.plugins.hook_registry import HookRegistry, HookType

    # always: the ops must be loadable by direct callers even when no route is installed
    HookRegistry.register(SGLANG_HOOKED_METHOD, _start_runtime, HookType.AFTER)
    env = RuntimeEnv()
    if env.is_sglang_plugin_enabled and not env.is_all_disabled:
        for module in ROUTE_MODULES:  # a route module declares its routes when imported
            importlib.import_module(f"{__name__}.models.{module}")
        hook.install()


def register() -> None:
    """What sglang's ``sglang.srt.plugins`` entry point calls, once per process.  sglang only logs an
    exception raised by a plugin and carries on without it; a deployment that asked for this plugin
    should not run silently unaccelerated, so a failed start exits the process instead."""
    try:
        _hook_up()
    except Exception as failure:
        raise SystemExit(f"aklr_b200: the sglang plugin cannot start: {failure!r}") from failure
