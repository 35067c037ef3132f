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
ROUTE_MODULES = ("deepseek_v2", "qwen3_moe", "minimax_m2")


def register() -> None:
    """Entry point sglang calls once per process; a plugin that cannot start ends the process
    (sglang would only log the error)."""
    try:
        _register()
    except Exception as e:
        raise SystemExit(f"aklr_b200: the sglang plugin cannot start: {e!r}") from e


def _register() -> None:
    from sglang.srt.plugins.hook_registry import HookRegistry, HookType

    HookRegistry.register(
        SGLANG_HOOKED_METHOD,
        lambda result, *args, **kwargs: DispatcherRegistry.default().init_once(),
        HookType.AFTER,
    )
    env = RuntimeEnv()
    if env.is_all_disabled or not env.is_sglang_plugin_enabled:
        return
    for name in ROUTE_MODULES:  # importing a module declares its routes
        importlib.import_module(f"{__name__}.models.{name}")
    hook.install()
