"""vLLM plugin, loaded through the ``vllm.general_plugins`` entry point
(the reference's: aklr/plugins/vllm/__init__.py:20-56)."""

from __future__ import annotations

import importlib

from aklr_b200.core.dispatch import DispatcherRegistry
from aklr_b200.core.env import RuntimeEnv
from aklr_b200.plugins.vllm import hook

__all__ = ["VLLM_HOOKED_METHOD", "register"]

VLLM_HOOKED_METHOD = "vllm.v1.worker.gpu_worker.Worker.init_device"
ROUTE_MODULES = ("fused_experts",)


def register() -> None:
    """Entry point vLLM calls in every process; a plugin that cannot start ends the process."""
    try:
        _register()
    except Exception as e:
        raise SystemExit(f"aklr_b200: the vLLM plugin cannot start: {e!r}") from e


def _register() -> None:
    env = RuntimeEnv()
    if env.is_all_disabled or not env.is_vllm_plugin_enabled:
        return
    _start_after_device_init()
    for name in ROUTE_MODULES:
        importlib.import_module(f"{__name__}.{name}")


def _start_after_device_init() -> None:
    """Start the runtime and bind the routes once the worker's device is set."""
    import pkgutil

    worker_cls = pkgutil.resolve_name(VLLM_HOOKED_METHOD.rsplit(".", 1)[0])
    orig = worker_cls.init_device
    if getattr(orig, "_aklr_b200_hooked", False):
        return

    def init_device(self, *args, **kwargs):
        result = orig(self, *args, **kwargs)
        DispatcherRegistry.default().init_once()
        hook.install()
        return result

    init_device._aklr_b200_hooked = True
    worker_cls.init_device = init_device
