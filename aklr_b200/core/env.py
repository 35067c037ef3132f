"""Environment switches, named as the reference names them (aklr/core/platform/env.py:27-104)."""

from __future__ import annotations

import os

ENV_DISABLE = "AKLR_DISABLE"
ENV_SGLANG_PLUGIN = "AKLR_SGLANG_PLUGIN"
ENV_VLLM_PLUGIN = "AKLR_VLLM_PLUGIN"
ENV_AITER_PLUGIN = "AKLR_AITER_PLUGIN"
ENV_TRACE = "AKLR_TRACE"
ENV_EXPORT = "AKLR_EXPORT"
ENV_EXPORT_DIR = "AKLR_EXPORT_DIR"
DEFAULT_EXPORT_DIR = "aklr_export"

_ALL = (ENV_DISABLE, ENV_SGLANG_PLUGIN, ENV_VLLM_PLUGIN, ENV_AITER_PLUGIN, ENV_TRACE, ENV_EXPORT, ENV_EXPORT_DIR)


def _switch(name: str) -> bool:
    value = os.environ.get(name) or "0"
    if value not in ("0", "1"):
        raise ValueError(f"{name}={value!r}: expected '1' or '0'")
    return value == "1"


def trace_mode() -> str:
    """AKLR_TRACE: '0'/unset nothing, 'plugin' the routes, 'op' the dispatches, 'all' both."""
    mode = os.environ.get(ENV_TRACE) or "0"
    if mode not in ("0", "plugin", "op", "all"):
        raise ValueError(f"{ENV_TRACE}={mode!r}: expected '0', 'plugin', 'op' or 'all'")
    return mode


class RuntimeEnv:
    """What the environment asks of the runtime, read once; '' counts as unset and a bad
    value raises ValueError naming its variable."""

    def __init__(self) -> None:
        disable = os.environ.get(ENV_DISABLE) or "0"
        self.is_all_disabled = disable == "1"
        self.disabled_contracts = (
            frozenset() if disable in ("0", "1") else frozenset(part.strip() for part in disable.split(","))
        )
        self.is_sglang_plugin_enabled = _switch(ENV_SGLANG_PLUGIN)
        self.is_vllm_plugin_enabled = _switch(ENV_VLLM_PLUGIN)
        self.is_aiter_plugin_enabled = _switch(ENV_AITER_PLUGIN)
        self.is_export_enabled = _switch(ENV_EXPORT)
        self.export_dir = os.path.abspath(os.environ.get(ENV_EXPORT_DIR) or DEFAULT_EXPORT_DIR)
        self.trace_mode = trace_mode()


def all_names() -> tuple[str, ...]:
    return _ALL
