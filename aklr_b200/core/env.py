"""The environment variables the runtime obeys.

The names and accepted values are the reference's (aklr/core/platform/env.py:27-104), so a deployment
script written for it keeps working: AKLR_DISABLE ("1" for everything, or a comma-separated list of
contract ids), AKLR_SGLANG_PLUGIN / AKLR_VLLM_PLUGIN / AKLR_AITER_PLUGIN / AKLR_EXPORT ("0" or "1"),
AKLR_EXPORT_DIR (a path) and AKLR_TRACE ("0", "plugin", "op", "all").  An empty value counts as unset;
any other value raises ``ValueError`` naming the variable, so a typo stops the start instead of being
read as "off".
"""

from __future__ import annotations

import os

DEFAULT_EXPORT_DIR = "aklr_export"
TRACE_MODES = ("0", "plugin", "op", "all")

# variable -> RuntimeEnv attribute holding its on/off value
_ON_OFF = {
    "AKLR_SGLANG_PLUGIN": "is_sglang_plugin_enabled",
    "AKLR_VLLM_PLUGIN": "is_vllm_plugin_enabled",
    "AKLR_AITER_PLUGIN": "is_aiter_plugin_enabled",
    "AKLR_EXPORT": "is_export_enabled",
}


def _read(name: str, unset: str) -> str:
    return os.environ.get(name) or unset


def _one_of(name: str, allowed: tuple[str, ...]) -> str:
    value = _read(name, allowed[0])
    if value not in allowed:
        raise ValueError(f"{name}={value!r}: expected {' or '.join(repr(a) for a in allowed)}")
    return value


def trace_mode() -> str:
    """AKLR_TRACE: nothing ("0" or unset), the plugin routes, the op dispatches, or both."""
    return _one_of("AKLR_TRACE", TRACE_MODES)


def all_names() -> tuple[str, ...]:
    """Every variable read here (tests clear them)."""
    return ("AKLR_DISABLE", *_ON_OFF, "AKLR_TRACE", "AKLR_EXPORT_DIR")


class RuntimeEnv:
    """A snapshot of the variables above, validated when taken."""

    def __init__(self) -> None:
        for name, field in _ON_OFF.items():
            setattr(self, field, _one_of(name, ("0", "1")) == "1")
        self.trace_mode = trace_mode()
        self.export_dir = os.path.abspath(_read("AKLR_EXPORT_DIR", DEFAULT_EXPORT_DIR))
        disable = _read("AKLR_DISABLE", "0")
        self.is_all_disabled = disable == "1"
        named = () if disable in ("0", "1") else (part.strip() for part in disable.split(","))
        self.disabled_contracts = frozenset(named)
