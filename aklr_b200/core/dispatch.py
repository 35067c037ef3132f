"""Op contracts and their dispatch: the reference's `@api(CONTRACT)` surface with one backend.

The reference serves each op from a table of measured kernels per device and falls back to the
engine's own code for anything else (aklr/core/runtime/dispatch/_dispatcher.py:53-240,
_registry.py:38-215).  Here there is exactly one kernel set (libaklr_b200.so, sm_100a), so the
table collapses: a call is served when its contract's ``key`` accepts it, the registry has been
initialised on a capability-10.0 device, and the contract is not disabled; otherwise the api
function returns a ``FallbackReason`` -- never an exception for "unsupported", never a CPU path.
"""

from __future__ import annotations

import inspect
import json
import logging
import os
import threading
from collections import Counter
from collections.abc import Callable, Mapping, Sequence
from dataclasses import dataclass, field
from enum import Enum
from typing import Any

import torch

from aklr_b200.core.env import RuntimeEnv

_LOGGER = logging.getLogger("aklr_b200.dispatch")
_TRACE_OP = logging.getLogger("aklr.trace.op")
_INIT_LOCK = threading.Lock()
ALIGNMENT = 16  # bytes: every tensor argument's address (TMA and 128-bit loads need it)


class LoadError(RuntimeError):
    """The runtime cannot start here (no GPU, wrong architecture, library missing)."""


class FallbackReason(str, Enum):
    """Why an api call did not run a kernel; the caller then runs its own code.  Values as
    the reference's (aklr/core/runtime/dispatch/_dispatcher.py:53-69); with one kernel set the
    measurement-related reasons never occur."""

    NO_SCHEMA = "no_schema"
    DISABLED = "disabled"
    OUT_OF_CONTRACT = "out_of_contract"
    NO_WORKLOAD = "no_workload"
    NOT_MEASURED = "not_measured"
    INACCURATE = "inaccurate"
    NOT_QUALIFIED = "not_qualified"
    NOT_WARMED = "not_warmed"


@dataclass(frozen=True)
class Param:
    name: str
    default: Any = inspect.Parameter.empty


@dataclass(frozen=True)
class ServingInfo:
    """What serves a call (the reference's RunnableMetadata, runtime/builder/runnable.py:27-74)."""

    contract_id: str
    kernel: str = "libaklr_b200.so"
    build_type: str = "cuda"
    arch: str = "sm_100a"


@dataclass
class OpContract:
    """One op: its id, api parameters in order, and three callables.

    ``key(call)``: the call's Point as a hashable tuple, or None when no Point describes it
    (wrong dtype/shape/layout/alignment/attr) -- the reference's generated fast_key
    (aklr/core/contract/fastkey/_fast_key_fn.py).  ``alloc(call, key)``: the outputs, the
    caller's buffers where ``call`` holds them.  ``run(call, outputs)``: launches on the current
    stream; no sync, no host reads -- unless the contract says ``capturable=False`` (its ``run`` reads
    something back on the host, e.g. the split sizes of an uneven all-to-all): such an op is never
    served inside a CUDA-graph capture, where it returns ``OUT_OF_CONTRACT`` instead."""

    contract_id: str
    params: Sequence[Param]
    outputs: Sequence[str]
    key: Callable[[Mapping[str, Any]], tuple | None]
    alloc: Callable[[Mapping[str, Any], tuple], Any]
    run: Callable[[Mapping[str, Any], Any], None]
    description: str = ""
    ranks: str | None = None
    group_init: Callable[[], None] | None = None
    capturable: bool = True

    @property
    def name(self) -> str:
        return self.contract_id.split("@")[0]

    def check_api_signature(self, fn: Callable) -> None:
        got = list(inspect.signature(fn).parameters.values())
        want = list(self.params)
        if [p.name for p in got] != [p.name for p in want]:
            raise TypeError(
                f"{self.contract_id}: api function {fn.__name__} takes {[p.name for p in got]}, "
                f"the contract {[p.name for p in want]}"
            )
        for g, w in zip(got, want):
            if g.default != w.default:
                raise TypeError(f"{self.contract_id}: default of {g.name} is {g.default!r}, the contract's {w.default!r}")


def tensor_ok(t: Any, dtype: torch.dtype | tuple, ndim: int, device: torch.device | None = None) -> bool:
    """The per-tensor checks of a dispatch key: a strided, contiguous, 16-byte-aligned CUDA tensor
    of the dtype and rank, not a negated view, on ``device`` if given."""
    dtypes = dtype if isinstance(dtype, tuple) else (dtype,)
    return (
        isinstance(t, torch.Tensor)
        and t.layout is torch.strided
        and t.dtype in dtypes
        and t.dim() == ndim
        and t.is_cuda
        and (device is None or t.device == device)
        and t.is_contiguous()
        and not t.is_neg()
        and (t.numel() == 0 or t.data_ptr() % ALIGNMENT == 0)
    )


def overlaps(a: torch.Tensor, b: torch.Tensor) -> bool:
    if a.numel() == 0 or b.numel() == 0:
        return False
    a0, b0 = a.data_ptr(), b.data_ptr()
    return a0 < b0 + b.numel() * b.element_size() and b0 < a0 + a.numel() * a.element_size()


def _is_capturing() -> bool:
    return torch.cuda.is_available() and torch.cuda.is_current_stream_capturing()


class Trace:
    """AKLR_TRACE: logs each distinct dispatch (op, key, outcome) once, as the reference's
    tracer does (aklr/core/runtime/dispatch/_trace.py:36-100)."""

    def __init__(self, mode: str):
        self.is_op = mode in ("op", "all")
        self.is_plugin = mode in ("plugin", "all")
        self._seen: set = set()
        self._lock = threading.Lock()

    def op(self, contract: OpContract, key, outcome) -> None:
        what = outcome.value if isinstance(outcome, FallbackReason) else "served"
        item = ("op", contract.contract_id, key, what)
        with self._lock:
            if item in self._seen:
                return
            self._seen.add(item)
        _TRACE_OP.info("%s %s -> %s", contract.contract_id, key, what)

    def plugin(self, engine: str, target: str, route: str, fallback) -> None:
        item = ("plugin", engine, target, fallback)
        with self._lock:
            if item in self._seen:
                return
            self._seen.add(item)
        logging.getLogger("aklr.trace.plugin").info(
            "%s %s via %s -> %s", engine, target, route, "served" if fallback is None else fallback.value
        )


_trace: Trace | None = None


def trace() -> Trace | None:
    return _trace


class CallRecorder:
    """AKLR_EXPORT=1: counts calls per (contract, key, outcome) and writes them as JSON lines at
    exit (the reference's recorder, aklr/core/runtime/dispatch/_recorder.py:61-167)."""

    def __init__(self, directory: str):
        self.directory = directory
        self.counts: Counter = Counter()
        self._lock = threading.Lock()

    def count(self, contract: OpContract, key, fallback: FallbackReason | None) -> None:
        with self._lock:
            self.counts[(contract.contract_id, repr(key), None if fallback is None else fallback.value)] += 1

    def save(self) -> str:
        os.makedirs(self.directory, exist_ok=True)
        path = os.path.join(self.directory, f"calls.pid{os.getpid()}.jsonl")
        with open(path, "w") as fh:
            for (contract_id, key, fallback), n in sorted(self.counts.items(), key=repr):
                fh.write(json.dumps({"contract": contract_id, "key": key, "fallback": fallback, "calls": n}) + "\n")
        return path


@dataclass
class KernelDispatcher:
    """Serves one contract.  Closed (every call returns ``closed_reason``) until the registry opens
    it; then ``dispatch`` keys the call, allocates outputs and runs the kernel."""

    contract: OpContract
    is_open: bool = False
    closed_reason: FallbackReason = FallbackReason.NO_SCHEMA
    warmed_keys: set = field(default_factory=set)
    recorder: CallRecorder | None = None
    has_warned_not_warmed: bool = False

    def _lookup(self, call: Mapping[str, Any]):
        """(key, outcome): outcome is a FallbackReason or None when the call is served."""
        if not self.is_open:
            return None, self.closed_reason
        if not self.contract.capturable and _is_capturing():
            return None, FallbackReason.OUT_OF_CONTRACT  # its run() reads from the host: not inside a capture
        key = self.contract.key(call)
        if key is None:
            return None, FallbackReason.OUT_OF_CONTRACT
        if key not in self.warmed_keys and _is_capturing():
            # a Point first seen inside a graph capture would do its first-call set-up there
            return key, FallbackReason.NOT_WARMED
        return key, None

    def _note(self, key, outcome) -> None:
        if (tracer := trace()) is not None and tracer.is_op:
            tracer.op(self.contract, key, outcome)
        if self.recorder is not None:
            self.recorder.count(self.contract, key, outcome)

    def dispatch(self, call: Mapping[str, Any]) -> Any:
        key, outcome = self._lookup(call)
        if outcome is not None:
            if outcome is FallbackReason.NOT_WARMED and not self.has_warned_not_warmed:
                self.has_warned_not_warmed = True
                _LOGGER.warning(
                    "%s: %s was first called inside a graph capture: it falls back there and in every "
                    "replay; call each shape once outside a capture first",
                    self.contract.contract_id,
                    key,
                )
            self._note(key, outcome)
            return outcome
        result = self.contract.alloc(call, key)
        try:
            self.contract.run(call, result)
        except Exception:
            _LOGGER.error(
                "%s: the sm_100a kernel serving %s failed; AKLR_DISABLE=%s turns this op off",
                self.contract.contract_id,
                key,
                self.contract.contract_id,
            )
            raise
        self.warmed_keys.add(key)
        self._note(key, None)
        return result

    def serving(self, call: Mapping[str, Any]) -> ServingInfo | FallbackReason:
        key, outcome = self._lookup(call)
        if outcome is not None:
            self._note(key, outcome)
            return outcome
        return ServingInfo(self.contract.contract_id)

    def fallback_reason(self, call: Mapping[str, Any]) -> FallbackReason | None:
        served = self.serving(call)
        return served if isinstance(served, FallbackReason) else None

    def open(self, recorder: CallRecorder | None = None) -> None:
        self.is_open, self.recorder = True, recorder

    def close(self, reason: FallbackReason) -> None:
        self.is_open, self.closed_reason, self.recorder = False, reason, None

    def make_api_fn(self, fn: Callable) -> Callable:
        """The api function replacing the signature-only ``fn``; its ``fallback_reason`` and
        ``serving`` attributes ask without running."""
        self.contract.check_api_signature(fn)
        signature = inspect.signature(fn)

        def bind(args, kwargs) -> dict:
            bound = signature.bind(*args, **kwargs)
            bound.apply_defaults()
            return dict(bound.arguments)

        def api_fn(*args, **kwargs):
            return self.dispatch(bind(args, kwargs))

        def fallback_reason(*args, **kwargs):
            return self.fallback_reason(bind(args, kwargs))

        def serving(*args, **kwargs):
            return self.serving(bind(args, kwargs))

        for generated in (api_fn, fallback_reason, serving):
            generated.__name__ = fn.__name__
            generated.__qualname__ = fn.__qualname__
            generated.__doc__ = fn.__doc__
            generated.__signature__ = signature
        api_fn.__module__ = fn.__module__
        api_fn.fallback_reason = fallback_reason
        api_fn.serving = serving
        api_fn.contract = self.contract
        return api_fn


class DispatcherRegistry:
    """The dispatchers of this process by contract id."""

    _default: DispatcherRegistry | None = None

    def __init__(self) -> None:
        self._dispatchers: dict[str, KernelDispatcher] = {}
        self.is_initialized = False
        self.recorder: CallRecorder | None = None
        self.device: torch.device | None = None

    @classmethod
    def default(cls) -> DispatcherRegistry:
        if cls._default is None:
            cls._default = cls()
        return cls._default

    def dispatcher(self, contract: OpContract) -> KernelDispatcher:
        existing = self._dispatchers.get(contract.contract_id)
        if existing is None:
            existing = self._dispatchers[contract.contract_id] = KernelDispatcher(contract)
        elif existing.contract is not contract:
            raise ValueError(f"{contract.contract_id}: another contract already has this id")
        return existing

    def dispatchers(self) -> Mapping[str, KernelDispatcher]:
        return dict(self._dispatchers)

    @staticmethod
    def _probe_device() -> torch.device:
        hint = "AKLR_DISABLE=1 starts without the B200 kernels"
        if not torch.cuda.is_available():
            raise LoadError(f"no GPU visible: {hint}")
        device = torch.device("cuda", torch.cuda.current_device())
        major, minor = torch.cuda.get_device_capability(device)
        if major != 10:
            raise LoadError(f"device {device.index} has capability {major}.{minor}; the kernels are sm_100a only: {hint}")
        return device

    def init(self) -> None:
        """Read the environment, probe the device, load the library, open the dispatchers."""
        global _trace
        env = RuntimeEnv()
        _trace = Trace(env.trace_mode) if env.trace_mode != "0" else None
        if env.is_all_disabled:
            for d in self._dispatchers.values():
                d.close(FallbackReason.DISABLED)
            self.is_initialized = True
            return
        unknown = env.disabled_contracts - set(self._dispatchers)
        if unknown:
            raise LoadError(f"AKLR_DISABLE names unknown contracts: {sorted(unknown)}")
        self.device = self._probe_device()
        from aklr_b200 import _lib

        try:
            _lib.load()
        except (ImportError, OSError) as e:
            raise LoadError(str(e)) from e
        if env.is_export_enabled and self.recorder is None:
            import atexit

            self.recorder = CallRecorder(env.export_dir)
            atexit.register(self.recorder.save)
        served = 0
        for contract_id, d in self._dispatchers.items():
            if contract_id in env.disabled_contracts:
                d.close(FallbackReason.DISABLED)
            else:
                d.open(self.recorder)
                if d.contract.group_init is not None and torch.distributed.is_available() and torch.distributed.is_initialized():
                    d.contract.group_init()
                served += 1
        self.is_initialized = True
        _LOGGER.info("aklr_b200 serves %d of %d contracts on %s (sm_100a)", served, len(self._dispatchers), self.device)

    def init_once(self) -> None:
        with _INIT_LOCK:
            if not self.is_initialized:
                self.init()

    def reset(self) -> None:
        """Close everything (tests)."""
        for d in self._dispatchers.values():
            d.close(FallbackReason.NO_SCHEMA)
            d.warmed_keys.clear()
        self.is_initialized = False
        self.recorder = None


def api(contract: OpContract) -> Callable[[Callable], Callable]:
    """The decorator of an op's api function (aklr/core/runtime/dispatch/_registry.py:213-215)."""
    return DispatcherRegistry.default().dispatcher(contract).make_api_fn
