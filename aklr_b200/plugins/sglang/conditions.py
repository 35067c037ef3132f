"""Named conditions: the route layer's way of saying why a call stays on sglang.

A route serves a sglang call only while the module in front of it is configured exactly as the op
behind the route computes.  Each such requirement is a ``Condition``: a label a person can read and a
test of one subject.  ``first_unmet`` walks a table of them and returns the label of the first that
does not hold, which the routes log once per label, so that "why is this layer not accelerated" has
an answer in the log instead of in a debugger.
"""

from __future__ import annotations

import logging
from collections.abc import Callable, Iterable
from typing import Any, NamedTuple

__all__ = ["Condition", "attr", "first_unmet", "leave_to_sglang", "report_once", "when"]

_LOGGER = logging.getLogger(__name__)
_REPORTED: set[tuple[str, str]] = set()
_ABSENT = object()


class Condition(NamedTuple):
    label: str
    holds: Callable[[Any], bool]


def attr(subject: Any, path: str, default: Any = _ABSENT) -> Any:
    """``subject.a.b.c`` for ``path`` "a.b.c"; ``default`` (when given) where a link is missing."""
    for name in path.split("."):
        subject = getattr(subject, name, _ABSENT)
        if subject is _ABSENT:
            if default is _ABSENT:
                raise AttributeError(f"{path!r}: no attribute {name!r}")
            return default
    return subject


def first_unmet(subject: Any, conditions: Iterable[Condition]) -> str | None:
    """The label of the first condition ``subject`` does not meet, else None."""
    for condition in conditions:
        if not condition.holds(subject):
            return condition.label
    return None


def report_once(route: str, label: str) -> None:
    """Log, once per (route, label), that ``route`` left a call to sglang because of ``label``."""
    if (route, label) not in _REPORTED:
        _REPORTED.add((route, label))
        _LOGGER.info("%s stays on sglang: %s", route, label)


def when(flag: Any, label: str) -> str | None:
    """``label`` if ``flag`` is true, else None: turns a bare predicate into a reason."""
    return label if flag else None


def leave_to_sglang(route: str, label: str):
    """Report ``label`` for ``route`` and return the value that hands the call back to sglang."""
    from aklr_b200.core.dispatch import FallbackReason

    report_once(route, label)
    return FallbackReason.OUT_OF_CONTRACT
