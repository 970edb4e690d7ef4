"""Deprecation helpers.

  @Deprecated(deprecated_date="2026-06-30", suggestion="use X")      warns once per call site category, names the date
  AutoExecuteFunction(fn)                                            a module-level side effect that runs at import
                                                                     unless side effects are disabled
  NoExecuteFunction                                                  context manager / switch that disables them (tools
                                                                     that only want to import a module for inspection)
reference: mindspeed/deprecate.py:45-144.
"""
from __future__ import annotations

import datetime
import functools
import warnings
from typing import Callable, Optional, Sequence

_SIDE_EFFECTS_ENABLED = True
_WARNED = set()


class Deprecated:
    def __init__(self, deprecated_date: str, deprecated_codes: Optional[Sequence[str]] = None, suggestion: str = ""):
        self.date = datetime.date.fromisoformat(deprecated_date)
        self.codes, self.suggestion = list(deprecated_codes or []), suggestion

    def message(self, name: str) -> str:
        today = datetime.date.today()
        when = f"will be removed after {self.date.isoformat()}" if today <= self.date else f"was scheduled for removal on {self.date.isoformat()}"
        msg = f"{name} is deprecated and {when}."
        if self.codes:
            msg += " Affected: " + ", ".join(self.codes) + "."
        if self.suggestion:
            msg += " " + self.suggestion
        return msg

    def __call__(self, obj):
        name = getattr(obj, "__qualname__", getattr(obj, "__name__", str(obj)))
        text = self.message(name)
        if isinstance(obj, type):
            orig_init = obj.__init__

            @functools.wraps(orig_init)
            def init(self_, *a, **kw):
                if name not in _WARNED:
                    _WARNED.add(name)
                    warnings.warn(text, DeprecationWarning, stacklevel=2)
                orig_init(self_, *a, **kw)
            obj.__init__ = init
            obj.__deprecated__ = text
            return obj

        @functools.wraps(obj)
        def wrapper(*a, **kw):
            if name not in _WARNED:
                _WARNED.add(name)
                warnings.warn(text, DeprecationWarning, stacklevel=2)
            return obj(*a, **kw)
        wrapper.__deprecated__ = text
        return wrapper


class NoExecuteFunction:
    """``with NoExecuteFunction(): import something`` - AutoExecuteFunction instances created inside do not run."""

    def __enter__(self):
        global _SIDE_EFFECTS_ENABLED
        self._prev = _SIDE_EFFECTS_ENABLED
        _SIDE_EFFECTS_ENABLED = False
        return self

    def __exit__(self, *exc):
        global _SIDE_EFFECTS_ENABLED
        _SIDE_EFFECTS_ENABLED = self._prev
        return False


class AutoExecuteFunction:
    """Runs ``fn(*args, **kw)`` on construction when side effects are enabled; ``run()`` forces it later."""

    def __init__(self, fn: Callable, *args, **kw):
        self.fn, self.args, self.kw = fn, args, kw
        self.executed = False
        self.result = None
        if _SIDE_EFFECTS_ENABLED:
            self.run()

    def run(self):
        if not self.executed:
            self.result = self.fn(*self.args, **self.kw)
            self.executed = True
        return self.result
