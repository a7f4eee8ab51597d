# SPDX-License-Identifier: Apache-2.0
"""One bound callback: an event name, the user function and the wrapped method it observes.

Behaviour parity: arctic_training/callback/callback.py:26-156.  A *pre* callback receives ``self`` plus
any subset of the wrapped method's parameters (by name) and must return the possibly modified values
in the same order; a *post* callback receives ``self`` and the return value and returns the new return
value (when the method is annotated ``-> None`` it receives only ``self``).
"""

from __future__ import annotations

import inspect
from typing import Any
from typing import Callable
from typing import Dict
from typing import Tuple

from ..logging import logger

_VARIADIC = (inspect.Parameter.VAR_POSITIONAL, inspect.Parameter.VAR_KEYWORD)


class Callback:
    def __init__(self, event: str, fn: Callable, method: Callable) -> None:
        self.event = event
        self.fn = fn
        self.method = method
        self._method_sig = inspect.signature(method)
        self._fn_sig = inspect.signature(fn)
        self.is_pre_cb = event.startswith("pre-")
        self.is_post_cb = event.startswith("post-")
        self.params_to_pass: Tuple[str, ...] = ()
        self.pass_return_val = True
        if self.is_pre_cb:
            self._check_pre()
        elif self.is_post_cb:
            self._check_post()
        else:
            raise ValueError(f"Invalid event type: {event}. Expected 'pre-' or 'post-' prefix.")

    def _check_pre(self) -> None:
        method_params = set(self._method_sig.parameters)
        names = []
        for p in self._fn_sig.parameters.values():
            if p.default is not p.empty:
                raise ValueError(f"Callback {self.fn.__name__}: parameter {p.name} must not have a default value.")
            if p.kind in _VARIADIC:
                raise ValueError(f"Callback {self.fn.__name__} must not take *args or **kwargs.")
            if p.name not in method_params:
                raise ValueError(
                    f"Callback {self.fn.__name__}: parameter {p.name} is not present in the method signature."
                )
            names.append(p.name)
        if not names:
            raise ValueError(f"Pre-callback {self.fn} should have at least one parameter: `self`.")
        self.params_to_pass = tuple(names[1:])

    def _check_post(self) -> None:
        ret = self._method_sig.return_annotation
        n = len(self._fn_sig.parameters)
        if ret is inspect.Signature.empty:
            logger.debug(f"{self.method} has no return annotation; post-callback {self.fn} is not validated.")
            self.pass_return_val = n >= 2
        elif ret is None or ret == "None":
            self.pass_return_val = False
            if n != 1:
                raise ValueError(f"Post-callback {self.fn} should have exactly one parameter: `self`.")
        elif n != 2:
            raise ValueError(f"Post-callback {self.fn} should take `self` and the wrapped method's return value.")

    def _run_pre(self, obj: object, args: Tuple[Any, ...], kwargs: Dict[str, Any]) -> Dict[str, Any]:
        bound = self._method_sig.bind(obj, *args, **kwargs)
        bound.apply_defaults()
        call_kwargs = {k: v for k, v in bound.arguments.items() if k not in ("self", "args", "kwargs")}
        out = self.fn(obj, **{k: call_kwargs[k] for k in self.params_to_pass})
        n = len(self.params_to_pass)
        if n == 0:
            if out is not None:
                raise ValueError(f"Pre-callback {self.fn} should not return any values.")
            return call_kwargs
        if n == 1:
            out = (out,)
        elif out is None or len(out) != n:
            got = 0 if out is None else len(out)
            raise ValueError(f"Pre-callback {self.fn} returned {got} arguments, but expected {n} arguments.")
        call_kwargs.update(dict(zip(self.params_to_pass, out)))
        return call_kwargs

    def __call__(self, obj: object, args: Any, kwargs: Dict[str, Any]) -> Tuple[Any, Dict[str, Any]]:
        if self.is_pre_cb:
            return (), self._run_pre(obj, args, kwargs)
        if self.pass_return_val:
            return self.fn(obj, args), {}
        return self.fn(obj), {}

    def __repr__(self) -> str:
        return f"<Callback event={self.event} fn={self.fn.__name__}>"
