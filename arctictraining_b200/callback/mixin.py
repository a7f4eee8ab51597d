# SPDX-License-Identifier: Apache-2.0
"""Mixin giving a class ``pre-<event>`` / ``post-<event>`` hooks around selected methods.

Behaviour parity: arctic_training/callback/mixin.py:35-162.  ``@callback_wrapper("step")`` marks a
method as observable.  Callbacks come from the ``callbacks`` class attribute (a list of
``(event, fn)`` tuples, accumulated over the inheritance chain) and from methods named
``pre_<event>_callback`` / ``post_<event>_callback``.  A subclass that overrides a wrapped method gets
the override wrapped again automatically, so hooks keep firing.
"""

from __future__ import annotations

import functools
import inspect
import re
from typing import Any
from typing import Callable
from typing import Dict
from typing import List
from typing import Tuple

from .callback import Callback
from .logging import post_init_callback_ordering_cb
from .logging import post_init_log_cb
from .logging import pre_init_log_cb

WRAPPER_NAME_ATTR = "__at_wrapped_name__"
_CB_METHOD_RE = re.compile(r"^(pre|post)_(.+)_callback$")


def callback_wrapper(name: str) -> Callable[[Callable], Callable]:
    """Decorator: run ``pre-<name>`` callbacks before and ``post-<name>`` callbacks after the method."""

    def decorator(method: Callable) -> Callable:
        if hasattr(method, WRAPPER_NAME_ATTR):
            return method

        @functools.wraps(method)
        def wrapper(self, *args, **kwargs):
            # an override that calls ``super().<method>()`` enters the parent's wrapper while its own is running:
            # the callbacks of the event belong to the outermost call only (otherwise a post-create-model callback
            # such as the adapter wrapping would be applied twice)
            running = self.__dict__.setdefault("_callback_events_running", set())
            if name in running:
                return method(self, *args, **kwargs)
            running.add(name)
            try:
                args, kwargs = self._run_callbacks(f"pre-{name}", args, kwargs)
                result = method(self, *args, **kwargs)
                result, _ = self._run_callbacks(f"post-{name}", result, {})
            finally:
                running.discard(name)
            return result

        setattr(wrapper, WRAPPER_NAME_ATTR, name)
        return wrapper

    return decorator


class CallbackMixin:
    _class_callbacks: List[Tuple[str, Callable]] = []
    _initialized_callbacks: List[Callback] = []

    callbacks: List[Tuple[str, Callable]] = [pre_init_log_cb, post_init_log_cb, post_init_callback_ordering_cb]
    """ ``(event, function)`` pairs applied to every instance of the class. """

    @callback_wrapper("init")
    def __init__(self, *args, **kwargs) -> None:
        super().__init__(*args, **kwargs)

    def __new__(cls, *args, **kwargs):
        cls._class_callbacks = cls._get_all_callbacks()
        cls._initialized_callbacks = cls._init_callbacks()
        return super().__new__(cls)

    def __init_subclass__(cls, **kwargs) -> None:
        super().__init_subclass__(**kwargs)
        # re-wrap overrides of wrapped parent methods
        for parent in cls.__mro__[1:]:
            for attr, member in vars(parent).items():
                event = getattr(member, WRAPPER_NAME_ATTR, None)
                if event is None:
                    continue
                own = cls.__dict__.get(attr)
                if own is not None and inspect.isfunction(own) and not hasattr(own, WRAPPER_NAME_ATTR):
                    setattr(cls, attr, callback_wrapper(event)(own))
        merged = list(cls._class_callbacks)
        merged.extend(cb for cb in cls.callbacks if cb not in merged)
        cls._class_callbacks = merged

    @classmethod
    def _get_all_callback_event_methods(cls) -> Dict[str, Callable]:
        out: Dict[str, Callable] = {}
        for _, member in inspect.getmembers(cls, predicate=inspect.isfunction):
            event = getattr(member, WRAPPER_NAME_ATTR, None)
            if event is not None:
                out[f"pre-{event}"] = member
                out[f"post-{event}"] = member
        return out

    @classmethod
    def _get_all_callbacks(cls) -> List[Tuple[str, Callable]]:
        found = list(cls._class_callbacks)
        for attr, member in inspect.getmembers(cls, predicate=inspect.isfunction):
            m = _CB_METHOD_RE.match(attr)
            if m:
                item = (f"{m.group(1)}-{m.group(2).replace('_', '-')}", member)
                if item not in found:
                    found.append(item)
        return found

    @classmethod
    def _init_callbacks(cls) -> List[Callback]:
        methods = cls._get_all_callback_event_methods()
        bound = []
        for event, fn in cls._class_callbacks:
            if event not in methods:
                raise ValueError(f"Callback {fn} for event {event} does not have a corresponding wrapped method.")
            bound.append(Callback(event, fn, inspect.unwrap(methods[event])))
        return bound

    def _run_callbacks(self, name: str, args: Any, kwargs: Dict[str, Any]) -> Tuple[Any, Dict[str, Any]]:
        for cb in self._initialized_callbacks:
            if cb.event == name:
                args, kwargs = cb(self, args, kwargs)
        return args, kwargs
