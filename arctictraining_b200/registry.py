# SPDX-License-Identifier: Apache-2.0
"""Class registry: every concrete subclass of a framework base class registers itself by ``name``.

Behaviour parity: arctic_training/registry.py:66-212 (auto-registration through a metaclass,
``get_registered_*`` look-ups, signature / type-hint validation helpers, deprecated ``@register``).

The registry is keyed first by the *root* class (the one that lists ``abc.ABC`` among its direct
bases, e.g. ``Trainer``) and then by the subclass' ``name`` attribute.  Root classes themselves are
never registered.  A class that does not override ``name`` (it inherits the parent's) is treated as
an intermediate helper and is validated but registered only if the name is still free.
"""

from __future__ import annotations

import inspect
from abc import ABC
from abc import ABCMeta
from typing import Any
from typing import Callable
from typing import Dict
from typing import Iterable
from typing import Optional
from typing import Tuple
from typing import Type
from typing import Union
from typing import get_args
from typing import get_origin

from .exceptions import RegistryError
from .exceptions import RegistryValidationError


def _root_of(cls: type) -> Optional[type]:
    """Return the registry root of ``cls``: the first class in the MRO that directly lists ABC."""
    for klass in cls.__mro__[1:]:
        if ABC in getattr(klass, "__bases__", ()):
            return klass
    return None


class RegistryMeta(ABCMeta):
    """Metaclass that validates and records subclasses as they are declared."""

    _registry: Dict[str, Dict[str, type]] = {}

    def __init__(cls, name: str, bases: Tuple[type, ...], namespace: Dict[str, Any]) -> None:
        super().__init__(name, bases, namespace)
        _validate_class_method(cls, "_validate_subclass", ["cls"])
        if ABC in bases:
            return  # a root class: declares the contract, is not itself selectable
        root = _root_of(cls)
        if root is None:
            return
        _validate_class_attribute_set(cls, "name")
        cls._validate_subclass()
        table = RegistryMeta._registry.setdefault(root.__name__, {})
        key = cls.name
        if "name" not in namespace:
            # inherited name: helper/intermediate class, keep the first owner of that name
            if key in table:
                return
        elif key in table:
            raise RegistryValidationError(f"{key} is already registered as a {root.__name__}.")
        table[key] = cls


def register(cls: Optional[type] = None, force: bool = False) -> Union[Callable, type]:
    """Deprecated no-op kept so that older user code ``@register`` still imports and runs."""
    from .logging import logger

    logger.warning("The @register decorator is deprecated and does nothing: subclasses register themselves when they are declared.")
    if isinstance(cls, type):
        return cls
    return lambda klass: klass


def get_registered_class(class_type: str, name: str) -> type:
    table = RegistryMeta._registry.get(class_type)
    if table is None:
        raise RegistryError(
            f"No classes of type {class_type} have been registered; import the module that declares them first."
        )
    if name not in table:
        raise RegistryError(f"{name} is not a registered {class_type}. Known: {sorted(table)}")
    return table[name]


def _getter(class_type: str) -> Callable[[str], type]:
    def get(name: str) -> type:
        return get_registered_class(class_type=class_type, name=name)

    get.__name__ = f"get_registered_{class_type}"
    return get


get_registered_checkpoint_engine = _getter("CheckpointEngine")
get_registered_data_factory = _getter("DataFactory")
get_registered_data_source = _getter("DataSource")
get_registered_model_factory = _getter("ModelFactory")
get_registered_optimizer_factory = _getter("OptimizerFactory")
get_registered_scheduler_factory = _getter("SchedulerFactory")
get_registered_tokenizer_factory = _getter("TokenizerFactory")
get_registered_trainer = _getter("Trainer")


def _validate_class_method(cls: type, method_name: str, expected_args: Iterable[str] = ()) -> None:
    """Check that ``cls.method_name`` exists, is callable and takes exactly ``expected_args``."""
    if not hasattr(cls, method_name):
        raise RegistryValidationError(f"{cls.__name__} must define a '{method_name}' method.")
    fn = getattr(cls, method_name)
    if not callable(fn):
        raise RegistryValidationError(f"{cls.__name__}.{method_name} must be a callable method.")
    if inspect.ismethod(fn):
        fn = fn.__func__
    got = set(inspect.signature(fn).parameters)
    want = set(expected_args)
    if got != want:
        raise RegistryValidationError(
            f"{cls.__name__}.{method_name} must accept exactly {want} as parameters, but got {got}."
        )


def _validate_class_attribute_set(cls: type, attribute: str) -> None:
    if not hasattr(cls, attribute):
        raise RegistryValidationError(f"{cls.__name__} must define a '{attribute}' attribute.")


def _get_class_attr_type_hints(cls: type, attribute: str) -> Tuple[type, ...]:
    """Type hints of one class attribute as a tuple (a ``Union`` is flattened).  Only the annotation of
    that attribute is evaluated (in the namespace of the class that declares it), so unrelated forward
    references elsewhere in the hierarchy cannot break the look-up."""
    import sys
    import typing

    for klass in cls.__mro__:
        ann = klass.__dict__.get("__annotations__", {})
        if attribute not in ann:
            continue
        hint = ann[attribute]
        if isinstance(hint, str):
            module = sys.modules.get(klass.__module__)
            globalns = dict(vars(typing))
            globalns.update(getattr(module, "__dict__", {}))
            hint = eval(hint, globalns, dict(vars(klass)))  # noqa: S307 - annotations of our own classes
        if get_origin(hint) is Union:
            return tuple(get_args(hint))
        return (hint,)
    return ()


def _validate_class_attribute_type(cls: type, attribute: str, type_: type) -> None:
    hints = _get_class_attr_type_hints(cls, attribute)
    if not hints:
        raise RegistryValidationError(f"{cls.__name__}.{attribute} must have a type hint.")
    bad = [h.__name__ for h in hints if not (isinstance(h, type) and issubclass(h, type_))]
    if bad:
        raise RegistryValidationError(
            f"{cls.__name__}.{attribute} must be hinted with subclasses of {type_.__name__}; offending: {bad}."
        )
