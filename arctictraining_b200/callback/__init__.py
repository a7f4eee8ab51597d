from .callback import Callback
from .mixin import CallbackMixin
from .mixin import callback_wrapper

__all__ = ["Callback", "CallbackMixin", "callback_wrapper"]
