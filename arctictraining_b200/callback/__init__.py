# SPDX-License-Identifier: Apache-2.0
from .callback import Callback
from .mixin import CallbackMixin
from .mixin import callback_wrapper

__all__ = ["Callback", "CallbackMixin", "callback_wrapper"]
