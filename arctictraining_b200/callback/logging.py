# SPDX-License-Identifier: Apache-2.0
"""Built-in logging callbacks.  Parity: arctic_training/callback/logging.py:21-68."""

from __future__ import annotations

from typing import Any

from ..logging import logger


def _pre_init_log(self) -> None:
    logger.info(f"Initializing {self.__class__.__name__}")


def _post_init_log(self) -> None:
    logger.info(f"Initialized {self.__class__.__name__}")


def _log_loss_value(self, loss: Any) -> Any:
    every = self.config.loss_log_interval
    if every and self.global_step % every == 0:
        logger.info(f"Global Step: {self.global_step}/{self.training_horizon}, Loss: {loss}")
    return loss


def _log_callback_ordering(self) -> None:
    lines = [f"Callback methods for {self.__class__.__name__}:"]
    for event in sorted({e.split("-", 1)[1] for e in self._get_all_callback_event_methods()}):
        pre = [cb for cb in self._initialized_callbacks if cb.event == f"pre-{event}"]
        post = [cb for cb in self._initialized_callbacks if cb.event == f"post-{event}"]
        lines.append(f"  {event}:\n\tPre-callbacks: {pre}\n\tPost-callbacks: {post}")
    logger.debug("\n".join(lines))


pre_init_log_cb = ("pre-init", _pre_init_log)
post_init_log_cb = ("post-init", _post_init_log)
post_loss_log_cb = ("post-loss", _log_loss_value)
post_init_callback_ordering_cb = ("post-init", _log_callback_ordering)
