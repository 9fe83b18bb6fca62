"""Running loss statistics of the example trainer: a sliding-window mean and a lifetime mean,
their cross-rank averages (two scalar all-reduces), optional TensorBoard output.

Reference counterpart: ``distributed_shampoo/examples/loss_metrics.py:25-98``.
"""

from __future__ import annotations

import logging
from collections import deque

import torch
import torch.distributed as dist

logger: logging.Logger = logging.getLogger(__name__)


class LossMetrics:
    def __init__(self, window_size: int = 100, device: torch.device = torch.device("cpu"), world_size: int = 1, metrics_dir: str | None = None) -> None:
        self._world_size = world_size
        self._iteration = 0
        self._window: deque[torch.Tensor] = deque(maxlen=window_size)
        zero = lambda: torch.tensor(0.0, device=device)  # noqa: E731
        self._window_loss, self._accumulated_loss, self._lifetime_loss = zero(), zero(), zero()
        self._global_window_loss, self._global_lifetime_loss = zero(), zero()
        self._writer = None
        if metrics_dir:
            from torch.utils.tensorboard import SummaryWriter

            self._writer = SummaryWriter(log_dir=metrics_dir)

    def update(self, loss: torch.Tensor) -> None:
        self._iteration += 1
        self._window.append(loss.detach())
        self._window_loss = torch.stack(tuple(self._window)).mean()
        self._accumulated_loss += loss.detach()
        self._lifetime_loss = self._accumulated_loss / self._iteration

    def _emit(self, scope: str, lifetime: torch.Tensor, window: torch.Tensor) -> None:
        logger.info(f"Iteration: {self._iteration} | {scope} Lifetime Loss: {lifetime} | {scope} Window Loss: {window}")
        if self._writer is not None:
            self._writer.add_scalars(f"{scope} Loss", {"Lifetime": lifetime, "Window": window}, global_step=self._iteration)

    def log(self) -> None:
        self._emit("Local", self._lifetime_loss, self._window_loss)

    def update_global_metrics(self) -> None:
        if dist.is_initialized() and self._world_size > 1:
            self._global_window_loss = self._window_loss / self._world_size
            self._global_lifetime_loss = self._lifetime_loss / self._world_size
            dist.all_reduce(self._global_window_loss, op=dist.ReduceOp.SUM)
            dist.all_reduce(self._global_lifetime_loss, op=dist.ReduceOp.SUM)

    def log_global_metrics(self) -> None:
        if self._world_size > 1:
            self._emit("Global", self._global_lifetime_loss, self._global_window_loss)

    def flush(self) -> None:
        if self._writer is not None:
            self._writer.flush()

    @property
    def lifetime_loss(self) -> torch.Tensor:
        return self._lifetime_loss

    @property
    def window_loss(self) -> torch.Tensor:
        return self._window_loss
