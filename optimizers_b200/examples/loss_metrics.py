"""Running loss statistics of the example trainer: a sliding-window mean and a lifetime mean
(API of ``distributed_shampoo/examples/loss_metrics.py:25-98`` in the reference).

Everything lives on the device and ``update`` never waits for it: the window is a ring buffer
tensor with a running sum (the sample that leaves is subtracted, the new one added; the sum is
recomputed from the ring once per turn of the ring, so rounding does not accumulate), and the
two cross-rank means travel in one all-reduce of a two-element tensor.  The host only
synchronises when a value is formatted for the log.
"""

from __future__ import annotations

import logging

import torch
import torch.distributed as dist

logger: logging.Logger = logging.getLogger(__name__)


class LossMetrics:
    def __init__(
        self,
        window_size: int = 100,
        device: torch.device = torch.device("cpu"),
        world_size: int = 1,
        metrics_dir: str | None = None,
    ) -> None:
        self._world_size = world_size
        self._iteration = 0
        self._ring = torch.zeros(max(window_size, 1), device=device)
        # [window sum, lifetime sum] and the means derived from them, local and cross-rank
        self._sums = torch.zeros(2, device=device)
        self._means = torch.zeros(2, device=device)
        self._global_means = torch.zeros(2, device=device)
        self._writer = None
        if metrics_dir:
            from torch.utils.tensorboard import SummaryWriter

            self._writer = SummaryWriter(log_dir=metrics_dir)

    def update(self, loss: torch.Tensor) -> None:
        value = loss.detach().to(self._ring.dtype)
        size = self._ring.numel()
        slot = self._iteration % size
        self._iteration += 1
        leaving = self._ring[slot].clone()
        self._ring[slot] = value
        if slot == size - 1:
            self._sums[0] = self._ring.sum()  # once per turn: resynchronise the running sum
        else:
            self._sums[0] += value - leaving
        self._sums[1] += value
        filled = min(self._iteration, size)
        self._means[0] = self._sums[0] / filled
        self._means[1] = self._sums[1] / self._iteration

    @property
    def window_loss(self) -> torch.Tensor:
        return self._means[0]

    @property
    def lifetime_loss(self) -> torch.Tensor:
        return self._means[1]

    def update_global_metrics(self) -> None:
        """Mean over ranks of both statistics: one collective."""
        if self._world_size > 1 and dist.is_initialized():
            self._global_means = self._means / self._world_size
            dist.all_reduce(self._global_means, op=dist.ReduceOp.SUM)

    def _emit(self, scope: str, means: torch.Tensor) -> None:
        window, lifetime = means.tolist()  # the one synchronisation
        logger.info(f"Iteration: {self._iteration} | {scope} Lifetime Loss: {lifetime} | {scope} Window Loss: {window}")
        if self._writer is not None:
            self._writer.add_scalars(f"{scope} Loss", {"Lifetime": lifetime, "Window": window}, global_step=self._iteration)

    def log(self) -> None:
        self._emit("Local", self._means)

    def log_global_metrics(self) -> None:
        if self._world_size > 1:
            self._emit("Global", self._global_means)

    def flush(self) -> None:
        if self._writer is not None:
            self._writer.flush()
