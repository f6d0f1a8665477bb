"""One optimisation step as a reusable object: forward, loss, backward, gradient reduction, optimiser update.

This is the unit the `Trainer` iterates and the benchmark times.  The reference spreads the same sequence over
`Trainer.train_one_epoch` (makani/utils/trainer.py:683-754): copy the batch, zero grads, autocast forward and
loss, backward, optimiser step.
"""

from __future__ import annotations

from typing import Callable, Optional

import torch

from ..parallel.grad_reduce import GradReducer


class TrainStep:
    def __init__(self, model: torch.nn.Module, loss_fn: Callable, optimizer: torch.optim.Optimizer,
                 reducer: Optional[GradReducer] = None, amp_dtype: Optional[torch.dtype] = None):
        self.model, self.loss_fn, self.optimizer, self.reducer = model, loss_fn, optimizer, reducer
        self.amp_dtype = amp_dtype

    def forward_backward(self, inp: torch.Tensor, tgt: torch.Tensor) -> torch.Tensor:
        if self.reducer is not None:
            self.reducer.zero_grad()
        else:
            self.optimizer.zero_grad(set_to_none=True)
        use_amp = self.amp_dtype is not None and inp.is_cuda
        with torch.autocast(device_type=inp.device.type, dtype=self.amp_dtype, enabled=use_amp):
            pred = self.model(inp)
            loss = self.loss_fn(pred, tgt, inp)
        loss.backward()
        return loss.detach()

    def __call__(self, inp: torch.Tensor, tgt: torch.Tensor) -> torch.Tensor:
        loss = self.forward_backward(inp, tgt)
        if self.reducer is not None:
            self.reducer.reduce()
        self.optimizer.step()
        return loss
