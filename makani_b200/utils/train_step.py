"""One optimisation step as a reusable object: forward, loss, backward, gradient reduction, optimiser update.

This is the unit the `Trainer` iterates and the benchmark times.  The reference spreads the same sequence over
`Trainer.train_one_epoch` (makani/utils/trainer.py:683-754): copy the batch, zero grads, autocast forward and
loss, backward, optimiser step.
"""

from __future__ import annotations

from typing import Callable, Optional

import torch

from ..ops import _ext
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


class GraphedTrainStep(TrainStep):
    """The same step replayed from one CUDA graph: forward, loss, backward, gradient reduction (peer-memory and
    NCCL collectives included) and the fused optimiser kernels are captured once on static input buffers; each
    call then copies the batch into those buffers, uploads the optimiser's hyper-parameters and replays.

    This removes the per-launch host cost (about a thousand launches per step for the flagship model), which
    dominates when the work per GPU is small, e.g. under spatial model parallelism.  Every rank of a job must use
    it or none (the captured collectives must match).  The reference offers the same idea for forward+backward
    only (`cuda_graph_mode`, makani/utils/trainer.py:226-265).
    """

    def __init__(self, model, loss_fn, optimizer, reducer=None, amp_dtype=None, warmup_steps: int = 3):
        super().__init__(model, loss_fn, optimizer, reducer, amp_dtype)
        self.warmup_steps = warmup_steps
        self.graph = None
        self._calls = 0
        self._capturable = hasattr(optimizer, "prepare_step") and hasattr(optimizer, "launch_step")

    def _capture(self, inp, tgt):
        dev = inp.device
        self.static_inp, self.static_tgt = inp.clone(), tgt.clone()
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            self.graph = torch.cuda.CUDAGraph()
            n0 = _ext.launch_count()
            with torch.cuda.graph(self.graph, stream=side):
                loss = self.forward_backward(self.static_inp, self.static_tgt)
                if self.reducer is not None:
                    self.reducer.reduce()
                self.optimizer.launch_step()
                self.static_loss = loss
            self.launches_per_replay = _ext.launch_count() - n0      # kernels of the extension inside the graph
            _ext.add_launches(-self.launches_per_replay)            # capturing launched nothing
        torch.cuda.current_stream(dev).wait_stream(side)

    def __call__(self, inp, tgt):
        if not (inp.is_cuda and self._capturable):
            return super().__call__(inp, tgt)
        self._calls += 1
        if self._calls <= self.warmup_steps:
            return super().__call__(inp, tgt)        # eager warm-up: allocator pools, peer buffers, plan caches
        if self.graph is not None and (inp.shape != self.static_inp.shape or tgt.shape != self.static_tgt.shape
                                       or inp.dtype != self.static_inp.dtype or tgt.dtype != self.static_tgt.dtype):
            # a different batch geometry (e.g. the last, shorter batch of an epoch): this call runs eagerly and the
            # captured graph stays valid for the usual shape
            return super().__call__(inp, tgt)
        if self.graph is None:
            self._capture(inp, tgt)
        self.static_inp.copy_(inp, non_blocking=True)
        self.static_tgt.copy_(tgt, non_blocking=True)
        self.optimizer.prepare_step()
        self.graph.replay()
        _ext.add_launches(self.launches_per_replay)
        return self.static_loss
