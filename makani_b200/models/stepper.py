"""Wrappers that turn a network into a forecast step (single) or an unrolled multi-step rollout (training with
`n_future > 0`).  Contract: makani/models/stepper.py:21-130.  Parameter names keep the `model.` / `preprocessor.`
prefixes so that checkpoints are interchangeable."""

from __future__ import annotations

import torch
import torch.nn as nn

from .preprocessor import Preprocessor2D


class SingleStepWrapper(nn.Module):
    def __init__(self, params, model_handle):
        super().__init__()
        self.preprocessor = Preprocessor2D(params)
        self.model = model_handle(params)

    def forward(self, inp):
        pp = self.preprocessor
        inpa = pp.append_unpredicted_features(inp)
        pp.history_compute_stats(inpa)
        inpan = pp.history_normalize(inpa, target=False)
        inpans = pp.add_static_features(inpan)
        yn = self.model(inpans)
        y = pp.history_denormalize(yn, target=True)
        return pp.add_residual(inp.to(y.dtype) if pp.learn_residual else inp, y)


class MultiStepWrapper(nn.Module):
    def __init__(self, params, model_handle):
        super().__init__()
        self.preprocessor = Preprocessor2D(params)
        self.model = model_handle(params)
        self.n_future = params.n_future

    def _one(self, inpt):
        pp = self.preprocessor
        inpa = pp.append_unpredicted_features(inpt)
        pp.history_compute_stats(inpa)
        inpans = pp.add_static_features(pp.history_normalize(inpa, target=False))
        pred = pp.history_denormalize(self.model(inpans), target=True)
        return pp.add_residual(inpt.to(pred.dtype) if pp.learn_residual else inpt, pred)

    def _forward_train(self, inp):
        result = []
        inpt = inp
        for step in range(self.n_future + 1):
            pred = self._one(inpt)
            result.append(pred)
            if step == self.n_future:
                break
            inpt = self.preprocessor.append_history(inpt.to(pred.dtype), pred, step)
        return torch.cat(result, dim=1)

    def forward(self, inp):
        return self._forward_train(inp) if self.training else self._one(inp)
