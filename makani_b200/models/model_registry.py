"""Registry of network constructors and the factory that wraps them into forecast steppers.

Contract: makani/models/model_registry.py:34-170 — names `AFNOv1, AFNO, FNO, SFNO, DebugNet, ViT`
(the reference discovers them through the `makani.models` entry-point group, pyproject.toml:106-112; additional
entry points of that group are honoured here too), `register_model(cls | "path.py:Class", name)`,
`list_models()`, `get_model(params)`.
"""

from __future__ import annotations

import importlib
import importlib.util
import logging
import os
from functools import partial
from typing import Callable, Dict, List, Union

import torch.nn as nn

from .stepper import MultiStepWrapper, SingleStepWrapper

_BUILTIN = {
    "AFNOv1": "makani_b200.models.networks.afnonet:AdaptiveFourierNeuralOperatorNet",
    "AFNO": "makani_b200.models.networks.afnonet_v2:AdaptiveFourierNeuralOperatorNet",
    "FNO": "makani_b200.models.networks.sfnonet:FourierNeuralOperatorNet",
    "SFNO": "makani_b200.models.networks.sfnonet:SphericalFourierNeuralOperatorNet",
    "DebugNet": "makani_b200.models.networks.debug:DebugNet",
    "ViT": "makani_b200.models.networks.vit:VisionTransformer",
}

_REGISTRY: Dict[str, Union[str, Callable]] = dict(_BUILTIN)


def _discover_entry_points():
    try:
        from importlib.metadata import entry_points
        for group in ("makani_b200.models", "makani.models"):     # own group, and plug-ins written for the reference
            for ep in entry_points(group=group):
                _REGISTRY.setdefault(ep.name, ep.value)
    except Exception:
        pass


_discover_entry_points()


def _resolve(spec):
    if not isinstance(spec, str):
        return spec
    mod, _, attr = spec.partition(":")
    if mod.endswith(".py") and os.path.exists(mod):
        s = importlib.util.spec_from_file_location(os.path.splitext(os.path.basename(mod))[0], mod)
        m = importlib.util.module_from_spec(s)
        s.loader.exec_module(m)
    else:
        m = importlib.import_module(mod)
    return getattr(m, attr)


def list_models() -> List[str]:
    return list(_REGISTRY.keys())


def register_model(model: Union[str, Callable], name: Union[str, None] = None) -> None:
    if isinstance(model, str):
        name = name or model.rpartition(":")[2]
    else:
        name = name or model.__name__
    if name in _REGISTRY:
        raise ValueError(f"Name {name} already in use")
    _REGISTRY[name] = model


def get_model_class(name: str):
    if name not in _REGISTRY:
        raise KeyError(f"No model is registered under the name {name}; available: {list_models()}")
    return _resolve(_REGISTRY[name])


def get_model(params, **kwargs) -> nn.Module:
    """Network named `params.nettype`, wrapped in a single- or multi-step stepper."""
    if params.nettype not in _REGISTRY:
        logging.warning(f"Net type {params.nettype} does not exist: registering")
        register_model(params.nettype)
    cls = get_model_class(params.nettype)
    inp_shape = (params.img_crop_shape_x, params.img_crop_shape_y)
    out_shape = (params.get("out_shape_x", params.img_crop_shape_x), params.get("out_shape_y", params.img_crop_shape_y))
    cfg = params.to_dict()
    for k in ("inp_shape", "out_shape", "inp_chans", "out_chans"):
        cfg.pop(k, None)
    model_handle = partial(cls, inp_shape=inp_shape, out_shape=out_shape, inp_chans=params.N_in_channels,
                           out_chans=params.N_out_channels, **cfg, **kwargs)

    def handle(_params):
        return model_handle()

    if params.get("n_future", 0) > 0:
        return MultiStepWrapper(params, handle)
    return SingleStepWrapper(params, handle)
