"""The upstream module name of the synthetic-data loader (makani/utils/dataloaders/data_loader_dummy.py:35-190):
`DummyLoader(params, location, train, device)` is `SyntheticLoader` of `data_loader_synthetic.py`, which has the same
constructor, normalisation getters, length and iteration protocol (and, unlike the upstream class, can be iterated)."""

from .data_loader_synthetic import SyntheticLoader


class DummyLoader(SyntheticLoader):
    pass
