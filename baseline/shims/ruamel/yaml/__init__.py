"""Stand-in for `ruamel.yaml` (absent from this image): `YAML().load(stream)` on top of PyYAML."""

import yaml as _yaml


class YAML:
    def __init__(self, typ=None, pure=False, **kwargs):
        self.typ = typ

    def load(self, stream):
        return _yaml.safe_load(stream)

    def dump(self, data, stream=None):
        return _yaml.safe_dump(data, stream)
