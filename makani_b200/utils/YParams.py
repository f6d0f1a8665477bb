"""Recipe/configuration container.

Behaviour contract of the reference's `ParamsBase` / `YParams` (makani/utils/YParams.py:19-93): a bag with both
attribute and item access, `"None"` strings mapped to `None`, `YParams(yaml_file, section)` loading one named
section of a YAML file that may use anchors and merge keys, `from_json`, `to_dict`, `update_params`, `log`.
PyYAML's safe loader resolves anchors/merge keys, so no other YAML package is needed.
"""

from __future__ import annotations

import json
import logging

import yaml


class ParamsBase:
    """Attribute + dict style parameter bag."""

    def __init__(self):
        self._yaml_filename = "no file"
        self._config_name = "no config"
        self.params = {}

    def __getitem__(self, key):
        return self.params[key]

    def __setitem__(self, key, val):
        self.params[key] = val
        self.__dict__[key] = val

    def __setattr__(self, key, val):
        object.__setattr__(self, key, val)
        if not key.startswith("_") and key != "params" and "params" in self.__dict__:
            self.__dict__["params"][key] = val

    def __contains__(self, key):
        return key in self.params

    def get(self, key, default=None):
        if key in self.params:
            return self.params[key]
        return getattr(self, key, default)

    def keys(self):
        return self.params.keys()

    def to_dict(self):
        return dict(self.params)

    @classmethod
    def from_json(cls, path):
        with open(path) as f:
            d = json.load(f)
        obj = cls()
        obj.update_params(d)
        return obj

    def update_params(self, config):
        for key, val in config.items():
            if val == "None":
                val = None
            self[key] = val

    def log(self, logger=None):
        logger = logger or logging.getLogger()
        logger.info("------------------ Configuration ------------------")
        logger.info("Configuration file: " + str(self._yaml_filename))
        logger.info("Configuration name: " + str(self._config_name))
        for key, val in self.to_dict().items():
            logger.info(f"{key} {val}")
        logger.info("---------------------------------------------------")


class YParams(ParamsBase):
    """Loads the section `config_name` of `yaml_filename`."""

    def __init__(self, yaml_filename, config_name, print_params=False):
        super().__init__()
        self._yaml_filename = yaml_filename
        self._config_name = config_name
        with open(yaml_filename) as f:
            doc = yaml.safe_load(f)
        if config_name not in doc:
            raise KeyError(f"config '{config_name}' not found in {yaml_filename}; available: {sorted(doc.keys())}")
        self.update_params(doc[config_name])
        if print_params:
            self.log()

    def __reduce__(self):
        # pickles (legacy checkpoints store the params object) rebuild without re-reading the YAML file
        return (_rebuild_params, (self.to_dict(), self._yaml_filename, self._config_name))


def _rebuild_params(d, yaml_filename, config_name):
    obj = ParamsBase()
    obj._yaml_filename = yaml_filename
    obj._config_name = config_name
    obj.update_params(d)
    return obj
