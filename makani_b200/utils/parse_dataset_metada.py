"""The upstream spelling of this module's name (makani/utils/parse_dataset_metada.py); see `parse_dataset_metadata.py`."""

from .parse_dataset_metadata import parse_dataset_metadata  # noqa: F401
