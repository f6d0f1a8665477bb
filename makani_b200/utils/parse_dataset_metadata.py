"""Parser for the dataset descriptor `data.json` (contract: makani/utils/parse_dataset_metada.py:19-56)."""

import json


def parse_dataset_metadata(metadata_json_path, params):
    with open(metadata_json_path, "r") as f:
        metadata = json.load(f)
    coords = metadata.get("coords", metadata.get("coord"))
    params["h5_path"] = metadata["h5_path"]
    params["dhours"] = metadata["dhours"]
    params["lat"] = coords["lat"]
    params["lon"] = coords["lon"]
    params["data_grid_type"] = coords["grid_type"]
    channel_names = coords["channel"]
    if params.get("channel_names") is not None:
        idx = []
        for name in params["channel_names"]:
            if name not in channel_names:
                raise ValueError(f"Error, requested channel {name} not found in dataset.")
            idx.append(channel_names.index(name))
    else:
        params["channel_names"] = channel_names
        idx = list(range(len(channel_names)))
    params["in_channels"] = idx
    params["out_channels"] = idx
    params["dataset"] = dict(name=metadata.get("dataset_name", ""), description=metadata.get("attrs", {}).get("description", ""),
                             metadata_file=metadata_json_path)
    return params, metadata
