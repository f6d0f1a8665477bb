"""Names of the auxiliary input channels appended by the loader / preprocessor (zenith angle, coordinate grid,
orography, land-sea mask); must stay in sync with `Preprocessor2D` (contract: makani/utils/features.py:17-47)."""


def get_auxiliary_channels(add_zenith=False, add_grid=False, gridtype=None, grid_type=None, grid_num_frequencies=0,
                           add_orography=False, add_landmask=False, **kwargs):
    names = []
    gtype = gridtype if gridtype is not None else grid_type
    if add_zenith:
        names.append("xzen")
    if add_grid:
        if gtype == "sinusoidal":
            for f in range(1, int(grid_num_frequencies or 1) + 1):
                names += [f"xsgrlat{f}", f"xsgrlon{f}"]
        else:
            names += ["xgrlat", "xgrlon"]
    if add_orography:
        names.append("xoro")
    if add_landmask:
        names += ["xlsml", "xlsms"]
    return names
