"""Dataset descriptors and helpers (ERA5 year files, Copernicus download requests)."""
