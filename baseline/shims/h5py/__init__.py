"""Import-time stand-in for `h5py` (absent from this image).  The benchmark feeds synthetic tensors; opening a file fails."""


class File:
    def __init__(self, *args, **kwargs):
        raise ImportError("h5py is not installed in this image; the reference arm runs on synthetic tensors only")
