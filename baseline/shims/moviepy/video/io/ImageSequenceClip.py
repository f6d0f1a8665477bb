"""Import-time stand-in: the reference only builds clips when it logs videos, which the benchmark never does."""


class ImageSequenceClip:
    def __init__(self, *args, **kwargs):
        raise ImportError("moviepy is not installed in this image")
