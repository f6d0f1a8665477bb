"""Import-time stand-in for `moviepy.video.io` (absent from this image)."""

from . import ImageSequenceClip  # noqa: F401
