from .manager import DistributedManager  # noqa: F401
