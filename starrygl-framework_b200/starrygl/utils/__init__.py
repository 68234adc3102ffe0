from .context import DistributedContext  # noqa: F401
