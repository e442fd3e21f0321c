"""Runtime (ranks, symmetric heap) and the data-parallel wrapper."""
from .env import GaspiEnvironment, LoopbackWorld  # noqa: F401
