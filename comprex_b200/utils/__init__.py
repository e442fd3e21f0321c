"""Configuration, tracing, logging."""
from .config import ComprexConfig
from .data import AsyncScalar, DevicePrefetcher
from .log import JsonlWriter, StepLogger, get_logger
from .trace import PhaseTimer, TictocTimer, enable_nvtx, nvtx_range

__all__ = ["ComprexConfig", "AsyncScalar", "DevicePrefetcher", "JsonlWriter", "StepLogger", "get_logger", "PhaseTimer", "TictocTimer",
           "enable_nvtx", "nvtx_range"]
