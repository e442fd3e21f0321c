"""Configuration, tracing, logging."""
from .config import ComprexConfig
from .log import JsonlWriter, StepLogger, get_logger
from .trace import PhaseTimer, TictocTimer, enable_nvtx, nvtx_range

__all__ = ["ComprexConfig", "JsonlWriter", "StepLogger", "get_logger", "PhaseTimer", "TictocTimer",
           "enable_nvtx", "nvtx_range"]
