"""comprex_b200: compressed vector exchange and allreduce for NVLink-connected B200 GPUs.

Same capabilities and Python surface as the ComprEx library (GaspiEx / ComprEx
point-to-point engines, top-k thresholds with local residual accumulation, the
AllToOne / Ring / BigRing allreduce variants, the compressed data-parallel
optimizer), built on hand-written sm_100a kernels that store compressed
payloads directly into peer GPUs' memory.
"""
from ._lib import ComprexError, launch_count  # noqa: F401
from .common import Getable, Gettable, Subscribable  # noqa: F401
from .gpi import GaspiEnvironment, Gaspi_Runtime, Gaspi_Segment, LoopbackWorld, gaspi_printf, initGaspiCxx  # noqa: F401
from .GaspiEx import GaspiEx  # noqa: F401
from .ComprEx import (Comprex, FastComprex, ThresholdNone, ThresholdConst, ThresholdTopK,  # noqa: F401
                      CompressorNone, CompressorRLE, CompressorIndexPairs)
from .allreduce import (AllToOneAllreduce, RingAllreduce, BigRingAllreduce, AutoAllreduce,  # noqa: F401
                        Comprex_AllToOneAllreduce, Comprex_RingAllreduce, Comprex_BigRingAllreduce,
                        select_schedule)
from .utils import ComprexConfig  # noqa: F401

__version__ = "0.1.0"
