from .clip_grad import clip_grad_norm
from .common import free_port, get_current_device, seed, set_device, set_seed
from .data import SyntheticLoader, get_dataloader
from .logging import get_logger, init_logger, write_logger_to_file
from .profiling import CommProfiler, MemoryTracker, calc_model_size, calc_tflops

__all__ = [
    "clip_grad_norm", "free_port", "get_current_device", "seed", "set_device", "set_seed", "get_dataloader",
    "SyntheticLoader", "get_logger", "init_logger", "write_logger_to_file", "CommProfiler", "MemoryTracker",
    "calc_model_size", "calc_tflops"
]

from . import checkpoint  # noqa: E402  (after the names above: it imports the parallel package)
