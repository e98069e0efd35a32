from .communication import CommProfiler
from .flops import calc_model_size, calc_tflops
from .memory_tracker import MemoryTracker

__all__ = ["CommProfiler", "calc_model_size", "calc_tflops", "MemoryTracker"]
