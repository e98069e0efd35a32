"""cubework_b200 — multi-dimensional (1D / 2D SUMMA / 3D cube) tensor parallelism for B200.

Public API parity with ``cubework`` (cubework/__init__.py:1-3): ``get_args``, ``parse_args``,
``initialize_distributed``, ``destroy_distributed``; sub-packages ``module`` (layers, losses, metrics,
initializers), ``distributed`` (topology + collectives) and ``utils``.
"""
from .arguments import get_args, parse_args
from .initialize import __version__, initialize_distributed
from .parallel.mesh import destroy_distributed

__all__ = ["get_args", "parse_args", "initialize_distributed", "destroy_distributed", "__version__"]
