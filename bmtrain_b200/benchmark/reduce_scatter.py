"""``bmt.benchmark.reduce_scatter`` under its historical module path (reference: ``bmtrain/benchmark/reduce_scatter.py``)."""
from .collectives import reduce_scatter  # noqa: F401
