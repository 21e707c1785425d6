"""``bmt.benchmark.all_gather`` under its historical module path (reference: ``bmtrain/benchmark/all_gather.py``)."""
from .collectives import all_gather  # noqa: F401
