"""``bmt.benchmark.send_recv`` under its historical module path (reference: ``bmtrain/benchmark/send_recv.py``)."""
from .collectives import send_recv  # noqa: F401
