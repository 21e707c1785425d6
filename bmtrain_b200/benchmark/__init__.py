"""Collective micro-benchmarks (reference: ``bmtrain/benchmark/*.py``): device-timed, warmed up, max over ranks."""
from .collectives import all_gather, reduce_scatter, send_recv
