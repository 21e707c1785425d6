"""Message sizes of the collective sweeps in bytes (reference: ``bmtrain/benchmark/shape.py``: 1 KiB ... 4 GiB)."""
SHAPES = [2 ** i for i in range(10, 33)]
