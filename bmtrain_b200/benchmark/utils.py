"""Size formatting of the benchmark printouts (reference: ``bmtrain/benchmark/utils.py``)."""


def format_size_(x: int) -> str:
    for unit, shift in (("B", 0), ("KB", 10), ("MB", 20)):
        if x < 1 << (shift + 10):
            return f"{x:d}B" if shift == 0 else f"{x / (1 << shift):4.2f}{unit}"
    return f"{x / (1 << 30):4.2f}GB"


def format_size(x: int) -> str:
    """At most six characters."""
    return format_size_(x)[:6]
