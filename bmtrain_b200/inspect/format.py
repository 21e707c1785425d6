"""Fixed-width text table for inspection summaries (reference: ``bmtrain/inspect/format.py:25-62``).

Columns: name (width = longest name + 4), shape (20), then max / min / std /
mean / grad_std / grad_mean (10 each).  Every cell is prefixed by one blank and
cut to its column; floats print with four decimals.
"""
from typing import Any, Dict, List

_COLUMNS = ("name", "shape", "max", "min", "std", "mean", "grad_std", "grad_mean")


def _cell(value: Any, width: int) -> str:
    text = f"{value:.4f}" if isinstance(value, float) else str(value)
    text = " " + (text[: width - 1] if len(text) + 1 > width else text)
    return text.ljust(width)


def item_formater(x: Any) -> str:
    """Cell text of one value: floats with four decimals, everything else through ``str``."""
    return f"{x:.4f}" if isinstance(x, float) else str(x)


def align_str(s: str, align: int, left: bool) -> str:
    """Pad ``s`` with blanks to ``align`` characters on the right (``left``) or on the left."""
    return s.ljust(align) if left else s.rjust(align)


def format_line(strs: List[str], length: List[int]) -> str:
    """One table row: every string gets a leading blank, is cut to its column and padded to the column width."""
    return "".join(_cell(v, w) for v, w in zip(strs, length))


def format_summary(summary: List[Dict[str, Any]]) -> str:
    """Render a list of summary dicts (from ``inspect_model`` / ``InspectTensor.get_summary``)."""
    name_width = max([len("name")] + [len(item["name"]) for item in summary]) + 4
    widths = [name_width, 20] + [10] * 6
    lines = ["".join(_cell(h, w) for h, w in zip(_COLUMNS, widths))]
    for item in summary:
        lines.append("".join(_cell(item[h], w) for h, w in zip(_COLUMNS, widths)))
    return "\n".join(lines)
