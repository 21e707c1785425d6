from .format import format_summary
from .model import inspect_model
from .tensor import inspect_tensor, record_tensor, InspectTensor
