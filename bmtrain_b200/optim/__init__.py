from .adam import AdamOptimizer
from .adam_offload import AdamOffloadOptimizer
from .optim_manager import OptimManager, check_overflow, grad_rescale
