"""bmtrain_b200 -- a Blackwell-native toolkit for training big models.

Public surface follows OpenBMB/BMTrain (``import bmtrain_b200 as bmt``):
``init_distributed``, ``DistributedParameter`` / ``DistributedModule``,
``Block`` (ZeRO-2/3 + checkpointing), ``TransformerBlockList``,
``PipelineTransformerBlockList``, ``nn`` (tensor-parallel layers), ``optim``
(Adam, host-offloaded Adam, ``OptimManager`` loss scaling), ``lr_scheduler``,
``loss.FusedCrossEntropy``, ``save`` / ``load``, ``inspect`` and ``benchmark``.
"""
from .global_var import config, world_size, rank
from .init import init_distributed, is_initialized, shutdown
from .parameter import DistributedParameter, ParameterInitializer
from .layer import DistributedModule
from .param_init import init_parameters, grouped_parameters
from .synchronize import synchronize, sum_loss, wait_loader, gather_result
from .block_layer import Block, TransformerBlockList
from .wrapper import BMTrainModelWrapper
from .pipe_layer import PipelineTransformerBlockList
from .utils import print_block, print_dict, print_rank, see_memory, load_nccl_pypi
from . import debug
from . import watchdog
from .store import save, load

from . import loss
from . import distributed
from . import nn
from . import optim
from . import inspect
from . import lr_scheduler
from . import benchmark
from . import nccl
from . import models

CheckpointBlock = Block

__version__ = "0.1.0"
