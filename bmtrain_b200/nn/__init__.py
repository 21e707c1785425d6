from .linear import Linear, OpLinear
from .column_parallel_linear import ColumnParallelLinear
from .row_parallel_linear import RowParallelLinear
from .parallel_embedding import VPEmbedding, ParallelEmbedding
from .parallel_linear_func import OpParallelLinear, ReduceType
from .layers import Embedding, LayerNorm, RMSNorm
