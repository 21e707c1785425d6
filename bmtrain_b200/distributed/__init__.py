from .ops import all_gather, all_reduce, reduce_scatter, broadcast, send_activations, recv_activations
