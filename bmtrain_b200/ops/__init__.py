"""Hot operators.  CUDA tensors run the hand-written sm_100a kernels in ``_C.so``;
CPU tensors run the plain PyTorch definition of the same op (the numerical oracle)."""
