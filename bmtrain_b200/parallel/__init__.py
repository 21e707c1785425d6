"""Multi-GPU building blocks: peer-memory (NVLink) buffers and the fused compute+collective operators."""
