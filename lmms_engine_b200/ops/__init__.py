"""Operators of the engine.  CUDA bf16 tensors run hand-written sm_100a kernels; other
tensors run the fp32 PyTorch formulations that double as test oracles."""
