"""B200 implementation of vkllama's Llama-2 token loop.

Python is only a thin ctypes layer over the C ABI in include/vkllama_b200.h
(the same entry points a C++ caller of the reference would bind); the classes
keep the reference's names and argument order (src/ops/*.h, models/llama2.h).
The shared library is built in-tree by `python -m vkllama_b200.build`; there is
no fallback when it, or a CUDA device, is missing.
"""
from .api import (  # noqa: F401
    FP32, FP16, UINT32, INT8, Q8_0,
    VklError, Device, Tensor, Command,
    MatMul, FeedForward, MultiHeadAttentionV2, UpdateKVCache, RMSNorm, Rope, Softmax,
    ArgOp, ArgMax, ArgMin, Embedding, ElementWise, Transpose, Slice, Cast, Concat, Reduce, ReadKVCache,
    Model, ModelConfig, q8_0_quantize, q8_0_quantize36, q8_0_dequantize, blocks36_to_34,
    kernel_launches, library_path, load_library, matmul_run_many,
    Gguf, Sampler, TopkSampler, TopPSampler,
)
