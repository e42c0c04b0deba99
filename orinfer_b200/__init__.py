"""orinfer_b200: a Blackwell (sm_100a) native LLM inference engine.

Layers, top to bottom: ``api`` (OpenAI / Ollama HTTP surface, CLI), ``engine``
(continuous batching, prefix cache, MTP, CUDA-graph pool), ``models`` (dense /
MoE / hybrid decoders), ``parallel`` (tensor / expert parallel plumbing and the
fused compute+collective kernels), ``ops`` (hand-written CUDA kernels bound via
ctypes), ``quant`` (E8P / W8 / A8 / INT8-KV codecs) and ``core`` (C++ policy
core: scheduler, radix prefix cache, sampling law, MTP controller).
"""

__version__ = "0.1.0"
