"""b200serve: a Blackwell-native LLM inference server.

Subpackages
-----------
models    model descriptors, the fp32 CPU oracle, the GPU decoder models
ops       hand-written sm_100a kernels (``ops/csrc``) and their Python bindings
parallel  tensor / expert / pipeline parallel engines and replica mode
runtime   CUDA-graph decode engine, paged KV, memory planner, speculative decoding
loader    safetensors reader, quantisation config checks, weight repacking
server    OpenAI-compatible HTTP server, scheduler, prefix cache bindings
native    C++ host library (allocator, prefix cache, tokenizer, parsers, HTTP)
cli       ``serve`` and ``decode`` entry points
utils     int4 formats, synthetic checkpoints, timing helpers
"""
__version__ = "0.1.0"
