"""mlxcel_b200 — a Blackwell-native (B200, sm_100a) LLM inference engine and server.

Layers, bottom up:

* ``csrc/``      hand-written sm_100a CUDA kernels behind a C ABI (``lib/libmlxcel_b200.so``)
* ``host/``      C++ host runtime: KV block manager, prefix index, tick policy
* ``ops/``       Python bindings of the kernels + plain PyTorch reference implementations
* ``loading/``   MLX safetensors checkpoints, quantization formats, TP/EP/PP sharding
* ``models/``    decoder families on top of ``ops``
* ``cache/``     paged / quantized KV pool, prompt cache
* ``engine/``    Engine (open/prefill/step/verify_round/close), samplers, scheduler
* ``parallel/``  tensor / expert / pipeline parallel runtime, fused compute+collective ops
* ``speculative/`` MTP / draft-model / prompt-lookup drafters
* ``server/``    OpenAI- and llama-server-compatible HTTP API
* ``cli.py``     ``mlxcel`` command line
"""
__version__ = "0.1.0"

from .config import ModelConfig  # noqa: F401
