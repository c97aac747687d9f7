"""owl_engine_b200 -- a Blackwell (B200, sm_100a) native LLM inference engine.

Package map:

* ``models``   model specs, the fp32 CPU reference model, the GPU runner, vision / draft heads
* ``ops``      Python entry points of the CUDA kernels plus their fp32 PyTorch references
* ``formats``  checkpoint readers and quantised-weight codecs (safetensors, AWQ, NVFP4, GGUF)
* ``parallel`` tensor-parallel plan / shard rules, symmetric memory, fused collectives
* ``engine``   scheduler, executor, CUDA-graph fleet, state pool, sampler, speculative decoding
* ``store``    KV block ledger, prefix tree, host / disk tiers, budget and admission
* ``server``   OpenAI-compatible HTTP/SSE surface, chat template, tool-call splitter, /debug
* ``utils``    config profiles, logging, metrics, step gate, GPU lock, test kit
"""
__version__ = "0.1.0"
