"""fastllm_b200 -- a Blackwell (sm_100a) native LLM inference framework.

Layers: ``ops`` (hand-written CUDA kernels behind a small functional API, PyTorch definitions on CPU),
``models`` (paged-KV decoder families), ``parallel`` (tensor / expert parallel communication over
NVLink), ``engine`` (continuous batching, paged KV with prefix cache, CUDA-graph decode), ``loader``
(safetensors / .flm / GGUF readers, quantiser, exporter), ``serving`` (OpenAI-style server, CLI).
"""
__version__ = "0.1.0"
