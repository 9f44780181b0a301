"""KV-cache size models of common LLM architectures (what a transfer has to move).

The library moves bytes, not activations; these classes answer "how many bytes is the KV cache
of one request on one GPU under this parallelism", which sizes buffers, descriptor lists and
benchmark traffic.  Parity: the model files of the reference's kvbench tool
(benchmark/kvbench/models/*.py, e.g. llama3_1.py:62-93, utils.py:34)."""
from .kv_models import (  # noqa: F401
    MODELS,
    DeepSeekV3,
    GptOss,
    KVModel,
    Llama3,
    ModelConfig,
    ParallelConfig,
    Qwen3,
    batch_descriptor_count,
    get_model,
    model_from_yaml,
)
