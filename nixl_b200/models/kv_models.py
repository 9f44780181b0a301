"""KV-cache geometry per model family and parallel layout."""
from __future__ import annotations

import math
from dataclasses import dataclass, field


@dataclass(frozen=True)
class ParallelConfig:
    """Model-parallel layout of one serving instance."""

    tp: int = 1  # tensor parallel: KV heads are split
    pp: int = 1  # pipeline parallel: layers are split
    cp: int = 1  # context parallel: tokens are split
    ep: int = 1  # expert parallel (no effect on KV size; kept for workload generators)


@dataclass(frozen=True)
class ModelConfig:
    name: str
    num_layers: int
    num_heads: int
    num_kv_heads: int
    hidden: int
    head_dim: int = 0
    kv_bytes: int = 2  # bf16
    extra: dict = field(default_factory=dict)

    def __post_init__(self):
        if self.head_dim == 0:
            object.__setattr__(self, "head_dim", self.hidden // self.num_heads)


class KVModel:
    """Multi-head / grouped-query attention: K and V of ``num_kv_heads x head_dim`` per token per layer."""

    def __init__(self, cfg: ModelConfig):
        self.cfg = cfg

    def kv_heads_per_gpu(self, par: ParallelConfig) -> int:
        # With more TP ranks than KV heads the heads are replicated, never split below one.
        return max(1, self.cfg.num_kv_heads // par.tp)

    def layers_per_gpu(self, par: ParallelConfig) -> int:
        return math.ceil(self.cfg.num_layers / par.pp)

    def bytes_per_token_per_gpu(self, par: ParallelConfig) -> int:
        return 2 * self.layers_per_gpu(par) * self.kv_heads_per_gpu(par) * self.cfg.head_dim * self.cfg.kv_bytes

    def kv_bytes_per_gpu(self, tokens: int, par: ParallelConfig) -> int:
        return math.ceil(tokens / par.cp) * self.bytes_per_token_per_gpu(par)

    def block_bytes(self, block_tokens: int, par: ParallelConfig) -> int:
        """Bytes of one paged block of one cache tensor (K or V of one layer) on one GPU."""
        return block_tokens * self.kv_heads_per_gpu(par) * self.cfg.head_dim * self.cfg.kv_bytes

    def cache_tensors_per_gpu(self, par: ParallelConfig) -> int:
        return 2 * self.layers_per_gpu(par)


class Llama3(KVModel):
    pass


class DeepSeekV3(KVModel):
    """Multi-head latent attention: one compressed KV vector (kv_lora_rank + rope dim) per token per
    layer, shared by all heads, so tensor parallelism does not shrink it."""

    def bytes_per_token_per_gpu(self, par: ParallelConfig) -> int:
        latent = self.cfg.extra.get("kv_lora_rank", 512) + self.cfg.extra.get("qk_rope_head_dim", 64)
        return self.layers_per_gpu(par) * latent * self.cfg.kv_bytes

    def block_bytes(self, block_tokens: int, par: ParallelConfig) -> int:
        latent = self.cfg.extra.get("kv_lora_rank", 512) + self.cfg.extra.get("qk_rope_head_dim", 64)
        return block_tokens * latent * self.cfg.kv_bytes

    def cache_tensors_per_gpu(self, par: ParallelConfig) -> int:
        return self.layers_per_gpu(par)


class GptOss(KVModel):
    """Grouped-query attention with 64-wide heads (gpt-oss 20B / 120B)."""


class Qwen3(KVModel):
    """Grouped-query attention with 128-wide heads that are not hidden / num_heads (Qwen3 dense and MoE)."""


_MLA = {"kv_lora_rank": 512, "qk_rope_head_dim": 64, "routed_experts": 256, "topk": 8, "moe_intermediate": 2048}

MODELS = {
    "llama-3-8b": Llama3(ModelConfig("llama-3-8b", 32, 32, 8, 4096)),
    "llama-3-70b": Llama3(ModelConfig("llama-3-70b", 80, 64, 8, 8192)),
    "llama-3.1-405b": Llama3(ModelConfig("llama-3.1-405b", 126, 128, 8, 16384)),
    "deepseek-v3": DeepSeekV3(ModelConfig("deepseek-v3", 61, 128, 128, 7168, head_dim=128, extra=dict(_MLA))),
    "deepseek-r1": DeepSeekV3(ModelConfig("deepseek-r1", 61, 128, 128, 7168, head_dim=128, extra=dict(_MLA))),
    "gpt-oss-20b": GptOss(ModelConfig("gpt-oss-20b", 24, 64, 8, 2880, head_dim=64, extra={"routed_experts": 32, "topk": 4})),
    "gpt-oss-120b": GptOss(ModelConfig("gpt-oss-120b", 36, 64, 8, 2880, head_dim=64, extra={"routed_experts": 128, "topk": 4})),
    "qwen3-8b": Qwen3(ModelConfig("qwen3-8b", 36, 32, 8, 4096, head_dim=128)),
    "qwen3-235b-a22b": Qwen3(ModelConfig("qwen3-235b-a22b", 94, 64, 4, 4096, head_dim=128, extra={"routed_experts": 128, "topk": 8})),
}
MODELS["llama-3.1-8b"] = MODELS["llama-3-8b"]
MODELS["llama-3.1-70b"] = MODELS["llama-3-70b"]

_QUANT_BYTES = {"fp8": 1, "int8": 1, "fp16": 2, "bf16": 2, "fp32": 4}


def model_from_yaml(path: str, kvcache_quant: str = "") -> KVModel:
    """A model from an architecture file with the keys the reference's kvbench uses
    (benchmark/kvbench/examples/model_*.yaml): ``model_name, num_layers, num_query_heads,
    query_head_dimension`` and either ``num_kv_heads`` (grouped-query attention) or
    ``mla_latent_vector_dimension`` + ``rope_mla_dimension`` (multi-head latent attention)."""
    import yaml

    with open(path) as f:
        d = yaml.safe_load(f)
    name = str(d["model_name"]).lower().replace("_", "-")
    layers, heads, head_dim = int(d["num_layers"]), int(d["num_query_heads"]), int(d["query_head_dimension"])
    kv_bytes = _QUANT_BYTES.get(kvcache_quant.lower(), 2) if kvcache_quant else 2
    if "mla_latent_vector_dimension" in d:
        extra = {"kv_lora_rank": int(d["mla_latent_vector_dimension"]), "qk_rope_head_dim": int(d.get("rope_mla_dimension", 64))}
        cfg = ModelConfig(name, layers, heads, heads, int(d.get("embedding_dimension", heads * head_dim)), head_dim=head_dim, kv_bytes=kv_bytes,
                          extra=extra)
        return DeepSeekV3(cfg)
    cfg = ModelConfig(name, layers, heads, int(d["num_kv_heads"]), int(d.get("embedding_dimension", heads * head_dim)), head_dim=head_dim,
                      kv_bytes=kv_bytes)
    return KVModel(cfg)


def get_model(name: str, kvcache_quant: str = "") -> KVModel:
    """A built-in model by name, or an architecture YAML file by path.  ``kvcache_quant``
    (``fp8``, ``bf16``, ...) sets the bytes per cached element."""
    if name.endswith((".yaml", ".yml")):
        return model_from_yaml(name, kvcache_quant)
    try:
        m = MODELS[name.lower()]
    except KeyError:
        raise KeyError(f"unknown model {name!r}; known: {sorted(MODELS)}") from None
    if kvcache_quant:
        import dataclasses

        m = type(m)(dataclasses.replace(m.cfg, kv_bytes=_QUANT_BYTES.get(kvcache_quant.lower(), 2)))
    return m


def batch_descriptor_count(model: KVModel, tokens: int, requests: int, par: ParallelConfig, io_bytes: int) -> int:
    """Descriptors a descriptor-list transfer needs: ceil(KV bytes of the batch / bytes per descriptor)."""
    return math.ceil(model.kv_bytes_per_gpu(tokens, par) * requests / io_bytes)
