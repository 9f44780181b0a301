"""KV-size math against hand-computed values of the benchmark shapes."""
from nixl_b200.models import ParallelConfig, batch_descriptor_count, get_model


def test_llama3_8b_kv_geometry():
    m = get_model("llama-3-8b")
    tp4, tp2 = ParallelConfig(tp=4), ParallelConfig(tp=2)
    assert m.kv_heads_per_gpu(tp4) == 2 and m.kv_heads_per_gpu(tp2) == 4
    assert m.block_bytes(16, tp4) == 16 * 2 * 128 * 2 == 8192
    assert m.cache_tensors_per_gpu(tp4) == 64
    # 8 requests x 4096 tokens: 1 GiB per prefill GPU at TP4 (the kvbench figure)
    assert m.kv_bytes_per_gpu(4096, tp4) * 8 == 1 << 30
    assert batch_descriptor_count(m, 4096, 8, tp4, 8192) == 131072
    assert m.kv_bytes_per_gpu(4096, ParallelConfig(tp=16)) == m.kv_bytes_per_gpu(4096, ParallelConfig(tp=8))  # heads replicate below 1


def test_pipeline_and_context_parallel_and_mla():
    m = get_model("llama-3-70b")
    assert m.layers_per_gpu(ParallelConfig(pp=4)) == 20
    assert m.kv_bytes_per_gpu(1000, ParallelConfig(cp=4)) == 250 * m.bytes_per_token_per_gpu(ParallelConfig())
    d = get_model("deepseek-v3")
    assert d.bytes_per_token_per_gpu(ParallelConfig(tp=8)) == 61 * 576 * 2  # latent KV is not split by TP
