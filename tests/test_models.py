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


def test_gpt_oss_qwen3_and_deepseek_r1_families():
    g = get_model("gpt-oss-120b")
    # 36 layers, 8 KV heads of 64 channels, K and V, bf16
    assert g.bytes_per_token_per_gpu(ParallelConfig()) == 36 * 2 * 8 * 64 * 2
    assert get_model("gpt-oss-20b").bytes_per_token_per_gpu(ParallelConfig(tp=8)) == 24 * 2 * 1 * 64 * 2
    q = get_model("qwen3-235b-a22b")
    assert q.cfg.head_dim == 128 and q.kv_heads_per_gpu(ParallelConfig(tp=4)) == 1
    assert q.bytes_per_token_per_gpu(ParallelConfig(tp=4, pp=2)) == 47 * 2 * 1 * 128 * 2
    assert get_model("qwen3-8b").block_bytes(16, ParallelConfig(tp=2)) == 16 * 4 * 128 * 2
    assert get_model("deepseek-r1").bytes_per_token_per_gpu(ParallelConfig(tp=8)) == get_model("deepseek-v3").bytes_per_token_per_gpu(ParallelConfig())
    assert get_model("llama-3.1-70b") is get_model("llama-3-70b")
    # fp8 cache halves everything
    assert get_model("gpt-oss-120b", "fp8").bytes_per_token_per_gpu(ParallelConfig()) * 2 == g.bytes_per_token_per_gpu(ParallelConfig())


def test_models_and_serving_configs_from_yaml(tmp_path):
    import json
    import subprocess
    import sys

    from nixl_b200.models import DeepSeekV3, model_from_yaml

    gqa = tmp_path / "m.yaml"
    gqa.write_text("model_name: 'MY_MODEL'\nnum_layers: 10\nnum_query_heads: 16\nnum_kv_heads: 2\nquery_head_dimension: 96\n")
    m = model_from_yaml(str(gqa))
    assert m.cfg.name == "my-model" and m.bytes_per_token_per_gpu(ParallelConfig(tp=2)) == 10 * 2 * 1 * 96 * 2
    mla = tmp_path / "mla.yaml"
    mla.write_text("model_name: 'X'\nnum_layers: 4\nnum_query_heads: 8\nquery_head_dimension: 128\nembedding_dimension: 1024\n"
                   "rope_mla_dimension: 64\nmla_latent_vector_dimension: 512\n")
    d = model_from_yaml(str(mla), "fp8")
    assert isinstance(d, DeepSeekV3) and d.bytes_per_token_per_gpu(ParallelConfig(tp=4)) == 4 * 576
    serving = tmp_path / "serve.yaml"
    serving.write_text("strategy:\n  tp_size: 2\n  pp_size: 5\n  kvcache_quant_mode: 'fp8'\nruntime:\n  isl: 320\n  num_requests: 3\nsystem:\n  page_size: 32\n")
    out = subprocess.run([sys.executable, "-m", "benchmarks.kvbench", "kvcache", "--model", str(gqa), "--model_config", str(serving)],
                         capture_output=True, text=True, check=True)
    rep = json.loads(out.stdout)
    assert (rep["tp"], rep["pp"], rep["isl"], rep["num_requests"], rep["page_size"]) == (2, 5, 320, 3, 32)
    assert rep["bytes_per_token_per_gpu"] == 2 * 2 * 1 * 96 * 1 and rep["io_size"] == 32 * 1 * 96
