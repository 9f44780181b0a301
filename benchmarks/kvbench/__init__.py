"""KV-cache benchmarking tools: size math, nixlbench plans, traffic-matrix workloads, fused KV transfer.

Covers what the reference's benchmark/kvbench offers (main.py commands plan / profile / kvcache /
ct-perftest / sequential-ct-perftest and test/inference_workload_matgen.py), driven through
``python -m benchmarks.kvbench <command>``; the etcd runtime is replaced by torch.distributed."""
