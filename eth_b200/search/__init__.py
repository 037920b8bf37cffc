"""HPP configuration search (CPU only): profile tables -> cost model -> pipeline split,
stage boundaries, per-stage TP/DP, micro-batch size, recompute -> normalized gpt_config.json."""
