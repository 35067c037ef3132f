"""Engine hooks: how sglang and vLLM calls reach the B200 fused-MoE ops (and fall back to the engine)."""
