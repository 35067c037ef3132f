"""Contract, environment and dispatch layer of the B200 fused-MoE ops (one backend: sm_100a)."""
