"""miles_b200 — a Blackwell-native RL post-training framework (GRPO/GSPO/PPO, colocated and async
rollout, R3 routing replay, LoRA, HF + torch_dist checkpoints) with hand-written sm_100a kernels."""

__version__ = "0.1.0"
