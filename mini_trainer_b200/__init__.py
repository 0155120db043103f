"""mini_trainer_b200 — a Blackwell-native fine-tuning framework.

Same capabilities, CLI and checkpoint format as Red-Hat-AI-Innovation-Team/mini_trainer:
padding-free packed SFT / pretraining, LPT minibatch packing to a per-GPU token budget, automatic
gradient accumulation, fully sharded training, JSONL metrics and bf16 HF-safetensors checkpoints.
"""
__version__ = "0.1.0"
