"""B200-native LLM stack: tokenizer, decoder-only dense/MoE training with TP/EP/FSDP,
and a paged-KV inference engine, on hand-written sm_100a kernels.

The user-facing contract (YAML configs, workflows, run directories, checkpoint dictionary)
follows Huangsj1/ajLLM (``ajllm_project/src/ajllm/__init__.py:1-3``).
"""

__version__ = "0.1.0"
