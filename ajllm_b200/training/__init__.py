"""Training primitives and the run loop."""

from ajllm_b200.training.checkpoint import load_checkpoint, save_checkpoint
from ajllm_b200.training.data import BatchStager, SyntheticTokens, TokenDataset
from ajllm_b200.training.logger import RunLogger
from ajllm_b200.training.losses import cross_entropy
from ajllm_b200.training.optim import AdamW, FlatAdamW, clip_gradients
from ajllm_b200.training.schedulers import warmup_cosine_learning_rate
from ajllm_b200.training.trainer import Trainer, optimizer_step

__all__ = [
    "load_checkpoint", "save_checkpoint", "BatchStager", "SyntheticTokens", "TokenDataset", "RunLogger",
    "cross_entropy", "AdamW", "FlatAdamW", "clip_gradients", "warmup_cosine_learning_rate", "Trainer",
    "optimizer_step",
]
