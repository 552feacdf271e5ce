"""Text generation: sampling rules and the single-prompt ``generate`` helper."""

from ajllm_b200.generation.sampling import sample_batch, sample_next_token, sampling_probabilities


def generate(*args, **kwargs):
    """See :func:`ajllm_b200.generation.generator.generate` (imported on first use: the generator
    depends on the engine, which itself uses this package's sampling rules)."""
    from ajllm_b200.generation.generator import generate as _generate

    return _generate(*args, **kwargs)


__all__ = ["generate", "sample_batch", "sample_next_token", "sampling_probabilities"]
