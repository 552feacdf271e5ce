"""One module per user verb; each exposes ``run(LoadedConfig) -> dict``."""
