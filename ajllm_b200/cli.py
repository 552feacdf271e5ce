"""Command line: ``ajllm-b200 {tokenizer {train,encode} | lm {train,sweep,evaluate,compare,generate} |
model report} --config FILE`` (reference: ``ajllm/cli.py:25-65``). The workflow's result dictionary is
printed as JSON; configuration and file errors become argparse errors."""

from __future__ import annotations

import argparse
import importlib
import json
from typing import Any

from ajllm_b200.config import load_run_config

VERBS = {
    "tokenizer": {"train": ("tokenizer_train", "Train a byte-level BPE tokenizer"),
                  "encode": ("tokenizer_encode", "Encode dataset splits to uint32")},
    "lm": {"train": ("lm_train", "Train a language model"),
           "sweep": ("lm_sweep", "Run a hyperparameter grid"),
           "evaluate": ("lm_evaluate", "Evaluate loss and perplexity"),
           "compare": ("lm_compare", "Compare completed runs"),
           "generate": ("lm_generate", "Generate text")},
    "model": {"report": ("model_report", "Write a Markdown architecture report")},
}
DOMAIN_HELP = {"tokenizer": "Tokenizer workflows", "lm": "Language-model workflows", "model": "Model inspection"}


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="ajllm-b200", description="Train tokenizers and Transformer language models")
    domains = parser.add_subparsers(dest="domain", required=True)
    for domain, commands in VERBS.items():
        sub = domains.add_parser(domain, help=DOMAIN_HELP[domain]).add_subparsers(dest="command", required=True)
        for command, (module, text) in commands.items():
            leaf = sub.add_parser(command, help=text)
            leaf.add_argument("--config", "-c", required=True, help="Path to a YAML configuration file")
            leaf.set_defaults(workflow_module=module)
    return parser


def resolve_workflow(module: str):
    return importlib.import_module(f"ajllm_b200.workflows.{module}").run


def main(argv: list[str] | None = None) -> None:
    parser = build_parser()
    arguments = parser.parse_args(argv)
    try:
        result: dict[str, Any] = resolve_workflow(arguments.workflow_module)(load_run_config(arguments.config))
    except (FileNotFoundError, KeyError, TypeError, ValueError) as error:
        parser.error(str(error))
    import torch.distributed as dist
    if not dist.is_initialized() or dist.get_rank() == 0:
        print(json.dumps(result, indent=2, ensure_ascii=False, default=str))
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
