"""Launcher: ``python -m ajllm_b200.workflows.lm_train_distributed --config X --nproc-per-node N``
starts ``torchrun ... -m ajllm_b200 lm train --config X`` (reference:
``ajllm/workflows/lm_train_distributed.py:25-74``). The rendezvous address defaults to 127.0.0.1; the
child's exit code is passed through and Ctrl-C maps to 130."""

from __future__ import annotations

import argparse
import subprocess
import sys


def build_command(args: argparse.Namespace) -> list[str]:
    return [sys.executable, "-m", "torch.distributed.run", "--nproc-per-node", str(args.nproc_per_node),
            "--nnodes", str(args.nnodes), "--node-rank", str(args.node_rank), "--master-addr", args.master_addr,
            "--master-port", str(args.master_port), "--max-restarts", str(args.max_restarts),
            "-m", "ajllm_b200", "lm", "train", "--config", args.config]


def parse(argv: list[str] | None = None) -> argparse.Namespace:
    parser = argparse.ArgumentParser(description="Launch multi-GPU language-model training")
    parser.add_argument("--config", "-c", required=True)
    parser.add_argument("--nproc-per-node", type=int, default=2)
    parser.add_argument("--master-port", type=int, default=29500)
    parser.add_argument("--nnodes", type=int, default=1)
    parser.add_argument("--node-rank", type=int, default=0)
    parser.add_argument("--master-addr", default="127.0.0.1")
    parser.add_argument("--max-restarts", type=int, default=0,
                        help="torchrun restarts the worker group this many times; training resumes from "
                             "training.resume_from / the latest checkpoint")
    return parser.parse_args(argv)


def main(argv: list[str] | None = None) -> int:
    args = parse(argv)
    command = build_command(args)
    print("Launching:", " ".join(command), flush=True)
    try:
        return subprocess.run(command, check=False).returncode
    except KeyboardInterrupt:
        return 130


if __name__ == "__main__":
    sys.exit(main())
