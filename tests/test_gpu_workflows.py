"""The user-facing workflows on a GPU: the default (no ``mixed_precision`` key) debug configuration must train,
evaluate and generate on this package's kernels, not on eager PyTorch."""

import json
from pathlib import Path

import pytest
import torch

from tests.helpers import loaded, make_project, prepare_artifacts, train_config

pytestmark = pytest.mark.gpu

# the shape of configs/models/transformer_tiny.yaml: 4 heads of 16, 2 KV heads, a 290-entry vocabulary
TINY = {"name": "transformer_tiny", "context_length": 32, "d_model": 64, "num_layers": 2, "num_heads": 4, "num_kv_heads": 2,
        "d_ff": 128, "position_encoding": {"type": "rope", "theta": 10000},
        "normalization": {"type": "rmsnorm", "placement": "pre"}, "feed_forward": {"type": "swiglu"}}


@pytest.fixture(scope="module")
def project(tmp_path_factory):
    root = make_project(tmp_path_factory.mktemp("gpu_project"))
    prepare_artifacts(root)
    return root


def test_default_debug_training_runs_on_the_kernels_and_serves(project):
    from ajllm_b200.ops import native
    from ajllm_b200.workflows import lm_evaluate, lm_generate, lm_train

    config = train_config(project, max_steps=3)
    config["model"] = dict(TINY)
    config["runtime"] = {"device": "cuda", "seed": 3}
    before = native.launch_count
    result = lm_train.run(loaded(project, config))
    assert native.launch_count - before > 50, "training on a GPU must go through the native kernels"
    assert result["status"] == "completed" and result["compute_dtype"] == "bfloat16"
    run_dir = Path(result["run_directory"])
    manifest = json.loads((run_dir / "manifest.json").read_text())
    assert manifest["compute_dtype"] == "bfloat16" and manifest["tp_backend"] == "none"
    events = [json.loads(line) for line in (run_dir / "metrics.jsonl").read_text().splitlines()]
    losses = [e["loss"] for e in events if e["event"] == "train"]
    assert all(v == v for v in losses) and losses[-1] < losses[0] + 0.5
    before = native.launch_count
    ev = lm_evaluate.run(loaded(project, {"name": "e", "run_directory": str(run_dir), "checkpoint": "final",
                                          "batches": 2, "batch_size": 2, "device": "cuda"}))
    gen = lm_generate.run(loaded(project, {"name": "g", "run_directory": str(run_dir), "checkpoint": "best",
                                           "prompts": ["The night train"], "max_new_tokens": 5, "temperature": 0.0,
                                           "device": "cuda"}))
    assert native.launch_count - before > 20
    assert ev["loss"] == ev["loss"] and len(gen["results"][0]["completions"]) == 1
    assert native.check_status() == 0


def test_an_fp32_cuda_tensor_is_refused_unless_eager_math_is_requested():
    from ajllm_b200 import ops

    x = torch.randn(4, 64, device="cuda")
    w = torch.randn(16, 64, device="cuda")
    with pytest.raises(TypeError, match="bfloat16"):
        ops.linear(x, w)
    with ops.eager_cuda():
        assert ops.linear(x, w).shape == (4, 16)
