import json

import pytest
import torch
import yaml

from ajllm_b200.cli import build_parser
from ajllm_b200.workflows import lm_compare, lm_evaluate, lm_generate, lm_sweep, lm_train, model_report
from ajllm_b200.workflows.lm_train_distributed import build_command, parse
from tests.helpers import base_run, loaded, make_project, prepare_artifacts, train_config


@pytest.fixture(scope="module")
def project(tmp_path_factory):
    root = make_project(tmp_path_factory.mktemp("project"))
    prepare_artifacts(root)
    return root


def test_tokenizer_artifacts_are_registered(project):
    tok = json.loads((project / "artifacts/tokenizers/toy_bpe/manifest.json").read_text())
    enc = json.loads((project / "artifacts/encoded/toy/toy_bpe/manifest.json").read_text())
    assert tok["artifact_type"] == "tokenizer" and tok["vocab_size"] == 290 and "fingerprint" in tok
    assert enc["dtype"] == "uint32" and enc["tokenizer_fingerprint"] == tok["fingerprint"]
    for split in ("train", "validation"):
        entry = enc["splits"][split]
        assert (project / "artifacts/encoded/toy/toy_bpe" / entry["path"]).stat().st_size == 4 * entry["token_count"]


def test_train_then_resume_then_generate_with_best(project):
    first = lm_train.run(loaded(project, train_config(project, max_steps=1)))
    run_dir = project / first["run_directory"] if not first["run_directory"].startswith("/") else None
    from pathlib import Path
    run_dir = Path(first["run_directory"])
    names = {p.name for p in (run_dir / "checkpoints").iterdir()}
    assert {"final.pt", "latest.pt", "best.pt", "step_00000001.pt"} <= names
    for name in ("resolved_config.yaml", "manifest.json", "metrics.jsonl", "summary.json", "model_report.md"):
        assert (run_dir / name).is_file()
    events = [json.loads(line) for line in (run_dir / "metrics.jsonl").read_text().splitlines()]
    assert {"train", "evaluation"} <= {e["event"] for e in events}
    train_event = next(e for e in events if e["event"] == "train")
    assert {"loss", "learning_rate", "gradient_norm", "tokens_per_second"} <= set(train_event)
    resumed = lm_train.run(loaded(project, train_config(project, max_steps=2,
                                                       resume_from=str(run_dir / "checkpoints" / "final.pt"))))
    assert resumed["steps"] == 2 and resumed["status"] == "completed"
    ckpt = torch.load(Path(resumed["run_directory"]) / "checkpoints" / "final.pt", weights_only=False)
    assert ckpt["step"] == 2 and ckpt["optimizer_state_dict"]["state"][0]["step"] == 2

    gen = lm_generate.run(loaded(project, {"name": "g", "run_directory": str(run_dir), "checkpoint": "best",
                                           "prompts": ["The night train", "A small robot"], "max_new_tokens": 5,
                                           "temperature": 0.0, "samples_per_prompt": 2, "device": "cpu"}))
    assert len(gen["results"]) == 2 and len(gen["results"][0]["completions"]) == 2
    a, b = gen["results"][0]["completions"]
    assert a["text"] == b["text"] and a["text"].startswith("The night train")      # greedy is deterministic
    ev = lm_evaluate.run(loaded(project, {"name": "e", "run_directory": str(run_dir), "checkpoint": "final",
                                          "batches": 2, "batch_size": 2, "device": "cpu"}))
    assert ev["perplexity"] == pytest.approx(pytest.importorskip("math").exp(ev["loss"]))


def test_sweep_compare_and_report(project):
    cfg = train_config(project, max_steps=1)
    cfg.update({"name": "lr", "grid": {"optimizer.max_lr": [1e-3, 3e-3]}, "comparison": {"generate_plot": True}})
    sweep = lm_sweep.run(loaded(project, cfg))
    assert len(sweep["trials"]) == 2 and sweep["best_run"] is not None
    out = sweep["output_dir"]
    from pathlib import Path
    assert (Path(out) / "comparison.csv").is_file() and (Path(out) / "trials.json").is_file()
    assert any(Path(out).glob("learning_curves.*"))
    runs = [t["run_directory"] for t in sweep["trials"]]
    cmp = lm_compare.run(loaded(project, {"name": "c", "runs": runs, "generate_plot": False}))
    losses = [r["validation_loss"] for r in cmp["results"]]
    assert losses == sorted(losses)
    rep = model_report.run(loaded(project, {"model": base_run(project)["model"], "report_vocab_size": 290}))
    assert Path(rep["output_path"]).is_file() and rep["parameter_count"] > 0


def test_sweep_records_failed_trials_when_asked(project):
    cfg = train_config(project, max_steps=1)
    cfg.update({"name": "bad", "grid": {"model.num_heads": [4, 5]}, "continue_on_error": True,
                "comparison": {"generate_plot": False}})
    sweep = lm_sweep.run(loaded(project, cfg))
    assert [t.get("status") for t in sweep["trials"]].count("failed") == 1


def test_training_refuses_a_mismatched_tokenizer(project):
    manifest_path = project / "artifacts/encoded/toy/toy_bpe/manifest.json"
    original = manifest_path.read_text()
    data = json.loads(original)
    data["tokenizer_fingerprint"] = "0" * 64
    manifest_path.write_text(json.dumps(data))
    try:
        with pytest.raises(ValueError, match="different tokenizer"):
            lm_train.run(loaded(project, train_config(project, max_steps=1)))
    finally:
        manifest_path.write_text(original)


def test_cli_accepts_every_verb_and_launcher_builds_torchrun():
    parser = build_parser()
    for argv in (["tokenizer", "train"], ["tokenizer", "encode"], ["lm", "train"], ["lm", "sweep"], ["lm", "evaluate"],
                 ["lm", "compare"], ["lm", "generate"], ["model", "report"]):
        assert parser.parse_args([*argv, "--config", "x.yaml"]).config == "x.yaml"
    command = build_command(parse(["--config", "c.yaml", "--nproc-per-node", "4"]))
    assert "torch.distributed.run" in command and command[-5:] == ["ajllm_b200", "lm", "train", "--config", "c.yaml"]
    assert command[command.index("--master-addr") + 1] == "127.0.0.1"


def test_acceleration_benchmark_writes_json_csv_and_figure(tmp_path):
    """The acceleration benchmark (reference: ajllm/workflows/benchmark_distributed.py) on CPU: every configuration
    and phase appears in the JSON / CSV, the sharded configurations run on two gloo ranks."""
    import csv
    import json

    from ajllm_b200.workflows import benchmark_distributed as bench
    from tests.conftest import free_port

    out = bench.main(["--device", "cpu", "--world-size", "2", "--vocab-size", "64", "--d-model", "32", "--num-layers", "2",
                      "--num-heads", "4", "--batch-size", "4", "--context-length", "16", "--steps", "2", "--warmup", "1",
                      "--master-port", str(free_port()), "--output-dir", str(tmp_path)])
    payload = json.loads((tmp_path / "benchmark_acceleration.json").read_text())
    assert {r["config"] for r in payload} == set(bench.CONFIGS)
    assert sum(1 for r in payload if r["config"] == "fsdp_ac") == 2           # one record per rank
    for record in payload:
        for phase in bench.PHASES:
            assert record[phase]["mean_ms"] >= 0.0
        assert record["tokens_per_second"] > 0
    rows = list(csv.DictReader((tmp_path / "benchmark_acceleration.csv").open()))
    assert len(rows) == len(payload) * len(bench.PHASES)
    assert (tmp_path / "benchmark_acceleration.png").exists() or (tmp_path / "benchmark_time.svg").exists()
    assert out["json"].endswith("benchmark_acceleration.json")


def _train_rank(rank, world, root, config):
    from pathlib import Path

    from ajllm_b200.workflows import lm_train as workflow

    out = workflow.run(loaded(Path(root), config))
    assert out["status"] == "completed" and out["steps"] == 2
    if rank == 0:
        run_dir = Path(out["run_directory"])
        ckpt = torch.load(run_dir / "checkpoints" / "final.pt", weights_only=False)
        # whole-model, un-prefixed keys whatever the parallel mode
        assert "token_embeddings.weight" in ckpt["model_state_dict"]
        assert any(k.startswith("layers.1.") for k in ckpt["model_state_dict"])
        events = [json.loads(line) for line in (run_dir / "metrics.jsonl").read_text().splitlines()]
        losses = [e["loss"] for e in events if e["event"] == "train"]
        assert len(losses) == 2 and all(2.0 < value < 8.0 for value in losses), losses


@pytest.mark.parametrize("mode", ["fsdp", "replicas", "pipeline", "tensor", "experts"])
def test_train_workflow_on_two_ranks(project, mode):
    """`lm train` end to end on two gloo ranks in each multi-rank mode: sharded, replicated, pipelined, tensor-parallel, expert-parallel."""
    from tests.conftest import run_ranks

    config = train_config(project, max_steps=2)
    config["model"] = {**config["model"], "tie_embeddings": False}
    config["experiment"] = f"two_ranks_{mode}"
    if mode == "fsdp":
        config["acceleration"] = {"use_fsdp": True}
    elif mode == "replicas":
        config["acceleration"] = {"use_fsdp": False}
        config["parallel"] = {"fsdp": 2}
    elif mode == "pipeline":
        config["acceleration"] = {"use_fsdp": False}
        config["parallel"] = {"pp": 2, "fsdp": 1, "pp_microbatches": 2}
    elif mode == "tensor":
        config["acceleration"] = {"use_fsdp": False}
        config["parallel"] = {"tp": 2, "fsdp": 1}
    else:
        config["model"] = {**config["model"], "d_ff": 32,
                           "moe": {"num_experts": 4, "top_k": 2, "shared_experts": 1, "d_ff": 32, "capacity_factor": 4.0}}
        config["acceleration"] = {"use_fsdp": True}
        config["parallel"] = {"fsdp": 2, "ep": 2}
    run_ranks(_train_rank, 2, str(project), config)


def _generate_tensor_parallel(rank, world, root, run_dir, want):
    from pathlib import Path

    out = lm_generate.run(loaded(Path(root), {"name": "g_tp", "run_directory": run_dir, "checkpoint": "final",
                                              "prompts": ["The night train", "A small robot"], "max_new_tokens": 6,
                                              "temperature": 0.0, "device": "cpu"}))
    assert out["tensor_parallel"] == {"size": 2, "backend": "nccl"}
    assert [r["completions"][0]["text"] for r in out["results"]] == want
    assert Path(out["output_dir"]).is_dir() == (rank == 0) or rank != 0


def test_generate_serves_tensor_parallel_over_two_ranks(project):
    from tests.conftest import run_ranks

    first = lm_train.run(loaded(project, train_config(project, max_steps=1)))
    single = lm_generate.run(loaded(project, {"name": "g_one", "run_directory": first["run_directory"], "checkpoint": "final",
                                              "prompts": ["The night train", "A small robot"], "max_new_tokens": 6,
                                              "temperature": 0.0, "device": "cpu"}))
    want = [r["completions"][0]["text"] for r in single["results"]]
    run_ranks(_generate_tensor_parallel, 2, str(project), first["run_directory"], want)
