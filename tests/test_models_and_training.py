import json
import math

import pytest
import torch

from ajllm_b200.models import build_model, count_parameters
from ajllm_b200.models.moe import capacity_for, route_tokens
from ajllm_b200.reporting import estimate_resources, write_model_report
from ajllm_b200.training import (AdamW, FlatAdamW, clip_gradients, cross_entropy, load_checkpoint, save_checkpoint,
                                 warmup_cosine_learning_rate)
from tests.helpers import TINY_MODEL

VARIANTS = [
    {},
    {"position_encoding": {"type": "none"}, "normalization": {"type": "none"}, "feed_forward": {"type": "silu"}},
    {"position_encoding": {"type": "learned"}, "normalization": {"type": "rmsnorm", "placement": "post"},
     "tie_embeddings": True},
    {"num_kv_heads": 1},
    {"moe": {"num_experts": 4, "top_k": 2, "shared_experts": 1, "d_ff": 32, "aux_loss_coef": 0.01}},
]


@pytest.mark.parametrize("override", VARIANTS)
def test_architecture_variants_produce_finite_logits_and_counts(override):
    config = {**TINY_MODEL, **override}
    model = build_model(config, 37)
    logits = model(torch.randint(0, 37, (3, 8)))
    assert logits.shape == (3, 8, 37) and torch.isfinite(logits).all()
    assert sum(p.numel() for p in model.parameters()) == count_parameters(config, 37)
    with pytest.raises(ValueError):
        model(torch.randint(0, 37, (1, config["context_length"] + 1)))
    loss = model.loss(torch.randint(0, 37, (2, 8)), torch.randint(0, 37, (2, 8)))
    loss.backward()
    assert all(p.grad is not None for p in model.parameters())


def test_state_dict_uses_reference_key_names_and_round_trips():
    model = build_model(TINY_MODEL, 40)
    keys = set(model.state_dict())
    for name in ("token_embeddings.weight", "layers.0.norm1.weight", "layers.0.attention.q_proj.weight",
                 "layers.0.attention.k_proj.weight", "layers.0.attention.v_proj.weight",
                 "layers.0.attention.output_proj.weight", "layers.1.feed_forward.w1.weight",
                 "layers.1.feed_forward.w2.weight", "layers.1.feed_forward.w3.weight", "final_norm.weight",
                 "lm_head.weight"):
        assert name in keys
    assert model.state_dict()["layers.0.attention.k_proj.weight"].shape == (16, 32)   # 2 KV heads x 8
    other = build_model(TINY_MODEL, 40)
    other.load_state_dict(model.state_dict())
    x = torch.randint(0, 40, (2, 8))
    assert torch.equal(model(x), other(x))


@pytest.mark.needs_reference
def test_logits_and_gradients_match_the_reference_model(reference_path):
    from ajllm.modeling.factory import build_model as ref_build
    from ajllm.training.losses import cross_entropy as ref_ce

    config = {k: v for k, v in TINY_MODEL.items() if k != "num_kv_heads"}
    for extra in ({}, {"tie_embeddings": True, "feed_forward": {"type": "silu"}}):
        cfg = {**config, **extra}
        ref, ours = ref_build(cfg, 50), build_model(cfg, 50)
        ours.load_state_dict(ref.state_dict())
        x, t = torch.randint(0, 50, (2, 9)), torch.randint(0, 50, (2, 9))
        assert torch.allclose(ours(x), ref(x), atol=1e-5)
        ours.loss(x, t).backward()
        ref_ce(ref(x), t).backward()
        got = ours.layers[0].attention.qkv_proj.grad[:32]
        assert torch.allclose(got, ref.layers[0].attention.q_proj.weight.grad, atol=1e-6)


def test_cross_entropy_schedule_and_clip():
    logits, targets = torch.randn(4, 5, 11), torch.randint(0, 11, (4, 5))
    assert torch.allclose(cross_entropy(logits, targets), torch.nn.functional.cross_entropy(logits.view(-1, 11), targets.view(-1)))
    assert warmup_cosine_learning_rate(0, 1.0, 0.1, 10, 100) == 0.0
    assert warmup_cosine_learning_rate(5, 1.0, 0.1, 10, 100) == pytest.approx(0.5)
    assert warmup_cosine_learning_rate(10, 1.0, 0.1, 10, 100) == pytest.approx(1.0)
    assert warmup_cosine_learning_rate(55, 1.0, 0.1, 10, 100) == pytest.approx(0.55)
    assert warmup_cosine_learning_rate(100, 1.0, 0.1, 10, 100) == pytest.approx(0.1)
    assert warmup_cosine_learning_rate(500, 1.0, 0.1, 10, 100) == pytest.approx(0.1)
    p = torch.nn.Parameter(torch.zeros(4))
    p.grad = torch.full((4,), 3.0)
    assert clip_gradients([p], 1.0) == pytest.approx(6.0)
    assert float(p.grad.norm()) == pytest.approx(1.0, rel=1e-4)


@pytest.mark.needs_reference
def test_flat_adamw_follows_the_reference_update(reference_path):
    from ajllm.training.optimizers import AdamW as RefAdamW

    torch.manual_seed(0)
    ours, ref = build_model(TINY_MODEL, 30), build_model(TINY_MODEL, 30)
    ref.load_state_dict(ours.state_dict())
    flat = FlatAdamW(ours, 1e-2, (0.9, 0.95), 1e-8, 0.1)
    plain = RefAdamW(ref.parameters(), 1e-2, (0.9, 0.95), 1e-8, 0.1)
    for _ in range(3):
        x, t = torch.randint(0, 30, (2, 8)), torch.randint(0, 30, (2, 8))
        flat.zero_grad(); ours.loss(x, t).backward(); flat.step(0.0)
        plain.zero_grad(); ref.loss(x, t).backward(); plain.step()
    for (_, a), (_, b) in zip(ours.state_dict().items(), ref.state_dict().items()):
        assert torch.allclose(a, b, atol=1e-6)
    state = flat.state_dict()
    assert set(state["state"][0]) == {"step", "first_moment", "second_moment"}
    assert state["param_names"][0] == "token_embeddings.weight"


def test_checkpoint_round_trip_restores_model_optimizer_and_step(tmp_path):
    model = build_model(TINY_MODEL, 30)
    opt = FlatAdamW(model, 1e-3)
    x, t = torch.randint(0, 30, (2, 8)), torch.randint(0, 30, (2, 8))
    opt.zero_grad(); model.loss(x, t).backward(); opt.step(1.0)
    path = save_checkpoint(tmp_path / "ck.pt", model, opt, 7, {"note": "x"}, aliases=("latest.pt",))
    assert (tmp_path / "latest.pt").is_file() and not list(tmp_path.glob("*.tmp"))
    raw = torch.load(path, weights_only=False)
    assert set(raw) >= {"model_state_dict", "optimizer_state_dict", "step", "metadata"} and raw["step"] == 7
    clone = build_model(TINY_MODEL, 30)
    clone_opt = FlatAdamW(clone, 1e-3)
    loaded = load_checkpoint(path, clone, clone_opt)
    assert loaded["step"] == 7 and clone_opt.step_count == 1
    assert torch.equal(clone_opt.m, opt.m) and torch.equal(clone_opt.v, opt.v)
    assert all(torch.equal(a, b) for a, b in zip(model.state_dict().values(), clone.state_dict().values()))
    (tmp_path / "broken.pt").write_bytes(path.read_bytes()[:100])
    with pytest.raises(RuntimeError, match="unreadable"):
        load_checkpoint(tmp_path / "broken.pt", clone)


def test_per_tensor_adamw_keeps_reference_state_names():
    p = torch.nn.Parameter(torch.ones(3))
    opt = AdamW([p], 0.1, (0.9, 0.999), 1e-8, 0.1)
    p.grad = torch.ones(3)
    opt.step()
    assert set(opt.state[p]) == {"step", "first_moment", "second_moment"}
    assert torch.allclose(p, torch.full((3,), (1 - 0.1) * (1 - 0.01)), atol=1e-6)


def test_moe_routing_capacity_and_aux_terms():
    torch.manual_seed(0)
    logits = torch.randn(64, 8)
    cap = capacity_for(64, 2, 8, 1.0)
    gates, experts, slots, (fraction, mean_prob, kept_counts) = route_tokens(logits, 2, cap)
    assert torch.allclose(gates.sum(-1), torch.ones(64))
    assert fraction.sum() == pytest.approx(1.0) and mean_prob.sum() == pytest.approx(1.0, rel=1e-5)
    kept = slots[slots >= 0]
    assert kept.unique().numel() == kept.numel()                        # one assignment per slot
    for e in range(8):
        mine = (experts == e)
        assert int((slots[mine] >= 0).sum()) == min(int(mine.sum()), cap)  # overflow is dropped, in order
        assert ((slots[mine][slots[mine] >= 0] // cap) == e).all()
    # earlier (token, choice) pairs win the capacity race
    flat_e, flat_s = experts.reshape(-1), slots.reshape(-1)
    for e in range(8):
        order = flat_s[flat_e == e]
        dropped = (order < 0).nonzero()
        if dropped.numel():
            assert (order[int(dropped[0]):] < 0).all()


def test_resource_estimate_and_report_sections(tmp_path):
    config = {**TINY_MODEL, "num_kv_heads": 4}
    model = build_model(config, 40)
    n = sum(p.numel() for p in model.parameters())
    est = estimate_resources({**config, "vocab_size": 40}, n, 4, {"max_steps": 10})
    assert est.optimizer_bytes == n * 8
    assert est.total_memory_bytes == est.parameter_bytes + est.activation_bytes + est.gradient_bytes + est.optimizer_bytes
    assert est.total_training_flops == est.training_flops_per_step * 10 and est.forward_flops_per_step > 0
    tokens, d, f, layers = 4 * 16, 32, 64, 2
    expected = layers * (8 * tokens * d * d + 4 * 4 * 16 * 16 * d + 3 * 2 * tokens * d * f) + 2 * tokens * d * 40
    assert est.forward_flops_per_step == expected
    report = write_model_report(tmp_path / "m.md", model, config, 40, 4, {"max_steps": 10}).read_text()
    for needle in ("Estimated Training Memory", "Estimated Matrix FLOPs", "AdamW first and second moments",
                   "Total training FLOPs", "layers.0.attention.q_proj.weight"):
        assert needle in report
