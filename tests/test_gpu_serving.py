"""Serving path on a GPU: the paged-attention kernel against the CPU statement of the same op, and the
engine (continuous batching, speculative decoding) against itself run one request at a time."""

import pytest
import torch

from ajllm_b200.engine import LLMEngine, PagedKVCache, SamplingParams
from ajllm_b200.models import build_model
from ajllm_b200.ops import native, reference, serving

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda", 0)


@pytest.mark.parametrize("heads,kv_heads,hd,q_len,lens", [(8, 2, 128, 1, [1, 17, 130, 500]), (8, 2, 128, 5, [5, 40, 260]),
                                                          (4, 4, 64, 3, [3, 129]), (16, 2, 128, 11, [11, 300])])
def test_paged_attention_kernel_matches_reference(heads, kv_heads, hd, q_len, lens):
    torch.manual_seed(0)
    dev = _dev()
    cache = PagedKVCache(1, 128, 16, kv_heads, hd, torch.bfloat16, dev)
    for sid, n in enumerate(lens):
        slots = torch.tensor(cache.append_slots(sid, n), device=dev)
        cache.write(0, slots, torch.randn(n, kv_heads, hd, device=dev) * 0.5, torch.randn(n, kv_heads, hd, device=dev) * 0.5)
    q = (torch.randn(len(lens) * q_len, heads, hd, device=dev) * 0.5).to(torch.bfloat16)
    tables = cache.block_table_tensor(list(range(len(lens))), dev)
    got = serving.paged_attention(q, cache.keys[0], cache.values[0], tables, None, None, [q_len] * len(lens), lens)
    want = reference.paged_attention(q.float().cpu().view(len(lens), q_len, heads, hd), cache.keys[0].float().cpu(),
                                     cache.values[0].float().cpu(), tables.cpu(), torch.tensor(lens))
    err = (got.float().cpu().view_as(want) - want).norm() / want.norm()
    assert float(err) < 1.5e-2, float(err)
    assert native.lib().ajb_check_status() == 0


CFG = {"name": "s", "context_length": 512, "d_model": 512, "num_layers": 2, "num_heads": 4, "num_kv_heads": 2,
       "d_ff": 1408, "init": {"type": "normal", "std": 0.05}}


@pytest.fixture(scope="module")
def models():
    torch.manual_seed(0)
    target = build_model(CFG, 1024).to(device=_dev(), dtype=torch.bfloat16)
    draft = build_model({**CFG, "num_layers": 1}, 1024).to(device=_dev(), dtype=torch.bfloat16)
    return target, draft


def _prompts():
    gen = torch.Generator().manual_seed(3)
    return [torch.randint(0, 1024, (n,), generator=gen).tolist() for n in (5, 40, 130, 17, 64, 9)]


def test_engine_prefill_logits_match_training_forward(models):
    """The serving forward (paged cache, flash prompt attention) must agree with the training forward."""
    target, _ = models
    from ajllm_b200.engine.model_runner import ModelRunner, RunItem
    prompt = _prompts()[2]
    cache = PagedKVCache(target.num_layers, 64, 16, 2, 128, torch.bfloat16, _dev())
    runner = ModelRunner(target, cache)
    got = runner.forward([RunItem(0, prompt, len(prompt))])
    with torch.no_grad():
        want = target(torch.tensor([prompt], device=_dev()))[0].float()
    assert float((got - want).abs().max()) < 0.08 * float(want.abs().max())
    # decode one more token through the paged kernel and compare with a full re-forward
    nxt = int(got[-1].argmax())
    step = runner.forward([RunItem(0, [nxt], 1)])
    with torch.no_grad():
        full = target(torch.tensor([prompt + [nxt]], device=_dev()))[0, -1].float()
    assert float((step[0] - full).abs().max()) < 0.08 * float(full.abs().max())


def test_engine_serves_32_wide_heads_like_the_training_forward():
    """Head sizes the kernels do not exist for (the reference's flagship has 16 heads of 32) are cached zero-padded."""
    from ajllm_b200.engine.model_runner import RunItem
    torch.manual_seed(1)
    config = {**CFG, "num_heads": 16, "num_kv_heads": 16}
    model = build_model(config, 1024).to(device=_dev(), dtype=torch.bfloat16)
    engine = LLMEngine(model, num_blocks=64)
    assert engine.cache.head_dim == 64 and engine.runner.head_dim == 32
    prompt = _prompts()[2]
    got = engine.runner.forward([RunItem(0, prompt, len(prompt))])
    with torch.no_grad():
        want = model(torch.tensor([prompt], device=_dev()))[0].float()
    assert float((got - want).abs().max()) < 0.08 * float(want.abs().max())
    nxt = int(got[-1].argmax())
    step = engine.runner.forward([RunItem(0, [nxt], 1)])
    with torch.no_grad():
        full = model(torch.tensor([prompt + [nxt]], device=_dev()))[0, -1].float()
    assert float((step[0] - full).abs().max()) < 0.08 * float(full.abs().max())
    outs = LLMEngine(model, num_blocks=128).generate(_prompts()[:3], SamplingParams(12, 0.0, None))
    assert all(len(o.output) == 12 for o in outs)
    assert native.lib().ajb_check_status() == 0


def test_gpu_engine_batched_equals_sequential_and_speculative(models):
    target, draft = models
    prompts = _prompts()
    params = SamplingParams(24, 0.0, None)
    batched = LLMEngine(target, num_blocks=256, max_num_seqs=4, max_batched_tokens=160).generate(prompts, params)
    assert all(len(o.output) == 24 for o in batched)
    spec = LLMEngine(target, num_blocks=256, max_num_seqs=4, draft_model=target, num_speculative_tokens=3)
    outs = spec.generate(prompts, params)
    # a model drafting for itself accepts nearly everything; ties in bf16 logits may flip an argmax
    assert spec.stats.acceptance_rate > 0.9
    agree = sum(a.output == b.output for a, b in zip(batched, outs))
    assert agree >= len(prompts) - 1
    small = LLMEngine(target, num_blocks=256, draft_model=draft, num_speculative_tokens=4).generate(prompts[:3], params)
    assert all(len(o.output) == 24 for o in small)
    sampled = LLMEngine(target, num_blocks=256).generate(prompts[:3], SamplingParams(8, 0.9, 0.95))
    assert all(len(o.output) == 8 for o in sampled)
    assert native.lib().ajb_check_status() == 0


@pytest.mark.parametrize("m,n,k", [(7, 256, 512), (256, 4096, 4096), (130, 1000, 1408), (64, 14336, 4096)])
def test_fp8_block_scaled_gemm_matches_dequantised_reference(m, n, k):
    from ajllm_b200.engine.quant import Fp8Weight
    from ajllm_b200.ops import fp8

    torch.manual_seed(1)
    x = torch.randn(m, k, device=_dev(), dtype=torch.bfloat16)
    w = (torch.randn(n, k, device=_dev()) * 0.05).to(torch.bfloat16)
    weight = Fp8Weight.from_dense(w)
    xq, sx = fp8.quantize_rows(x)
    rq, rs = reference.quantize_activation_fp8_rows(x, 128)
    assert torch.allclose(sx, rs, rtol=1e-3) and float((xq.float() - rq.float()).abs().max()) <= 32.0
    got = fp8.fp8_block_gemm(x, weight)
    want = reference.fp8_block_linear(xq, sx, weight.q, weight.scale, 128)       # same quantised operands, fp32 math
    assert float((got.float() - want).norm() / want.norm()) < 6e-3
    exact = x.float() @ w.float().t()
    assert float((got.float() - exact).norm() / exact.norm()) < 6e-2               # quantisation error itself
    assert native.lib().ajb_check_status() == 0


def test_fp8_engine_generates(models):
    target, _ = models
    outs = LLMEngine(target, num_blocks=128, quantization="fp8").generate(_prompts()[:3], SamplingParams(8, 0.0, None))
    assert all(len(o.output) == 8 for o in outs)


def test_sampler_kernel_greedy_top_p_and_distribution():
    dev = _dev()
    torch.manual_seed(2)
    logits = torch.randn(4, 1000, device=dev)
    zeros = torch.zeros(4, device=dev)
    ones = torch.ones(4, device=dev)
    seeds = torch.arange(4, device=dev, dtype=torch.int64)
    greedy = serving.sample_rows(logits, zeros, ones, seeds, seeds)
    assert greedy.tolist() == logits.argmax(-1).tolist()
    # empirical distribution of one row over many draws, with and without top-p
    row = torch.log(torch.tensor([0.5, 0.3, 0.15, 0.05], device=dev)).repeat(20000, 1)
    n = row.shape[0]
    temps, seeds = torch.ones(n, device=dev), torch.full((n,), 7, device=dev, dtype=torch.int64)
    counters = torch.arange(n, device=dev, dtype=torch.int64)
    free = torch.bincount(serving.sample_rows(row, temps, torch.ones(n, device=dev), seeds, counters).long(), minlength=4) / n
    assert torch.allclose(free.cpu(), torch.tensor([0.5, 0.3, 0.15, 0.05]), atol=0.015)
    nucleus = torch.bincount(serving.sample_rows(row, temps, torch.full((n,), 0.6, device=dev), seeds, counters).long(),
                             minlength=4) / n
    assert torch.allclose(nucleus.cpu(), torch.tensor([0.625, 0.375, 0.0, 0.0]), atol=0.015)
    # same (seed, counter) -> same token
    again = serving.sample_rows(row[:64], temps[:64], torch.ones(64, device=dev), seeds[:64], counters[:64])
    first = serving.sample_rows(row[:64], temps[:64], torch.ones(64, device=dev), seeds[:64], counters[:64])
    assert torch.equal(again, first)


def test_spec_verify_kernel_preserves_target_distribution():
    dev = _dev()
    n, k, vocab = 20000, 1, 4
    p = torch.tensor([0.5, 0.2, 0.2, 0.1], device=dev)
    q = torch.tensor([0.1, 0.6, 0.2, 0.1], device=dev)
    gen = torch.Generator(device=dev).manual_seed(0)
    drafts = torch.multinomial(q.repeat(n, 1), 1, generator=gen).to(torch.int32)
    target = torch.log(p).repeat(n, k + 1, 1).contiguous()
    draft = torch.log(q).repeat(n, k, 1).contiguous()
    temps = torch.ones(n, device=dev)
    seeds = torch.full((n,), 11, device=dev, dtype=torch.int64)
    counters = torch.arange(n, device=dev, dtype=torch.int64) * 8
    verdict = serving.spec_verify(target, draft, drafts, temps, seeds, counters)
    first = torch.where(verdict[:, 0] == 1, drafts[:, 0], verdict[:, 1]).long()
    freq = torch.bincount(first, minlength=vocab) / n
    assert torch.allclose(freq.cpu(), p.cpu(), atol=0.015)
    # greedy: accept while the draft equals the target argmax
    tl = torch.eye(5, device=dev)[[3, 1, 4, 0]].unsqueeze(0).contiguous() * 5
    out = serving.spec_verify(tl, torch.zeros(1, 3, 5, device=dev), torch.tensor([[3, 1, 2]], dtype=torch.int32, device=dev),
                              torch.zeros(1, device=dev), seeds[:1], counters[:1])
    assert out.tolist() == [[2, 4]]
