import pytest
import torch

from ajllm_b200.engine import BlockAllocator, LLMEngine, OutOfBlocks, PagedKVCache, SamplingParams, Scheduler
from ajllm_b200.engine.quant import Fp8Weight, fp8_linear
from ajllm_b200.engine.spec_decode import verify_greedy, verify_rejection
from ajllm_b200.generation import generate, sample_next_token, sampling_probabilities
from ajllm_b200.models import build_model
from ajllm_b200.ops import reference

CFG = {"name": "e", "context_length": 128, "d_model": 64, "num_layers": 2, "num_heads": 4, "num_kv_heads": 2, "d_ff": 128}


@pytest.fixture(scope="module")
def models():
    torch.manual_seed(0)
    return build_model(CFG, 300), build_model({**CFG, "num_layers": 1}, 300)


def _prompts():
    gen = torch.Generator().manual_seed(5)
    return [torch.randint(0, 300, (n,), generator=gen).tolist() for n in (5, 17, 33, 9)]


def test_block_allocator_and_rollback():
    alloc = BlockAllocator(3)
    a, b, c = alloc.allocate(), alloc.allocate(), alloc.allocate()
    with pytest.raises(OutOfBlocks):
        alloc.allocate()
    alloc.share(a)
    alloc.release(a)
    assert alloc.free_blocks == 0
    alloc.release(a)
    assert alloc.free_blocks == 1
    cache = PagedKVCache(1, 8, 4, 1, 8, torch.float32, torch.device("cpu"))
    slots = cache.append_slots(7, 10)
    assert len(slots) == 10 and len(cache.tables[7].blocks) == 3
    cache.truncate(7, 5)
    assert cache.length(7) == 5 and len(cache.tables[7].blocks) == 2 and cache.allocator.free_blocks == 6
    cache.fork(7, 8)
    assert cache.allocator.ref_count(cache.tables[7].blocks[0]) == 2
    cache.free(7); cache.free(8)
    assert cache.allocator.free_blocks == 8


def test_paged_attention_matches_contiguous_attention():
    torch.manual_seed(1)
    cache = PagedKVCache(1, 16, 4, 2, 8, torch.float32, torch.device("cpu"))
    lens = [9, 4, 13]
    ks, vs = [torch.randn(n, 2, 8) for n in lens], [torch.randn(n, 2, 8) for n in lens]
    for sid, (k, v) in enumerate(zip(ks, vs)):
        cache.write(0, torch.tensor(cache.append_slots(sid, k.shape[0])), k, v)
    q = torch.randn(3, 2, 4, 8)     # two query rows per sequence (verify-style)
    out = reference.paged_attention(q, cache.keys[0], cache.values[0], cache.block_table_tensor([0, 1, 2], torch.device("cpu")),
                                    torch.tensor(lens))
    for i in range(3):
        want = reference.attention(q[i:i + 1], ks[i][None], vs[i][None], causal=True)
        assert torch.allclose(out[i:i + 1], want, atol=1e-5)


@pytest.mark.needs_reference
def test_sampling_and_greedy_generation_match_the_reference(reference_path):
    from ajllm.generation.generator import generate as ref_generate
    from ajllm.generation.sampling import sample_next_token as ref_sample
    from ajllm.modeling.factory import build_model as ref_build

    cfg = {k: v for k, v in CFG.items() if k != "num_kv_heads"}
    torch.manual_seed(0)
    ref, ours = ref_build(cfg, 300), build_model(cfg, 300)
    ours.load_state_dict(ref.state_dict())
    prompt = torch.randint(0, 300, (7,))
    assert ref_generate(ref, prompt, 20, 0.0, None, None).tolist() == generate(ours, prompt, 20, 0.0, None, None).tolist()
    logits = torch.randn(3, 50)
    for top_p in (None, 0.3, 0.9):
        torch.manual_seed(11); a = ref_sample(logits, 0.7, top_p)
        torch.manual_seed(11); b = sample_next_token(logits, 0.7, top_p)
        assert torch.equal(a, b)


def test_top_p_keeps_the_token_that_crosses_the_threshold():
    probs = sampling_probabilities(torch.log(torch.tensor([[0.5, 0.3, 0.15, 0.05]])), 1.0, 0.6)
    assert torch.allclose(probs, torch.tensor([[0.625, 0.375, 0.0, 0.0]]), atol=1e-6)
    with pytest.raises(ValueError):
        sampling_probabilities(torch.zeros(1, 4), 1.0, 0.0)


def test_continuous_batching_equals_one_at_a_time(models):
    target, _ = models
    prompts = _prompts()
    batched = LLMEngine(target, num_blocks=64, max_num_seqs=3, max_batched_tokens=24).generate(prompts, SamplingParams(20, 0.0, None))
    single = [generate(target, torch.tensor(p), 20, 0.0).tolist()[len(p):] for p in prompts]
    assert [o.output for o in batched] == single
    assert all(o.finish_reason == "length" for o in batched)


def test_preemption_by_recompute_preserves_outputs(models):
    target, _ = models
    prompts = _prompts()
    roomy = LLMEngine(target, num_blocks=64, max_num_seqs=4).generate(prompts, SamplingParams(20, 0.0, None))
    tight_engine = LLMEngine(target, num_blocks=8, max_num_seqs=4, max_batched_tokens=64)
    tight = tight_engine.generate(prompts, SamplingParams(20, 0.0, None))
    assert tight_engine.stats.preemptions > 0
    assert [o.output for o in tight] == [o.output for o in roomy]
    assert tight_engine.cache.allocator.free_blocks == 8


def test_eos_stops_a_sequence(models):
    target, _ = models
    prompt = _prompts()[0]
    free_run = LLMEngine(target, num_blocks=32).generate([prompt], SamplingParams(10, 0.0, None))[0].output
    stopped = LLMEngine(target, num_blocks=32).generate([prompt], SamplingParams(10, 0.0, None, eos_token_id=free_run[3]))[0]
    assert stopped.finish_reason == "eos" and stopped.output == free_run[:free_run.index(free_run[3]) + 1]


def test_speculative_greedy_is_lossless_and_self_draft_accepts_everything(models):
    target, draft = models
    prompts = _prompts()
    plain = LLMEngine(target, num_blocks=64).generate(prompts, SamplingParams(20, 0.0, None))
    spec_engine = LLMEngine(target, num_blocks=64, draft_model=draft, num_speculative_tokens=4)
    assert [o.output for o in spec_engine.generate(prompts, SamplingParams(20, 0.0, None))] == [o.output for o in plain]
    self_engine = LLMEngine(target, num_blocks=64, draft_model=target, num_speculative_tokens=3)
    outs = self_engine.generate(prompts, SamplingParams(12, 0.0, None))
    assert [o.output for o in outs] == [o.output[:12] for o in plain]
    assert self_engine.stats.acceptance_rate == 1.0 and self_engine.stats.steps < 12
    assert self_engine.cache.allocator.free_blocks == 64 and self_engine.draft_cache.allocator.free_blocks == 64


def test_speculative_decoding_runs_into_the_context_limit_like_the_plain_engine(models):
    target, draft = models
    gen = torch.Generator().manual_seed(9)
    prompts = [torch.randint(0, 300, (n,), generator=gen).tolist() for n in (100, 90)]
    params = SamplingParams(100, 0.0, None)
    plain = LLMEngine(target, num_blocks=64).generate(prompts, params)
    spec = LLMEngine(target, num_blocks=64, draft_model=draft, num_speculative_tokens=4).generate(prompts, params)
    assert [o.finish_reason for o in plain] == ["context", "context"]
    assert [o.finish_reason for o in spec] == ["context", "context"]
    assert [o.output for o in spec] == [o.output for o in plain]


def test_rejection_sampling_preserves_the_target_distribution():
    torch.manual_seed(0)
    gen = torch.Generator().manual_seed(0)
    p = torch.tensor([0.5, 0.2, 0.2, 0.1])
    q = torch.tensor([0.1, 0.6, 0.2, 0.1])
    counts = torch.zeros(4)
    trials = 20000
    for _ in range(trials):
        d = torch.multinomial(q, 1, generator=gen)
        accepted, nxt = verify_rejection(d, q[None], torch.stack([p, p]), gen)
        counts[int(d) if accepted == 1 else nxt] += 1      # first emitted token
    assert torch.allclose(counts / trials, p, atol=0.015)
    assert verify_greedy(torch.tensor([3, 1, 2]), torch.eye(5)[[3, 1, 4, 0]]) == (2, 4)


def test_fp8_block_quantisation_error_is_small():
    torch.manual_seed(0)
    w, x = torch.randn(200, 300) * 0.05, torch.randn(7, 300)
    q = Fp8Weight.from_dense(w)
    assert q.q.dtype == torch.float8_e4m3fn and q.scale.shape == (2, 3)
    assert (q.dequantize() - w).abs().max() / w.abs().max() < 0.07
    y = fp8_linear(x, q)
    assert (y - x @ w.t()).norm() / (x @ w.t()).norm() < 0.06


def test_scheduler_rejects_impossible_requests(models):
    target, _ = models
    cache = PagedKVCache(1, 2, 4, 1, 8, torch.float32, torch.device("cpu"))
    sched = Scheduler(cache, max_num_seqs=2, max_batched_tokens=64, context_length=128)
    with pytest.raises(ValueError):
        sched.add([], SamplingParams())
    sched.add(list(range(30)), SamplingParams())
    assert sched.schedule() == []          # the prompt can never fit in two blocks of four tokens


def test_decode_staging_mirrors_the_block_tables_under_churn():
    """The persistent host arrays of a replayed decoding step against the cache's own tables while sequences come,
    go, change rows and are rolled back (rejected draft tokens give blocks back and take other ones later)."""
    import random

    from ajllm_b200.engine.kv_cache import PagedKVCache
    from ajllm_b200.engine.model_runner import DecodeStaging, RunItem

    random.seed(0)
    for q_len in (1, 5):
        cache = PagedKVCache(1, 400, 16, 1, 8, torch.float32, torch.device("cpu"))
        scratch = cache.allocator.allocate()
        st = DecodeStaging(8, q_len, 16, scratch, 16, pinned=False)
        live = {}
        nxt = 0
        for step in range(300):
            # random churn: add / remove / rollback sequences
            while len(live) < 8 and random.random() < 0.5:
                cache.append_slots(nxt, random.randint(1, 40)); live[nxt] = True; nxt += 1
            for s in list(live):
                r = random.random()
                if r < 0.05 or cache.length(s) + q_len > 250:
                    cache.free(s); del live[s]
                elif r < 0.3 and q_len > 1:
                    cache.truncate(s, max(1, cache.length(s) - random.randint(0, q_len - 1)))
            ids = list(live)
            random.shuffle(ids)
            ids = ids[:random.randint(0, len(ids))]
            if not ids: continue
            items = [RunItem(s, [random.randint(0, 99) for _ in range(q_len)], q_len) for s in ids]
            before = {s: cache.length(s) for s in ids}
            st.fill(items, cache)
            rows, meta = st.rows.numpy(), st.meta.numpy()
            ctx, tables = meta[:8], meta[8:].reshape(8, 16)
            for i, it in enumerate(items):
                lo = i * q_len
                assert list(rows[0, lo:lo+q_len]) == it.token_ids
                assert list(rows[1, lo:lo+q_len]) == list(range(before[it.seq_id], before[it.seq_id] + q_len))
                blocks = cache.tables[it.seq_id].blocks
                assert list(tables[i, :len(blocks)]) == blocks, (step, i)
                for j, p in enumerate(range(before[it.seq_id], before[it.seq_id] + q_len)):
                    assert rows[2, lo + j] == blocks[p // 16] * 16 + p % 16
                assert ctx[i] == before[it.seq_id] + q_len
            for i in range(len(items), 8):
                lo = i * q_len
                assert ctx[i] == q_len and tables[i, 0] == scratch
                assert list(rows[2, lo:lo+q_len]) == [scratch * 16 + r for r in range(q_len)]
                assert list(rows[1, lo:lo+q_len]) == list(range(q_len))


def test_token_slice_equals_slicing_the_joined_tokens():
    from ajllm_b200.engine.scheduler import SamplingParams, Sequence

    seq = Sequence(0, list(range(10)), SamplingParams())
    seq.output.extend(range(100, 107))
    joined = seq.tokens
    for start in range(0, 19):
        for stop in range(start, 19):
            assert seq.token_slice(start, stop) == joined[start:stop], (start, stop)
    other = Sequence(0, list(range(10)), SamplingParams())
    assert seq != other and seq == seq and len({seq, other}) == 2      # identity, not field-wise comparison


def test_warm_up_is_a_no_op_without_graphs():
    import torch

    from ajllm_b200.engine import LLMEngine, SamplingParams
    from ajllm_b200.models import build_model

    torch.manual_seed(0)
    model = build_model({**CFG, "num_layers": 1}, 300)
    engine = LLMEngine(model, block_size=16, max_num_seqs=4)
    assert engine.warm_up() == 0
    out = engine.generate([[1, 2, 3]], SamplingParams(4, 0.0, None, None))
    assert len(out[0].output) == 4


def test_sampling_state_is_reused_while_the_batch_keeps_its_composition():
    """Seeds and draw counters of the device sampler: rebuilt when the batch changes, advanced in place otherwise, and
    always equal to what the per-request bookkeeping on the host says."""
    import torch

    from ajllm_b200.engine import LLMEngine, SamplingParams
    from ajllm_b200.models import build_model

    torch.manual_seed(0)
    engine = LLMEngine(build_model({**CFG, "num_layers": 1}, 300), block_size=16, max_num_seqs=4)
    for seed in (11, 12, 13):
        engine.add_request([1, 2, 3], SamplingParams(4, 0.7, 0.9, None, seed=seed))
    seqs = list(engine.scheduler.waiting)
    cpu = torch.device("cpu")
    temps, top_ps, seeds, counters = engine._device_sampling_state(seqs, cpu, draws=1)
    assert seeds.tolist() == [11, 12, 13] and counters.tolist() == [0, 0, 0] and top_ps.tolist() == pytest.approx([0.9] * 3)
    again = engine._device_sampling_state(seqs, cpu, draws=1)
    assert again[3] is counters and counters.tolist() == [1, 1, 1]             # same tensors, advanced in place
    _, _, _, wide = engine._device_sampling_state(seqs, cpu, draws=9)           # another draw width: rebuilt from the host
    assert wide.tolist() == [2, 2, 2]
    _, _, seeds2, fewer = engine._device_sampling_state(seqs[1:], cpu, draws=1)  # another composition: rebuilt
    assert seeds2.tolist() == [12, 13] and fewer.tolist() == [11, 11]
    assert [engine._draws[s.request_id] for s in seqs] == [11, 12, 12]
