"""Sampler rules, rollout generator, scheduler (stop strings, token queue, enforcer hook, out-of-memory retry, runaway
guards), batch generator and state cache on a tiny CPU model."""
import pytest
import torch

from rwkvtune_b200.data.tokenizers import RWKVTokenizer, get_vocab_path
from rwkvtune_b200.inference import (BatchGenerator, GenerationConfig, GRPOBatchGenerator, SchedulerCore, SequenceState,
                                     TokenSampler, create_state_cache)
from rwkvtune_b200.models import RWKVConfig, RWKV7Model


@pytest.fixture(scope="module")
def model():
    torch.manual_seed(0)
    m = RWKV7Model(RWKVConfig(n_layer=2, n_embd=64, vocab_size=256, eos_token_id=7))
    with torch.no_grad():
        for n, p in m.named_parameters():
            if n.endswith(("output.weight", "ffn.value.weight")):
                p.normal_(0, 0.05)
    return m.eval()


class _Tok:
    eos_token_id = 7
    vocab_size = 250
    idx2token = {i: bytes([65 + i % 26]) for i in range(1, 250)}

    def decode(self, ids, **kw):
        return "".join(chr(65 + int(i) % 26) for i in ids)

    def encode(self, s):
        return [ord(c) - 64 for c in s]


def test_top_p_rule_keeps_prefix_and_bans_oov():
    logits = torch.log(torch.tensor([[0.5, 0.3, 0.15, 0.05, 0.0001]]))
    f = TokenSampler.filter_logits(logits, 1.0, 0.8, 0, max_valid_token_id=3)
    assert torch.isfinite(f[0, :2]).all() and torch.isinf(f[0, 2:]).all()
    f = TokenSampler.filter_logits(logits, 1.0, 0.3, 0)      # top token alone exceeds p: still kept
    assert torch.isfinite(f[0, 0]) and torch.isinf(f[0, 1:]).all()
    tok, lp = TokenSampler.sample_batch(logits.repeat(8, 1), temperature=0.0)
    assert (tok == 0).all()
    g = torch.Generator().manual_seed(1)
    tok, lp = TokenSampler.sample_batch(logits.repeat(4000, 1), 1.0, 0.8, generator=g)
    frac = (tok == 0).float().mean().item()
    assert set(tok.tolist()) <= {0, 1} and abs(frac - 0.625) < 0.03
    assert torch.allclose(lp[tok == 0], torch.log(torch.tensor(0.625)), atol=1e-4)


def test_grpo_generator_matches_stepwise_greedy(model):
    gen = GRPOBatchGenerator(model, _Tok(), sync_every=2)
    prompts = [[3, 4, 5, 6], [9, 8], [3, 4, 5, 6]]
    out = gen.generate(prompts, max_new_tokens=6, num_generations=2, temperature=0.0)
    assert out["completion_ids"].shape[0] == 6 and gen.last_stats["unique_prompts"] == 2
    ref = model.generate(torch.tensor([[3, 4, 5, 6]]), max_new_tokens=6, do_sample=False, eos_token_id=7)[0, 4:]
    ids, mask = out["completion_ids"][0], out["masks"][0]
    n = int(mask.sum())
    assert torch.equal(ids[:n], ref[:n])
    assert torch.equal(out["completion_ids"][0], out["completion_ids"][1])      # greedy paths agree
    assert torch.equal(out["completion_ids"][0], out["completion_ids"][4])      # duplicated prompt
    assert (out["completion_ids"][~out["masks"]] == 0).all()
    assert len(out["completions"]) == 6


def test_grpo_generator_sampling_stops_at_eos(model):
    gen = GRPOBatchGenerator(model, _Tok())
    out = gen.generate([[1, 2, 3]] * 2, max_new_tokens=40, num_generations=4, temperature=1.0, top_p=0.95,
                       repetition_penalty=1.1, seed=5)
    ids, masks = out["completion_ids"], out["masks"]
    for row, m in zip(ids, masks):
        n = int(m.sum())
        assert 1 <= n <= 40
        body = row[:n - 1]
        assert (body != 7).all()                   # EOS only ever as the last kept token
        assert row[:n].max() <= 249                # ids beyond the tokenizer are banned
    out2 = gen.generate([[1, 2, 3]] * 2, max_new_tokens=40, num_generations=4, temperature=1.0, top_p=0.95,
                        repetition_penalty=1.1, seed=5)
    assert torch.equal(out2["completion_ids"], ids)


def test_scheduler_equals_plain_generate(model):
    tok = _Tok()
    sched = SchedulerCore(model, tok, max_batch_size=2, max_batch_tokens=8, prefill_chunk_size=3)
    seqs = [SequenceState(i, p, max_new_tokens=5, temperature=0.0, eos_token_id=7)
            for i, p in enumerate([[3, 4, 5, 6, 7, 8, 9], [9, 8], [20, 21, 22]])]
    sched.add_sequences(seqs)
    for _ in sched.run_to_completion_sync():
        pass
    for s in seqs:
        ref = model.generate(torch.tensor([s.prompt_tokens]), max_new_tokens=5, do_sample=False, eos_token_id=7)
        assert s.generated_tokens == ref[0, len(s.prompt_tokens):].tolist()[:len(s.generated_tokens)]
        assert s.is_finished and s.finish_reason in ("eos", "length")
    assert sched.get_stats()["free_slots"] == 2


def test_state_cache_prefix_hit_gives_same_tokens(model):
    tok = _Tok()
    cache = create_state_cache(model, max_cache_memory_gb=0.01, max_cache_entries=2)
    sys_prompt = [3, 4, 5, 6, 10, 11]
    assert cache.create_checkpoints(sys_prompt + [20, 21], system_prompt_len=6) == 2
    pos, state, out = cache.lookup(sys_prompt + [30, 31, 32])
    assert pos == 6 and state is not None
    bg = BatchGenerator(model, tok, GenerationConfig(max_length=4, temperature=0.0), max_batch_size=2)
    bg.scheduler.state_cache = cache
    a = bg.generate(input_ids=[sys_prompt + [30, 31, 32]])["completion_ids"]
    bg.scheduler.state_cache = None
    b = bg.generate(input_ids=[sys_prompt + [30, 31, 32]])["completion_ids"]
    assert torch.equal(a, b)
    cache.create_checkpoints([40, 41, 42])
    assert cache.get_stats()["entries"] <= 2 and cache.get_stats()["evictions"] >= 1


def test_structured_output_masks_to_json():
    from rwkvtune_b200.inference import create_enforcer, is_structured_output_available
    if not is_structured_output_available():
        pytest.skip("lm-format-enforcer not installed")
    tok = RWKVTokenizer(get_vocab_path())
    enf = create_enforcer(tok, {"type": "json_schema", "json_schema": {"schema": {
        "type": "object", "properties": {"ok": {"type": "boolean"}}, "required": ["ok"]}}})
    text = ""
    for _ in range(40):
        logits = torch.zeros(65536)
        masked = enf.mask_logits(logits)
        if enf.is_finished():
            break
        allowed = torch.isfinite(masked).nonzero().flatten().tolist()
        pick = max(allowed, key=lambda t: len(tok.idx2token.get(t, b"")))
        text += tok.decode([pick])
        if enf.update(pick):
            break
    import json
    assert json.loads(text)["ok"] in (True, False)


def test_state_cache_checkpoints_from_messages(model):
    cache = create_state_cache(model, max_cache_memory_gb=0.01, max_cache_entries=4)
    tokens = list(range(3, 15))                         # 12 tokens
    messages = [{"role": "system", "content": "x" * 30}, {"role": "user", "content": "y" * 10}]
    assert cache.create_checkpoints(tokens, messages) == 2           # first message ~ 30/40 of the tokens
    pos, state, _ = cache.lookup(tokens[:9] + [99, 98])
    assert pos == 9 and state is not None
    assert cache.create_checkpoints(tokens, messages) == 0           # both prefixes already cached


def test_scheduler_retries_after_out_of_memory_and_stops_runaway_loops(model, monkeypatch):
    """An out-of-memory error inside a step is retried after the allocator cache is emptied; a loop that keeps
    scheduling without finishing anything ends with an error that carries the scheduler's counters."""
    tok = _Tok()
    sched = SchedulerCore(model, tok, max_batch_size=2, max_batch_tokens=16, prefill_chunk_size=8)
    seq = SequenceState(0, [3, 4, 5], max_new_tokens=3, temperature=0.0, eos_token_id=7)
    sched.add_sequences([seq])
    real = sched._execute_prefill
    failures = {"left": 2}

    def flaky(batch):
        if failures["left"] > 0:
            failures["left"] -= 1
            raise torch.cuda.OutOfMemoryError("synthetic")
        return real(batch)

    emptied = []
    monkeypatch.setattr(sched, "_execute_prefill", flaky)
    monkeypatch.setattr(torch.cuda, "empty_cache", lambda: emptied.append(1))
    monkeypatch.setattr("time.sleep", lambda s: None)
    for _ in sched.run_to_completion_sync():
        pass
    assert seq.is_finished and len(emptied) == 2 and failures["left"] == 0
    want = model.generate(torch.tensor([[3, 4, 5]]), max_new_tokens=3, do_sample=False, eos_token_id=7)[0, 3:].tolist()
    assert seq.generated_tokens == want[:len(seq.generated_tokens)]

    always = SchedulerCore(model, tok, max_batch_size=2, max_batch_tokens=16, prefill_chunk_size=8)
    always.add_sequences([SequenceState(1, [3, 4], max_new_tokens=2, temperature=0.0, eos_token_id=7)])
    monkeypatch.setattr(always, "_execute_prefill", lambda batch: (_ for _ in ()).throw(torch.cuda.OutOfMemoryError("again")))
    with pytest.raises(torch.cuda.OutOfMemoryError):
        always.step_sync()                                              # ten attempts, then the error is the caller's

    stuck = SchedulerCore(model, tok, max_batch_size=2, max_batch_tokens=16, prefill_chunk_size=8)
    stuck.add_sequences([SequenceState(2, [3, 4], max_new_tokens=2, temperature=0.0, eos_token_id=7)])
    monkeypatch.setattr(stuck, "step_sync", lambda: [])
    with pytest.raises(RuntimeError, match="exceeded 5 steps"):
        for _ in stuck.run_to_completion_sync(max_steps=5):
            pass
    with pytest.raises(RuntimeError, match="no progress for 3 steps"):
        for _ in stuck.run_to_completion_sync(stall_steps=3, stall_seconds=0.0):
            pass


def test_sampler_rules_one_by_one():
    """Greedy below the temperature threshold, bias clamping, the processor hook, top-k, seeds, the single-row form,
    rows that went non-finite, and the shape check."""
    TokenSampler.set_max_valid_token_id(None)
    logits = torch.tensor([[0.0, 1.0, 3.0, 2.0, -1.0]])
    tok, lp = TokenSampler.sample_batch(logits, temperature=0.0)
    assert tok.tolist() == [2] and float(lp) == pytest.approx(float(torch.log_softmax(logits, -1)[0, 2]))
    # a bias beyond +-100 is clamped: +1e9 on id 0 still loses to nothing, -1e9 on the arg-max removes it
    tok, _ = TokenSampler.sample_batch(logits, temperature=0.0, logit_bias={2: -1e9, "3": 0.5})
    assert tok.tolist() == [3]
    filtered = TokenSampler.filter_logits(logits, 1.0, 1.0, 0, logit_bias={0: 1e9, 99: 5.0})
    assert float(filtered[0, 0]) == 100.0 and filtered.shape == logits.shape             # clamped; id 99 is out of range
    # the processor sees the logits after temperature and bias and before top-k / top-p
    seen = {}

    def processor(x):
        seen["x"] = x.clone()
        x = x.clone()
        x[..., 2] = float("-inf")
        return x

    out = TokenSampler.filter_logits(logits, 0.5, 1.0, 2, logits_processor=processor)
    assert torch.allclose(seen["x"], logits / 0.5) and torch.isinf(out[0, 2])
    assert torch.isfinite(out[0]).sum() == 2 and torch.isfinite(out[0, [1, 3]]).all()    # top-2 of what the processor left
    # top-p keeps the sorted prefix whose mass stays within p, and always the most likely id
    sharp = torch.tensor([[10.0, 0.0, 0.0, 0.0]])
    assert torch.isfinite(TokenSampler.filter_logits(sharp, 1.0, 0.5, 0)[0]).tolist() == [True, False, False, False]
    # seeds and generators reproduce a draw
    flat = torch.zeros(3, 50)
    a, _ = TokenSampler.sample_batch(flat, seed=11)
    b, _ = TokenSampler.sample_batch(flat, seed=11)
    c, _ = TokenSampler.sample_batch(flat, generator=torch.Generator().manual_seed(11))
    assert a.tolist() == b.tolist() == c.tolist()
    tok, lp = TokenSampler.sample(torch.tensor([0.0, 5.0, 1.0]), temperature=0.0)
    assert (tok, lp) == (1, pytest.approx(float(torch.log_softmax(torch.tensor([0.0, 5.0, 1.0]), -1)[1])))
    # a row of NaNs falls back to a uniform draw instead of raising
    broken = torch.tensor([[float("nan")] * 4, [0.0, 1.0, 2.0, 3.0]])
    tok, _ = TokenSampler.sample_batch(broken, seed=0)
    assert 0 <= int(tok[0]) < 4 and 0 <= int(tok[1]) < 4
    with pytest.raises(ValueError):
        TokenSampler.sample_batch(torch.zeros(5))
    # ids above the tokenizer's range are never drawn
    TokenSampler.set_max_valid_token_id(2)
    try:
        draws, _ = TokenSampler.sample_batch(torch.zeros(200, 6), seed=1)
        assert int(draws.max()) <= 2
    finally:
        TokenSampler.set_max_valid_token_id(None)


def test_scheduler_stop_strings_token_queue_enforcer_and_fully_cached_prompts(model):
    import queue

    from rwkvtune_b200.inference import CacheConfig, CacheLevel, StateCache

    tok = _Tok()
    greedy = model.generate(torch.tensor([[3, 4, 5]]), max_new_tokens=6, do_sample=False, eos_token_id=999)[0, 3:].tolist()
    text = tok.decode(greedy)

    # a stop string ends the sequence as soon as the decoded text contains it; tokens also arrive on the queue
    q = queue.Queue()
    sched = SchedulerCore(model, tok, max_batch_size=2, max_batch_tokens=16, prefill_chunk_size=8)
    seq = SequenceState("s", [3, 4, 5], max_new_tokens=6, temperature=0.0, eos_token_id=999, stop=[text[1:3]], output_queue=q)
    sched.add_sequences([seq])
    for _ in sched.run_to_completion_sync():
        pass
    assert seq.finish_reason == "stop" and seq.generated_tokens == greedy[:3] and text[1:3] in seq.generated_text
    drained = []
    while not q.empty():
        drained.append(q.get())
    assert drained == greedy[:3] + [None]                                # the end marker follows the last token

    # an enforcer masks the logits, is told every token, and ends the sequence when it is satisfied
    class TwoTokens:
        def __init__(self):
            self.seen = []

        def mask_logits(self, logits):
            out = torch.full_like(logits, float("-inf"))
            out[..., 20 + len(self.seen)] = 0.0
            return out

        def update(self, token):
            self.seen.append(token)

        def is_finished(self):
            return len(self.seen) == 2

    enf = TwoTokens()
    sched2 = SchedulerCore(model, tok, max_batch_size=2, max_batch_tokens=16, prefill_chunk_size=8)
    forced = SequenceState(1, [3, 4, 5], max_new_tokens=6, temperature=1.0, eos_token_id=999, enforcer=enf)
    sched2.add_sequences([forced])
    for _ in sched2.run_to_completion_sync():
        pass
    assert forced.generated_tokens == [20, 21] == enf.seen and forced.finish_reason == "schema_complete"

    # a prompt that is in the cache to its last token needs no prefill at all: its stored logits seed the first draw
    cache = StateCache(model, CacheConfig(max_cache_memory_gb=0.01, cache_level=CacheLevel.EXACT), auto_config=False)
    cache.create_checkpoints([3, 4, 5])
    pos, state, output = cache.lookup([3, 4, 5])
    assert pos == 3 and state is not None and cache.lookup([3, 4])[0] == 0          # exact level: no prefix hits
    assert cache.get_stats()["exact_hits"] >= 1
    sched3 = SchedulerCore(model, tok, max_batch_size=2, max_batch_tokens=16, prefill_chunk_size=8, state_cache=cache)
    hit = SequenceState(2, [3, 4, 5], max_new_tokens=6, temperature=0.0, eos_token_id=999)
    sched3.add_sequences([hit])
    for _ in sched3.run_to_completion_sync():
        pass
    assert hit.cached_prefix_len == 3 and hit.generated_tokens == greedy
    off = StateCache(model, CacheConfig(max_cache_memory_gb=0.01, cache_level=CacheLevel.NONE), auto_config=False)
    assert off.lookup([3, 4, 5]) == (0, None, None) and off.get_stats()["total_misses"] == 1
    with pytest.raises(ValueError):
        CacheConfig(max_cache_memory_gb=0.0)
    with pytest.raises(ValueError):
        sched3.add_sequences([SequenceState(3, [], max_new_tokens=1)])


def test_batch_generator_token_inputs_eos_stripping_and_mode_restore(model, capsys):
    from rwkvtune_b200.inference import BatchGenerator, GenerationConfig

    class Tok(_Tok):
        pass

    tok = Tok()
    first = int(model.generate(torch.tensor([[3, 4, 5]]), max_new_tokens=1, do_sample=False)[0, -1])
    tok.eos_token_id = first                       # the very first greedy token ends the sequence
    gen = BatchGenerator(model, tok, max_batch_size=4, verbose=True)
    model.train()
    out = gen.generate(input_ids=[[3, 4, 5], [9, 8]], generation_config=GenerationConfig(max_length=4, temperature=0.0,
                                                                                        num_generations=2))
    assert model.training                                                  # the caller's mode is put back
    model.eval()
    assert out["completion_ids"].shape[0] == 4 and out["masks"].dtype == torch.float32
    assert out["masks"][0].sum() == 0 and out["completions"][0] == ""      # only an EOS was produced, and it is stripped
    assert out["masks"][0].tolist() == out["masks"][1].tolist()            # both generations of a prompt, prompt-major
    assert "eos 2" in capsys.readouterr().out
    with pytest.raises(ValueError):
        gen.generate()
