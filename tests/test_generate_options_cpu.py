"""``generate()`` options (ban list, repetition penalty, several returns, carried states, EOS lists) and small
accessors of the adapter layer, the flat parameter space, the tokenizer output and the structured-output adapter."""
import pytest
import torch

from rwkvtune_b200.models import RWKVConfig, RWKV7Model


@pytest.fixture(scope="module")
def model():
    torch.manual_seed(0)
    m = RWKV7Model(RWKVConfig(n_layer=2, n_embd=64, vocab_size=64, dim_att_lora=16, dim_gate_lora=16, dim_mv_lora=16))
    with torch.no_grad():
        for n, p in m.named_parameters():
            if n.endswith(("output.weight", "ffn.value.weight")):
                p.normal_(0, 0.1)
    return m.eval()


def test_greedy_generate_equals_stepwise_argmax_and_respects_the_ban_list(model):
    prompt = torch.tensor([[3, 9, 4]])
    out = model.generate(prompt, max_new_tokens=6, do_sample=False)
    assert out.shape == (1, 9) and torch.equal(out[:, :3], prompt)
    with torch.no_grad():
        logits, st = model.forward_with_state(prompt)
        expect = []
        for _ in range(6):
            tok = int(logits[0, -1].argmax())
            expect.append(tok)
            logits, st = model.forward_with_state(torch.tensor([[tok]]), st)
    assert out[0, 3:].tolist() == expect
    banned = model.generate(prompt, max_new_tokens=6, do_sample=False, token_ban=expect[:1])
    assert expect[0] not in banned[0, 3:].tolist()
    # one-dimensional input and max_length are accepted
    assert model.generate(prompt[0], max_length=5, do_sample=False).shape == (1, 5)
    with pytest.raises(ValueError):
        model.generate()


def test_repetition_penalty_changes_the_greedy_path_only_through_seen_tokens(model):
    from rwkvtune_b200.models.generation_mixin import apply_repetition_penalty_

    logits = torch.tensor([[2.0, -2.0, 1.0, -1.0]])
    seen = torch.tensor([[True, True, False, False]])
    apply_repetition_penalty_(logits, seen, 2.0)
    assert logits.tolist() == [[1.0, -4.0, 1.0, -1.0]]
    apply_repetition_penalty_(logits, seen, 1.0)
    assert logits.tolist() == [[1.0, -4.0, 1.0, -1.0]]
    prompt = torch.tensor([[5, 5, 5, 5]])
    plain = model.generate(prompt, max_new_tokens=12, do_sample=False)[0, 4:].tolist()
    pen = model.generate(prompt, max_new_tokens=12, do_sample=False, repetition_penalty=8.0)[0, 4:].tolist()
    assert len(set(pen)) >= len(set(plain))
    assert len(set(pen)) > len(pen) // 2          # a strong penalty keeps the path from looping


def test_several_returns_states_and_eos(model):
    prompt = torch.tensor([[7, 8], [9, 10]])
    g = torch.Generator().manual_seed(0)
    res = model.generate(prompt, max_new_tokens=5, do_sample=True, temperature=1.0, top_p=0.9, top_k=20,
                         num_return_sequences=3, return_dict_in_generate=True, generator=g)
    seqs, states = res["sequences"], res["states"]
    assert seqs.shape == (6, 7) and torch.equal(seqs[:3, :2], prompt[:1].expand(3, 2)) and torch.equal(seqs[3:, :2], prompt[1:].expand(3, 2))
    assert len(states) == 2 and states[0]["att_kv"].shape[0] == 6
    # carried states: generating from the stored state of a prefix equals generating from the whole prompt
    with torch.no_grad():
        _, st = model.forward_with_state(torch.tensor([[7, 8, 9]]))
    a = model.generate(torch.tensor([[11]]), max_new_tokens=4, do_sample=False, initial_states=st)
    b = model.generate(torch.tensor([[7, 8, 9, 11]]), max_new_tokens=4, do_sample=False)
    assert a[0, 1:].tolist() == b[0, 4:].tolist()
    first = int(model.generate(torch.tensor([[7, 8]]), max_new_tokens=1, do_sample=False)[0, -1])
    stopped = model.generate(torch.tensor([[7, 8]]), max_new_tokens=9, do_sample=False, eos_token_id=[first, 63])
    assert stopped.shape == (1, 3)                 # the EOS token is kept, nothing follows it


def test_adapter_layer_accessors():
    from rwkvtune_b200.peft.lora.layer import LoraLinear

    torch.manual_seed(0)
    layer = LoraLinear(torch.nn.Linear(8, 6, bias=False), r=2, lora_alpha=4)
    assert layer.weight is layer.base_layer.weight and "r=2" in layer.extra_repr() and "merged=False" in repr(layer)
    assert torch.equal(layer.effective_weight(), layer.base_layer.weight)          # B starts at zero
    sd = layer.get_lora_state_dict()
    assert set(sd) == {"lora_A", "lora_B"} and sd["lora_A"].shape == (2, 8) and sd["lora_B"].shape == (6, 2)
    sd["lora_B"] = torch.randn(6, 2)
    layer.load_lora_state_dict(sd)
    want = layer.base_layer.weight + (sd["lora_B"] @ sd["lora_A"]) * layer.scaling
    assert torch.allclose(layer.effective_weight(), want)
    x = torch.randn(3, 8)
    assert torch.allclose(layer(x), x @ want.t(), atol=1e-5)
    layer.disable_adapter()
    assert torch.equal(layer.effective_weight(), layer.base_layer.weight)
    layer.enable_adapter()
    layer.reset_lora_parameters("gaussian")
    assert float(layer.lora_B.detach().abs().sum()) == 0 and float(layer.lora_A.detach().abs().sum()) > 0


def test_flat_parameter_space_views_and_shards():
    from rwkvtune_b200.parallel import FlatParamSpace, build_param_groups

    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(5, 7), torch.nn.LayerNorm(7))
    before = {n: p.detach().clone() for n, p in net.named_parameters()}
    groups = build_param_groups(net.named_parameters(), weight_decay=0.1)
    space = FlatParamSpace(groups, world_size=4)
    assert space.padded % 4 == 0 and space.shard_numel * 4 == space.padded >= space.numel
    assert [space.shard_range(r) for r in (0, 3)] == [(0, space.shard_numel), (3 * space.shard_numel, space.padded)]
    views = dict(space.named_views())
    assert set(views) == set(before) and all(torch.equal(views[n], before[n]) for n in before)
    for n, p in net.named_parameters():             # parameters now live in the flat buffer
        assert p.data_ptr() == views[n].data_ptr() and p.grad is not None and p.grad.shape == p.shape
    net(torch.randn(2, 5)).sum().backward()
    assert float(space.grads.abs().sum()) > 0
    for p in net.parameters():
        p.grad = None
    space.rebind_grads()
    assert all(p.grad is not None for p in net.parameters())
    space.zero_grads()
    assert float(space.grads.abs().sum()) == 0 and float(next(net.parameters()).grad.abs().sum()) == 0
    decayed = [g for g in groups if g.weight_decay > 0]
    assert decayed and all(n.endswith(".weight") and p.dim() >= 2 for g in decayed for n, p in g.params)


def test_tokenizer_output_and_formatter_getters():
    from rwkvtune_b200.data.chat_formatter import ChatFormatter, get_default_formatter, get_formatter
    from rwkvtune_b200.data.tokenizers import RWKVTokenizer, get_vocab_path

    enc = RWKVTokenizer(get_vocab_path())(["hi", "hello there"], return_tensors="pt")
    assert enc.input_ids is enc["input_ids"] and enc.to("cpu") is enc and enc.attention_mask.dtype in (torch.long, torch.int64)
    with pytest.raises(AttributeError):
        enc.nothing
    assert isinstance(get_default_formatter(), ChatFormatter) and isinstance(get_formatter(None), ChatFormatter)
    text = get_default_formatter().format_messages([{"role": "user", "content": "hi"}], add_generation_prompt=True) \
        if hasattr(ChatFormatter, "format_messages") else get_default_formatter().format([{"role": "user", "content": "hi"}])
    assert "hi" in text


def test_structured_output_adapter_reports_specials_and_vocabulary():
    from rwkvtune_b200.data.tokenizers import get_tokenizer
    from rwkvtune_b200.inference.structured_output import TokenizerAdapter

    tok = get_tokenizer()
    ad = TokenizerAdapter(tok)
    assert ad.vocab_size == len(ad) == tok.vocab_size and ad.eos_token_id == tok.eos_token_id      # falls through
    assert 0 in ad.all_special_ids and tok.eos_token_id in ad.all_special_ids
    a_id = tok.encode("a")[0]
    assert ad.convert_ids_to_tokens(a_id) == "a" and ad.convert_ids_to_tokens(tok.encode("ab c")) == [tok.decode([i]) for i in tok.encode("ab c")]
    vocab = ad.get_vocab()
    assert vocab["a"] == a_id and len(vocab) > 60000
