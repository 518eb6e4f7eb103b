"""The network must reproduce the reference model's numbers from the same state_dict."""
import torch
import pytest

from rwkvtune_b200.models import RWKVConfig, RWKV7Model


def _randomise(model, seed=0):
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if p.abs().sum() == 0 or name.endswith(("output.weight", "ffn.value.weight", "w1", "a1", "v1", "g1")):
                p.copy_(torch.randn(p.shape, generator=g) * 0.05)


def test_forward_backward_matches_reference(reference_pkg):
    from rwkvtune.models.rwkv7.model import RWKV7Model as RefModel
    from rwkvtune.models.configuration import RWKVConfig as RefConfig

    kw = dict(n_layer=3, n_embd=128, vocab_size=384, dim_att_lora=32, dim_gate_lora=32, dim_mv_lora=32)
    torch.manual_seed(1)
    ours = RWKV7Model(RWKVConfig(**kw))
    _randomise(ours)
    ref = RefModel(RefConfig(**kw))
    missing, unexpected = ref.load_state_dict(ours.state_dict())
    assert not missing and not unexpected
    ref.train(); ours.train()
    idx = torch.randint(0, 384, (2, 32))
    out_ref = ref(idx)
    out = ours(idx)
    assert torch.allclose(out, out_ref, atol=2e-5, rtol=1e-4), (out - out_ref).abs().max()
    out.square().mean().backward()
    out_ref.square().mean().backward()
    ref_grads = dict(ref.named_parameters())
    for name, p in ours.named_parameters():
        g_ref = ref_grads[name].grad
        assert g_ref is not None, name
        assert torch.allclose(p.grad, g_ref, atol=1e-6, rtol=2e-3), (name, (p.grad - g_ref).abs().max())


def test_state_dict_schema():
    cfg = RWKVConfig(n_layer=2, n_embd=128, vocab_size=256, dim_att_lora=32, dim_gate_lora=48, dim_mv_lora=16)
    sd = RWKV7Model(cfg).state_dict()
    C, H = 128, 2
    expect = {
        "emb.weight": (256, C), "head.weight": (256, C), "ln_out.weight": (C,), "blocks.0.ln0.weight": (C,),
        "blocks.1.att.x_r": (1, 1, C), "blocks.1.att.w1": (C, 32), "blocks.1.att.w2": (32, C),
        "blocks.1.att.v1": (C, 16), "blocks.1.att.g1": (C, 48), "blocks.1.att.g2": (48, C),
        "blocks.1.att.r_k": (H, 64), "blocks.1.att.ln_x.weight": (C,), "blocks.1.ffn.key.weight": (4 * C, C),
        "blocks.1.ffn.value.weight": (C, 4 * C), "blocks.1.ffn.x_k": (1, 1, C), "blocks.0.att.k_k": (1, 1, C),
    }
    for k, shape in expect.items():
        assert tuple(sd[k].shape) == shape, k
    assert "blocks.0.att.v1" not in sd and "blocks.1.ln0.weight" not in sd


def test_official_checkpoint_quirks():
    cfg = RWKVConfig(n_layer=2, n_embd=128, vocab_size=256)
    m = RWKV7Model(cfg)
    sd = {k: v.clone() for k, v in m.state_dict().items()}
    sd["blocks.0.att.r_k"] = sd["blocks.0.att.r_k"].flatten()
    sd["blocks.0.att.v0"] = torch.zeros(1, 1, 128)
    del sd["blocks.0.ln0.weight"], sd["blocks.0.ln0.bias"]
    m2 = RWKV7Model(cfg)
    m2.load_state_dict({"model": sd})
    assert m2.blocks[0].skip_ln0 and m2._emb_preprocessed
    assert m2.blocks[0].att.r_k.shape == (2, 64)


def test_chunked_state_equals_full():
    torch.manual_seed(0)
    m = RWKV7Model(RWKVConfig(n_layer=2, n_embd=128, vocab_size=256))
    _randomise(m)
    idx = torch.randint(0, 256, (2, 24))
    full = m(idx)
    a, st = m.forward_with_state(idx[:, :10])
    b, st = m.forward_with_state(idx[:, 10:11], st)
    c, st = m.forward_with_state(idx[:, 11:], st)
    assert torch.allclose(torch.cat([a, b, c], 1), full, atol=1e-5)


def test_loss_matches_logits_path():
    torch.manual_seed(0)
    m = RWKV7Model(RWKVConfig(n_layer=1, n_embd=64, vocab_size=128))
    _randomise(m)
    idx = torch.randint(0, 128, (2, 16))
    labels = idx.clone(); labels[:, :4] = -100
    loss = m.loss(idx, labels, l2wrap=False)
    ref = torch.nn.functional.cross_entropy(m(idx).reshape(-1, 128), labels.reshape(-1), ignore_index=-100)
    assert torch.allclose(loss, ref, atol=1e-6)


def test_block_recompute_matches_plain_backward():
    """Per-block activation checkpointing (own recompute node) gives the same loss and gradients, also when no
    block input requires grad (frozen embedding) and through the stateful chunked path."""
    import torch
    from rwkvtune_b200.models import RWKVConfig, RWKV7Model

    torch.manual_seed(0)
    cfg = RWKVConfig(n_layer=3, n_embd=64, vocab_size=128, dim_att_lora=8, dim_gate_lora=8, dim_mv_lora=8, ctx_len=64)
    m = RWKV7Model(cfg).train()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if n.endswith(("output.weight", "ffn.value.weight", "w1", "a1", "v1", "g1")):
                p.normal_(0, 0.05)
    m.emb.weight.requires_grad_(False)
    idx = torch.randint(0, 128, (2, 24))
    labels = torch.randint(0, 128, (2, 24))

    def grads(cp):
        m.config.grad_cp = cp
        m.zero_grad()
        loss = m.loss(idx, labels)
        loss.backward()
        return float(loss), {n: p.grad.clone() for n, p in m.named_parameters() if p.grad is not None}

    l0, g0 = grads(0)
    l1, g1 = grads(1)
    assert abs(l0 - l1) < 1e-6 and g0.keys() == g1.keys() and len(g0) > 10
    for n in g0:
        assert torch.allclose(g0[n], g1[n], atol=1e-6, rtol=1e-5), n


def test_tokenizer_matches_reference_trie_on_mixed_text(reference_pkg):
    """Encode / decode parity with the reference's ``TRIE_TOKENIZER`` (``rwkvtune/data/tokenizers/rwkv_tokenizer.py``)
    on ASCII, CJK, emoji, control characters and raw bytes that are not valid UTF-8."""
    from rwkvtune.data.tokenizers.rwkv_tokenizer import TRIE_TOKENIZER as RefTok

    from rwkvtune_b200.data.tokenizers import get_tokenizer
    from rwkvtune_b200.data.tokenizers.rwkv_tokenizer import TRIE_TOKENIZER

    import rwkvtune.data.tokenizers as ref_tok_pkg
    import os

    vocab = os.path.join(os.path.dirname(ref_tok_pkg.__file__), "vocab", "rwkv_vocab_v20230424.txt")
    ref = RefTok(vocab)
    ours = get_tokenizer()
    assert isinstance(ours, TRIE_TOKENIZER)
    texts = [
        "Hello, world!\n\nUser: hi\n\nAssistant: hello",
        "The quick brown fox jumps over the lazy dog 1234567890 times.",
        "中文分词测试：今天天气很好，我们去公园散步吧。",
        "日本語のテキストと한국어 텍스트 mixed with English",
        "emoji 🎉🚀👩‍💻 and symbols ∑∫√≠≈ ©®™",
        "tabs\tand\r\nnewlines\n\n\nand    spaces",
        "def f(x):\n    return x ** 2  # comment\n",
        "<|im_start|>system\nYou are helpful.<|im_end|>",
        "",
        " ",
        "a" * 300,
    ]
    for t in texts:
        a, b = ref.encode(t), ours.encode(t)
        assert a == b, t
        assert ref.decode(a) == ours.decode(b) == t
    raw = [bytes([0xff, 0xfe, 0x41, 0x00, 0x80]), bytes(range(256)), "héllo".encode("latin-1")]
    for bts in raw:
        a, b = ref.encodeBytes(bts), ours.encodeBytes(bts)
        assert a == b
        assert ref.decodeBytes(a) == ours.decodeBytes(b) == bts
        assert ref.decode(a) == ours.decode(b)      # tolerant decoding of invalid UTF-8
    import random

    rng = random.Random(0)
    for _ in range(50):
        ids = [rng.randrange(1, 65530) for _ in range(40)]
        assert ref.decode(ids) == ours.decode(ids)
        assert ref.decodeBytes(ids) == ours.decodeBytes(ids)
