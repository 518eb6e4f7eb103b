"""Small contracts: adapter settings, training-time model config checks, kernel switches, engine health on CPU,
adapter weight files written by the model's own method, cache reset, tokenizer odds and ends."""
import math
import os

import pytest
import torch

from rwkvtune_b200 import LoraConfig, get_peft_model
from rwkvtune_b200.models import RWKVConfig, RWKV7Config, RWKV7Model


def _model():
    torch.manual_seed(0)
    return RWKV7Model(RWKVConfig(n_layer=2, n_embd=64, vocab_size=64, dim_att_lora=8, dim_gate_lora=8, dim_mv_lora=8))


def test_adapter_settings_scaling_targets_and_validation():
    assert LoraConfig(r=16, lora_alpha=32).scaling == 2.0
    assert LoraConfig(r=16, lora_alpha=32, use_rslora=True).scaling == pytest.approx(32 / math.sqrt(16))
    cfg = LoraConfig()
    assert cfg.target_modules == ["receptance", "key", "value", "output", "key_ffn", "value_ffn"]
    assert cfg.modules_to_save == ["ln", "time"] and cfg.to_dict()["r"] == 64
    assert LoraConfig(target_modules="att").target_modules == ["receptance", "key", "value", "output"]
    assert LoraConfig(target_modules="receptance").target_modules == ["receptance"]
    with pytest.raises(ValueError):
        LoraConfig(r=0)
    # names are matched as substrings of the qualified module name: "key" and "value" reach both halves of a block
    m = get_peft_model(_model(), LoraConfig(r=4, lora_alpha=8))
    adapted = sorted(n for n, mod in m.named_modules() if type(mod).__name__ == "LoraLinear")
    assert adapted == sorted(f"blocks.{i}.{h}" for i in range(2)
                             for h in ("att.receptance", "att.key", "att.value", "att.output", "ffn.key", "ffn.value"))
    only_r = get_peft_model(_model(), LoraConfig(r=4, lora_alpha=8, target_modules="receptance"))
    assert sum(type(mod).__name__ == "LoraLinear" for mod in only_r.modules()) == 2
    trainable = {n for n, p in m.named_parameters() if p.requires_grad}
    assert any("lora_A" in n for n in trainable) and any(".ln1." in n for n in trainable)
    assert not any(n.endswith("att.key.base_layer.weight") or n == "emb.weight" for n in trainable)
    with pytest.raises(ValueError):
        get_peft_model(_model(), LoraConfig(target_modules="no_such_layer"))


def test_training_time_model_config_checks_infctx_chunks():
    ok = RWKV7Config(n_layer=2, n_embd=64, vocab_size=64, ctx_len=256, train_type="infctx", chunk_ctx=64)
    assert ok.chunk_ctx == 64 and ok.adam_eps == 1e-18
    for bad in (dict(chunk_ctx=0), dict(chunk_ctx=512), dict(chunk_ctx=96)):
        with pytest.raises(ValueError):
            RWKV7Config(n_layer=2, n_embd=64, vocab_size=64, ctx_len=256, train_type="infctx", **bad)
    RWKV7Config(n_layer=2, n_embd=64, vocab_size=64, ctx_len=256, train_type="normal", chunk_ctx=96)      # only checked for infctx


def test_kernel_family_switches_are_named_and_checked():
    from rwkvtune_b200 import ops

    names = sorted(ops._KERNELS)
    assert names and all(ops.kernel_enabled(n) for n in names)
    ops.set_kernel_enabled(names[0], False)
    try:
        assert not ops.kernel_enabled(names[0])
    finally:
        ops.set_kernel_enabled(names[0], True)
    with pytest.raises(KeyError):
        ops.set_kernel_enabled("no_such_family", False)


def test_engine_health_and_peak_memory_are_defined_on_cpu():
    from rwkvtune_b200.engine import EngineConfig, TrainEngine
    from rwkvtune_b200.parallel import DistContext

    eng = TrainEngine(_model(), EngineConfig(lr_init=1e-3, precision="fp32"), DistContext())
    idx = torch.randint(0, 64, (2, 16))
    loss = eng.train_step(idx, idx.roll(-1, 1), 1e-3)
    assert float(loss) == float(loss) and eng.health_ok()
    assert eng.phases.peak_bytes() == 0             # nothing to report without a CUDA device
    assert eng.start_guard() is None                # a single process has no peers to watch


def test_adapter_files_written_and_read_by_the_model_methods(tmp_path):
    m = get_peft_model(_model(), LoraConfig(r=4, lora_alpha=8))
    with torch.no_grad():
        for n, p in m.named_parameters():
            if "lora_B" in n:
                p.normal_(0, 0.1)
            if n.endswith("ln1.weight"):
                p.add_(0.25)
    idx = torch.tensor([[1, 2, 3, 4, 5]])
    want = m(idx)
    path = str(tmp_path / "deep" / "dir" / "adapter.pth")
    m.save_lora_weights(path)
    sd = torch.load(path)
    assert any("lora_A" in k for k in sd) and any("ln1.weight" in k for k in sd)          # the unfrozen norms travel too
    assert not any("base_layer" in k for k in sd)
    other = get_peft_model(_model(), LoraConfig(r=4, lora_alpha=8))
    other.load_lora_weights(path)
    assert torch.allclose(other(idx), want, atol=1e-6)


def test_state_cache_clear_and_tokenizer_odds_and_ends(capsys):
    from rwkvtune_b200.data.tokenizers import RWKVTokenizer, chatml_utils, get_tokenizer, get_vocab_path
    from rwkvtune_b200.inference import create_state_cache

    cache = create_state_cache(_model().eval(), max_cache_memory_gb=0.01)
    cache.create_checkpoints([1, 2, 3, 4, 5, 6])
    assert cache.get_stats()["entries"] >= 1 and cache.is_enabled()
    cache.clear()
    assert cache.get_stats()["entries"] == 0 and cache.lookup([1, 2, 3, 4, 5, 6]) == (0, None, None)

    tok = get_tokenizer()
    assert tok.get_vocab_size() == tok.vocab_size == 65530
    tok.printTokens(tok.encode("ab c"))
    assert capsys.readouterr().out.strip()
    full = RWKVTokenizer(get_vocab_path())
    chatml_utils.print_chatml_diagnostics(full)
    assert "INVALID" in capsys.readouterr().out
    chatml_utils.setup_chatml_tokenizer(full)
    chatml_utils.print_chatml_diagnostics(full, verbose=True)
    out = capsys.readouterr().out
    assert "ChatML configuration: OK" in out and "<|im_end|>" in out
