"""On-disk formats: every weight / adapter file name and container the loaders accept, and what the savers write."""
import json
import os

import pytest
import torch

from rwkvtune_b200 import AutoModel, LoraConfig, get_peft_model, is_peft_model, load_peft_model
from rwkvtune_b200.models import RWKVConfig, RWKV7Model


def _model(seed=0):
    torch.manual_seed(seed)
    m = RWKV7Model(RWKVConfig(n_layer=2, n_embd=64, vocab_size=128, dim_att_lora=16, dim_gate_lora=16, dim_mv_lora=16))
    with torch.no_grad():
        for n, p in m.named_parameters():
            if n.endswith(("output.weight", "ffn.value.weight")):
                p.normal_(0, 0.05)
    return m


IDX = torch.tensor([[3, 9, 27, 81, 5, 15, 45, 7]])


@pytest.mark.parametrize("layout", ["model.pth", "pytorch_model.pth", "model.safetensors", "wrapped", "bare_file"])
def test_auto_model_reads_every_weight_layout(tmp_path, layout):
    m = _model()
    want = m(IDX)
    d = tmp_path / "hub"
    d.mkdir()
    m.config.save_pretrained(str(d))
    sd = {k: v.detach().clone() for k, v in m.state_dict().items()}
    if layout == "model.safetensors":
        from safetensors.torch import save_file

        save_file({k: v.contiguous() for k, v in sd.items()}, str(d / layout))
        target = str(d)
    elif layout == "wrapped":                     # training frameworks wrap the weights as {"model": state_dict}
        torch.save({"model": sd}, str(d / "model.pth"))
        target = str(d)
    elif layout == "bare_file":                   # a weight file with its config.json beside it
        torch.save(sd, str(d / "anything.pth"))
        target = str(d / "anything.pth")
    else:
        torch.save(sd, str(d / layout))
        target = str(d)
    got = AutoModel.from_pretrained(target)
    assert torch.allclose(got(IDX), want, atol=1e-6)
    half = AutoModel.from_pretrained(target, dtype="bf16")
    assert next(half.parameters()).dtype == torch.bfloat16


def test_auto_model_errors_and_config_only_load(tmp_path):
    with pytest.raises(ValueError):
        AutoModel.from_pretrained(str(tmp_path / "missing"))
    d = tmp_path / "cfg_only"
    d.mkdir()
    _model().config.save_pretrained(str(d))
    with pytest.raises(FileNotFoundError):
        AutoModel.from_pretrained(str(d))
    fresh = AutoModel.from_pretrained(str(d), load_weights=False)
    assert fresh.config.n_embd == 64 and sum(p.numel() for p in fresh.parameters()) > 0


@pytest.mark.parametrize("fmt", ["pth", "safetensors"])
def test_save_pretrained_round_trip(tmp_path, fmt):
    m = _model(1)
    path = AutoModel.save_pretrained(m, str(tmp_path / "out"), save_format=fmt)
    assert os.path.basename(path) == ("model.pth" if fmt == "pth" else "model.safetensors")
    cfg = json.load(open(tmp_path / "out" / "config.json"))
    assert cfg["n_layer"] == 2 and cfg["n_embd"] == 64 and cfg["vocab_size"] == 128
    assert torch.allclose(AutoModel.from_pretrained(str(tmp_path / "out"))(IDX), m(IDX), atol=1e-6)


def _trained_adapter():
    m = get_peft_model(_model(), LoraConfig(r=4, lora_alpha=8))
    with torch.no_grad():
        for n, p in m.named_parameters():
            if "lora_B" in n:
                p.normal_(0, 0.05)
    return m


@pytest.mark.parametrize("cfg_name,weights_name", [("adapter_config.json", "adapter_model.bin"),
                                                   ("lora_config.json", "lora_weights.pth"),
                                                   ("adapter_config.json", "adapter_model.safetensors")])
def test_load_peft_model_reads_current_and_legacy_names(tmp_path, cfg_name, weights_name):
    src = _trained_adapter()
    want = src(IDX)
    d = tmp_path / "adapter"
    d.mkdir()
    json.dump({"r": 4, "lora_alpha": 8, "lora_dropout": 0.0}, open(d / cfg_name, "w"))
    sd = {k: v.detach().clone().contiguous() for k, v in src.get_lora_state_dict().items()}
    assert sd and all("lora_" in k or "ln" in k for k in sd)
    if weights_name.endswith(".safetensors"):
        from safetensors.torch import save_file

        save_file(sd, str(d / weights_name))
    else:
        torch.save(sd, str(d / weights_name))
    loaded = load_peft_model(_model(), str(d))
    assert is_peft_model(loaded) and torch.allclose(loaded(IDX), want, atol=1e-6)
    with pytest.raises(ValueError):
        load_peft_model(_model(), str(tmp_path / "no_such_dir"))
    empty = tmp_path / "empty"
    empty.mkdir()
    with pytest.raises(ValueError):
        load_peft_model(_model(), str(empty))


def test_adapter_switches_and_merged_state_dict():
    m = _trained_adapter()
    base = _model()
    with_adapter = m(IDX)
    m.disable_adapter()
    assert torch.allclose(m(IDX), base(IDX), atol=1e-6)
    m.enable_adapter()
    assert torch.allclose(m(IDX), with_adapter, atol=1e-6)
    merged_sd = m.get_merged_state_dict()
    assert not any("lora_" in k or "base_layer" in k for k in merged_sd) and set(merged_sd) == set(base.state_dict())
    plain = _model(5)
    plain.load_state_dict(merged_sd)
    assert torch.allclose(plain(IDX), with_adapter, atol=1e-5)
    # forming the merged dictionary leaves the adapter model itself as it was
    assert torch.allclose(m(IDX), with_adapter, atol=1e-6)
    m.merge_adapter()
    assert torch.allclose(m(IDX), with_adapter, atol=1e-5)
    m.unmerge_adapter()
    assert torch.allclose(m(IDX), with_adapter, atol=1e-5)


def test_hub_directory_layout_and_link_mode(tmp_path):
    from rwkvtune_b200.utils import create_model_hub

    m = _model()
    raw = tmp_path / "raw.pth"
    torch.save(m.state_dict(), str(raw))
    hub = create_model_hub(str(tmp_path / "hub"), model_file=str(raw), model_name="tiny", description="two layers",
                           temperature=0.7, top_p=0.5)
    files = set(os.listdir(hub))
    assert {"config.json", "generation_config.json", "tokenizer_config.json", "vocab.txt", "model.pth", "README.md"} <= files
    gen = json.load(open(os.path.join(hub, "generation_config.json")))
    assert gen["temperature"] == 0.7 and gen["top_p"] == 0.5
    cfg = json.load(open(os.path.join(hub, "config.json")))
    assert (cfg["n_layer"], cfg["n_embd"], cfg["vocab_size"]) == (2, 64, 128)           # read off the tensor shapes
    assert torch.allclose(AutoModel.from_pretrained(hub)(IDX), m(IDX), atol=1e-6)
    with pytest.raises(FileExistsError):
        create_model_hub(hub, model_file=str(raw))
    linked = create_model_hub(str(tmp_path / "linked"), model_file=str(raw), copy_weights=False)
    assert os.path.islink(os.path.join(linked, "model.pth"))
    st = create_model_hub(str(tmp_path / "st"), model_file=str(raw), save_format="safetensors")
    assert os.path.exists(os.path.join(st, "model.safetensors"))
    assert torch.allclose(AutoModel.from_pretrained(st)(IDX), m(IDX), atol=1e-6)


def test_merge_cli_syncs_eos_prefers_adapter_tokenizer_files_and_records_provenance(tmp_path, capsys):
    from rwkvtune_b200.cli import merge_lora
    from rwkvtune_b200.data.tokenizers import RWKVTokenizer, chatml_utils, get_vocab_path
    from rwkvtune_b200.training.model_save_utils import save_lora_checkpoint
    from rwkvtune_b200.utils import create_model_hub

    torch.manual_seed(0)
    base = RWKV7Model(RWKVConfig(n_layer=2, n_embd=64, vocab_size=65536, dim_att_lora=16, dim_gate_lora=16, dim_mv_lora=16))
    raw = tmp_path / "raw.pth"
    torch.save(base.state_dict(), str(raw))
    hub = create_model_hub(str(tmp_path / "hub"), model_file=str(raw))
    assert json.load(open(os.path.join(hub, "config.json")))["eos_token_id"] == 261

    adapted = get_peft_model(AutoModel.from_pretrained(hub), LoraConfig(r=4, lora_alpha=8))
    with torch.no_grad():
        for n, p in adapted.named_parameters():
            if "lora_B" in n:
                p.normal_(0, 0.05)
    tok = RWKVTokenizer(get_vocab_path())
    chatml_utils.setup_chatml_tokenizer(tok)                   # <|im_end|> becomes the EOS, on id 0
    adapter_dir = str(tmp_path / "adapter")
    save_lora_checkpoint(adapted, adapter_dir, base_model_path=hub, tokenizer=tok)
    idx = torch.tensor([[11, 12, 13, 14]])
    want = adapted(idx)

    out = str(tmp_path / "merged")
    assert merge_lora.main(["--base-model", hub, "--lora-model", adapter_dir, "--output", out, "--precision", "fp32",
                            "--save-format", "safetensors"]) == 0
    files = set(os.listdir(out))
    assert {"model.safetensors", "config.json", "tokenizer_config.json", "vocab.txt", "merge_info.json"} <= files
    assert json.load(open(os.path.join(out, "config.json")))["eos_token_id"] == 0           # synced from the adapter side
    merged_tok_cfg = json.load(open(os.path.join(out, "tokenizer_config.json")))
    assert merged_tok_cfg["eos_token"] == "<|im_end|>"                                       # the adapter's tokenizer wins
    info = json.load(open(os.path.join(out, "merge_info.json")))
    assert info["weights_file"] == "model.safetensors" and info["precision"] == "fp32"
    assert info["base_model"].endswith("hub") and info["lora_model"].endswith("adapter")
    merged = AutoModel.from_pretrained(out)
    assert not any("lora" in k for k in merged.state_dict()) and torch.allclose(merged(idx), want, atol=1e-5)
    assert merge_lora.main(["-b", str(tmp_path / "nowhere"), "-l", adapter_dir, "-o", out]) == 1
    assert "merge failed" in capsys.readouterr().err
