"""Small pieces of the public surface that have no other test: buffer, config files, parameter dictionaries,
the dictionary-state block step and the stand-alone L2Wrap."""
import json

import torch

from rwkvtune_b200.models import GenerationConfig, GenerationMixin, RWKV7Model, RWKVConfig
from rwkvtune_b200.sampling_params import SamplingParams
from rwkvtune_b200.training import L2Wrap
from rwkvtune_b200.training.grpo import GRPODataBuffer, RepeatBatchSampler


def test_grpo_data_buffer_per_sample_interface():
    buf = GRPODataBuffer(buffer_size=6)
    n, P, L = 4, 3, 5
    for start in (0, 4):
        buf.add_batch([f"p{start + i}" for i in range(n)], torch.arange(n * P).view(n, P) + start,
                      [f"c{start + i}" for i in range(n)], torch.arange(n * L).view(n, L), torch.zeros(n, L),
                      torch.arange(n, dtype=torch.float32) + start, torch.ones(n), torch.ones(n, L))
    assert len(buf) == 6 and buf.is_full()                      # the two oldest samples were dropped
    assert sorted(r["prompt"] for r in buf.items) == [f"p{i}" for i in range(2, 8)]
    batch = buf.sample_batch(4, generator=torch.Generator().manual_seed(0))
    assert batch["prompt_ids"].shape == (4, P) and batch["completion_ids"].shape == (4, L)
    assert len(set(batch["rewards"].tolist())) == 4             # without replacement
    buf.clear()
    assert buf.sample_batch(2) is None and not buf.is_full()
    buf.add("slice")
    assert buf.pop() == "slice" and buf.pop() is None


def test_repeat_batch_sampler_properties():
    s = RepeatBatchSampler(10, 4, repeat_count=3, shuffle=False)
    assert s.batch_size == 4 and s.sampler is s and isinstance(s.drop_last, bool)
    batches = list(s)
    assert batches[0] == batches[1] == batches[2]


def test_config_json_files(tmp_path):
    cfg = RWKVConfig(n_layer=2, n_embd=128, vocab_size=512)
    cfg.to_json_file(str(tmp_path / "c.json"))
    assert RWKVConfig.from_json_file(str(tmp_path / "c.json")).to_dict() == cfg.to_dict()
    g = GenerationConfig(temperature=0.7, top_k=5)
    g.to_json_file(str(tmp_path / "g.json"))
    assert json.load(open(tmp_path / "g.json"))["top_k"] == 5
    assert GenerationConfig.from_json_file(str(tmp_path / "g.json")) == g


def test_sampling_params_dict_round_trip():
    p = SamplingParams(max_tokens=7, temperature=0.5, stop="###", logit_bias={3: -1.0})
    d = p.to_dict()
    assert d["stop"] == ["###"] and d["max_tokens"] == 7
    assert SamplingParams.from_dict({**d, "unknown_key": 1}) == p


def test_l2wrap_gradient_at_argmax():
    logits = torch.randn(2, 3, 11, requires_grad=True)
    loss = L2Wrap.apply(logits.sum() * 0.0, logits)
    loss.backward()
    g = logits.grad
    mx, ids = logits.detach().max(-1, keepdim=True)
    expect = torch.zeros_like(g).scatter_(-1, ids, mx * 1e-4 / 6)
    assert torch.allclose(g, expect, atol=1e-9)


def test_block_forward_with_state_matches_model_state_step():
    torch.manual_seed(0)
    cfg = RWKVConfig(n_layer=2, n_embd=128, vocab_size=256)
    model = RWKV7Model(cfg).eval()
    assert isinstance(model, GenerationMixin)
    idx = torch.randint(0, 256, (1, 6))
    with torch.no_grad():
        x = model.emb(idx)
        H, N = cfg.n_embd // 64, 64
        v_first = torch.empty_like(x)
        for blk in model.blocks:
            st = {"att_x_prev": torch.zeros(1, cfg.n_embd), "att_kv": torch.zeros(1, H, N, N),
                  "ffn_x_prev": torch.zeros(1, cfg.n_embd)}
            x, v_first, new = blk.forward_with_state(x, v_first, st)
            assert new["att_kv"].shape == (1, H, N, N) and new["att_kv"].dtype == torch.float32
        x = torch.nn.functional.layer_norm(x, (cfg.n_embd,), model.ln_out.weight, model.ln_out.bias)
        ref = model.forward_hidden(idx)
    assert torch.allclose(x, ref, atol=1e-4, rtol=1e-4)


def test_half_block_steps_follow_the_reference_contract():
    """``att.forward_with_state`` / ``ffn.forward_with_state`` take the normalised input and return the bare
    projection; composed by hand with the residual sums they reproduce the block's own stateful step, over two
    calls that carry the state."""
    torch.manual_seed(0)
    cfg = RWKVConfig(n_layer=2, n_embd=128, vocab_size=256)
    model = RWKV7Model(cfg).eval()
    with torch.no_grad():
        for p in model.parameters():        # zero-initialised projections would make the comparison vacuous
            if p.dim() >= 2 and float(p.abs().sum()) == 0:
                p.normal_(0, 0.02)
    H, N, C = cfg.n_embd // 64, 64, cfg.n_embd
    ln = lambda m, t: torch.nn.functional.layer_norm(t, (C,), m.weight, m.bias)
    with torch.no_grad():
        x_all = model.emb(torch.randint(0, 256, (2, 7)))
        for blk in model.blocks:
            st = {"att_x_prev": torch.zeros(2, C), "att_kv": torch.zeros(2, H, N, N), "ffn_x_prev": torch.zeros(2, C)}
            a_prev, kv, f_prev = st["att_x_prev"], st["att_kv"], st["ffn_x_prev"]
            v_in = torch.randn_like(x_all)      # stands for layer 0's value rows when the block is not layer 0
            t0 = 0
            outs = []
            for part in (x_all[:, :4], x_all[:, 4:]):
                vf = v_in[:, t0:t0 + part.shape[1]]
                t0 += part.shape[1]
                want, vf_a, st = blk.forward_with_state(part, vf, st)
                h = ln(blk.ln0, part) if blk.layer_id == 0 else part
                y, vf_b, a_prev, kv = blk.att.forward_with_state(ln(blk.ln1, h), vf, a_prev, kv)
                assert torch.allclose(vf_a, vf_b, atol=1e-5)
                h = h + y
                y, f_prev = blk.ffn.forward_with_state(ln(blk.ln2, h), f_prev)
                got = h + y
                assert a_prev.dtype == f_prev.dtype == kv.dtype == torch.float32 and a_prev.shape == (2, C)
                assert torch.allclose(got, want, atol=1e-4, rtol=1e-4)
                assert torch.allclose(kv, st["att_kv"], atol=1e-4) and torch.allclose(f_prev, st["ffn_x_prev"], atol=1e-5)
                outs.append(want)
            x_all = torch.cat(outs, 1)


def test_operator_entry_points_follow_reference_conventions():
    from rwkvtune_b200.models.rwkv7 import operators as O
    from rwkvtune_b200.ops import reference
    torch.manual_seed(1)
    B, T, H, N = 2, 5, 2, 64
    C = H * N
    r, k, v = (torch.randn(B, T, C) * 0.5 for _ in range(3))
    w = -torch.nn.functional.softplus(-torch.randn(B, T, C)) - 0.5
    kk = torch.nn.functional.normalize(torch.randn(B, T, H, N), dim=-1).reshape(B, T, C)
    a, b = -kk, kk * torch.sigmoid(torch.randn(B, T, C))
    y_ref, s_ref = reference.wkv7(r, w, k, v, a, b, N)
    op = O.load_wkv_operator(device="cpu")
    assert torch.allclose(op(r, w, k, v, a, b), y_ref)
    y, s = op(r, w, k, v, a, b, state=None, return_state=True)
    assert torch.allclose(s, s_ref)
    assert O.load_wkv7_operator is O.load_wkv_operator
    y2, s2 = O.rwkv7_wkv(r, w, k, v, a, b, head_size=N, return_state=True)
    assert torch.allclose(y2, y_ref, atol=1e-5) and torch.allclose(s2, s_ref, atol=1e-5)
    y1, s1 = O.rwkv7_wkv_cpu(r[0], w[0], k[0], v[0], a[0], b[0], HEAD_SIZE=N)
    assert y1.shape == (T, C) and torch.allclose(s1, s_ref[0], atol=1e-5)
    # infctx form: [B, T, H, N], w first, two half chunks carry the state
    f4 = lambda t: t.reshape(B, T, H, N)
    ya, sa = O.rwkv7_wkv_infctx(f4(w)[:, :3], f4(r)[:, :3], f4(k)[:, :3], f4(v)[:, :3], f4(a)[:, :3], f4(b)[:, :3])
    yb, sb = O.load_cuda_operator_infctx()(f4(w)[:, 3:], f4(r)[:, 3:], f4(k)[:, 3:], f4(v)[:, 3:], f4(a)[:, 3:],
                                           f4(b)[:, 3:], state=sa)
    assert torch.allclose(torch.cat([ya, yb], 1).reshape(B, T, C), y_ref, atol=1e-5)
    assert torch.allclose(sb, s_ref, atol=1e-5)
    # the oracle takes q, k, v, w (the order of the reference's naive operator), unlike the chunk step above
    yn, sn = O.rwkv7_wkv_infctx_naive(f4(r), f4(k), f4(v), f4(w), f4(a), f4(b), scale=0.5)
    assert torch.allclose(yn.reshape(B, T, C), 0.5 * y_ref, atol=1e-5) and torch.allclose(sn, s_ref, atol=1e-5)
    try:
        O.load_wkv_operator(device="tpu")
        raise AssertionError("expected ValueError")
    except ValueError:
        pass


def test_save_model_checkpoint_layout(tmp_path):
    from rwkvtune_b200.training.model_save_utils import save_model_checkpoint

    class Holder:
        pass

    h = Holder()
    h.model = RWKV7Model(RWKVConfig(n_layer=1, n_embd=64, vocab_size=128))
    path = save_model_checkpoint(h, str(tmp_path), "step-10")
    assert path == str(tmp_path / "step-10" / "model.pth") and (tmp_path / "step-10" / "config.json").exists()
    sd = torch.load(path)
    assert set(sd) == set(h.model.state_dict())


def test_trainer_accepts_lora_settings_as_dict():
    from rwkvtune_b200 import SFTConfig, SFTTrainer, is_peft_model
    m = RWKV7Model(RWKVConfig(n_layer=1, n_embd=64, vocab_size=128))
    tr = SFTTrainer(m, SFTConfig(accelerator="cpu", precision="fp32"), [{"input_ids": [1, 2, 3], "labels": [2, 3, 4]}],
                    lora_config={"r": 4, "lora_alpha": 8, "not_a_field": 1})
    assert is_peft_model(tr.model) and tr.args.use_lora
    assert any("lora_A" in n for n, _ in tr.model.named_parameters())


def test_pipeline_generate_forms_and_chat_prompt():
    from rwkvtune_b200.inference import InferencePipeline
    torch.manual_seed(0)
    model = RWKV7Model(RWKVConfig(n_layer=1, n_embd=64, vocab_size=65536))
    pipe = InferencePipeline(model=model, device="cpu", precision="fp32")
    one = pipe.generate("hello", max_tokens=3)
    assert isinstance(one, str)
    many = pipe.generate(["a b", "c"], max_tokens=2, num_generations=2)
    assert isinstance(many, list) and len(many) == 4
    assert isinstance(pipe.generate("x", max_tokens=2, num_generations=2), list)
    seen = {}
    pipe.generate = lambda prompt, **kw: seen.update(prompt=prompt, kw=kw) or " ok "
    assert pipe.chat("How?", system_prompt="Be brief.", history=[("Hi", "Hello")], temperature=0.5) == "ok"
    assert seen["prompt"] == "System: Be brief.\n\nUser: Hi\n\nAssistant: Hello\n\nUser: How?\n\nAssistant:"
    assert seen["kw"] == {"temperature": 0.5, "max_tokens": 256}


def test_sharegpt_conversion_and_text_generator_complete():
    from rwkvtune_b200.data.chat_formatter import ChatFormatter
    conv = [{"from": "human", "value": "q"}, {"from": "gpt_ignore", "value": "draft"}, {"from": "gpt", "value": "a"}]
    kept = ChatFormatter.convert_sharegpt_to_messages(conv)
    assert [m["role"] for m in kept] == ["user", "assistant", "assistant"] and kept[1]["_ignore"] is True
    dropped = ChatFormatter.convert_sharegpt_to_messages(conv, include_gpt_ignore=False)
    assert [m["content"] for m in dropped] == ["q", "a"]
    text = ChatFormatter().format_sharegpt(conv, add_generation_prompt=True, include_gpt_ignore=False)
    assert "q" in text and "draft" not in text

    from rwkvtune_b200.inference import TextGenerator

    class _Pipe:
        def generate(self, prompt, max_tokens=100, num_generations=1, **kw):
            return "x" if num_generations == 1 else ["x"] * num_generations

    g = TextGenerator(_Pipe())
    assert g.complete("p") == ["x"] and g.complete("p", n=3) == ["x", "x", "x"]


def test_save_utilities_follow_reference_signatures(tmp_path):
    from rwkvtune_b200 import LoraConfig, get_peft_model
    from rwkvtune_b200.training.model_save_utils import (get_lora_state_dict, save_checkpoint_with_lora_support,
                                                         save_lora_checkpoint, save_model_with_config)
    base = RWKV7Model(RWKVConfig(n_layer=1, n_embd=64, vocab_size=128))
    p = save_model_with_config(base, str(tmp_path / "a"), "weights")
    assert p.endswith("weights.pth") and (tmp_path / "a" / "config.json").exists()
    assert save_model_with_config(base, str(tmp_path / "skip"), is_main_process=False) is None
    assert not (tmp_path / "skip").exists()
    p = save_model_with_config(base.state_dict(), str(tmp_path / "b"), model_config_obj=base.config,
                               save_format="safetensors")
    assert p.endswith("model.safetensors") and (tmp_path / "b" / "config.json").exists()

    lora = get_peft_model(base, peft_config=LoraConfig(r=4, lora_alpha=8))
    assert get_lora_state_dict(model=lora)
    save_lora_checkpoint(lora, str(tmp_path / "c"), lora_config={"note": "x"}, base_model_path="hub/x",
                         safe_serialization=True)
    cfg = json.load(open(tmp_path / "c" / "adapter_config.json"))
    assert cfg["r"] == 4 and cfg["note"] == "x" and cfg["base_model_name_or_path"] == "hub/x"
    assert (tmp_path / "c" / "adapter_model.safetensors").exists()

    class Holder:
        model = lora

    out = save_checkpoint_with_lora_support(Holder(), str(tmp_path), "ckpt-1", use_lora=True, lora_save_mode="both")
    assert out == str(tmp_path / "ckpt-1")
    assert (tmp_path / "ckpt-1" / "adapter_model.bin").exists() and (tmp_path / "ckpt-1" / "merged" / "model.pth").exists()


def test_repeat_batch_sampler_wraps_a_batch_sampler():
    from torch.utils.data import BatchSampler, SequentialSampler
    inner = BatchSampler(SequentialSampler(range(7)), batch_size=3, drop_last=False)
    s = RepeatBatchSampler(inner, 2)
    assert list(s) == [[0, 1, 2], [0, 1, 2], [3, 4, 5], [3, 4, 5], [6], [6]] and len(s) == 6
    assert s.batch_size == 3 and s.drop_last is False and s.sampler is inner.sampler
    assert len(RepeatBatchSampler(batch_sampler := inner, repeat_batch_count=3)) == 9 and batch_sampler is inner
    try:
        RepeatBatchSampler(inner, 0)
        raise AssertionError("expected ValueError")
    except ValueError:
        pass


def test_public_names_of_the_reference_are_importable():
    import importlib
    expected = {
        "rwkvtune_b200": ["AutoModel", "AutoTokenizer", "GRPOConfig", "GRPOTrainer", "GenerationConfig", "LoraConfig",
                          "PretrainConfig", "PretrainTrainer", "RWKV7Config", "RWKV7Model",
                          "RWKV7_DEFAULT_TARGET_MODULES", "RWKVConfig", "RWKVTokenizer", "SFTConfig", "SFTTrainer",
                          "TRIE_TOKENIZER", "__author__", "__license__", "__version__", "create_model_hub",
                          "get_peft_model", "get_tokenizer", "is_peft_model", "load_peft_model"],
        "rwkvtune_b200.inference": ["InferencePipeline", "TextGenerator", "BatchGenerator", "GenerationConfig",
                                    "GRPOBatchGenerator", "TokenSampler", "SchedulerCore", "SequenceState", "SeqStatus",
                                    "create_scheduler_core", "JsonSchemaEnforcer", "JsonObjectEnforcer",
                                    "create_enforcer", "is_structured_output_available", "StateCache", "CacheConfig",
                                    "CacheLevel", "create_state_cache"],
        "rwkvtune_b200.training": ["PretrainConfig", "PretrainTrainer", "SFTConfig", "SFTTrainer", "GRPOConfig",
                                   "GRPOTrainer"],
        "rwkvtune_b200.peft": ["LoraConfig", "get_peft_model", "is_peft_model", "load_peft_model",
                               "RWKV7_DEFAULT_TARGET_MODULES"],
        "rwkvtune_b200.models": ["RWKVConfig", "GenerationConfig", "AutoModel", "RWKV7Model", "RWKV7Config",
                                 "GenerationMixin"],
        "rwkvtune_b200.models.rwkv7.operators": ["load_wkv_operator", "rwkv7_wkv", "load_wkv7_operator",
                                                 "load_cpu_operator", "load_cuda_operator_train",
                                                 "load_cuda_operator_inference", "load_cuda_operator_infctx",
                                                 "rwkv7_wkv_infctx", "rwkv7_wkv_infctx_naive", "rwkv7_wkv_cpu",
                                                 "naive_recurrent_rwkv7_fwd", "naive_recurrent_rwkv7_bwd",
                                                 "RWKV7InfctxNaiveFunction", "WKV7InfctxFunction"],
        "rwkvtune_b200.training.callbacks": ["TrainingCallback"],
        "rwkvtune_b200.training.grpo": ["get_gpu_memory_info", "monitor_memory_and_time", "AdvantageCalculator",
                                        "get_loss_function", "create_grpo_dataloader", "RepeatBatchSampler"],
        "rwkvtune_b200.configs": ["load_model_config", "list_available_models", "print_model_info", "ModelConfig"],
        "rwkvtune_b200.training.model_save_utils": ["save_model_with_config", "save_model_checkpoint",
                                                    "get_lora_state_dict", "save_lora_checkpoint",
                                                    "save_checkpoint_with_lora_support"],
    }
    for module, names in expected.items():
        mod = importlib.import_module(module)
        missing = [n for n in names if not hasattr(mod, n)]
        assert not missing, f"{module} lacks {missing}"
