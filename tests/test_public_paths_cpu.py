"""Public entry points that nothing else in the CPU suite calls: state containers and the infinite-context view,
ragged batches, size presets, the hub CLI, generation presets, small dataclasses and helpers."""
import asyncio
import json
import os

import pytest
import torch

from rwkvtune_b200.models import RWKVConfig, RWKV7Model


def _model(**kw):
    torch.manual_seed(0)
    m = RWKV7Model(RWKVConfig(n_layer=2, n_embd=128, vocab_size=96, dim_att_lora=16, dim_gate_lora=16, dim_mv_lora=16, **kw))
    with torch.no_grad():
        for n, p in m.named_parameters():
            if n.endswith(("output.weight", "ffn.value.weight")):
                p.normal_(0, 0.05)
    return m.eval()


def test_state_list_and_infctx_view_carry_chunks():
    from rwkvtune_b200.models.rwkv7.infctx_module import BlockState, BlockStateList, ChannelMixState, TimeMixState
    from rwkvtune_b200.models.rwkv7.model_infctx import RWKV7Infctx, as_infctx

    model = _model()
    cfg = model.config
    states = BlockStateList.create(cfg.n_layer, 2, cfg.n_embd, cfg.n_head, "cpu", dtype=torch.float32)
    assert len(states) == 2 and states.shift_states.shape == (2, 2, 2, 128) and states.wkv_states.shape == (2, 2, 2, 64, 64)
    assert states.wkv_states.dtype == torch.float32 and float(states.shift_states.abs().sum()) == 0
    assert BlockStateList.empty(2, 3, 128, 2, "cpu").shift_states.dtype == torch.bfloat16
    layer = states[1]
    assert isinstance(layer, BlockState) and layer.time_mix_state.wkv_state.shape == (2, 2, 64, 64)
    states[0] = BlockState(TimeMixState(torch.ones(2, 128), torch.full((2, 2, 64, 64), 2.0)), ChannelMixState(torch.full((2, 128), 3.0)))
    assert float(states.shift_states[0, 0].mean()) == 1 and float(states.wkv_states[0].mean()) == 2
    assert float(states.shift_states[0, 1].mean()) == 3 and float(states.shift_states[1].abs().sum()) == 0
    copy = states.clone()
    copy.shift_states.zero_()
    assert float(states.shift_states[0, 0].mean()) == 1 and states.detach().wkv_states.requires_grad is False
    assert states.to("cpu").wkv_states.device.type == "cpu"

    view = as_infctx(model)
    assert isinstance(view, RWKV7Infctx) and as_infctx(view) is view
    idx = torch.randint(0, 96, (2, 12))
    zero = BlockStateList.create(cfg.n_layer, 2, cfg.n_embd, cfg.n_head, "cpu", dtype=torch.float32)
    with torch.no_grad():
        whole = model(idx)
        l1, shift, wkv = view.forward_infctx(idx[:, :5], zero.shift_states, zero.wkv_states)
        l2, shift2, wkv2 = view.forward_infctx(idx[:, 5:], shift, wkv)
    assert shift.shape == zero.shift_states.shape and wkv.shape == zero.wkv_states.shape
    assert torch.allclose(torch.cat([l1, l2], 1), whole, atol=1e-4, rtol=1e-4)
    assert not torch.equal(wkv, wkv2)


def test_ragged_batch_forward_matches_one_sequence_at_a_time():
    model = _model()
    seqs = [[5, 6, 7, 8, 9, 10, 11], [20, 21], [30, 31, 32, 33]]
    with torch.no_grad():
        last, states = model.forward_batch_dynamic(seqs)
        full, _ = model.forward_batch_dynamic(seqs, full_output=True)
        for i, s in enumerate(seqs):
            want, st = model.forward_with_state(torch.tensor([s]))
            assert torch.allclose(last[i], want[0, -1], atol=1e-4, rtol=1e-4)
            assert full[i].shape == (len(s), 96) and torch.allclose(full[i], want[0], atol=1e-4, rtol=1e-4)
            for layer, ref in zip(states, st):
                assert torch.allclose(layer["att_kv"][i], ref["att_kv"][0], atol=1e-4)
                assert torch.allclose(layer["att_x_prev"][i], ref["att_x_prev"][0], atol=1e-5)
        # continuing from the returned states equals one longer pass
        more, _ = model.forward_batch_dynamic([[1], [2, 3], [4]], states=states)
        want, _ = model.forward_with_state(torch.tensor([seqs[1] + [2, 3]]))
    assert torch.allclose(more[1], want[0, -1], atol=1e-4, rtol=1e-4)
    assert model.num_parameters() == sum(p.numel() for p in model.parameters())


def test_size_presets_resolve_by_short_name_full_name_and_path(capsys):
    from rwkvtune_b200.configs import ModelConfig, list_available_models, load_model_config, print_model_info

    models = list_available_models()
    assert {"rwkv7-0.1b", "rwkv7-0.4b", "rwkv7-1.5b", "rwkv7-2.9b", "rwkv7-7.2b", "rwkv7-13.3b"} <= set(models)
    a, b, c = load_model_config("1.5b"), load_model_config("RWKV7-1.5B"), load_model_config(models["rwkv7-1.5b"])
    assert isinstance(a, ModelConfig) and a.to_train_config_dict() == b.to_train_config_dict() == c.to_train_config_dict()
    assert (a.n_layer, a.n_embd, a.vocab_size, a.head_size_a) == (24, 2048, 65536, 64) and "1.5" in repr(a)
    cfg = load_model_config("0.1b").to_rwkv_config()
    assert (cfg.n_layer, cfg.n_embd, cfg.n_head, cfg.ffn_width) == (12, 768, 12, 3072)
    assert a.model_path is None or os.path.exists(a.model_path)
    with pytest.raises(ValueError):
        load_model_config("9000b")
    print_model_info(a)
    out = capsys.readouterr().out
    assert "n_layer: 24" in out and "recommended" in out


def test_hub_cli_builds_from_a_preset_and_lists_presets(tmp_path, capsys):
    from rwkvtune_b200 import AutoModel
    from rwkvtune_b200.cli import create_model_hub as cli

    assert cli.main(["--list-configs"]) == 0
    assert "rwkv7-0.1b" in capsys.readouterr().out
    weights = tmp_path / "w.pth"
    tiny = _model()
    torch.save(tiny.state_dict(), str(weights))
    out = tmp_path / "hub"
    rc = cli.main(["--output-dir", str(out), "--model-file", str(weights), "--config-name", "0.1b", "--n-layer", "2",
                   "--n-embd", "128", "--vocab-size", "96", "--dim-att-lora", "16", "--dim-gate-lora", "16",
                   "--dim-mv-lora", "16", "--ctx-len", "256", "--top-p", "0.3", "--model-name", "tiny", "--link-weights",
                   "--verbose"])
    assert rc == 0 and os.path.islink(out / "model.pth")
    cfg = json.load(open(out / "config.json"))
    assert (cfg["n_layer"], cfg["n_embd"], cfg["vocab_size"], cfg["ctx_len"]) == (2, 128, 96, 256)   # flags override the preset
    assert json.load(open(out / "generation_config.json"))["top_p"] == 0.3
    idx = torch.tensor([[1, 2, 3]])
    assert torch.allclose(AutoModel.from_pretrained(str(out))(idx), tiny(idx), atol=1e-6)
    assert cli.main(["--output-dir", str(out), "--model-file", str(weights), "--config-name", "0.1b"]) == 1      # exists
    assert "error" in capsys.readouterr().err


def test_generation_presets_and_repl():
    from rwkvtune_b200.inference import TextGenerator

    class Pipe:
        def __init__(self):
            self.calls = []

        def generate(self, prompt, **kw):
            self.calls.append(("generate", prompt, kw))
            n = kw.get("num_generations", 1)
            return "out" if n == 1 else ["out"] * n

        def chat(self, user, system_prompt=None, history=None):
            self.calls.append(("chat", user, list(history)))
            return f"re:{user}"

    pipe = Pipe()
    gen = TextGenerator(pipe)
    assert gen.generate("hi", preset="precise", max_tokens=7, top_k=5) == "out"
    assert pipe.calls[-1] == ("generate", "hi", {"max_tokens": 7, "temperature": 0.3, "top_p": 0.5, "top_k": 5})
    assert set(TextGenerator.PRESETS) == {"greedy", "creative", "precise", "balanced"}
    with pytest.raises(ValueError):
        gen.generate("hi", preset="wild")
    assert gen.complete("hi", n=3) == ["out"] * 3 and gen.complete("hi") == ["out"]
    lines = iter(["", "one", "clear", "two", "quit", "never"])
    gen.interactive_chat(system_prompt="sys", input_fn=lambda _prompt: next(lines))
    chats = [c for c in pipe.calls if c[0] == "chat"]
    assert [c[1] for c in chats] == ["one", "two"] and chats[1][2] == []          # "clear" dropped the first turn
    gen.interactive_chat(input_fn=lambda _p: "again", max_turns=2)
    assert len([c for c in pipe.calls if c[0] == "chat"]) == 4


def test_small_dataclasses_and_config_helpers(tmp_path):
    from rwkvtune_b200.outputs import CompletionOutput, RequestOutput
    from rwkvtune_b200.sampling_params import SamplingParams

    done = CompletionOutput(0, "hi", [1, 2], cumulative_logprob=-0.5, finish_reason="stop")
    assert done.finished() and not CompletionOutput(1, "", []).finished()
    req = RequestOutput("r1", "p", [3, 4], [done])
    assert req.finished and "outputs=1" in repr(req) and "r1" in repr(req)
    assert SamplingParams(temperature=0.0, max_tokens=9).greedy and not SamplingParams().greedy
    assert SamplingParams(stop="\n").stop == ["\n"]
    with pytest.raises(ValueError):
        SamplingParams(top_p=1.5)
    cfg = RWKVConfig(n_layer=2, n_embd=128, vocab_size=96).update(ctx_len=512, note="kept")
    assert cfg.ctx_len == 512 and cfg._extra_config["note"] == "kept"
    cfg.save_pretrained(str(tmp_path))
    back = RWKVConfig.from_pretrained(str(tmp_path))
    assert (back.n_layer, back.n_embd, back.ctx_len) == (2, 128, 512)
    with pytest.raises(FileNotFoundError):
        RWKVConfig.from_pretrained(str(tmp_path / "none"))


def test_group_statistics_and_loss_aggregations():
    from rwkvtune_b200.training.grpo import AdvantageCalculator, BNPOLoss, DAPOLoss, DrGRPOLoss, GRPOLossBase

    calc = AdvantageCalculator(num_generations=2)
    r = torch.tensor([1.0, 3.0, 2.0, 2.0])
    st = calc.compute_group_statistics(r)
    assert st["group_mean_rewards"].tolist() == [2.0, 2.0] and st["group_std_rewards"].tolist() == [1.0, 0.0]
    assert float(st["global_mean_reward"]) == 2.0
    per_token = torch.tensor([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]])
    mask = torch.tensor([[1.0, 1.0, 0.0], [1.0, 0.0, 0.0]])
    assert float(DAPOLoss().compute_loss(per_token, mask)) == pytest.approx(7.0 / 3)
    assert float(BNPOLoss().compute_loss(per_token, mask)) == pytest.approx(7.0 / 3)
    assert float(DrGRPOLoss(4).compute_loss(per_token, mask)) == pytest.approx(7.0 / 8)
    with pytest.raises(NotImplementedError):
        GRPOLossBase().compute_loss(per_token, mask)


def test_scheduler_factory_and_async_step():
    from rwkvtune_b200.inference import SequenceState, create_scheduler_core

    class Tok:
        eos_token_id = 7
        vocab_size = 96

        def decode(self, ids, **kw):
            return " ".join(map(str, ids))

    model = _model(eos_token_id=7)
    sched = create_scheduler_core(model, Tok(), max_batch_size=2, max_batch_tokens=16, prefill_chunk_size=4,
                                  use_state_cache=True, max_cache_memory_gb=0.01)
    assert sched.state_cache is not None and sched.get_stats()["free_slots"] == 2
    seq = SequenceState(0, [3, 4, 5], max_new_tokens=3, temperature=0.0, eos_token_id=7)
    sched.add_sequences([seq])
    steps = 0
    while sched.has_pending_work() and steps < 20:
        asyncio.run(sched.step_async())
        steps += 1
    want = model.generate(torch.tensor([[3, 4, 5]]), max_new_tokens=3, do_sample=False, eos_token_id=7)[0, 3:].tolist()
    assert seq.is_finished and seq.generated_tokens == want[:len(seq.generated_tokens)]
