"""The example scripts' data preparation and reward functions, and tiny end-to-end runs of all three scripts on CPU:
SFT with an adapter, GRPO, and generation with the adapter GRPO saved."""
import json
import os
import sys

import pytest
import torch

EXAMPLES = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples")
sys.path.insert(0, EXAMPLES)

import rewards  # noqa: E402
import sharegpt  # noqa: E402


class CharTokenizer:
    """One token per character (offset so that 0 stays the padding id)."""
    eos_token_id = 1
    vocab_size = 300

    def encode(self, text):
        return [min(ord(c), 255) + 2 for c in text]

    def decode(self, ids):
        return "".join(chr(i - 2) for i in ids if i >= 2)


CONV = [{"from": "system", "value": "Be brief."}, {"from": "human", "value": "Hi"}, {"from": "gpt", "value": "Yo"},
        {"from": "user", "value": "Bye"}, {"from": "assistant", "value": "Ok"}]


def test_sft_sample_is_shifted_and_role_masked():
    tok = CharTokenizer()
    s = sharegpt.encode_sft_sample(CONV, tok, eos_token_id=tok.eos_token_id)
    assert len(s["input_ids"]) == len(s["labels"])
    learned = [t for t in s["labels"] if t != sharegpt.IGNORE_INDEX]
    assert tok.decode(learned) == "YoOk" and learned.count(tok.eos_token_id) == 2     # both replies, each with its eos
    # label i is the token after input i wherever it is learned
    full = s["input_ids"] + [s["labels"][-1]]
    assert all(l == sharegpt.IGNORE_INDEX or l == full[i + 1] for i, l in enumerate(s["labels"]))
    text = tok.decode(s["input_ids"])
    assert text.startswith("System: Be brief.\n\nUser: Hi") and "Assistant:<think>\n\n</think>Yo" in text
    last = sharegpt.encode_sft_sample(CONV, tok, last_reply_only=True, eos_token_id=tok.eos_token_id)
    assert tok.decode([t for t in last["labels"] if t != sharegpt.IGNORE_INDEX]) == "Ok"


def test_grpo_dataset_unrolls_turns():
    tok = CharTokenizer()
    ds = sharegpt.build_grpo_dataset([{"conversations": CONV}], tok, max_prompt_length=4096, instructions="RULES\n")
    assert [d["ground_truth_answer"] for d in ds] == ["Yo", "Ok"]
    assert ds[0]["prompt"].endswith("User: Hi\n\nAssistant: <think")
    assert "Assistant: Yo\n\nUser: Bye\n\nAssistant: <think" in ds[1]["prompt"]
    assert ds[1]["input_ids"] == tok.encode(ds[1]["prompt"]) and ds[1]["turn_index"] == 1
    short = sharegpt.build_grpo_dataset([{"conversations": CONV}], tok, max_prompt_length=20, instructions="")
    assert all(len(d["input_ids"]) == 20 for d in short)


def test_reward_functions_score_structure():
    fns, weights = rewards.build_reward_functions(CharTokenizer())
    assert len(fns) == 7 and weights == [1.0, 0.5, 0.6, 0.8, 0.5, 0.8, 1.2]
    good = "x" * 600 + "</think>*nods slowly* Follow the lamps to the bridge.\n\n"
    bad = "\"Hello\" (waves) Name: hi"
    scores = {f.__name__: f(["p", "p", "p"], [good, bad, None], ground_truth_answer=["Follow the lamps", "zzz", "a"])
              for f in fns}
    assert scores["reward_has_think"] == [1.0, -1.0, -1.0]
    assert scores["reward_think_len"][0] == 1.0 and scores["reward_think_len"][1] == -0.5
    assert scores["reward_reply_len"][0] == pytest.approx(rewards.band_score(len("*nods slowly* Follow the lamps to the bridge."), 5, 10, 30, 50))
    assert scores["reward_actions_style"][:2] == [1.0, -0.3]
    assert scores["reward_similarity"][0] == pytest.approx(0.8) and scores["reward_similarity"][1] == pytest.approx(-0.2)
    assert scores["reward_format_clean"] == [1.0, -1.0, 0.0]
    assert scores["reward_eos_ending"] == [1.0, -0.5, -1.0]
    assert rewards.band_score(0, 5, 10, 30, 50) == -0.5 and rewards.band_score(7, 5, 10, 30, 50) == pytest.approx(0.4)
    assert rewards.band_score(40, 5, 10, 30, 50) == pytest.approx(0.5)


def test_sft_example_runs_end_to_end_on_cpu(tmp_path, monkeypatch):
    from rwkvtune_b200.models import RWKVConfig, RWKV7Model
    from rwkvtune_b200.utils import create_model_hub
    import train_sft_single_gpu as script

    torch.manual_seed(0)
    cfg = RWKVConfig(n_layer=2, n_embd=64, vocab_size=65536, dim_att_lora=8, dim_gate_lora=8, dim_mv_lora=8, ctx_len=128)
    raw = str(tmp_path / "raw.pth")
    torch.save(RWKV7Model(cfg).state_dict(), raw)
    hub = create_model_hub(str(tmp_path / "hub"), model_file=raw)
    out = str(tmp_path / "out")
    argv = ["train_sft_single_gpu.py", "--model_path", hub, "--data_file", os.path.join(EXAMPLES, "data", "sharegpt_sample.jsonl"),
            "--output_dir", out, "--ctx_len", "96", "--micro_bsz", "4", "--accumulate_grad_batches", "1", "--epoch_count", "1",
            "--use_lora", "--lora_r", "4", "--lora_alpha", "8", "--precision", "fp32", "--accelerator", "cpu"]
    monkeypatch.setattr(sys, "argv", argv)
    script.main()
    saved = [d for d in os.listdir(out) if os.path.isdir(os.path.join(out, d))]
    assert any("adapter_model.bin" in os.listdir(os.path.join(out, d)) for d in saved)


def _tiny_hub(tmp_path):
    from rwkvtune_b200.models import RWKVConfig, RWKV7Model
    from rwkvtune_b200.utils import create_model_hub

    torch.manual_seed(0)
    cfg = RWKVConfig(n_layer=2, n_embd=64, vocab_size=65536, dim_att_lora=8, dim_gate_lora=8, dim_mv_lora=8, ctx_len=128)
    raw = str(tmp_path / "raw.pth")
    torch.save(RWKV7Model(cfg).state_dict(), raw)
    return create_model_hub(str(tmp_path / "hub"), model_file=raw)


def test_grpo_and_generation_examples_run_on_cpu(tmp_path, monkeypatch):
    """``train_grpo_single_gpu.py`` trains adapters against the seven reward functions and dumps its rollouts;
    ``test_generation.py`` then loads the adapter directory it saved and writes its JSON report."""
    import test_generation as gen_script
    import train_grpo_single_gpu as grpo_script

    hub = _tiny_hub(tmp_path)
    data = os.path.join(EXAMPLES, "data", "sharegpt_sample.jsonl")
    out = str(tmp_path / "grpo")
    monkeypatch.setattr(sys, "argv", [
        "train_grpo_single_gpu.py", "--model_path", hub, "--data_file", data, "--output_dir", out, "--max_samples", "4",
        "--micro_bsz", "2", "--num_generations", "2", "--steps_per_generation", "2", "--max_prompt_length", "48",
        "--max_completion_length", "6", "--lora_r", "4", "--lora_alpha", "8", "--warmup_steps", "0", "--precision", "fp32",
        "--accelerator", "cpu", "--save_rollout_steps", "1", "--beta", "0.02"])
    grpo_script.main()
    recs = [json.loads(l) for l in open(os.path.join(out, "grpo_loss_data.jsonl"))]
    assert len(recs) == 4 and all(r["loss"] == r["loss"] for r in recs)
    rollouts = os.listdir(os.path.join(out, "rollouts"))
    first = json.loads(open(os.path.join(out, "rollouts", sorted(rollouts)[0])).readline())
    assert {"prompt", "completion", "reward", "advantage"} <= set(first)
    final = os.path.join(out, "checkpoint_epoch_1")
    assert {"adapter_model.bin", "adapter_config.json"} <= set(os.listdir(final))

    report = str(tmp_path / "gen.json")
    monkeypatch.setattr(sys, "argv", [
        "test_generation.py", "--model_path", hub, "--lora_path", final, "--data_file", data, "--num_samples", "2",
        "--max_new_tokens", "5", "--device", "cpu", "--output_json", report])
    gen_script.main()
    rows = json.load(open(report))
    assert len(rows) == 2 and all(isinstance(r, dict) and r for r in rows)
