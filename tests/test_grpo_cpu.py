"""GRPO pieces against closed forms, and the trainer end to end on a tiny CPU model."""
import json
import os

import pytest
import torch

from rwkvtune_b200.models import RWKVConfig, RWKV7Model
from rwkvtune_b200.peft import LoraConfig
from rwkvtune_b200.training import GRPOConfig, GRPOTrainer
from rwkvtune_b200.training.grpo import AdvantageCalculator, get_loss_function, selective_log_softmax, entropy_from_logits


def test_advantages_closed_form():
    r = torch.tensor([1.0, 2.0, 3.0, 4.0, 0.0, 0.0, 0.0, 0.0])
    adv = AdvantageCalculator("group", 4).compute_advantages(r)
    g = r[:4]
    assert torch.allclose(adv[:4], (g - g.mean()) / g.std(unbiased=False))
    assert torch.equal(adv[4:], torch.zeros(4))
    adv = AdvantageCalculator("group", 4, advantage_clip=1.0, low_reward_threshold=0.5, low_reward_scale=0.1).compute_advantages(r)
    assert adv[:4].abs().max() <= 1.0 and torch.equal(adv[4:], torch.zeros(4))
    assert torch.allclose(AdvantageCalculator("batch", 4).compute_advantages(r), (r - r.mean()) / r.std(unbiased=False))
    assert torch.equal(AdvantageCalculator("none", 4).compute_advantages(r), r)


def test_losses_match_manual():
    torch.manual_seed(0)
    n, C = 6, 5
    lp, old, ref = torch.randn(n, C) * 0.1 - 2, torch.randn(n, C) * 0.1 - 2, torch.randn(n, C) * 0.1 - 2
    adv = torch.randn(n)
    mask = (torch.rand(n, C) > 0.3).float()
    cfg = GRPOConfig(loss_type="dapo", epsilon=0.2, epsilon_high=0.3, beta=0.04, max_completion_length=8)
    fn = get_loss_function("dapo", cfg)
    pt = fn.compute_per_token_loss(lp, ref, old, adv, mask, 0.04)
    ratio = torch.exp(lp - old)
    manual = -torch.min(ratio * adv[:, None], ratio.clamp(0.8, 1.3) * adv[:, None])
    d = ref - lp
    manual = (manual + 0.04 * (torch.exp(d) - d - 1)) * mask
    assert torch.allclose(pt, manual, atol=1e-6)
    assert torch.allclose(fn.compute_loss(pt, mask), manual.sum() / mask.sum())
    dr = get_loss_function("dr_grpo", cfg)
    assert torch.allclose(dr.compute_loss(pt, mask), manual.sum() / (n * 8))
    cfg.importance_sampling_level = "sequence"
    seq = get_loss_function("grpo", cfg).importance_ratio(lp, old, mask)
    assert seq.shape == (n, 1)


def test_logprob_helpers():
    logits = torch.randn(2, 3, 11)
    idx = torch.randint(0, 11, (2, 3))
    assert torch.allclose(selective_log_softmax(logits, idx), torch.log_softmax(logits, -1).gather(-1, idx[..., None]).squeeze(-1), atol=1e-6)
    p = torch.softmax(logits, -1)
    assert torch.allclose(entropy_from_logits(logits), -(p * p.log()).sum(-1), atol=1e-5)


class _Tok:
    eos_token_id = 7
    vocab_size = 128

    def decode(self, ids, **kw):
        return " ".join(str(int(i)) for i in ids)

    def save_pretrained(self, d):
        pass


def _low_id_reward(prompts, completions, **kw):
    out = []
    for c in completions:
        toks = [int(t) for t in c.split()] if c else []
        out.append(sum(t < 64 for t in toks) / max(len(toks), 1))
    return out


def test_grpo_trainer_end_to_end(tmp_path):
    torch.manual_seed(0)
    model = RWKV7Model(RWKVConfig(n_layer=2, n_embd=64, vocab_size=128, dim_att_lora=16, dim_gate_lora=16, dim_mv_lora=16,
                                  eos_token_id=7))
    with torch.no_grad():
        for n, p in model.named_parameters():
            if n.endswith(("output.weight", "ffn.value.weight")):
                p.normal_(0, 0.05)
    data = [{"prompt": f"p{i}", "input_ids": [10 + i, 11 + i, 12 + i], "tag": i} for i in range(4)]
    proj = str(tmp_path / "grpo")
    args = GRPOConfig(micro_bsz=2, num_generations=4, steps_per_generation=2, max_prompt_length=8, max_completion_length=6,
                      temperature=1.0, top_p=0.95, beta=0.04, lr_init=1e-3, lr_final=1e-4, warmup_steps=0, accelerator="cpu",
                      precision="fp32", proj_dir=proj, epoch_count=1, save_rollout_steps=1, log_steps=1)
    seen_kwargs = {}

    def reward(prompts, completions, **kw):
        seen_kwargs.update(kw)
        return _low_id_reward(prompts, completions)

    tr = GRPOTrainer(model, reward, args, data, processing_class=_Tok(), peft_config=LoraConfig(r=4, lora_alpha=8))
    tr.train()
    recs = [json.loads(l) for l in open(os.path.join(proj, "grpo_loss_data.jsonl"))]
    assert len(recs) == 4                       # 2 prompt batches x generate_every 2
    assert "tag" in seen_kwargs and len(seen_kwargs["tag"]) == 8
    m = tr.last_metrics
    for key in ("train_loss", "clip_ratio", "kl_div", "entropy", "train/reward/mean", "completions/mean_length"):
        assert key in m and m[key] == m[key], key
    assert m["kl_div"] >= 0
    rollouts = os.listdir(os.path.join(proj, "rollouts"))
    assert rollouts and {"prompt", "completion", "reward", "advantage", "tag"} <= set(
        json.loads(open(os.path.join(proj, "rollouts", rollouts[0])).readline()))
    final = os.path.join(proj, "checkpoint_epoch_1")
    assert {"adapter_model.bin", "adapter_config.json", "trainer_state"} <= set(os.listdir(final))
    moved = any(float(p.abs().sum()) > 0 for n, p in tr.engine.model.named_parameters() if "lora_B" in n)
    assert moved, "LoRA B matrices never received an update"


def test_completion_postprocess_hook_contract(tmp_path):
    """The hook gets texts, ids, masks, the tokenizer and the dataset columns, and what it returns is what gets
    scored and trained on; a result of the wrong kind is rejected."""
    torch.manual_seed(0)
    model = RWKV7Model(RWKVConfig(n_layer=1, n_embd=64, vocab_size=128, dim_att_lora=16, dim_gate_lora=16, dim_mv_lora=16,
                                  eos_token_id=7))
    data = [{"prompt": f"p{i}", "input_ids": [10 + i, 11 + i], "tag": i} for i in range(2)]
    args = GRPOConfig(micro_bsz=2, num_generations=2, steps_per_generation=1, max_prompt_length=4, max_completion_length=5,
                      lr_init=1e-3, lr_final=1e-4, warmup_steps=0, accelerator="cpu", precision="fp32",
                      proj_dir=str(tmp_path / "g"), epoch_count=1, log_steps=1)
    calls = {}

    def keep_two_tokens(prompts, completions, completion_ids, masks, tokenizer, **columns):
        calls.update(n=len(prompts), shape=tuple(completion_ids.shape), tok=tokenizer, columns=sorted(columns))
        ids = completion_ids.clone()
        ids[:, 2:] = 0
        new_masks = masks.clone()
        new_masks[:, 2:] = False
        return {"completions": ["cut"] * len(completions), "completion_ids": ids, "masks": new_masks}

    scored = []

    def reward(prompts, completions, **kw):
        scored.extend(completions)
        return [float(i % 2) for i in range(len(completions))]

    tok = _Tok()
    tr = GRPOTrainer(model, reward, args, data, processing_class=tok, peft_config=LoraConfig(r=4, lora_alpha=8),
                     completion_postprocess_fn=keep_two_tokens)
    tr.train()
    assert calls["n"] == 4 and calls["shape"][0] == 4 and calls["tok"] is tok and calls["columns"] == ["tag"]
    assert scored and set(scored) == {"cut"}
    assert tr.last_metrics["completions/mean_length"] <= 2.0

    tr2 = GRPOTrainer(model, reward, args, data, processing_class=tok,
                      completion_postprocess_fn=lambda **kw: ["not", "a", "dict", "!"])
    try:
        tr2.train()
        raise AssertionError("expected TypeError")
    except TypeError as e:
        assert "dict" in str(e)


def test_loss_mask_hook_is_called_with_keywords(tmp_path):
    torch.manual_seed(0)
    model = RWKV7Model(RWKVConfig(n_layer=1, n_embd=64, vocab_size=128, dim_att_lora=16, dim_gate_lora=16, dim_mv_lora=16,
                                  eos_token_id=7))
    data = [{"prompt": f"p{i}", "input_ids": [10 + i, 11 + i]} for i in range(2)]
    args = GRPOConfig(micro_bsz=2, num_generations=2, steps_per_generation=1, max_prompt_length=4, max_completion_length=5,
                      lr_init=1e-3, lr_final=1e-4, warmup_steps=0, accelerator="cpu", precision="fp32",
                      proj_dir=str(tmp_path / "g"), epoch_count=1, log_steps=1)
    seen = {}

    def first_token_only(**kw):
        seen.update({k: type(v).__name__ for k, v in kw.items()})
        m = torch.zeros_like(kw["completion_ids"], dtype=torch.float32)
        m[:, 0] = 1
        return m

    tr = GRPOTrainer(model, lambda prompts, completions, **k: [float(i % 2) for i in range(len(completions))], args, data,
                     processing_class=_Tok(), peft_config=LoraConfig(r=4, lora_alpha=8), loss_mask_func=first_token_only)
    tr.train()
    assert set(seen) == {"prompts", "completions", "completion_ids", "tokenizer"}
    assert tr.last_metrics["train_loss"] == tr.last_metrics["train_loss"]


def test_reward_functions_are_weighted_named_and_checked():
    """Several reward functions: weights from the config, names from the functions, lists or tensors as results, and a
    result of the wrong length is an error that names the function."""
    model = RWKV7Model(RWKVConfig(n_layer=1, n_embd=64, vocab_size=128, dim_att_lora=8, dim_gate_lora=8, dim_mv_lora=8))
    data = [{"prompt": "p", "input_ids": [5, 6, 7]}]

    def fmt(prompts, completions, **kw):
        return [1.0, 0.0, 1.0]

    def quality(prompts, completions, **kw):
        return torch.tensor([0.5, 2.0, -1.0])

    args = GRPOConfig(micro_bsz=1, num_generations=3, steps_per_generation=1, max_prompt_length=8, max_completion_length=4,
                      accelerator="cpu", precision="fp32", reward_weights=[0.5, 2.0])
    tr = GRPOTrainer(model, [fmt, quality], args, data, processing_class=_Tok(), peft_config=LoraConfig(r=4, lora_alpha=8))
    assert tr.reward_names == ["fmt", "quality"] and tr.reward_weights == [0.5, 2.0]
    total, per_func = tr._compute_rewards(["p"] * 3, ["a", "b", "c"], {})
    assert per_func.shape == (3, 2) and per_func[:, 0].tolist() == [1.0, 0.0, 1.0]
    assert torch.allclose(total, torch.tensor([0.5 + 1.0, 0.0 + 4.0, 0.5 - 2.0]))
    single = GRPOTrainer(model, fmt, GRPOConfig(micro_bsz=1, num_generations=3, steps_per_generation=1, accelerator="cpu",
                                                precision="fp32"), data, processing_class=_Tok())
    assert single.reward_weights == [1.0] and len(single.reward_funcs) == 1          # a bare callable is one function
    with pytest.raises(ValueError, match="reward_weights has 1 entries for 2"):
        GRPOTrainer(model, [fmt, quality], GRPOConfig(micro_bsz=1, num_generations=3, steps_per_generation=1,
                                                     accelerator="cpu", precision="fp32", reward_weights=[1.0]),
                    data, processing_class=_Tok())
    with pytest.raises(ValueError, match="fmt returned 3 values for 2 completions"):
        tr._compute_rewards(["p"] * 2, ["a", "b"], {})


def test_full_parameter_grpo_keeps_a_frozen_reference_saves_per_batch_and_resumes(tmp_path):
    """Without an adapter and with ``beta > 0`` the KL reference is a frozen copy of the starting weights; save points
    every n batches; a second trainer picks the run up from one of them; ``save_model`` writes the final directory."""
    def make():
        torch.manual_seed(0)
        m = RWKV7Model(RWKVConfig(n_layer=2, n_embd=64, vocab_size=128, dim_att_lora=16, dim_gate_lora=16, dim_mv_lora=16,
                                  eos_token_id=7))
        with torch.no_grad():
            for n, p in m.named_parameters():
                if n.endswith(("output.weight", "ffn.value.weight")):
                    p.normal_(0, 0.05)
        return m

    data = [{"prompt": f"p{i}", "input_ids": [10 + i, 11 + i, 12 + i]} for i in range(4)]
    proj = str(tmp_path / "full")
    common = dict(micro_bsz=2, num_generations=2, steps_per_generation=1, max_prompt_length=8, max_completion_length=5,
                  beta=0.1, lr_init=5e-3, lr_final=1e-3, warmup_steps=0, accelerator="cpu", precision="fp32", epoch_count=1,
                  log_steps=1, save_every_n_batches=1, save_total_limit=0)
    with pytest.warns(UserWarning) as caught:
        tr = GRPOTrainer(make(), _low_id_reward, GRPOConfig(proj_dir=proj, **common), data, eval_dataset=data,
                         processing_class=_Tok(), optimizers=(object(), None))
    msgs = " ".join(str(w.message) for w in caught)
    assert "eval_dataset is accepted but not used" in msgs and "`optimizers` is ignored" in msgs
    start = {n: p.detach().clone() for n, p in tr.model.named_parameters()}
    tr.train()
    assert tr.ref_model is not None and not any(p.requires_grad for p in tr.ref_model.parameters())
    for n, p in tr.ref_model.named_parameters():                       # the reference did not move, the policy did
        assert torch.equal(p, start[n])
    assert any(not torch.equal(p, start[n]) for n, p in tr.engine.model.named_parameters())
    assert tr.last_metrics["kl_div"] >= 0
    saved = sorted(d for d in os.listdir(proj) if d.startswith("rwkv7-batch"))
    assert saved == ["rwkv7-batch1", "rwkv7-batch2"]
    assert {"model.pth", "config.json", "trainer_state"} <= set(os.listdir(os.path.join(proj, "rwkv7-batch1")))
    final = tr.save_model()
    assert final.endswith("final") and os.path.exists(os.path.join(final, "model.pth"))

    again = GRPOTrainer(make(), _low_id_reward,
                        GRPOConfig(proj_dir=str(tmp_path / "again"), resume_from_checkpoint=os.path.join(proj, "rwkv7-batch1"),
                                   **common), data, processing_class=_Tok())
    again.train()
    assert again.state["global_step"] == 2                               # one step was already done
    recs = [json.loads(l) for l in open(os.path.join(str(tmp_path / "again"), "grpo_loss_data.jsonl"))]
    assert len(recs) == 1
    with pytest.raises(FileNotFoundError):
        GRPOTrainer(make(), _low_id_reward, GRPOConfig(proj_dir=str(tmp_path / "x"), resume_from_checkpoint=str(tmp_path / "none"),
                                                       **common), data, processing_class=_Tok()).train()
    with pytest.raises(ValueError):
        GRPOTrainer(make(), _low_id_reward, GRPOConfig(proj_dir=str(tmp_path / "y"), **common), None, processing_class=_Tok())
    with pytest.raises(ValueError):
        GRPOTrainer(make(), [], GRPOConfig(proj_dir=str(tmp_path / "z"), **common), data, processing_class=_Tok())
