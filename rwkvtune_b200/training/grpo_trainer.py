"""``GRPOTrainer``: group-relative policy optimisation with on-policy rollouts.

Algorithm and public surface follow ``rwkvtune/training/grpo_trainer.py:311-901`` and
``rwkvtune/training/grpo/lightning_module.py:534-1789``:

1. every prompt batch arrives ``steps_per_generation * num_iterations`` times; on the first arrival
   ``G`` completions per prompt are rolled out (:class:`GRPOBatchGenerator`), optionally post-processed,
   scored by the reward functions, rewards are all-gathered so that group / batch statistics see the
   whole job, advantages are computed and this rank keeps its slice;
2. old log-probabilities are taken with the current policy under ``no_grad``; rows are shuffled and
   split into ``steps_per_generation`` slices;
3. each training step consumes one slice: policy log-probs (with grad), reference log-probs when
   ``beta > 0`` (adapter disabled for LoRA, otherwise a frozen copy), optional ``loss_mask_func``,
   clipped objective, aggregation by ``loss_type``, AdamW with ``att.w0`` at twice the learning rate,
   warm-up + cosine schedule per optimiser step.

Log-probabilities never touch ``[n, L, V]`` logits: the hidden states of the completion positions are
gathered and go through the fused head + log-softmax + entropy operator.  Sequences are right-padded
(to a multiple of 16), so padding never enters a row's recurrent state.
"""
from __future__ import annotations

import copy
import json
import os
import time
from typing import Any, Callable, Dict, List, Optional, Sequence, Union

import torch

from .. import ops
from ..engine import EngineConfig, TrainEngine, grpo_lr_scale
from ..engine import checkpoint as ckpt
from ..engine.metrics import MetricLogger
from ..inference.grpo_batch_generator import GRPOBatchGenerator
from ..models import AutoModel
from ..parallel import init_distributed
from ..peft import get_peft_model, is_peft_model
from .callbacks import CallbackList
from .grpo.advantage import AdvantageCalculator
from .grpo.dataset import create_grpo_dataloader
from .grpo.loss import get_loss_function
from .grpo_config import GRPOConfig
from .model_save_utils import save_model_or_adapter

RewardFunc = Callable[..., Union[List[float], torch.Tensor]]


class GRPOTrainer:
    def __init__(self, model, reward_funcs: Union[RewardFunc, Sequence[RewardFunc]], args: Optional[GRPOConfig] = None,
                 train_dataset=None, eval_dataset=None, processing_class=None, callbacks=None, optimizers=None,
                 peft_config=None, loss_mask_func: Optional[Callable] = None,
                 completion_postprocess_fn: Optional[Callable] = None):
        self.args = args or GRPOConfig()
        if train_dataset is None:
            raise ValueError("train_dataset is required")
        self.train_dataset, self.eval_dataset = train_dataset, eval_dataset
        import warnings

        if eval_dataset is not None:   # accepted for signature parity; the reference stores it and never evaluates either
            warnings.warn("GRPOTrainer: eval_dataset is accepted but not used (no evaluation loop runs during GRPO)")
        if optimizers is not None and tuple(optimizers) != (None, None):
            warnings.warn("GRPOTrainer: `optimizers` is ignored; the engine builds its own sharded AdamW and schedule "
                          "from lr_init / lr_final / warmup_steps / weight_decay")
        if processing_class is None:    # as in the reference (grpo_trainer.py:540-549): the default RWKV vocabulary,
            from ..data.tokenizers import AutoTokenizer, get_tokenizer   # or the model directory's own tokenizer

            if isinstance(model, str) and os.path.exists(os.path.join(model, "tokenizer_config.json")):
                processing_class = AutoTokenizer.from_pretrained(model)
            else:
                processing_class = get_tokenizer()
        self.processing_class = self.tokenizer = processing_class
        self.callbacks = CallbackList(callbacks)
        self.loss_mask_func = loss_mask_func
        self.completion_postprocess_fn = completion_postprocess_fn
        self.reward_funcs = [reward_funcs] if callable(reward_funcs) else list(reward_funcs)
        if not self.reward_funcs:
            raise ValueError("at least one reward function is required")
        w = self.args.reward_weights
        if w is not None and len(w) != len(self.reward_funcs):
            raise ValueError(f"reward_weights has {len(w)} entries for {len(self.reward_funcs)} reward functions")
        self.reward_weights = list(w) if w is not None else [1.0] * len(self.reward_funcs)
        self.reward_names = [getattr(f, "__name__", f"reward_{i}") for i, f in enumerate(self.reward_funcs)]
        self.base_model_path = model if isinstance(model, str) else ""
        if isinstance(model, str):
            model = AutoModel.from_pretrained(model, device="cpu")
        if peft_config is not None and not is_peft_model(model):
            model = get_peft_model(model, peft_config)
        self.model = model
        self.args.use_lora = is_peft_model(model)
        self.ref_model = None
        for f in ("n_layer", "n_embd", "vocab_size", "head_size_a", "dim_att_lora", "dim_gate_lora", "dim_mv_lora",
                  "dim_att", "dim_ffn"):
            if hasattr(model.config, f):
                setattr(self.args, f, getattr(model.config, f))
        model.config.grad_cp = self.args.grad_cp
        model.config.ctx_len = max(getattr(model.config, "ctx_len", 0), self.args.ctx_len + 16)
        self.loss_fn = get_loss_function(self.args.loss_type, self.args)
        self.advantage = AdvantageCalculator(self.args.scale_rewards, self.args.num_generations, self.args.advantage_clip,
                                             self.args.low_reward_threshold, self.args.low_reward_scale)
        self.engine: Optional[TrainEngine] = None
        self.ctx = None
        self.buffer: List[Dict[str, torch.Tensor]] = []
        self.state = {"global_step": 0, "samples_seen": 0, "rollouts": 0}
        self.last_metrics: Dict[str, float] = {}

    # ------------------------------------------------------------------ log-probabilities
    def _hidden_at_completions(self, model, prompt_ids: List[List[int]], completion_ids: torch.Tensor):
        """Runs ``[prompt; completion[:-1]]`` (right-padded to a multiple of 16) and returns the hidden states
        that predict each completion token: ``[n, C, hidden]``."""
        dev = completion_ids.device
        n, C = completion_ids.shape
        plens = torch.tensor([len(p) for p in prompt_ids], device=dev)
        width = int(plens.max()) + max(C - 1, 0)
        width = (width + 15) // 16 * 16
        seq = torch.zeros(n, width, dtype=torch.long, device=dev)
        for i, p in enumerate(prompt_ids):
            seq[i, :len(p)] = torch.tensor(p, dtype=torch.long, device=dev)
        if C > 1:
            cols = plens[:, None] + torch.arange(C - 1, device=dev)[None, :]
            seq.scatter_(1, cols, completion_ids[:, :-1])
        x = model.forward_hidden(seq)
        pos = (plens[:, None] - 1 + torch.arange(C, device=dev)[None, :]).clamp(max=width - 1)
        return x.gather(1, pos[:, :, None].expand(n, C, x.shape[-1]))

    def _per_token_logps(self, model, prompt_ids, completion_ids, with_entropy: bool = False, batch_size: Optional[int] = None):
        n, C = completion_ids.shape
        bs = batch_size or self.args.logprob_batch_size or n
        lps, ents = [], []
        temp = self.args.temperature if self.args.temperature > 0 else 1.0
        for s in range(0, n, bs):
            h = self._hidden_at_completions(model, prompt_ids[s:s + bs], completion_ids[s:s + bs])
            m = h.shape[0]
            lp, ent = ops.linear_logprob_entropy(h.reshape(m * C, -1), model._head_weight(),
                                                 completion_ids[s:s + bs].reshape(-1), 1.0, with_entropy)
            lps.append(lp.reshape(m, C))
            if with_entropy:
                ents.append(ent.reshape(m, C))
        return torch.cat(lps), (torch.cat(ents) if with_entropy else None)

    def _reference_logps(self, prompt_ids, completion_ids):
        model = self.engine.model
        with torch.no_grad():
            if is_peft_model(model):
                model.disable_adapter()
                try:
                    lp, _ = self._per_token_logps(model, prompt_ids, completion_ids)
                finally:
                    model.enable_adapter()
                return lp
            if self.ref_model is None:
                return None
            return self._per_token_logps(self.ref_model, prompt_ids, completion_ids)[0]

    # ------------------------------------------------------------------ rollout
    def _compute_rewards(self, prompts: List[str], completions: List[str], extra: Dict[str, List[Any]]):
        per_func = []
        for f in self.reward_funcs:
            r = f(prompts=prompts, completions=completions, **extra)
            r = r.detach().float().cpu() if isinstance(r, torch.Tensor) else torch.tensor([float(x) for x in r])
            if r.numel() != len(completions):
                raise ValueError(f"reward function {getattr(f, '__name__', f)} returned {r.numel()} values for "
                                 f"{len(completions)} completions")
            per_func.append(r)
        per_func_t = torch.stack(per_func, dim=1)
        total = (per_func_t * torch.tensor(self.reward_weights)[None, :]).sum(1)
        return total, per_func_t

    def _postprocess(self, prompts, completions, comp_ids, masks, extra):
        """Hook between rollout and rewards (``rwkvtune/training/grpo/lightning_module.py:876-905``): called with
        ``prompts, completions, completion_ids [B*G, C], masks [B*G, C], tokenizer`` and the extra dataset columns as
        keywords; returns a dict with ``completions``, ``completion_ids`` and ``masks`` of the same shapes (the hook
        re-encodes what it edits).  The edited ids are what the policy is trained on."""
        result = self.completion_postprocess_fn(prompts=prompts, completions=list(completions), completion_ids=comp_ids,
                                                masks=masks, tokenizer=self.processing_class, **extra)
        if not isinstance(result, dict):
            raise TypeError("completion_postprocess_fn must return a dict with keys 'completions', 'completion_ids', "
                            f"'masks'; got {type(result).__name__}")
        for key in ("completions", "completion_ids", "masks"):
            if key not in result:
                raise KeyError(f"completion_postprocess_fn result lacks {key!r}; got {sorted(result)}")
        new_text = list(result["completions"])
        new_ids = torch.as_tensor(result["completion_ids"]).to(device=comp_ids.device, dtype=comp_ids.dtype)
        new_masks = torch.as_tensor(result["masks"]).to(device=masks.device, dtype=masks.dtype)
        if len(new_text) != len(prompts) or new_ids.shape != comp_ids.shape or new_masks.shape != masks.shape:
            raise ValueError(f"completion_postprocess_fn must keep {len(prompts)} completions and the shape "
                             f"{tuple(comp_ids.shape)}; got {len(new_text)}, {tuple(new_ids.shape)}, "
                             f"{tuple(new_masks.shape)}")
        return new_text, new_ids, new_masks

    def _generate_and_buffer(self, batch: Dict[str, Any]) -> None:
        a, ctx, eng = self.args, self.ctx, self.engine
        G = a.num_generations
        prompts_ids = [list(p)[-a.max_prompt_length:] for p in batch["input_ids"]]
        phases = eng.phases
        t0 = time.perf_counter()
        with phases.phase("rollout"):
            out = self.generator.generate(prompts_ids, max_new_tokens=a.max_completion_length, num_generations=G,
                                          temperature=a.temperature, top_p=a.top_p, top_k=a.top_k,
                                          repetition_penalty=a.repetition_penalty, logit_bias=a.logit_bias)
        t_roll = time.perf_counter() - t0
        completions, comp_ids, masks = out["completions"], out["completion_ids"], out["masks"]
        prompts_rep = [p for p in batch["prompts"] for _ in range(G)]
        ids_rep = [p for p in prompts_ids for _ in range(G)]
        extra = {k: [v for v in vals for _ in range(G)] for k, vals in batch.items() if k not in ("prompts", "input_ids")}
        if self.completion_postprocess_fn is not None:
            completions, comp_ids, masks = self._postprocess(prompts_rep, completions, comp_ids, masks, extra)
        with phases.phase("rewards"):
            rewards, per_func = self._compute_rewards(prompts_rep, completions, extra)
        rewards, per_func = rewards.to(ctx.device), per_func.to(ctx.device)
        n_local = rewards.numel()
        if ctx.world_size > 1:
            import torch.distributed as dist

            counts = [torch.zeros(1, dtype=torch.long, device=ctx.device) for _ in range(ctx.world_size)]
            dist.all_gather(counts, torch.tensor([n_local], device=ctx.device))
            if len({int(c) for c in counts}) != 1:
                raise RuntimeError(f"ranks produced different numbers of rewards: {[int(c) for c in counts]}")
            gathered = [torch.zeros_like(rewards) for _ in range(ctx.world_size)]
            dist.all_gather(gathered, rewards)
            all_rewards = torch.cat(gathered)
            # the per-function columns too, so that the logged train/rewards/<func>/* describe the whole job
            # (rwkvtune/training/grpo/lightning_module.py:980-988 gathers both)
            gathered_pf = [torch.zeros_like(per_func) for _ in range(ctx.world_size)]
            dist.all_gather(gathered_pf, per_func.contiguous())
            all_per_func = torch.cat(gathered_pf)
        else:
            all_rewards, all_per_func = rewards, per_func
        adv_all = self.advantage.compute_advantages(all_rewards)
        adv = adv_all[ctx.rank * n_local:(ctx.rank + 1) * n_local]
        if comp_ids.shape[1] == 0:
            comp_ids = torch.zeros(n_local, 1, dtype=torch.long, device=ctx.device)
            masks = torch.zeros(n_local, 1, dtype=torch.bool, device=ctx.device)
        with torch.no_grad(), phases.phase("old_logps"):
            old_logps, _ = self._per_token_logps(eng.model, ids_rep, comp_ids)
        order = torch.randperm(n_local, device=ctx.device) if a.shuffle_buffer else torch.arange(n_local, device=ctx.device)
        S = a.steps_per_generation
        per = n_local // S
        self.buffer = []
        for s in range(S):
            sel = order[s * per:(s + 1) * per]
            self.buffer.append({"prompt_ids": [ids_rep[i] for i in sel.tolist()], "completion_ids": comp_ids[sel],
                                "mask": masks[sel].float(), "advantages": adv[sel], "old_logps": old_logps[sel],
                                "prompts": [prompts_rep[i] for i in sel.tolist()],
                                "completions": [completions[i] for i in sel.tolist()]})
        lengths = masks.sum(1).float()
        self.rollout_stats = {"train/reward/mean": float(all_rewards.mean()), "train/reward/std": float(all_rewards.std(unbiased=False)),
                              "train/reward/min": float(all_rewards.min()), "train/reward/max": float(all_rewards.max()),
                              "completions/mean_length": float(lengths.mean()), "completions/min_length": float(lengths.min()),
                              "completions/max_length": float(lengths.max()), "rollout/seconds": t_roll,
                              "rollout/tokens_per_sec": float(lengths.sum()) / max(t_roll, 1e-9),
                              "mean_advantage": float(adv.mean()),
                              "phase/prefill/seconds": float(self.generator.last_stats.get("prefill_s", 0.0)),
                              "phase/decode/seconds": float(self.generator.last_stats.get("decode_s", 0.0))}
        for j, name in enumerate(self.reward_names):
            col = all_per_func[:, j]
            self.rollout_stats.update({f"train/rewards/{name}/mean": float(col.mean()), f"train/rewards/{name}/std": float(col.std(unbiased=False)),
                                       f"train/rewards/{name}/min": float(col.min()), f"train/rewards/{name}/max": float(col.max())})
        self.state["rollouts"] += 1
        if a.save_rollout_steps > 0 and ctx.is_main and self.state["rollouts"] % a.save_rollout_steps == 0:
            self._save_rollout(prompts_rep, completions, rewards, adv, comp_ids, masks, per_func, extra)
        ctx.barrier()

    def _save_rollout(self, prompts, completions, rewards, adv, comp_ids, masks, per_func, extra) -> None:
        os.makedirs(self.args.save_rollout_path, exist_ok=True)
        path = os.path.join(self.args.save_rollout_path, f"rollout_step_{self.state['global_step']}.jsonl")
        with open(path, "w", encoding="utf-8") as fh:
            for i in range(len(prompts)):
                n = int(masks[i].sum())
                rec = {"step": self.state["global_step"], "index": i, "prompt": prompts[i], "completion": completions[i],
                       "reward": float(rewards[i]), "advantage": float(adv[i]), "completion_ids": comp_ids[i, :n].tolist(),
                       "rewards_per_func": {nm: float(per_func[i, j]) for j, nm in enumerate(self.reward_names)}}
                for k, v in extra.items():
                    try:
                        json.dumps(v[i])
                        rec[k] = v[i]
                    except TypeError:
                        rec[k] = str(v[i])
                fh.write(json.dumps(rec, ensure_ascii=False) + "\n")

    # ------------------------------------------------------------------ training step
    def _training_step(self, data: Dict[str, Any], lr: float) -> Dict[str, float]:
        a, eng = self.args, self.engine
        model = eng.model
        comp, mask, adv, old = data["completion_ids"], data["mask"], data["advantages"], data["old_logps"]
        policy, ent = self._per_token_logps(model, data["prompt_ids"], comp, with_entropy=a.log_entropy)
        if not policy.requires_grad:
            raise RuntimeError("policy log-probabilities carry no gradient (no trainable parameters on the path)")
        ref = self._reference_logps(data["prompt_ids"], comp) if a.beta > 0 else None
        if self.loss_mask_func is not None:
            custom = self.loss_mask_func(prompts=data["prompts"], completions=data["completions"], completion_ids=comp,
                                         tokenizer=self.processing_class)
            custom = torch.as_tensor(custom, dtype=mask.dtype, device=mask.device)
            if custom.shape == mask.shape and float((custom * mask).sum()) > 0:
                mask = mask * custom
        per_tok = self.loss_fn.compute_per_token_loss(policy, ref, old, adv, mask, a.beta)
        loss = self.loss_fn.compute_loss(per_tok, mask)
        stepped = eng.backward_and_step(loss, lr)
        with torch.no_grad():
            denom = mask.sum().clamp(min=1.0)
            ratio = self.loss_fn.importance_ratio(policy.detach(), old, mask).expand_as(mask)
            low = ((ratio < 1 - a.epsilon) & (adv[:, None] < 0)).float()
            high = ((ratio > 1 + a.epsilon_high) & (adv[:, None] > 0)).float()
            metrics = {"train_loss": float(loss.detach()), "clip_ratio/low_mean": float((low * mask).sum() / denom),
                       "clip_ratio/high_mean": float((high * mask).sum() / denom),
                       "clip_ratio/region_mean": float(((low + high) * mask).sum() / denom), "lr": lr,
                       "optimizer_stepped": float(stepped)}
            metrics["clip_ratio"] = metrics["clip_ratio/region_mean"]
            if ref is not None:
                d = ref - policy.detach()
                metrics["kl_div"] = float(((torch.exp(d) - d - 1) * mask).sum() / denom)
            if ent is not None:
                metrics["entropy"] = float((ent.detach() * mask).sum() / denom)
        return metrics

    # ------------------------------------------------------------------ main loop
    def train(self) -> None:
        a = self.args
        launched = int(os.environ.get("WORLD_SIZE", "1")) > 1
        if a.devices > 1 and not launched and a.accelerator != "cpu":
            import torch.multiprocessing as mp

            from .trainer_base import _spawn_entry

            mp.start_processes(_spawn_entry, args=(self, 29500 + os.getpid() % 2000), nprocs=a.devices, join=True,
                               start_method="spawn")
            return
        self._train_worker()

    def _train_worker(self) -> None:
        a = self.args
        ctx = self.ctx = init_distributed("cpu" if a.accelerator == "cpu" else "gpu")
        if a.seed >= 0:
            torch.manual_seed(a.seed + ctx.rank)
        if a.beta > 0 and not is_peft_model(self.model):
            src = AutoModel.from_pretrained(a.ref_model_path, device="cpu") if a.ref_model_path else copy.deepcopy(self.model)
            self.ref_model = src
        cfg = EngineConfig(lr_init=a.lr_init, beta1=a.beta1, beta2=a.beta2, adam_eps=a.adam_eps, weight_decay=a.weight_decay,
                           grad_clip=a.grad_clip, accumulate_grad_batches=a.accumulate_grad_batches, strategy=a.strategy,
                           precision=a.precision if a.accelerator != "cpu" else "fp32", grad_cp=a.grad_cp,
                           lr_2x_patterns=("att.w0",), transport=os.environ.get("RWKVTUNE_TRANSPORT", "auto"),
                           cuda_graph=os.environ.get("RWKVTUNE_CUDA_GRAPH", "0") == "1")
        self.engine = eng = TrainEngine(self.model, cfg, ctx)
        self.model = eng.model
        if self.ref_model is not None:
            self.ref_model = self.ref_model.to(device=ctx.device, dtype=eng.model.dtype).eval()
            for p in self.ref_model.parameters():
                p.requires_grad_(False)
        self.generator = GRPOBatchGenerator(eng.model, self.processing_class, ctx.device,
                                            prefill_chunk_size=a.prefill_chunk_size,
                                            max_prefill_batch_size=a.max_prefill_batch_size,
                                            max_decode_batch_size=a.max_decode_batch_size)
        loader = create_grpo_dataloader(self.train_dataset, a.micro_bsz, a.generate_every, True, max(a.seed, 0), ctx.rank,
                                        ctx.world_size, a.num_workers)
        epoch_steps = a.epoch_steps if a.epoch_steps is not None else len(loader)
        total_steps = a.epoch_count * epoch_steps
        total_opt = max(1, total_steps // a.accumulate_grad_batches)
        logger = MetricLogger(a.proj_dir, a.report_to or "", a.run_name or "", ctx.is_main, "grpo_loss_data.jsonl",
                              "grpo_train_log.txt", vars(a))
        self._maybe_resume()
        from ..engine.profiling import StepProfiler, profile_steps_requested

        profiler = StepProfiler(profile_steps_requested(a), a.proj_dir, is_main=ctx.is_main)
        done = False
        self.callbacks.fire("on_train_start", self)
        for epoch in range(a.epoch_count):
            loader.sampler.set_epoch(epoch)
            for b, batch in enumerate(loader):
                if b >= epoch_steps or self.state["global_step"] >= total_steps:
                    done = self.state["global_step"] >= total_steps
                    break
                step = self.state["global_step"]
                if step % a.generate_every == 0 or not self.buffer:
                    self._generate_and_buffer(batch)
                data = self.buffer[(step % a.generate_every) % len(self.buffer)]
                lr = a.lr_init * grpo_lr_scale(eng.optimizer_steps, a.lr_init, a.lr_final, a.warmup_steps, total_opt,
                                               a.accumulate_grad_batches)
                t0 = time.perf_counter()
                self.callbacks.fire("on_train_batch_start", self, batch, b)
                profiler.step_begin()
                with eng.phases.phase("policy_step"):
                    metrics = self._training_step(data, lr)
                profiler.step_end()
                eng.check_health()
                metrics.update(self.rollout_stats)
                metrics.update(eng.phases.scalars())
                self.state["global_step"] += 1
                self.state["samples_seen"] += a.micro_bsz * ctx.world_size
                self.last_metrics = metrics
                if ctx.world_size > 1:
                    t = torch.tensor([metrics["train_loss"]], device=ctx.device)
                    torch.distributed.all_reduce(t)
                    metrics["train_loss"] = float(t) / ctx.world_size
                tokens = int(data["mask"].sum()) * ctx.world_size
                logger.log_step(self.state["global_step"], metrics["train_loss"], lr, tokens, time.perf_counter() - t0,
                                {k: v for k, v in metrics.items() if k != "train_loss"})
                if ctx.is_main and self.state["global_step"] % max(1, a.log_steps) == 0:
                    print(f"step {self.state['global_step']}/{total_steps} loss {metrics['train_loss']:.5f} "
                          f"reward {metrics['train/reward/mean']:.4f} len {metrics['completions/mean_length']:.1f} "
                          f"lr {lr:.2e}", flush=True)
                self.callbacks.fire("on_train_batch_end", self, {"loss": metrics["train_loss"], **metrics}, batch, b)
                self.callbacks.fire("on_step_end", self, metrics)
                if a.save_every_n_batches > 0 and self.state["global_step"] % a.save_every_n_batches == 0:
                    self._save_checkpoint(f"rwkv7-batch{self.state['global_step']}")
            self.callbacks.fire("on_train_epoch_end", self, epoch)
            if done:
                break
        self._save_checkpoint(f"checkpoint_epoch_{a.epoch_count}")
        self.callbacks.fire("on_train_end", self)
        logger.close()
        ctx.barrier()

    # ------------------------------------------------------------------ checkpoints
    def _save_checkpoint(self, name: str) -> None:
        a, ctx, eng = self.args, self.ctx, self.engine
        final = os.path.join(a.proj_dir, name)
        meta = {"samples_seen": self.state["samples_seen"], "devices": ctx.world_size, "micro_bsz": a.micro_bsz,
                "accumulate_grad_batches": a.accumulate_grad_batches, "grpo_generate_every": a.generate_every,
                "global_step": self.state["global_step"], "trainer": "grpo"}

        def write(tmp: str) -> None:
            if ctx.is_main:
                save_model_or_adapter(eng.model, tmp, self.processing_class, a.lora_save_mode, self.base_model_path)
            ckpt.save_trainer_state(tmp, eng, ctx, meta, a.save_optimizer_state)

        ckpt.atomic_checkpoint(final, ctx, write)
        if ctx.is_main and a.save_total_limit > 0:
            ckpt.rotate_checkpoints(a.proj_dir, a.save_total_limit, "rwkv7-batch*")
        self.callbacks.fire("on_save_checkpoint", self, final)

    def _maybe_resume(self) -> None:
        a, ctx, eng = self.args, self.ctx, self.engine
        if not a.resume_from_checkpoint:
            return
        found = ckpt.find_checkpoint(a.resume_from_checkpoint)
        if found is None:
            raise FileNotFoundError(f"no checkpoint found at {a.resume_from_checkpoint}")
        from .trainer_base import SupervisedTrainer

        SupervisedTrainer._load_weights(self, found)
        meta = ckpt.read_meta(found) if os.path.isdir(found) else {}
        if not (os.path.isdir(found) and ckpt.load_optimizer_state(found, eng, ctx)):
            eng.opt.master.copy_(eng.space.params[eng.opt.lo:eng.opt.hi].float())
        self.state["samples_seen"] = int(meta.get("samples_seen", 0))
        self.state["global_step"] = int(meta.get("global_step", 0))

    def save_model(self, output_dir: Optional[str] = None) -> str:
        out = output_dir or os.path.join(self.args.proj_dir, "final")
        if self.ctx is None or self.ctx.is_main:
            save_model_or_adapter(self.model, out, self.processing_class, self.args.lora_save_mode,
                                              self.base_model_path)
        return out
