"""``grpo_trainer`` (alias ``rl_trainer``): group-relative policy optimisation for the packed
decoders.

The reference registers no RL trainer; its RL surface is the flow-GRPO loss inside the Bagel
model driven by an external loop (src/lmms_engine/models/bagel/bagel.py:1046-1360) and a
preference-data schema (src/lmms_engine/protocol/data_proto.py:63-67).  This trainer makes the
loop first class: for every prompt it samples a group of completions from the current policy,
scores them with a registered reward function, normalises rewards inside the group, and
optimises the clipped-ratio objective with a k3 KL penalty to a frozen reference copy.  All
sequences of a step are evaluated as ONE packed varlen batch.

``trainer_args.rl_config``: ``group_size`` (8), ``max_new_tokens`` (64), ``temperature`` (1.0),
``clip_range`` (0.2), ``beta`` (0.04), ``num_iterations`` (1), ``reward`` (registered name or
``module:function``), ``eos_token_id``.
"""
from __future__ import annotations

import copy
import importlib
from typing import Any, Callable, Dict, List, Optional, Sequence

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ...ops import cross_entropy as ce_ops
from ...utils.logging_utils import logger
from ..fsdp2.fsdp2_trainer import FSDP2SFTTrainer
from ..registry import TRAINER_REGISTER

REWARD_FUNCTIONS: Dict[str, Callable[[torch.Tensor, torch.Tensor], float]] = {}


def register_reward(name: str):
    def deco(fn):
        REWARD_FUNCTIONS[name] = fn
        return fn

    return deco


@register_reward("length")
def _reward_length(prompt: torch.Tensor, completion: torch.Tensor) -> float:
    return -abs(int(completion.numel()) - 16) / 16.0


@register_reward("repeat_last_prompt_token")
def _reward_repeat(prompt: torch.Tensor, completion: torch.Tensor) -> float:
    if completion.numel() == 0:
        return 0.0
    return float((completion == prompt[-1]).float().mean())


def resolve_reward(spec) -> Callable:
    if callable(spec):
        return spec
    if spec in REWARD_FUNCTIONS:
        return REWARD_FUNCTIONS[spec]
    if isinstance(spec, str) and ":" in spec:
        mod, fn = spec.split(":", 1)
        return getattr(importlib.import_module(mod), fn)
    raise KeyError(f"unknown reward '{spec}'; registered: {sorted(REWARD_FUNCTIONS)}")


def group_advantages(rewards: torch.Tensor, group_size: int, eps: float = 1e-4) -> torch.Tensor:
    r = rewards.view(-1, group_size)
    return ((r - r.mean(1, keepdim=True)) / (r.std(1, keepdim=True, unbiased=False) + eps)).view(-1)


def grpo_token_loss(logp, old_logp, ref_logp, adv_tok, mask, clip_range: float, beta: float):
    """Token-level clipped surrogate + k3 KL estimate, averaged over completion tokens."""
    ratio = torch.exp(logp - old_logp)
    surr = torch.minimum(ratio * adv_tok, torch.clamp(ratio, 1 - clip_range, 1 + clip_range) * adv_tok)
    loss = -surr
    kl = None
    if beta > 0 and ref_logp is not None:
        d = ref_logp - logp
        kl = torch.exp(d) - d - 1
        loss = loss + beta * kl
    n = mask.sum().clamp(min=1.0)
    return (loss * mask).sum() / n, ((kl * mask).sum() / n).detach() if kl is not None else None


@torch.no_grad()
def sample_completions(model, prompts: Sequence[torch.Tensor], max_new_tokens: int, temperature: float,
                       eos_token_id: Optional[int], generator=None, sync_group=None, token_group=None,
                       use_cache: Optional[bool] = None) -> List[torch.Tensor]:
    """Ancestral sampling for a list of prompts, all sequences advanced together as one packed batch per step.

    ``use_cache`` (default: when the model supports it and is not sequence-parallel): the prompts are run once and
    every later step feeds ONE token per sequence against the cached keys / values (``models/kv_cache.py``); otherwise
    every step re-runs the whole sequences.  Both draw the same tokens from the same generator state.
    ``sync_group``: ranks whose forward passes contain collectives (sharded parameters, sequence
    parallelism).  They must run the same number of forwards, so the loop ends only when NO rank of
    the group has an unfinished sequence, and a rank that is done keeps forwarding its (finished)
    batch; tokens sampled for a finished sequence are dropped.
    ``token_group``: ranks that hold the SAME prompts (a sequence-parallel group).  The tokens drawn
    by its first rank are broadcast, so that all of them continue the same text."""
    from ...models.kv_cache import PackedKVCache

    dev = prompts[0].device
    seqs = [p.clone() for p in prompts]
    done = [False] * len(seqs)
    inner = getattr(model, "module", model)
    if use_cache is None:
        use_cache = bool(getattr(inner, "supports_kv_cache", False)) and token_group is None and getattr(inner, "sp_group", None) is None
    cache = None
    if use_cache:
        n_layers = len(inner.model.layers)
        cache = PackedKVCache(n_layers, [p.numel() + max_new_tokens for p in prompts], device=dev)
    fed = [0] * len(seqs)  # tokens of every sequence that the cache holds
    head = inner.lm_head.weight.detach()
    if hasattr(head, "full_tensor"):  # held in shards by a wrapper outside the forward pass: gather once per rollout
        head = head.full_tensor()
    for _ in range(max_new_tokens):
        live = [i for i, d in enumerate(done) if not d]
        if sync_group is not None:
            flag = torch.tensor([1 if live else 0], dtype=torch.int32, device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=sync_group)
            if int(flag) == 0:
                break
            live = list(range(len(seqs)))  # same shapes of work on every rank
        elif not live:
            break
        if cache is not None:
            # a finished sequence that must keep running (sync_group) re-feeds its last token without growing
            new = [seqs[i][fed[i]:] if seqs[i].numel() > fed[i] else seqs[i][-1:] for i in live]
            counts = [0] * len(seqs)
            for i, t in zip(live, new):
                counts[i] = t.numel()
            for i in live:
                if seqs[i].numel() == fed[i]:  # nothing new: overwrite the last row instead of appending
                    cache.lens[i] -= 1
                    fed[i] -= 1
            pos = cache.advance(counts)
            for i in live:
                fed[i] += counts[i]
            ids = torch.cat(new)
            lens = torch.tensor([t.numel() for t in new], dtype=torch.int32, device=dev)
            cu = F.pad(torch.cumsum(lens, 0, dtype=torch.int32), (1, 0))
            hidden = model(input_ids=ids, cu_seqlens=cu, position_ids=pos, kv_cache=cache)["hidden_states"]
        else:
            ids = torch.cat([seqs[i] for i in live])
            lens = torch.tensor([seqs[i].numel() for i in live], dtype=torch.int32, device=dev)
            cu = F.pad(torch.cumsum(lens, 0, dtype=torch.int32), (1, 0))
            hidden = model(input_ids=ids, cu_seqlens=cu)["hidden_states"]
        last = hidden.index_select(0, (cu[1:] - 1).long())
        logits = F.linear(last, head).float() / max(temperature, 1e-5)
        nxt = torch.multinomial(torch.softmax(logits, -1), 1, generator=generator).flatten()
        if token_group is not None:
            dist.broadcast(nxt, src=dist.get_global_rank(token_group, 0), group=token_group)
        for j, i in enumerate(live):
            if done[i]:
                continue
            seqs[i] = torch.cat([seqs[i], nxt[j:j + 1]])
            if eos_token_id is not None and int(nxt[j]) == eos_token_id:
                done[i] = True
    return [s[p.numel():] for s, p in zip(seqs, prompts)]


def packed_logprobs(model, ids: torch.Tensor, cu: torch.Tensor) -> torch.Tensor:
    """log p(token_t | prefix) for every position (0 at each document's first token)."""
    from ...models.decoder_lm import IGNORE_INDEX, shift_labels_per_document

    shifted = shift_labels_per_document(ids, cu)
    inner = getattr(model, "module", model)
    if getattr(inner, "sp_group", None) is None and getattr(inner, "tp_group", None) is None and hasattr(inner, "loss_reduction"):
        # the head runs inside the forward pass, where a sharding wrapper has gathered its weight and will reduce its gradient
        keep, inner.loss_reduction = inner.loss_reduction, "none"
        try:
            nll = model(input_ids=ids, labels=ids, cu_seqlens=cu)["loss"]
        finally:
            inner.loss_reduction = keep
    else:
        hidden = model(input_ids=ids, cu_seqlens=cu)["hidden_states"]
        nll = ce_ops.fused_linear_cross_entropy(hidden, model.lm_head.weight, shifted, "none")
    # position t holds -log p(ids[t+1]); move it onto the token it scores
    out = torch.zeros_like(nll)
    out[1:] = -nll[:-1]
    out = out.masked_fill(torch.roll(shifted, 1, 0) == IGNORE_INDEX, 0.0)
    out[0] = 0.0
    return out


@TRAINER_REGISTER.register("grpo_trainer")
class GRPOTrainer(FSDP2SFTTrainer):
    def __init__(self, *a, **k):
        super().__init__(*a, **k)
        cfg = dict(self.args.rl_config or {})
        self.group_size = int(cfg.get("group_size", 8))
        self.max_new_tokens = int(cfg.get("max_new_tokens", 64))
        self.temperature = float(cfg.get("temperature", 1.0))
        clip = cfg.get("clip_range", 0.2)
        self.clip_range = float(clip[0] if isinstance(clip, (list, tuple)) else clip)
        self.beta = float(cfg.get("beta", 0.04))
        self.num_iterations = int(cfg.get("num_iterations", 1))
        self.eos_token_id = cfg.get("eos_token_id")
        self.reward_fn = resolve_reward(cfg.get("reward", "length"))
        self.ref_model = None
        self.enable_perf_metrics = False
        self.rl_metrics: Dict[str, float] = {}
        if self.num_iterations > 1 and max(int(self.args.gradient_accumulation_steps or 1), 1) > 1:
            raise ValueError("rl_config.num_iterations > 1 updates the policy several times per batch and cannot be "
                             "combined with gradient_accumulation_steps > 1")

    def prepare_model(self):
        twin = copy.deepcopy(self.model) if self.beta > 0 else None  # before a sharding wrapper is applied
        super().prepare_model()
        if twin is not None:
            self.ref_model = self.prepare_frozen_twin(twin)

    def prompts_of(self, batch) -> List[torch.Tensor]:
        ids, cu = batch["input_ids"], batch["cu_seqlens"].tolist()
        labels = batch.get("labels")
        out = []
        for a, b in zip(cu[:-1], cu[1:]):
            p = ids[a:b]
            if labels is not None:  # the prompt is the unsupervised prefix
                sup = (labels[a:b] != -100).nonzero()
                if sup.numel():
                    p = p[: int(sup[0])]
            out.append(p)
        return out

    def training_step(self, batch, do_step):
        model = self.model
        prompts = [p for p in self.prompts_of(batch) for _ in range(self.group_size)]
        model.eval()
        sync_group = token_group = None
        if self.world_size > 1 and dist.is_initialized():
            if self.sp_size > 1 and self.pgm is not None:
                token_group = self.pgm.cp_group
                sync_group = self.pgm.cp_group
            if getattr(self, "runtime_kind", "native") != "native":
                sync_group = dist.group.WORLD  # sharded parameters: every forward gathers them
        completions = sample_completions(model, prompts, self.max_new_tokens, self.temperature, self.eos_token_id,
                                         sync_group=sync_group, token_group=token_group)
        rewards = torch.tensor([self.reward_fn(p, c) for p, c in zip(prompts, completions)], dtype=torch.float32, device=self.device)
        adv = group_advantages(rewards, self.group_size)
        ids = torch.cat([torch.cat([p, c]) for p, c in zip(prompts, completions)])
        lens = torch.tensor([p.numel() + c.numel() for p, c in zip(prompts, completions)], dtype=torch.int32, device=self.device)
        cu = F.pad(torch.cumsum(lens, 0, dtype=torch.int32), (1, 0))
        mask = torch.cat([torch.cat([torch.zeros(p.numel()), torch.ones(c.numel())]) for p, c in zip(prompts, completions)]).to(self.device)
        adv_tok = torch.repeat_interleave(adv, lens.long())
        with torch.no_grad():
            old_logp = packed_logprobs(model, ids, cu)
            ref_logp = packed_logprobs(self.ref_model, ids, cu) if self.ref_model is not None else None
        model.train()
        loss = None
        grad_norm = None
        ga = max(int(self.args.gradient_accumulation_steps or 1), 1)
        for _ in range(self.num_iterations):
            logp = packed_logprobs(model, ids, cu)
            loss, kl = grpo_token_loss(logp, old_logp, ref_logp, adv_tok, mask, self.clip_range, self.beta)
            (loss / ga).backward()
            self.accumulated_grad_steps += 1
            # with accumulation the optimizer moves once per ``gradient_accumulation_steps`` batches, in step
            # with ``global_step`` and the schedule; without it, once per policy iteration
            if do_step:
                self.lr_factor = self.current_lr_factor(self.global_step)
                grad_norm = self.runtime.step(self.lr_factor) if self.runtime is not None else self._torch_step()
                self.accumulated_grad_steps = 0
        self.rl_metrics = {"rl/reward_mean": float(rewards.mean()), "rl/reward_std": float(rewards.std(unbiased=False)),
                           "rl/completion_len": float(mask.sum() / max(len(prompts), 1)),
                           "rl/kl": float(kl) if kl is not None else 0.0}
        return loss.detach(), grad_norm

    def _torch_step(self):
        from ...utils.fsdp2_utils import fsdp2_clip_grad_norm_

        gn = fsdp2_clip_grad_norm_(self.model.parameters(), self.args.max_grad_norm)
        for g in self.optimizer.param_groups:
            g["lr"] = g["initial_lr"] * self.lr_factor
        self.optimizer.step()
        self.optimizer.zero_grad(set_to_none=True)
        return gn

    def extra_metrics(self):
        return dict(self.rl_metrics)


TRAINER_REGISTER.register("rl_trainer")(GRPOTrainer)
