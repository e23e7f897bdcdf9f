"""Reinforcement-learning trainers: GRPO, PPO, DPO, RLVR, the Bradley-Terry reward model, the rollout
worker / buffer and the RLHF pipeline that strings them together.

GRPO follows the reference's public behaviour (src/trainer/trainer_rl.cpp:1129-1350): a group of G
completions per prompt (default 8, at most 32 new tokens when sampled internally), advantages
``(r - mean) / sqrt(var + 1e-8)``, loss ``(1/G) * sum_i adv_i * CE_i`` on the completion tokens, ``beta``
as a gradient damping ``(1 - 0.01 * beta)``; zero-variance rewards make the step a no-op.  Log-probs
use correctly shifted targets (the reference feeds labels == inputs).  Optional and off by default:
PPO-style ratio clipping (``clip_eps``) and a KL penalty against a frozen reference model
(``kl_coef``).  Rollouts come from the paged-KV inference engine.

PPO: clip 0.2, GAE gamma .99 lambda .95, adaptive KL (trainer_rl.cpp:557-1127).  DPO: beta .1.  RLVR:
verifiable (substring / exact-match) rewards (trainer_rl.cpp:1352-1433).  RewardModel: Bradley-Terry
pairwise loss on a scalar head (src/trainer/reward.cpp).  RolloutWorker: deterministic,
sequence-numbered buffer (src/trainer/rollout_worker.cpp, include/quant/rollout_worker.h:27-80).
"""
from __future__ import annotations

import copy
import math
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

import torch
import torch.nn.functional as TF

from .fused_optim import FlatAdamW


def collect_params(model):
    """Every trainable tensor of a dense or MoE model (reference: GRPO collects Dense + MoE params)."""
    return [p for p in model.parameters() if p.requires_grad]


def token_logprobs(model, ids):
    """log p(ids[:, t+1] | ids[:, :t+1]) for t = 0..S-2 -> [B, S-1] (graph attached)."""
    logits = model(ids).float()
    lp = torch.log_softmax(logits[:, :-1], -1)
    return lp.gather(-1, ids[:, 1:].unsqueeze(-1)).squeeze(-1)


class _RLBase:
    def __init__(self, model, tokenizer=None, lr=1e-5, weight_decay=0.0, max_grad_norm=1.0):
        self.model, self.tok = model, tokenizer
        self.flat = model.flatten()
        self.opt = FlatAdamW(self.flat, lr=lr, betas=(0.9, 0.999), weight_decay=weight_decay, max_grad_norm=max_grad_norm)
        self.steps = 0

    def _backward_and_step(self, loss, grad_scale=1.0):
        loss.backward()
        for p in self.flat.params_list:      # tensors that went through plain autograd
            if p.grad is not None:
                p.main_grad.add_(p.grad.float())
                p.grad = None
        if grad_scale != 1.0:
            self.flat.grads.mul_(grad_scale)
        self.opt.step()
        self.steps += 1

    def generate(self, prompt_ids: List[int], n: int, max_new: int, temperature=1.0, top_k=0, top_p=1.0, seed=0):
        """n sampled completions of one prompt through the inference engine."""
        from ..inference.engine import EngineConfig, InferenceEngine
        from ..inference.sampler import SamplerConfig
        eng = InferenceEngine(self.model, self.tok, EngineConfig(max_batch=max(1, n), num_pages=max(64, n * 8),
                                                                 enable_prefix_cache=True, seed=seed + self.steps))
        sc = SamplerConfig(temperature=temperature, top_k=top_k, top_p=top_p)
        return eng.generate_batch([list(prompt_ids)] * n, max_new, sc)


# ------------------------------------------------------------------------------------------------
# GRPO
# ------------------------------------------------------------------------------------------------
def default_reward(text_ids: Sequence[int]) -> float:
    """Heuristic used when no reward function is given: favour longer, less repetitive completions."""
    if not text_ids:
        return 0.0
    return len(set(text_ids)) / len(text_ids) + 0.01 * len(text_ids)


class GRPOTrainer(_RLBase):
    def __init__(self, model, tokenizer=None, group_size=8, beta=0.04, lr=1e-5, clip_eps=0.0, kl_coef=0.0,
                 reward_fn: Optional[Callable] = None, max_new_tokens=32):
        super().__init__(model, tokenizer, lr=lr)
        self.G, self.beta, self.clip_eps, self.kl_coef = group_size, beta, clip_eps, kl_coef
        self.reward_fn = reward_fn or default_reward
        self.max_new = max_new_tokens
        self.ref_model = copy.deepcopy(model).eval() if kl_coef > 0 else None
        self.last_advantages = None

    @staticmethod
    def advantages(rewards: torch.Tensor) -> torch.Tensor:
        r = rewards.float()
        return (r - r.mean()) / torch.sqrt(r.var(unbiased=False) + 1e-8)

    def train_step(self, ids=None, mask=None, rewards=None, prompt: Optional[List[int]] = None):
        """Either (ids [G, S], mask [G, S] marking completion tokens, rewards [G]) or ``prompt`` (token ids):
        the group is then sampled and scored here.  Returns the loss value (0.0 for a no-op step)."""
        dev = self.model.tok_embeddings.device
        if prompt is not None:
            outs = self.generate(prompt, self.G, self.max_new, temperature=1.0)
            S = len(prompt) + max(len(o) for o in outs)
            ids = torch.zeros((self.G, S), dtype=torch.long)
            mask = torch.zeros((self.G, S))
            for i, o in enumerate(outs):
                seq = list(prompt) + o
                ids[i, :len(seq)] = torch.tensor(seq)
                mask[i, len(prompt):len(seq)] = 1
            rewards = torch.tensor([self.reward_fn(o) for o in outs])
        ids, mask, rewards = ids.to(dev), mask.to(dev).float(), rewards.to(dev).float()
        adv = self.advantages(rewards)
        self.last_advantages = adv
        if float(rewards.var(unbiased=False)) < 1e-12:
            return 0.0                                    # zero-variance group: no update
        lp = token_logprobs(self.model, ids)              # [G, S-1]
        m = mask[:, 1:]
        denom = m.sum(-1).clamp(min=1)
        if self.clip_eps > 0:
            old = lp.detach()
            ratio = torch.exp(lp - old)
            a = adv[:, None]
            per_tok = -torch.minimum(ratio * a, ratio.clamp(1 - self.clip_eps, 1 + self.clip_eps) * a)
            seq_loss = (per_tok * m).sum(-1) / denom
        else:
            ce = -(lp * m).sum(-1) / denom                # CE_i over completion tokens
            seq_loss = adv * ce
        loss = seq_loss.mean()
        if self.ref_model is not None:
            with torch.no_grad():
                ref_lp = token_logprobs(self.ref_model, ids)
            kl = (torch.exp(ref_lp - lp) - (ref_lp - lp) - 1) * m
            loss = loss + self.kl_coef * (kl.sum(-1) / denom).mean()
        self._backward_and_step(loss, grad_scale=1.0 - 0.01 * self.beta)
        return float(loss.detach())


# ------------------------------------------------------------------------------------------------
# PPO
# ------------------------------------------------------------------------------------------------
def gae(rewards, values, gamma=0.99, lam=0.95):
    """rewards, values [T] (values has T+1 entries) -> (advantages, returns)."""
    T = rewards.shape[0]
    adv = torch.zeros(T)
    last = 0.0
    for t in reversed(range(T)):
        delta = rewards[t] + gamma * values[t + 1] - values[t]
        last = delta + gamma * lam * last
        adv[t] = last
    return adv, adv + values[:T]


class PPOTrainer(_RLBase):
    def __init__(self, model, tokenizer=None, clip=0.2, gamma=0.99, lam=0.95, kl_target=0.01, kl_coef=0.1, lr=1e-5,
                 value_coef=0.5):
        super().__init__(model, tokenizer, lr=lr)
        self.clip, self.gamma, self.lam, self.kl_target, self.kl_coef, self.value_coef = clip, gamma, lam, kl_target, kl_coef, value_coef
        H = model.cfg.hidden_size
        dev, dt = model.tok_embeddings.device, torch.float32
        self.value_head = torch.nn.Linear(H, 1).to(dev, dt)
        self.value_opt = torch.optim.Adam(self.value_head.parameters(), lr=1e-3)

    def values(self, ids):
        B, S = ids.shape
        with torch.no_grad():
            h = self.model.hidden_states(ids).float().view(B, S, -1)
        return self.value_head(h).squeeze(-1)

    def train_step(self, ids, mask, rewards, old_logprobs=None):
        """ids [B,S]; mask marks action tokens; rewards [B] terminal rewards."""
        dev = self.model.tok_embeddings.device
        ids, mask = ids.to(dev), mask.to(dev).float()
        m = mask[:, 1:]
        lp = token_logprobs(self.model, ids)
        old = lp.detach() if old_logprobs is None else old_logprobs.to(dev)
        v = self.values(ids)
        advs, rets = [], []
        for b in range(ids.shape[0]):
            T = ids.shape[1] - 1
            r = torch.zeros(T)
            last = int(m[b].nonzero().max()) if m[b].any() else T - 1
            r[last] = float(rewards[b])
            a, ret = gae(r, torch.cat([v[b, :T].detach().cpu(), torch.zeros(1)]), self.gamma, self.lam)
            advs.append(a)
            rets.append(ret)
        adv = torch.stack(advs).to(dev)
        ret = torch.stack(rets).to(dev)
        adv = (adv - (adv * m).sum() / m.sum().clamp(min=1)) / (adv[m > 0].std() + 1e-8 if (m > 0).sum() > 1 else 1.0)
        ratio = torch.exp(lp - old)
        pol = -torch.minimum(ratio * adv, ratio.clamp(1 - self.clip, 1 + self.clip) * adv)
        approx_kl = ((old - lp) * m).sum() / m.sum().clamp(min=1)
        loss = (pol * m).sum() / m.sum().clamp(min=1) + self.kl_coef * approx_kl
        self._backward_and_step(loss)
        vloss = (((self.values(ids)[:, :-1] - ret) ** 2) * m).sum() / m.sum().clamp(min=1)
        self.value_opt.zero_grad()
        (self.value_coef * vloss).backward()
        self.value_opt.step()
        kl = float(approx_kl.detach())
        if kl > 1.5 * self.kl_target:                 # adaptive KL coefficient
            self.kl_coef *= 1.5
        elif kl < self.kl_target / 1.5:
            self.kl_coef /= 1.5
        return float(loss.detach()), float(vloss.detach()), kl


# ------------------------------------------------------------------------------------------------
# DPO
# ------------------------------------------------------------------------------------------------
class DPOTrainer(_RLBase):
    def __init__(self, model, ref_model=None, tokenizer=None, beta=0.1, lr=1e-6):
        super().__init__(model, tokenizer, lr=lr)
        self.beta = beta
        self.ref = (ref_model or copy.deepcopy(model)).eval()

    def train_step(self, chosen, rejected, chosen_mask, rejected_mask):
        dev = self.model.tok_embeddings.device

        def seq_lp(model, ids, mask):
            return (token_logprobs(model, ids.to(dev)) * mask.to(dev).float()[:, 1:]).sum(-1)
        pc, pr = seq_lp(self.model, chosen, chosen_mask), seq_lp(self.model, rejected, rejected_mask)
        with torch.no_grad():
            rc, rr = seq_lp(self.ref, chosen, chosen_mask), seq_lp(self.ref, rejected, rejected_mask)
        margin = self.beta * ((pc - rc) - (pr - rr))
        loss = -TF.logsigmoid(margin).mean()
        self._backward_and_step(loss)
        return float(loss.detach()), float((margin > 0).float().mean())


# ------------------------------------------------------------------------------------------------
# RLVR: verifiable rewards
# ------------------------------------------------------------------------------------------------
class RLVRTrainer(GRPOTrainer):
    """GRPO whose reward is a verifier: 1 when the expected answer appears in the completion, else 0."""

    def __init__(self, model, tokenizer, verifier: Optional[Callable[[str, str], float]] = None, **kw):
        super().__init__(model, tokenizer, **kw)
        self.verifier = verifier or (lambda completion, answer: 1.0 if answer.strip() and answer.strip() in completion else 0.0)

    def train_on_example(self, prompt: str, answer: str):
        p = self.tok.encode(prompt)
        self.reward_fn = lambda ids: self.verifier(self.tok.decode(ids), answer)
        return self.train_step(prompt=p)


# ------------------------------------------------------------------------------------------------
# reward model, rollouts, pipeline
# ------------------------------------------------------------------------------------------------
class RewardModel(torch.nn.Module):
    """Scalar head on the final hidden state of the last token; Bradley-Terry pairwise loss."""

    def __init__(self, backbone, hidden=None):
        super().__init__()
        self.backbone = backbone
        H = backbone.cfg.hidden_size
        dev = backbone.tok_embeddings.device
        self.head = torch.nn.Sequential(torch.nn.Linear(H, hidden or H), torch.nn.Tanh(), torch.nn.Linear(hidden or H, 1)).to(dev)

    def score(self, ids, lengths=None):
        B, S = ids.shape
        with torch.no_grad():
            h = self.backbone.hidden_states(ids).float().view(B, S, -1)
        last = (lengths - 1) if lengths is not None else torch.full((B,), S - 1, device=ids.device)
        return self.head(h[torch.arange(B, device=ids.device), last]).squeeze(-1)

    def pairwise_loss(self, chosen, rejected):
        return -TF.logsigmoid(self.score(chosen) - self.score(rejected)).mean()


@dataclass
class Rollout:
    seq: int
    prompt: List[int]
    completion: List[int]
    reward: float


class RolloutWorker:
    """Produces rollouts in a deterministic, sequence-numbered order into a bounded buffer."""

    def __init__(self, trainer: _RLBase, reward_fn: Callable, capacity=1024, max_new=32, temperature=1.0):
        self.tr, self.reward_fn, self.max_new, self.temperature = trainer, reward_fn, max_new, temperature
        self.buffer = deque(maxlen=capacity)
        self.next_seq = 0

    def collect(self, prompts: List[List[int]], per_prompt=1):
        for p in prompts:
            for o in self.tr.generate(p, per_prompt, self.max_new, self.temperature, seed=self.next_seq):
                self.buffer.append(Rollout(self.next_seq, list(p), o, float(self.reward_fn(o))))
                self.next_seq += 1
        return len(self.buffer)

    def drain(self, n=None):
        n = len(self.buffer) if n is None else min(n, len(self.buffer))
        return [self.buffer.popleft() for _ in range(n)]


class RLHFPipeline:
    """reward-model fit -> rollouts -> policy optimisation, one round per ``run_round``."""

    def __init__(self, policy_trainer: GRPOTrainer, reward_model: Optional[RewardModel] = None):
        self.policy, self.rm = policy_trainer, reward_model
        self.rm_opt = torch.optim.Adam(reward_model.head.parameters(), lr=1e-3) if reward_model is not None else None

    def fit_reward_model(self, chosen, rejected, steps=10):
        losses = []
        for _ in range(steps):
            loss = self.rm.pairwise_loss(chosen, rejected)
            self.rm_opt.zero_grad()
            loss.backward()
            self.rm_opt.step()
            losses.append(float(loss))
        return losses

    def run_round(self, prompts: List[List[int]]):
        if self.rm is not None:
            dev = self.policy.model.tok_embeddings.device
            self.policy.reward_fn = lambda ids: float(self.rm.score(torch.tensor([ids or [0]], device=dev)))
        return [self.policy.train_step(prompt=p) for p in prompts]
