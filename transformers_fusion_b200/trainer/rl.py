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

    # ---- reference-named helpers (include/quant/trainer.h:347-465)
    def set_optimizer(self, opt):
        """Use another flat optimizer (anything with ``step()`` over this model's flat buffers)."""
        self.opt = opt

    def optimizer(self):
        return self.opt

    @staticmethod
    def compute_log_probs(logits, ids):
        """log p of the tokens that follow: logits [B, S, V], ids [B, S] -> [B, S-1] (position t scores ids[:, t+1])."""
        lp = torch.log_softmax(logits.float()[:, :-1], -1)
        return lp.gather(-1, ids[:, 1:].unsqueeze(-1)).squeeze(-1)

    @staticmethod
    def compute_kl_divergence(logits_a, logits_b) -> float:
        """Mean over positions of KL(softmax(a) || softmax(b))."""
        la, lb = torch.log_softmax(logits_a.float(), -1), torch.log_softmax(logits_b.float(), -1)
        return float((la.exp() * (la - lb)).sum(-1).mean())

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
        self._last_loss = 0.0

    def set_beta(self, b: float): self.beta = float(b)
    def group_size(self) -> int: return self.G
    def last_loss(self) -> float: return self._last_loss

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
        self._last_loss = float(loss.detach())
        return self._last_loss


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


def _set_log_callback(self, cb):
    """``cb`` is called at the end of every train_step (PPO: policy loss, value loss, entropy, KL; DPO: loss, KL)."""
    self.log_cb = cb


class PPOTrainer(_RLBase):
    def __init__(self, model, tokenizer=None, clip=0.2, gamma=0.99, lam=0.95, kl_target=0.01, kl_coef=0.1, lr=1e-5,
                 value_coef=0.5):
        super().__init__(model, tokenizer, lr=lr)
        self.clip, self.gamma, self.lam, self.kl_target, self.kl_coef, self.value_coef = clip, gamma, lam, kl_target, kl_coef, value_coef
        H = model.cfg.hidden_size
        dev, dt = model.tok_embeddings.device, torch.float32
        self.value_head = torch.nn.Linear(H, 1).to(dev, dt)
        self.value_opt = torch.optim.Adam(self.value_head.parameters(), lr=1e-3)

    def critic_forward(self, hidden):
        """Value of every position from final hidden states [..., H]."""
        return self.value_head(hidden.float()).squeeze(-1)

    def critic_parameters(self):
        return list(self.value_head.parameters())

    @staticmethod
    def compute_gae(rewards, values, gamma=0.99, lam=0.95):
        """Advantages of one trajectory: rewards [T], values [T] or [T + 1] (a missing bootstrap value counts as 0)."""
        r, v = torch.as_tensor(rewards).float().cpu(), torch.as_tensor(values).float().cpu()
        if v.numel() == r.numel():
            v = torch.cat([v, torch.zeros(1)])
        return gae(r, v, gamma, lam)[0]

    def kl_alpha(self) -> float: return self.kl_coef
    def last_kl(self) -> float: return getattr(self, "_last_kl", 0.0)

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
        kl = self._last_kl = float(approx_kl.detach())
        if getattr(self, "log_cb", None):
            # policy loss, value loss, mean entropy estimate of the action tokens (-log-prob of the taken actions), KL to the old policy
            ent = float((-(lp.detach()) * m).sum() / m.sum().clamp(min=1))
            self.log_cb(float(loss.detach()), float(vloss.detach()), ent, kl)
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
        self._last_loss = 0.0

    def set_beta(self, b: float): self.beta = float(b)
    def last_loss(self) -> float: return self._last_loss

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
        self._last_loss = float(loss.detach())
        if getattr(self, "log_cb", None):
            # loss and the sequence-level KL estimate to the frozen reference on the chosen answers
            self.log_cb(self._last_loss, float((pc.detach() - rc).mean()))
        return self._last_loss, float((margin > 0).float().mean())


# ------------------------------------------------------------------------------------------------
# RLVR: verifiable rewards
# ------------------------------------------------------------------------------------------------
PPOTrainer.set_log_callback = _set_log_callback
DPOTrainer.set_log_callback = _set_log_callback


class RLVRTrainer(GRPOTrainer):
    """GRPO whose reward is a verifier: 1 when the expected answer appears in the completion, else 0."""

    def __init__(self, model, tokenizer, verifier: Optional[Callable[[str, str], float]] = None, **kw):
        super().__init__(model, tokenizer, **kw)
        self.verifier = verifier or (lambda completion, answer: 1.0 if answer.strip() and answer.strip() in completion else 0.0)

    def verify(self, output: str, answer: str) -> bool:
        return self.verifier(output, answer) > 0

    def last_reward(self) -> float:
        return getattr(self, "_last_reward", 0.0)

    def train_on_example(self, prompt: str, answer: str):
        p = self.tok.encode(prompt)
        got = []

        def reward(ids):
            got.append(self.verifier(self.tok.decode(ids), answer))
            return got[-1]
        self.reward_fn = reward
        loss = GRPOTrainer.train_step(self, prompt=p)
        self._last_reward = sum(got) / max(1, len(got))
        return loss

    def train_step(self, ids=None, mask=None, rewards=None, prompt=None, answer: Optional[str] = None):
        """``train_step(prompt_text, answer_text)`` (the reference's verifiable form: sample a group, reward = the
        verifier's verdict) or the group form of GRPO (ids, mask, rewards)."""
        if isinstance(ids, str):
            return self.train_on_example(ids, mask if isinstance(mask, str) else (answer or ""))
        if isinstance(prompt, str):
            return self.train_on_example(prompt, answer or "")
        return GRPOTrainer.train_step(self, ids, mask, rewards, prompt)


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

    # ---- the reference's surface (include/quant/reward.h:18-52)
    def hidden_size(self) -> int: return self.backbone.cfg.hidden_size
    def num_layers(self) -> int: return sum(1 for m in self.head if isinstance(m, torch.nn.Linear))
    def last_loss(self) -> float: return getattr(self, "_last_loss", 0.0)
    def set_log_callback(self, cb): self.log_cb = cb

    def score_pair(self, chosen, rejected):
        """(score of chosen, score of rejected), each [B]."""
        return self.score(chosen), self.score(rejected)

    @staticmethod
    def reward_loss(chosen_rewards, rejected_rewards):
        """Bradley-Terry: -log sigmoid(r_chosen - r_rejected), mean over the pairs."""
        return -TF.logsigmoid(chosen_rewards - rejected_rewards).mean()

    def train_step(self, chosen, rejected, opt=None, loss_scale: float = 1.0) -> float:
        """One optimizer step on the head from a batch of pairs; reports (loss, pair accuracy) to the log callback."""
        if opt is None:
            opt = self.__dict__.setdefault("_opt", torch.optim.Adam(self.head.parameters(), lr=1e-3))
        rc, rr = self.score_pair(chosen, rejected)
        loss = self.reward_loss(rc, rr)
        opt.zero_grad()
        (loss * loss_scale).backward()
        if loss_scale != 1.0:
            for p in self.head.parameters():
                if p.grad is not None:
                    p.grad.div_(loss_scale)
        opt.step()
        self._last_loss = float(loss.detach())
        if getattr(self, "log_cb", None):
            self.log_cb(self._last_loss, float((rc > rr).float().mean()))
        return self._last_loss

    @staticmethod
    def compute_abstention_reward(output: str, confidence: float) -> float:
        """Reward shaping for "I don't know"-style answers: abstaining is worth a small positive reward when the model is
        unsure (confidence < 0.5) and is penalised when it was confident; a committed answer earns its confidence."""
        text = output.lower()
        abstains = any(k in text for k in ("i don't know", "i do not know", "not sure", "cannot answer", "unsure", "no idea"))
        c = min(1.0, max(0.0, float(confidence)))
        if abstains:
            return 0.3 * (1.0 - c) - 0.5 * max(0.0, c - 0.5)
        return c - 0.5

    def save(self, path: str):
        torch.save({"head": self.head.state_dict(), "hidden": self.hidden_size()}, path)

    def load(self, path: str):
        st = torch.load(path, map_location="cpu", weights_only=True)
        if st["hidden"] != self.hidden_size():
            raise ValueError(f"{path}: head for hidden size {st['hidden']}, this backbone has {self.hidden_size()}")
        self.head.load_state_dict(st["head"])
        return self


@dataclass
class Rollout:
    seq: int
    prompt: List[int]
    completion: List[int]
    reward: float


@dataclass
class Trajectory:
    seq: int = 0                     # global push order: the deterministic replay key
    tokens: List[int] = field(default_factory=list)      # prompt + generated tokens
    reward: float = 0.0
    done: bool = True


class AsyncRolloutBuffer:
    """Bounded hand-over between rollout producers and the trainer.  Trajectories are numbered in push order and popped in
    that order, so a run can be replayed exactly; ``push`` blocks while the buffer is full, ``pop`` while it is empty (both
    give up on ``close``).  Reference: AsyncRolloutBuffer, include/quant/rollout_worker.h:36-62."""

    def __init__(self, capacity: int = 64):
        import threading
        self._cap, self._items, self._next, self._closed = int(capacity), {}, 0, False
        self._det, self._log = True, []
        self._cv = threading.Condition()

    def set_deterministic_replay(self, v: bool): self._det = bool(v)
    def deterministic_replay(self) -> bool: return self._det
    def capacity(self) -> int: return self._cap
    def closed(self) -> bool: return self._closed

    def size(self) -> int:
        with self._cv:
            return len(self._items)

    def push(self, t: Trajectory, timeout_s: Optional[float] = None) -> bool:
        with self._cv:
            if not self._cv.wait_for(lambda: self._closed or len(self._items) < self._cap, timeout_s) or self._closed:
                return False
            t.seq = self._next
            self._next += 1
            self._items[t.seq] = t
            if self._det:
                self._log.append(Trajectory(t.seq, list(t.tokens), t.reward, t.done))
            self._cv.notify_all()
            return True

    def _take(self):
        k = min(self._items)
        t = self._items.pop(k)
        self._cv.notify_all()
        return t

    def pop(self, timeout_s: Optional[float] = None) -> Optional[Trajectory]:
        with self._cv:
            if not self._cv.wait_for(lambda: self._closed or self._items, timeout_s):
                return None
            return self._take() if self._items else None

    def try_pop(self) -> Optional[Trajectory]:
        with self._cv:
            return self._take() if self._items else None

    def close(self):
        with self._cv:
            self._closed = True
            self._cv.notify_all()

    def replay(self) -> List[Trajectory]:
        """Every trajectory pushed so far, in push order (kept only under deterministic replay)."""
        with self._cv:
            return list(self._log)


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

    # ---- text-prompt form of the reference (include/quant/rollout_worker.h:64-80)
    def _ids(self, prompt):
        tok = self.tr.tok
        return list(prompt) if not isinstance(prompt, str) else (tok.encode(prompt) if tok is not None else [ord(c) % 250 + 5 for c in prompt])

    def generate(self, prompt) -> List[int]:
        """Prompt ids followed by one sampled completion."""
        ids = self._ids(prompt)
        out = self.tr.generate(ids, 1, self.max_new, self.temperature, seed=self.next_seq)[0]
        self.next_seq += 1
        return ids + out

    def generate_batch(self, prompts) -> List[List[int]]:
        return [self.generate(p) for p in prompts]

    def generate_trajectory(self, prompt, reward: Optional[float] = None) -> Trajectory:
        ids = self._ids(prompt)
        toks = self.generate(ids)
        r = float(self.reward_fn(toks[len(ids):])) if reward is None else float(reward)
        return Trajectory(0, toks, r, True)

    def produce_to(self, buf: AsyncRolloutBuffer, prompts) -> int:
        """Push one trajectory per prompt; stops early when the buffer is closed.  Returns how many were pushed."""
        n = 0
        for p in prompts:
            if not buf.push(self.generate_trajectory(p)):
                break
            n += 1
        return n

    def param_count(self) -> int:
        return sum(p.numel() for p in self.tr.model.parameters())


@dataclass
class Comparison:
    prompt: str = ""
    chosen_ids: List[int] = field(default_factory=list)
    rejected_ids: List[int] = field(default_factory=list)
    reward_chosen: float = 0.0
    reward_rejected: float = 0.0


@dataclass
class RLHFMetrics:
    step: int = 0
    reward_loss: float = 0.0
    reward_accuracy: float = 0.0
    ppo_loss: float = 0.0
    ppo_kl: float = 0.0
    dpo_loss: float = 0.0
    grpo_loss: float = 0.0
    mean_reward: float = 0.0


DEFAULT_PROMPTS = ("Explain why the sky is blue.", "Write a short poem about AI.", "What is machine learning?",
                   "Describe how a computer works.", "Tell me a joke.", "What is the capital of France?")


class RLHFPipeline:
    """Preference alignment loop: sample pairs of completions and rank them -> fit the reward model -> optimise the policy
    (PPO against the reward model, DPO on the stored pairs, GRPO / verifiable-reward steps) - one round per ``run_round``
    or the whole schedule with ``run``.  Reference: RLHFPipeline, include/quant/trainer.h:466-521,
    src/trainer/trainer_rl.cpp:1021-1127, trainer_rl_ops.cpp:28-526 (whose ``generate_comparisons`` stores one greedy
    sequence as both members of a pair; here the two members are two sampled completions ranked by reward)."""

    def __init__(self, policy_trainer: GRPOTrainer, reward_model: Optional[RewardModel] = None):
        self.policy, self.rm = policy_trainer, reward_model
        self.rm_opt = torch.optim.Adam(reward_model.head.parameters(), lr=1e-3) if reward_model is not None else None
        self._comparisons: List[Comparison] = []
        self._metrics = RLHFMetrics()
        self.log_cb = None
        self.verbose = False
        self._ppo = self._dpo = None

    # ---- bookkeeping
    def comparisons(self) -> List[Comparison]: return self._comparisons
    def metrics(self) -> RLHFMetrics: return self._metrics
    def set_log_callback(self, cb): self.log_cb = cb
    def set_verbose(self, v: bool): self.verbose = bool(v)

    def _say(self, text):
        if self.verbose:
            print(text)

    def _encode(self, prompt):
        tok = self.policy.tok
        if isinstance(prompt, str):
            ids = tok.encode(prompt) if tok is not None else []
            V = self.policy.model.cfg.vocab_size
            return ids or [ord(c) % max(1, V - 5) + 5 for c in prompt]      # the reference's fallback without a tokenizer
        return list(prompt)

    def _score(self, ids: List[int]) -> float:
        if self.rm is not None:
            dev = self.policy.model.tok_embeddings.device
            with torch.no_grad():
                return float(self.rm.score(torch.tensor([ids or [0]], device=dev)))
        return float(self.policy.reward_fn(ids))

    # ---- math helpers with the reference's names
    compute_gae = staticmethod(lambda rewards, values, gamma=0.99, lam=0.95: PPOTrainer.compute_gae(rewards, values, gamma, lam))

    @staticmethod
    def compute_returns_discounted(rewards, gamma: float = 0.99):
        r = torch.as_tensor(rewards).float()
        out, acc = torch.zeros_like(r), 0.0
        for t in reversed(range(r.numel())):
            acc = float(r[t]) + gamma * acc
            out[t] = acc
        return out

    @staticmethod
    def compute_kl_between_policies(logits_pi, logits_ref, actions) -> float:
        """Mean over positions of log pi(a) - log ref(a) on the taken actions (the sampled-action KL estimate)."""
        lp = torch.log_softmax(logits_pi.float(), -1).gather(-1, actions.long().unsqueeze(-1)).squeeze(-1)
        lr_ = torch.log_softmax(logits_ref.float(), -1).gather(-1, actions.long().unsqueeze(-1)).squeeze(-1)
        return float((lp - lr_).mean())

    # ---- data
    def generate_comparisons(self, prompts, max_new_tokens: int = 64):
        """Two sampled completions per prompt, ranked by the reward model (or the policy trainer's reward function)."""
        for i, p in enumerate(prompts):
            ids = self._encode(p)
            a, b = self.policy.generate(ids, 2, max_new_tokens, temperature=1.0, seed=len(self._comparisons))
            ra, rb = self._score(ids + a), self._score(ids + b)
            if rb > ra:
                a, b, ra, rb = b, a, rb, ra
            self._comparisons.append(Comparison(p if isinstance(p, str) else "", ids + a, ids + b, ra, rb))
            self._say(f"[RLHF] Comparison {i + 1}/{len(prompts)} | reward_chosen={ra:.4f} reward_rejected={rb:.4f}")
        return self._comparisons

    def _pair_batch(self, data: Sequence[Comparison]):
        dev = self.policy.model.tok_embeddings.device
        S = max(max(len(c.chosen_ids), len(c.rejected_ids)) for c in data)

        def pad(rows):
            ids = torch.zeros((len(rows), S), dtype=torch.long)
            mask = torch.zeros((len(rows), S))
            for i, r in enumerate(rows):
                ids[i, :len(r)] = torch.tensor(r)
                mask[i, :len(r)] = 1
            return ids.to(dev), mask.to(dev)
        return pad([c.chosen_ids for c in data]), pad([c.rejected_ids for c in data])

    def _rm_scores(self, ids, mask):
        return self.rm.score(ids, mask.sum(-1).long().clamp(min=1))

    # ---- reward model
    def compute_reward_accuracy(self, data: Optional[Sequence[Comparison]] = None) -> float:
        """Fraction of pairs whose chosen member the reward model scores higher."""
        data = list(data if data is not None else self._comparisons)
        data = [c for c in data if c.chosen_ids and c.rejected_ids]
        if not data or self.rm is None:
            return 0.0
        (ci, cm), (ri, rm_) = self._pair_batch(data)
        with torch.no_grad():
            return float((self._rm_scores(ci, cm) > self._rm_scores(ri, rm_)).float().mean())

    def train_reward_model(self, data: Optional[Sequence[Comparison]] = None, epochs: int = 3, batch_size: int = 8):
        data = [c for c in (data if data is not None else self._comparisons) if c.chosen_ids and c.rejected_ids]
        last = 0.0
        for _ in range(epochs):
            for o in range(0, len(data), batch_size):
                (ci, cm), (ri, rm_) = self._pair_batch(data[o:o + batch_size])
                loss = -TF.logsigmoid(self._rm_scores(ci, cm) - self._rm_scores(ri, rm_)).mean()
                self.rm_opt.zero_grad()
                loss.backward()
                self.rm_opt.step()
                last = float(loss.detach())
        self._metrics.reward_loss = last
        return last

    def train_reward_model_epoch_with_accuracy(self, train_data, val_data, epochs: int = 3, batch_size: int = 8, split_name=None):
        """Fit on ``train_data`` and report the pairwise accuracy on ``val_data`` after every epoch; returns the last."""
        acc = 0.0
        for e in range(epochs):
            loss = self.train_reward_model(train_data, 1, batch_size)
            acc = self.compute_reward_accuracy(val_data if val_data else train_data)
            self._say(f"[{split_name or 'RM'}] epoch {e + 1}/{epochs} loss={loss:.4f} val_acc={acc:.3f}")
        self._metrics.reward_accuracy = acc
        return acc

    # ---- policy optimisation stages
    def _share_optimizer(self, trainer):
        trainer.flat, trainer.opt = self.policy.flat, self.policy.opt        # one optimizer state per policy
        return trainer

    def ppo_finetune(self, prompts, n_ppo_steps: int = 100, ppo_batch_size: int = 8, max_new_tokens: int = 64):
        """PPO steps on sampled completions whose terminal reward is the reward model's score."""
        if self._ppo is None:
            self._ppo = self._share_optimizer(PPOTrainer(self.policy.model, self.policy.tok))
        dev = self.policy.model.tok_embeddings.device
        out = (0.0, 0.0, 0.0)
        for step in range(n_ppo_steps):
            ids_p = self._encode(prompts[step % len(prompts)])
            outs = self.policy.generate(ids_p, ppo_batch_size, max_new_tokens, temperature=1.0, seed=step)
            S = len(ids_p) + max(1, max(len(o) for o in outs))
            ids, mask = torch.zeros((len(outs), S), dtype=torch.long), torch.zeros((len(outs), S))
            for i, o in enumerate(outs):
                seq = ids_p + o
                ids[i, :len(seq)] = torch.tensor(seq)
                mask[i, len(ids_p):len(seq)] = 1
            rewards = torch.tensor([self._score(ids_p + o) for o in outs])
            out = self._ppo.train_step(ids.to(dev), mask.to(dev), rewards)
            self._metrics.mean_reward = float(rewards.mean())
        self._metrics.ppo_loss, self._metrics.ppo_kl = out[0], out[2]
        return out

    def dpo_finetune(self, comparisons: Optional[Sequence[Comparison]] = None, n_steps: int = 10, batch_size: int = 4):
        data = [c for c in (comparisons if comparisons is not None else self._comparisons) if c.chosen_ids and c.rejected_ids]
        if not data:
            return 0.0
        if self._dpo is None:
            self._dpo = self._share_optimizer(DPOTrainer(self.policy.model, tokenizer=self.policy.tok))
        loss = 0.0
        for step in range(n_steps):
            o = (step * batch_size) % len(data)
            (ci, cm), (ri, rm_) = self._pair_batch((data + data)[o:o + batch_size])
            loss, _ = self._dpo.train_step(ci, ri, cm, rm_)
        self._metrics.dpo_loss = loss
        return loss

    def grpo_finetune(self, prompts, n_steps: int = 20, max_new_tokens: int = 32):
        self.policy.max_new = max_new_tokens
        if self.rm is not None:
            self.policy.reward_fn = lambda ids: self._score(ids)
        loss = 0.0
        for step in range(n_steps):
            loss = self.policy.train_step(prompt=self._encode(prompts[step % len(prompts)]))
        self._metrics.grpo_loss = loss
        return loss

    def rlvf_finetune(self, qa_pairs, n_steps: int = 20, max_new_tokens: int = 32, verifier=None):
        """Verifiable-reward steps: the reward of a completion is whether it contains the pair's answer."""
        verifier = verifier or (lambda completion, answer: 1.0 if answer.strip() and answer.strip() in completion else 0.0)
        tok = self.policy.tok
        self.policy.max_new = max_new_tokens
        loss = 0.0
        for step in range(n_steps):
            q, a = qa_pairs[step % len(qa_pairs)]
            self.policy.reward_fn = lambda ids, a=a: verifier(tok.decode(ids) if tok is not None else "", a)
            loss = self.policy.train_step(prompt=self._encode(q))
        self._metrics.grpo_loss = loss
        return loss

    def run(self, n_rounds: int = 3, n_prompts: int = 50, n_ppo_steps: int = 200, prompts=None, max_new_tokens: int = 32):
        """Rounds of: new comparisons -> reward model (one more epoch each round, a fifth of the prompts held out) -> PPO
        -> DPO on everything gathered so far."""
        prompts = list(prompts) if prompts else [DEFAULT_PROMPTS[i % len(DEFAULT_PROMPTS)] for i in range(n_prompts)]
        hold = max(1, len(prompts) // 5)
        train_prompts = prompts[:-hold] or prompts
        heldout: List[Comparison] = []
        for rnd in range(n_rounds):
            self._say(f"=== RLHF Round {rnd + 1}/{n_rounds} ===")
            self._metrics.step = rnd
            if not heldout and self.rm is not None:
                before = len(self._comparisons)
                self.generate_comparisons(prompts[-hold:], max_new_tokens)
                heldout, self._comparisons = self._comparisons[before:], self._comparisons[:before]
            self.generate_comparisons(train_prompts, max_new_tokens)
            if self.rm is not None:
                self.train_reward_model_epoch_with_accuracy(self._comparisons, heldout, max(1, 3 + rnd), 8, "RM")
            self.ppo_finetune(train_prompts, max(1, n_ppo_steps + rnd * 10), 8, max_new_tokens)
            if len(self._comparisons) > 4:
                self.dpo_finetune(self._comparisons, max(1, 2 + rnd), 4)
            if self.rm is not None:
                self._metrics.reward_accuracy = self.compute_reward_accuracy(self._comparisons)
            if self.log_cb:
                self.log_cb(self._metrics)
        return self._metrics

    def fit_reward_model(self, chosen, rejected, steps=10):
        losses = []
        for _ in range(steps):
            loss = self.rm.pairwise_loss(chosen, rejected)
            self.rm_opt.zero_grad()
            loss.backward()
            self.rm_opt.step()
            losses.append(float(loss.detach()))
        return losses

    def run_round(self, prompts: List[List[int]]):
        if self.rm is not None:
            dev = self.policy.model.tok_embeddings.device
            self.policy.reward_fn = lambda ids: float(self.rm.score(torch.tensor([ids or [0]], device=dev)).detach())
        return [self.policy.train_step(prompt=p) for p in prompts]
