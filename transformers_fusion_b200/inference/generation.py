"""Generation front ends on top of the paged engine.

* ``Generator``            - generate_tokens / generate / generate_stream / generate_full (text in, text out).
* ``StreamingGenerator``   - event stream (START, TOKEN, COMPLETE, ERROR, STOP) with stop strings, per-token log-probs and
                             a cooperative ``request_stop``.
* ``SpeculativeDecoder``   - a small draft model proposes ``gamma`` tokens, the target model scores all of them in one
                             chunked pass over its paged cache and accepts the longest prefix that survives rejection
                             sampling (exactly the target distribution; greedy when temperature is 0); ``gamma`` adapts
                             to the acceptance rate.  Rejected positions are simply overwritten: the cache is addressed
                             by position, so rewinding is resetting a counter.
* ``TreeDecoder``          - top-b branching draft tree flattened into candidate paths; the best-scoring path that the
                             target accepts wins.
* ``DynamicBatcher``       - groups queued requests by arrival window and pads them into one batch.
* ``EmbeddingEndpoint`` / ``Reranker`` - mean-pooled hidden states, cosine scoring.
* ``GrammarDecoder``       - token masks from a JSON-structure automaton or a regular expression over the decoded text.
* ``INT8Inference`` / ``FP8Inference`` / ``ModelShard`` - low-precision linear layers and layer-range shards.

Reference counterparts: src/inference/generator.cpp:16-363, inference_speculative.cpp, speculative_decoder.cpp,
inference_serve.cpp:25-325, inference_lowprec.cpp."""
from __future__ import annotations

import json
import math
import re
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

import torch

from ..ops import functional as F
from .engine import EngineConfig, InferenceEngine, Request
from .kv_cache import PAGE
from .sampler import SamplerConfig, _filtered_probs


@dataclass
class GenerationResult:
    text: str = ""
    tokens: List[int] = field(default_factory=list)
    duration: float = 0.0
    tokens_per_sec: float = 0.0
    truncated: bool = False


class Generator:
    def __init__(self, model, tokenizer, engine_cfg: Optional[EngineConfig] = None):
        self.model, self.tok = model, tokenizer
        self.engine = InferenceEngine(model, tokenizer, engine_cfg or EngineConfig(num_pages=max(64, 4 * model.cfg.max_seq_len // PAGE)))

    def generate_tokens(self, ids: Sequence[int], cfg: Optional[SamplerConfig] = None) -> List[int]:
        cfg = cfg or SamplerConfig()
        return self.engine.generate_batch([list(ids)], cfg.max_tokens, cfg)[0]

    def generate(self, prompt: str, cfg: Optional[SamplerConfig] = None) -> str:
        cfg = cfg or SamplerConfig()
        return self.engine.generate(prompt, cfg.max_tokens, cfg)

    def generate_stream(self, prompt: str, cfg: Optional[SamplerConfig], on_token: Callable[[str], None]) -> str:
        cfg = cfg or SamplerConfig()
        return self.engine.generate_stream(prompt, on_token, cfg.max_tokens, cfg)

    def generate_full(self, prompt: str, cfg: Optional[SamplerConfig] = None) -> GenerationResult:
        cfg = cfg or SamplerConfig()
        ids = self.tok.encode(prompt)
        limit = self.engine.max_len - 1
        t0 = time.perf_counter()
        out = self.generate_tokens(ids[:limit], cfg)
        dt = time.perf_counter() - t0
        eos = getattr(self.tok, "eos_id", -1)
        toks = [t for t in out if t != eos]
        return GenerationResult(self.tok.decode(toks), out, dt, len(out) / max(dt, 1e-9), len(ids) > limit)


@dataclass
class StreamingConfig:
    sampling: SamplerConfig = field(default_factory=SamplerConfig)
    max_tokens: int = 128
    stop_strings: Sequence[str] = ()
    top_logprobs: int = 0

    def effective_max_tokens(self, budget: Optional[str] = None) -> int:
        from .sampler import REASONING_BUDGET
        cap = REASONING_BUDGET.get((budget or "").lower())
        return min(self.max_tokens, cap) if cap else self.max_tokens


class StreamingGenerator:
    START, TOKEN, COMPLETE, ERROR, STOP = "START", "TOKEN", "COMPLETE", "ERROR", "STOP"

    def __init__(self, model, tokenizer, seed: int = 42):
        self.model, self.tok = model, tokenizer
        self.engine = InferenceEngine(model, tokenizer, EngineConfig(seed=seed, num_pages=max(64, 4 * model.cfg.max_seq_len // PAGE)))
        self.handler: Callable[[str, dict], None] = lambda kind, payload: None
        self._stop = threading.Event()
        self._out: List[int] = []
        self._logprobs: List[float] = []
        self._tps = 0.0

    def set_event_handler(self, fn):
        self.handler = fn

    def request_stop(self):
        self._stop.set()

    def output_ids(self):
        return list(self._out)

    def token_logprobs(self):
        return list(self._logprobs)

    def tokens_per_sec(self):
        return self._tps

    def num_tokens_generated(self) -> int:
        return len(self._out)

    def stopped(self) -> bool:
        """True when the last generation ended on a stop request or a stop string."""
        return getattr(self, "_stopped", False)

    @torch.no_grad()
    def generate(self, prompt, cfg: Optional[StreamingConfig] = None) -> str:
        cfg = cfg or StreamingConfig()
        eng, tok = self.engine, self.tok
        self._stop.clear()
        self._out, self._logprobs = [], []
        try:
            ids = list(prompt) if not isinstance(prompt, str) else tok.encode(prompt)
            ids = ids[-(eng.max_len - 2):] or [0]
            self.handler(self.START, {"prompt_tokens": len(ids)})
            t0 = time.perf_counter()
            text, reason = "", self.COMPLETE
            r = eng.add_request(ids, cfg.max_tokens, cfg.sampling)
            seen = 0
            while eng.has_pending():
                eng.step()
                for t in r.out[seen:]:
                    self._out.append(t)
                    if t == getattr(tok, "eos_id", -1):
                        continue
                    new_text = tok.decode([x for x in self._out if x != getattr(tok, "eos_id", -1)])
                    piece, text = new_text[len(text):], new_text
                    self.handler(self.TOKEN, {"token": t, "text": piece})
                seen = len(r.out)
                hit = next((s for s in cfg.stop_strings if s and s in text), None)
                if hit is not None:
                    text = text[: text.index(hit)]
                    reason = self.STOP
                if self._stop.is_set():
                    reason = self.STOP
                if reason == self.STOP and not r.finished:
                    r.max_tokens = len(r.out)          # finishes at the next emit
                    r.finished = True
                    eng._release(r)
                    eng.running = [x for x in eng.running if x is not r]
                    break
            dt = time.perf_counter() - t0
            self._tps = len(self._out) / max(dt, 1e-9)
            self._stopped = reason == self.STOP
            self.handler(reason, {"text": text, "tokens": len(self._out), "tokens_per_sec": self._tps})
            return text
        except Exception as e:                         # surface the failure as an event, then re-raise
            self.handler(self.ERROR, {"message": str(e)})
            raise


# ================================================================================================ speculative decoding
class _Seq:
    """One sequence on one engine: pages + position counter."""

    def __init__(self, eng: InferenceEngine, max_total: int):
        self.eng = eng
        self.r = Request([], max_total)
        self.r.pages = [eng.cache.allocator.alloc() for _ in range((max_total + PAGE - 1) // PAGE)]
        self.tokens: List[int] = []
        self.pos = 0                       # positions < pos hold valid K/V

    def extend(self, upto_tokens: List[int], all_positions=False):
        """Run tokens[pos:] through the model, return logits of the new positions (all or last)."""
        h = self.eng._layers_prefill(upto_tokens, self.pos, self.r, all_positions=all_positions)
        self.pos = len(upto_tokens)
        return self.eng._logits(h).float()

    def rewind(self, pos):
        self.pos = pos

    def free(self):
        self.eng._release(self.r)


@dataclass
class SpeculativeStats:
    proposed: int = 0
    accepted: int = 0
    target_passes: int = 0
    generated: int = 0

    @property
    def acceptance_rate(self):
        return self.accepted / max(1, self.proposed)

    @property
    def tokens_per_target_pass(self):
        return self.generated / max(1, self.target_passes)


@dataclass
class SpeculativeStepResult:
    tokens_accepted: List[int]
    tokens_rejected: int = 0
    total_proposed: int = 0
    acceptance_rate: float = 0.0


class SpeculativeDecoder:
    def __init__(self, target, draft, gamma: int = 4, adaptive: bool = True, max_gamma: int = 8, seed: int = 0, kv_mode="bf16"):
        pages = lambda m: max(64, 4 * m.cfg.max_seq_len // PAGE)
        self.te = InferenceEngine(target, None, EngineConfig(num_pages=pages(target), enable_prefix_cache=False, kv_mode=kv_mode))
        self.de = InferenceEngine(draft, None, EngineConfig(num_pages=pages(draft), enable_prefix_cache=False, kv_mode=kv_mode))
        self.gamma, self.adaptive, self.max_gamma = gamma, adaptive, max_gamma
        self.gen = torch.Generator().manual_seed(seed)
        self.stats = SpeculativeStats()

    # ---- counters with the reference's names (include/quant/inference_opt.h:41-49)
    def acceptance_rate(self) -> float: return self.stats.acceptance_rate
    def accepted_count(self) -> int: return self.stats.accepted
    def total_count(self) -> int: return self.stats.proposed
    def current_gamma(self) -> float: return float(self.gamma)
    def used_uniform_draft_fallback(self) -> bool: return False      # a draft model is mandatory here

    # ---- step-wise form (reference: include/quant/speculative_decoder.h:80-98)
    def current_draft_k(self) -> int: return self.gamma
    def total_accepted(self) -> int: return self.stats.accepted
    def total_proposed(self) -> int: return self.stats.proposed

    def update_draft_k(self, new_k: int):
        """Set the number of drafted tokens per round, clamped to [1, max]."""
        self.gamma = max(1, min(int(new_k), self.max_gamma))

    @torch.no_grad()
    def decode_step(self, context: List[int], sampling: Optional[SamplerConfig] = None) -> "SpeculativeStepResult":
        """One draft-and-verify round on ``context`` (extended in place by the accepted tokens and the target's own token).  Both
        caches are rebuilt from the context, so a caller that wants them kept across rounds uses ``generate``."""
        sc = sampling or SamplerConfig(temperature=0.0)
        g = self.gamma
        total = min(len(context) + g + 2, min(self.te.max_len, self.de.max_len))
        if not context or len(context) + g + 1 > total:
            return SpeculativeStepResult([], 0, 0, self.acceptance_rate())
        T, D = _Seq(self.te, total), _Seq(self.de, total)
        try:
            if len(context) > 1:
                T.extend(context[:-1])
            q_list, prop, cur = [], [], list(context)
            for _ in range(g):
                q = self._probs(D.extend(cur)[-1], sc)
                t = int(torch.multinomial(q.cpu(), 1, generator=self.gen))
                q_list.append(q), prop.append(t), cur.append(t)
            lt = T.extend(cur, all_positions=True)
            self.stats.target_passes += 1
            self.stats.proposed += g
            n_acc, bonus = 0, None
            for i in range(g):
                p, q, t = self._probs(lt[i], sc), q_list[i], prop[i]
                if float(torch.rand((), generator=self.gen)) < min(1.0, float(p[t]) / max(float(q[t]), 1e-30)):
                    n_acc += 1
                    continue
                resid = (p - q.to(p.device)).clamp(min=0)
                bonus = int(torch.multinomial((resid / resid.sum().clamp(min=1e-30)).cpu(), 1, generator=self.gen)) \
                    if float(resid.sum()) > 0 else int(p.argmax())
                break
            if bonus is None:
                bonus = int(torch.multinomial(self._probs(lt[g], sc).cpu(), 1, generator=self.gen))
            self.stats.accepted += n_acc
            new = prop[:n_acc] + [bonus]
            self.stats.generated += len(new)
            context.extend(new)
            if self.adaptive:
                if n_acc == g:
                    self.update_draft_k(self.gamma + 1)
                elif n_acc < g // 2:
                    self.update_draft_k(self.gamma - 1)
            return SpeculativeStepResult(new, g - n_acc, g, self.acceptance_rate())
        finally:
            T.free(), D.free()

    def _probs(self, logits_row, sc: SamplerConfig):
        if sc.temperature <= 0:
            p = torch.zeros_like(logits_row)
            p[int(logits_row.argmax())] = 1.0
            return p
        return _filtered_probs(logits_row.cpu(), sc.temperature, sc.top_k, sc.top_p, 1.0, None)

    @torch.no_grad()
    def generate(self, prompt_ids: Sequence[int], max_new_tokens: int = 64, sampling: Optional[SamplerConfig] = None, eos_id: int = -1):
        sc = sampling or SamplerConfig(temperature=0.0)
        total = min(len(prompt_ids) + max_new_tokens + self.max_gamma + 2, min(self.te.max_len, self.de.max_len))
        T, D = _Seq(self.te, total), _Seq(self.de, total)
        toks = list(prompt_ids)
        out: List[int] = []
        try:
            # prefill both; the target's last-position distribution gives the first token
            pt = self._probs(T.extend(toks)[-1], sc)
            D.extend(toks)
            self.stats.target_passes += 1
            nxt = int(torch.multinomial(pt.cpu(), 1, generator=self.gen))
            toks.append(nxt), out.append(nxt)
            while len(out) < max_new_tokens and nxt != eos_id and len(toks) + self.gamma + 1 < total:
                g = self.gamma
                # ---- draft proposes g tokens
                q_list, prop = [], []
                cur = list(toks)
                for _ in range(g):
                    q = self._probs(D.extend(cur)[-1], sc)
                    t = int(torch.multinomial(q.cpu(), 1, generator=self.gen))
                    q_list.append(q), prop.append(t), cur.append(t)
                # ---- target scores toks[-1], prop[0..g-1] in one pass: logits at the g+1 new positions
                lt = T.extend(cur, all_positions=True)           # rows: positions len(toks)-1 .. len(cur)-1
                self.stats.target_passes += 1
                self.stats.proposed += g
                n_acc, bonus = 0, None
                for i in range(g):
                    p = self._probs(lt[i], sc)
                    q = q_list[i]
                    t = prop[i]
                    if float(torch.rand((), generator=self.gen)) < min(1.0, float(p[t]) / max(float(q[t]), 1e-30)):
                        n_acc += 1
                        continue
                    resid = (p - q.to(p.device)).clamp(min=0)
                    bonus = int(torch.multinomial((resid / resid.sum().clamp(min=1e-30)).cpu(), 1, generator=self.gen)) \
                        if float(resid.sum()) > 0 else int(p.argmax())
                    break
                if bonus is None:                                 # everything accepted: one more token from the target for free
                    bonus = int(torch.multinomial(self._probs(lt[g], sc).cpu(), 1, generator=self.gen))
                self.stats.accepted += n_acc
                new = prop[:n_acc] + [bonus]
                for t in new:
                    toks.append(t), out.append(t)
                    if t == eos_id or len(out) >= max_new_tokens:
                        break
                nxt = out[-1]
                # positions beyond the accepted prefix are stale in both caches: rewind (they get overwritten)
                keep = len(toks) - 1
                T.rewind(min(T.pos, keep)), D.rewind(min(D.pos, keep))
                if self.adaptive:
                    if n_acc == g and self.gamma < self.max_gamma:
                        self.gamma += 1
                    elif n_acc < g // 2 and self.gamma > 1:
                        self.gamma -= 1
            self.stats.generated += len(out)
            return out[:max_new_tokens]
        finally:
            T.free(), D.free()


class TreeDecoder:
    """Draft tree with branching factor ``b`` and depth ``d``: the b^d candidate paths are verified greedily against the
    target; returns the longest accepted path plus the target's next token."""

    def __init__(self, target, draft, branching=2, depth=3):
        self.target, self.draft, self.b, self.d = target, draft, branching, depth

    @torch.no_grad()
    def step(self, ids: Sequence[int]):
        dev = self.target.tok_embeddings.device
        paths = [[]]
        for _ in range(self.d):
            nxt = []
            for p in paths:
                lg = self.draft.forward(torch.tensor([list(ids) + p], device=dev))[0, -1].float()
                for t in lg.topk(self.b).indices.tolist():
                    nxt.append(p + [t])
            paths = nxt
        best, best_tok = [], None
        for p in paths:
            lg = self.target.forward(torch.tensor([list(ids) + p], device=dev))[0].float()
            base = len(ids) - 1
            n = 0
            while n < len(p) and int(lg[base + n].argmax()) == p[n]:
                n += 1
            if n > len(best) or best_tok is None:
                best, best_tok = p[:n], int(lg[base + n].argmax())
        return best + [best_tok]

    def decode(self, prompt: Sequence[int], max_tokens: int, eos_id: int = -1) -> List[int]:
        """Generate up to ``max_tokens`` tokens, one verified tree step at a time; returns the new tokens."""
        out: List[int] = []
        while len(out) < max_tokens:
            step = self.step(list(prompt) + out)
            for t in step:
                out.append(t)
                if t == eos_id or len(out) >= max_tokens:
                    return out
        return out


# ================================================================================================ serving helpers
class DynamicBatcher:
    """Collects requests for up to ``window_s`` or ``max_batch`` items, then hands them out as one left-padded batch.
    With a model and tokenizer, ``batch_generate(prompts, max_tokens)`` answers a list of prompts in one continuous batch."""

    def __init__(self, max_batch=8, window_s=0.005, pad_id=0, model=None, tokenizer=None):
        self.max_batch, self.window_s, self.pad_id = max_batch, window_s, pad_id
        self.model, self.tok = model, tokenizer
        self.queue: List = []
        self.lock = threading.Condition()

    def batch_generate(self, prompts: Sequence[str], max_tokens: int, sampling: Optional[SamplerConfig] = None) -> List[str]:
        if self.model is None or self.tok is None:
            raise RuntimeError("batch_generate needs the batcher to be built with a model and a tokenizer")
        eng = InferenceEngine(self.model, self.tok, EngineConfig(max_batch=min(self.max_batch, max(1, len(prompts))),
                                                                 num_pages=max(64, 16 * len(prompts))))
        outs = eng.generate_batch([self.tok.encode(p) or [0] for p in prompts], max_tokens,
                                  sampling or SamplerConfig(temperature=0.0))
        eos = getattr(self.tok, "eos_id", -1)
        return [self.tok.decode([t for t in o if t != eos]) for o in outs]

    def submit(self, tokens: Sequence[int], tag=None):
        with self.lock:
            self.queue.append((time.perf_counter(), list(tokens), tag))
            self.lock.notify()

    def next_batch(self, timeout_s=1.0):
        """(ids [B, L] padded on the left, lengths, tags) or None when nothing arrived within the timeout."""
        end = time.perf_counter() + timeout_s
        with self.lock:
            while not self.queue:
                rest = end - time.perf_counter()
                if rest <= 0:
                    return None
                self.lock.wait(rest)
            first = self.queue[0][0]
            while len(self.queue) < self.max_batch and time.perf_counter() - first < self.window_s:
                self.lock.wait(self.window_s)
            items, self.queue = self.queue[: self.max_batch], self.queue[self.max_batch:]
        L = max(len(t) for _, t, _ in items)
        ids = torch.full((len(items), L), self.pad_id, dtype=torch.long)
        for i, (_, t, _) in enumerate(items):
            ids[i, L - len(t):] = torch.tensor(t)
        return ids, [len(t) for _, t, _ in items], [g for _, _, g in items]


class EmbeddingEndpoint:
    def __init__(self, model, tokenizer, normalize=True):
        self.model, self.tok, self.normalize = model, tokenizer, normalize

    @torch.no_grad()
    def embed(self, texts: Sequence[str]) -> torch.Tensor:
        dev = self.model.tok_embeddings.device
        out = []
        for t in texts:
            ids = self.tok.encode(t)[: self.model.cfg.max_seq_len] or [0]
            h = self.model.hidden_states(torch.tensor([ids], device=dev)).float().mean(0)
            out.append(torch.nn.functional.normalize(h, dim=0) if self.normalize else h)
        return torch.stack(out)


    embed_batch = embed


class Reranker:
    def __init__(self, endpoint: EmbeddingEndpoint):
        self.ep = endpoint

    def score(self, query: str, document: str) -> float:
        """Cosine similarity of the two mean-pooled embeddings."""
        return self.score_batch(query, [document])[0]

    def score_batch(self, query: str, documents: Sequence[str]) -> List[float]:
        e = torch.nn.functional.normalize(self.ep.embed([query] + list(documents)), dim=-1)
        return (e[1:] @ e[0]).tolist()

    def rerank(self, query: str, docs: Sequence[str], top_k: Optional[int] = None):
        e = self.ep.embed([query] + list(docs))
        scores = (e[1:] @ e[0]).tolist()
        order = sorted(range(len(docs)), key=lambda i: -scores[i])
        return [(i, scores[i]) for i in order[: top_k or len(docs)]]


class GrammarDecoder:
    """Token masks that keep generation inside a grammar.  ``mode='json'``: a prefix automaton of JSON (objects,
    arrays, strings, numbers, literals); ``mode='regex'``: the decoded text must stay a prefix of a match of ``pattern``
    (checked by partial matching).  ``mask(prefix_text)`` returns a bool tensor over the vocabulary."""

    def __init__(self, tokenizer, vocab_size: int, mode="json", pattern: Optional[str] = None, max_candidates: int = 0):
        self.tok, self.V, self.mode = tokenizer, vocab_size, mode
        self.pattern = pattern
        self.pieces = [tokenizer.decode([i]) for i in range(vocab_size)]
        self.max_candidates = max_candidates

    @staticmethod
    def json_prefix_ok(s: str) -> bool:
        """True when ``s`` can be extended to a valid JSON document."""
        stack, i, n = [], 0, len(s)
        state = "value"                     # value | after_value | key | colon
        while i < n:
            c = s[i]
            if c in " \t\n\r":
                i += 1
                continue
            if state in ("value", "value_or_close"):
                if state == "value_or_close" and c == "]":
                    stack.pop(); state = "after_value"; i += 1
                    continue
                if c == "{":
                    stack.append("{"); state = "key_or_close"; i += 1
                elif c == "[":
                    stack.append("["); state = "value_or_close"; i += 1
                elif c == '"':
                    j = GrammarDecoder._scan_string(s, i)
                    if j < 0:
                        return True          # inside an unfinished string: fine
                    i = j; state = "after_value"
                elif c in "-0123456789":
                    m = re.match(r"-?(0|[1-9]\d*)?(\.\d*)?([eE][+-]?\d*)?", s[i:])
                    j = i + m.end()
                    if m.end() == 0:
                        return False
                    if j == n:
                        return True
                    if not re.fullmatch(r"-?(0|[1-9]\d*)(\.\d+)?([eE][+-]?\d+)?", s[i:j]):
                        return False
                    i = j; state = "after_value"
                elif c in "tfn":
                    for lit in ("true", "false", "null"):
                        if s[i:i + len(lit)] == lit:
                            i += len(lit); state = "after_value"
                            break
                        if lit.startswith(s[i:]):
                            return True
                    else:
                        return False
                else:
                    return False
            elif state in ("key", "key_or_close"):
                if state == "key_or_close" and c == "}":
                    stack.pop(); state = "after_value"; i += 1
                    continue
                if c != '"':
                    return False
                j = GrammarDecoder._scan_string(s, i)
                if j < 0:
                    return True
                i = j; state = "colon"
            elif state == "colon":
                if c != ":":
                    return False
                i += 1; state = "value"
            elif state == "after_value":
                if not stack:
                    return False               # trailing garbage after a complete document
                if c == ",":
                    state = "key" if stack[-1] == "{" else "value"; i += 1
                elif c == "}" and stack[-1] == "{":
                    stack.pop(); i += 1
                elif c == "]" and stack[-1] == "[":
                    stack.pop(); i += 1
                else:
                    return False
        return True

    @staticmethod
    def _scan_string(s, i):
        j = i + 1
        while j < len(s):
            if s[j] == "\\":
                j += 2
                continue
            if s[j] == '"':
                return j + 1
            if ord(s[j]) < 0x20:
                return len(s) + 1              # control character inside a string: treated as a dead end by the caller
            j += 1
        return -1

    def regex_prefix_ok(self, s: str) -> bool:
        """Partial match by progressively truncating the pattern is not available in ``re``; accept when some extension
        of ``s`` by pattern-derived filler matches: checked with a fullmatch of s against every prefix-closed form."""
        if self._pfx is None:
            self._pfx = _prefix_regex(self.pattern)
        return self._pfx.fullmatch(s) is not None

    _pfx = None

    def mask(self, prefix_text: str, candidates: Optional[Sequence[int]] = None) -> torch.Tensor:
        ok = torch.zeros(self.V, dtype=torch.bool)
        check = self.json_prefix_ok if self.mode == "json" else self.regex_prefix_ok
        for i in (candidates if candidates is not None else range(self.V)):
            piece = self.pieces[i]
            if piece and check(prefix_text + piece):
                ok[i] = True
        return ok

    def constrain(self, logits: torch.Tensor, prefix_text: str, top: int = 64) -> torch.Tensor:
        """Mask ``logits`` [V]: only the ``top`` highest-scoring tokens are checked (all tokens if none of them fits)."""
        cand = logits.topk(min(top, self.V)).indices.tolist()
        m = self.mask(prefix_text, cand)
        if not m.any():
            m = self.mask(prefix_text)
        return logits.masked_fill(~m.to(logits.device), float("-inf"))


def _prefix_regex(pattern: str):
    """Regex accepting every prefix of a match of ``pattern`` (for patterns built from literals, classes, groups, |, ?, *, +)."""
    try:
        import re._parser as sre_parse
    except ImportError:      # Python < 3.11
        import sre_parse

    def pref(items):
        """alternatives: for a sequence x1 x2 ... xn -> (x1 x2 ... x_{k-1} prefix(x_k))? for every k"""
        alts = [""]
        done = ""
        for op, av in items:
            alts.append(done + one_prefix(op, av))
            done += emit(op, av)
        alts.append(done)
        return "(?:" + "|".join(a for a in alts) + ")"

    def emit(op, av):
        n = str(op)
        if n == "LITERAL":
            return re.escape(chr(av))
        if n == "NOT_LITERAL":
            return "[^" + re.escape(chr(av)) + "]"
        if n == "ANY":
            return "."
        if n == "IN":
            return "[" + "".join(emit_in(o, a) for o, a in av) + "]"
        if n in ("MAX_REPEAT", "MIN_REPEAT"):
            lo, hi, sub = av
            body = "(?:" + "".join(emit(o, a) for o, a in sub) + ")"
            return body + "{%d,%s}" % (lo, "" if hi >= 4294967295 or str(hi) == "MAXREPEAT" else hi)
        if n == "SUBPATTERN":
            return "(?:" + "".join(emit(o, a) for o, a in av[3]) + ")"
        if n == "BRANCH":
            return "(?:" + "|".join("".join(emit(o, a) for o, a in br) for br in av[1]) + ")"
        if n == "AT":
            return ""
        raise ValueError(f"unsupported regex element {n}")

    def emit_in(op, av):
        n = str(op)
        if n == "LITERAL":
            return re.escape(chr(av))
        if n == "RANGE":
            return re.escape(chr(av[0])) + "-" + re.escape(chr(av[1]))
        if n == "NEGATE":
            return "^"
        if n == "CATEGORY":
            return {"CATEGORY_DIGIT": "\\d", "CATEGORY_WORD": "\\w", "CATEGORY_SPACE": "\\s", "CATEGORY_NOT_DIGIT": "\\D",
                    "CATEGORY_NOT_WORD": "\\W", "CATEGORY_NOT_SPACE": "\\S"}[str(av)]
        raise ValueError(f"unsupported class element {n}")

    def one_prefix(op, av):
        n = str(op)
        if n in ("LITERAL", "NOT_LITERAL", "ANY", "IN", "AT"):
            return ""                                   # a single character has only the empty proper prefix
        if n in ("MAX_REPEAT", "MIN_REPEAT"):
            lo, hi, sub = av
            body = "(?:" + "".join(emit(o, a) for o, a in sub) + ")"
            cap = "" if hi >= 4294967295 or str(hi) == "MAXREPEAT" else max(0, hi - 1)
            return body + "{0,%s}" % cap + pref(list(sub))
        if n == "SUBPATTERN":
            return pref(list(av[3]))
        if n == "BRANCH":
            return "(?:" + "|".join(pref(list(br)) for br in av[1]) + ")"
        raise ValueError(f"unsupported regex element {n}")

    return re.compile(pref(list(sre_parse.parse(pattern))), re.S)


# ================================================================================================ low precision
class INT8Inference:
    """Weight-only int8 linear: per-output-row absmax scales; y = (x @ Wq^T) * scale."""

    def __init__(self, weight: torch.Tensor):
        w = weight.float()
        self.scale = (w.abs().amax(1, keepdim=True) / 127.0).clamp(min=1e-12)
        self.q = torch.clamp(torch.round(w / self.scale), -127, 127).to(torch.int8)

    def forward(self, x):
        return (x.float() @ self.q.float().t()) * self.scale.t()

    def error(self, weight):
        return float((self.q.float() * self.scale - weight.float()).abs().max())


class FP8Inference:
    """FP8 linear on the block-scaled tensor-core GEMM (1x128 activation scales, 128x128 weight scales); on CPU the
    dequantised operands are multiplied in fp32."""

    def __init__(self, weight: torch.Tensor):
        from ..quant import fp8
        self.fp8 = fp8
        self.N, self.K = weight.shape
        self.qw, self.sw = fp8.quant_weight_128x128(weight.contiguous())

    def forward(self, x):
        qa, sa = self.fp8.quant_act_1x128(x.contiguous())
        return self.fp8.gemm_fp8(qa, sa, self.qw, self.sw)

    def forward_two_stage(self, x):
        """Two-stage residual accumulation: what the 8-bit activations lost (x minus their dequantised value) is quantised
        again with its own, much smaller scales and sent through a second GEMM, so the activation rounding error drops by
        about the fp8 step (1/16) at twice the tensor-core work.  Meant for long contexts, where that error accumulates.
        Reference counterpart: FP8Inference::forward_two_stage (include/quant/inference_opt.h:151-158)."""
        x = x.contiguous()
        qa, sa = self.fp8.quant_act_1x128(x)
        resid = (x.float() - self.fp8.dequant(qa, sa, 1)).to(x.dtype)
        qr, sr = self.fp8.quant_act_1x128(resid.contiguous())
        y = self.fp8.gemm_fp8(qa, sa, self.qw, self.sw)
        return y + self.fp8.gemm_fp8(qr, sr, self.qw, self.sw)


class ModelShard:
    """Layers [lo, hi) of a model as a callable stage (embedding on the first shard, head on the last)."""

    def __init__(self, model, lo, hi):
        self.model, self.lo, self.hi = model, lo, hi

    @torch.no_grad()
    def forward(self, x, B, S):
        from ..models.dense import block_forward
        m = self.model
        h = m.embed(x) if self.lo == 0 else x
        rope = m.rope(h.device)
        for i in range(self.lo, self.hi):
            h, _ = block_forward(m.cfg, m.layers[i], h, B, S, rope, save=False)
        if self.hi == m.cfg.num_layers:
            from ..models.dense import _norm_fwd
            f, _ = _norm_fwd(m.cfg, h, m.norm, m.norm_bias)
            return F.gemm(f, m.lm_head.data)
        return h
