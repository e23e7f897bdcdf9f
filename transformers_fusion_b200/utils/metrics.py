"""Evaluation metrics and the model evaluator.

Scalar metrics (accuracy, perplexity, precision/recall/F1 with a confusion matrix, BLEU, ROUGE-N/L) and
``ModelEvaluator`` (sliding-window perplexity, next-token accuracy, generation speed).

Reference counterparts: include/quant/metrics.h (accuracy / perplexity / f1 / bleu / rouge /
confusion_matrix), ``eval_classification`` and ModelEvaluator (src/trainer/eval.cpp:20-393)."""
from __future__ import annotations

import math
import time
from collections import Counter
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch


def accuracy(pred: Sequence[int], target: Sequence[int]) -> float:
    n = min(len(pred), len(target))
    return sum(int(a == b) for a, b in zip(pred, target)) / n if n else 0.0


def topk_accuracy(logits: torch.Tensor, target: Sequence[int], k: int = 1) -> float:
    """Fraction of rows whose target is among the k largest logits."""
    t = torch.as_tensor(target, device=logits.device).long()
    if t.numel() == 0:
        return 0.0
    top = logits.float().topk(min(k, logits.shape[-1]), -1).indices
    return float((top == t[:, None]).any(-1).float().mean())


def average_precision(scores: Sequence[float], relevant: Sequence[int]) -> float:
    """Area under the precision-recall steps of one ranked list (ties keep input order)."""
    order = sorted(range(len(scores)), key=lambda i: -scores[i])
    hits, ap = 0, 0.0
    for rank, i in enumerate(order, 1):
        if relevant[i]:
            hits += 1
            ap += hits / rank
    return ap / hits if hits else 0.0


def mean_average_precision(score_lists: Sequence[Sequence[float]], relevant_lists: Sequence[Sequence[int]]) -> float:
    """Mean of the per-query (or per-class) average precision; queries without a relevant item are skipped."""
    aps = [average_precision(s, r) for s, r in zip(score_lists, relevant_lists) if any(r)]
    return sum(aps) / len(aps) if aps else 0.0


def perplexity(mean_nll: float) -> float:
    return math.exp(min(mean_nll, 80.0))


def confusion_matrix(pred: Sequence[int], target: Sequence[int], num_classes: int):
    m = torch.zeros((num_classes, num_classes), dtype=torch.long)
    for p, t in zip(pred, target):
        if 0 <= p < num_classes and 0 <= t < num_classes:
            m[t, p] += 1
    return m


@dataclass
class ClassificationReport:
    accuracy: float = 0.0
    precision: float = 0.0
    recall: float = 0.0
    f1_score: float = 0.0
    confusion: torch.Tensor = None


def eval_classification(logits: torch.Tensor, labels: Sequence[int]) -> ClassificationReport:
    """Macro precision / recall / F1 over the classes that occur (as label or prediction)."""
    pred = logits.float().argmax(-1).tolist()
    labels = [int(x) for x in labels]
    classes = sorted(set(pred) | set(labels))
    idx = {c: i for i, c in enumerate(classes)}
    cm = confusion_matrix([idx[p] for p in pred], [idx[t] for t in labels], len(classes)).double()
    tp = cm.diag()
    prec = tp / cm.sum(0).clamp(min=1)
    rec = tp / cm.sum(1).clamp(min=1)
    f1 = 2 * prec * rec / (prec + rec).clamp(min=1e-12)
    return ClassificationReport(accuracy(pred, labels), float(prec.mean()), float(rec.mean()), float(f1.mean()), cm.long())


def f1_score(pred, target, positive=1) -> float:
    tp = sum(1 for p, t in zip(pred, target) if p == positive and t == positive)
    fp = sum(1 for p, t in zip(pred, target) if p == positive and t != positive)
    fn = sum(1 for p, t in zip(pred, target) if p != positive and t == positive)
    return 2 * tp / (2 * tp + fp + fn) if tp else 0.0


def _ngrams(tokens, n):
    return Counter(tuple(tokens[i:i + n]) for i in range(len(tokens) - n + 1))


def bleu(candidate: Sequence, references: Sequence[Sequence], max_n: int = 4, smooth: bool = True) -> float:
    """Corpus-free sentence BLEU with brevity penalty and add-one smoothing of the higher orders."""
    if not candidate:
        return 0.0
    logs = 0.0
    for n in range(1, max_n + 1):
        c = _ngrams(candidate, n)
        best = Counter()
        for r in references:
            for g, k in _ngrams(r, n).items():
                best[g] = max(best[g], k)
        match = sum(min(k, best[g]) for g, k in c.items())
        total = max(1, sum(c.values()))
        if n > 1 and smooth:
            match, total = match + 1, total + 1
        if match == 0:
            return 0.0
        logs += math.log(match / total) / max_n
    ref_len = min((abs(len(r) - len(candidate)), len(r)) for r in references)[1]
    bp = 1.0 if len(candidate) >= ref_len else math.exp(1 - ref_len / len(candidate))
    return bp * math.exp(logs)


def rouge_n(candidate, reference, n=1):
    c, r = _ngrams(candidate, n), _ngrams(reference, n)
    overlap = sum(min(k, r[g]) for g, k in c.items())
    p = overlap / max(1, sum(c.values()))
    rc = overlap / max(1, sum(r.values()))
    return {"precision": p, "recall": rc, "f1": 2 * p * rc / (p + rc) if p + rc else 0.0}


def rouge_l(candidate, reference):
    a, b = list(candidate), list(reference)
    prev = [0] * (len(b) + 1)
    for x in a:
        cur = [0]
        for j, y in enumerate(b):
            cur.append(prev[j] + 1 if x == y else max(prev[j + 1], cur[j]))
        prev = cur
    l = prev[-1]
    p, r = l / max(1, len(a)), l / max(1, len(b))
    return {"precision": p, "recall": r, "f1": 2 * p * r / (p + r) if p + r else 0.0}


# ---- accumulating metric objects (reference: include/quant/metrics.h): ``update`` takes tensors of one batch and the
# object keeps running totals, so a metric can be fed batch by batch on the device and read at the end
def _ids(t) -> torch.Tensor:
    return t.reshape(-1).long() if torch.is_tensor(t) else torch.tensor(list(t), dtype=torch.long)


class Accuracy:
    """Top-k accuracy.  ``predictions``: class scores [N, C] (or class ids [N] for k = 1)."""

    def __init__(self, top_k: int = 1):
        self._k = top_k
        self.reset()

    def reset(self): self._correct = self._total = 0
    def correct(self) -> int: return self._correct
    def total(self) -> int: return self._total
    def top_k(self) -> int: return self._k
    def value(self) -> float: return self._correct / self._total if self._total else 0.0

    def update(self, predictions: torch.Tensor, targets) -> float:
        t = _ids(targets).to(predictions.device)
        if predictions.dim() == 1:
            hit = predictions.long() == t
        else:
            p = predictions.reshape(-1, predictions.shape[-1])
            hit = (p.topk(min(self._k, p.shape[-1]), -1).indices == t[:, None]).any(-1)
        self._correct += int(hit.sum())
        self._total += t.numel()
        return self.value()


class Perplexity:
    """exp(mean negative log-likelihood) over everything fed so far; targets equal to ``ignore_index`` are skipped."""

    def __init__(self, ignore_index: int = -100):
        self.ignore_index = ignore_index
        self.reset()

    def reset(self): self._nll, self._count = 0.0, 0
    def nll(self) -> float: return self._nll
    def count(self) -> int: return self._count
    def value(self) -> float: return perplexity(self._nll / self._count) if self._count else float("inf")

    def update(self, logits: torch.Tensor, targets) -> float:
        t = _ids(targets).to(logits.device)
        lp = torch.log_softmax(logits.reshape(-1, logits.shape[-1]).float(), -1)
        keep = t != self.ignore_index
        self._nll += float(-lp[keep].gather(1, t[keep][:, None]).sum())
        self._count += int(keep.sum())
        return self.value()


class ConfusionMatrix:
    """``at(pred, true)`` counts; rows are predictions."""

    def __init__(self, num_classes: int):
        self._n = num_classes
        self.reset()

    def reset(self): self.matrix = torch.zeros(self._n, self._n, dtype=torch.long)

    def update(self, predictions: torch.Tensor, targets, from_logits: Optional[bool] = None):
        if from_logits or (from_logits is None and torch.is_tensor(predictions) and predictions.dim() > 1):
            predictions = predictions.reshape(-1, predictions.shape[-1]).argmax(-1)
        p, t = _ids(predictions).cpu(), _ids(targets).cpu()
        ok = (p >= 0) & (p < self._n) & (t >= 0) & (t < self._n)
        self.matrix += torch.bincount(p[ok] * self._n + t[ok], minlength=self._n * self._n).view(self._n, self._n)

    def at(self, pred_class: int, true_class: int) -> int: return int(self.matrix[pred_class, true_class])
    def true_positive(self, c: int) -> int: return int(self.matrix[c, c])
    def false_positive(self, c: int) -> int: return int(self.matrix[c].sum() - self.matrix[c, c])
    def false_negative(self, c: int) -> int: return int(self.matrix[:, c].sum() - self.matrix[c, c])
    def total_samples(self) -> int: return int(self.matrix.sum())
    def num_classes(self) -> int: return self._n
    def data(self) -> List[int]: return self.matrix.reshape(-1).tolist()


class F1Score:
    """Per-class, macro and support-weighted precision / recall / F1 (``class_idx`` -1: the macro average)."""

    def __init__(self, num_classes: int = 2):
        self.cm = ConfusionMatrix(num_classes)

    def reset(self): self.cm.reset()
    def num_classes(self) -> int: return self.cm.num_classes()
    def update(self, predictions, targets): self.cm.update(predictions, targets)

    def _one(self, c: int):
        tp, fp, fn = self.cm.true_positive(c), self.cm.false_positive(c), self.cm.false_negative(c)
        p = tp / (tp + fp) if tp + fp else 0.0
        r = tp / (tp + fn) if tp + fn else 0.0
        return p, r, (2 * p * r / (p + r) if p + r else 0.0)

    def _avg(self, k: int, c: int) -> float:
        if c >= 0:
            return self._one(c)[k]
        return sum(self._one(i)[k] for i in range(self.num_classes())) / max(1, self.num_classes())

    def precision(self, class_idx: int = -1) -> float: return self._avg(0, class_idx)
    def recall(self, class_idx: int = -1) -> float: return self._avg(1, class_idx)
    def f1(self, class_idx: int = -1) -> float: return self._avg(2, class_idx)
    def macro_f1(self) -> float: return self._avg(2, -1)

    def weighted_f1(self) -> float:
        sup = self.cm.matrix.sum(0).tolist()
        return sum(self._one(i)[2] * sup[i] for i in range(self.num_classes())) / max(1, sum(sup))


class BLEUScore:
    def __init__(self, max_n: int = 4, smooth: bool = True):
        self._n, self.smooth = max_n, smooth

    def max_n(self) -> int: return self._n

    def compute(self, candidate, reference) -> float:
        return bleu(_ids(candidate).tolist(), [_ids(reference).tolist()], self._n, self.smooth)


class ROUGELScore:
    def compute(self, candidate, reference) -> float:
        """The F-measure of the longest common subsequence."""
        return rouge_l(_ids(candidate).tolist(), _ids(reference).tolist())["f1"]


class MeanAveragePrecision:
    """``compute(scores, labels)`` adds one query (scores of its candidates, 0 / 1 relevance labels) and returns its average
    precision; ``value`` is the mean over the queries so far."""

    def __init__(self): self.reset()
    def reset(self): self.ap_scores: List[float] = []
    def value(self) -> float: return sum(self.ap_scores) / len(self.ap_scores) if self.ap_scores else 0.0

    def compute(self, scores, labels) -> float:
        sc = scores.reshape(-1).tolist() if torch.is_tensor(scores) else list(scores)
        lb = _ids(labels).tolist()
        ap = average_precision(sc, [int(r > 0) for r in lb])
        self.ap_scores.append(ap)
        return ap


def load_eval_tokens(path, max_tokens=0, tokenizer=None) -> List[int]:
    """Whitespace-separated integer ids, or text run through ``tokenizer`` when the file is not numeric."""
    text = open(path, "r", encoding="utf-8", errors="ignore").read()
    parts = text.split()
    try:
        ids = [int(p) for p in parts[: max_tokens or None]]
    except ValueError:
        if tokenizer is None:
            raise
        ids = tokenizer.encode(text)
    return ids[:max_tokens] if max_tokens else ids


@dataclass
class EvalResult:
    name: str = ""
    loss: float = 0.0
    perplexity: float = 0.0
    accuracy: float = 0.0
    correct: int = 0
    total: int = 0
    total_tokens: int = 0
    tokens_per_sec: float = 0.0
    elapsed_s: float = 0.0


class ModelEvaluator:
    def __init__(self, model, batch_size: int = 1):
        self.model, self.batch_size = model, batch_size
        self.results: List[EvalResult] = []

    def set_batch_size(self, n):
        self.batch_size = max(1, int(n))

    def _device(self):
        return self.model.tok_embeddings.device

    @torch.no_grad()
    def _nll_windows(self, tokens, context, stride):
        """Yields (nll [n], pred [n], target [n]) for the scored tail of each window."""
        dev = self._device()
        V = self.model.cfg.vocab_size
        starts = list(range(0, max(1, len(tokens) - 1), stride))
        batch = []
        for s in starts:
            w = tokens[s:s + context + 1]
            if len(w) < 2:
                continue
            new_from = 0 if s == 0 else max(0, context - stride)
            batch.append((w, new_from))
            if s + context + 1 >= len(tokens):
                break
        for i in range(0, len(batch), self.batch_size):
            grp = batch[i:i + self.batch_size]
            L = max(len(w) for w, _ in grp) - 1
            ids = torch.zeros((len(grp), L), dtype=torch.long)
            for j, (w, _) in enumerate(grp):
                ids[j, : len(w) - 1] = torch.tensor(w[:-1])
            logits = self.model.forward(ids.to(dev)).float()
            lp = torch.log_softmax(logits, -1)
            for j, (w, nf) in enumerate(grp):
                n = len(w) - 1
                tgt = torch.tensor(w[1:], device=dev).clamp(0, V - 1)
                row = lp[j, :n]
                nll = -row.gather(1, tgt[:, None])[:, 0]
                yield nll[nf:], row.argmax(-1)[nf:], tgt[nf:]

    def evaluate_perplexity(self, tokens, name="perplexity", context=512, stride=0) -> EvalResult:
        stride = stride or max(1, context // 2)
        t0 = time.perf_counter()
        tot, n = 0.0, 0
        for nll, _, _ in self._nll_windows(tokens, context, stride):
            tot += float(nll.sum())
            n += nll.numel()
        r = EvalResult(name, tot / max(1, n), perplexity(tot / max(1, n)), total_tokens=n, elapsed_s=time.perf_counter() - t0)
        self.results.append(r)
        return r

    def evaluate_accuracy(self, tokens, name="accuracy", context=512) -> EvalResult:
        ok = n = 0
        for _, pred, tgt in self._nll_windows(tokens, context, context):
            ok += int((pred == tgt).sum())
            n += tgt.numel()
        r = EvalResult(name, accuracy=ok / max(1, n), correct=ok, total=n, total_tokens=n)
        self.results.append(r)
        return r

    def run_all(self, eval_tokens, context: int = 512, generation: Optional[bool] = None) -> List[EvalResult]:
        """Perplexity and next-token accuracy on ``eval_tokens`` and, where the model can be served (a CUDA device), the
        generation-speed measurement; returns the results in that order."""
        ctx = min(context, self.model.cfg.max_seq_len)
        out = [self.evaluate_perplexity(eval_tokens, context=ctx), self.evaluate_accuracy(eval_tokens, context=ctx)]
        if generation if generation is not None else self._device().type == "cuda":
            out.append(self.evaluate_generation(prompt_len=min(32, max(1, self.model.cfg.max_seq_len // 4))))
        return out

    def evaluate_generation(self, prompt_len=32, new_tokens=128, name="generation") -> EvalResult:
        from ..inference.engine import EngineConfig, InferenceEngine
        from ..inference.sampler import SamplerConfig
        cfg = self.model.cfg
        new_tokens = min(new_tokens, cfg.max_seq_len - prompt_len - 1)
        eng = InferenceEngine(self.model, None, EngineConfig(num_pages=max(64, 2 * cfg.max_seq_len // 16)))
        prompt = [int(x) % cfg.vocab_size for x in range(3, 3 + prompt_len)]
        t0 = time.perf_counter()
        out = eng.generate_batch([prompt], new_tokens, SamplerConfig(0.0))
        dt = time.perf_counter() - t0
        r = EvalResult(name, total_tokens=len(out[0]), tokens_per_sec=len(out[0]) / max(dt, 1e-9), elapsed_s=dt)
        self.results.append(r)
        return r
