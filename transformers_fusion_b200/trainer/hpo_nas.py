"""Hyper-parameter optimisation and architecture search around a user-supplied evaluation function.

``HPOEngine``: random search, Bayesian optimisation (RBF Gaussian-process surrogate, UCB acquisition), population-based
training (truncation selection, exploit + explore), successive halving; evaluation history, best / top-k, JSON save / load.
``NASEngine``: evolutionary search over (layers, width, heads, FFN, vocab, dropout) with mutation operators, a parameter /
memory / latency model and hardware-constraint penalties.

Reference counterparts: include/quant/hpo_nas.h:15-260, src/trainer/hpo_nas.cpp."""
from __future__ import annotations

import json
import math
import random
from dataclasses import asdict, dataclass, field
from typing import Callable, List, Optional, Sequence, Tuple


@dataclass
class SearchSpace:
    lr_min: float = 1e-5
    lr_max: float = 1e-1
    wd_min: float = 1e-6
    wd_max: float = 1e-1
    beta1_min: float = 0.7
    beta1_max: float = 0.999
    warmup_min: int = 0
    warmup_max: int = 1000
    batch_size_min: int = 1
    batch_size_max: int = 256
    depth_min: int = 1
    depth_max: int = 48
    width_min: int = 64
    width_max: int = 4096
    heads_min: int = 1
    heads_max: int = 64
    ffn_ratio_min: float = 1.0
    ffn_ratio_max: float = 8.0
    dropout_min: float = 0.0
    dropout_max: float = 0.5


@dataclass
class HPConfig:
    id: int = 0
    lr: float = 3e-4
    weight_decay: float = 1e-2
    beta1: float = 0.9
    beta2: float = 0.999
    warmup_steps: int = 100
    batch_size: int = 32
    dropout: float = 0.1
    depth: int = 12
    width: int = 768
    num_heads: int = 12
    ffn_ratio: float = 4.0
    score: float = 0.0
    val_loss: float = 1e10
    train_loss: float = 1e10
    epoch: int = 0
    alive: bool = True


@dataclass
class Architecture:
    id: int = 0
    num_layers: int = 12
    hidden_size: int = 768
    num_heads: int = 12
    ffn_size: int = 3072
    vocab_size: int = 32000
    dropout: float = 0.1
    score: float = 0.0
    val_loss: float = 1e10
    latency_ms: float = 0.0
    param_count: int = 0
    memory_bytes: int = 0
    alive: bool = True


@dataclass
class HardwareConstraints:
    target_latency_ms: float = 10.0
    target_memory_bytes: int = 1 << 30
    max_params: int = 1_000_000_000
    enabled: bool = False


@dataclass
class SuccessiveHalvingConfig:
    n_configs: int = 0
    n_rungs: int = 0
    reduction_factor: float = 3.0
    configs_per_rung: List[int] = field(default_factory=list)
    budget_per_rung: List[float] = field(default_factory=list)


class HPOEngine:
    """``evaluate(config, budget) -> score`` (higher is better) is supplied by the caller; ``budget`` is a relative
    amount of training (epochs, steps...) that successive halving and PBT grow."""

    def __init__(self, evaluate: Optional[Callable[[HPConfig, float], float]] = None, seed: int = 0):
        self.evaluate_fn = evaluate
        self.space = SearchSpace()
        self.hw = HardwareConstraints()
        self.history: List[Tuple[HPConfig, float]] = []
        self.gp_x: List[List[float]] = []
        self.gp_y: List[float] = []
        self.rng = random.Random(seed)
        self._next = 0

    def set_search_space(self, s):
        self.space = s

    # ---- a ready-made objective: short training runs of a given trainer (reference: HPOEngine::set_trainer / set_model,
    # include/quant/hpo_nas.h:146-147)
    def set_model(self, model):
        self.model = model

    def set_trainer(self, trainer, loader=None, steps_per_budget: int = 8):
        """Score a configuration by training ``trainer``'s model from its CURRENT weights for ``budget x steps_per_budget``
        steps with the configuration's learning rate, weight decay and warm-up, and returning minus the mean loss of the last
        quarter of the steps.  Weights, optimizer state and step counter are put back after every trial, so trials are
        comparable.  Used when no ``evaluate`` callable was given."""
        self.trainer, self.loader, self.steps_per_budget = trainer, loader, steps_per_budget
        self.model = getattr(trainer, "model", getattr(self, "model", None))
        if self.evaluate_fn is None:
            self.evaluate_fn = self._train_objective

    def _train_objective(self, c: HPConfig, budget: float) -> float:
        import torch
        t, dl = self.trainer, self.loader
        if dl is None:
            raise RuntimeError("set_trainer needs a data loader for the built-in objective")
        flat = t.model.flat
        w0 = flat.params.clone()
        opt_sd = {k: (v.clone() if torch.is_tensor(v) else ({a: b.clone() for a, b in v.items()} if isinstance(v, dict) else v))
                  for k, v in t.opt.state_dict().items()} if hasattr(t.opt, "state_dict") else None
        cfg0 = (t.cfg.learning_rate, t.cfg.weight_decay, t.cfg.warmup_steps, t.global_step)
        t.cfg.learning_rate, t.cfg.weight_decay, t.cfg.warmup_steps, t.global_step = c.lr, c.weight_decay, c.warmup_steps, 0
        for o in (t.opt, getattr(t, "engine", None) and getattr(t.engine, "opt", None)):
            if o is not None and hasattr(o, "wd"):
                o.wd = c.weight_decay
        n = max(1, int(round(budget * self.steps_per_budget)))
        losses = []
        try:
            for _ in range(n):
                if hasattr(dl, "has_next") and not dl.has_next():
                    dl.reset()
                losses.append(float(t.train_step(*dl.next_batch())))
        finally:
            flat.params.copy_(w0)
            if opt_sd is not None:
                t.opt.load_state_dict(opt_sd)
            t.cfg.learning_rate, t.cfg.weight_decay, t.cfg.warmup_steps, t.global_step = cfg0
        tail = losses[-max(1, n // 4):]
        c.val_loss = sum(tail) / len(tail)
        return -c.val_loss if math.isfinite(c.val_loss) else -1e30

    def get_search_space(self):
        return self.space

    def set_hardware_constraints(self, hc):
        self.hw = hc

    # ---- sampling
    def _log_uniform(self, lo, hi):
        return math.exp(self.rng.uniform(math.log(lo), math.log(hi)))

    def random_sample(self) -> HPConfig:
        s = self.space
        heads = self.rng.randint(s.heads_min, min(s.heads_max, 64))
        width = max(s.width_min, min(s.width_max, heads * 16 * self.rng.randint(1, max(1, s.width_max // (heads * 16)))))
        c = HPConfig(id=self._next, lr=self._log_uniform(s.lr_min, s.lr_max), weight_decay=self._log_uniform(s.wd_min, s.wd_max),
                     beta1=self.rng.uniform(s.beta1_min, s.beta1_max), warmup_steps=self.rng.randint(s.warmup_min, s.warmup_max),
                     batch_size=self.rng.randint(s.batch_size_min, s.batch_size_max), dropout=self.rng.uniform(s.dropout_min, s.dropout_max),
                     depth=self.rng.randint(s.depth_min, s.depth_max), width=width, num_heads=heads,
                     ffn_ratio=self.rng.uniform(s.ffn_ratio_min, s.ffn_ratio_max))
        self._next += 1
        return c

    def _eval(self, c: HPConfig, budget=1.0) -> float:
        score = float(self.evaluate_fn(c, budget)) if self.evaluate_fn else -c.val_loss
        if self.hw.enabled:
            score -= self.compute_hardware_penalty(Architecture(num_layers=c.depth, hidden_size=c.width, num_heads=c.num_heads,
                                                                ffn_size=int(c.width * c.ffn_ratio)))
        c.score = score
        self.record_eval(c, score)
        return score

    def record_eval(self, c, score):
        self.history.append((c, score))
        self.surrogate_update(c, score)

    def get_eval_history(self):
        return list(self.history)

    def random_search(self, n_configs) -> List[HPConfig]:
        cs = [self.random_sample() for _ in range(n_configs)]
        for c in cs:
            self._eval(c)
        return sorted(cs, key=lambda c: -c.score)

    # ---- Bayesian optimisation
    def config_to_features(self, c: HPConfig) -> List[float]:
        s = self.space

        def norm(v, lo, hi, log=False):
            if log:
                v, lo, hi = math.log(v), math.log(lo), math.log(hi)
            return (v - lo) / max(hi - lo, 1e-12)
        return [norm(c.lr, s.lr_min, s.lr_max, True), norm(c.weight_decay, s.wd_min, s.wd_max, True), norm(c.beta1, s.beta1_min, s.beta1_max),
                norm(c.warmup_steps, s.warmup_min, max(1, s.warmup_max)), norm(c.batch_size, s.batch_size_min, s.batch_size_max),
                norm(c.dropout, s.dropout_min, max(s.dropout_max, 1e-6)), norm(c.depth, s.depth_min, s.depth_max),
                norm(c.width, s.width_min, s.width_max), norm(c.ffn_ratio, s.ffn_ratio_min, s.ffn_ratio_max)]

    @staticmethod
    def rbf_kernel(x1, x2, length_scale=0.3):
        return math.exp(-sum((a - b) ** 2 for a, b in zip(x1, x2)) / (2 * length_scale ** 2))

    def surrogate_update(self, c, score):
        self.gp_x.append(self.config_to_features(c))
        self.gp_y.append(score)
        self._alpha = None

    def _fit(self):
        import numpy as np
        n = len(self.gp_x)
        K = np.array([[self.rbf_kernel(a, b) for b in self.gp_x] for a in self.gp_x]) + 1e-4 * np.eye(n)
        y = np.array(self.gp_y)
        self._mu, self._sd = float(y.mean()), float(y.std() + 1e-9)
        self._Kinv = np.linalg.inv(K)
        self._alpha = self._Kinv @ ((y - self._mu) / self._sd)

    def _posterior(self, c):
        import numpy as np
        if not self.gp_x:
            return 0.0, 1.0
        if getattr(self, "_alpha", None) is None:
            self._fit()
        k = np.array([self.rbf_kernel(self.config_to_features(c), x) for x in self.gp_x])
        mean = float(k @ self._alpha) * self._sd + self._mu
        var = max(1e-9, 1.0 - float(k @ self._Kinv @ k))
        return mean, math.sqrt(var) * self._sd

    def surrogate_predict(self, c):
        return self._posterior(c)[0]

    def acquisition_function(self, c, n_evaluations):
        m, s = self._posterior(c)
        return m + math.sqrt(2 * math.log(max(2, n_evaluations))) * s       # upper confidence bound

    def bayesian_optimization(self, n_initial=5, n_iterations=20, n_candidates=200) -> List[HPConfig]:
        cs = [self.random_sample() for _ in range(n_initial)]
        for c in cs:
            self._eval(c)
        for it in range(n_iterations):
            cand = [self.random_sample() for _ in range(n_candidates)]
            best = max(cand, key=lambda c: self.acquisition_function(c, len(self.history)))
            self._eval(best)
            cs.append(best)
        return sorted(cs, key=lambda c: -c.score)

    # ---- PBT
    def select_parent(self, population):
        top = sorted(population, key=lambda c: -c.score)[: max(1, len(population) // 4)]
        return self.rng.choice(top)

    def exploit_and_explore(self, child: HPConfig, parent: HPConfig, perturbation_factor=0.2):
        s = self.space
        for f in ("lr", "weight_decay", "beta1", "dropout", "ffn_ratio"):
            v = getattr(parent, f) * self.rng.choice([1 - perturbation_factor, 1 + perturbation_factor])
            lo, hi = {"lr": (s.lr_min, s.lr_max), "weight_decay": (s.wd_min, s.wd_max), "beta1": (s.beta1_min, s.beta1_max),
                      "dropout": (s.dropout_min, s.dropout_max), "ffn_ratio": (s.ffn_ratio_min, s.ffn_ratio_max)}[f]
            setattr(child, f, min(hi, max(lo, v)))
        for f in ("depth", "width", "num_heads", "batch_size", "warmup_steps"):
            setattr(child, f, getattr(parent, f))
        return child

    def population_based_training(self, n_population=8, n_generations=10) -> List[HPConfig]:
        pop = [self.random_sample() for _ in range(n_population)]
        for g in range(n_generations):
            for c in pop:
                c.epoch = g + 1
                self._eval(c, budget=g + 1)
            pop.sort(key=lambda c: -c.score)
            cut = max(1, n_population // 4)
            for loser in pop[-cut:]:
                self.exploit_and_explore(loser, self.select_parent(pop[:-cut] or pop))
        return pop

    # ---- successive halving
    def setup_successive_halving(self, n_configs=27, n_rungs=5, reduction_factor=3.0) -> SuccessiveHalvingConfig:
        cfg = SuccessiveHalvingConfig(n_configs, n_rungs, reduction_factor)
        n, b = n_configs, 1.0
        for _ in range(n_rungs):
            cfg.configs_per_rung.append(max(1, int(n)))
            cfg.budget_per_rung.append(b)
            n, b = n / reduction_factor, b * reduction_factor
            if cfg.configs_per_rung[-1] == 1:
                break
        cfg.n_rungs = len(cfg.configs_per_rung)
        return cfg

    def successive_halving(self, n_configs=27, n_rungs=5) -> List[HPConfig]:
        plan = self.setup_successive_halving(n_configs, n_rungs)
        alive = [self.random_sample() for _ in range(n_configs)]
        for keep, budget in zip(plan.configs_per_rung, plan.budget_per_rung):
            alive = alive[:keep]
            for c in alive:
                self._eval(c, budget)
            alive.sort(key=lambda c: -c.score)
        return alive

    def optimize(self, n_budget=100, method="pbt") -> HPConfig:
        if method == "random":
            self.random_search(n_budget)
        elif method in ("bayes", "bayesian"):
            self.bayesian_optimization(min(5, n_budget), max(0, n_budget - 5))
        elif method in ("sha", "successive_halving"):
            self.successive_halving(n_budget)
        else:
            pop = max(2, min(8, n_budget))
            self.population_based_training(pop, max(1, n_budget // pop))
        return self.get_best()

    def get_best(self) -> HPConfig:
        return max(self.history, key=lambda t: t[1])[0]

    def get_top_k(self, k):
        seen, out = set(), []
        for c, s in sorted(self.history, key=lambda t: -t[1]):
            if c.id not in seen:
                seen.add(c.id)
                out.append(c)
            if len(out) >= k:
                break
        return out

    def save_best_configs(self, path, top_k=5) -> bool:
        try:
            with open(path, "w") as f:
                json.dump([asdict(c) for c in self.get_top_k(top_k)], f, indent=1)
            return True
        except OSError:
            return False

    @staticmethod
    def load_configs(path) -> List[HPConfig]:
        with open(path) as f:
            return [HPConfig(**d) for d in json.load(f)]

    def compute_hardware_penalty(self, arch: Architecture) -> float:
        NASEngine.estimate(arch)
        h = self.hw
        pen = 0.0
        if arch.param_count > h.max_params:
            pen += arch.param_count / h.max_params - 1
        if arch.memory_bytes > h.target_memory_bytes:
            pen += arch.memory_bytes / h.target_memory_bytes - 1
        if arch.latency_ms > h.target_latency_ms:
            pen += arch.latency_ms / h.target_latency_ms - 1
        return pen


class NASMutateOp:
    ADD_LAYER, REMOVE_LAYER, CHANGE_WIDTH, CHANGE_HEADS, CHANGE_FFN, CHANGE_DROPOUT, CHANGE_VOCAB = range(7)


@dataclass
class NASConfig:
    population: int = 16
    generations: int = 10
    mutation_rate: float = 0.3
    elite_fraction: float = 0.25
    tflops: float = 1000.0           # sustained matrix throughput used by the latency model
    tokens: int = 4096               # tokens per forward pass in the latency model


class NASEngine:
    def __init__(self, evaluate: Optional[Callable[[Architecture], float]] = None, cfg: Optional[NASConfig] = None,
                 hw: Optional[HardwareConstraints] = None, seed=0):
        self.evaluate_fn, self.cfg, self.hw = evaluate, cfg or NASConfig(), hw or HardwareConstraints()
        self.rng = random.Random(seed)
        self.history: List[Architecture] = []
        self._next = 0

    @staticmethod
    def estimate(a: Architecture, tflops=1000.0, tokens=4096):
        per_layer = 4 * a.hidden_size * a.hidden_size + 3 * a.hidden_size * a.ffn_size + 2 * a.hidden_size
        a.param_count = a.num_layers * per_layer + 2 * a.vocab_size * a.hidden_size + a.hidden_size
        a.memory_bytes = a.param_count * 2
        a.latency_ms = 2.0 * a.param_count * tokens / (tflops * 1e12) * 1e3
        return a

    def random_architecture(self) -> Architecture:
        heads = self.rng.choice([4, 8, 12, 16, 32])
        hidden = heads * self.rng.choice([32, 64, 128])
        a = Architecture(id=self._next, num_layers=self.rng.randint(2, 32), hidden_size=hidden, num_heads=heads,
                         ffn_size=int(hidden * self.rng.choice([2, 2.75, 4])), dropout=self.rng.choice([0.0, 0.1]))
        self._next += 1
        return self.estimate(a, self.cfg.tflops, self.cfg.tokens)

    def mutate(self, a: Architecture, op: Optional[int] = None, magnitude=0.25) -> Architecture:
        b = Architecture(**asdict(a))
        b.id, self._next = self._next, self._next + 1
        op = self.rng.randrange(7) if op is None else op
        if op == NASMutateOp.ADD_LAYER:
            b.num_layers += 1
        elif op == NASMutateOp.REMOVE_LAYER:
            b.num_layers = max(1, b.num_layers - 1)
        elif op == NASMutateOp.CHANGE_WIDTH:
            hd = b.hidden_size // b.num_heads
            hd = max(16, int(round(hd * (1 + self.rng.choice([-1, 1]) * magnitude) / 16)) * 16)
            b.hidden_size = hd * b.num_heads
        elif op == NASMutateOp.CHANGE_HEADS:
            hd = max(16, b.hidden_size // b.num_heads)
            b.num_heads = max(1, b.num_heads + self.rng.choice([-1, 1]) * max(1, int(b.num_heads * magnitude)))
            b.hidden_size = hd * b.num_heads
        elif op == NASMutateOp.CHANGE_FFN:
            b.ffn_size = max(64, int(round(b.ffn_size * (1 + self.rng.choice([-1, 1]) * magnitude) / 64)) * 64)
        elif op == NASMutateOp.CHANGE_DROPOUT:
            b.dropout = min(0.5, max(0.0, b.dropout + self.rng.choice([-0.05, 0.05])))
        else:
            b.vocab_size = max(256, int(b.vocab_size * (1 + self.rng.choice([-1, 1]) * magnitude)))
        return self.estimate(b, self.cfg.tflops, self.cfg.tokens)

    def penalty(self, a: Architecture) -> float:
        if not self.hw.enabled:
            return 0.0
        h, pen = self.hw, 0.0
        pen += max(0.0, a.param_count / h.max_params - 1)
        pen += max(0.0, a.memory_bytes / h.target_memory_bytes - 1)
        pen += max(0.0, a.latency_ms / h.target_latency_ms - 1)
        return pen

    def score(self, a: Architecture) -> float:
        base = float(self.evaluate_fn(a)) if self.evaluate_fn else -a.val_loss
        a.score = base - self.penalty(a)
        self.history.append(a)
        return a.score

    def search(self, population: Optional[int] = None, generations: Optional[int] = None) -> Architecture:
        c = self.cfg
        if population or generations:
            c = NASConfig(**{**asdict(c), "population": population or c.population, "generations": generations or c.generations})
        pop = self.initialize_population(c.population)
        for a in pop:
            self.score(a)
        for _ in range(c.generations):
            pop.sort(key=lambda a: -a.score)
            elite = pop[: max(1, int(c.elite_fraction * c.population))]
            children = []
            while len(elite) + len(children) < c.population:
                child = self.mutate(self.rng.choice(elite))
                self.score(child)
                children.append(child)
            pop = elite + children
        return max(pop, key=lambda a: a.score)

    # ---- the reference's verbs (include/quant/hpo_nas.h: NASEngine) ------------------------------------------------
    def set_search_config(self, cfg: NASConfig): self.cfg = cfg
    def set_hardware_constraints(self, hw: HardwareConstraints): self.hw = hw

    def set_model(self, model):
        """Start the search around an existing model: its shape becomes the first member of every population."""
        c = model.cfg
        self.seed_arch = self.estimate(Architecture(id=-1, num_layers=c.num_layers, hidden_size=c.hidden_size, num_heads=c.num_heads,
                                                    ffn_size=c.ffn_hidden_size, vocab_size=c.vocab_size), self.cfg.tflops, self.cfg.tokens)

    def initialize_population(self, n: int) -> List[Architecture]:
        seed = [Architecture(**asdict(self.seed_arch))] if getattr(self, "seed_arch", None) is not None else []
        return seed + [self.random_architecture() for _ in range(n - len(seed))]

    def mutate_add_layer(self, a): return self.mutate(a, NASMutateOp.ADD_LAYER)
    def mutate_remove_layer(self, a): return self.mutate(a, NASMutateOp.REMOVE_LAYER)
    def mutate_change_width(self, a): return self.mutate(a, NASMutateOp.CHANGE_WIDTH)
    def mutate_change_heads(self, a): return self.mutate(a, NASMutateOp.CHANGE_HEADS)
    def mutate_change_ffn(self, a): return self.mutate(a, NASMutateOp.CHANGE_FFN)
    def mutate_change_dropout(self, a): return self.mutate(a, NASMutateOp.CHANGE_DROPOUT)

    def crossover(self, a: Architecture, b: Architecture) -> Architecture:
        """Each gene from one of the parents; the width is re-aligned to the chosen head count."""
        pick = lambda x, y: x if self.rng.random() < 0.5 else y
        heads = pick(a.num_heads, b.num_heads)
        hd = max(16, pick(a.hidden_size // a.num_heads, b.hidden_size // b.num_heads))
        c = Architecture(id=self._next, num_layers=pick(a.num_layers, b.num_layers), hidden_size=hd * heads, num_heads=heads,
                         ffn_size=pick(a.ffn_size, b.ffn_size), dropout=pick(a.dropout, b.dropout), vocab_size=pick(a.vocab_size, b.vocab_size))
        self._next += 1
        return self.estimate(c, self.cfg.tflops, self.cfg.tokens)

    def evaluate(self, a: Architecture) -> float:
        return self.score(a)

    def tournament_select(self, pop: Sequence[Architecture], k: int = 3) -> Architecture:
        return max(self.rng.sample(list(pop), min(k, len(pop))), key=lambda x: x.score)

    def hardware_aware_score(self, a: Architecture) -> float:
        """Quality proxy minus the hardware penalty, without calling the (expensive) evaluation function: larger models
        score higher with diminishing returns until a limit is crossed."""
        self.estimate(a, self.cfg.tflops, self.cfg.tokens)
        return math.log10(max(10.0, a.param_count)) - self.penalty(a)

    def estimate_latency_cycles(self, depth: int, width: int, num_heads: int, clock_ghz: float = 1.9) -> int:
        a = self.estimate(Architecture(id=-1, num_layers=depth, hidden_size=width, num_heads=num_heads, ffn_size=4 * width),
                          self.cfg.tflops, self.cfg.tokens)
        return int(a.latency_ms * 1e-3 * clock_ghz * 1e9)

    def estimate_memory(self, depth: int, width: int, ffn_size: int, vocab_size: int = 32000) -> int:
        return self.estimate(Architecture(id=-1, num_layers=depth, hidden_size=width, num_heads=max(1, width // 64), ffn_size=ffn_size,
                                          vocab_size=vocab_size)).memory_bytes

    def record_architecture(self, a: Architecture):
        self.history.append(a)

    def get_best_architecture(self) -> Optional[Architecture]:
        return max(self.history, key=lambda a: a.score) if self.history else None

    def get_pareto_front(self) -> List[Architecture]:
        """Architectures not dominated in (score up, parameters down, latency down)."""
        hist = list({a.id: a for a in self.history}.values())
        dom = lambda x, y: x.score >= y.score and x.param_count <= y.param_count and x.latency_ms <= y.latency_ms and \
            (x.score > y.score or x.param_count < y.param_count or x.latency_ms < y.latency_ms)
        return sorted((a for a in hist if not any(dom(b, a) for b in hist)), key=lambda a: -a.score)

    def save_architectures(self, path, top_k: int = 10) -> bool:
        try:
            best = sorted({a.id: a for a in self.history}.values(), key=lambda a: -a.score)[:top_k]
            with open(path, "w") as f:
                json.dump([asdict(a) for a in best], f, indent=1)
            return True
        except OSError:
            return False

    @staticmethod
    def load_architectures(path) -> List[Architecture]:
        with open(path) as f:
            return [Architecture(**d) for d in json.load(f)]

    # ---- differentiable-search flavour: a continuous relaxation over the same genes
    def darts_evaluate(self, a: Architecture) -> float:
        return self.score(a)

    def darts_migrate(self, a: Architecture, alpha: float = 0.1) -> Architecture:
        """One relaxed step: every gene moves by the fraction ``alpha`` towards the best architecture seen so far (then
        snaps back to valid sizes)."""
        best = self.get_best_architecture() or a
        mix = lambda x, y: x + alpha * (y - x)
        heads = max(1, int(round(mix(a.num_heads, best.num_heads))))
        hd = max(16, int(round(mix(a.hidden_size / a.num_heads, best.hidden_size / best.num_heads) / 16)) * 16)
        b = Architecture(id=self._next, num_layers=max(1, int(round(mix(a.num_layers, best.num_layers)))), hidden_size=hd * heads,
                         num_heads=heads, ffn_size=max(64, int(round(mix(a.ffn_size, best.ffn_size) / 64)) * 64),
                         dropout=mix(a.dropout, best.dropout), vocab_size=a.vocab_size)
        self._next += 1
        return self.estimate(b, self.cfg.tflops, self.cfg.tokens)

    def darts_search(self, n_iterations: int = 50, alpha: float = 0.3) -> Architecture:
        """Alternate a relaxed move towards the incumbent with a random mutation; keep whichever scores better."""
        cur = self.initialize_population(1)[0]
        self.darts_evaluate(cur)
        for _ in range(n_iterations):
            cand = self.mutate(self.darts_migrate(cur, alpha))
            if self.darts_evaluate(cand) > cur.score:
                cur = cand
        return self.get_best_architecture()

    def to_transformer_config(self, a: Architecture):
        from ..models.config import TransformerConfig
        return TransformerConfig(vocab_size=a.vocab_size, hidden_size=a.hidden_size, num_layers=a.num_layers, num_heads=a.num_heads,
                                 ffn_hidden_size=a.ffn_size)
