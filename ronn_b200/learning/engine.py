"""Continual-learning engine.

Structure of the reference: ``MultiTimescaleLearner`` with fast lr 0.01 / slow lr 1e-4 and
consolidation rate 0.1 over 100 weights (crates/ronn-learning/src/timescales.rs:8-135),
``ElasticWeightConsolidation`` with lambda 0.4 scaling updates by max(1 - lambda*importance, 0)
(ewc.rs:22-81), ``ExperienceReplay`` ring buffer with Random / Importance / Recent strategies
(replay.rs:9-90), and the engine loop store -> compute -> constrain -> apply -> replay every 10
updates (lib.rs:77-113).  The reference's gradients are synthetic (sin(i*0.01)*lr); here the update
is a real gradient of 0.5*||W x - target||^2 restricted to the learner's weight vector.
"""
from __future__ import annotations

import enum
import random
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, List, Optional

import torch


@dataclass
class TimescaleConfig:
    fast_lr: float = 0.01
    slow_lr: float = 1e-4
    consolidation_rate: float = 0.1
    num_weights: int = 100


class MultiTimescaleLearner:
    def __init__(self, config: TimescaleConfig = None):
        self.config = config or TimescaleConfig()
        n = self.config.num_weights
        self.fast = torch.zeros(n)
        self.slow = torch.zeros(n)
        self.updates = 0

    def effective_weights(self) -> torch.Tensor:
        return self.slow + self.fast

    def compute_update(self, x: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        """Gradient step direction for the elementwise linear model y = w * x on the first n features."""
        n = self.config.num_weights
        xf = torch.zeros(n)
        tf = torch.zeros(n)
        xv, tv = x.detach().float().reshape(-1)[:n], target.detach().float().reshape(-1)[:n]
        xf[: xv.numel()] = xv
        tf[: tv.numel()] = tv
        err = self.effective_weights() * xf - tf
        return -(err * xf)

    def apply_update(self, delta: torch.Tensor) -> None:
        self.fast += self.config.fast_lr * delta
        self.slow += self.config.slow_lr * delta
        self.updates += 1

    def consolidate(self) -> None:
        r = self.config.consolidation_rate
        self.slow += r * self.fast
        self.fast *= (1.0 - r)


class ElasticWeightConsolidation:
    def __init__(self, num_weights: int = 100, lam: float = 0.4):
        self.lam = lam
        self.importance = torch.zeros(num_weights)
        self.tasks = 0

    def consolidate_task(self, task_size: int, grads: Optional[torch.Tensor] = None) -> None:
        """Accumulate importance: squared gradients when given (Fisher diagonal), else the reference's
        heuristic min(0.1*|task|, 1)."""
        if grads is not None:
            g2 = grads.detach().float().reshape(-1)[: self.importance.numel()] ** 2
            self.importance[: g2.numel()] += g2 / (g2.max() + 1e-12)
        else:
            self.importance += min(0.1 * task_size, 1.0)
        self.importance.clamp_(max=1.0 / max(self.lam, 1e-12))
        self.tasks += 1

    def constrain_update(self, delta: torch.Tensor) -> torch.Tensor:
        return delta * torch.clamp(1.0 - self.lam * self.importance, min=0.0)


class ReplayStrategy(enum.Enum):
    RANDOM = "random"
    IMPORTANCE = "importance"
    RECENT = "recent"


@dataclass
class Experience:
    input: torch.Tensor
    target: torch.Tensor
    importance: float
    step: int = 0


class ExperienceReplay:
    def __init__(self, capacity: int = 1000, strategy: ReplayStrategy = ReplayStrategy.IMPORTANCE, seed: int = 0):
        self.capacity = capacity
        self.strategy = strategy
        self.buffer: Deque[Experience] = deque(maxlen=capacity)
        self._rng = random.Random(seed)
        self._step = 0

    def __len__(self):
        return len(self.buffer)

    def store(self, exp: Experience) -> None:
        exp.step = self._step
        self._step += 1
        self.buffer.append(exp)

    def sample(self, n: int) -> List[Experience]:
        items = list(self.buffer)
        if self.strategy == ReplayStrategy.IMPORTANCE:
            return sorted(items, key=lambda e: -e.importance)[:n]
        if self.strategy == ReplayStrategy.RECENT:
            return list(reversed(items))[:n]
        return self._rng.sample(items, min(n, len(items)))


@dataclass
class LearningConfig:
    timescales: TimescaleConfig = field(default_factory=TimescaleConfig)
    ewc_lambda: float = 0.4
    replay_capacity: int = 1000
    replay_interval: int = 10
    replay_batch: int = 32
    replay_scale: float = 0.5


@dataclass
class LearningResult:
    loss: float
    update_norm: float
    replayed: int


class ContinualLearningEngine:
    def __init__(self, config: LearningConfig = None):
        self.config = config or LearningConfig()
        self.learner = MultiTimescaleLearner(self.config.timescales)
        self.ewc = ElasticWeightConsolidation(self.config.timescales.num_weights, self.config.ewc_lambda)
        self.replay = ExperienceReplay(self.config.replay_capacity)
        self.updates = 0
        self._last_grad = None

    def learn(self, x: torch.Tensor, target: torch.Tensor, importance: float = 0.5) -> LearningResult:
        self.replay.store(Experience(x, target, importance))
        delta = self.learner.compute_update(x, target)
        self._last_grad = delta
        delta = self.ewc.constrain_update(delta)
        self.learner.apply_update(delta)
        self.updates += 1
        replayed = 0
        if self.updates % self.config.replay_interval == 0:
            for e in self.replay.sample(self.config.replay_batch):
                d = self.ewc.constrain_update(self.learner.compute_update(e.input, e.target))
                self.learner.apply_update(self.config.replay_scale * d)
                replayed += 1
        n = self.config.timescales.num_weights
        xv = torch.zeros(n)
        tv = torch.zeros(n)
        a, b = x.detach().float().reshape(-1)[:n], target.detach().float().reshape(-1)[:n]
        xv[: a.numel()], tv[: b.numel()] = a, b
        loss = 0.5 * float(((self.learner.effective_weights() * xv - tv) ** 2).sum())
        return LearningResult(loss, float(delta.norm()), replayed)

    def consolidate_task(self) -> None:
        self.ewc.consolidate_task(len(self.replay), self._last_grad)
        self.learner.consolidate()
