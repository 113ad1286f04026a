"""Continual learning: multi-timescale weights, EWC, experience replay (crates/ronn-learning/src/lib.rs:56-179)."""
from .engine import (ContinualLearningEngine, ElasticWeightConsolidation, Experience, ExperienceReplay,
                     LearningConfig, LearningResult, MultiTimescaleLearner, ReplayStrategy, TimescaleConfig)
