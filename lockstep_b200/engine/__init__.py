"""The step function and what drives it."""

from .batch import StepContext, StepEntry
from .engine import Engine
from .model import Model, expected_weights
from .policy import DefaultPolicy, FixedChunkPolicy, Policy, SchedulerState, ScriptedPolicy
from .runner import ModelRunner
from .scheduler import OversizedRequest, Request, Scheduler

__all__ = ["DefaultPolicy", "Engine", "FixedChunkPolicy", "Model", "ModelRunner", "OversizedRequest",
           "Policy", "Request", "Scheduler", "SchedulerState", "ScriptedPolicy", "StepContext",
           "StepEntry", "expected_weights"]
