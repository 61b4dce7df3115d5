"""lockstep_b200: a single-GPU inference engine for sm_100a built after LockStep."""

__version__ = "0.1.0"

from .engine import Engine, ModelRunner, Request, Scheduler, StepEntry  # noqa: E402,F401
