"""Model assembly, the step function, the generation loop and the entry point."""

from .engine import Engine, parse_dtype
from .generate import GenerationLoop, Sequence, split_into_batches
from .model import Model, PartTree, Runtime, expected_tensors
from .step import BatchMeta, StepContext, StepEntry, Stepper

__all__ = [n for n in dir() if not n.startswith("_")]
