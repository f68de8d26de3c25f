"""The model, the step function and the generation loop."""
from .batch import StepBatch, Workspace
from .engine import Engine, StepEntry, Stats, StepError, load_model, resolve_dtype
from .model import Model, plan_manifest
from .generate import GenerateOptions, GenerateResult, generate, plan_batches
