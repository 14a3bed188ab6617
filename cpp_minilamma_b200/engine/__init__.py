from .generate import Backend, Completion, GenerationError, generate, plan_batches
from .model import Model
from .step import Engine, StepEntry, StepError, Workspace
