from .engine import Engine, EngineStats, GenerationEvent, RequestHandle
from .scheduler import BatchConfig, FinishReason, Phase, Scheduler, StepPlan
from .step import ModelRunner, StepContext, StepEntry
