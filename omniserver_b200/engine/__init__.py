from .llm_engine import LLMEngine, StepDelta, build_runner
from .request import Request, SamplingParams, Sequence, Status
from .scheduler import ScheduledEntry, Scheduler, SchedulerConfig, SchedulerOutput
from .step import ModelRunner, StepContext, StepEntry
