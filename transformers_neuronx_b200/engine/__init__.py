from .step import HostBatch, StepEntry, StepRunner
from .loading import build_model, load_model, require_cuda
from .scheduler import Request, SamplingParams, Scheduled, Scheduler, StepPlan
from .llm_engine import LLMEngine
