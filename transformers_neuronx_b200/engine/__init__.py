from .step import HostBatch, StepEntry, StepRunner
from .loading import build_model, load_model, require_cuda
