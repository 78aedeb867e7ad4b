from .engine import Engine, EngineConfig, Sequence  # noqa: F401
from .params import FinishReason, SamplingParams, SeqStatus  # noqa: F401
