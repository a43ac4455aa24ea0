from .params import EngineStepResult, FinishReason, GenerateOutput, RequestOutput, SamplingParams
from .sampler import Sampler, uniform_for

__all__ = ["EngineStepResult", "FinishReason", "GenerateOutput", "RequestOutput", "Sampler", "SamplingParams",
           "uniform_for"]
