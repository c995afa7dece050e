from .handle import (EngineHandle, Error, Finished, GenerateRequest, GenerationResult, GenerationStream, Token,
                     TokenIds)
from .runner import ModelRunner, SequenceStep
from .scheduler import Scheduler

__all__ = ["EngineHandle", "Error", "Finished", "GenerateRequest", "GenerationResult", "GenerationStream", "Token",
           "TokenIds", "ModelRunner", "SequenceStep", "Scheduler"]
