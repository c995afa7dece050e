from .runner import ModelRunner, SequenceStep

__all__ = ["ModelRunner", "SequenceStep"]
