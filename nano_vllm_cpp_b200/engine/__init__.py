from .batch import StepEntry, StepBatch, EntryInfo

__all__ = ["StepEntry", "StepBatch", "EntryInfo"]
