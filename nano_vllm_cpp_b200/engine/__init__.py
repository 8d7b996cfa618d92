from .batch import StepEntry, StepBatch, EntryInfo, build_batch

__all__ = ["StepEntry", "StepBatch", "EntryInfo", "build_batch"]
