from .request import InferenceRequest, RequestState, SamplingParams
from .scheduler import ContinuousBatchScheduler, ScheduledBatch, ScheduledItem, SchedulerStats

__all__ = ["InferenceRequest", "RequestState", "SamplingParams", "ContinuousBatchScheduler", "ScheduledBatch",
           "ScheduledItem", "SchedulerStats"]
