from .timing import ClockSampler, L2Flusher, time_cuda

__all__ = ["ClockSampler", "L2Flusher", "time_cuda"]
