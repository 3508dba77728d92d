from .core import (NullProfiler, Profiler, bucket, get_active_profiler, register_active_profiler,
                   release_active_profiler)

__all__ = ["NullProfiler", "Profiler", "bucket", "get_active_profiler", "register_active_profiler",
           "release_active_profiler"]
