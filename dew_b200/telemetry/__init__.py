from .benchmark import DeviceTime, L2Flush, compared, device_time, max_over_ranks, measured_peaks

__all__ = ["DeviceTime", "L2Flush", "compared", "device_time", "max_over_ranks", "measured_peaks", "Profiler", "region"]


def __getattr__(name):
    if name in ("Profiler", "region", "CaptureOptions"):
        from . import profile
        return getattr(profile, name)
    raise AttributeError(name)
