from .params import RandomStream, SamplingParams

__all__ = ["RandomStream", "SamplingParams", "DeviceSampler"]


def __getattr__(name):
    if name == "DeviceSampler":
        from .device import DeviceSampler
        return DeviceSampler
    raise AttributeError(name)
