"""Sampling: the options a request carries, the device sampler, the host reference."""
from .params import SamplingParams
from .device import DeviceSampler
from .host import HostSampler, Rng, draw_greedy, draw_temperature

__all__ = ["SamplingParams", "DeviceSampler", "HostSampler", "Rng", "draw_greedy", "draw_temperature"]
