"""B200-native token sampling for the Stingray host: the host-side mirror of the reference's
``Sampler`` / ``SamplingParams`` API over the C-ABI CUDA library in ``csrc/``.

Importing this package never falls back to a CPU implementation: every operation goes through
``libstingray_sampler.so`` and raises if the library or a CUDA device is missing.
"""
from .sampler import (  # noqa: F401
    BatchSampler,
    Random,
    Sampler,
    SamplingParams,
    StingrayError,
)
