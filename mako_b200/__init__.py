"""mako_b200: the token-sampling path of jhanssen/mako as sm_100a CUDA kernels behind a C ABI.

Importing the package loads libmako_b200.so; it raises ImportError with the build command if the library has not
been built. Nothing here computes on the CPU.
"""
from ._lib import (FLAG_ALL_MASKED, FLAG_GUARD_BAND, FLAG_NEAR_CDF_BOUNDARY, FLAG_NO_CANDIDATE, FLAG_OVERFLOW,
                   FLAG_SECOND_PASS, FLAG_TIMEOUT, FLAG_VP_TRUNCATED, MakoError, lib)
from .sampler import BatchSampler, SampleResult, Sampler, SamplingParams, check_sampling, pack_bias, pack_params

__all__ = [
    "BatchSampler", "SampleResult", "Sampler", "SamplingParams", "check_sampling", "pack_bias", "pack_params",
    "MakoError", "lib", "FLAG_ALL_MASKED", "FLAG_GUARD_BAND", "FLAG_NEAR_CDF_BOUNDARY", "FLAG_NO_CANDIDATE",
    "FLAG_OVERFLOW", "FLAG_SECOND_PASS", "FLAG_TIMEOUT", "FLAG_VP_TRUNCATED",
]


def version() -> str:
    return lib.mk_version().decode()
