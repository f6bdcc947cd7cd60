"""mako_b200: the token-sampling path of jhanssen/mako as sm_100a CUDA kernels behind a C ABI.

The first use of any name below loads libmako_b200.so; that raises ImportError with the build command if the library
has not been built (`python -m mako_b200.build`, which itself needs no built library). Nothing here computes on the
CPU.
"""
_SAMPLER = {"BatchSampler", "SampleResult", "Sampler", "SamplingParams", "check_sampling", "pack_bias", "pack_params"}
_LIB = {"MakoError", "lib", "FLAG_ALL_MASKED", "FLAG_GUARD_BAND", "FLAG_NEAR_CDF_BOUNDARY", "FLAG_NO_CANDIDATE",
        "FLAG_OVERFLOW", "FLAG_TIMEOUT", "FLAG_HISTORY_FULL", "FLAG_VP_TRUNCATED"}
__all__ = sorted(_SAMPLER | _LIB | {"version", "synth"})


def __getattr__(name):
    import importlib
    if name in _SAMPLER:
        return getattr(importlib.import_module(".sampler", __name__), name)
    if name in _LIB:
        return getattr(importlib.import_module("._lib", __name__), name)
    if name in ("synth", "sampler", "build", "_lib"):
        return importlib.import_module("." + name, __name__)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def version() -> str:
    from ._lib import lib
    return lib.mk_version().decode()
