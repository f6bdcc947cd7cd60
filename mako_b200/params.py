"""The sampling parameters as a plain value, with the names and defaults of mako::gen::SamplingParams
(src/gen/sampler.hpp:12-20). Importing this module loads no native library."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class SamplingParams:
    """Applied in this order: penalties, temperature, min_p, top_k, top_p (src/gen/sampler.hpp:11-20)."""

    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0

    def to_c(self):
        """The same seven fields as the C ABI's mk_sampling_params (this loads the library)."""
        from ._lib import SamplingParamsC
        return SamplingParamsC(self.temperature, self.top_k, self.top_p, self.min_p, self.presence_penalty,
                               self.frequency_penalty, self.repetition_penalty)
