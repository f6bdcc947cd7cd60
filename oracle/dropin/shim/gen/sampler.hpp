// TEST INFRASTRUCTURE — the header swap a maintainer of the reference would make: this file takes the place of the
// reference's src/gen/sampler.hpp on the include path, so that the reference's own, unmodified src/gen/session.cpp
// (which includes "gen/sampler.hpp" through gen/session.hpp and constructs mako::gen::Sampler at session.cpp:416)
// compiles against the B200 sampler instead. Nothing else of the reference changes; src/gen/sampler.cpp is left out
// of the link.
#pragma once

#include "mako_b200/sampler.hpp"

namespace mako::gen {
using SamplingParams = mako_b200::gen::SamplingParams; // same fields, same defaults (src/gen/sampler.hpp:12-20)
using Sampler = mako_b200::gen::Sampler;               // same constructor and methods (src/gen/sampler.hpp:22-45)
} // namespace mako::gen
