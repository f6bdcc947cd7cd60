// Float exponential that returns, bit for bit, what the host C library returns for the same float.
//
// The reference sampler turns logits into weights with std::exp(float) (src/gen/sampler.cpp:33); which tokens
// survive min_p / top_k / top_p and which token a uniform selects depend on the exact float. On the build's hosts
// that function is glibc 2.39 expf (sysdeps/ieee754/flt-32/e_expf.c, from ARM's optimized routines): in double,
//     z = x * 32/ln2;  k = round(z);  r = z - k;  exp(x) = 2^(k/32) * (C0 r^3 + C1 r^2 + C2 r + 1)
// with 2^(k/32) from a 32-entry table and the scale folded into the exponent bits. The x86-64 build of that
// routine that runs on FMA-capable hosts contracts r = fma(32/ln2, x, -k) and the three polynomial steps; the
// same operations are issued here with explicit IEEE intrinsics. Checked exhaustively on the host against expf
// for every float in [-103.98, -0.0] (0 mismatches in 1,120,924,085 values); the sampler only ever evaluates
// non-positive arguments, NaN and -inf.
#pragma once
#include <cstdint>

namespace mk {

__device__ __constant__ unsigned long long kExp2Tab[32] = {
#include "exp2_table.inc"
};

__device__ __forceinline__ float expf_host_exact(float x)
{
    if (!(x >= -0x1.9fe368p6f)) {       // below log(2^-150), -inf, or NaN
        return (x != x) ? x : 0.0f;
    }
    if (x > 0x1.62e42ep6f)              // above log(2^128): overflow (not reached by the sampler)
        return __int_as_float(0x7f800000);
    const double inv_ln2_n = 0x1.71547652b82fep+0 * 32.0;
    const double shift = 0x1.8p+52;
    const double c0 = 0x1.c6af84b912394p-5 / 32.0 / 32.0 / 32.0;
    const double c1 = 0x1.ebfce50fac4f3p-3 / 32.0 / 32.0;
    const double c2 = 0x1.62e42ff0c52d6p-1 / 32.0;
    const double xd = (double)x;
    const double z = __dmul_rn(inv_ln2_n, xd);
    double kd = __dadd_rn(z, shift);
    const unsigned long long ki = (unsigned long long)__double_as_longlong(kd);
    kd = __dsub_rn(kd, shift);
    const double r = __fma_rn(inv_ln2_n, xd, -kd);
    const unsigned long long t = kExp2Tab[ki & 31ull] + (ki << 47);
    const double s = __longlong_as_double((long long)t);
    const double zz = __fma_rn(c0, r, c1);
    const double r2 = __dmul_rn(r, r);
    double y = __fma_rn(c2, r, 1.0);
    y = __fma_rn(zz, r2, y);
    y = __dmul_rn(y, s);
    return __double2float_rn(y);
}

} // namespace mk
