// Counter-based matrix generator shared by host and device code: element (i,j)
// of matrix `mat` under `seed` is a pure function of (seed, mat, i, j), so any
// sub-block of any operand can be regenerated anywhere, bit for bit.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define ULMB_GEN_HD __host__ __device__ __forceinline__
#else
#define ULMB_GEN_HD inline
#endif

namespace ulmb200 {

ULMB_GEN_HD uint64_t mix64(uint64_t z)
{
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// uniform in [0,1) with 53 random bits
ULMB_GEN_HD double gen_u01(uint64_t seed, uint32_t mat, int64_t i, int64_t j)
{
    const uint64_t key = mix64(seed ^ ((uint64_t)mat * 0xD1B54A32D192ED03ull));
    const uint64_t h = mix64(key ^ (((uint64_t)j << 32) | (uint64_t)(i & 0xFFFFFFFFll)));
    return (double)(h >> 11) * (1.0 / 9007199254740992.0);
}

// dist 0: uniform[-1,1).  dist 1: diagonal uniform[1,2), off-diagonal uniform[-1,1)*scale.
ULMB_GEN_HD double gen_value(uint64_t seed, uint32_t mat, int64_t i, int64_t j, int dist, double scale)
{
    const double u = gen_u01(seed, mat, i, j);
    if (dist == 1) return (i == j) ? 1.0 + u : (2.0 * u - 1.0) * scale;
    return 2.0 * u - 1.0;
}

}  // namespace ulmb200
