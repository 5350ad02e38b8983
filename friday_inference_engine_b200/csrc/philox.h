// Philox-4x32-10 and the normal numbers of the random-weights mode, for host and device alike.
//
// A tensor's numbers are a function of (key, element index) only, so any tensor, or any part of one, can be
// made alone, in any order, on the host or on the device, and comes out the same (up to the last bit of the
// library's log/sin/cos in double precision, which the rounding to 32 bits hides in all but a vanishing
// share of elements).  Element 2j and 2j+1 are the two results of one Box-Muller transform of the two 24-bit
// uniforms that counter j gives under the key.
#pragma once
#include <math.h>
#include <stdint.h>

#ifdef __CUDACC__
#define FR_HD __host__ __device__ __forceinline__
#else
#define FR_HD inline
#endif

FR_HD void fr_philox4x32_10(uint32_t c[4], uint32_t k0, uint32_t k1) {
    for (int r = 0; r < 10; ++r) {
        const uint64_t p0 = (uint64_t)0xD2511F53u * c[0], p1 = (uint64_t)0xCD9E8D57u * c[2];
        const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k0, n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k1;
        c[1] = (uint32_t)p1;
        c[3] = (uint32_t)p0;
        c[0] = n0;
        c[2] = n2;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
}

// Standard normal number for element `index` under `key`.
FR_HD double fr_normal_at(uint64_t key, uint64_t index) {
    const uint64_t pair = index >> 1;
    uint32_t c[4] = {(uint32_t)pair, (uint32_t)(pair >> 32), 0u, 0u};
    fr_philox4x32_10(c, (uint32_t)key, (uint32_t)(key >> 32));
    const double u1 = ((double)(c[0] >> 8) + 0.5) * (1.0 / 16777216.0);
    const double u2 = (double)(c[1] >> 8) * (1.0 / 16777216.0);
    const double r = sqrt(-2.0 * log(u1));
    const double a = 6.283185307179586476925286766559 * u2;
    return (index & 1) ? r * sin(a) : r * cos(a);
}
