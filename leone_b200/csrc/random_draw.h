// Seeded random weights as a pure function of (key, element index).
//
// The same function is compiled for the host (host_runtime.cpp, which fills CPU tensors) and
// for the device (random_weights.cu, which fills GPU tensors); both give the same bits, so a
// model drawn on the GPU from (configuration, seed) is the model a file written on the CPU
// from the same pair holds.  That needs arithmetic that rounds the same way everywhere:
// integer mixing, and fp64 +, -, *, /, sqrt, each rounded once to nearest (no fused
// multiply-add: the device side uses the _rn intrinsics, the host side is compiled with
// -ffp-contract=off).  No library log, sin or cos is used: those are not correctly rounded
// and differ between libm and CUDA.
//
// The definition (the tests' own restatement in numpy follows it operation by operation):
//   mix(z):  z ^= z >> 30; z *= 0xbf58476d1ce4e5b9; z ^= z >> 27; z *= 0x94d049bb133111eb;
//            z ^= z >> 31                                   (the splitmix64 finaliser)
//   bits(key, n) = mix(key + (n + 1) * 0x9e3779b97f4a7c15)  (n-th output of splitmix64(key))
//   element i of a tensor uses a = bits(key, 2 i) >> 12 and b = bits(key, 2 i + 1) >> 12
//   u  = (a + 0.5) * 2^-52                       in (0, 1), exact
//   ln u: u = m * 2^e with m in [1, 2); if m > 1.4142135623730951 then m /= 2, e += 1;
//        s = (m - 1) / (m + 1); w = s * s; p = Horner in w of 1/(2k+1), k = 11 .. 0;
//        ln u = e * 0.6931471805599453 + 2 * (s * p)
//   r  = sqrt(-2 * ln u)
//   angle: octant o = b >> 49, rest = b & (2^49 - 1); odd octants mirror: rest' = 2^49 - 1 - rest;
//        x = (rest' + 0.5) * ((pi / 4) * 2^-49)  in (0, pi / 4); w = x * x
//        cos x = Horner in w of (-1)^k / (2k)!, k = 9 .. 0; sin x = x * Horner of (-1)^k / (2k+1)!
//        cos(angle) = +-cos x or +-sin x by octant (0: c, 1: s, 2: -s, 3: -c, 4: -c, 5: -s, 6: s, 7: c)
//   z  = r * cos(angle)                          standard normal (Box-Muller, cosine branch)
//   value = float(mean + std * z)                rounded once from fp64 to fp32
//   bfloat16 storage holds round-to-nearest-even of that fp32 value.
//   Integer tables: bits(key, i) >> 49 (15 bits).
//
// The reference has no random-weight mode (crates/leone/tests/common/cpu_fixture.rs:67-106
// builds a zero-weight fixture); this generator is this engine's own.
#pragma once
#include <math.h>
#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define LEONE_RD_FN __host__ __device__ __forceinline__
#else
#define LEONE_RD_FN static inline
#endif

namespace leone_rd {

#if defined(__CUDA_ARCH__)
#define LEONE_RD_OP(dev, host) return dev
#else
#define LEONE_RD_OP(dev, host) return host
#endif
LEONE_RD_FN double add(double a, double b) { LEONE_RD_OP(__dadd_rn(a, b), a + b); }
LEONE_RD_FN double sub(double a, double b) { LEONE_RD_OP(__dsub_rn(a, b), a - b); }
LEONE_RD_FN double mul(double a, double b) { LEONE_RD_OP(__dmul_rn(a, b), a * b); }
LEONE_RD_FN double div(double a, double b) { LEONE_RD_OP(__ddiv_rn(a, b), a / b); }
LEONE_RD_FN double root(double a) { LEONE_RD_OP(__dsqrt_rn(a), sqrt(a)); }
LEONE_RD_FN uint64_t as_bits(double a) { uint64_t b; memcpy(&b, &a, 8); return b; }
LEONE_RD_FN double from_bits(uint64_t b) { double a; memcpy(&a, &b, 8); return a; }

LEONE_RD_FN uint64_t mix(uint64_t z) {
    z ^= z >> 30; z *= 0xbf58476d1ce4e5b9ULL;
    z ^= z >> 27; z *= 0x94d049bb133111ebULL;
    return z ^ (z >> 31);
}

LEONE_RD_FN uint64_t bits(uint64_t key, uint64_t n) {
    return mix(key + (n + 1) * 0x9e3779b97f4a7c15ULL);
}

// ln of a positive normal double
LEONE_RD_FN double ln(double u) {
    uint64_t b = as_bits(u);
    long long e = (long long)((b >> 52) & 0x7ff) - 1023;
    double m = from_bits((b & 0x000fffffffffffffULL) | 0x3ff0000000000000ULL);
    if (m > 1.4142135623730951) { m = mul(m, 0.5); e += 1; }
    double s = div(sub(m, 1.0), add(m, 1.0));
    double w = mul(s, s);
    double p = 1.0 / 23.0;
    p = add(mul(p, w), 1.0 / 21.0);
    p = add(mul(p, w), 1.0 / 19.0);
    p = add(mul(p, w), 1.0 / 17.0);
    p = add(mul(p, w), 1.0 / 15.0);
    p = add(mul(p, w), 1.0 / 13.0);
    p = add(mul(p, w), 1.0 / 11.0);
    p = add(mul(p, w), 1.0 / 9.0);
    p = add(mul(p, w), 1.0 / 7.0);
    p = add(mul(p, w), 1.0 / 5.0);
    p = add(mul(p, w), 1.0 / 3.0);
    p = add(mul(p, w), 1.0);
    return add(mul((double)e, 0.6931471805599453), mul(2.0, mul(s, p)));
}

// cos of the angle 2 pi (b + 0.5) / 2^52 for a 52-bit b
LEONE_RD_FN double cos_turn(uint64_t b) {
    unsigned o = (unsigned)(b >> 49);
    uint64_t rest = b & ((1ULL << 49) - 1);
    if (o & 1) rest = ((1ULL << 49) - 1) - rest;
    // (pi / 4) * 2^-49
    double x = mul(add((double)rest, 0.5), 0.7853981633974483 * (1.0 / 562949953421312.0));
    double w = mul(x, x);
    double v;
    if (o == 1 || o == 2 || o == 5 || o == 6) {
        double p = -1.0 / 121645100408832000.0;            // 19!
        p = add(mul(p, w), 1.0 / 355687428096000.0);       // 17!
        p = add(mul(p, w), -1.0 / 1307674368000.0);        // 15!
        p = add(mul(p, w), 1.0 / 6227020800.0);            // 13!
        p = add(mul(p, w), -1.0 / 39916800.0);             // 11!
        p = add(mul(p, w), 1.0 / 362880.0);                // 9!
        p = add(mul(p, w), -1.0 / 5040.0);                 // 7!
        p = add(mul(p, w), 1.0 / 120.0);                   // 5!
        p = add(mul(p, w), -1.0 / 6.0);                    // 3!
        p = add(mul(p, w), 1.0);
        v = mul(x, p);
    } else {
        double p = -1.0 / 6402373705728000.0;              // 18!
        p = add(mul(p, w), 1.0 / 20922789888000.0);        // 16!
        p = add(mul(p, w), -1.0 / 87178291200.0);          // 14!
        p = add(mul(p, w), 1.0 / 479001600.0);             // 12!
        p = add(mul(p, w), -1.0 / 3628800.0);              // 10!
        p = add(mul(p, w), 1.0 / 40320.0);                 // 8!
        p = add(mul(p, w), -1.0 / 720.0);                  // 6!
        p = add(mul(p, w), 1.0 / 24.0);                    // 4!
        p = add(mul(p, w), -1.0 / 2.0);                    // 2!
        v = add(mul(p, w), 1.0);
    }
    return (o >= 2 && o <= 5) ? -v : v;
}

// element `index` of the tensor keyed `key`: a standard normal draw in fp64
LEONE_RD_FN double normal(uint64_t key, uint64_t index) {
    uint64_t a = bits(key, 2 * index) >> 12;
    uint64_t b = bits(key, 2 * index + 1) >> 12;
    double u = mul(add((double)a, 0.5), 1.0 / 4503599627370496.0);     // 2^-52
    double r = root(mul(-2.0, ln(u)));
    return mul(r, cos_turn(b));
}

LEONE_RD_FN float weight(uint64_t key, uint64_t index, double mean, double std) {
    return (float)add(mean, mul(std, normal(key, index)));
}

LEONE_RD_FN int32_t table_entry(uint64_t key, uint64_t index) {
    return (int32_t)(bits(key, index) >> 49);
}

}  // namespace leone_rd
