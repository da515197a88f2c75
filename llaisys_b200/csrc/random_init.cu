// Counter-based normal random numbers for the random-weights mode: element i of a tensor with
// 64-bit key k is a function of (k, i) alone, so a tensor can be filled in any order, in pieces,
// on the device or on the host, and holds the same values.  (xsmccc/llaisys has no random
// initialisation; its models are always loaded from files.)
//
//   bits(c)  = splitmix64 finaliser of (k + (c + 1) * 0x9E3779B97F4A7C15)
//   u1       = ((bits(2i) >> 11) + 0.5) * 2^-53            in (0, 1)
//   q, f     = top two bits and remaining 51 bits of (bits(2i + 1) >> 11): the angle 2 pi u2 as a
//              quadrant and a fraction of a quarter turn
//   z        = sqrt(-2 ln u1) * cos(2 pi u2)               (Box-Muller)
//   value    = mean + std * z, rounded once to float32 and, for bfloat16 tensors, once more
//
// ln, cos and sin are evaluated here from additions, multiplications, divisions and square roots
// in double precision with explicit rounding (no contraction into fused multiply-adds): these
// operations give the same bits on every IEEE machine, which library logarithms and cosines do
// not.  The host twin (weights/rng.py) performs the same operations in the same order with numpy.
#include "common.cuh"

namespace {

__device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

#define ADD(a, b) __dadd_rn((a), (b))
#define MUL(a, b) __dmul_rn((a), (b))
#define DIV(a, b) __ddiv_rn((a), (b))

// ln(x) for x in (0, 1]: x = m * 2^e with m in [sqrt(1/2), sqrt(2)); s = (m - 1) / (m + 1);
// ln m = 2 (s + s^3/3 + ... + s^25/25), |s| < 0.1716; ln x = e * ln 2 + ln m.
__device__ double ln_exact_ops(double x) {
    int e;
    double m = frexp(x, &e);                      // exact: m in [0.5, 1)
    if (m < 0.70710678118654752440) {
        m = MUL(m, 2.0);
        e -= 1;
    }
    const double s = DIV(ADD(m, -1.0), ADD(m, 1.0));
    const double s2 = MUL(s, s);
    double acc = DIV(1.0, 25.0);
#pragma unroll
    for (int k = 23; k >= 1; k -= 2) acc = ADD(MUL(acc, s2), DIV(1.0, (double)k));
    const double ln_m = MUL(MUL(2.0, s), acc);
    return ADD(MUL((double)e, 0.69314718055994530942), ln_m);
}

// cos and sin of t in [0, pi/2] by their Taylor series up to t^26 / t^27.
__device__ void cos_sin_exact_ops(double t, double* c, double* s) {
    const double t2 = MUL(t, t);
    double ca = 0.0, sa = 0.0;
#pragma unroll
    for (int k = 13; k >= 1; --k) {
        ca = MUL(ADD(1.0, -ca), DIV(t2, (double)((2 * k - 1) * (2 * k))));
        sa = MUL(ADD(1.0, -sa), DIV(t2, (double)((2 * k) * (2 * k + 1))));
    }
    *c = ADD(1.0, -ca);
    *s = MUL(t, ADD(1.0, -sa));
}

__device__ double normal_at(uint64_t key, uint64_t i) {
    const uint64_t G = 0x9E3779B97F4A7C15ull;
    const uint64_t b1 = mix64(key + (2 * i + 1) * G) >> 11, b2 = mix64(key + (2 * i + 2) * G) >> 11;
    const double u1 = MUL(ADD((double)b1, 0.5), 1.1102230246251565e-16);          // 2^-53
    const int quadrant = (int)(b2 >> 51);
    const double frac = MUL((double)(b2 & ((1ull << 51) - 1)), 4.440892098500626e-16);   // 2^-51: [0, 1)
    double c, s;
    cos_sin_exact_ops(MUL(frac, 1.57079632679489661923), &c, &s);
    const double cosv = quadrant == 0 ? c : quadrant == 1 ? -s : quadrant == 2 ? -c : s;
    const double r = __dsqrt_rn(MUL(-2.0, ln_exact_ops(u1)));
    return MUL(r, cosv);
}

template <typename T>
__global__ void fill_normal_kernel(T* __restrict__ out, long long n, long long first, uint64_t key, double mean, double std) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const double v = ADD(mean, MUL(std, normal_at(key, (uint64_t)(first + i))));
    out[i] = from_f32<T>(__double2float_rn(v));
}

}  // namespace

// out[i] = value(key, first + i) for i < n, in float32 or bfloat16.
LLB_API int llb_fill_normal(void* out, int dtype, long long n, long long first, unsigned long long key,
                            double mean, double std, cudaStream_t stream) {
    if (n <= 0) return 0;
    const long long blocks = (n + 255) / 256;
    if (blocks > 0x7fffffffll) return (int)cudaErrorInvalidValue;
    LLB_DISPATCH_DTYPE(dtype, T, fill_normal_kernel<T><<<(unsigned)blocks, 256, 0, stream>>>((T*)out, n, first, key, mean, std));
    return llb_status();
}
