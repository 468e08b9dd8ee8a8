// Random weights on the device: out[i] = std * z(key, i), z a standard normal deviate that
// depends on nothing but a 64-bit key (made on the host from the seed and the tensor's name)
// and the element's index.  The reference's fixture is likewise a pure function of its seed
// (crates/bc-infer/src/fixtures.rs:7-60).
//
// Every step is either integer arithmetic or a single float operation that IEEE 754 rounds
// correctly (add, multiply, divide, square root; written with the _rn intrinsics so that the
// compiler cannot fuse a multiply with an add), so the NumPy mirror in
// weights/random_init.py, which does the same steps in the same order, produces the same
// bits.  The logarithm, sine and cosine of Box and Muller's transform are therefore
// polynomials written out here, not library calls.
#include "common.cuh"

__device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}

// Constants are double literals rounded once to float, as NumPy rounds the same literals.
#define F(x) ((float)(x))

__device__ __forceinline__ float mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float add(float a, float b) { return __fadd_rn(a, b); }

__device__ __forceinline__ float normal_deviate(uint64_t key, uint64_t index) {
    const uint64_t h = mix64(key + (index + 1ull) * 0x9e3779b97f4a7c15ull);
    const uint32_t a = (uint32_t)(h >> 40), b = (uint32_t)(h >> 16) & 0xffffffu;   // two draws of 24 bits
    // radius: sqrt(-2 ln u), u = (a + 1) / 2^24 in (0, 1]
    const float u = mul((float)(a + 1u), F(5.9604644775390625e-08));
    int e;
    float m = frexpf(u, &e);                       // u = m 2^e, m in [0.5, 1)
    if (m < F(0.70710678118654752)) {
        m = mul(m, F(2.0));
        e -= 1;
    }
    const float s = __fdiv_rn(add(m, F(-1.0)), add(m, F(1.0)));    // ln m = 2 atanh(s), |s| < 0.1716
    const float s2 = mul(s, s);
    float p = F(0.090909090909090909);
    p = add(F(0.11111111111111111), mul(s2, p));
    p = add(F(0.14285714285714285), mul(s2, p));
    p = add(F(0.2), mul(s2, p));
    p = add(F(0.33333333333333333), mul(s2, p));
    const float ln_m = mul(F(2.0), add(s, mul(s, mul(s2, p))));
    const float ln_u = add(mul((float)e, F(0.69314718055994531)), ln_m);
    const float radius = __fsqrt_rn(mul(F(-2.0), ln_u));
    // angle: 2 pi b / 2^24 = quadrant (top two bits) * pi/2 + x, x in [0, pi/2)
    const uint32_t quadrant = b >> 22;
    const float x = mul(mul((float)(b & 0x3fffffu), F(2.384185791015625e-07)), F(1.5707963267948966));
    const float x2 = mul(x, x);
    float sn = F(1.6059043836821613e-10);            // 1/13!
    sn = add(F(-2.5052108385441719e-08), mul(x2, sn));
    sn = add(F(2.7557319223985891e-06), mul(x2, sn));
    sn = add(F(-1.9841269841269841e-04), mul(x2, sn));
    sn = add(F(8.3333333333333333e-03), mul(x2, sn));
    sn = add(F(-1.6666666666666667e-01), mul(x2, sn));
    sn = add(x, mul(x, mul(x2, sn)));
    float cs = F(-1.1470745597729725e-11);           // -1/14!
    cs = add(F(2.0876756987868099e-09), mul(x2, cs));
    cs = add(F(-2.7557319223985888e-07), mul(x2, cs));
    cs = add(F(2.4801587301587302e-05), mul(x2, cs));
    cs = add(F(-1.3888888888888889e-03), mul(x2, cs));
    cs = add(F(4.1666666666666664e-02), mul(x2, cs));
    cs = add(F(-0.5), mul(x2, cs));
    cs = add(F(1.0), mul(x2, cs));
    const float c = quadrant == 0 ? cs : quadrant == 1 ? -sn : quadrant == 2 ? -cs : sn;   // cos(quadrant pi/2 + x)
    return mul(radius, c);
}

template <class T>
__global__ void random_normal_kernel(T* __restrict__ out, size_t n, uint64_t key, float std) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        out[i] = from_f32<T>(mul(normal_deviate(key, (uint64_t)i), std));
}

#define RANDOM_LAUNCHER(SUFFIX, T)                                                                                            \
    extern "C" int bc_random_normal_##SUFFIX(void* out, long long n, unsigned long long key, float std, cudaStream_t s) {   \
        BC_CHECK_ARG(n >= 0 && std >= 0.0f, "random_normal: bad sizes n=%lld std=%g", n, (double)std);                       \
        if (n == 0) return BC_OK;                                                                                             \
        const long long blocks = (n + 255) / 256, most = (long long)bc_sm_count() * 16;                                       \
        random_normal_kernel<T><<<(unsigned)(blocks < most ? blocks : most), 256, 0, s>>>((T*)out, (size_t)n, key, std);      \
        BC_LAUNCH_STATUS();                                                                                                   \
    }

RANDOM_LAUNCHER(f32, float)
RANDOM_LAUNCHER(bf16, bf16)
