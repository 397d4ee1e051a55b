// Seeded normal values written straight into their place in a weight buffer.
//
// Element i of the tensor with key `key` is a function of (key, i) alone:
//
//   h  = mix64(key + (i + 1) * 0x9E3779B97F4A7C15)          (the splitmix64 sequence)
//   u1 = ((h >> 40) + 1) * 2^-24                             in (0, 1]
//   a  = (h >> 8) & 0xFFFFFF                                 the angle 2 pi a / 2^24
//   z  = sqrt(-2 ln u1) * cos(2 pi a / 2^24)                 (Box-Muller)
//   w  = std * z, rounded to nearest even to bfloat16 when the tensor is stored so
//   value = w + offset (a norm's 1 + weight), rounded to the buffer's type
//
// ln and cos are evaluated with the fixed sequences of single 32-bit operations
// below (each multiply, add, divide and square root rounded on its own, nothing
// contracted into a fused multiply-add), so that a host restatement that does the
// same operations in the same order gives the same bits.  weights/random_init.py
// holds that restatement; it is how a model folder is written without a device.
// The reference has no random-weights mode (its tests hand-build identity, zero
// and ramp tensors, src/engine/generate.rs:1477-1584).
//
// The destination may interleave the rows of the stored tensor with another
// tensor's rows: stored row r goes to destination row
// (r / group) * group_stride + r % group (group 0: rows stay together).
#include "common.cuh"

namespace {

__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z ^= z >> 30;
    z *= 0xBF58476D1CE4E5B9ull;
    z ^= z >> 27;
    z *= 0x94D049BB133111EBull;
    z ^= z >> 31;
    return z;
}

// ln(u) for u = n * 2^-24, n in [1, 2^24]: u = m * 2^e with m in (1/sqrt2, sqrt2],
// ln m = 2 s (1 + s^2/3 + s^4/5 + s^6/7 + s^8/9) with s = (m - 1) / (m + 1).
__device__ __forceinline__ float ln_unit(float u) {
    int bits = __float_as_int(u);
    int e = (bits >> 23) - 127;
    float m = __int_as_float((bits & 0x007FFFFF) | 0x3F800000);    // [1, 2)
    if (m > 1.41421354f) {
        m = __fmul_rn(m, 0.5f);
        e += 1;
    }
    const float s = __fdiv_rn(__fadd_rn(m, -1.0f), __fadd_rn(m, 1.0f));
    const float s2 = __fmul_rn(s, s);
    float p = 0.111111111f;
    p = __fadd_rn(__fmul_rn(p, s2), 0.142857143f);
    p = __fadd_rn(__fmul_rn(p, s2), 0.2f);
    p = __fadd_rn(__fmul_rn(p, s2), 0.333333333f);
    p = __fadd_rn(__fmul_rn(p, s2), 1.0f);
    const float ln_m = __fmul_rn(__fmul_rn(2.0f, s), p);
    return __fadd_rn(__fmul_rn((float)e, 0.693147181f), ln_m);
}

// cos(pi/2 * t) for t in [0, 1]: the series in x = pi/2 * t up to x^14.
__device__ __forceinline__ float cos_quarter(float t) {
    const float x = __fmul_rn(t, 1.57079633f);
    const float x2 = __fmul_rn(x, x);
    float p = -1.14707456e-11f;                                   // -1/14!
    p = __fadd_rn(__fmul_rn(p, x2), 2.08767570e-9f);              //  1/12!
    p = __fadd_rn(__fmul_rn(p, x2), -2.75573192e-7f);             // -1/10!
    p = __fadd_rn(__fmul_rn(p, x2), 2.48015873e-5f);              //  1/8!
    p = __fadd_rn(__fmul_rn(p, x2), -1.38888889e-3f);             // -1/6!
    p = __fadd_rn(__fmul_rn(p, x2), 4.16666667e-2f);              //  1/4!
    p = __fadd_rn(__fmul_rn(p, x2), -0.5f);
    p = __fadd_rn(__fmul_rn(p, x2), 1.0f);
    return p;
}

__device__ __forceinline__ float normal_of(unsigned long long key, unsigned long long i) {
    const unsigned long long h = mix64(key + (i + 1ull) * 0x9E3779B97F4A7C15ull);
    const float u1 = __fmul_rn((float)((unsigned)(h >> 40) + 1u), 5.9604644775390625e-8f);
    const unsigned a = (unsigned)(h >> 8) & 0xFFFFFFu;
    const unsigned quadrant = a >> 22;
    const float t = __fmul_rn((float)(a & 0x3FFFFFu), 2.384185791015625e-7f);   // * 2^-22
    float c;
    if (quadrant == 0) c = cos_quarter(t);
    else if (quadrant == 1) c = -cos_quarter(__fadd_rn(1.0f, -t));
    else if (quadrant == 2) c = -cos_quarter(t);
    else c = cos_quarter(__fadd_rn(1.0f, -t));
    const float r = __fsqrt_rn(__fmul_rn(-2.0f, ln_unit(u1)));
    return __fmul_rn(r, c);
}

template <typename T>
__global__ void randn_fill_kernel(T* __restrict__ dst, long long rows, long long cols,
                                  long long group, long long group_stride,
                                  unsigned long long key, float offset, float std,
                                  int stored_bf16) {
    const long long n = rows * cols;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const long long r = i / cols, c = i - r * cols;
        const long long dr = group > 0 ? (r / group) * group_stride + r % group : r;
        float w = __fmul_rn(std, normal_of(key, (unsigned long long)i));
        if (stored_bf16) w = __bfloat162float(__float2bfloat16_rn(w));
        if (offset != 0.f) w = __fadd_rn(w, offset);
        dst[dr * cols + c] = from_f32<T>(w);
    }
}

}  // namespace

SIB_EXPORT int sib_randn_fill(void* dst, int dtype, long long rows, long long cols,
                              long long group, long long group_stride, unsigned long long key,
                              float offset, float std, int stored_dtype, void* stream) {
    SIB_REQUIRE(dst != nullptr && rows >= 0 && cols > 0, "randn_fill: rows=%lld cols=%lld", rows,
                cols);
    SIB_REQUIRE(group >= 0 && (group == 0 || (group_stride >= group && rows % group == 0)),
                "randn_fill: runs of %lld rows placed %lld rows apart do not fit %lld rows", group,
                group_stride, rows);
    if (rows == 0) return 0;
    const long long n = rows * cols;
    const int threads = 256;
    const long long want = (n + threads - 1) / threads;
    const unsigned blocks = (unsigned)(want < 8192 ? want : 8192);    // grid-stride beyond
    SIB_DISPATCH_DTYPE(dtype, randn_fill_kernel<T><<<blocks, threads, 0, (cudaStream_t)stream>>>(
                                  (T*)dst, rows, cols, group, group_stride, key, offset, std,
                                  stored_dtype == SIB_BF16 ? 1 : 0));
    return sib_check_launch("randn_fill");
}
