// RMS norm, alone and fused with the residual add around it.
//
//   rms(x, g) = x * 1/sqrt(mean(x^2) + eps) * g        (statistics in f32)
//
// The gain g arrives ready-made in f32 (the norm part adds the architecture's
// offset to the stored weight once, when it is built).
// Plain counterpart: tests/plain_gemma2.py rms_norm().
// Reference formula: src/backend/cpu.rs:797-810; the order "norm of the
// sub-layer's output, then the add" is src/model/layer.rs:1163-1170,1185-1192.
#include "common.cuh"

// out[i, :] = rms(x[rows ? rows[i] : i, :], gain).  The row is held in shared
// memory (hidden floats) between the two passes.
template <typename Tin, typename Tout>
__global__ void rms_norm_kernel(const Tin* __restrict__ x, const int* __restrict__ rows,
                                const float* __restrict__ gain, Tout* __restrict__ out,
                                int hidden, float eps) {
    extern __shared__ float row[];
    __shared__ float scratch[33];
    const int i = blockIdx.x;
    const Tin* src = x + (size_t)(rows ? rows[i] : i) * hidden;
    float ss = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float v = to_f32(src[c]);
        row[c] = v;
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
    Tout* dst = out + (size_t)i * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x)
        dst[c] = from_f32<Tout>(row[c] * inv * gain[c]);
}

// h[r, :] += post_gain ? rms(a[r, :], post_gain) : a[r, :]
// out[r, :] = rms(h[r, :], pre_gain)            (only if pre_gain)
// h is the 32-bit residual stream; a and out have the activation type.
template <typename T>
__global__ void add_rms_norm_kernel(const T* __restrict__ a, const float* __restrict__ post_gain,
                                    float post_eps, float* __restrict__ h,
                                    const float* __restrict__ pre_gain, float pre_eps,
                                    T* __restrict__ out, int hidden) {
    extern __shared__ float row[];
    __shared__ float scratch[33];
    const size_t base = (size_t)blockIdx.x * hidden;
    float ss = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float v = to_f32(a[base + c]);
        row[c] = v;
        ss += v * v;
    }
    float inv = 1.f;
    if (post_gain) {
        ss = block_sum(ss, scratch);
        inv = 1.0f / sqrtf(ss / (float)hidden + post_eps);
    }
    float ss2 = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float add = post_gain ? row[c] * inv * post_gain[c] : row[c];
        const float v = h[base + c] + add;
        h[base + c] = v;
        row[c] = v;
        ss2 += v * v;
    }
    if (!pre_gain) return;
    ss2 = block_sum(ss2, scratch);
    const float inv2 = 1.0f / sqrtf(ss2 / (float)hidden + pre_eps);
    for (int c = threadIdx.x; c < hidden; c += blockDim.x)
        out[base + c] = from_f32<T>(row[c] * inv2 * pre_gain[c]);
}

static int norm_threads(int hidden) {
    int t = 128;
    while (t < 1024 && t * 4 < hidden) t *= 2;
    return t;
}

static const int kMaxRowBytes = 200 * 1024;

template <typename K>
static int allow_row(K kernel, size_t bytes) {
    if (bytes <= 48 * 1024) return 0;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)bytes);
    if (e != cudaSuccess) {
        sib_set_error("norm: cannot reserve %zu bytes of shared memory: %s", bytes,
                      cudaGetErrorString(e));
        return (int)e;
    }
    return 0;
}

SIB_EXPORT int sib_rms_norm(const void* x, int in_dtype, const int* rows, const float* gain,
                            float eps, void* out, int out_dtype, int n_rows, int hidden,
                            void* stream) {
    if (n_rows == 0) return 0;
    SIB_REQUIRE(n_rows > 0 && hidden > 0, "rms_norm: rows=%d hidden=%d", n_rows, hidden);
    const size_t smem = (size_t)hidden * sizeof(float);
    SIB_REQUIRE(smem <= (size_t)kMaxRowBytes,
                "rms_norm: hidden=%d needs %zu bytes of shared memory; at most %d are supported",
                hidden, smem, kMaxRowBytes);
    const int threads = norm_threads(hidden);
    cudaStream_t s = (cudaStream_t)stream;
#define LAUNCH(TIN, TOUT)                                                              \
    do {                                                                               \
        int rc = allow_row(rms_norm_kernel<TIN, TOUT>, smem);                          \
        if (rc) return rc;                                                             \
        rms_norm_kernel<TIN, TOUT><<<n_rows, threads, smem, s>>>(                      \
            (const TIN*)x, rows, gain, (TOUT*)out, hidden, eps);                       \
    } while (0)
    if (in_dtype == SIB_F32 && out_dtype == SIB_F32) LAUNCH(float, float);
    else if (in_dtype == SIB_F32 && out_dtype == SIB_BF16) LAUNCH(float, __nv_bfloat16);
    else if (in_dtype == SIB_BF16 && out_dtype == SIB_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else if (in_dtype == SIB_BF16 && out_dtype == SIB_F32) LAUNCH(__nv_bfloat16, float);
    else SIB_REQUIRE(false, "rms_norm: unknown element types %d -> %d", in_dtype, out_dtype);
#undef LAUNCH
    return sib_check_launch("rms_norm");
}

SIB_EXPORT int sib_add_rms_norm(const void* a, int dtype, const float* post_gain, float post_eps,
                                float* h, const float* pre_gain, float pre_eps, void* out,
                                int n_rows, int hidden, void* stream) {
    if (n_rows == 0) return 0;
    SIB_REQUIRE(n_rows > 0 && hidden > 0, "add_rms_norm: rows=%d hidden=%d", n_rows, hidden);
    SIB_REQUIRE(pre_gain == nullptr || out != nullptr, "add_rms_norm: pre_gain without out");
    const size_t smem = (size_t)hidden * sizeof(float);
    SIB_REQUIRE(smem <= (size_t)kMaxRowBytes,
                "add_rms_norm: hidden=%d needs %zu bytes of shared memory; at most %d are supported",
                hidden, smem, kMaxRowBytes);
    const int threads = norm_threads(hidden);
    SIB_DISPATCH_DTYPE(dtype, {
        int rc = allow_row(add_rms_norm_kernel<T>, smem);
        if (rc) return rc;
        add_rms_norm_kernel<T><<<n_rows, threads, smem, (cudaStream_t)stream>>>(
            (const T*)a, post_gain, post_eps, h, pre_gain, pre_eps, (T*)out, hidden);
    });
    return sib_check_launch("add_rms_norm");
}
