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
    pdl_trigger();
    pdl_wait();
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
    pdl_trigger();
    pdl_wait();
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

// The same for bfloat16 activations and a hidden size in whole groups of 8: every
// access is 16 bytes wide (8 activations, 4 stream or gain values).
__global__ void add_rms_norm_bf16_kernel(const __nv_bfloat16* __restrict__ a,
                                         const float* __restrict__ post_gain, float post_eps,
                                         float* __restrict__ h, const float* __restrict__ pre_gain,
                                         float pre_eps, __nv_bfloat16* __restrict__ out, int hidden) {
    extern __shared__ float row[];
    __shared__ float scratch[33];
    pdl_trigger();
    pdl_wait();
    const size_t base = (size_t)blockIdx.x * hidden;
    const int groups = hidden / 8;
    float ss = 0.f;
    for (int v = threadIdx.x; v < groups; v += blockDim.x) {
        const uint4 raw = *reinterpret_cast<const uint4*>(a + base + 8 * v);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float lo = __uint_as_float(w[k] << 16), hi = __uint_as_float(w[k] & 0xffff0000u);
            row[8 * v + 2 * k] = lo;
            row[8 * v + 2 * k + 1] = hi;
            ss += lo * lo + hi * hi;
        }
    }
    float inv = 1.f;
    if (post_gain) {
        ss = block_sum(ss, scratch);
        inv = 1.0f / sqrtf(ss / (float)hidden + post_eps);
    } else {
        __syncthreads();   // the next pass reads the row in another order
    }
    float ss2 = 0.f;
    for (int v = threadIdx.x; v < 2 * groups; v += blockDim.x) {   // float4 at a time
        float4 hv = *reinterpret_cast<const float4*>(h + base + 4 * v);
        float4 av = *reinterpret_cast<const float4*>(row + 4 * v);
        if (post_gain) {
            const float4 gv = *reinterpret_cast<const float4*>(post_gain + 4 * v);
            av.x *= inv * gv.x; av.y *= inv * gv.y; av.z *= inv * gv.z; av.w *= inv * gv.w;
        }
        hv.x += av.x; hv.y += av.y; hv.z += av.z; hv.w += av.w;
        *reinterpret_cast<float4*>(h + base + 4 * v) = hv;
        *reinterpret_cast<float4*>(row + 4 * v) = hv;
        ss2 += hv.x * hv.x + hv.y * hv.y + hv.z * hv.z + hv.w * hv.w;
    }
    if (!pre_gain) return;
    ss2 = block_sum(ss2, scratch);
    const float inv2 = 1.0f / sqrtf(ss2 / (float)hidden + pre_eps);
    for (int v = threadIdx.x; v < groups; v += blockDim.x) {
        uint32_t w[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int c = 8 * v + 2 * k;
            const __nv_bfloat162 o = __floats2bfloat162_rn(row[c] * inv2 * pre_gain[c],
                                                           row[c + 1] * inv2 * pre_gain[c + 1]);
            w[k] = *reinterpret_cast<const uint32_t*>(&o);
        }
        *reinterpret_cast<uint4*>(out + base + 8 * v) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// One warp per row, the row in registers, no block-wide barrier: for hidden sizes that
// are NG x 256 (lane l owns the 8-element groups l, l + 32, ...).
template <int NG>
__global__ void __launch_bounds__(128)
add_rms_norm_bf16_warp_kernel(const __nv_bfloat16* __restrict__ a, const float* __restrict__ post_gain,
                              float post_eps, float* __restrict__ h,
                              const float* __restrict__ pre_gain, float pre_eps,
                              __nv_bfloat16* __restrict__ out, int n_rows) {
    pdl_trigger();
    pdl_wait();
    constexpr int hidden = NG * 256;
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (r >= n_rows) return;
    const size_t base = (size_t)r * hidden;
    float v[NG][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NG; ++i) {
        const uint4 raw = *reinterpret_cast<const uint4*>(a + base + 8 * (lane + 32 * i));
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            v[i][2 * k] = __uint_as_float(w[k] << 16);
            v[i][2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
            ss += v[i][2 * k] * v[i][2 * k] + v[i][2 * k + 1] * v[i][2 * k + 1];
        }
    }
    float inv = 1.f;
    if (post_gain) inv = 1.0f / sqrtf(warp_sum(ss) / (float)hidden + post_eps);
    float ss2 = 0.f;
#pragma unroll
    for (int i = 0; i < NG; ++i) {
        const int c = 8 * (lane + 32 * i);
        float4 h0 = *reinterpret_cast<const float4*>(h + base + c);
        float4 h1 = *reinterpret_cast<const float4*>(h + base + c + 4);
        if (post_gain) {
            const float4 g0 = *reinterpret_cast<const float4*>(post_gain + c);
            const float4 g1 = *reinterpret_cast<const float4*>(post_gain + c + 4);
            v[i][0] *= inv * g0.x; v[i][1] *= inv * g0.y; v[i][2] *= inv * g0.z; v[i][3] *= inv * g0.w;
            v[i][4] *= inv * g1.x; v[i][5] *= inv * g1.y; v[i][6] *= inv * g1.z; v[i][7] *= inv * g1.w;
        }
        h0.x += v[i][0]; h0.y += v[i][1]; h0.z += v[i][2]; h0.w += v[i][3];
        h1.x += v[i][4]; h1.y += v[i][5]; h1.z += v[i][6]; h1.w += v[i][7];
        *reinterpret_cast<float4*>(h + base + c) = h0;
        *reinterpret_cast<float4*>(h + base + c + 4) = h1;
        v[i][0] = h0.x; v[i][1] = h0.y; v[i][2] = h0.z; v[i][3] = h0.w;
        v[i][4] = h1.x; v[i][5] = h1.y; v[i][6] = h1.z; v[i][7] = h1.w;
#pragma unroll
        for (int e = 0; e < 8; ++e) ss2 += v[i][e] * v[i][e];
    }
    if (!pre_gain) return;
    const float inv2 = 1.0f / sqrtf(warp_sum(ss2) / (float)hidden + pre_eps);
#pragma unroll
    for (int i = 0; i < NG; ++i) {
        const int c = 8 * (lane + 32 * i);
        const float4 g0 = *reinterpret_cast<const float4*>(pre_gain + c);
        const float4 g1 = *reinterpret_cast<const float4*>(pre_gain + c + 4);
        const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
        uint32_t w[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const __nv_bfloat162 o = __floats2bfloat162_rn(v[i][2 * k] * inv2 * g[2 * k],
                                                           v[i][2 * k + 1] * inv2 * g[2 * k + 1]);
            w[k] = *reinterpret_cast<const uint32_t*>(&o);
        }
        *reinterpret_cast<uint4*>(out + base + c) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// One block per row, one 8-element group per thread, the row in registers: every load of a
// row is issued before anything is computed (the gains even before the kernel ahead of this
// one has finished), so a row costs two block-wide sums and no pass over shared memory.
__global__ void __launch_bounds__(1024)
add_rms_norm_bf16_group_kernel(const __nv_bfloat16* __restrict__ a, const float* __restrict__ post_gain,
                               float post_eps, float* __restrict__ h,
                               const float* __restrict__ pre_gain, float pre_eps,
                               __nv_bfloat16* __restrict__ out, int hidden) {
    __shared__ float scratch[33];
    pdl_trigger();
    const int c = 8 * threadIdx.x;
    const bool live = c < hidden;
    const float4 one = make_float4(1.f, 1.f, 1.f, 1.f);
    float4 pg0 = one, pg1 = one, qg0 = one, qg1 = one;
    if (live && post_gain) {
        pg0 = *reinterpret_cast<const float4*>(post_gain + c);
        pg1 = *reinterpret_cast<const float4*>(post_gain + c + 4);
    }
    if (live && pre_gain) {
        qg0 = *reinterpret_cast<const float4*>(pre_gain + c);
        qg1 = *reinterpret_cast<const float4*>(pre_gain + c + 4);
    }
    pdl_wait();
    const size_t base = (size_t)blockIdx.x * hidden + c;
    uint4 raw = make_uint4(0, 0, 0, 0);
    float4 h0 = make_float4(0.f, 0.f, 0.f, 0.f), h1 = h0;
    if (live) {
        raw = *reinterpret_cast<const uint4*>(a + base);
        h0 = *reinterpret_cast<const float4*>(h + base);
        h1 = *reinterpret_cast<const float4*>(h + base + 4);
    }
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    float v[8];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        v[2 * k] = __uint_as_float(w[k] << 16);
        v[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
        ss += v[2 * k] * v[2 * k] + v[2 * k + 1] * v[2 * k + 1];
    }
    if (post_gain) {
        ss = block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)hidden + post_eps);
        v[0] *= inv * pg0.x; v[1] *= inv * pg0.y; v[2] *= inv * pg0.z; v[3] *= inv * pg0.w;
        v[4] *= inv * pg1.x; v[5] *= inv * pg1.y; v[6] *= inv * pg1.z; v[7] *= inv * pg1.w;
    }
    h0.x += v[0]; h0.y += v[1]; h0.z += v[2]; h0.w += v[3];
    h1.x += v[4]; h1.y += v[5]; h1.z += v[6]; h1.w += v[7];
    if (live) {
        *reinterpret_cast<float4*>(h + base) = h0;
        *reinterpret_cast<float4*>(h + base + 4) = h1;
    }
    if (!pre_gain) return;
    float ss2 = h0.x * h0.x + h0.y * h0.y + h0.z * h0.z + h0.w * h0.w +
                h1.x * h1.x + h1.y * h1.y + h1.z * h1.z + h1.w * h1.w;
    ss2 = block_sum(ss2, scratch);
    const float inv2 = 1.0f / sqrtf(ss2 / (float)hidden + pre_eps);
    if (live) {
        const __nv_bfloat162 o0 = __floats2bfloat162_rn(h0.x * inv2 * qg0.x, h0.y * inv2 * qg0.y);
        const __nv_bfloat162 o1 = __floats2bfloat162_rn(h0.z * inv2 * qg0.z, h0.w * inv2 * qg0.w);
        const __nv_bfloat162 o2 = __floats2bfloat162_rn(h1.x * inv2 * qg1.x, h1.y * inv2 * qg1.y);
        const __nv_bfloat162 o3 = __floats2bfloat162_rn(h1.z * inv2 * qg1.z, h1.w * inv2 * qg1.w);
        *reinterpret_cast<uint4*>(out + base) =
            make_uint4(*reinterpret_cast<const uint32_t*>(&o0), *reinterpret_cast<const uint32_t*>(&o1),
                       *reinterpret_cast<const uint32_t*>(&o2), *reinterpret_cast<const uint32_t*>(&o3));
    }
}

template <int NG>
static int launch_warp_norm(const void* a, const float* post_gain, float post_eps, float* h,
                            const float* pre_gain, float pre_eps, void* out, int n_rows,
                            cudaStream_t s) {
    sib_launch_chained(add_rms_norm_bf16_warp_kernel<NG>, dim3((n_rows + 3) / 4), dim3(128), 0, s,
                       (const __nv_bfloat16*)a, post_gain, post_eps, h, pre_gain, pre_eps,
                       (__nv_bfloat16*)out, n_rows);
    return sib_check_launch("add_rms_norm");
}

#include <stdlib.h>
#include <string.h>

// SIB_NORM_KERNEL=warp keeps the warp-per-row kernel for many rows.
static int norm_kernel_mode() {
    const char* v = getenv("SIB_NORM_KERNEL");
    return (v && strcmp(v, "warp") == 0) ? 1 : 0;
}
// From this many rows on the group-per-thread kernel runs (SIB_NORM_GROUP_ROWS overrides).
// It is the faster one at every number of rows: single-token steps of the Gemma2-2B shape gain
// 5 % at batch 8 and 6 % at batch 1 over the kernel that stages the row in shared memory, the 9B
// and 27B shapes 3 % and 1 %.
static int group_rows_threshold() {
    static int t = -1;
    if (t < 0) {
        const char* v = getenv("SIB_NORM_GROUP_ROWS");
        t = v ? atoi(v) : 1;
        if (t < 1) t = 1;
    }
    return t;
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
        sib_launch_chained(rms_norm_kernel<TIN, TOUT>, dim3(n_rows), dim3(threads), smem, s, \
                           (const TIN*)x, rows, gain, (TOUT*)out, hidden, eps);        \
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
    if (dtype == SIB_BF16 && hidden % 8 == 0 && ((uintptr_t)a % 16) == 0 &&
        ((uintptr_t)h % 16) == 0 && ((uintptr_t)out % 16) == 0 &&
        ((uintptr_t)post_gain % 16) == 0 && ((uintptr_t)pre_gain % 16) == 0) {
        // a block per row with one 8-element group per thread, every load issued at once
        // (SIB_NORM_KERNEL=warp: for many rows a warp per row, for few the row in shared memory)
        static const int mode = norm_kernel_mode();
        if (n_rows >= group_rows_threshold() && hidden / 8 <= 1024 && mode != 1) {
            const int threads = (hidden / 8 + 31) / 32 * 32;
            sib_launch_chained(add_rms_norm_bf16_group_kernel, dim3(n_rows), dim3(threads), 0,
                               (cudaStream_t)stream, (const __nv_bfloat16*)a, post_gain, post_eps, h,
                               pre_gain, pre_eps, (__nv_bfloat16*)out, hidden);
            return sib_check_launch("add_rms_norm");
        }
        if (n_rows >= 512 && hidden % 256 == 0 && hidden / 256 <= 18) {
            cudaStream_t s = (cudaStream_t)stream;
#define NORM_CASE(NG) \
    case NG: return launch_warp_norm<NG>(a, post_gain, post_eps, h, pre_gain, pre_eps, out, n_rows, s)
            switch (hidden / 256) {
                NORM_CASE(1); NORM_CASE(2); NORM_CASE(3); NORM_CASE(4); NORM_CASE(5); NORM_CASE(6);
                NORM_CASE(7); NORM_CASE(8); NORM_CASE(9); NORM_CASE(10); NORM_CASE(11); NORM_CASE(12);
                NORM_CASE(13); NORM_CASE(14); NORM_CASE(15); NORM_CASE(16); NORM_CASE(17); NORM_CASE(18);
            }
#undef NORM_CASE
        }
        int rc = allow_row(add_rms_norm_bf16_kernel, smem);
        if (rc) return rc;
        sib_launch_chained(add_rms_norm_bf16_kernel, dim3(n_rows),
                           dim3(threads < 256 ? threads : 256), smem, (cudaStream_t)stream,
                           (const __nv_bfloat16*)a, post_gain, post_eps, h, pre_gain, pre_eps,
                           (__nv_bfloat16*)out, hidden);
        return sib_check_launch("add_rms_norm");
    }
    SIB_DISPATCH_DTYPE(dtype, {
        int rc = allow_row(add_rms_norm_kernel<T>, smem);
        if (rc) return rc;
        sib_launch_chained(add_rms_norm_kernel<T>, dim3(n_rows), dim3(threads), smem,
                           (cudaStream_t)stream, (const T*)a, post_gain, post_eps, h, pre_gain,
                           pre_eps, (T*)out, hidden);
    });
    return sib_check_launch("add_rms_norm");
}
