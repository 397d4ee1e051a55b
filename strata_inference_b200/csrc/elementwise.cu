// Embedding gather with scale, gated tanh-GELU, soft cap.
//
// Plain counterparts: tests/plain_gemma2.py embed(), gelu_tanh(), lm_head().
// Reference formulas: src/backend/cpu.rs:1086-1136 (row gather),
// src/model/layer.rs:1285-1288 (scale), src/backend/cpu.rs:1190-1199 (GeGLU).
#include "common.cuh"

// out[r, :] = scale * table[tokens[r], :], accumulated stream in f32.
template <typename T>
__global__ void embed_rows_kernel(const int* __restrict__ tokens, const T* __restrict__ table,
                                  float* __restrict__ out, int hidden, float scale) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    const T* src = table + (size_t)tokens[r] * hidden;
    float* dst = out + (size_t)r * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_f32(src[i]) * scale;
}

SIB_EXPORT int sib_embed_rows(const int* tokens, const void* table, int table_dtype, float* out,
                              int rows, int hidden, float scale, void* stream) {
    if (rows == 0) return 0;
    SIB_REQUIRE(rows > 0 && hidden > 0, "embed_rows: rows=%d hidden=%d", rows, hidden);
    SIB_DISPATCH_DTYPE(table_dtype,
                       sib_launch_chained(embed_rows_kernel<T>, dim3(rows), dim3(256), 0,
                                          (cudaStream_t)stream, tokens, (const T*)table, out, hidden,
                                          scale));
    return sib_check_launch("embed_rows");
}

__device__ __forceinline__ float gelu_tanh(float g) {
    const float c = 0.7978845608028654f;  // sqrt(2/pi)
    return 0.5f * g * (1.0f + tanhf(c * (g + 0.044715f * g * g * g)));
}

// out[r, i] = gelu_tanh(gate(r, i)) * up(r, i).  The two halves of gate_up[r, :]
// are laid out either as [all gates | all ups] (group == 0) or in groups of
// `group` gates followed by the `group` matching ups.
template <typename T>
__global__ void gelu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter,
                                int group, size_t total) {
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t r = idx / inter;
        const int i = (int)(idx - r * inter);
        const T* row = gate_up + r * 2 * (size_t)inter;
        const int gi = group ? (i / group) * 2 * group + i % group : i;
        const int ui = group ? gi + group : inter + i;
        const float g = to_f32(row[gi]), u = to_f32(row[ui]);
        out[idx] = from_f32<T>(gelu_tanh(g) * u);
    }
}

// The bfloat16 case with groups of 8: a group is 32 contiguous bytes (8 gates,
// 8 ups) and gives 16 contiguous bytes of output; one thread per group, every
// access 16 bytes wide.
__global__ void gelu_mul_group8_bf16_kernel(const uint4* __restrict__ gate_up,
                                            uint4* __restrict__ out, size_t groups) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < groups;
         i += (size_t)gridDim.x * blockDim.x) {
        const uint4 gv = gate_up[2 * i], uv = gate_up[2 * i + 1];
        const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
        uint32_t ow[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float g0 = __uint_as_float(gw[k] << 16), g1 = __uint_as_float(gw[k] & 0xffff0000u);
            const float u0 = __uint_as_float(uw[k] << 16), u1 = __uint_as_float(uw[k] & 0xffff0000u);
            const __nv_bfloat162 o = __floats2bfloat162_rn(gelu_tanh(g0) * u0, gelu_tanh(g1) * u1);
            ow[k] = *reinterpret_cast<const uint32_t*>(&o);
        }
        out[i] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
}

SIB_EXPORT int sib_gelu_mul(const void* gate_up, void* out, int dtype, int rows, int inter,
                            int group, void* stream) {
    if (rows == 0) return 0;
    SIB_REQUIRE(rows > 0 && inter > 0, "gelu_mul: rows=%d inter=%d", rows, inter);
    SIB_REQUIRE(group >= 0 && (group == 0 || inter % group == 0),
                "gelu_mul: %d columns do not come in groups of %d", inter, group);
    const size_t total = (size_t)rows * inter;
    if (dtype == SIB_BF16 && group == 8 && ((uintptr_t)gate_up % 16) == 0 &&
        ((uintptr_t)out % 16) == 0) {
        const size_t groups = total / 8;
        const size_t want = (groups + 255) / 256;
        const int blocks = (int)(want < 148 * 32 ? want : 148 * 32);
        gelu_mul_group8_bf16_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(
            (const uint4*)gate_up, (uint4*)out, groups);
        return sib_check_launch("gelu_mul");
    }
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    SIB_DISPATCH_DTYPE(dtype, (gelu_mul_kernel<T><<<blocks, 256, 0, (cudaStream_t)stream>>>(
                                  (const T*)gate_up, (T*)out, inter, group, total)));
    return sib_check_launch("gelu_mul");
}

// x = cap * tanh(x / cap), in place, 32-bit.
__global__ void softcap_kernel(float* x, size_t total, float cap) {
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x)
        x[idx] = cap * tanhf(x[idx] / cap);
}

SIB_EXPORT int sib_softcap(float* x, long long total, float cap, void* stream) {
    if (total == 0 || cap <= 0.f) return 0;
    const long long want = (total + 255) / 256;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    softcap_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(x, (size_t)total, cap);
    return sib_check_launch("softcap");
}
