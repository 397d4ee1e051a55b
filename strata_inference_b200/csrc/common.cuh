// Shared helpers of the sm_100a kernels: element types, warp and block
// reductions, launch checks.  Every exported function is plain C, takes raw
// device pointers and the stream to launch on, and returns 0 or an error
// code whose text sib_last_error() gives.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define SIB_EXPORT extern "C" __attribute__((visibility("default")))

enum SibDtype { SIB_F32 = 0, SIB_BF16 = 1 };

void sib_set_error(const char* fmt, ...);
int sib_check_launch(const char* what);

// Programmatic dependent launch: a kernel launched with sib_launch_chained may begin
// while the kernel before it on the stream is still running.  It may do work
// that reads nothing the earlier kernel writes (prefetching weights), then calls
// pdl_wait(), which returns once the earlier kernel has completed and its writes
// are visible.  pdl_trigger() lets the NEXT kernel of the stream begin in the same
// way.  Without the launch attribute both are no-ops.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_trigger() {
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
#endif

bool sib_chained_launches();   // false when the environment sets SIB_CHAINED_LAUNCH=0
int sib_carveout();            // the shared-memory carve-out (percent) every kernel asks for, or -1

// Every kernel of a step asks for the same split of an SM's memory between shared memory
// and L1: a kernel that needs another split than its predecessor cannot start under it.
template <typename K> inline void sib_same_carveout(K kernel) {
    const int c = sib_carveout();
    if (c >= 0) cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, c);
}

// Kernels whose waits are bounded (mbarrier waits of the tcgen05 kernels) leave a code in
// "their" word of a small per-device table when a wait ran out.  The table is allocated
// at the first use on a device; the host fetches it with an asynchronous copy on the
// step's stream and looks at it wherever it synchronises anyway (runtime.cu).
enum SibErrorWord {
    SIB_ERR_GEMM_TCGEN05 = 0, SIB_ERR_ATTENTION_PREFILL_TC = 1, SIB_ERR_LINEAR_STREAM = 2,
    SIB_ERR_DECODE_CHAIN = 3, SIB_ERR_LINEAR_ROWS_TC = 4,
    SIB_ERROR_WORDS = 8
};
int* sib_error_word(int word);   // device address of the current device's word; null on failure

template <typename... KArgs, typename... Args>
inline cudaError_t sib_launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                      cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = sib_chained_launches() ? 1 : 0;
    sib_same_carveout(kernel);
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

#define SIB_REQUIRE(cond, ...)            \
    do {                                  \
        if (!(cond)) {                    \
            sib_set_error(__VA_ARGS__);   \
            return -1;                    \
        }                                 \
    } while (0)

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
    return __bfloat162float(v);
}
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` holds 33 floats of shared memory and may be reused after return.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// Dispatch on a SibDtype code: BODY sees the element type as T.
#define SIB_DISPATCH_DTYPE(code, ...)                                         \
    do {                                                                      \
        if ((code) == SIB_F32) { typedef float T; __VA_ARGS__; }              \
        else if ((code) == SIB_BF16) { typedef __nv_bfloat16 T; __VA_ARGS__; } \
        else { sib_set_error("unknown element type code %d", (int)(code)); return -1; } \
    } while (0)
