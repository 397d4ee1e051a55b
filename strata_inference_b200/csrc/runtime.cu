// Error reporting shared by all exported launchers.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>

#include "common.cuh"
#include "tma.cuh"

static thread_local char g_error[512] = "";

void sib_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

// After a launch: 0, or the CUDA error's code with its text recorded.
int sib_check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) return 0;
    sib_set_error("%s: %s", what, cudaGetErrorString(e));
    return (int)e;
}

bool sib_chained_launches() {
    static int enabled = -1;
    if (enabled < 0) {
        const char* v = getenv("SIB_CHAINED_LAUNCH");
        enabled = (v && v[0] == '0') ? 0 : 1;
    }
    return enabled == 1;
}

int sib_carveout() {
    static int value = -2;
    if (value == -2) {
        const char* v = getenv("SIB_CARVEOUT");
        value = v ? atoi(v) : -1;
        if (value > 100) value = 100;
    }
    return value;
}

SIB_EXPORT const char* sib_last_error() { return g_error; }

// The architecture this library was compiled for; the loader refuses any other.
SIB_EXPORT int sib_compiled_arch() {
#ifdef SIB_ARCH
    return SIB_ARCH;
#else
    return 0;
#endif
}

// ---------------------------------------------------------------------------
// The per-device table of error words (common.cuh).
// ---------------------------------------------------------------------------
#include <mutex>

static int* g_error_words[64] = {};
static std::mutex g_error_mutex;
static const char* const kErrorWordNames[SIB_ERROR_WORDS] = {
    "gemm_tcgen05", "attention_prefill_tc", "linear_stream", "decode_chain", "linear_rows_tc", "", "", ""};

static int* error_table() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        sib_set_error("no current CUDA device for the table of error words");
        return nullptr;
    }
    std::lock_guard<std::mutex> guard(g_error_mutex);
    if (!g_error_words[dev]) {
        int* p = nullptr;
        cudaError_t e = cudaMalloc(&p, SIB_ERROR_WORDS * sizeof(int));
        if (e != cudaSuccess) {
            sib_set_error("table of error words: %s", cudaGetErrorString(e));
            return nullptr;
        }
        cudaMemset(p, 0, SIB_ERROR_WORDS * sizeof(int));
        g_error_words[dev] = p;
    }
    return g_error_words[dev];
}

int* sib_error_word(int word) {
    int* t = (word >= 0 && word < SIB_ERROR_WORDS) ? error_table() : nullptr;
    return t ? t + word : nullptr;
}

SIB_EXPORT int sib_error_words() { return SIB_ERROR_WORDS; }

SIB_EXPORT const char* sib_error_word_name(int word) {
    return (word >= 0 && word < SIB_ERROR_WORDS) ? kErrorWordNames[word] : "";
}

// Copy the table to `host` (SIB_ERROR_WORDS ints, pinned for the copy to be asynchronous)
// on `stream`: the words are valid once the stream has reached this point.
SIB_EXPORT int sib_kernel_errors_fetch(int* host, void* stream) {
    int* t = error_table();
    if (!t) return -1;
    cudaError_t e = cudaMemcpyAsync(host, t, SIB_ERROR_WORDS * sizeof(int), cudaMemcpyDeviceToHost,
                                    (cudaStream_t)stream);
    if (e != cudaSuccess) {
        sib_set_error("fetching the error words: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return 0;
}

// Set one word (0 clears it).  The kernels set their words themselves; the host sets one
// to clear it after a report, and tests set one to stand for a failure.
SIB_EXPORT int sib_kernel_error_set(int word, int code, void* stream) {
    int* w = sib_error_word(word);
    if (!w) return -1;
    // (a 4-byte pattern needs the 32-bit memset of the driver API; codes fit a byte)
    SIB_REQUIRE(code >= 0 && code < 256, "error codes are 0..255, got %d", code);
    cudaError_t e = cudaMemsetAsync(w, 0, sizeof(int), (cudaStream_t)stream);
    if (e == cudaSuccess && code) e = cudaMemsetAsync(w, code, 1, (cudaStream_t)stream);
    if (e != cudaSuccess) {
        sib_set_error("setting an error word: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return 0;
}

// One word, read with a synchronous copy (tests, and after a failure).
static int error_word_now(int word, int clear) {
    int* w = sib_error_word(word);
    if (!w) return 0;
    int v = 0;
    cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost);
    if (clear && v) cudaMemset(w, 0, sizeof(int));
    return v;
}

// 0, or the code a block of gemm_tcgen05 left when one of its waits ran out (1: a stage
// never became free, 2: a load never arrived, 3: the accumulator never became ready).
SIB_EXPORT int sib_gemm_tcgen05_error(int clear) { return error_word_now(SIB_ERR_GEMM_TCGEN05, clear); }

SIB_EXPORT int sib_attention_prefill_tc_error(int clear) {
    return error_word_now(SIB_ERR_ATTENTION_PREFILL_TC, clear);
}

// ---------------------------------------------------------------------------
// Tensor maps (tma.cuh).
// ---------------------------------------------------------------------------
SibEncodeTiledFn sib_encode_tiled_fn() {
    static SibEncodeTiledFn fn = nullptr;
    if (fn) return fn;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
        return nullptr;
    fn = (SibEncodeTiledFn)ptr;
    return fn;
}

int sib_make_bf16_map(CUtensorMap* map, const void* base, long long rows, long long cols,
                      long long row_stride, int box_rows, const char* who) {
    SibEncodeTiledFn enc = sib_encode_tiled_fn();
    if (!enc) {
        sib_set_error("%s: cuTensorMapEncodeTiled is not available", who);
        return -1;
    }
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)row_stride * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                     box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        sib_set_error("%s: cuTensorMapEncodeTiled failed with code %d", who, (int)r);
        return -1;
    }
    return 0;
}

int sib_make_bf16_map_k_tiles(CUtensorMap* map, const void* base, long long rows, long long cols,
                              long long row_stride, int box_rows, int box_tiles, const char* who) {
    SibEncodeTiledFn enc = sib_encode_tiled_fn();
    if (!enc) {
        sib_set_error("%s: cuTensorMapEncodeTiled is not available", who);
        return -1;
    }
    if (cols % 64 != 0) {
        sib_set_error("%s: %lld columns are not whole blocks of 64", who, cols);
        return -1;
    }
    cuuint64_t dims[3] = {64u, (cuuint64_t)rows, (cuuint64_t)(cols / 64)};
    cuuint64_t strides[2] = {(cuuint64_t)row_stride * 2, 128u};
    cuuint32_t box[3] = {64u, (cuuint32_t)box_rows, (cuuint32_t)box_tiles};
    cuuint32_t elem[3] = {1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides,
                     box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        sib_set_error("%s: cuTensorMapEncodeTiled (3-d) failed with code %d", who, (int)r);
        return -1;
    }
    return 0;
}
