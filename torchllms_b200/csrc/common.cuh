// Shared helpers of the sm_100a kernels: element conversion, launch checks, the C ABI convention.
//
// Every exported function is `extern "C" int tl_<name>(..., void* stream)`.  It
// validates what only the host can see cheaply, launches on `stream`, and returns 0
// or a negative code from the enum below (positive values are cudaError_t).  The
// Python side turns a non-zero return into an exception; nothing here allocates
// memory, synchronises a stream or keeps state between calls.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdlib.h>

enum TlStatus : int {
    TL_OK = 0,
    TL_BAD_DTYPE = -1,      // dtype code is not one of TL_F32 / TL_BF16
    TL_BAD_SIZE = -2,       // a size the kernel refuses (see the message of the Python wrapper)
    TL_BAD_ALIGN = -3,      // a pointer or row pitch is not aligned as the kernel needs
    TL_TOO_LARGE = -4,      // needs more shared memory or scratch than there is
};

enum TlDtype : int { TL_F32 = 0, TL_BF16 = 1 };

#define TL_LAUNCH_CHECK()                                  \
    do {                                                   \
        cudaError_t e__ = cudaGetLastError();              \
        if (e__ != cudaSuccess) return (int)e__;           \
    } while (0)

__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// 16-byte vector of elements: 4 floats or 8 bfloat16.
template <typename T> struct Vec16;
template <> struct Vec16<float> {
    static constexpr int N = 4;
    float4 v;
    __device__ __forceinline__ void load(const float* p) { v = *reinterpret_cast<const float4*>(p); }
    __device__ __forceinline__ void store(float* p) const { *reinterpret_cast<float4*>(p) = v; }
    __device__ __forceinline__ float get(int i) const { return reinterpret_cast<const float*>(&v)[i]; }
    __device__ __forceinline__ void set(int i, float x) { reinterpret_cast<float*>(&v)[i] = x; }
};
template <> struct Vec16<__nv_bfloat16> {
    static constexpr int N = 8;
    uint4 v;
    __device__ __forceinline__ void load(const __nv_bfloat16* p) { v = *reinterpret_cast<const uint4*>(p); }
    __device__ __forceinline__ void store(__nv_bfloat16* p) const { *reinterpret_cast<uint4*>(p) = v; }
    __device__ __forceinline__ float get(int i) const {
        return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(&v)[i]);
    }
    __device__ __forceinline__ void set(int i, float x) {
        reinterpret_cast<__nv_bfloat16*>(&v)[i] = __float2bfloat16_rn(x);
    }
};

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}
__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
    return x;
}

// ---- debug builds (-DTL_DEBUG): every index that a kernel takes from the step's index data is
// range-checked before it is used.  A bad one is not followed (the access is skipped or reads
// zeros) and its kind is left in the library's debug word, which the host reads with
// tl_debug_take(); nothing traps.  The limits that a kernel's arguments do not carry (pages of the
// page tensor in use, rows of the stream) are set by the host before the launch, in stream order.
// Release builds compile the checks away.
enum : int { TL_DBG_TOKEN_ID = 901, TL_DBG_POSITION = 902, TL_DBG_SLOT = 903, TL_DBG_PAGE = 904, TL_DBG_ROW = 905 };
#ifdef TL_DEBUG
__device__ int tl_debug_word = 0;
__device__ long long tl_debug_limits[2] = {0, 0};      // pages of the page tensor, rows of the stream (0: unknown)
__device__ __forceinline__ bool tl_debug_ok(bool cond, int code) {
    if (!cond) atomicCAS(&tl_debug_word, 0, code);
    return cond;
}
__device__ __forceinline__ bool tl_check_page(long long page) {
    return tl_debug_ok(page >= 0 && (tl_debug_limits[0] == 0 || page < tl_debug_limits[0]), TL_DBG_PAGE);
}
__device__ __forceinline__ bool tl_check_row(long long row) {
    return tl_debug_ok(row >= 0 && (tl_debug_limits[1] == 0 || row < tl_debug_limits[1]), TL_DBG_ROW);
}
#define TL_CHECK(cond, code) tl_debug_ok((cond), (code))
// which limit (0: pages, 1: rows), its value; ordered with the launches on `stream`
extern "C" int tl_debug_set_limit(int which, long long value, void* stream) {
    if (which < 0 || which > 1) return TL_BAD_SIZE;
    return (int)cudaMemcpyToSymbolAsync(tl_debug_limits, &value, sizeof(value), which * sizeof(long long),
                                        cudaMemcpyHostToDevice, (cudaStream_t)stream);
}
// the code of the first bad index since the last call (0: none); waits for the device
extern "C" int tl_debug_take() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, tl_debug_word, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(tl_debug_word, &zero, sizeof(int));
    return v;
}
#else
__device__ __forceinline__ bool tl_check_page(long long) { return true; }
__device__ __forceinline__ bool tl_check_row(long long) { return true; }
#define TL_CHECK(cond, code) true
#endif

// ---- rows whose RMS normalisation was deferred: the kernel that produced them left the weighted rows
// and, beside them, the parts of every row's sum of squares (one part per strip of columns that a
// CTA of the producer owned).  Whoever ends the chain of products multiplies by
// rsqrt(sum of the parts * inv_dim + eps); ssq == nullptr means there is nothing to apply.
struct RowScale {
    const float* ssq;       // [rows, parts]
    int parts;
    float inv_dim, eps;
};
// every thread on its own (rows that differ from thread to thread)
__device__ __forceinline__ float row_scale(const RowScale& rs, long long row) {
    if (rs.ssq == nullptr) return 1.f;
    float v = 0.f;
    for (int q = 0; q < rs.parts; ++q) v += __ldcg(rs.ssq + row * rs.parts + q);
    return rsqrtf(v * rs.inv_dim + rs.eps);
}
// all 32 lanes of a warp for the same row: the parts are read side by side
__device__ __forceinline__ float warp_row_scale(const RowScale& rs, long long row) {
    if (rs.ssq == nullptr) return 1.f;
    float v = 0.f;
    for (int q = threadIdx.x & 31; q < rs.parts; q += 32) v += __ldcg(rs.ssq + row * rs.parts + q);
    return rsqrtf(warp_sum(v) * rs.inv_dim + rs.eps);
}

// ---- programmatic dependent launch: a kernel may start while its predecessor in the stream is
// still running, do what does not depend on it (set-up, prefetching weights), and must call
// grid_dependency_wait() before it touches anything the predecessor writes or reads.  Every
// kernel launched through tl_launch calls it, so completion of a kernel still implies completion
// of everything before it.  grid_launch_dependents() lets the successor be scheduled early.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

static inline bool pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* off = getenv("TORCHLLMS_B200_NO_PDL");
        on = (off != nullptr && off[0] == '1') ? 0 : 1;
    }
    return on == 1;
}

// Launch with the programmatic-stream-serialization attribute (works in stream capture too).
template <typename... KArgs, typename... Args>
static inline cudaError_t tl_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
