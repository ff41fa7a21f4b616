// Choosing the next token from float32 logits: greedy, temperature, optional top-k.
//
// Reference: torchllms/inference/utils.py:18-48.  Greedy is argmax (the first maximal index wins
// a tie).  With a temperature the reference divides the logits by max(T, 1e-5), optionally sets
// everything below the k-th largest logit to -inf, takes the softmax and returns
// argmax(probs / q) with q ~ Exp(1).  That argmax equals argmax(logit / T - log q), which is what
// this kernel evaluates without ever forming the probabilities.
//
// The noise is a pure function of a 64-bit key per row and the vocabulary index, so a request's
// samples depend neither on the batch it sits in nor on how its prompt was cut; the host derives
// the row key from (seed, request, index of the generated token).
//   bits(i) = mix64(key + (i + 1) * 0x9E3779B97F4A7C15),  u = ((bits >> 41) + 0.5) * 2^-23,
//   -log q = -log(-log u).
//
// One CTA per row.  top-k first finds the k-th largest logit with a 4-pass radix select over
// the order-preserving integer image of the floats.
#include "common.cuh"
#include <math.h>

namespace {

constexpr int NT = 1024;

__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z ^= z >> 30; z *= 0xBF58476D1CE4E5B9ull;
    z ^= z >> 27; z *= 0x94D049BB133111EBull;
    z ^= z >> 31;
    return z;
}

__device__ __forceinline__ float neg_log_exp1(unsigned long long key, unsigned i) {
    const unsigned long long bits = mix64(key + (unsigned long long)(i + 1u) * 0x9E3779B97F4A7C15ull);
    const float u = ((float)(bits >> 41) + 0.5f) * 1.1920928955078125e-07f;  // 2^-23
    return -logf(-logf(u));
}

__device__ __forceinline__ unsigned ordered_bits(float x) {
    const unsigned b = __float_as_uint(x);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ float from_ordered_bits(unsigned k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// k-th largest value of row[0..V) (k >= 1), every thread returns it
__device__ float kth_largest(const float* __restrict__ row, int V, int k, unsigned* hist, unsigned* shared) {
    unsigned prefix = 0, mask = 0;
    int remaining = k;
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
        __syncthreads();
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const unsigned key = ordered_bits(row[i]);
            if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int left = remaining;
            int bucket = 255;
            for (; bucket > 0; --bucket) {
                const int n = (int)hist[bucket];
                if (n >= left) break;
                left -= n;
            }
            shared[0] = (unsigned)bucket;
            shared[1] = (unsigned)left;
        }
        __syncthreads();
        prefix |= shared[0] << shift;
        mask |= 255u << shift;
        remaining = (int)shared[1];
        __syncthreads();
    }
    return from_ordered_bits(prefix);
}

__global__ void __launch_bounds__(NT) sample_kernel(const float* __restrict__ logits, long long row_stride, int V,
                                                    const float* __restrict__ temperature,
                                                    const int* __restrict__ top_k,
                                                    const unsigned long long* __restrict__ row_keys,
                                                    int* __restrict__ out) {
    __shared__ unsigned hist[256];
    __shared__ unsigned pick[2];
    __shared__ float best_v[32];
    __shared__ int best_i[32];
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * row_stride;
    const float temp = temperature ? temperature[r] : 0.f;
    const bool greedy = !(temp > 0.f);
    float pivot = -INFINITY;
    if (!greedy && top_k) {
        const int k = top_k[r];
        if (k > 0 && k < V) pivot = kth_largest(row, V, k, hist, pick);
    }
    const float t = fmaxf(temp, 1e-5f);
    const unsigned long long key = greedy ? 0ull : row_keys[r];
    float bv = -INFINITY;
    int bi = V;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float x = row[i];
        float s;
        if (greedy) s = x;
        else if (x < pivot) continue;
        else s = x / t + neg_log_exp1(key, (unsigned)i);
        if (s > bv || (s == bv && i < bi)) { bv = s; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        bv = lane < (blockDim.x >> 5) ? best_v[lane] : -INFINITY;
        bi = lane < (blockDim.x >> 5) ? best_i[lane] : V;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) out[r] = bi < V ? bi : 0;
    }
}

// ---- two-stage form for rows without top-k: many CTAs per row, then one warp per row
constexpr int CHUNK = 4096;      // vocabulary entries per stage-one CTA
constexpr int NT1 = 256;

__device__ __forceinline__ void better(float& bv, int& bi, float ov, int oi) {
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
}

__global__ void __launch_bounds__(NT1) sample_stage1_kernel(const float* __restrict__ logits, long long row_stride, int V,
                                                            const float* __restrict__ temperature,
                                                            const unsigned long long* __restrict__ row_keys,
                                                            float* __restrict__ part_v, int* __restrict__ part_i) {
    __shared__ float best_v[NT1 / 32];
    __shared__ int best_i[NT1 / 32];
    grid_launch_dependents();
    grid_dependency_wait();
    const int r = blockIdx.y, chunk = blockIdx.x;
    const float* row = logits + (size_t)r * row_stride;
    const float temp = temperature ? temperature[r] : 0.f;
    const bool greedy = !(temp > 0.f);
    const float t = fmaxf(temp, 1e-5f);
    const unsigned long long key = greedy ? 0ull : row_keys[r];
    const int hi = min(V, (chunk + 1) * CHUNK);
    float bv = -INFINITY;
    int bi = V;
    for (int i = chunk * CHUNK + threadIdx.x; i < hi; i += NT1) {
        const float x = row[i];
        const float s = greedy ? x : x / t + neg_log_exp1(key, (unsigned)i);
        better(bv, bi, s, i);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        better(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        bv = lane < NT1 / 32 ? best_v[lane] : -INFINITY;
        bi = lane < NT1 / 32 ? best_i[lane] : V;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
            better(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
        if (lane == 0) {
            part_v[(size_t)r * gridDim.x + chunk] = bv;
            part_i[(size_t)r * gridDim.x + chunk] = bi;
        }
    }
}

__global__ void sample_stage2_kernel(const float* __restrict__ part_v, const int* __restrict__ part_i,
                                     int n_chunks, int V, int* __restrict__ out) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int r = blockIdx.x, lane = threadIdx.x;
    float bv = -INFINITY;
    int bi = V;
    for (int c = lane; c < n_chunks; c += 32) better(bv, bi, part_v[(size_t)r * n_chunks + c], part_i[(size_t)r * n_chunks + c]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        better(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
    if (lane == 0) out[r] = bi < V ? bi : 0;
}

}  // namespace

// How many 4-byte words of scratch tl_sample_wide needs for this many rows of this vocabulary.
extern "C" long long tl_sample_wide_scratch(int n_rows, int vocab) {
    const long long chunks = (vocab + CHUNK - 1) / CHUNK;
    return 2 * chunks * n_rows;
}

// Rows without top-k, spread over many CTAs: same result as tl_sample.  scratch: see above.
extern "C" int tl_sample_wide(const float* logits, long long row_stride, int n_rows, int vocab,
                              const float* temperature, const unsigned long long* row_keys,
                              void* scratch, int* out, void* stream) {
    if (n_rows <= 0) return TL_OK;
    if (vocab <= 0 || row_stride < vocab || n_rows > 65535 || scratch == nullptr) return TL_BAD_SIZE;
    if (temperature != nullptr && row_keys == nullptr) return TL_BAD_SIZE;
    const int chunks = (vocab + CHUNK - 1) / CHUNK;
    float* part_v = (float*)scratch;
    int* part_i = (int*)scratch + (size_t)chunks * n_rows;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e = tl_launch(sample_stage1_kernel, dim3(chunks, n_rows), dim3(NT1), 0, s, logits, row_stride, vocab,
                              temperature, row_keys, part_v, part_i);
    if (e != cudaSuccess) return (int)e;
    return (int)tl_launch(sample_stage2_kernel, dim3(n_rows), dim3(32), 0, s, (const float*)part_v, (const int*)part_i,
                          chunks, vocab, out);
}

// temperature, top_k and row_keys may be null: then every row is greedy / unfiltered.  A row
// whose temperature is not positive is greedy.  All arrays live on the device.
extern "C" int tl_sample(const float* logits, long long row_stride, int n_rows, int vocab,
                         const float* temperature, const int* top_k,
                         const unsigned long long* row_keys, int* out, void* stream) {
    if (n_rows <= 0) return TL_OK;
    if (vocab <= 0 || row_stride < vocab) return TL_BAD_SIZE;
    if (temperature != nullptr && row_keys == nullptr) return TL_BAD_SIZE;
    sample_kernel<<<n_rows, NT, 0, (cudaStream_t)stream>>>(logits, row_stride, vocab, temperature, top_k, row_keys, out);
    TL_LAUNCH_CHECK();
    return TL_OK;
}
