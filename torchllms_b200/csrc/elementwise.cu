// Embedding gather, residual sum + RMS norm, and the SwiGLU gate.
//
// embed:    h[t, :] = float(table[ids[t], :])                 (the residual stream is float32)
// rmsnorm:  x = h[row] (+ delta[row]);  y = x * rsqrt(mean(x^2) + eps) * w   -- all in float32,
//           rounded once to the output dtype; with `write_back` the sum x replaces h[row].
//           The reference normalises in float32 too (torchllms/models/networks.py:195-200).
//           Deferred form: y = x * w without the rsqrt, and ssq_out[row] = sum(x^2): the kernels that
//           consume the product of y with a weight matrix apply rsqrt(ssq / dim + eps) to the product's
//           rows instead (a matrix product is linear in its input, so the scale commutes with it).
// swiglu:   out[t, f] = silu(in[t, f]) * in[t, F + f],  silu(g) = g / (1 + exp(-g)), in float32
//           (torchllms/models/networks.py:604-605).  With a row scale (see above) gate and up are
//           multiplied by it first.
#include "common.cuh"

template <typename T>
__global__ void embed_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                             float* __restrict__ out, int dim, int vocab) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int t = blockIdx.x;
    int id = ids[t];
    (void)TL_CHECK(id >= 0 && id < vocab, TL_DBG_TOKEN_ID);
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);  // the host rejects such ids; stay in bounds anyway
    const T* src = table + (size_t)id * dim;
    float* dst = out + (size_t)t * dim;
    for (int d = threadIdx.x; d < dim; d += blockDim.x) dst[d] = to_float(src[d]);
}

// bfloat16 table, dim a multiple of 8, 16-byte aligned rows: eight elements per thread and turn
__global__ void embed_bf16x8_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                    float* __restrict__ out, int dim, int vocab) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int t = blockIdx.x;
    int id = ids[t];
    (void)TL_CHECK(id >= 0 && id < vocab, TL_DBG_TOKEN_ID);
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    const __nv_bfloat16* src = table + (size_t)id * dim;
    float* dst = out + (size_t)t * dim;
    for (int d = threadIdx.x * 8; d < dim; d += blockDim.x * 8) {
        const uint4 raw = *reinterpret_cast<const uint4*>(src + d);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
        const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
        const float2 c = __bfloat1622float2(h[2]), e = __bfloat1622float2(h[3]);
        *reinterpret_cast<float4*>(dst + d) = make_float4(a.x, a.y, b.x, b.y);
        *reinterpret_cast<float4*>(dst + d + 4) = make_float4(c.x, c.y, e.x, e.y);
    }
}

// four contiguous elements as floats
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<unsigned*>(&a);
    raw.y = *reinterpret_cast<unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
}

// VEC = 4: dim is a multiple of 4 and every row starts 16-byte aligned; VEC = 1: anything.
// delta holds `splits` planes `plane` elements apart (partial sums of a split-K product); they
// are added in order, then to the stream.
template <typename TD, typename TO, int VEC>
__global__ void rmsnorm_kernel(float* __restrict__ h, const TD* __restrict__ delta, int splits, long long plane,
                               const float* __restrict__ weight, TO* __restrict__ out,
                               const int* __restrict__ rows, int dim, float eps, int write_back,
                               float* __restrict__ ssq_out) {
    extern __shared__ __align__(16) float row_buf[];  // the summed row, kept for the second pass
    __shared__ float warp_part[32];
    grid_launch_dependents();
    // the row index and the norm's weight do not come from the kernel before this one
    const int o = blockIdx.x;
    int r = rows ? rows[o] : o;
    if (!tl_check_row(r)) r = 0;                     // (debug builds: a bad row is reported, row 0 read in its place)
    float4 w_first = make_float4(0.f, 0.f, 0.f, 0.f);
    if (VEC == 4 && threadIdx.x * 4 < dim) w_first = load4(weight + threadIdx.x * 4);
    grid_dependency_wait();
    float* hr = h + (size_t)r * dim;
    const TD* dr = delta ? delta + (size_t)r * dim : nullptr;
    float ss = 0.f;
    if (VEC == 4 && ssq_out != nullptr) {
        // deferred form: what is written does not depend on the row's sum, so one walk does it all and
        // nothing waits for the sum (no staging in shared memory, no second pass)
        TO* orow = out + (size_t)o * dim;
        for (int d = threadIdx.x * 4; d < dim; d += blockDim.x * 4) {
            float4 x = load4(hr + d);
            if (dr) {
                float4 y = load4(dr + d);
                for (int sp = 1; sp < splits; ++sp) {
                    const float4 z = load4(dr + sp * plane + d);
                    y.x += z.x; y.y += z.y; y.z += z.z; y.w += z.w;
                }
                x.x += y.x; x.y += y.y; x.z += y.z; x.w += y.w;
            }
            const float4 w = d == (int)threadIdx.x * 4 ? w_first : load4(weight + d);
            if (write_back) store4(hr + d, x);
            store4(orow + d, make_float4(x.x * w.x, x.y * w.y, x.z * w.z, x.w * w.w));
            ss += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
        }
        ss = warp_sum(ss);
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
        if (lane == 0) warp_part[warp] = ss;
        __syncthreads();
        if (warp == 0) {
            float v = lane < n_warps ? warp_part[lane] : 0.f;
            v = warp_sum(v);
            if (lane == 0) ssq_out[o] = v;
        }
        return;
    }
    if (VEC == 4) {
        for (int d = threadIdx.x * 4; d < dim; d += blockDim.x * 4) {
            float4 x = load4(hr + d);
            if (dr) {
                float4 y = load4(dr + d);
                for (int sp = 1; sp < splits; ++sp) {
                    const float4 z = load4(dr + sp * plane + d);
                    y.x += z.x; y.y += z.y; y.z += z.z; y.w += z.w;
                }
                x.x += y.x; x.y += y.y; x.z += y.z; x.w += y.w;
            }
            store4(row_buf + d, x);
            ss += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
        }
    } else {
        for (int d = threadIdx.x; d < dim; d += blockDim.x) {
            float x = hr[d];
            if (dr) {
                float y = to_float(dr[d]);
                for (int sp = 1; sp < splits; ++sp) y += to_float(dr[sp * plane + d]);
                x += y;
            }
            row_buf[d] = x;
            ss += x * x;
        }
    }
    ss = warp_sum(ss);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    if (lane == 0) warp_part[warp] = ss;
    __syncthreads();
    if (warp == 0) {
        float v = lane < n_warps ? warp_part[lane] : 0.f;
        v = warp_sum(v);
        if (lane == 0) warp_part[0] = v;
    }
    __syncthreads();
    // deferred form: the rows leave weighted but not normalised, with their sum of squares beside them
    const float rstd = ssq_out ? 1.f : rsqrtf(warp_part[0] / (float)dim + eps);
    if (ssq_out && threadIdx.x == 0) ssq_out[o] = warp_part[0];
    TO* orow = out + (size_t)o * dim;
    if (VEC == 4) {
        for (int d = threadIdx.x * 4; d < dim; d += blockDim.x * 4) {   // each thread re-reads what it wrote
            const float4 x = load4(row_buf + d);
            const float4 w = d == (int)threadIdx.x * 4 ? w_first : load4(weight + d);
            if (write_back) store4(hr + d, x);
            store4(orow + d, make_float4(x.x * rstd * w.x, x.y * rstd * w.y, x.z * rstd * w.z, x.w * rstd * w.w));
        }
    } else {
        for (int d = threadIdx.x; d < dim; d += blockDim.x) {
            const float x = row_buf[d];
            if (write_back) hr[d] = x;
            orow[d] = from_float<TO>(x * rstd * weight[d]);
        }
    }
}

// `in` holds `splits` planes of [tokens, 2 * hidden] (partial sums of a split-K product), summed first.
// VEC = 4: hidden is a multiple of 4 and rows are 16-byte aligned: four gates and four ups per thread.
template <typename TI, typename T, int VEC>
__global__ void swiglu_kernel(const TI* __restrict__ in, int splits, long long plane, T* __restrict__ out,
                              int hidden, int n_tokens, const RowScale rs) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int per_row = hidden / VEC;
    for (int t = blockIdx.y; t < n_tokens; t += gridDim.y) {
        const TI* row = in + (size_t)t * 2 * hidden;
        T* orow = out + (size_t)t * hidden;
        const float sc = warp_row_scale(rs, t);        // (t is the same for the whole CTA)
        for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < per_row; c += gridDim.x * blockDim.x) {
            const int f = c * VEC;
            if (VEC == 4) {
                float4 g = load4(row + f), u = load4(row + hidden + f);
                for (int sp = 1; sp < splits; ++sp) {
                    const float4 g2 = load4(row + sp * plane + f), u2 = load4(row + sp * plane + hidden + f);
                    g.x += g2.x; g.y += g2.y; g.z += g2.z; g.w += g2.w;
                    u.x += u2.x; u.y += u2.y; u.z += u2.z; u.w += u2.w;
                }
                g.x *= sc; g.y *= sc; g.z *= sc; g.w *= sc;
                u.x *= sc; u.y *= sc; u.z *= sc; u.w *= sc;
                store4(orow + f, make_float4(g.x / (1.f + expf(-g.x)) * u.x, g.y / (1.f + expf(-g.y)) * u.y,
                                             g.z / (1.f + expf(-g.z)) * u.z, g.w / (1.f + expf(-g.w)) * u.w));
            } else {
                float g = 0.f, u = 0.f;
                for (int sp = 0; sp < splits; ++sp) {
                    g += to_float(row[sp * plane + f]);
                    u += to_float(row[sp * plane + hidden + f]);
                }
                g *= sc;
                u *= sc;
                orow[f] = from_float<T>(g / (1.f + expf(-g)) * u);
            }
        }
    }
}

extern "C" int tl_embed(const int* ids, const void* table, int table_dtype, float* out,
                        int n_tokens, int dim, int vocab, void* stream) {
    if (n_tokens <= 0) return TL_OK;
    if (dim <= 0 || vocab <= 0) return TL_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = dim >= 1024 ? 256 : 128;
    cudaError_t e;
    if (table_dtype == TL_F32)
        e = tl_launch(embed_kernel<float>, dim3(n_tokens), dim3(threads), 0, s, ids, (const float*)table, out, dim, vocab);
    else if (table_dtype == TL_BF16 && dim % 8 == 0 && aligned16(table) && aligned16(out))
        e = tl_launch(embed_bf16x8_kernel, dim3(n_tokens), dim3(dim / 8 >= 256 ? 256 : (dim / 8 + 31) / 32 * 32), 0, s, ids,
                      (const __nv_bfloat16*)table, out, dim, vocab);
    else if (table_dtype == TL_BF16)
        e = tl_launch(embed_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, s, ids, (const __nv_bfloat16*)table, out, dim, vocab);
    else
        return TL_BAD_DTYPE;
    return (int)e;
}

template <typename TD, typename TO>
static int launch_rmsnorm(float* h, const void* delta, int splits, long long plane, const float* w, void* out,
                          const int* rows, int n_out, int dim, float eps, int write_back, float* ssq_out, cudaStream_t s) {
    const bool vec = dim % 4 == 0 && plane % 4 == 0 && aligned16(h) && aligned16(w) && aligned16(out) &&
                     (delta == nullptr || aligned16(delta));
    const size_t smem = (vec && ssq_out != nullptr) ? 0 : (size_t)dim * sizeof(float);    // (the deferred form stages nothing)
    if (smem > 200 * 1024) return TL_TOO_LARGE;
    auto kern = vec ? rmsnorm_kernel<TD, TO, 4> : rmsnorm_kernel<TD, TO, 1>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    const int per_thread = vec ? 4 : 1;
    int threads = (dim / per_thread + 31) / 32 * 32;
    threads = threads < 64 ? 64 : (threads > 1024 ? 1024 : threads);
    if (n_out >= 512 && threads > 256) threads = 256;   // many rows: smaller CTAs, more of them resident
    return (int)tl_launch(kern, dim3(n_out), dim3(threads), smem, s, h, (const TD*)delta, splits, plane, w, (TO*)out, rows,
                          dim, eps, write_back, ssq_out);
}

// delta may be null (then nothing is added); it may hold `delta_splits` planes of [rows of h, dim],
// `delta_plane` elements apart, which are summed.  rows may be null (then row o is row o of h).
// ssq_out may be null; else [n_out] floats receive the rows' sums of squares and the rows are
// written weighted but not normalised (the deferred form).
extern "C" int tl_rmsnorm(float* h, const void* delta, int delta_dtype, int delta_splits, long long delta_plane,
                          const float* weight, void* out, int out_dtype, const int* rows, int n_out, int dim,
                          float eps, int write_back, float* ssq_out, void* stream) {
    if (n_out <= 0) return TL_OK;
    if (dim <= 0 || delta_splits < 1) return TL_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    if (delta_dtype == TL_F32 && out_dtype == TL_F32)
        return launch_rmsnorm<float, float>(h, delta, delta_splits, delta_plane, weight, out, rows, n_out, dim, eps, write_back, ssq_out, s);
    if (delta_dtype == TL_BF16 && out_dtype == TL_BF16)
        return launch_rmsnorm<__nv_bfloat16, __nv_bfloat16>(h, delta, delta_splits, delta_plane, weight, out, rows, n_out, dim, eps, write_back, ssq_out, s);
    if (delta_dtype == TL_F32 && out_dtype == TL_BF16)
        return launch_rmsnorm<float, __nv_bfloat16>(h, delta, delta_splits, delta_plane, weight, out, rows, n_out, dim, eps, write_back, ssq_out, s);
    if (delta_dtype == TL_BF16 && out_dtype == TL_F32)
        return launch_rmsnorm<__nv_bfloat16, float>(h, delta, delta_splits, delta_plane, weight, out, rows, n_out, dim, eps, write_back, ssq_out, s);
    return TL_BAD_DTYPE;
}

// silu(g) * u with the fast exponential and division: their error (a few units in the last place of a
// float) disappears when the result is rounded to bfloat16, and the exact forms cost more
// instructions than the kernel has time for at full memory bandwidth
__device__ __forceinline__ float silu_mul_fast(float g, float u) { return __fdividef(g, 1.f + __expf(-g)) * u; }

// bfloat16 in and out, hidden a multiple of 8, one plane: eight gates and eight ups per thread (16-byte accesses)
__global__ void swiglu_bf16x8_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out,
                                     int hidden, long long n_chunks, const RowScale rs) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int per_row = hidden >> 3;
    for (long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x; c < n_chunks; c += (long long)gridDim.x * blockDim.x) {
        const long long t = c / per_row;
        const int f = (int)(c - t * per_row) << 3;
        const float sc = row_scale(rs, t);
        const uint4 graw = *reinterpret_cast<const uint4*>(in + t * 2 * hidden + f);
        const uint4 uraw = *reinterpret_cast<const uint4*>(in + t * 2 * hidden + hidden + f);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&graw);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uraw);
        uint4 oraw;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&oraw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 g = __bfloat1622float2(g2[i]), u = __bfloat1622float2(u2[i]);
            o2[i] = __floats2bfloat162_rn(silu_mul_fast(g.x * sc, u.x * sc), silu_mul_fast(g.y * sc, u.y * sc));
        }
        *reinterpret_cast<uint4*>(out + t * hidden + f) = oraw;
    }
}

template <typename TI, typename T>
static int launch_swiglu(const void* in, int splits, void* out, int n_tokens, int hidden, const RowScale& rs, cudaStream_t s) {
    const long long plane = 2LL * n_tokens * hidden;
    const bool vec = hidden % 4 == 0 && aligned16(in) && aligned16(out) && sizeof(T) * hidden % 8 == 0;
    const int per_row = vec ? hidden / 4 : hidden;
    const int threads = 256;
    int bx = (per_row + threads - 1) / threads;
    if (bx > 64) bx = 64;
    int by = n_tokens < 4096 ? n_tokens : 4096;
    const dim3 grid(bx, by), block(threads);
    if (vec)
        return (int)tl_launch(swiglu_kernel<TI, T, 4>, grid, block, 0, s, (const TI*)in, splits, plane, (T*)out, hidden, n_tokens, rs);
    return (int)tl_launch(swiglu_kernel<TI, T, 1>, grid, block, 0, s, (const TI*)in, splits, plane, (T*)out, hidden, n_tokens, rs);
}

// in: [splits, n_tokens, 2 * hidden] of in_dtype (splits > 1 only for float32 partial sums); out: [n_tokens, hidden].
// in_ssq may be null; else [n_tokens, in_parts] floats: gate and up of a token are multiplied by
// rsqrt(sum_p in_ssq[token, p] * in_inv_dim + in_eps) before the activation.
extern "C" int tl_swiglu(const void* in, int in_dtype, int splits, void* out, int dtype, int n_tokens, int hidden,
                         const float* in_ssq, int in_parts, float in_inv_dim, float in_eps, void* stream) {
    if ((long long)n_tokens * hidden <= 0) return TL_OK;
    if (splits < 1 || (in_ssq != nullptr && in_parts < 1)) return TL_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const RowScale rs = {in_ssq, in_parts, in_inv_dim, in_eps};
    if (in_dtype == TL_F32 && dtype == TL_F32) return launch_swiglu<float, float>(in, splits, out, n_tokens, hidden, rs, s);
    if (in_dtype == TL_BF16 && dtype == TL_BF16) {
        if (splits == 1 && hidden % 8 == 0 && aligned16(in) && aligned16(out)) {
            const long long n_chunks = (long long)n_tokens * (hidden / 8);
            long long blocks = (n_chunks + 255) / 256;
            if (blocks > 148 * 16) blocks = 148 * 16;
            return (int)tl_launch(swiglu_bf16x8_kernel, dim3((unsigned)blocks), dim3(256), 0, s, (const __nv_bfloat16*)in,
                                  (__nv_bfloat16*)out, hidden, n_chunks, rs);
        }
        return launch_swiglu<__nv_bfloat16, __nv_bfloat16>(in, splits, out, n_tokens, hidden, rs, s);
    }
    if (in_dtype == TL_F32 && dtype == TL_BF16) return launch_swiglu<float, __nv_bfloat16>(in, splits, out, n_tokens, hidden, rs, s);
    return TL_BAD_DTYPE;
}
