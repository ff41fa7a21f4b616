// Causal grouped-query attention over paged keys and values, for any mix of prompt portions
// and single decoded tokens (the general kernel: float32 and bfloat16, any head_dim that is a
// multiple of 16 up to 256, any number of heads and groups, optional sliding window).
//
// What it computes, per query token at absolute position p of request b and query head h
// (kv head h / (H / KV)):   o = softmax_k( q . k_k * scale ) v_k   over keys k <= p
// (and k > p - window when a window is set), as torchllms/models/networks.py:355-397 does for
// whole sequences; the query's position is kv_len[b] - q_len[b] + its index in the portion, the
// bottom-right aligned mask the reference relies on for a suffix after a cached prefix
// (torchllms/models/networks.py:435-445).  Scores, the running maximum and sum, and the output
// accumulator are float32.
//
// Work split: one CTA takes up to 16 rows, a row being (token, query head of one kv group), so
// the heads of a group share every key and value it loads.  Keys are walked in tiles of 32
// through shared memory with the streaming-softmax update.  When the batch offers too few CTAs
// (decoding a few long requests), the key range is cut into splits whose partial (max, sum,
// accumulator) go to a float32 workspace that tl_attention_merge combines.
#include "common.cuh"
#include <math.h>

namespace {

constexpr int R = 16;    // rows per CTA
constexpr int TK = 32;   // keys per tile
constexpr int NT = 128;  // threads per CTA: 8 threads per row
constexpr int TARGET_CTAS = 296;
constexpr int MIN_SPLIT = 128;

struct AttnParams {
    const void* q;
    const void* k_pages;
    const void* v_pages;
    void* out;
    const int* block_table;
    const int* q_start;
    const int* kv_len;
    float* part_o;   // [T * H, n_splits, head_dim]
    float* part_ml;  // [T * H, n_splits, 2]
    int table_stride;
    int n_heads, n_kv_heads, head_dim, page_size;
    int group, gchunk, n_gchunks, tokens_per_tile;
    int window;  // 0: none
    int n_splits;
    float scale;
};

template <typename T, int HD_MAX>
__global__ void __launch_bounds__(NT) paged_attention_kernel(const AttnParams p) {
    extern __shared__ float smem[];
    const int hd = p.head_dim;
    const int qpitch = hd + 1;
    float* Qs = smem;                 // [R][hd + 1]
    float* Ks = Qs + R * qpitch;      // [TK][hd + 1]
    float* Vs = Ks + TK * qpitch;     // [TK][hd]
    float* Ss = Vs + TK * hd;         // [R][TK + 1]

    const int b = blockIdx.z;
    const int qs = p.q_start[b];
    const int ql = p.q_start[b + 1] - qs;
    const int kl = p.kv_len[b];
    const int tile = blockIdx.x / p.n_splits;
    const int split = blockIdx.x - tile * p.n_splits;
    const int tok0 = tile * p.tokens_per_tile;
    if (tok0 >= ql) return;
    const int ntok = min(p.tokens_per_tile, ql - tok0);
    const int kvh = blockIdx.y / p.n_gchunks;
    const int g0 = (blockIdx.y - kvh * p.n_gchunks) * p.gchunk;
    const int ng = min(p.gchunk, p.group - g0);
    const int n_rows = ntok * ng;

    const int tid = threadIdx.x;
    const int rr = tid >> 3;  // row of this thread
    const int c = tid & 7;

    const T* q = reinterpret_cast<const T*>(p.q);
    const T* k_pages = reinterpret_cast<const T*>(p.k_pages);
    const T* v_pages = reinterpret_cast<const T*>(p.v_pages);

    // ---- queries of the tile, as float
    for (int i = tid; i < R * hd; i += NT) {
        const int r = i / hd, d = i - r * hd;
        float v = 0.f;
        if (r < n_rows) {
            const int tok = qs + tok0 + r / ng;
            const int head = kvh * p.group + g0 + r % ng;
            v = to_float(q[((size_t)tok * p.n_heads + head) * hd + d]);
        }
        Qs[r * qpitch + d] = v;
    }

    const int qpos_min = kl - ql + tok0;
    const int qpos_max = qpos_min + ntok - 1;
    const int my_qpos = rr < n_rows ? qpos_min + rr / ng : -1;
    int k_lo = p.window > 0 ? max(0, qpos_min - p.window + 1) : 0;
    int k_hi = qpos_max + 1;
    if (p.n_splits > 1) {
        // every request cuts its own visible keys evenly, in whole tiles, so the launch shape
        // depends on the batch only and not on how long the requests have grown
        const int len = max(k_hi - k_lo, 0);
        const int chunk = ((len + p.n_splits - 1) / p.n_splits + TK - 1) / TK * TK;
        const int lo = k_lo + split * chunk;
        k_hi = min(k_hi, lo + chunk);
        k_lo = lo;
    }

    float m = -INFINITY, l = 0.f;
    float acc[HD_MAX / 8];
#pragma unroll
    for (int j = 0; j < HD_MAX / 8; ++j) acc[j] = 0.f;

    constexpr int VEC = Vec16<T>::N;
    const int vec_per_row = hd / VEC;
    const int* table = p.block_table + (size_t)b * p.table_stride;

    for (int k0 = k_lo; k0 < k_hi; k0 += TK) {
        __syncthreads();  // the previous tile's Ks / Vs / Ss are no longer read (and Qs is written)
        for (int i = tid; i < TK * vec_per_row; i += NT) {
            const int j = i / vec_per_row, v = i - j * vec_per_row;
            const int kpos = k0 + j;
            float* kd = Ks + j * qpitch + v * VEC;
            float* vd = Vs + j * hd + v * VEC;
            if (kpos < k_hi && tl_check_page(table[kpos / p.page_size])) {     // (debug builds: a bad page reads as zeros)
                const int page = table[kpos / p.page_size];
                const size_t off = (((size_t)page * p.n_kv_heads + kvh) * p.page_size + kpos % p.page_size) * hd + v * VEC;
                Vec16<T> kv, vv;
                kv.load(k_pages + off);
                vv.load(v_pages + off);
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
                    kd[e] = kv.get(e);
                    vd[e] = vv.get(e);
                }
            } else {
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
                    kd[e] = 0.f;
                    vd[e] = 0.f;
                }
            }
        }
        __syncthreads();

        // ---- scores of row rr against keys c, c + 8, c + 16, c + 24
        float s[4] = {0.f, 0.f, 0.f, 0.f};
        const float* qrow = Qs + rr * qpitch;
        for (int d = 0; d < hd; ++d) {
            const float qv = qrow[d];
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) s[jj] = fmaf(qv, Ks[(c + 8 * jj) * qpitch + d], s[jj]);
        }
        float tile_max = -INFINITY;
        bool ok[4];
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            const int kpos = k0 + c + 8 * jj;
            ok[jj] = kpos < k_hi && kpos <= my_qpos && (p.window <= 0 || kpos > my_qpos - p.window);
            s[jj] *= p.scale;
            if (ok[jj]) tile_max = fmaxf(tile_max, s[jj]);
        }
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, o));
        const float m_new = fmaxf(m, tile_max);
        float alpha = 1.f, row_sum = 0.f;
        float pr[4] = {0.f, 0.f, 0.f, 0.f};
        if (m_new != -INFINITY) {
            alpha = expf(m - m_new);  // m = -inf gives 0
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
                pr[jj] = ok[jj] ? expf(s[jj] - m_new) : 0.f;
                row_sum += pr[jj];
            }
        }
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) row_sum += __shfl_xor_sync(0xffffffffu, row_sum, o);
        l = l * alpha + row_sum;
        m = m_new;
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) Ss[rr * (TK + 1) + c + 8 * jj] = pr[jj];
#pragma unroll
        for (int j = 0; j < HD_MAX / 8; ++j) acc[j] *= alpha;
        __syncthreads();

        // ---- accumulate probabilities times values; this thread owns lanes c, c + 8, ...
        const float* prow = Ss + rr * (TK + 1);
        for (int j = 0; j < TK; ++j) {
            const float pj = prow[j];
            const float* vrow = Vs + j * hd + c;
#pragma unroll
            for (int jd = 0; jd < HD_MAX / 8; ++jd)
                if (jd * 8 < hd) acc[jd] = fmaf(pj, vrow[jd * 8], acc[jd]);
        }
    }

    if (rr >= n_rows) return;
    const int tok = qs + tok0 + rr / ng;
    const int head = kvh * p.group + g0 + rr % ng;
    const size_t row = (size_t)tok * p.n_heads + head;
    if (p.n_splits == 1) {
        T* o = reinterpret_cast<T*>(p.out) + row * hd;
        const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
        for (int jd = 0; jd < HD_MAX / 8; ++jd)
            if (jd * 8 < hd) o[c + jd * 8] = from_float<T>(acc[jd] * inv);
    } else {
        float* o = p.part_o + (row * p.n_splits + split) * hd;
#pragma unroll
        for (int jd = 0; jd < HD_MAX / 8; ++jd)
            if (jd * 8 < hd) o[c + jd * 8] = acc[jd];
        if (c == 0) {
            float* ml = p.part_ml + (row * p.n_splits + split) * 2;
            ml[0] = m;
            ml[1] = l;
        }
    }
}

// out[row, d] = sum_i e^{m_i - M} o_i[d] / sum_i e^{m_i - M} l_i,  M = max_i m_i
template <typename T>
__global__ void attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                       T* __restrict__ out, int n_splits, int head_dim) {
    const size_t row = blockIdx.x;
    const float* ml = part_ml + row * n_splits * 2;
    float M = -INFINITY;
    for (int i = 0; i < n_splits; ++i) M = fmaxf(M, ml[2 * i]);
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
        float num = 0.f, den = 0.f;
        for (int i = 0; i < n_splits; ++i) {
            const float mi = ml[2 * i];
            if (mi == -INFINITY) continue;
            const float w = expf(mi - M);
            num = fmaf(w, part_o[(row * n_splits + i) * head_dim + d], num);
            den = fmaf(w, ml[2 * i + 1], den);
        }
        out[row * head_dim + d] = from_float<T>(den > 0.f ? num / den : 0.f);
    }
}

struct Plan {
    int gchunk, n_gchunks, tokens_per_tile, n_q_tiles, n_splits;
};

Plan make_plan(int n_seqs, int n_heads, int n_kv_heads, int max_q_len, int max_kv_len, int allow_split) {
    Plan pl;
    const int group = n_heads / n_kv_heads;
    pl.gchunk = group < R ? group : R;
    pl.n_gchunks = (group + pl.gchunk - 1) / pl.gchunk;
    pl.tokens_per_tile = R / pl.gchunk;
    pl.n_q_tiles = (max_q_len + pl.tokens_per_tile - 1) / pl.tokens_per_tile;
    pl.n_splits = 1;
    const long long base = (long long)pl.n_q_tiles * n_kv_heads * pl.n_gchunks * n_seqs;
    if (allow_split && base < TARGET_CTAS && max_kv_len >= 2 * MIN_SPLIT) {
        const int want = (int)((TARGET_CTAS + base - 1) / base);
        const int most = max_kv_len / MIN_SPLIT;
        pl.n_splits = want < most ? want : most;
        if (pl.n_splits < 1) pl.n_splits = 1;
    }
    return pl;
}

size_t smem_bytes(int hd) { return (size_t)(R * (hd + 1) + TK * (hd + 1) + TK * hd + R * (TK + 1)) * sizeof(float); }

template <typename T, int HD_MAX>
int launch(const AttnParams& p, dim3 grid, cudaStream_t s) {
    const size_t smem = smem_bytes(p.head_dim);
    auto kern = paged_attention_kernel<T, HD_MAX>;
    static int raised = 0;         // per instantiation: the largest limit set so far
    if (smem > 48 * 1024 && (int)smem > raised) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        raised = (int)smem;
    }
    kern<<<grid, NT, smem, s>>>(p);
    TL_LAUNCH_CHECK();
    return TL_OK;
}

template <typename T>
int launch_hd(const AttnParams& p, dim3 grid, cudaStream_t s) {
    if (p.head_dim <= 64) return launch<T, 64>(p, grid, s);
    if (p.head_dim <= 128) return launch<T, 128>(p, grid, s);
    return launch<T, 256>(p, grid, s);
}

}  // namespace

// How many key splits the general kernel would use for this batch, and how many float32 words of
// workspace (partials and their max / sum) the caller must provide.  n_splits == 1 needs none.
extern "C" int tl_attention_plan(int n_tokens, int n_seqs, int n_heads, int n_kv_heads, int head_dim,
                                 int max_q_len, int max_kv_len, int allow_split,
                                 int* n_splits, long long* workspace_floats) {
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0) return TL_BAD_SIZE;
    if (head_dim <= 0 || head_dim % 16 != 0 || head_dim > 256) return TL_BAD_SIZE;
    const Plan pl = make_plan(n_seqs, n_heads, n_kv_heads, max_q_len, max_kv_len, allow_split);
    *n_splits = pl.n_splits;
    *workspace_floats = pl.n_splits > 1 ? (long long)n_tokens * n_heads * pl.n_splits * (head_dim + 2) : 0;
    return TL_OK;
}

// q, out: [n_tokens, n_heads, head_dim]; pages: [n_pages, n_kv_heads, page_size, head_dim];
// block_table: [n_seqs, table_stride]; q_start: [n_seqs + 1]; kv_len: [n_seqs] (length after this
// step's tokens were appended).  workspace: float32, as large as tl_attention_plan said (may be
// null when it said 0).  window <= 0 means no window.
extern "C" int tl_paged_attention(const void* q, const void* k_pages, const void* v_pages, void* out,
                                  const int* block_table, int table_stride, const int* q_start,
                                  const int* kv_len, float* workspace, int dtype, int n_tokens, int n_seqs,
                                  int n_heads, int n_kv_heads, int head_dim, int page_size, int max_q_len,
                                  int max_kv_len, int window, float scale, int allow_split, void* stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return TL_OK;
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || page_size <= 0) return TL_BAD_SIZE;
    if (head_dim <= 0 || head_dim % 16 != 0 || head_dim > 256) return TL_BAD_SIZE;
    if (max_q_len <= 0 || max_kv_len <= 0) return TL_BAD_SIZE;
    if (!aligned16(q) || !aligned16(k_pages) || !aligned16(v_pages) || !aligned16(out)) return TL_BAD_ALIGN;
    const Plan pl = make_plan(n_seqs, n_heads, n_kv_heads, max_q_len, max_kv_len, allow_split);
    if (pl.n_splits > 1 && workspace == nullptr) return TL_BAD_SIZE;
    if (n_seqs > 65535 || (long long)n_kv_heads * pl.n_gchunks > 65535) return TL_BAD_SIZE;

    AttnParams p;
    p.q = q; p.k_pages = k_pages; p.v_pages = v_pages; p.out = out;
    p.block_table = block_table; p.q_start = q_start; p.kv_len = kv_len;
    p.table_stride = table_stride;
    p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.head_dim = head_dim; p.page_size = page_size;
    p.group = n_heads / n_kv_heads; p.gchunk = pl.gchunk; p.n_gchunks = pl.n_gchunks;
    p.tokens_per_tile = pl.tokens_per_tile;
    p.window = window > 0 ? window : 0;
    p.n_splits = pl.n_splits;
    p.scale = scale;
    p.part_o = workspace;
    p.part_ml = workspace ? workspace + (size_t)n_tokens * n_heads * pl.n_splits * head_dim : nullptr;

    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(pl.n_q_tiles * pl.n_splits, n_kv_heads * pl.n_gchunks, n_seqs);
    int rc;
    if (dtype == TL_F32) rc = launch_hd<float>(p, grid, s);
    else if (dtype == TL_BF16) rc = launch_hd<__nv_bfloat16>(p, grid, s);
    else return TL_BAD_DTYPE;
    if (rc != TL_OK) return rc;
    if (pl.n_splits > 1) {
        const int threads = head_dim >= 128 ? 128 : 64;
        const unsigned rows = (unsigned)n_tokens * n_heads;
        if (dtype == TL_F32)
            attention_merge_kernel<float><<<rows, threads, 0, s>>>(p.part_o, p.part_ml, (float*)out, pl.n_splits, head_dim);
        else
            attention_merge_kernel<__nv_bfloat16><<<rows, threads, 0, s>>>(p.part_o, p.part_ml, (__nv_bfloat16*)out, pl.n_splits, head_dim);
        TL_LAUNCH_CHECK();
    }
    return TL_OK;
}

// ---------------------------------------------------------------------------------------------
// The same attention for callers that may not allocate: the split-KV partials live in a fixed
// array inside this library instead of a workspace the caller brings.  See
// attention_static_scratch.h for who needs this and for the rules of use.
#include "attention_static_scratch.h"

namespace {

// Part of the library image: present on every device that loads it, until the process ends.
static __device__ __align__(256) float tl_static_scratch[TL_STATIC_SCRATCH_FLOATS];

constexpr int MAX_DEVICES = 64;
float* static_scratch_address[MAX_DEVICES] = {};   // per device, asked for once

// In host code the array's name is only a handle for the runtime, not a pointer a kernel could
// use; the device address has to be asked for, with the right device current.
int static_scratch_for_current_device(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= MAX_DEVICES) return TL_STATIC_SCRATCH_NO_ADDRESS;
    if (static_scratch_address[dev] == nullptr) {
        float* ptr = nullptr;
        e = cudaGetSymbolAddress((void**)&ptr, tl_static_scratch);
        if (e != cudaSuccess) return (int)e;
        if (ptr == nullptr) return TL_STATIC_SCRATCH_NO_ADDRESS;
        static_scratch_address[dev] = ptr;
    }
    *out = static_scratch_address[dev];
    return TL_OK;
}

}  // namespace

extern "C" int tl_paged_attention_static_scratch(const void* q, const void* k_pages, const void* v_pages, void* out,
                                                 const int* block_table, int table_stride, const int* q_start,
                                                 const int* kv_len, int dtype, int n_tokens, int n_seqs, int n_heads,
                                                 int n_kv_heads, int head_dim, int page_size, int max_q_len,
                                                 int max_kv_len, int window, float scale, int allow_split, void* stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return TL_OK;
    int n_splits = 0;
    long long floats = 0;
    int rc = tl_attention_plan(n_tokens, n_seqs, n_heads, n_kv_heads, head_dim, max_q_len, max_kv_len, allow_split,
                               &n_splits, &floats);
    if (rc != TL_OK) return rc;
    if (floats > (long long)TL_STATIC_SCRATCH_FLOATS) return TL_STATIC_SCRATCH_TOO_SMALL;   // nothing was launched
    float* scratch = nullptr;
    rc = static_scratch_for_current_device(&scratch);
    if (rc != TL_OK) return rc;
    // Every (row, split) cell that the merge reads is written by the attention kernel of this same
    // call first, so what an earlier call left in the array does not matter and nothing is cleared.
    return tl_paged_attention(q, k_pages, v_pages, out, block_table, table_stride, q_start, kv_len, scratch, dtype,
                              n_tokens, n_seqs, n_heads, n_kv_heads, head_dim, page_size, max_q_len, max_kv_len,
                              window, scale, allow_split, stream);
}

extern "C" const char* tl_static_scratch_strerror(int code) {
    switch (code) {
        case TL_OK: return "ok";
        case TL_STATIC_SCRATCH_TOO_SMALL:
            return "this step needs more split-KV scratch than the 8 MiB array built into the library holds; "
                   "use fewer tokens, heads or splits per call, or tl_paged_attention with a workspace of your own";
        case TL_STATIC_SCRATCH_NO_ADDRESS:
            return "the runtime gave no device address for the built-in scratch array on the current device";
        default: return "see the status codes of tl_paged_attention";
    }
}
