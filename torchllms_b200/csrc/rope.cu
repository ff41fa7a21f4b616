// Rotary encoding of q and k fused with the write of k and v into their cache pages.
//
// Input is the packed projection row [q heads | k heads | v heads] of every token.  q and k are
// rotated in float32 with (cos, sin) gathered from a float32 table at the token's absolute
// position; v is copied.  Reference: torchllms/models/networks.py:332-352 (rotation of adjacent
// lanes) and :551-553 (k is stored after rotation, v as it is).  `interleaved` pairs lanes
// (2i, 2i+1); otherwise lanes (i, i + head_dim/2) are paired.
//
// Pages are laid out [page, kv_head, slot_in_page, head_dim]; slot_mapping[t] = page * page_size + slot.
#include "common.cuh"

template <typename T>
__global__ void rope_kv_write_kernel(const T* __restrict__ qkv, const int* __restrict__ positions,
                                     const float* __restrict__ table, const int* __restrict__ slot_mapping,
                                     T* __restrict__ q_out, T* __restrict__ k_pages, T* __restrict__ v_pages,
                                     int n_heads, int n_kv_heads, int head_dim, int page_size,
                                     int table_rows, int interleaved) {
    const int t = blockIdx.x;
    const int half = head_dim >> 1;
    int pos = positions[t];
    pos = pos < 0 ? 0 : (pos >= table_rows ? table_rows - 1 : pos);  // the host keeps positions inside the table
    const float* cs = table + (size_t)pos * head_dim;                 // [half][2]
    const int row = (n_heads + 2 * n_kv_heads) * head_dim;
    const T* src = qkv + (size_t)t * row;
    const int n_rot_pairs = (n_heads + n_kv_heads) * half;
    const int n_pairs = (n_heads + 2 * n_kv_heads) * half;
    int page = 0, slot = 0;
    const bool write = k_pages != nullptr;
    if (write) {
        const int sm = slot_mapping[t];
        page = sm / page_size;
        slot = sm - page * page_size;
    }
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int head = p / half;       // 0 .. H + 2 KV - 1 over the packed row
        const int i = p - head * half;
        const int l0 = interleaved ? 2 * i : i;
        const int l1 = interleaved ? 2 * i + 1 : i + half;
        float x0 = to_float(src[head * head_dim + l0]);
        float x1 = to_float(src[head * head_dim + l1]);
        if (p < n_rot_pairs) {
            const float c = cs[2 * i], s = cs[2 * i + 1];
            const float y0 = x0 * c - x1 * s;
            const float y1 = x1 * c + x0 * s;
            x0 = y0;
            x1 = y1;
        }
        if (head < n_heads) {
            T* dst = q_out + ((size_t)t * n_heads + head) * head_dim;
            dst[l0] = from_float<T>(x0);
            dst[l1] = from_float<T>(x1);
        } else if (write) {
            const bool is_k = head < n_heads + n_kv_heads;
            const int kvh = is_k ? head - n_heads : head - n_heads - n_kv_heads;
            T* base = is_k ? k_pages : v_pages;
            T* dst = base + (((size_t)page * n_kv_heads + kvh) * page_size + slot) * head_dim;
            dst[l0] = from_float<T>(x0);
            dst[l1] = from_float<T>(x1);
        }
    }
}

// k_pages / v_pages may both be null: then only q is produced (a run that reads another run's cache).
extern "C" int tl_rope_kv_write(const void* qkv, const int* positions, const float* table,
                                const int* slot_mapping, void* q_out, void* k_pages, void* v_pages,
                                int dtype, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                int page_size, int table_rows, int interleaved, void* stream) {
    if (n_tokens <= 0) return TL_OK;
    if (head_dim <= 0 || (head_dim & 1) || n_heads <= 0 || n_kv_heads <= 0 || page_size <= 0 || table_rows <= 0)
        return TL_BAD_SIZE;
    if ((k_pages == nullptr) != (v_pages == nullptr)) return TL_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const int pairs = (n_heads + 2 * n_kv_heads) * (head_dim / 2);
    const int threads = pairs >= 1024 ? 256 : 128;
    if (dtype == TL_F32)
        rope_kv_write_kernel<float><<<n_tokens, threads, 0, s>>>(
            (const float*)qkv, positions, table, slot_mapping, (float*)q_out, (float*)k_pages, (float*)v_pages,
            n_heads, n_kv_heads, head_dim, page_size, table_rows, interleaved);
    else if (dtype == TL_BF16)
        rope_kv_write_kernel<__nv_bfloat16><<<n_tokens, threads, 0, s>>>(
            (const __nv_bfloat16*)qkv, positions, table, slot_mapping, (__nv_bfloat16*)q_out,
            (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages,
            n_heads, n_kv_heads, head_dim, page_size, table_rows, interleaved);
    else
        return TL_BAD_DTYPE;
    TL_LAUNCH_CHECK();
    return TL_OK;
}
