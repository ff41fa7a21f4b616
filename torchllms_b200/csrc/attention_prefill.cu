// Prefill attention over paged bfloat16 keys and values on the fifth-generation tensor cores
// (head_dim 64 or 128): for steps whose requests bring long portions of their prompts.
//
// Same contract as the kernels in attention_mma.cu (causal, optional sliding window, grouped
// heads, float32 scores / running maximum / sum / accumulator), other machinery: both products
// are tcgen05.mma with accumulators in tensor memory, operands arrive by TMA, and a thread owns
// a whole query row, so the softmax needs no exchange between threads.
//
// A CTA serves 128 consecutive tokens of one request and one query head (M = 128), walking the
// visible keys in tiles of 128.  192 threads:
//   warps 0-3      : softmax.  Thread r owns row r = TMEM lane r: reads its 128 scores
//                    (tcgen05.ld), masks, keeps the running maximum and sum, writes the
//                    probabilities into shared memory in the operand layout, rescales
//                    its accumulator row in TMEM when the maximum has grown, and at the end
//                    divides the row by the sum and stores it.
//   warp 4, lane 0 : issues the products.  S_j = Q K_j^T into one of two score buffers in TMEM
//                    (so that S_{j+1} is computed while the softmax works on S_j), then
//                    O += P_j V_j once the probabilities are in place.
//   warp 5, lane 0 : TMA producer: the Q tile once, then per key tile one box per page (or per
//                    128 rows of a larger page) and 64-element column block of K and of V into
//                    128-byte-swizzled shared memory; no multicast.
// Q and K are K-major operands (rows of 128 bytes, swizzled); V is used as stored, keys x
// columns, as an MN-major operand.  Probabilities are multiplied as value + remainder, both
// bfloat16 (two products), so that the product keeps 16 bits of them, as in the other kernels.
//
// The maximum that exponents are taken against is allowed to lag behind the true running
// maximum by up to 2^8: the accumulator row is rescaled (a round trip through registers) only
// when a row's maximum has grown by more than that.  The result is the same up to rounding,
// since numerator and denominator carry the same factor.
//
// Every mbarrier wait is bounded in time; on a time-out the CTA records a code in the status word,
// stops, frees its tensor memory and returns without writing.
#include "common.cuh"
#include <cuda.h>
#include <limits.h>
#include <math.h>
#include <map>
#include <mutex>
#include <tuple>

namespace {

constexpr int BM = 128;                 // query rows (tokens) per CTA
constexpr int BN = 128;                 // keys per tile
constexpr int NTHREADS = 192;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LAG = 8.f;              // how far (in powers of two) the maximum in use may lag
constexpr unsigned long long WAIT_NS = 2000ull * 1000ull * 1000ull;
enum : int { ERR_PRODUCER_WAIT = 301, ERR_ISSUER_WAIT = 302, ERR_SOFTMAX_WAIT = 303, ERR_BAD_COPY = 304 };
constexpr unsigned TMEM_COLS = 512;     // two score buffers of 128 columns and the accumulator
constexpr unsigned COL_S = 0, COL_O = 256;

struct PrefillParams {
    __nv_bfloat16* out;
    const int* block_table;
    const int* q_start;
    const int* kv_len;
    int* status;
    int table_stride;
    int n_heads, n_kv_heads, page_size, page_shift, box_rows;
    int total_rows;             // rows of the page tensor: a copy that starts there reads only the zero fill
    int n_q_tiles;
    int window;
    float scale_log2;
};

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// false once WAIT_NS have passed, or as soon as another role has given up
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity, volatile int* failed) {
    if (mbar_try_wait(bar, parity)) return true;
    unsigned long long t0;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
    for (unsigned i = 1;; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 0u) {
            unsigned long long t1;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
            if (*failed || t1 - t0 > WAIT_NS) return false;
        }
    }
}
// a copy must start on 16 bytes in global memory (x a multiple of 8 elements) and, for the
// 128-byte swizzle, on 128 bytes in shared memory; y must not be negative
__device__ __forceinline__ bool copy_is_sound(const void* dst, int x, int y) {
    return (x & 7) == 0 && x >= 0 && y >= 0 && (smem_u32(dst) & 127u) == 0u;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, unsigned long long* bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}

// shared-memory matrix descriptors, 128-byte swizzle, rows of 128 bytes, 8-row groups 1024 bytes apart.
// K-major (Q, K, P): the row is the M or N index, K runs along the 128-byte row.
__device__ __forceinline__ unsigned long long desc_k_major(unsigned addr) {
    unsigned long long d = 0;
    d |= (unsigned long long)((addr & 0x3FFFFu) >> 4);
    d |= (unsigned long long)(1024u >> 4) << 32;                 // between 8-row groups
    d |= (unsigned long long)1u << 46;
    d |= (unsigned long long)2u << 61;
    return d;
}
// MN-major (V as stored): the 128-byte row is a key (the K index) holding 64 consecutive columns
// (the N index); 8 keys make a 1024-byte group, the next 64 columns lie block_bytes further on.
__device__ __forceinline__ unsigned long long desc_mn_major(unsigned addr, unsigned block_bytes) {
    unsigned long long d = 0;
    d |= (unsigned long long)((addr & 0x3FFFFu) >> 4);
    d |= (unsigned long long)((block_bytes >> 4) & 0x3FFFu) << 16;   // between 64-column blocks
    d |= (unsigned long long)(1024u >> 4) << 32;                     // between 8-key groups
    d |= (unsigned long long)1u << 46;
    d |= (unsigned long long)2u << 61;
    return d;
}
// instruction descriptor: float32 accumulator, M = 128, N = n; formats 0 = float16, 1 = bfloat16
__host__ __device__ constexpr unsigned idesc(int n, unsigned a_fmt, unsigned b_fmt, unsigned b_mn_major) {
    return (1u << 4) | (a_fmt << 7) | (b_fmt << 10) | (b_mn_major << 16) | ((unsigned)(n >> 3) << 17) | ((unsigned)(BM >> 4) << 24);
}
__device__ __forceinline__ void umma(unsigned tmem_d, unsigned long long a_desc, unsigned long long b_desc,
                                     unsigned id, unsigned accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(id), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(unsigned taddr, unsigned (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
}
__device__ __forceinline__ void tmem_st32(unsigned taddr, const unsigned (&r)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                   "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                   "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
                 : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ float ex2(float x) {     // 2^x, one instruction; 2^-inf = 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

template <int HD, int STAGES>
__global__ void __launch_bounds__(NTHREADS, 1) attention_prefill_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                       const __grid_constant__ CUtensorMap map_k,
                                                                       const __grid_constant__ CUtensorMap map_v,
                                                                       const PrefillParams p) {
    constexpr int HALVES = HD / 64;                      // 64-element (128-byte) column blocks of a row
    constexpr unsigned HALF_BYTES = BN * 128;            // one [128 rows x 128 B] block
    constexpr unsigned Q_BYTES = HALVES * HALF_BYTES;
    constexpr unsigned KV_BYTES = HALVES * HALF_BYTES;   // K (or V) of a tile
    constexpr unsigned STAGE_BYTES = 2 * KV_BYTES;
    constexpr unsigned P_BYTES = 2 * HALF_BYTES;         // [128 rows x 128 keys] bfloat16 as two 64-key blocks; value, then remainder
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~uintptr_t(1023));
    unsigned char* Qs = base;
    unsigned char* Ps = base + Q_BYTES;
    unsigned char* tiles = Ps + 2 * P_BYTES;
    __shared__ __align__(8) unsigned long long q_full;
    __shared__ __align__(8) unsigned long long kv_full[STAGES];
    __shared__ __align__(8) unsigned long long kv_empty[STAGES];
    __shared__ __align__(8) unsigned long long s_full[2];
    __shared__ __align__(8) unsigned long long s_empty[2];
    __shared__ __align__(8) unsigned long long p_full;
    __shared__ __align__(8) unsigned long long pv_done;
    __shared__ unsigned tmem_base_slot;
    __shared__ int failed_flag;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        failed_flag = 0;
        mbar_init(&q_full, 1);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&kv_full[s], 1);
            mbar_init(&kv_empty[s], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&s_full[i], 1);
            mbar_init(&s_empty[i], 4);
        }
        mbar_init(&p_full, 4);
        mbar_init(&pv_done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = tmem_base_slot;
    volatile int* failed = &failed_flag;
    grid_launch_dependents();
    grid_dependency_wait();

    const int b = blockIdx.z;
    const int head = blockIdx.y;
    const int kvh = head / (p.n_heads / p.n_kv_heads);
    const int qs = p.q_start[b];
    const int ql = p.q_start[b + 1] - qs;
    const int kl = p.kv_len[b];
    const int tok0 = (p.n_q_tiles - 1 - (int)blockIdx.x) * BM;      // the tiles with most keys start first
    const bool active = tok0 < ql;
    const int qpos_base = kl - ql;
    const int rows = active ? min(BM, ql - tok0) : 0;
    // keys this tile can see: from the window's start of its first row to its last row's own position
    const int k_lo = p.window > 0 ? max(0, qpos_base + tok0 - p.window + 1) : 0;
    const int k_hi = qpos_base + tok0 + rows;
    const int k_start = k_lo & ~(BN - 1);
    const int n_tiles = active ? (k_hi - k_start + BN - 1) / BN : 0;

    if (warp == 5) {
        if (lane == 0 && active) {
            // ---- producer
            bool sound = (smem_u32(base) & 1023u) == 0u;
#pragma unroll
            for (int h = 0; h < HALVES; ++h) sound = sound && copy_is_sound(Qs + h * HALF_BYTES, head * HD + h * 64, qs + tok0);
            if (!sound) {
                failed_flag = 1;
                atomicExch(p.status, ERR_BAD_COPY);
            }
            mbar_expect_tx(&q_full, Q_BYTES);
#pragma unroll
            for (int h = 0; h < HALVES; ++h)
                if (sound) tma_load_2d(Qs + h * HALF_BYTES, &map_q, &q_full, head * HD + h * 64, qs + tok0);
            const int* table = p.block_table + (size_t)b * p.table_stride;
            for (int j = 0; j < n_tiles && sound; ++j) {
                const int s = j % STAGES;
                if (j >= STAGES && !mbar_wait(&kv_empty[s], ((j / STAGES) - 1) & 1, failed)) {
                    failed_flag = 1;
                    atomicExch(p.status, ERR_PRODUCER_WAIT);
                    break;
                }
                mbar_expect_tx(&kv_full[s], STAGE_BYTES);
                unsigned char* kt = tiles + s * STAGE_BYTES;
                const int k0 = k_start + j * BN;
                for (int c = 0; c < BN / p.box_rows; ++c) {
                    const int kpos = k0 + c * p.box_rows;
                    // boxes past the last key start outside the tensor: the copy writes the zero fill, so
                    // that what is multiplied by probability 0 there is finite
                    int row = p.total_rows;
                    if (kpos < k_hi) {
                        const int page = table[kpos >> p.page_shift];
                        row = (page * p.n_kv_heads + kvh) * p.page_size + (kpos & (p.page_size - 1));
                    }
#pragma unroll
                    for (int h = 0; h < HALVES; ++h) {
                        unsigned char* dst = kt + h * HALF_BYTES + c * p.box_rows * 128;
                        if (!copy_is_sound(dst, h * 64, row) || !copy_is_sound(dst + KV_BYTES, h * 64, row)) {
                            failed_flag = 1;
                            atomicExch(p.status, ERR_BAD_COPY);
                            sound = false;
                            continue;
                        }
                        tma_load_2d(dst, &map_k, &kv_full[s], h * 64, row);
                        tma_load_2d(dst + KV_BYTES, &map_v, &kv_full[s], h * 64, row);
                    }
                }
            }
        }
    } else if (warp == 4) {
        if (lane == 0 && active) {
            // ---- issuer: S_0, then per tile S_{j+1} (while the softmax works on S_j) and O += P_j V_j
            constexpr unsigned id_s = idesc(BN, 1u, 1u, 0u);     // bf16 x bf16, both K-major
            constexpr unsigned id_o = idesc(HD, 1u, 1u, 1u);     // bf16 probabilities x bf16 values as stored (MN-major)
            bool ok = mbar_wait(&q_full, 0, failed);
            auto issue_s = [&](int j) -> bool {
                const int s = j % STAGES, sb = j & 1;
                if (!mbar_wait(&kv_full[s], (j / STAGES) & 1, failed)) return false;
                if (j >= 2 && !mbar_wait(&s_empty[sb], ((j >> 1) - 1) & 1, failed)) return false;
                tc_fence_after();
                const unsigned qa = smem_u32(Qs), ka = smem_u32(tiles + s * STAGE_BYTES);
#pragma unroll
                for (int kd = 0; kd < HD / 16; ++kd) {
                    const unsigned off = (kd / 4) * HALF_BYTES + (kd % 4) * 32;
                    umma(tmem + COL_S + sb * BN, desc_k_major(qa + off), desc_k_major(ka + off), id_s, kd > 0 ? 1u : 0u);
                }
                umma_commit(&s_full[sb]);
                return true;
            };
            ok = ok && issue_s(0);
            for (int j = 0; j < n_tiles && ok; ++j) {
                if (j + 1 < n_tiles) ok = issue_s(j + 1);
                if (!ok || !mbar_wait(&p_full, j & 1, failed)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const int s = j % STAGES;
                const unsigned pa = smem_u32(Ps), va = smem_u32(tiles + s * STAGE_BYTES + KV_BYTES);
#pragma unroll
                for (int part = 0; part < 2; ++part)             // value, then remainder
#pragma unroll
                    for (int kk = 0; kk < BN / 16; ++kk)
                        umma(tmem + COL_O, desc_k_major(pa + part * P_BYTES + (kk / 4) * HALF_BYTES + (kk % 4) * 32),
                             desc_mn_major(va + kk * 2048, HALF_BYTES), id_o, (j > 0 || part > 0 || kk > 0) ? 1u : 0u);
                umma_commit(&kv_empty[s]);       // the stage is free once these products have read it
                umma_commit(&pv_done);           // and so are the probabilities; the accumulator is up to date
            }
            if (!ok) {
                failed_flag = 1;
                atomicExch(p.status, ERR_ISSUER_WAIT);
            }
        }
    } else if (active) {
        // ---- softmax: thread r owns row r of the tile, TMEM lane r
        const int r = tid;                                   // warp w reads lanes 32 w .. 32 w + 31
        const unsigned lane_addr = tmem + ((unsigned)(warp * 32) << 16);
        const bool valid = r < rows;
        const int qpos = qpos_base + tok0 + (valid ? r : rows - 1);      // idle rows follow the last real one
        const int tile_qmin = qpos_base + tok0;
        float m_used = -INFINITY, l = 0.f;
        unsigned char* prow = Ps + r * 128;
        bool ok = true;
        for (int j = 0; j < n_tiles; ++j) {
            const int sb = j & 1;
            // (a wait's verdict is taken by the whole warp: the loads below need all of its lanes)
            if (!__all_sync(0xffffffffu, mbar_wait(&s_full[sb], (j >> 1) & 1, failed))) {
                ok = false;
                break;
            }
            tc_fence_after();
            unsigned raw[BN];
#pragma unroll
            for (int c = 0; c < BN / 32; ++c)
                tmem_ld32(lane_addr + COL_S + sb * BN + c * 32, *reinterpret_cast<unsigned(*)[32]>(&raw[c * 32]));
            tmem_wait_ld();
            float sc[BN];
#pragma unroll
            for (int i = 0; i < BN; ++i) sc[i] = __uint_as_float(raw[i]);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_empty[sb]);        // the score buffer may be written again
            const int k0 = k_start + j * BN;
            // the whole tile is visible to every row of this CTA?
            const bool clear = k0 + BN - 1 <= tile_qmin && k0 >= k_lo &&
                               (p.window <= 0 || k0 > qpos_base + tok0 + rows - 1 - p.window);
            if (!clear) {
#pragma unroll
                for (int i = 0; i < BN; ++i) {
                    const int kpos = k0 + i;
                    const bool vis = kpos <= qpos && (p.window <= 0 || kpos > qpos - p.window);
                    if (!vis) sc[i] = -INFINITY;
                }
            }
            float mx0 = sc[0], mx1 = sc[1], mx2 = sc[2], mx3 = sc[3];
#pragma unroll
            for (int i = 4; i < BN; i += 4) {
                mx0 = fmaxf(mx0, sc[i]); mx1 = fmaxf(mx1, sc[i + 1]);
                mx2 = fmaxf(mx2, sc[i + 2]); mx3 = fmaxf(mx3, sc[i + 3]);
            }
            const float m_new = fmaxf(m_used, fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2);
            const bool grow = m_new > m_used + LAG;          // also true for the first keys a row sees
            // before the probabilities are overwritten and the accumulator is touched, the product
            // that reads them must be over
            if (j > 0 && !__all_sync(0xffffffffu, mbar_wait(&pv_done, (j - 1) & 1, failed))) {
                ok = false;
                break;
            }
            if (j > 0 && __any_sync(0xffffffffu, grow)) {
                tc_fence_after();
                const float alpha = grow ? ex2(m_used - m_new) : 1.f;     // 0 for a row that had seen nothing
                l *= alpha;
#pragma unroll
                for (int c = 0; c < HD / 32; ++c) {
                    unsigned v[32];
                    tmem_ld32(lane_addr + COL_O + c * 32, v);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                    tmem_st32(lane_addr + COL_O + c * 32, v);
                }
                tmem_wait_st();
            }
            if (grow) m_used = m_new;
            const float m_safe = (m_used == -INFINITY) ? 0.f : m_used;   // nothing seen yet: keep exponents finite
            float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
#pragma unroll
            for (int c = 0; c < BN / 8; ++c) {
                float e[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) e[i] = ex2(fmaf(sc[c * 8 + i], p.scale_log2, -m_safe));
                l0 += e[0] + e[4]; l1 += e[1] + e[5]; l2 += e[2] + e[6]; l3 += e[3] + e[7];
                unsigned hi[4], lo[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const __nv_bfloat162 h2 = __floats2bfloat162_rn(e[2 * i], e[2 * i + 1]);
                    const float2 back = __bfloat1622float2(h2);
                    hi[i] = *reinterpret_cast<const unsigned*>(&h2);
                    lo[i] = pack_bf16(e[2 * i] - back.x, e[2 * i + 1] - back.y);
                }
                // chunk c of this row: 64-key block c / 8, 16-byte chunk c % 8, swizzled with the row
                unsigned char* at = prow + (c >> 3) * HALF_BYTES + (((c & 7) ^ (r & 7)) << 4);
                *reinterpret_cast<uint4*>(at) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                *reinterpret_cast<uint4*>(at + P_BYTES) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
            }
            l += (l0 + l1) + (l2 + l3);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the tensor core reads what threads wrote
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full);
        }
        if (ok && n_tiles > 0) ok = mbar_wait(&pv_done, (n_tiles - 1) & 1, failed);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
            if (lane == 0) {
                failed_flag = 1;
                atomicExch(p.status, ERR_SOFTMAX_WAIT);
            }
        } else {
            tc_fence_after();
            const float inv = l > 0.f ? 1.f / l : 0.f;
            __nv_bfloat16* orow = p.out + ((size_t)(qs + tok0 + r) * p.n_heads + head) * HD;
#pragma unroll
            for (int c = 0; c < HD / 32; ++c) {
                unsigned v[32];
                tmem_ld32(lane_addr + COL_O + c * 32, v);     // every lane takes part in the load
                tmem_wait_ld();
                if (valid) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint4 w;
                        w.x = pack_bf16(__uint_as_float(v[8 * i]) * inv, __uint_as_float(v[8 * i + 1]) * inv);
                        w.y = pack_bf16(__uint_as_float(v[8 * i + 2]) * inv, __uint_as_float(v[8 * i + 3]) * inv);
                        w.z = pack_bf16(__uint_as_float(v[8 * i + 4]) * inv, __uint_as_float(v[8 * i + 5]) * inv);
                        w.w = pack_bf16(__uint_as_float(v[8 * i + 6]) * inv, __uint_as_float(v[8 * i + 7]) * inv);
                        *reinterpret_cast<uint4*>(orow + c * 32 + i * 8) = w;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 4) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

// ---- host side ---------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// rows x cols bfloat16, row-major; box = box_rows x 64 elements, 128-byte swizzle, zero fill outside.
// Maps are kept per (pointer, rows, cols, box): page tensors live as long as the engine, and the
// query buffer of a recorded step keeps its address.
int tiled_map(CUtensorMap* out, const void* base, long long rows, long long cols, int box_rows) {
    static std::map<std::tuple<const void*, long long, long long, int>, CUtensorMap> cache;
    static std::mutex lock;
    std::lock_guard<std::mutex> guard(lock);
    auto key = std::make_tuple(base, rows, cols, box_rows);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return TL_OK;
    }
    EncodeTiledFn fn = encode_tiled();
    if (fn == nullptr) return TL_BAD_SIZE;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUtensorMap m;
    CUresult rc = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return TL_BAD_SIZE;
    if (cache.size() > 4096) cache.clear();
    cache[key] = m;
    *out = m;
    return TL_OK;
}

template <int HD> constexpr int stages_for() { return HD == 128 ? 2 : 3; }
template <int HD> constexpr size_t smem_for() {
    return (size_t)(HD / 64) * BN * 128 + 2 * 2 * BN * 128 + (size_t)stages_for<HD>() * 2 * (HD / 64) * BN * 128 + 1024;
}

bool takes(int n_heads, int n_kv_heads, int head_dim, int page_size) {
    if (head_dim != 64 && head_dim != 128) return false;
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0) return false;
    return page_size >= 1 && (page_size & (page_size - 1)) == 0;           // a power of two
}

template <int HD>
int launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const PrefillParams& p, dim3 grid, cudaStream_t s) {
    constexpr size_t smem = smem_for<HD>();
    auto kern = attention_prefill_kernel<HD, stages_for<HD>()>;
    static bool raised = false;
    if (!raised) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        raised = true;
    }
    return (int)tl_launch(kern, grid, dim3(NTHREADS), smem, s, mq, mk, mv, p);
}

}  // namespace

// 1 if this kernel takes the shapes: head_dim 64 or 128 and a page size that is a power of two.
extern "C" int tl_attention_prefill_supports(int n_heads, int n_kv_heads, int head_dim, int page_size) {
    return takes(n_heads, n_kv_heads, head_dim, page_size) ? 1 : 0;
}

// q, out: [q_rows, n_heads, head_dim] bfloat16 (q_rows: all rows of the buffer, n_tokens of them in
// use by the n_seqs requests given); pages: [n_pages, n_kv_heads, page_size, head_dim].
extern "C" int tl_paged_attention_prefill(const void* q, const void* k_pages, const void* v_pages, void* out,
                                          const int* block_table, int table_stride, const int* q_start,
                                          const int* kv_len, int* status, long long q_rows, int n_tokens, int n_seqs,
                                          int n_heads, int n_kv_heads, int head_dim, int page_size, long long n_pages,
                                          int max_q_len, int window, float scale, void* stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return TL_OK;
    if (!takes(n_heads, n_kv_heads, head_dim, page_size) || max_q_len <= 0 || n_pages <= 0 || q_rows < n_tokens) return TL_BAD_SIZE;
    if (n_pages * n_kv_heads * page_size >= (1LL << 31)) return TL_BAD_SIZE;
    if (!aligned16(q) || !aligned16(k_pages) || !aligned16(v_pages) || !aligned16(out) || status == nullptr) return TL_BAD_ALIGN;
    if (n_seqs > 65535 || n_heads > 65535) return TL_BAD_SIZE;

    PrefillParams p;
    p.out = (__nv_bfloat16*)out;
    p.block_table = block_table; p.q_start = q_start; p.kv_len = kv_len; p.table_stride = table_stride;
    p.status = status;
    p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.page_size = page_size;
    p.page_shift = 0;
    while ((1 << p.page_shift) < page_size) ++p.page_shift;
    p.box_rows = page_size < BN ? page_size : BN;
    p.total_rows = (int)(n_pages * n_kv_heads * page_size);
    p.n_q_tiles = (max_q_len + BM - 1) / BM;
    p.window = window > 0 ? window : 0;
    p.scale_log2 = scale * LOG2E;

    const long long rows = n_pages * n_kv_heads * page_size;
    CUtensorMap mq, mk, mv;
    int rc = tiled_map(&mq, q, q_rows, (long long)n_heads * head_dim, BM);
    if (rc != TL_OK) return rc;
    rc = tiled_map(&mk, k_pages, rows, head_dim, p.box_rows);
    if (rc != TL_OK) return rc;
    rc = tiled_map(&mv, v_pages, rows, head_dim, p.box_rows);
    if (rc != TL_OK) return rc;

    dim3 grid(p.n_q_tiles, n_heads, n_seqs);
    cudaStream_t s = (cudaStream_t)stream;
    return head_dim == 128 ? launch<128>(mq, mk, mv, p, grid, s) : launch<64>(mq, mk, mv, p, grid, s);
}
