// Prefill attention over paged bfloat16 keys and values on the fifth-generation tensor cores
// (head_dim 64 or 128): for steps whose requests bring long portions of their prompts.
//
// Same contract as the kernels in attention_mma.cu (causal, optional sliding window, grouped
// heads, float32 scores / running maximum / sum / accumulator), other machinery: both products
// are tcgen05.mma with accumulators in tensor memory, K and V arrive by TMA.
//
// Two kernels.  The one that is used by default is the second in this file: one bfloat16 per
// probability, a thread to a query row, 512 threads.  The first, described next, multiplies every
// probability as value + remainder (half the rounding error, a third slower); it has two threads
// to a query row that exchange one number per key tile.  Both share the tiling, the producer and
// the issuers' order of work.
//
// A CTA serves 256 consecutive tokens of one request and one query head as two query tiles of
// 128 rows (M = 128 each), walking the visible keys in tiles of 128.  Every K and V tile that is
// loaded serves both query tiles: the step is bound by what the SMs can pull out of L2 otherwise.
// 352 threads:
//   warps 0-7      : softmax, for one query tile after the other.  Row r = TMEM lane r belongs to
//                    two threads, one in warp r / 32 for the key tile's first 64 keys and one in
//                    warp 4 + r / 32 for the other 64 (a warp reaches the lanes 32 (w mod 4) ..
//                    + 31 only).  At the start each writes its half of its query rows into shared
//                    memory in the operand layout.  Per (key tile, query tile) each reads its
//                    scores (tcgen05.ld), masks, and the two swap their maxima through shared
//                    memory; both then keep the same running maximum, a sum of their own, write
//                    their probabilities back into tensor memory where the scores were
//                    (tcgen05.st), rescale their half of the accumulator row when the maximum has
//                    grown, and at the end divide it by the sum and store it.
//   warp 8         : TMA producer: per key tile one box per page (or per 128 rows of a larger
//                    page) and 64-element column block of K and of V into 128-byte-swizzled
//                    shared memory, each in a ring of its own; no multicast.
//   warps 9 and 10 : each issues the products of one query tile (the whole warp in step, one
//                    elected lane issuing): S_j = Q K_j^T, then, once the probabilities are in
//                    place, O += P_j V_j with the probabilities read from tensor memory, and the
//                    scores of the next key tile right behind it.  While the softmax works on one
//                    query tile the tensor core works for the other.  (One thread polling for both
//                    tiles left the tensor core idle between its turns.)
// Q and K are K-major operands (rows of 128 bytes, swizzled); V is used as stored, keys x
// columns, as an MN-major operand.  In this kernel probabilities are multiplied as value +
// remainder, both bfloat16 (two products), so that the product keeps 16 bits of them, as in the
// mma.sync kernels.
// (A float16 left operand against a bfloat16 right operand in one tcgen05.mma.kind::f16 raised
// "illegal instruction" on a B200: the two formats have to be the same.)
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

constexpr int BM = 128;                 // rows of a query tile (tokens of one head)
constexpr int QT = 2;                   // query tiles per CTA: they share every K and V tile that is loaded
constexpr int BN = 128;                 // keys per tile
constexpr int RT = 2;                   // threads that share a query row in the softmax (warps w, w + 4, ..: same TMEM lanes);
                                        // 4 measured the same speed: the softmax is bound by instruction issue, not by latency
constexpr int W_COPY = 4 * RT, W_ISSUE = 4 * RT + 1;   // warps 0 .. 4 RT - 1 are the softmax, then one copies, two issue
constexpr int NTHREADS = (4 * RT + 3) * 32;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LAG = 8.f;              // how far (in powers of two) the maximum in use may lag
constexpr unsigned long long WAIT_NS = 2000ull * 1000ull * 1000ull;
enum : int { ERR_PRODUCER_WAIT = 301, ERR_ISSUER_WAIT = 302, ERR_SOFTMAX_WAIT = 303, ERR_BAD_COPY = 304 };
constexpr unsigned TMEM_COLS = 512;     // two score buffers of 128 columns, the accumulator, the queries
constexpr unsigned COL_S = 0, COL_O = 256;     // scores (then probabilities) of tile t at COL_S + 128 t, its accumulator at COL_O + 128 t

struct PrefillParams {
    const __nv_bfloat16* q;
    __nv_bfloat16* out;
    const int* block_table;
    const int* q_start;
    const int* kv_len;
    int* status;
    int table_stride;
    int n_heads, n_kv_heads, page_size, page_shift, box_rows;
    int total_rows;             // rows of the page tensor: a copy that starts there reads only the zero fill
    int n_q_blocks;             // blocks of QT query tiles
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
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, unsigned long long* bar, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z) : "memory");
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
// The three tensor-core instructions below are for a whole warp in step: one elected lane issues.  So
// the descriptors stay warp-uniform values (uniform registers); a lone lane inside a divergent branch
// cannot have those, and its instructions issued a fifth slower.
// D[tmem] (+)= A[shared] . B[shared]
__device__ __forceinline__ void umma_ss_elect(unsigned tmem_d, unsigned long long a_desc, unsigned long long b_desc,
                                              unsigned id, unsigned accumulate) {
    asm volatile("{\n\t.reg .pred p, e;\n\telect.sync _|e, 0xffffffff;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(id), "r"(accumulate) : "memory");
}
// D[tmem] (+)= A[tmem] . B[shared]: the left operand lies in tensor memory, row = lane, two 16-bit
// elements of K to a column
__device__ __forceinline__ void umma_ts_elect(unsigned tmem_d, unsigned tmem_a, unsigned long long b_desc,
                                              unsigned id, unsigned accumulate) {
    asm volatile("{\n\t.reg .pred p, e;\n\telect.sync _|e, 0xffffffff;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(b_desc), "r"(id), "r"(accumulate) : "memory");
}
// the barrier gets an arrival when everything this lane has issued so far is done
__device__ __forceinline__ void umma_commit_elect(unsigned long long* bar) {
    asm volatile("{\n\t.reg .pred e;\n\telect.sync _|e, 0xffffffff;\n\t"
                 "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld16(unsigned taddr, unsigned (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
}
__device__ __forceinline__ void tmem_st16(unsigned taddr, const unsigned (&r)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
                 : "memory");
}
// N words (a multiple of 16) of this thread's lane, in pieces of 16 columns
template <int N> __device__ __forceinline__ void tmem_ld(unsigned taddr, unsigned (&r)[N]) {
    static_assert(N % 16 == 0, "whole pieces of 16 columns");
#pragma unroll
    for (int c = 0; c < N / 16; ++c) tmem_ld16(taddr + c * 16, *reinterpret_cast<unsigned(*)[16]>(&r[c * 16]));
}
template <int N> __device__ __forceinline__ void tmem_st(unsigned taddr, const unsigned (&r)[N]) {
    static_assert(N % 16 == 0, "whole pieces of 16 columns");
#pragma unroll
    for (int c = 0; c < N / 16; ++c) tmem_st16(taddr + c * 16, *reinterpret_cast<const unsigned(*)[16]>(&r[c * 16]));
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

template <int STAGES>
struct Tail {                   // what lies behind the tiles in shared memory
    unsigned long long q_full, k_full[STAGES], k_empty[STAGES], v_full[STAGES], v_empty[STAGES];
    unsigned long long s_full[QT], p_full[QT], pv_done[QT];
    unsigned tmem_base_slot;
    int failed_flag;
    float swap[2][RT][BM];      // [parity of the softmax's step][part of the row][row]
};

// What a query tile has to do with the CTA's key tiles: it works on tiles first .. last - 1.
struct TileRange {
    int rows, first, last;
};

// PARTS: 2 = probabilities as value + remainder (two products, 16 bits of every probability kept);
// 1 = probabilities rounded to bfloat16 once (one product; the kernel further down does that faster).
template <int HD, int STAGES, int PARTS>
__global__ void __launch_bounds__(NTHREADS, 1) attention_prefill_kernel(const __grid_constant__ CUtensorMap map_k,
                                                                       const __grid_constant__ CUtensorMap map_v,
                                                                       const PrefillParams p) {
    constexpr int HALVES = HD / 64;                      // 64-element (128-byte) column blocks of a row
    constexpr unsigned HALF_BYTES = BN * 128;            // one [128 rows x 128 B] block
    constexpr unsigned KV_BYTES = HALVES * HALF_BYTES;   // K (or V) of a tile; a query tile has the same layout
    // All shared memory is dynamic and laid out by hand: the two query tiles and the K and V rings
    // first (they need 1024-byte alignment for the 128-byte swizzle, which the start of the window
    // has; the producer checks), then the barriers and the little that threads exchange.
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* Qs = smem_raw;                        // [QT] query tiles
    unsigned char* tiles = Qs + QT * KV_BYTES;           // K ring, then V ring
    Tail<STAGES>& tail = *reinterpret_cast<Tail<STAGES>*>(tiles + 2 * STAGES * KV_BYTES);
    unsigned long long& q_full = tail.q_full;
    unsigned long long (&k_full)[STAGES] = tail.k_full;
    unsigned long long (&k_empty)[STAGES] = tail.k_empty;
    unsigned long long (&v_full)[STAGES] = tail.v_full;
    unsigned long long (&v_empty)[STAGES] = tail.v_empty;
    unsigned long long (&s_full)[QT] = tail.s_full;
    unsigned long long (&p_full)[QT] = tail.p_full;
    unsigned long long (&pv_done)[QT] = tail.pv_done;
    unsigned& tmem_base_slot = tail.tmem_base_slot;
    int& failed_flag = tail.failed_flag;
    float (&swap_max)[2][RT][BM] = tail.swap;                // the threads of a row tell each other their maximum

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        failed_flag = 0;
        mbar_init(&q_full, 4 * RT);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&k_full[s], 1);
            mbar_init(&k_empty[s], QT);       // every query tile's issuer lets go of a stage
            mbar_init(&v_full[s], 1);
            mbar_init(&v_empty[s], QT);
        }
        for (int t = 0; t < QT; ++t) {
            mbar_init(&s_full[t], 1);
            mbar_init(&p_full[t], 4 * RT);
            mbar_init(&pv_done[t], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == W_ISSUE) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = tmem_base_slot;
    volatile int* failed = &failed_flag;
    grid_launch_dependents();
    // (what is read down to the dependency wait does not come from the kernels just before this one: the
    // step's index data were uploaded before its first kernel; so this runs while the predecessor still works)

    // CTAs start in the order x, then y, then z: the heads run along x, so that all heads of the
    // query block with most keys start first and the short blocks fill the gaps at the end
    const int b = blockIdx.z;
    const int head = blockIdx.x;
    const int kvh = head / (p.n_heads / p.n_kv_heads);
    const int qs = p.q_start[b];
    const int ql = p.q_start[b + 1] - qs;
    const int kl = p.kv_len[b];
    const int tok0 = (p.n_q_blocks - 1 - (int)blockIdx.y) * (QT * BM);
    const bool active = tok0 < ql;
    const int qpos_base = kl - ql;
    // Keys the CTA walks: from the window's start of its first row to its last row's own position, in
    // tiles of 128 counted from k_start.  Each query tile takes part in the key tiles it can see.
    const int k_lo = p.window > 0 ? max(0, qpos_base + tok0 - p.window + 1) : 0;      // the first key anybody here sees
    const int k_start = k_lo & ~(BN - 1);
    TileRange range[QT];
    int n_tiles = 0;
#pragma unroll
    for (int t = 0; t < QT; ++t) {
        const int t0 = tok0 + t * BM;
        const int rows = active ? max(0, min(BM, ql - t0)) : 0;
        const int lo = p.window > 0 ? max(0, qpos_base + t0 - p.window + 1) : 0;
        range[t].rows = rows;
        range[t].first = rows > 0 ? ((lo & ~(BN - 1)) - k_start) / BN : 0;
        range[t].last = rows > 0 ? (qpos_base + t0 + rows - k_start + BN - 1) / BN : 0;
        n_tiles = max(n_tiles, range[t].last);
    }
    const int k_hi = qpos_base + min(ql, tok0 + QT * BM);    // one past the last key anybody here sees
    grid_dependency_wait();

    if (warp == W_COPY) {
        if (active) {
            // ---- producer (the whole warp: lanes look pages up and issue copies side by side).
            // K and V have rings of their own: a K stage is free as soon as the scores of its tile
            // are computed, long before the V stage of the same tile.
            bool sound = (smem_u32(Qs) & 1023u) == 0u;
            if (!sound && lane == 0) {
                failed_flag = 1;
                atomicExch(p.status, ERR_BAD_COPY);
            }
            const int* table = p.block_table + (size_t)b * p.table_stride;
            const int n_boxes = BN / p.box_rows;
            for (int j = 0; j < n_tiles && sound; ++j) {
                const int s = j % STAGES;
                const int k0 = k_start + j * BN;
                for (int which = 0; which < 2 && sound; ++which) {
                    unsigned long long* full = which == 0 ? &k_full[s] : &v_full[s];
                    unsigned long long* empty = which == 0 ? &k_empty[s] : &v_empty[s];
                    if (j >= STAGES && !__all_sync(0xffffffffu, mbar_wait(empty, ((j / STAGES) - 1) & 1, failed))) {
                        if (lane == 0) {
                            failed_flag = 1;
                            atomicExch(p.status, ERR_PRODUCER_WAIT);
                        }
                        sound = false;
                        break;
                    }
                    if (lane == 0) mbar_expect_tx(full, KV_BYTES);
                    __syncwarp();
                    unsigned char* dst0 = tiles + (which * STAGES + s) * KV_BYTES;
                    const CUtensorMap* map = which == 0 ? &map_k : &map_v;
                    for (int c = lane; c < n_boxes; c += 32) {
                        const int kpos = k0 + c * p.box_rows;
                        // boxes past the last key start outside the tensor: the copy writes the zero fill,
                        // so that what is multiplied by probability 0 there is finite.  So do boxes that
                        // end before the first key of a window: their pages may have been given back
                        // (the table then holds no page for them), and every score there is masked.
                        int row = p.total_rows;
                        if (kpos < k_hi && kpos + p.box_rows > k_lo) {
                            const int page = table[kpos >> p.page_shift];
                            if (tl_check_page(page))               // (debug builds: a bad page reads as the zero fill)
                                row = (page * p.n_kv_heads + kvh) * p.page_size + (kpos & (p.page_size - 1));
                        }
#pragma unroll
                        for (int h = 0; h < HALVES; ++h) {
                            unsigned char* dst = dst0 + h * HALF_BYTES + c * p.box_rows * 128;
                            if (!copy_is_sound(dst, h * 64, row)) {
                                failed_flag = 1;
                                atomicExch(p.status, ERR_BAD_COPY);
                                continue;
                            }
                            tma_load_2d(dst, map, full, h * 64, row);
                        }
                    }
                    __syncwarp();
                }
            }
        }
    } else if (warp >= W_ISSUE) {
        if (active) {
            // ---- issuers, one per query tile (warp W_ISSUE + t); the whole warp runs in step and one
            // elected lane issues.  For every key tile its query tile takes part in: scores
            // S_j = Q K_j^T, then, once the softmax has put the probabilities where the scores were, the
            // product O += P_j V_j with the probabilities read from tensor memory, and right behind it
            // the scores of the next key tile (the tensor core takes its instructions in order, so they
            // overwrite the probabilities only after the product has read them).  What is not on the
            // softmax's path (K, V) is waited for before the probabilities are.  The two tiles' chains
            // do not depend on each other: while one issuer waits for its softmax, the other keeps the
            // tensor core busy.  A stage of K or V is released by both.
            constexpr unsigned id_s = idesc(BN, 1u, 1u, 0u);     // bf16 x bf16, K as stored (K-major)
            constexpr unsigned id_o = idesc(HD, 1u, 1u, 1u);     // bf16 probabilities x bf16 values as stored (MN-major)
            const int t = warp - W_ISSUE;
            const int first = t ? range[1].first : range[0].first, last = t ? range[1].last : range[0].last;
            bool ok = __all_sync(0xffffffffu, mbar_wait(&q_full, 0, failed));
            tc_fence_after();
            const unsigned long long qd0 = desc_k_major(smem_u32(Qs + t * KV_BYTES));
            const unsigned d_s = tmem + COL_S + t * BN, d_o = tmem + COL_O + t * BN;
            // scores of key tile j (its K stage has arrived), or this tile's leave to reuse the stage
            auto scores = [&](int j) {
                const int s = j % STAGES;
                if (j >= first && j < last) {
                    tc_fence_after();
                    // (the address is the low field of a descriptor, in units of 16 bytes: moving
                    // along K is an addition to the descriptor as a whole)
                    const unsigned long long kd0 = desc_k_major(smem_u32(tiles + s * KV_BYTES));
#pragma unroll
                    for (int kd = 0; kd < HD / 16; ++kd) {
                        const unsigned off = ((kd / 4) * HALF_BYTES + (kd % 4) * 32) >> 4;
                        umma_ss_elect(d_s, qd0 + off, kd0 + off, id_s, kd > 0 ? 1u : 0u);
                    }
                    umma_commit_elect(&s_full[t]);
                    umma_commit_elect(&k_empty[s]);        // this tile is done with the K stage once its scores are computed
                } else if (lane == 0) {
                    mbar_arrive(&k_empty[s]);              // not this tile's keys: nothing to wait for
                }
            };
            if (ok && n_tiles > 0) {
                ok = __all_sync(0xffffffffu, mbar_wait(&k_full[0], 0, failed));
                if (ok) scores(0);
            }
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int s = j % STAGES;
                const unsigned ring = (j / STAGES) & 1;
                const bool mine = j >= first && j < last;
                ok = __all_sync(0xffffffffu, mbar_wait(&v_full[s], ring, failed));
                if (ok && j + 1 < n_tiles) ok = __all_sync(0xffffffffu, mbar_wait(&k_full[(j + 1) % STAGES], ((j + 1) / STAGES) & 1, failed));
                if (!ok) break;
                if (mine) {
                    ok = __all_sync(0xffffffffu, mbar_wait(&p_full[t], (j - first) & 1, failed));
                    if (!ok) break;
                    tc_fence_after();
                    const unsigned long long vd0 = desc_mn_major(smem_u32(tiles + (STAGES + s) * KV_BYTES), HALF_BYTES);
                    const unsigned acc = j > first ? 1u : 0u;
#pragma unroll
                    for (int part = 0; part < PARTS; ++part)         // value, then remainder
#pragma unroll
                        for (int kk = 0; kk < BN / 16; ++kk)         // 16 keys on: 2048 bytes of V, 8 columns of P
                            umma_ts_elect(d_o, d_s + part * (BN / 2) + kk * 8, vd0 + kk * (2048 >> 4), id_o,
                                          (part > 0 || kk > 0) ? 1u : acc);
                    umma_commit_elect(&pv_done[t]);        // the accumulator is up to date
                    umma_commit_elect(&v_empty[s]);        // and this tile is done with the V stage
                } else if (lane == 0) {
                    mbar_arrive(&v_empty[s]);
                }
                if (j + 1 < n_tiles) scores(j + 1);
            }
            if (!ok && lane == 0) {
                failed_flag = 1;
                atomicExch(p.status, ERR_ISSUER_WAIT);
            }
        }
    } else if (active) {
        // ---- softmax: row r = TMEM lane r of either query tile; this thread has the keys
        // HN half .. HN half + HN - 1 of every key tile (half: which of the row's RT threads this is)
        constexpr int HN = BN / RT;                          // keys per thread and tile
        constexpr int HO = HD / RT;                          // accumulator columns per thread
        const int half = warp >> 2;
        const int r = (warp & 3) * 32 + lane;
        const unsigned lane_addr = tmem + ((unsigned)((warp & 3) * 32) << 16);
        const int pair_barrier = 1 + (warp & 3);             // named barrier of the RT warps that share 32 rows
        // this thread's half of its query rows goes into shared memory in the layout of a K tile:
        // rows of 128 bytes (64 elements), 16-byte chunks swizzled with the row
#pragma unroll
        for (int t = 0; t < QT; ++t) {
            const bool valid = r < range[t].rows;
            const uint4* src = reinterpret_cast<const uint4*>(p.q + ((size_t)(qs + tok0 + t * BM + r) * p.n_heads + head) * HD + half * HO);
#pragma unroll
            for (int i = 0; i < HO / 8; ++i) {
                const uint4 v = valid ? src[i] : make_uint4(0u, 0u, 0u, 0u);
                const int chunk = (half * HO) / 8 + i;              // of the row: block chunk / 8, chunk % 8 within it
                *reinterpret_cast<uint4*>(Qs + t * KV_BYTES + (chunk >> 3) * HALF_BYTES + r * 128 + (((chunk & 7) ^ (r & 7)) << 4)) = v;
            }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the tensor core reads what threads wrote
        __syncwarp();
        if (lane == 0) mbar_arrive(&q_full);

        // The state of the two query tiles lives in scalars picked by hand, and the loop over the
        // tiles is not unrolled: one copy of the body, no indexed arrays, fewer registers.
        static_assert(QT == 2, "the softmax keeps the state of two query tiles");
        float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
        const int rows_a = range[0].rows, rows_b = range[1].rows;
        const int first_a = range[0].first, first_b = range[1].first, last_a = range[0].last, last_b = range[1].last;
        bool ok = true;
        int step = 0;                                        // counts the (key tile, query tile) pairs done: slot of the swap
        // Once a wait has failed (ok = false) the loop only keeps its appointments at the pair's
        // barrier: both warps of a pair pass it once per step whatever happens, so neither can be
        // left waiting there.
        for (int j = 0; j < n_tiles; ++j) {
            const int k0 = k_start + j * BN;
#pragma unroll 1
            for (int t = 0; t < QT; ++t) {
                const int first = t ? first_b : first_a, last = t ? last_b : last_a, rows = t ? rows_b : rows_a;
                if (j < first || j >= last) continue;
                const int it = j - first;                    // how many tiles this query tile has done
                const int slot = step & 1;
                ++step;
                float m_used = t ? m_b : m_a;
                const int t0 = qpos_base + tok0 + t * BM;    // position of the tile's first row
                const int qpos = t0 + (r < rows ? r : rows - 1);         // idle rows follow the last real one
                const unsigned col_s = COL_S + t * BN, col_o = COL_O + t * BN;
                // (a wait's outcome is taken by the whole warp: the loads below need all of its lanes)
                if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&s_full[t], it & 1, failed));
                if (!ok) failed_flag = 1;
                unsigned raw[HN];                            // the scores
                float mine = -INFINITY;
                if (ok) {
                    tc_fence_after();
                    tmem_ld<HN>(lane_addr + col_s + half * HN, raw);
                    tmem_wait_ld();
                    // the whole key tile is visible to every row of this query tile?
                    const bool clear = k0 + BN - 1 <= t0 && (p.window <= 0 || k0 > t0 + rows - 1 - p.window);
                    if (!clear) {
#pragma unroll
                        for (int i = 0; i < HN; ++i) {
                            const int kpos = k0 + half * HN + i;
                            const bool vis = kpos <= qpos && (p.window <= 0 || kpos > qpos - p.window);
                            if (!vis) raw[i] = 0xff800000u;  // -inf
                        }
                    }
                    float mx0 = __uint_as_float(raw[0]), mx1 = __uint_as_float(raw[1]);
                    float mx2 = __uint_as_float(raw[2]), mx3 = __uint_as_float(raw[3]);
#pragma unroll
                    for (int i = 4; i < HN; i += 4) {
                        mx0 = fmaxf(mx0, __uint_as_float(raw[i])); mx1 = fmaxf(mx1, __uint_as_float(raw[i + 1]));
                        mx2 = fmaxf(mx2, __uint_as_float(raw[i + 2])); mx3 = fmaxf(mx3, __uint_as_float(raw[i + 3]));
                    }
                    mine = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
                }
                // The partner can be one step ahead at most (it stops at the next barrier until this
                // thread gets there), so two slots, used in turn, are never overwritten unread.  Past the
                // barrier both have their scores in registers: the probabilities may go where they were.
                swap_max[slot][half][r] = mine;
                asm volatile("bar.sync %0, %1;" ::"r"(pair_barrier), "n"(32 * RT) : "memory");
                if (!ok) continue;
                float both = mine;
#pragma unroll
                for (int o = 1; o < RT; ++o) both = fmaxf(both, swap_max[slot][(half + o) % RT][r]);
                const float m_new = fmaxf(m_used, both * p.scale_log2);
                const bool grow = m_new > m_used + LAG;      // also true for the first keys a row sees
                const bool rescale = it > 0 && __any_sync(0xffffffffu, grow);
                const float alpha = grow ? ex2(m_used - m_new) : 1.f;        // 0 for a row that had seen nothing
                if (grow) m_used = m_new;
                const float m_safe = (m_used == -INFINITY) ? 0.f : m_used;   // nothing seen yet: keep exponents finite
                // probabilities as value + remainder, two bfloat16 to a column: columns 32 half .. of the
                // tile's buffer hold the values of this thread's keys, columns 64 + 32 half .. the remainders
                unsigned hi[HN / 2], lo[HN / 2];
                // (arithmetic two floats at a time, fma.f32x2 and add.f32x2 of this architecture: the softmax
                // is bound by how many instructions it issues)
                float2 la = make_float2(0.f, 0.f), lb = make_float2(0.f, 0.f);
                const float2 sc2 = make_float2(p.scale_log2, p.scale_log2), nm2 = make_float2(-m_safe, -m_safe);
                const float2 neg1 = make_float2(-1.f, -1.f);
#pragma unroll
                for (int i = 0; i < HN; i += 4) {
                    const float2 xa = __ffma2_rn(make_float2(__uint_as_float(raw[i]), __uint_as_float(raw[i + 1])), sc2, nm2);
                    const float2 xb = __ffma2_rn(make_float2(__uint_as_float(raw[i + 2]), __uint_as_float(raw[i + 3])), sc2, nm2);
                    const float2 ea = make_float2(ex2(xa.x), ex2(xa.y)), eb = make_float2(ex2(xb.x), ex2(xb.y));
                    la = __fadd2_rn(la, ea);
                    lb = __fadd2_rn(lb, eb);
                    const __nv_bfloat162 ha = __floats2bfloat162_rn(ea.x, ea.y), hb = __floats2bfloat162_rn(eb.x, eb.y);
                    hi[i / 2] = *reinterpret_cast<const unsigned*>(&ha);
                    hi[i / 2 + 1] = *reinterpret_cast<const unsigned*>(&hb);
                    if (PARTS == 2) {
                        const float2 ra = __ffma2_rn(__bfloat1622float2(ha), neg1, ea);      // what the rounding left, exactly
                        const float2 rb = __ffma2_rn(__bfloat1622float2(hb), neg1, eb);
                        lo[i / 2] = pack_bf16(ra.x, ra.y);
                        lo[i / 2 + 1] = pack_bf16(rb.x, rb.y);
                    }
                }
                const float l0 = la.x, l1 = la.y, l2 = lb.x, l3 = lb.y;
                float l_sum = (t ? l_b : l_a);
                if (rescale) {
                    // the product that last wrote the accumulator must be over
                    ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[t], (it - 1) & 1, failed));
                    if (!ok) {
                        failed_flag = 1;
                        continue;
                    }
                    tc_fence_after();
                    l_sum *= alpha;
                    unsigned v[HO];
                    tmem_ld<HO>(lane_addr + col_o + half * HO, v);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < HO; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                    tmem_st<HO>(lane_addr + col_o + half * HO, v);
                }
                l_sum += (l0 + l1) + (l2 + l3);
                if (t) { m_b = m_used; l_b = l_sum; } else { m_a = m_used; l_a = l_sum; }
                tmem_st<HN / 2>(lane_addr + col_s + half * (HN / 2), hi);
                if (PARTS == 2) tmem_st<HN / 2>(lane_addr + col_s + BN / 2 + half * (HN / 2), lo);
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&p_full[t]);
            }
        }
        float l[QT] = {l_a, l_b};
        // ---- the end: wait for the last products, add the two halves' sums, divide, store
#pragma unroll
        for (int t = 0; t < QT; ++t) {
            const int n = range[t].last - range[t].first;
            if (ok && n > 0) ok = mbar_wait(&pv_done[t], (n - 1) & 1, failed);
        }
        ok = __all_sync(0xffffffffu, ok);
        // (both warps of a pair come here, failed or not; the slot is the one the last step did not
        // use: the partner has read that one before it came to the last step's barrier)
        float (&swap_sum)[RT][BM] = swap_max[step & 1];
        float (&swap_sum2)[RT][BM] = swap_max[(step & 1) ^ 1];
        swap_sum[half][r] = l[0];
        asm volatile("bar.sync %0, %1;" ::"r"(pair_barrier), "n"(32 * RT) : "memory");
#pragma unroll
        for (int o = 1; o < RT; ++o) l[0] += swap_sum[(half + o) % RT][r];
        swap_sum2[half][r] = l[1];
        asm volatile("bar.sync %0, %1;" ::"r"(pair_barrier), "n"(32 * RT) : "memory");
#pragma unroll
        for (int o = 1; o < RT; ++o) l[1] += swap_sum2[(half + o) % RT][r];
        if (!ok) {
            if (lane == 0) {
                failed_flag = 1;
                atomicExch(p.status, ERR_SOFTMAX_WAIT);
            }
        } else {
            tc_fence_after();
#pragma unroll
            for (int t = 0; t < QT; ++t) {
                if (range[t].rows == 0) continue;
                const bool valid = r < range[t].rows;
                const float inv = l[t] > 0.f ? 1.f / l[t] : 0.f;
                __nv_bfloat16* orow = p.out + ((size_t)(qs + tok0 + t * BM + r) * p.n_heads + head) * HD + half * HO;
                unsigned v[HO];
                tmem_ld<HO>(lane_addr + COL_O + t * BN + half * HO, v);     // every lane takes part in the load
                tmem_wait_ld();
                if (valid) {
#pragma unroll
                    for (int i = 0; i < HO / 8; ++i) {
                        uint4 w;
                        w.x = pack_bf16(__uint_as_float(v[8 * i]) * inv, __uint_as_float(v[8 * i + 1]) * inv);
                        w.y = pack_bf16(__uint_as_float(v[8 * i + 2]) * inv, __uint_as_float(v[8 * i + 3]) * inv);
                        w.z = pack_bf16(__uint_as_float(v[8 * i + 4]) * inv, __uint_as_float(v[8 * i + 5]) * inv);
                        w.w = pack_bf16(__uint_as_float(v[8 * i + 6]) * inv, __uint_as_float(v[8 * i + 7]) * inv);
                        *reinterpret_cast<uint4*>(orow + i * 8) = w;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == W_ISSUE) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}


// ================================================================================================
// The same work with one bfloat16 per probability and the roles spread over four warp groups (512
// threads), so that a query row's softmax is one thread's business and waits for no neighbour:
//   warps 0-3, 4-7 : softmax of query tile 0, of query tile 1.  Row r = TMEM lane r belongs to one
//                    thread, which reads the 128 scores of a key tile into registers once (192
//                    registers a thread: the warp groups trade registers at the start with
//                    setmaxnreg), takes their maximum, tells the correction warps by how much the
//                    row's accumulator has to shrink, and writes the probabilities where the scores were.
//   warps 8-11     : correction.  When a row's maximum in use has grown they rescale its accumulator
//                    (a round trip through registers) off the softmax's path; at the end they divide
//                    by the row's sum and store it.
//   warp 12        : TMA producer (the two query tiles through a three-dimensional map of q, then K and V);
//                    warps 13, 14 : the issuers of the two query tiles (the whole warp
//                    runs in step and one elected lane issues: a lone lane inside a divergent branch
//                    cannot keep the descriptors in uniform registers, and issued a fifth slower);
//                    warp 15 is there to complete the warp group.
// Barriers beside those of the kernel above: alpha_ready (softmax -> correction: factors are in
// shared memory), o_ready (correction -> issuer: the accumulator may take the next product),
// p_half (softmax -> issuer: the probabilities of the tile's first 64 keys are in place, the product may
// start on them), l_ready (softmax -> correction: the row sums are in shared memory), turn (softmax ->
// the other tile's softmax: the exponential unit is yours).
constexpr int NTHREADS_ROWS = 512;
// Registers a thread after the trade: softmax / correction / the rest.  A warp group can only be given
// what another has handed back, so the sum stays within what the launch allots (128 a thread).
constexpr int REGS_SOFTMAX = 192, REGS_CORRECTION = 72, REGS_REST = 40;
static_assert(QT * REGS_SOFTMAX + REGS_CORRECTION + REGS_REST <= 4 * 128, "registers are traded, not made");
constexpr int WR_CORR = 4 * QT, WR_COPY = 4 * QT + 4, WR_ISSUE = 4 * QT + 5;

template <int STAGES>
struct TailRows {
    unsigned long long q_full, k_full[STAGES], k_empty[STAGES], v_full[STAGES], v_empty[STAGES];
    unsigned long long s_full[QT], p_half[QT], p_full[QT], pv_done[QT], alpha_ready[QT], o_ready[QT], l_ready[QT], turn[QT];
    unsigned tmem_base_slot;
    int failed_flag;
    int grow_any[QT][2][4];     // [tile][parity of the tile's step][warp of the tile]: did a row of the warp grow
    float alpha[QT][2][BM];     // [tile][parity of the tile's step][row]: what the row's accumulator shrinks by
    float l_final[QT][BM];
};

template <int N> __device__ __forceinline__ void regs_up() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N> __device__ __forceinline__ void regs_down() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

template <int HD, int STAGES>
__global__ void __launch_bounds__(NTHREADS_ROWS, 1) attention_prefill_rows_kernel(const __grid_constant__ CUtensorMap map_k,
                                                                                 const __grid_constant__ CUtensorMap map_v,
                                                                                 const __grid_constant__ CUtensorMap map_q,
                                                                                 const PrefillParams p) {
    constexpr int HALVES = HD / 64;
    constexpr unsigned HALF_BYTES = BN * 128;
    constexpr unsigned KV_BYTES = HALVES * HALF_BYTES;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* Qs = smem_raw;
    unsigned char* tiles = Qs + QT * KV_BYTES;
    TailRows<STAGES>& tail = *reinterpret_cast<TailRows<STAGES>*>(tiles + 2 * STAGES * KV_BYTES);
    unsigned long long& q_full = tail.q_full;
    unsigned long long (&k_full)[STAGES] = tail.k_full;
    unsigned long long (&k_empty)[STAGES] = tail.k_empty;
    unsigned long long (&v_full)[STAGES] = tail.v_full;
    unsigned long long (&v_empty)[STAGES] = tail.v_empty;
    unsigned long long (&s_full)[QT] = tail.s_full;
    unsigned long long (&p_full)[QT] = tail.p_full;
    unsigned long long (&p_half)[QT] = tail.p_half;
    unsigned long long (&pv_done)[QT] = tail.pv_done;
    unsigned long long (&alpha_ready)[QT] = tail.alpha_ready;
    unsigned long long (&o_ready)[QT] = tail.o_ready;
    unsigned long long (&l_ready)[QT] = tail.l_ready;
    unsigned long long (&turn)[QT] = tail.turn;
    unsigned& tmem_base_slot = tail.tmem_base_slot;
    int& failed_flag = tail.failed_flag;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        failed_flag = 0;
        mbar_init(&q_full, 1);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&k_full[s], 1);
            mbar_init(&k_empty[s], QT);
            mbar_init(&v_full[s], 1);
            mbar_init(&v_empty[s], QT);
        }
        for (int t = 0; t < QT; ++t) {
            mbar_init(&s_full[t], 1);
            mbar_init(&p_full[t], 4);
            mbar_init(&p_half[t], 4);
            mbar_init(&pv_done[t], 1);
            mbar_init(&alpha_ready[t], 4);
            mbar_init(&o_ready[t], 4);
            mbar_init(&l_ready[t], 4);
            mbar_init(&turn[t], 4);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == WR_ISSUE) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = tmem_base_slot;
    volatile int* failed = &failed_flag;
    grid_launch_dependents();
    // (what is read down to the dependency wait does not come from the kernels just before this one: the
    // step's index data were uploaded before its first kernel; so this runs while the predecessor still works)

    const int b = blockIdx.z;
    const int head = blockIdx.x;
    const int kvh = head / (p.n_heads / p.n_kv_heads);
    const int qs = p.q_start[b];
    const int ql = p.q_start[b + 1] - qs;
    const int kl = p.kv_len[b];
    const int tok0 = (p.n_q_blocks - 1 - (int)blockIdx.y) * (QT * BM);
    const bool active = tok0 < ql;
    const int qpos_base = kl - ql;
    const int k_lo = p.window > 0 ? max(0, qpos_base + tok0 - p.window + 1) : 0;
    const int k_start = k_lo & ~(BN - 1);
    TileRange range[QT];
    int n_tiles = 0;
#pragma unroll
    for (int t = 0; t < QT; ++t) {
        const int t0 = tok0 + t * BM;
        const int rows = active ? max(0, min(BM, ql - t0)) : 0;
        const int lo = p.window > 0 ? max(0, qpos_base + t0 - p.window + 1) : 0;
        range[t].rows = rows;
        range[t].first = rows > 0 ? ((lo & ~(BN - 1)) - k_start) / BN : 0;
        range[t].last = rows > 0 ? (qpos_base + t0 + rows - k_start + BN - 1) / BN : 0;
        n_tiles = max(n_tiles, range[t].last);
    }
    const int k_hi = qpos_base + min(ql, tok0 + QT * BM);
    grid_dependency_wait();

    if (warp >= WR_COPY) {
        regs_down<REGS_REST>();
        if (warp == WR_COPY) {
            if (active) {
                // ---- producer: as in the kernel above
                bool sound = (smem_u32(Qs) & 1023u) == 0u;
                if (!sound && lane == 0) {
                    failed_flag = 1;
                    atomicExch(p.status, ERR_BAD_COPY);
                }
                // the queries of both tiles: [128 tokens x 64 elements] boxes of this head, which land in the
                // layout of a K tile (rows past the request's own are another request's or the zero fill:
                // their results are never stored)
                if (sound && lane == 0) {
                    int tiles_q = 0;
                    for (int t = 0; t < QT; ++t) tiles_q += (t ? range[1].rows : range[0].rows) > 0 ? 1 : 0;
                    mbar_expect_tx(&q_full, tiles_q * KV_BYTES);
                    for (int t = 0; t < QT; ++t)
                        if ((t ? range[1].rows : range[0].rows) > 0)
                            for (int h = 0; h < HALVES; ++h)
                                tma_load_3d(Qs + t * KV_BYTES + h * HALF_BYTES, &map_q, &q_full, h * 64, head, qs + tok0 + t * BM);
                }
                __syncwarp();
                const int* table = p.block_table + (size_t)b * p.table_stride;
                const int n_boxes = BN / p.box_rows;
                for (int j = 0; j < n_tiles && sound; ++j) {
                    const int s = j % STAGES;
                    const int k0 = k_start + j * BN;
                    for (int which = 0; which < 2 && sound; ++which) {
                        unsigned long long* full = which == 0 ? &k_full[s] : &v_full[s];
                        unsigned long long* empty = which == 0 ? &k_empty[s] : &v_empty[s];
                        if (j >= STAGES && !__all_sync(0xffffffffu, mbar_wait(empty, ((j / STAGES) - 1) & 1, failed))) {
                            if (lane == 0) {
                                failed_flag = 1;
                                atomicExch(p.status, ERR_PRODUCER_WAIT);
                            }
                            sound = false;
                            break;
                        }
                        if (lane == 0) mbar_expect_tx(full, KV_BYTES);
                        __syncwarp();
                        unsigned char* dst0 = tiles + (which * STAGES + s) * KV_BYTES;
                        const CUtensorMap* map = which == 0 ? &map_k : &map_v;
                        for (int c = lane; c < n_boxes; c += 32) {
                            const int kpos = k0 + c * p.box_rows;
                            int row = p.total_rows;
                            if (kpos < k_hi && kpos + p.box_rows > k_lo) {
                                const int page = table[kpos >> p.page_shift];
                                if (tl_check_page(page))
                                    row = (page * p.n_kv_heads + kvh) * p.page_size + (kpos & (p.page_size - 1));
                            }
#pragma unroll
                            for (int h = 0; h < HALVES; ++h) {
                                unsigned char* dst = dst0 + h * HALF_BYTES + c * p.box_rows * 128;
                                if (!copy_is_sound(dst, h * 64, row)) {
                                    failed_flag = 1;
                                    atomicExch(p.status, ERR_BAD_COPY);
                                    continue;
                                }
                                tma_load_2d(dst, map, full, h * 64, row);
                            }
                        }
                        __syncwarp();
                    }
                }
            }
        } else if (warp < WR_ISSUE + QT) {
            if (active) {
                // ---- issuers, one per query tile; the whole warp runs in step and one elected lane issues.
                // As in the kernel above, with two differences.  The product into the accumulator also waits
                // for the correction warps' word that the accumulator is ready for it.  And the scores of the
                // next key tile are queued right behind that product (the tensor core takes its instructions
                // in order, so the scores overwrite the probabilities only after the product has read them):
                // everything else the two wait for (K, V) is waited for before the probabilities are, so
                // that nothing but the products themselves stands between one softmax and the next.
                constexpr unsigned id_s = idesc(BN, 1u, 1u, 0u);
                constexpr unsigned id_o = idesc(HD, 1u, 1u, 1u);
                const int t = warp - WR_ISSUE;
                const int first = t ? range[1].first : range[0].first, last = t ? range[1].last : range[0].last;
                bool ok = __all_sync(0xffffffffu, mbar_wait(&q_full, 0, failed));
                tc_fence_after();
                const unsigned long long qd0 = desc_k_major(smem_u32(Qs + t * KV_BYTES));
                const unsigned d_s = tmem + COL_S + t * BN, d_o = tmem + COL_O + t * BN;
                // scores of key tile j (its K stage has arrived), or this tile's leave to reuse the stage
                auto scores = [&](int j) {
                    const int s = j % STAGES;
                    if (j >= first && j < last) {
                        tc_fence_after();
                        const unsigned long long kd0 = desc_k_major(smem_u32(tiles + s * KV_BYTES));
#pragma unroll
                        for (int kd = 0; kd < HD / 16; ++kd) {
                            const unsigned off = ((kd / 4) * HALF_BYTES + (kd % 4) * 32) >> 4;
                            umma_ss_elect(d_s, qd0 + off, kd0 + off, id_s, kd > 0 ? 1u : 0u);
                        }
                        umma_commit_elect(&s_full[t]);
                        umma_commit_elect(&k_empty[s]);
                    } else if (lane == 0) {
                        mbar_arrive(&k_empty[s]);
                    }
                };
                if (ok && n_tiles > 0) {
                    ok = __all_sync(0xffffffffu, mbar_wait(&k_full[0], 0, failed));
                    if (ok) scores(0);
                }
                for (int j = 0; j < n_tiles && ok; ++j) {
                    const int s = j % STAGES;
                    const unsigned ring = (j / STAGES) & 1;
                    const bool mine = j >= first && j < last;
                    ok = __all_sync(0xffffffffu, mbar_wait(&v_full[s], ring, failed));
                    if (ok && j + 1 < n_tiles) ok = __all_sync(0xffffffffu, mbar_wait(&k_full[(j + 1) % STAGES], ((j + 1) / STAGES) & 1, failed));
                    if (!ok) break;
                    if (mine) {
                        // the product starts on the first half of the probabilities while the second is still being taken
                        ok = __all_sync(0xffffffffu, mbar_wait(&p_half[t], (j - first) & 1, failed) && mbar_wait(&o_ready[t], (j - first) & 1, failed));
                        if (!ok) break;
                        tc_fence_after();
                        const unsigned long long vd0 = desc_mn_major(smem_u32(tiles + (STAGES + s) * KV_BYTES), HALF_BYTES);
                        const unsigned acc = j > first ? 1u : 0u;
#pragma unroll
                        for (int kk = 0; kk < BN / 32; ++kk)
                            umma_ts_elect(d_o, d_s + kk * 8, vd0 + kk * (2048 >> 4), id_o, kk > 0 ? 1u : acc);
                        ok = __all_sync(0xffffffffu, mbar_wait(&p_full[t], (j - first) & 1, failed));
                        if (!ok) break;
                        tc_fence_after();
#pragma unroll
                        for (int kk = BN / 32; kk < BN / 16; ++kk)
                            umma_ts_elect(d_o, d_s + kk * 8, vd0 + kk * (2048 >> 4), id_o, 1u);
                        umma_commit_elect(&pv_done[t]);
                        umma_commit_elect(&v_empty[s]);
                    } else if (lane == 0) {
                        mbar_arrive(&v_empty[s]);
                    }
                    if (j + 1 < n_tiles) scores(j + 1);
                }
                if (!ok && lane == 0) {
                    failed_flag = 1;
                    atomicExch(p.status, ERR_ISSUER_WAIT);
                }
            }
        }
    } else if (warp >= WR_CORR) {
        regs_down<REGS_CORRECTION>();
        if (active) {
            // ---- correction: row r of either query tile
            constexpr int PIECE = 32;
            const int cw = warp & 3;
            const int r = cw * 32 + lane;
            const unsigned lane_addr = tmem + ((unsigned)(cw * 32) << 16);
            bool ok = true;
            for (int j = 0; j < n_tiles && ok; ++j) {
#pragma unroll 1
                for (int t = 0; t < QT && ok; ++t) {
                    const int first = t ? range[1].first : range[0].first, last = t ? range[1].last : range[0].last;
                    if (j < first || j >= last) continue;
                    const int it = j - first, par = it & 1;
                    ok = __all_sync(0xffffffffu, mbar_wait(&alpha_ready[t], par, failed));
                    if (!ok) break;
                    if (it > 0 && tail.grow_any[t][par][cw]) {
                        ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[t], (it - 1) & 1, failed));     // the product that last wrote the accumulator
                        if (!ok) break;
                        tc_fence_after();
                        const float a = tail.alpha[t][par][r];
#pragma unroll
                        for (int c = 0; c < HD / PIECE; ++c) {
                            unsigned v[PIECE];
                            tmem_ld<PIECE>(lane_addr + COL_O + t * BN + c * PIECE, v);
                            tmem_wait_ld();
#pragma unroll
                            for (int i = 0; i < PIECE; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * a);
                            tmem_st<PIECE>(lane_addr + COL_O + t * BN + c * PIECE, v);
                        }
                        tmem_wait_st();
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&o_ready[t]);
                }
            }
            // ---- the end: the rows' sums, the last products, divide, store
#pragma unroll 1
            for (int t = 0; t < QT && ok; ++t) {
                const int rows = t ? range[1].rows : range[0].rows;
                const int n = (t ? range[1].last : range[0].last) - (t ? range[1].first : range[0].first);
                if (rows == 0 || n <= 0) continue;
                ok = __all_sync(0xffffffffu, mbar_wait(&l_ready[t], 0, failed) && mbar_wait(&pv_done[t], (n - 1) & 1, failed));
                if (!ok) break;
                tc_fence_after();
                const float l = tail.l_final[t][r];
                const float inv = l > 0.f ? 1.f / l : 0.f;
                // The rows leave through shared memory (the query tile's place: its last product is over), in
                // the swizzled layout the queries had, so that they are written to global memory a row
                // at a time; a thread writing 16 bytes of its own row, 8 KB from its neighbour's, took 6 us.
                unsigned char* stage = Qs + t * KV_BYTES;
#pragma unroll
                for (int c = 0; c < HD / PIECE; ++c) {
                    unsigned v[PIECE];
                    tmem_ld<PIECE>(lane_addr + COL_O + t * BN + c * PIECE, v);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < PIECE / 8; ++i) {
                        uint4 w;
                        w.x = pack_bf16(__uint_as_float(v[8 * i]) * inv, __uint_as_float(v[8 * i + 1]) * inv);
                        w.y = pack_bf16(__uint_as_float(v[8 * i + 2]) * inv, __uint_as_float(v[8 * i + 3]) * inv);
                        w.z = pack_bf16(__uint_as_float(v[8 * i + 4]) * inv, __uint_as_float(v[8 * i + 5]) * inv);
                        w.w = pack_bf16(__uint_as_float(v[8 * i + 6]) * inv, __uint_as_float(v[8 * i + 7]) * inv);
                        const int chunk = c * (PIECE / 8) + i;
                        *reinterpret_cast<uint4*>(stage + (chunk >> 3) * HALF_BYTES + r * 128 + (((chunk & 7) ^ (r & 7)) << 4)) = w;
                    }
                }
                __syncwarp();                                // (a warp writes out the 32 rows it staged itself)
                constexpr int CH = HD / 8;
#pragma unroll
                for (int i = 0; i < CH; ++i) {
                    const int row = cw * 32 + i * (32 / CH) + lane / CH, chunk = lane % CH;
                    const uint4 w = *reinterpret_cast<const uint4*>(stage + (chunk >> 3) * HALF_BYTES + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
                    if (row < rows)
                        *reinterpret_cast<uint4*>(p.out + ((size_t)(qs + tok0 + t * BM + row) * p.n_heads + head) * HD + chunk * 8) = w;
                }
            }
            if (!ok && lane == 0) {
                failed_flag = 1;
                atomicExch(p.status, ERR_SOFTMAX_WAIT);
            }
        }
    } else {
        regs_up<REGS_SOFTMAX>();
        if (active) {
            // ---- softmax of query tile t: one thread to a row
            const int t = warp >> 2;
            const int sw = warp & 3;
            const int r = sw * 32 + lane;
            const unsigned lane_addr = tmem + ((unsigned)(sw * 32) << 16);
            const int rows = t ? range[1].rows : range[0].rows;
            const int first = t ? range[1].first : range[0].first, last = t ? range[1].last : range[0].last;
            const unsigned col_s = COL_S + t * BN;
            float m_used = -INFINITY, l_sum = 0.f;
            const int t0 = qpos_base + tok0 + t * BM;
            const int qpos = t0 + (r < rows ? r : rows - 1);
            const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
            bool ok = true;
            // The exponentials of the two query tiles take turns (turn[t]: tile t may go), so that one tile's
            // softmax has the exponential unit to itself while the tensor core works for the other tile;
            // side by side they would both wait for the unit and then both for the tensor core.
            if (t == 1 && lane == 0) mbar_arrive(&turn[0]);
            for (int j = 0; j < n_tiles; ++j) {
                if (j < first || j >= last) {      // not this tile's keys: pass the turn on
                    ok = __all_sync(0xffffffffu, mbar_wait(&turn[t], j & 1, failed));
                    if (!ok) break;
                    if (lane == 0) mbar_arrive(&turn[t ^ 1]);
                    continue;
                }
                const int k0 = k_start + j * BN;
                const int it = j - first, par = it & 1;
                ok = __all_sync(0xffffffffu, mbar_wait(&s_full[t], par, failed));
                if (!ok) break;
                tc_fence_after();
                unsigned raw[BN];
                tmem_ld<BN>(lane_addr + col_s, raw);
                tmem_wait_ld();
                const bool clear = k0 + BN - 1 <= t0 && (p.window <= 0 || k0 > t0 + rows - 1 - p.window);
                if (!clear) {
#pragma unroll
                    for (int i = 0; i < BN; ++i) {
                        const int kpos = k0 + i;
                        const bool vis = kpos <= qpos && (p.window <= 0 || kpos > qpos - p.window);
                        if (!vis) raw[i] = 0xff800000u;      // -inf
                    }
                }
                float mx[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) mx[i] = __uint_as_float(raw[i]);
#pragma unroll
                for (int i = 8; i < BN; i += 8)
#pragma unroll
                    for (int k = 0; k < 8; ++k) mx[k] = fmaxf(mx[k], __uint_as_float(raw[i + k]));
                const float m_new = fmaxf(m_used, fmaxf(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])), fmaxf(fmaxf(mx[4], mx[5]), fmaxf(mx[6], mx[7]))) * p.scale_log2);
                const bool grow = m_new > m_used + LAG;      // also true for the first keys a row sees
                const float alpha = grow ? ex2(m_used - m_new) : 1.f;
                if (grow) m_used = m_new;
                // the correction warps learn what this row's accumulator shrinks by, and whether any row of the warp does
                const bool any = __any_sync(0xffffffffu, grow);
                tail.alpha[t][par][r] = alpha;
                if (lane == 0) tail.grow_any[t][par][sw] = any ? 1 : 0;
                __syncwarp();
                if (lane == 0) mbar_arrive(&alpha_ready[t]);
                ok = __all_sync(0xffffffffu, mbar_wait(&turn[t], j & 1, failed));
                if (!ok) break;
                l_sum *= alpha;
                const float m_safe = (m_used == -INFINITY) ? 0.f : m_used;
                const float2 nm2 = make_float2(-m_safe, -m_safe);
                float2 la = make_float2(0.f, 0.f), lb = make_float2(0.f, 0.f);
#pragma unroll
                for (int c = 0; c < BN / 32; ++c) {
                    unsigned packed[16];
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        const int k = c * 32 + i;
                        const float2 xa = __ffma2_rn(make_float2(__uint_as_float(raw[k]), __uint_as_float(raw[k + 1])), sc2, nm2);
                        const float2 xb = __ffma2_rn(make_float2(__uint_as_float(raw[k + 2]), __uint_as_float(raw[k + 3])), sc2, nm2);
                        const float2 ea = make_float2(ex2(xa.x), ex2(xa.y)), eb = make_float2(ex2(xb.x), ex2(xb.y));
                        la = __fadd2_rn(la, ea);
                        lb = __fadd2_rn(lb, eb);
                        packed[i / 2] = pack_bf16(ea.x, ea.y);
                        packed[i / 2 + 1] = pack_bf16(eb.x, eb.y);
                    }
                    tmem_st<16>(lane_addr + col_s + c * 16, packed);      // (all scores are in registers: nothing is overwritten unread)
                    if (c == BN / 64 - 1) {          // half of the keys' probabilities are in place
                        tmem_wait_st();
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&p_half[t]);
                    }
                }
                l_sum += (la.x + la.y) + (lb.x + lb.y);
                __syncwarp();
                if (lane == 0) mbar_arrive(&turn[t ^ 1]);
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&p_full[t]);
            }
            if (ok) {
                tail.l_final[t][r] = l_sum;
                __syncwarp();
                if (lane == 0) mbar_arrive(&l_ready[t]);
            } else if (lane == 0) {
                failed_flag = 1;
                atomicExch(p.status, ERR_SOFTMAX_WAIT);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == WR_ISSUE) {
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
// Maps are kept per (pointer, rows, cols, box): page tensors live as long as the engine.
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

// the queries [rows, n_heads, head_dim] bfloat16 as a three-dimensional tensor; box = 128 tokens of one head
// x 64 elements, 128-byte swizzle, zero fill outside
int query_map(CUtensorMap* out, const void* base, long long rows, int n_heads, int head_dim) {
    static std::map<std::tuple<const void*, long long, int, int>, CUtensorMap> cache;
    static std::mutex lock;
    std::lock_guard<std::mutex> guard(lock);
    auto key = std::make_tuple(base, rows, n_heads, head_dim);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return TL_OK;
    }
    EncodeTiledFn fn = encode_tiled();
    if (fn == nullptr) return TL_BAD_SIZE;
    cuuint64_t dims[3] = {(cuuint64_t)head_dim, (cuuint64_t)n_heads, (cuuint64_t)rows};
    cuuint64_t strides[2] = {(cuuint64_t)head_dim * 2, (cuuint64_t)n_heads * head_dim * 2};
    cuuint32_t box[3] = {64u, 1u, (cuuint32_t)BM};
    cuuint32_t elem[3] = {1, 1, 1};
    CUtensorMap m;
    CUresult rc = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, elem,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return TL_BAD_SIZE;
    if (cache.size() > 4096) cache.clear();
    cache[key] = m;
    *out = m;
    return TL_OK;
}

template <int HD> constexpr int stages_for() { return HD == 128 ? 2 : 4; }
template <int HD> constexpr size_t smem_for() {
    return (size_t)(QT + 2 * stages_for<HD>()) * (HD / 64) * BN * 128 + sizeof(Tail<stages_for<HD>()>);
}
static_assert(smem_for<128>() <= 227 * 1024 && smem_for<64>() <= 227 * 1024, "a CTA has 227 KB of shared memory");
static_assert(COL_O + QT * 128 <= TMEM_COLS && COL_S + QT * 128 <= COL_O, "scores and accumulators of the query tiles must fit the tensor memory of a CTA");

bool takes(int n_heads, int n_kv_heads, int head_dim, int page_size) {
    if (head_dim != 64 && head_dim != 128) return false;
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0) return false;
    return page_size >= 1 && (page_size & (page_size - 1)) == 0;           // a power of two
}

bool p_blocks_too_many(int max_q_len) { return (max_q_len + QT * BM - 1) / (QT * BM) > 65535; }

template <int HD> constexpr size_t smem_rows_for() {
    return (size_t)(QT + 2 * stages_for<HD>()) * (HD / 64) * BN * 128 + sizeof(TailRows<stages_for<HD>()>);
}
static_assert(smem_rows_for<128>() <= 227 * 1024 && smem_rows_for<64>() <= 227 * 1024, "a CTA has 227 KB of shared memory");

template <int HD>
int launch_rows(const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mq, const PrefillParams& p, dim3 grid, cudaStream_t s) {
    constexpr size_t smem = smem_rows_for<HD>();
    auto kern = attention_prefill_rows_kernel<HD, stages_for<HD>()>;
    static bool raised = false;
    if (!raised) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        raised = true;
    }
    return (int)tl_launch(kern, grid, dim3(NTHREADS_ROWS), smem, s, mk, mv, mq, p);
}

template <int HD, int PARTS>
int launch(const CUtensorMap& mk, const CUtensorMap& mv, const PrefillParams& p, dim3 grid, cudaStream_t s) {
    constexpr size_t smem = smem_for<HD>();
    auto kern = attention_prefill_kernel<HD, stages_for<HD>(), PARTS>;
    static bool raised = false;
    if (!raised) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        raised = true;
    }
    return (int)tl_launch(kern, grid, dim3(NTHREADS), smem, s, mk, mv, p);
}

}  // namespace

// 1 if this kernel takes the shapes: head_dim 64 or 128 and a page size that is a power of two.
extern "C" int tl_attention_prefill_supports(int n_heads, int n_kv_heads, int head_dim, int page_size) {
    return takes(n_heads, n_kv_heads, head_dim, page_size) ? 1 : 0;
}

// q, out: [q_rows, n_heads, head_dim] bfloat16 (q_rows: all rows of the buffer, n_tokens of them in
// use by the n_seqs requests given); pages: [n_pages, n_kv_heads, page_size, head_dim].
// parts: 1 multiplies every probability as one bfloat16 (the kernel of 512 threads), 2 as bfloat16 value +
// bfloat16 remainder (the kernel of 352 threads: a third slower, half the rounding error).
extern "C" int tl_paged_attention_prefill(const void* q, const void* k_pages, const void* v_pages, void* out,
                                          const int* block_table, int table_stride, const int* q_start,
                                          const int* kv_len, int* status, long long q_rows, int n_tokens, int n_seqs,
                                          int n_heads, int n_kv_heads, int head_dim, int page_size, long long n_pages,
                                          int max_q_len, int window, float scale, int parts, void* stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return TL_OK;
    if (!takes(n_heads, n_kv_heads, head_dim, page_size) || max_q_len <= 0 || n_pages <= 0 || q_rows < n_tokens) return TL_BAD_SIZE;
    if (parts != 1 && parts != 2) return TL_BAD_SIZE;
    if (n_pages * n_kv_heads * page_size >= (1LL << 31)) return TL_BAD_SIZE;
    if (!aligned16(q) || !aligned16(k_pages) || !aligned16(v_pages) || !aligned16(out) || status == nullptr) return TL_BAD_ALIGN;
    if (n_seqs > 65535 || p_blocks_too_many(max_q_len)) return TL_BAD_SIZE;

    PrefillParams p;
    p.q = (const __nv_bfloat16*)q;
    p.out = (__nv_bfloat16*)out;
    p.block_table = block_table; p.q_start = q_start; p.kv_len = kv_len; p.table_stride = table_stride;
    p.status = status;
    p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.page_size = page_size;
    p.page_shift = 0;
    while ((1 << p.page_shift) < page_size) ++p.page_shift;
    p.box_rows = page_size < BN ? page_size : BN;
    p.total_rows = (int)(n_pages * n_kv_heads * page_size);
    p.n_q_blocks = (max_q_len + QT * BM - 1) / (QT * BM);
    p.window = window > 0 ? window : 0;
    p.scale_log2 = scale * LOG2E;

    const long long rows = n_pages * n_kv_heads * page_size;
    CUtensorMap mk, mv;
    int rc = tiled_map(&mk, k_pages, rows, head_dim, p.box_rows);
    if (rc != TL_OK) return rc;
    rc = tiled_map(&mv, v_pages, rows, head_dim, p.box_rows);
    if (rc != TL_OK) return rc;

    dim3 grid(n_heads, p.n_q_blocks, n_seqs);
    cudaStream_t s = (cudaStream_t)stream;
    if (parts == 2) return head_dim == 128 ? launch<128, 2>(mk, mv, p, grid, s) : launch<64, 2>(mk, mv, p, grid, s);
    CUtensorMap mq;
    rc = query_map(&mq, q, q_rows, n_heads, head_dim);
    if (rc != TL_OK) return rc;
    return head_dim == 128 ? launch_rows<128>(mk, mv, mq, p, grid, s) : launch_rows<64>(mk, mv, mq, p, grid, s);
}
