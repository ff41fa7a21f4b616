// C[M, N] = A[M, K] . W[N, K]^T in bfloat16 on the fifth-generation tensor cores, for few rows
// (the projections of a decode step, where the work is streaming W once from HBM).
//
// Both operands are K-major as stored (activations row-major, weights [out, in] as nn.Linear
// keeps them, torchllms/models/networks.py:474-493, :600-602).  The operands are swapped so that
// 128 rows of W fill the 128 rows of a tcgen05.mma and the (padded) tokens are its N:
//   D[w_row, token] = sum_k W[w_row, k] * A[token, k]        -> written out as C[token, w_row].
//
// One CTA computes one 128-row slab of W over one slice of K (split-K): the grid is
// (slabs, splits), so that a narrow projection still puts a CTA or two on every SM.  Splits write
// float32 partial sums C[split, M, N]; the kernels that read them (residual + norm, rope, swiglu)
// add them up, in a fixed order, so nothing is reduced by atomics and results are reproducible.
//
// Inside a CTA (192 threads):
//   warp 0, one lane : TMA producer - cp.async.bulk.tensor (no multicast) of a [128 x 64] tile of W
//                      and a [BQ x 64] tile of A per stage into 128-byte-swizzled shared memory
//   warp 1, one lane : issues tcgen05.mma (M 128, N BQ, K 16; four per stage), accumulator in TMEM,
//                      tcgen05.commit frees the stage and finally signals the epilogue
//   warps 2-5        : epilogue - tcgen05.ld of their 32 TMEM lanes, convert, coalesced stores
// Every mbarrier wait is bounded: on a time-out the CTA records a code in the status word, drains,
// frees its TMEM and returns.
//
// Three forms of the epilogue:
//   plain     partial sums (or, with one split, the product itself) as described above;
//   gated     SwiGLU of a stacked gate/up weight (below);
//   residual  the product is added to the float32 residual stream and prepared for the RMS norm that
//             follows (TransformerBlock, torchllms/models/networks.py:635-644: h = x + attn(..),
//             then ffn_norm(h)).  The K splits of a slab form one thread-block cluster; each CTA
//             sends its partial sums, token by token, into the shared memory of the CTA of the
//             cluster that owns the token (st.async through distributed shared memory, counted by
//             an mbarrier there: plain stores between CTAs of this GPU, no multicast), and every CTA
//             adds up what it receives for its tokens in the order of the splits, rounds the sum to
//             bfloat16 as a product that passes through memory is, adds it to h, and writes h, the
//             weighted but not yet normalised activations bf16(h * norm_weight), and its rows' share
//             of sum(h^2) per token.  The kernels that consume the next product (rotary encoding,
//             the gated epilogue here) multiply by rsqrt(sum / dim + eps): a product is linear in
//             its input, so the scale may follow it.  No partial sum passes through global memory
//             and no norm kernel stands between two products.
#include "common.cuh"
#include <cuda.h>

namespace {

constexpr int BP = 128;          // rows of W per CTA (MMA M)
constexpr int BK = 64;           // K per stage: 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int NTHREADS = 192;
constexpr unsigned long long WAIT_LIMIT_NS = 2000ull * 1000ull * 1000ull;   // two seconds, then give up

enum : int { ERR_TMA_WAIT = 101, ERR_MMA_WAIT = 102, ERR_EPI_WAIT = 103, ERR_REDUCE_WAIT = 104, ERR_SELFTEST_WAIT = 109 };

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// false once limit_ns have passed, or as soon as another role has given up
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity, volatile int* abort_flag,
                                          unsigned long long limit_ns = WAIT_LIMIT_NS) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (unsigned i = 1;; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 0u && (*abort_flag || global_ns() - t0 > limit_ns)) return false;
    }
}

// A wait that nothing will ever satisfy, with a short limit: it must give up, report, and leave the
// context usable.  What the tests run to see that the bounded waits of the kernels do what they say.
__global__ void wait_selftest_kernel(int* status, unsigned long long limit_ns, unsigned long long* waited_ns) {
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned long long t0 = global_ns();
        const bool ok = mbar_wait(&bar, 0, &abort_flag, limit_ns);      // nobody arrives
        *waited_ns = global_ns() - t0;
        if (!ok) atomicExch(status, ERR_SELFTEST_WAIT);
    }
}

// The producer's two instructions are for a whole warp in step, of which one elected lane issues.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, unsigned long long* bar, int x, int y) {
    asm volatile("{\n\t.reg .pred e;\n\telect.sync _|e, 0xffffffff;\n\t"
                 "@e cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n\t}"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
// the same with a cache policy: weights are read once, they should be the first to leave L2
__device__ __forceinline__ unsigned long long policy_evict_first() {
    unsigned long long pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void tma_load_2d_hint(void* dst, const CUtensorMap* map, unsigned long long* bar, int x, int y, unsigned long long pol) {
    asm volatile("{\n\t.reg .pred e;\n\telect.sync _|e, 0xffffffff;\n\t"
                 "@e cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;\n\t}"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "l"(pol) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx_elect(unsigned long long* bar, unsigned bytes) {
    asm volatile("{\n\t.reg .pred e;\n\telect.sync _|e, 0xffffffff;\n\t"
                 "@e mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n\t}" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

// shared-memory matrix descriptor: K-major tile, 128-byte swizzle, rows of 128 bytes, 8-row groups 1024 bytes apart
__device__ __forceinline__ unsigned long long umma_desc(const void* tile, int k_byte_offset) {
    const unsigned addr = smem_u32(tile) + (unsigned)k_byte_offset;
    unsigned long long d = 0;
    d |= (unsigned long long)((addr & 0x3FFFFu) >> 4);           // start address
    d |= (unsigned long long)(0u) << 16;                         // leading byte offset: unused for swizzled K-major
    d |= (unsigned long long)(1024u >> 4) << 32;                 // stride byte offset between 8-row groups
    d |= (unsigned long long)1u << 46;                           // descriptor version of this architecture
    d |= (unsigned long long)2u << 61;                           // layout: 128-byte swizzle
    return d;
}

// instruction descriptor: bf16 x bf16 -> f32, both K-major, M = 128, N = n
__host__ __device__ constexpr unsigned umma_idesc(int n) {
    return (1u << 4)                  // accumulator format: f32
         | (1u << 7)                  // a format: bf16
         | (1u << 10)                 // b format: bf16
         | ((unsigned)(n >> 3) << 17)
         | ((unsigned)(BP >> 4) << 24);
}

// Both for a whole warp in step, of which one elected lane issues: the descriptors then stay warp-uniform
// values (a lone lane inside a divergent branch cannot have those).
__device__ __forceinline__ void umma_bf16(unsigned tmem_d, unsigned long long a_desc, unsigned long long b_desc,
                                          unsigned idesc, unsigned accumulate) {
    asm volatile("{\n\t.reg .pred p, e;\n\telect.sync _|e, 0xffffffff;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
    asm volatile("{\n\t.reg .pred e;\n\telect.sync _|e, 0xffffffff;\n\t"
                 "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(smem_u32(bar)) : "memory");
}

// ---- distributed shared memory: addresses of the same variable in another CTA of the cluster, and
// a store there that counts its bytes on an mbarrier there when it has landed
__device__ __forceinline__ unsigned cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ unsigned map_to_cta(unsigned local_addr, unsigned rank) {
    unsigned remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    return remote;
}
__device__ __forceinline__ void st_async_f32(unsigned remote_addr, float v, unsigned remote_bar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];"
                 ::"r"(remote_addr), "r"(__float_as_uint(v)), "r"(remote_bar) : "memory");
}
// The cluster's barrier in two halves: every thread arrives once and waits once, possibly much later.
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

template <int N> struct TmemLoad;
template <> struct TmemLoad<16> {
    __device__ static __forceinline__ void run(unsigned taddr, unsigned (&r)[16]) {
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                     : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                       "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                     : "r"(taddr));
    }
};

struct GemmParams {
    void* out;              // [splits, M, N], float32 or bfloat16 (bfloat16 only with one split)
    int* status;            // error word (may live in mapped host memory)
    int M, N, K;
    int k_blocks_per_split; // stages each split walks
    int out_is_f32;
    int hidden;             // gated form: W is [2 * hidden, K], gate rows above up rows; out is [M, hidden] bfloat16
    // gated form, optional: the input rows were not normalised yet; gate and up are multiplied by
    // rsqrt(sum_p in_ssq[tok, p] * in_inv_dim + in_eps) before the activation
    const float* in_ssq;
    int in_parts;
    float in_inv_dim, in_eps;
    // residual form
    int splits;             // = CTAs of a cluster
    float* h;               // [M, N] residual stream, updated in place
    const float* norm_w;    // [N]
    __nv_bfloat16* xw;      // [M, N]: bf16(h * norm_w)
    float* ssq;             // [M, 4 * slabs]: the share of sum(h^2) of every 32 columns
};

enum : int { MODE_PLAIN = 0, MODE_GATED = 1, MODE_RESID = 2 };

// GATED: the slab is 64 rows of the gate projection and the 64 matching rows of the up projection
// (two TMA boxes per stage), and the epilogue writes silu(gate) * up in bfloat16: the SwiGLU costs
// no kernel and no round trip of the projections through memory.  One K split only.
template <int BQ, int STAGES, int MODE>
__global__ void __launch_bounds__(NTHREADS) gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                const __grid_constant__ CUtensorMap map_a,
                                                                const GemmParams p) {
    constexpr unsigned W_BYTES = BP * BK * 2, A_BYTES = BQ * BK * 2;
    constexpr unsigned STAGE_BYTES = W_BYTES + A_BYTES;
    constexpr unsigned TMEM_COLS = BQ < 32 ? 32 : BQ;
    extern __shared__ unsigned char smem_raw[];
    // tiles want 1024-byte alignment for the 128-byte swizzle
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~uintptr_t(1023));
    __shared__ __align__(8) unsigned long long full_bar[STAGES];
    __shared__ __align__(8) unsigned long long empty_bar[STAGES];
    __shared__ __align__(8) unsigned long long accum_bar;
    __shared__ unsigned tmem_base_slot;
    __shared__ int abort_flag;
    __shared__ __align__(8) unsigned long long red_bar;      // residual form: counts the bytes other CTAs send here
    __shared__ __align__(16) float rstd_s[BQ];
    constexpr bool GATED = MODE == MODE_GATED;
    constexpr bool CLUSTERED = MODE == MODE_RESID;     // the K splits of a slab are one cluster

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int slab = blockIdx.x, split = blockIdx.y;
    const int total_k_blocks = (p.K + BK - 1) / BK;
    const int kb0 = split * p.k_blocks_per_split;
    const int n_kb = max(0, min(p.k_blocks_per_split, total_k_blocks - kb0));

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&accum_bar, 1);
        if (CLUSTERED) mbar_init(&red_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_d = tmem_base_slot;
    volatile int* aborted = &abort_flag;
    // residual form: this CTA is split `rank` of its slab's cluster and owns the tokens rank, rank + S, ..:
    // n_owned of them, each arriving as one row of 128 floats from every split
    const int S = CLUSTERED ? p.splits : 1;
    const int rank = CLUSTERED ? (int)cluster_rank() : 0;
    const int n_owned = (CLUSTERED && p.M > rank) ? (p.M - rank - 1) / S + 1 : 0;
    float* red = reinterpret_cast<float*>(tiles + STAGES * STAGE_BYTES);     // [owned token][split][row of the slab]
    if (CLUSTERED) {
        // Every CTA's barrier must be set up before anybody sends to it.  The threads only say here that
        // theirs is; each waits for the others where it needs them (the epilogue before it sends, the two
        // other roles when they are done), so that the weights start to stream before the whole cluster
        // is on the machine.
        if (threadIdx.x == 0) mbar_expect_tx(&red_bar, (unsigned)(n_owned * S * BP * 4));
        cluster_arrive();
    }
    grid_launch_dependents();

    if (warp == 0) {
        {
            // ---- producer (the whole warp in step, one elected lane issuing).  The weights depend on no
            // earlier kernel: their first tiles are fetched before the dependency on the predecessor is
            // resolved, the activations after it.
            const int pre = n_kb < STAGES ? n_kb : STAGES;
            // With more than 16 tokens the weights are marked to leave L2 first: the tokens' tiles, which
            // every slab reads again, and the partial sums then stay (w2 with 64 tokens: 24.3 -> 21.8 us; with
            // 8 tokens a step was 2 % slower with the mark, so it is not set there).
            const bool mark = p.M > 16;
            const unsigned long long pol = policy_evict_first();
            auto load_one = [&](unsigned char* dst, unsigned long long* bar, int x, int y) {
                if (mark) tma_load_2d_hint(dst, &map_w, bar, x, y, pol);
                else tma_load_2d(dst, &map_w, bar, x, y);
            };
            auto load_w = [&](unsigned char* dst, unsigned long long* bar, int kb) {
                if (GATED) {
                    load_one(dst, bar, kb * BK, slab * (BP / 2));
                    load_one(dst + (BP / 2) * BK * 2, bar, kb * BK, p.hidden + slab * (BP / 2));
                } else {
                    load_one(dst, bar, kb * BK, slab * BP);
                }
            };
            for (int i = 0; i < pre; ++i) {
                mbar_expect_tx_elect(&full_bar[i], STAGE_BYTES);
                load_w(tiles + i * STAGE_BYTES, &full_bar[i], kb0 + i);
            }
            grid_dependency_wait();
            for (int i = 0; i < pre; ++i)
                tma_load_2d(tiles + i * STAGE_BYTES + W_BYTES, &map_a, &full_bar[i], (kb0 + i) * BK, 0);
            for (int i = pre; i < n_kb; ++i) {
                const int s = i % STAGES;
                if (!__all_sync(0xffffffffu, mbar_wait(&empty_bar[s], ((i / STAGES) - 1) & 1, aborted))) {
                    if (lane == 0) {
                        abort_flag = 1;
                        atomicExch(p.status, ERR_TMA_WAIT);
                    }
                    break;
                }
                unsigned char* wt = tiles + s * STAGE_BYTES;
                mbar_expect_tx_elect(&full_bar[s], STAGE_BYTES);
                load_w(wt, &full_bar[s], kb0 + i);
                tma_load_2d(wt + W_BYTES, &map_a, &full_bar[s], (kb0 + i) * BK, 0);
            }
        }
        __syncwarp();
        if (CLUSTERED) cluster_wait();
    } else if (warp == 1) {
        {
            // ---- tensor-core issuer: the whole warp in step, one elected lane issuing
            constexpr unsigned idesc = umma_idesc(BQ);
            bool ok = true;
            for (int i = 0; i < n_kb && ok; ++i) {
                const int s = i % STAGES;
                if (!__all_sync(0xffffffffu, mbar_wait(&full_bar[s], (i / STAGES) & 1, aborted))) {
                    if (lane == 0) {
                        abort_flag = 1;
                        atomicExch(p.status, ERR_MMA_WAIT);
                    }
                    ok = false;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                unsigned char* wt = tiles + s * STAGE_BYTES;
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)
                    umma_bf16(tmem_d, umma_desc(wt, k * UMMA_K * 2), umma_desc(wt + W_BYTES, k * UMMA_K * 2), idesc,
                              (i > 0 || k > 0) ? 1u : 0u);
                umma_commit(&empty_bar[s]);      // the stage is free once these MMAs have read it
            }
            if (ok) umma_commit(&accum_bar);     // everything issued so far has landed in TMEM
        }
        __syncwarp();
        if (CLUSTERED) cluster_wait();
    } else {
        // ---- epilogue: warp w owns TMEM lanes 32 * (w % 4) .. + 31, i.e. rows of W of this slab
        const int quarter = warp & 3;
        const int w_row = slab * BP + quarter * 32 + lane;
        bool ok = true;
        if (GATED) {
            // the scale of every token's row, while the products run
            if (p.in_ssq != nullptr) {
                grid_dependency_wait();
                for (int tok = quarter; tok < BQ; tok += 4) {
                    float v = 0.f;
                    if (tok < p.M)
                        for (int q = lane; q < p.in_parts; q += 32) v += __ldcg(p.in_ssq + (size_t)tok * p.in_parts + q);
                    v = warp_sum(v);
                    if (lane == 0) rstd_s[tok] = rsqrtf(v * p.in_inv_dim + p.in_eps);
                }
            } else {
                for (int tok = quarter * 32 + lane; tok < BQ; tok += 128) rstd_s[tok] = 1.f;
            }
        }
        // residual form: what this CTA's own tokens need besides the sums (their rows of the stream, the
        // norm's weight) is fetched now, while the products run
        constexpr int AHEAD = 4;
        const int own_row = quarter * 32 + lane;
        const int own_col = slab * BP + own_row;
        float pre_h[AHEAD], pre_nw = 0.f;
        if (CLUSTERED && n_owned > 0) {
            grid_dependency_wait();
            if (own_col < p.N) pre_nw = p.norm_w[own_col];
#pragma unroll
            for (int slot = 0; slot < AHEAD; ++slot)
                pre_h[slot] = (slot < n_owned && own_col < p.N) ? p.h[(size_t)(slot * S + rank) * p.N + own_col] : 0.f;
        }
        if (n_kb > 0) {
            ok = mbar_wait(&accum_bar, 0, aborted);
            if (!ok && lane == 0) {
                abort_flag = 1;
                atomicExch(p.status, ERR_EPI_WAIT);
            }
        }
        ok = __all_sync(0xffffffffu, ok);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (GATED) {
            // Rows 0-63 of the accumulator are gates, rows 64-127 the matching ups.  The ups go through
            // shared memory (the stages are done with: every product has finished) to the threads
            // that hold the gates.  All four warps keep the appointment at the barrier, failed or not.
            float* xch = reinterpret_cast<float*>(tiles);              // [64][BQ + 1]
            const int row = quarter * 32 + lane;
            if (ok && n_kb > 0 && row >= BP / 2) {
#pragma unroll
                for (int c0 = 0; c0 < BQ; c0 += 16) {
                    unsigned r[16];
                    TmemLoad<16>::run(tmem_d + ((unsigned)(quarter * 32) << 16) + (unsigned)c0, r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int j = 0; j < 16; ++j) xch[(row - BP / 2) * (BQ + 1) + c0 + j] = __uint_as_float(r[j]);
                }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (ok && row < BP / 2) {
                const int f = slab * (BP / 2) + row;                   // column of the output
#pragma unroll
                for (int c0 = 0; c0 < BQ; c0 += 16) {
                    unsigned r[16];
                    if (n_kb > 0) TmemLoad<16>::run(tmem_d + ((unsigned)(quarter * 32) << 16) + (unsigned)c0, r);
                    // the sixteen tokens' scales in four loads, under way while the accumulator is fetched (one
                    // load per element behind the wait cost 2 us with 64 tokens)
                    float scales[16];
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        const float4 v = *reinterpret_cast<const float4*>(&rstd_s[c0 + 4 * q4]);
                        scales[4 * q4] = v.x; scales[4 * q4 + 1] = v.y; scales[4 * q4 + 2] = v.z; scales[4 * q4 + 3] = v.w;
                    }
                    if (n_kb > 0) {
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) r[j] = 0u;
                    }
                    if (f < p.hidden) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int tok = c0 + j;
                            if (tok < p.M) {
                                // (rounded to bfloat16 first, as they are when they pass through memory:
                                // this form and the two-kernel form give the same numbers)
                                const float sc = scales[j];
                                const float g = __bfloat162float(__float2bfloat16_rn(__uint_as_float(r[j]))) * sc;
                                const float u = __bfloat162float(__float2bfloat16_rn(n_kb > 0 ? xch[row * (BQ + 1) + tok] : 0.f)) * sc;
                                reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)tok * p.hidden + f] =
                                    __float2bfloat16_rn(__fdividef(g, 1.f + __expf(-g)) * u);
                            }
                        }
                    }
                }
            }
        } else if (CLUSTERED) {
            // Every token's partial sums go to the CTA of the cluster that owns the token (token mod S),
            // one row of the slab per thread; the store counts itself on the owner's barrier when it
            // has landed.  A CTA whose waits did not hold sends nothing: its owners' waits run out in
            // turn and say so.
            const int row = quarter * 32 + lane;
            cluster_wait();          // the owners' barriers are set up
            if (ok) {
                const unsigned red_addr = smem_u32(red), bar_addr = smem_u32(&red_bar);
#pragma unroll
                for (int c0 = 0; c0 < BQ; c0 += 16) {
                    unsigned r[16];
                    TmemLoad<16>::run(tmem_d + ((unsigned)(quarter * 32) << 16) + (unsigned)c0, r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int tok = c0 + j;
                        if (tok < p.M) {
                            const unsigned owner = (unsigned)(tok % S);
                            const unsigned slot = (unsigned)(tok / S);
                            st_async_f32(map_to_cta(red_addr + ((slot * S + split) * BP + row) * 4u, owner), __uint_as_float(r[j]),
                                         map_to_cta(bar_addr, owner));
                        }
                    }
                }
            }
            if (MODE == MODE_RESID && n_owned > 0) {
                const int col = own_col;
                const float nw = pre_nw;
                bool got = mbar_wait(&red_bar, 0, aborted);
                if (!got && lane == 0) {
                    abort_flag = 1;
                    atomicExch(p.status, ERR_REDUCE_WAIT);
                }
                got = __all_sync(0xffffffffu, got);
                if (got) {
#pragma unroll 1
                    for (int slot = 0; slot < n_owned; ++slot) {
                        const int tok = slot * S + rank;
                        float acc = 0.f;
                        for (int sp = 0; sp < S; ++sp) acc += red[(slot * S + sp) * BP + row];      // in the order of the splits
                        float hv = 0.f;
                        float h_old = 0.f;
#pragma unroll
                        for (int a = 0; a < AHEAD; ++a) if (a == slot) h_old = pre_h[a];
                        if (slot >= AHEAD && col < p.N) h_old = p.h[(size_t)tok * p.N + col];
                        if (col < p.N) {
                            // the product enters the stream as it does when it passes through memory in
                            // bfloat16 (prompt portions, whose products the library takes): one arithmetic
                            // however a request is cut into steps
                            hv = h_old + __bfloat162float(__float2bfloat16_rn(acc));
                            p.h[(size_t)tok * p.N + col] = hv;
                            p.xw[(size_t)tok * p.N + col] = __float2bfloat16_rn(hv * nw);
                        }
                        const float ss = warp_sum(hv * hv);
                        if (lane == 0) p.ssq[(size_t)tok * (gridDim.x * 4) + slab * 4 + quarter] = ss;
                    }
                }
            }
        } else if (ok) {
            const size_t plane = (size_t)p.M * p.N;
#pragma unroll
            for (int c0 = 0; c0 < BQ; c0 += 16) {
                unsigned r[16];
                if (n_kb > 0) {
                    TmemLoad<16>::run(tmem_d + ((unsigned)(quarter * 32) << 16) + (unsigned)c0, r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) r[j] = 0u;
                }
                if (w_row < p.N) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int tok = c0 + j;
                        if (tok < p.M) {
                            const float v = __uint_as_float(r[j]);
                            const size_t at = (size_t)split * plane + (size_t)tok * p.N + w_row;
                            if (p.out_is_f32) reinterpret_cast<float*>(p.out)[at] = v;
                            else reinterpret_cast<__nv_bfloat16*>(p.out)[at] = __float2bfloat16_rn(v);
                        }
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(TMEM_COLS) : "memory");
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

// rows x K bf16, row-major; box = box_rows x 64 elements, 128-byte swizzle, zero fill outside
int make_map(CUtensorMap* map, const void* base, long long rows, long long K, int box_rows) {
    EncodeTiledFn fn = encode_tiled();
    if (fn == nullptr) return TL_BAD_SIZE;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult rc = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return rc == CUDA_SUCCESS ? TL_OK : TL_BAD_SIZE;
}


int tl_gemm_tcgen05_splits_impl(int M, int N, int K) {
    // Two CTAs fit an SM; all CTAs of a launch should be resident at once (one wave), because a
    // second, partly filled wave streams at a fraction of the bandwidth.  So: as many splits as
    // keep slabs * splits within 2 * 148, each with at least four stages of work.  (Fewer splits
    // for the wider token buckets, to save the float32 partial sums' traffic, measured slower: the
    // CTAs they would save are what keeps the stream busy.)  M is taken so that this can change.
    const int slabs = (N + BP - 1) / BP;
    const int k_blocks = (K + BK - 1) / BK;
    int splits = (2 * 148) / slabs;
    const int most = k_blocks / 4 > 0 ? k_blocks / 4 : 1;
    if (splits > most) splits = most;
    (void)M;
    if (splits < 1) splits = 1;
    const int per = (k_blocks + splits - 1) / splits;
    return (k_blocks + per - 1) / per;                          // no empty split
}

template <int BQ, int STAGES, int MODE = MODE_PLAIN>
int launch(const CUtensorMap& mw, const CUtensorMap& ma, const GemmParams& p, int slabs, int splits, cudaStream_t s) {
    // the residual form keeps, behind the stages, the rows that the other CTAs of its cluster send it
    constexpr size_t red_bytes = MODE == MODE_RESID ? (size_t)(BQ + 8) * BP * 4 : 0;
    constexpr size_t smem = (size_t)STAGES * (BP * BK * 2 + BQ * BK * 2) + red_bytes + 1024;
    static_assert(MODE != MODE_GATED || (size_t)64 * (BQ + 1) * 4 <= (size_t)STAGES * (BP * BK * 2 + BQ * BK * 2), "the ups pass through the stages' memory");
    auto kern = gemm_tcgen05_kernel<BQ, STAGES, MODE>;
    static bool raised = false;
    if (!raised) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        raised = true;
    }
    if (MODE == MODE_RESID) {
        // the splits of a slab as one cluster (at most 8 CTAs, the portable size)
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(slabs, splits);
        cfg.blockDim = dim3(NTHREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = s;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = 1;
        attr[1].val.clusterDim.y = (unsigned)splits;
        attr[1].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 2;
        return (int)cudaLaunchKernelEx(&cfg, kern, mw, ma, p);
    }
    return (int)tl_launch(kern, dim3(slabs, splits), dim3(NTHREADS), smem, s, mw, ma, p);
}

// K splits of the residual form: as the plain form has them, but no more than a cluster holds.
// (Measured at batch 8 on the 8B shape, a step with clusters of 8 / 7 / 6 / 4 CTAs: 3.25 / 3.25 /
// 3.28 / 3.39 ms.)
int clustered_splits(int M, int N, int K) {
    int splits = tl_gemm_tcgen05_splits_impl(M, N, K);
    if (splits > 8) splits = 8;
    const int k_blocks = (K + BK - 1) / BK;
    const int per = (k_blocks + splits - 1) / splits;
    return (k_blocks + per - 1) / per;            // no empty split
}

}  // namespace

// Launches a kernel whose only wait can never be satisfied and gives up after limit_ns (at most a
// second): the status word receives code 109, waited_ns (device memory) the time the wait took.
extern "C" int tl_wait_selftest(int* status, unsigned long long limit_ns, unsigned long long* waited_ns, void* stream) {
    if (status == nullptr || waited_ns == nullptr || limit_ns == 0 || limit_ns > 1000ull * 1000ull * 1000ull) return TL_BAD_SIZE;
    return (int)tl_launch(wait_selftest_kernel, dim3(1), dim3(32), 0, (cudaStream_t)stream, status, limit_ns, waited_ns);
}

// How many K splits the kernel uses for M rows against a [N, K] weight.
extern "C" int tl_gemm_tcgen05_splits(int M, int N, int K) { return tl_gemm_tcgen05_splits_impl(M, N, K); }

// 1 if the kernel takes this problem: at most 64 rows, K a multiple of 8 (TMA wants 16-byte row
// pitches), operands 16-byte aligned.
extern "C" int tl_gemm_tcgen05_supports(int M, int N, int K) {
    return (M >= 1 && M <= 64 && N >= 1 && K >= 8 && K % 8 == 0) ? 1 : 0;
}

// A: [M, K] bf16, W: [N, K] bf16, out: [splits, M, N] with splits = tl_gemm_tcgen05_splits(M, N, K);
// float32 when out_is_f32, else bfloat16 (then splits must be 1).  status: one int the kernel sets
// to a non-zero code if a wait ran out (it then leaves its output unwritten).
extern "C" int tl_gemm_tcgen05(const void* A, const void* W, void* out, int out_is_f32, int M, int N, int K,
                               int splits, int* status, void* stream) {
    if (M <= 0 || N <= 0) return TL_OK;
    if (!tl_gemm_tcgen05_supports(M, N, K)) return TL_BAD_SIZE;
    if (!aligned16(A) || !aligned16(W) || !aligned16(out) || status == nullptr) return TL_BAD_ALIGN;
    if (splits != tl_gemm_tcgen05_splits(M, N, K)) return TL_BAD_SIZE;
    if (!out_is_f32 && splits != 1) return TL_BAD_SIZE;
    const int slabs = (N + BP - 1) / BP;
    const int k_blocks = (K + BK - 1) / BK;
    const int bq = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    CUtensorMap mw, ma;
    int rc = make_map(&mw, W, N, K, BP);
    if (rc != TL_OK) return rc;
    rc = make_map(&ma, A, M, K, bq);
    if (rc != TL_OK) return rc;
    GemmParams p = {};
    p.out = out; p.status = status; p.M = M; p.N = N; p.K = K;
    p.k_blocks_per_split = (k_blocks + splits - 1) / splits;
    p.out_is_f32 = out_is_f32;
    p.hidden = 0;
    p.splits = splits;
    cudaStream_t s = (cudaStream_t)stream;
    if (bq == 16) return launch<16, 6>(mw, ma, p, slabs, splits, s);
    if (bq == 32) return launch<32, 5>(mw, ma, p, slabs, splits, s);
    return launch<64, 4>(mw, ma, p, slabs, splits, s);
}

// 1 if the residual form takes this problem: what tl_gemm_tcgen05 takes.
extern "C" int tl_gemm_tcgen05_residual_supports(int M, int N, int K) { return tl_gemm_tcgen05_supports(M, N, K); }

// Width of `ssq` for a weight of N rows: one part per 32 columns of every 128-row slab.
extern "C" int tl_gemm_tcgen05_residual_parts(int N) { return 4 * ((N + BP - 1) / BP); }

// h[M, N] += bf16(A[M, K] . W[N, K]^T) (float32, in place); xw[M, N] = bf16(h * norm_w);
// ssq[M, tl_gemm_tcgen05_residual_parts(N)] = the parts of every row's sum of h^2 (all of them are
// written, zeros beyond N).  No scratch memory: the K splits of a slab are one cluster and add up
// through shared memory.
extern "C" int tl_gemm_tcgen05_residual(const void* A, const void* W, float* h, const float* norm_w, void* xw, float* ssq,
                                        int M, int N, int K, int* status, void* stream) {
    if (M <= 0 || N <= 0) return TL_OK;
    if (!tl_gemm_tcgen05_residual_supports(M, N, K)) return TL_BAD_SIZE;
    if (!aligned16(A) || !aligned16(W) || !aligned16(h) || !aligned16(norm_w) || !aligned16(xw) || status == nullptr || ssq == nullptr)
        return TL_BAD_ALIGN;
    const int slabs = (N + BP - 1) / BP;
    const int k_blocks = (K + BK - 1) / BK;
    const int bq = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    const int splits = clustered_splits(M, N, K);
    CUtensorMap mw, ma;
    int rc = make_map(&mw, W, N, K, BP);
    if (rc != TL_OK) return rc;
    rc = make_map(&ma, A, M, K, bq);
    if (rc != TL_OK) return rc;
    GemmParams p = {};
    p.status = status; p.M = M; p.N = N; p.K = K;
    p.k_blocks_per_split = (k_blocks + splits - 1) / splits;
    p.out_is_f32 = 1;
    p.splits = splits;
    p.h = h; p.norm_w = norm_w; p.xw = (__nv_bfloat16*)xw; p.ssq = ssq;
    cudaStream_t s = (cudaStream_t)stream;
    // (a stage less than the plain form: the rows that the cluster sends need their room)
    if (bq == 16) return launch<16, 5, MODE_RESID>(mw, ma, p, slabs, splits, s);
    if (bq == 32) return launch<32, 4, MODE_RESID>(mw, ma, p, slabs, splits, s);
    return launch<64, 3, MODE_RESID>(mw, ma, p, slabs, splits, s);
}


// 1 if the gated form takes this problem (W is [2 * hidden, K]) and is the better choice: what
// tl_gemm_tcgen05 takes, hidden a multiple of 64, and a shape that the plain form would not split
// over K either (a split has no whole sums to gate).
extern "C" int tl_gemm_tcgen05_gated_supports(int M, int hidden, int K) {
    if (hidden <= 0 || hidden % (BP / 2) != 0) return 0;
    if (!tl_gemm_tcgen05_supports(M, 2 * hidden, K)) return 0;
    return tl_gemm_tcgen05_splits(M, 2 * hidden, K) == 1 ? 1 : 0;
}

// out[M, hidden] (bfloat16) = silu(s . A . W[:hidden]^T) * (s . A . W[hidden:]^T), A: [M, K] bf16, W: [2 * hidden, K] bf16.
// s is one scale per row of A: 1 when in_ssq is null, else rsqrt(sum_p in_ssq[row, p] * in_inv_dim + in_eps)
// (rows that were weighted for an RMS norm but not normalised yet).
// Any hidden that is a multiple of 64 is computed correctly; tl_gemm_tcgen05_gated_supports says when
// it is also the faster way.
extern "C" int tl_gemm_tcgen05_gated(const void* A, const void* W, void* out, int M, int hidden, int K,
                                     const float* in_ssq, int in_parts, float in_inv_dim, float in_eps, int* status,
                                     void* stream) {
    if (M <= 0 || hidden <= 0) return TL_OK;
    if (hidden % (BP / 2) != 0 || !tl_gemm_tcgen05_supports(M, 2 * hidden, K)) return TL_BAD_SIZE;
    if (!aligned16(A) || !aligned16(W) || !aligned16(out) || status == nullptr) return TL_BAD_ALIGN;
    const int slabs = hidden / (BP / 2);
    const int bq = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    CUtensorMap mw, ma;
    int rc = make_map(&mw, W, 2LL * hidden, K, BP / 2);
    if (rc != TL_OK) return rc;
    rc = make_map(&ma, A, M, K, bq);
    if (rc != TL_OK) return rc;
    if (in_ssq != nullptr && in_parts < 1) return TL_BAD_SIZE;
    GemmParams p = {};
    p.out = out; p.status = status; p.M = M; p.N = 2 * hidden; p.K = K;
    p.k_blocks_per_split = (K + BK - 1) / BK;
    p.out_is_f32 = 0;
    p.hidden = hidden;
    p.splits = 1;
    p.in_ssq = in_ssq; p.in_parts = in_parts; p.in_inv_dim = in_inv_dim; p.in_eps = in_eps;
    cudaStream_t s = (cudaStream_t)stream;
    if (bq == 16) return launch<16, 6, MODE_GATED>(mw, ma, p, slabs, 1, s);
    if (bq == 32) return launch<32, 5, MODE_GATED>(mw, ma, p, slabs, 1, s);
    return launch<64, 4, MODE_GATED>(mw, ma, p, slabs, 1, s);
}
