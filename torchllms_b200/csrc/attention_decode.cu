// Decode attention over paged bfloat16 keys and values with TMA-fed tiles (head_dim 64 or 128).
//
// For steps where every request brings so few tokens that its rows (token x query heads of one kv
// group) fit one 16-row tensor-core tile: single decoded tokens above all.  Same contract and
// the same arithmetic as the kernels in attention_mma.cu (float32 scores, running maximum and
// sum, accumulators; probabilities multiplied as value + remainder), but the tiles are moved by
// the TMA unit instead of by every thread: the decode step is bound by streaming K and V once
// from HBM, and issuing 16-byte copies from all threads cost more instructions than the math.
//
// A CTA serves one (request, kv head, key split).  Warp 4 is the producer: for every 64-key tile it
// looks up the pages, and issues cp.async.bulk.tensor copies (no multicast) of [page rows x 64
// elements] boxes into 128-byte-swizzled shared memory, completing on an mbarrier per stage.
// Warps 0-3 share the rows and each takes 16 keys of every tile; they hand a stage back through a
// second mbarrier.  No CTA-wide barrier is used until the four partial results are merged.  Key
// splits over CTAs write float32 partials that merge_partials_kernel combines.
//
// The products are taken transposed: scores^T = K Q^T and out^T = V^T P^T, so that the 16 rows of
// a tensor-core tile are keys (or value columns), all of them real, and the few query rows (four
// for a group of four heads) sit in the 8-wide direction.  With the queries as the 16 rows, three
// quarters of every product were padding, and instruction issue, not memory, set the pace.  The
// probabilities change sides between the two products (result columns -> operand columns),
// which is one movmatrix per 8 x 8 block.
// Every mbarrier wait is bounded in time; on a time-out the CTA records a code in the status
// word, writes nothing and returns.
#include "common.cuh"
#include <cuda.h>
#include <limits.h>
#include <math.h>
#include <map>
#include <mutex>
#include <tuple>

namespace {

constexpr int BN = 64;                  // keys per tile
constexpr int NCW = 4;                  // consumer warps
constexpr int NTHREADS = (NCW + 1) * 32;
constexpr int MIN_SPLIT = 128;
constexpr int MERGE_MAX_SPLITS = 64;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;
constexpr unsigned long long WAIT_NS = 2000ull * 1000ull * 1000ull;
enum : int { ERR_PRODUCER_WAIT = 211, ERR_CONSUMER_WAIT = 212 };

struct DecodeParams {
    const __nv_bfloat16* q;
    __nv_bfloat16* out;
    const int* block_table;
    const int* q_start;
    const int* kv_len;
    float* part_o;   // [T * H, n_splits, head_dim]
    float* part_ml;  // [T * H, n_splits, 2]
    int* status;
    int table_stride;
    int n_heads, n_kv_heads, page_size, page_shift, box_rows;
    int total_rows;             // rows of the page tensor: a copy that starts there reads only the zero fill
    int group, ng, n_gchunks, tpw;
    int window;
    int streamed;               // the call reads more keys and values than L2 holds: their copies are marked to leave it first
    int n_splits;
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
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, unsigned long long* bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
// the same with the mark "first to leave L2": keys and values that are read once and are more than L2 holds
__device__ __forceinline__ void tma_load_2d_streamed(void* dst, const CUtensorMap* map, unsigned long long* bar, int x, int y) {
    unsigned long long pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "l"(pol) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float ex2(float x) {     // 2^x, one instruction; 2^-inf = 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}
// byte offset of (row, 16-byte chunk c of a 128-byte row) inside a 128-byte-swizzled [rows x 128 B] tile
__device__ __forceinline__ unsigned swz(int row, int c) { return (unsigned)(row * 128 + ((c ^ (row & 7)) << 4)); }

__device__ __forceinline__ unsigned movmatrix_trans(unsigned a) {     // 8 x 8 bfloat16 block, transposed across the warp
    unsigned d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}

// NT: 8-row blocks of query rows (1: up to 8 rows, 2: up to 16)
template <int HD, int STAGES, int NT>
__global__ void __launch_bounds__(NTHREADS, NT == 1 ? 3 : 2) attention_decode_kernel(const __grid_constant__ CUtensorMap map_k,
                                                                                  const __grid_constant__ CUtensorMap map_v,
                                                                                  const DecodeParams p) {
    constexpr int HALVES = HD / 64;                     // 64-element (128-byte) column blocks of a row
    constexpr unsigned HALF_BYTES = BN * 128;           // one [64 keys x 128 B] block
    constexpr unsigned KV_BYTES = HALVES * HALF_BYTES;  // K (or V) of a tile
    constexpr unsigned STAGE_BYTES = 2 * KV_BYTES;
    constexpr int QPITCH = HD + 8;
    constexpr int KSTEPS = HD / 16;
    constexpr int NROWS = 8 * NT;
    constexpr int OPITCH = HD + 4;                      // of the merge buffer: rows two apart fall on different banks
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~uintptr_t(1023));
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(tiles + STAGES * STAGE_BYTES);   // [16][QPITCH]
    __shared__ __align__(8) unsigned long long full_bar[STAGES];
    __shared__ __align__(8) unsigned long long empty_bar[STAGES];
    __shared__ int failed_flag;

    grid_launch_dependents();
    // What follows, down to the dependency wait, reads nothing that the kernels just before this one
    // write: the step's index data were uploaded before its first kernel, and keys and values of
    // positions before the step's own tokens were written by earlier steps.  Under programmatic
    // dependent launch this part runs while the predecessor is still at work.
    const int b = blockIdx.z;
    const int qs = p.q_start[b];
    const int ql = p.q_start[b + 1] - qs;
    const int kl = p.kv_len[b];
    const int tile = blockIdx.x / p.n_splits;
    const int split = blockIdx.x - tile * p.n_splits;
    const int tok0 = tile * p.tpw;
    if (tok0 >= ql) return;
    const int kvh = blockIdx.y / p.n_gchunks;
    const int g0 = (blockIdx.y - kvh * p.n_gchunks) * p.ng;
    const int ng = min(p.ng, p.group - g0);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    volatile int* failed = &failed_flag;

    // ---- which keys this CTA walks: its share of the request's visible keys, in whole tiles
    const int cta_tok_hi = min(ql, tok0 + p.tpw);
    const int qpos_base = kl - ql;
    int k_lo = p.window > 0 ? max(0, qpos_base + tok0 - p.window + 1) : 0;
    int k_hi = qpos_base + cta_tok_hi;
    if (p.n_splits > 1) {
        const int len = max(k_hi - k_lo, 0);
        const int chunk = ((len + p.n_splits - 1) / p.n_splits + BN - 1) / BN * BN;
        const int lo = k_lo + split * chunk;
        k_hi = min(k_hi, lo + chunk);
        k_lo = lo;
    }
    const int k_start = k_lo & ~(p.box_rows - 1);      // copies start on a box (page) boundary; keys below k_lo are masked
    const int n_tiles = k_hi > k_start ? (k_hi - k_start + BN - 1) / BN : 0;
    const int* table = p.block_table + (size_t)b * p.table_stride;

    // one tile: a box per page (or per 64 rows of a larger page) and 64-element column block, K and V.
    // The whole producer warp issues it, a lane to a box: the page lookups go side by side.
    auto issue_tile = [&](int it) {
        const int s = it % STAGES;
        const int k0 = k_start + it * BN;
        if (lane == 0) mbar_expect_tx(&full_bar[s], STAGE_BYTES);
        __syncwarp();
        unsigned char* kt = tiles + s * STAGE_BYTES;
        for (int c = lane; c < BN / p.box_rows; c += 32) {
            const int kpos = k0 + c * p.box_rows;
            // boxes past the last key start outside the tensor: the copy writes the zero fill, so
            // that what is multiplied by probability 0 there is finite
            int row = p.total_rows;
            if (kpos < k_hi) {
                const int page = table[kpos >> p.page_shift];
                if (tl_check_page(page))                           // (debug builds: a bad page reads as the zero fill)
                    row = (page * p.n_kv_heads + kvh) * p.page_size + (kpos & (p.page_size - 1));
            }
#pragma unroll
            for (int h = 0; h < HALVES; ++h) {
                unsigned char* dst = kt + h * HALF_BYTES + c * p.box_rows * 128;
                if (p.streamed) {
                    tma_load_2d_streamed(dst, &map_k, &full_bar[s], h * 64, row);
                    tma_load_2d_streamed(dst + KV_BYTES, &map_v, &full_bar[s], h * 64, row);
                } else {
                    tma_load_2d(dst, &map_k, &full_bar[s], h * 64, row);
                    tma_load_2d(dst + KV_BYTES, &map_v, &full_bar[s], h * 64, row);
                }
            }
        }
        __syncwarp();
    };

    if (warp == NCW) {
        // the producer warp sets the barriers up and sends the first tiles on their way while the
        // other warps are still fetching the queries
        if (lane == 0) {
            failed_flag = 0;
            for (int s = 0; s < STAGES; ++s) {
                mbar_init(&full_bar[s], 1);
                mbar_init(&empty_bar[s], NCW);
            }
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __syncwarp();
        // tiles that end before the step's first new position can go now; a tile that may hold a key
        // written by the predecessor (only the last tile of the last split can) waits for it
        int it = 0;
        for (; it < STAGES && it < n_tiles && k_start + (it + 1) * BN <= qpos_base; ++it) issue_tile(it);
        grid_dependency_wait();
        for (; it < STAGES && it < n_tiles; ++it) issue_tile(it);
    } else {
        grid_dependency_wait();
    }
    // queries (zero rows where the tile has none)
    for (int c = tid; c < 16 * (HD / 8); c += NTHREADS) {
        const int rr = c / (HD / 8), part = c - rr * (HD / 8);
        const int tok = tok0 + rr / ng;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (rr < p.tpw * ng && tok < ql) {
            const int head = kvh * p.group + g0 + rr % ng;
            v = *reinterpret_cast<const uint4*>(p.q + ((size_t)(qs + tok) * p.n_heads + head) * HD + part * 8);
        }
        *reinterpret_cast<uint4*>(Qs + rr * QPITCH + part * 8) = v;
    }
    __syncthreads();

    // this thread's two query rows of every 8-row block are 2t and 2t + 1: of the scores^T tile it
    // holds keys g and g + 8 for them, of the out^T tile value columns g and g + 8
    float m[NT][2], l[NT][2];
    float o[NT][KSTEPS][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        m[nt][0] = m[nt][1] = -INFINITY;
        l[nt][0] = l[nt][1] = 0.f;
#pragma unroll
        for (int i = 0; i < KSTEPS; ++i) o[nt][i][0] = o[nt][i][1] = o[nt][i][2] = o[nt][i][3] = 0.f;
    }
    const int g = lane >> 2, t = lane & 3;

    if (warp == NCW) {
        // ---- producer: the first tiles are on their way; keep the ring full
        for (int it = STAGES; it < n_tiles; ++it) {
            if (!__all_sync(0xffffffffu, mbar_wait(&empty_bar[it % STAGES], ((it / STAGES) - 1) & 1, failed))) {
                if (lane == 0) {
                    failed_flag = 1;
                    atomicExch(p.status, ERR_PRODUCER_WAIT);
                }
                break;
            }
            issue_tile(it);
        }
    } else {
        // ---- consumers: the same rows, 16 keys of every tile each
        int qpos[NT][2];
        int qmax = -1, qmin = INT_MAX;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int rr = nt * 8 + 2 * t + j;
                const int tok = tok0 + rr / ng;
                const int qp = (rr < p.tpw * ng && tok < ql) ? qpos_base + tok : -1;
                qpos[nt][j] = qp;
                qmax = max(qmax, qp);
                if (qp >= 0) qmin = min(qmin, qp);
            }
        const int warp_qmax = __reduce_max_sync(0xffffffffu, qmax);
        const int warp_qmin = __reduce_min_sync(0xffffffffu, qmin);
        // Q^T as the 8-wide operand: this thread holds columns 2t, 2t + 1 (and + 8) of row g
        unsigned qf[NT][KSTEPS][2];
        const int mi = lane >> 3;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int kd2 = 0; kd2 < KSTEPS / 2; ++kd2) {
                unsigned r[4];
                ldmatrix_x4(r, smem_u32(Qs + (nt * 8 + (lane & 7)) * QPITCH + (kd2 * 4 + mi) * 8));
                qf[nt][2 * kd2][0] = r[0]; qf[nt][2 * kd2][1] = r[1];
                qf[nt][2 * kd2 + 1][0] = r[2]; qf[nt][2 * kd2 + 1][1] = r[3];
            }
        const int key_off = warp * 16;
        // this lane's row and first chunk inside a tile: K as the 16-row operand [keys x 16 columns],
        // V through a transposing load as [16 columns x keys]
        const int k_row = key_off + (lane & 7) + ((mi & 1) ? 8 : 0);
        const int v_row = key_off + (lane & 7) + ((mi & 2) ? 8 : 0);
        const unsigned k_lane_off = swz(k_row, (mi & 2) ? 1 : 0);
        const unsigned v_lane_off = swz(v_row, mi & 1);
        bool ok = true;
        for (int it = 0; it < n_tiles; ++it) {
            const int s = it % STAGES;
            if (!mbar_wait(&full_bar[s], (it / STAGES) & 1, failed)) {
                ok = false;
                break;
            }
            const int share_lo = k_start + it * BN + key_off;
            if (share_lo <= warp_qmax && share_lo + 16 > k_lo) {
                const unsigned kt = smem_u32(tiles + s * STAGE_BYTES);
                // rows are 128 bytes and tiles 1024-byte aligned, so bits 4-6 of a row's address are the
                // swizzled chunk: xor-ing a constant chunk number in is all it takes to move along a row
                const unsigned ka = kt + k_lane_off, va = kt + KV_BYTES + v_lane_off;
                float sc[NT][4];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
#pragma unroll
                for (int kd = 0; kd < KSTEPS; ++kd) {
                    unsigned kf[4];
                    ldmatrix_x4(kf, (ka ^ (unsigned)(((kd * 2) & 7) << 4)) + (kd / 4) * HALF_BYTES);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) mma_bf16(sc[nt], kf, qf[nt][kd][0], qf[nt][kd][1]);
                }
                const bool all_visible = share_lo >= k_lo && share_lo + 16 <= k_hi && share_lo + 15 <= warp_qmin &&
                                         (p.window <= 0 || share_lo > warp_qmax - p.window);
                if (!all_visible) {
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int qp = qpos[nt][e & 1];
                            const int kpos = share_lo + g + 8 * (e >> 1);
                            const bool vis = kpos >= k_lo && kpos < k_hi && kpos <= qp && (p.window <= 0 || kpos > qp - p.window);
                            if (!vis) sc[nt][e] = -INFINITY;
                        }
                }
                unsigned ph[NT][2], pl[NT][2];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    float m_safe[2], alpha[2];
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        float mx = fmaxf(sc[nt][j], sc[nt][j + 2]);            // over the 16 keys: the lanes that share t
                        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
                        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
                        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
                        const float m_new = fmaxf(m[nt][j], mx * p.scale_log2);   // maxima live on the base-2 scale
                        m_safe[j] = (m_new == -INFINITY) ? 0.f : m_new;           // no key seen yet: keep exponents finite
                        alpha[j] = ex2(m[nt][j] - m_safe[j]);
                        m[nt][j] = m_new;
                        l[nt][j] *= alpha[j];
                    }
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float pv = ex2(fmaf(sc[nt][e], p.scale_log2, -m_safe[e & 1]));
                        sc[nt][e] = pv;
                        l[nt][e & 1] += pv;
                    }
                    if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
                        for (int i = 0; i < KSTEPS; ++i) {
                            o[nt][i][0] *= alpha[0]; o[nt][i][1] *= alpha[1];
                            o[nt][i][2] *= alpha[0]; o[nt][i][3] *= alpha[1];
                        }
                    }
                    // probabilities as value + remainder in bfloat16 (the product keeps 16 bits of them),
                    // moved from result layout [key g][rows 2t, 2t+1] to operand layout [keys 2t, 2t+1][row g]
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const float a = sc[nt][2 * h], c = sc[nt][2 * h + 1];
                        const __nv_bfloat162 hi = __floats2bfloat162_rn(a, c);
                        const float2 back = __bfloat1622float2(hi);
                        ph[nt][h] = movmatrix_trans(*reinterpret_cast<const unsigned*>(&hi));
                        pl[nt][h] = movmatrix_trans(pack_bf16(a - back.x, c - back.y));
                    }
                }
#pragma unroll
                for (int dp = 0; dp < KSTEPS; ++dp) {
                    unsigned vf[4];
                    ldmatrix_x4_trans(vf, (va ^ (unsigned)(((dp * 2) & 7) << 4)) + (dp / 4) * HALF_BYTES);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        mma_bf16(o[nt][dp], vf, ph[nt][0], ph[nt][1]);
                        mma_bf16(o[nt][dp], vf, pl[nt][0], pl[nt][1]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[s]);     // this warp is done with the stage
        }
        if (!__all_sync(0xffffffffu, ok) && lane == 0) {
            failed_flag = 1;
            atomicExch(p.status, ERR_CONSUMER_WAIT);
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                l[nt][j] += __shfl_xor_sync(0xffffffffu, l[nt][j], 4);
                l[nt][j] += __shfl_xor_sync(0xffffffffu, l[nt][j], 8);
                l[nt][j] += __shfl_xor_sync(0xffffffffu, l[nt][j], 16);
            }
    }

    // ---- merge the four warps' partials through shared memory (the stages are done with)
    __syncthreads();
    if (failed_flag) return;
    float* Om = reinterpret_cast<float*>(tiles);          // [NCW][NROWS][OPITCH]
    float* Mm = Om + NCW * NROWS * OPITCH;                // [NCW][NROWS]
    float* Lm = Mm + NCW * NROWS;                         // [NCW][NROWS]
    if (warp < NCW) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
            for (int dp = 0; dp < KSTEPS; ++dp)
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    Om[(warp * NROWS + nt * 8 + 2 * t + (e & 1)) * OPITCH + dp * 16 + g + 8 * (e >> 1)] = o[nt][dp][e];
            if (g == 0) {
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    Mm[warp * NROWS + nt * 8 + 2 * t + j] = m[nt][j];
                    Lm[warp * NROWS + nt * 8 + 2 * t + j] = l[nt][j];
                }
            }
        }
    }
    __syncthreads();
    const int n_rows = min(p.tpw, ql - tok0) * ng;
    for (int idx = tid; idx < n_rows * (HD / 4); idx += NTHREADS) {      // four columns of a row per turn
        const int rr = idx / (HD / 4), d = (idx - rr * (HD / 4)) * 4;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NCW; ++w) M = fmaxf(M, Mm[w * NROWS + rr]);
        float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
        float den = 0.f;
#pragma unroll
        for (int w = 0; w < NCW; ++w) {
            const float mw = Mm[w * NROWS + rr];
            if (mw == -INFINITY) continue;
            const float f = exp2f(mw - M);
            const float4 o4 = *reinterpret_cast<const float4*>(Om + (w * NROWS + rr) * OPITCH + d);
            num.x = fmaf(f, o4.x, num.x); num.y = fmaf(f, o4.y, num.y);
            num.z = fmaf(f, o4.z, num.z); num.w = fmaf(f, o4.w, num.w);
            den = fmaf(f, Lm[w * NROWS + rr], den);
        }
        const int tok = qs + tok0 + rr / ng;
        const int head = kvh * p.group + g0 + rr % ng;
        const size_t row = (size_t)tok * p.n_heads + head;
        if (p.n_splits == 1) {
            const float inv = den > 0.f ? 1.f / den : 0.f;
            uint2 w2;
            w2.x = pack_bf16(num.x * inv, num.y * inv);
            w2.y = pack_bf16(num.z * inv, num.w * inv);
            *reinterpret_cast<uint2*>(p.out + row * HD + d) = w2;
        } else {
            *reinterpret_cast<float4*>(p.part_o + (row * p.n_splits + split) * HD + d) = num;
            if (d == 0) {
                p.part_ml[(row * p.n_splits + split) * 2] = (M == -INFINITY) ? -INFINITY : M * LN2;   // natural-log scale
                p.part_ml[(row * p.n_splits + split) * 2 + 1] = den;
            }
        }
    }
}

// out[row, d] = sum_i e^{m_i - M} o_i[d] / sum_i e^{m_i - M} l_i,  M = max_i m_i: the weights are
// computed once per row (lanes over splits), then every thread sums its lanes over the splits in order
__global__ void merge_partials_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                      __nv_bfloat16* __restrict__ out, int n_splits, int head_dim) {
    __shared__ float wgt[MERGE_MAX_SPLITS];
    __shared__ float red;
    grid_launch_dependents();
    grid_dependency_wait();
    const size_t row = blockIdx.x;
    const float* ml = part_ml + row * n_splits * 2;
    if (threadIdx.x < 32) {
        float M = -INFINITY;
        for (int i = threadIdx.x; i < n_splits; i += 32) M = fmaxf(M, ml[2 * i]);
        M = warp_max(M);
        float den = 0.f;
        for (int i = threadIdx.x; i < n_splits; i += 32) {
            const float mi = ml[2 * i];
            const float w = (mi == -INFINITY) ? 0.f : __expf(mi - M);
            wgt[i] = w;
            den = fmaf(w, ml[2 * i + 1], den);
        }
        den = warp_sum(den);
        if (threadIdx.x == 0) red = den;
    }
    __syncthreads();
    const float inv = red > 0.f ? 1.f / red : 0.f;
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
        float num = 0.f;
        for (int i = 0; i < n_splits; ++i) num = fmaf(wgt[i], part_o[(row * n_splits + i) * head_dim + d], num);
        out[row * head_dim + d] = __float2bfloat16_rn(num * inv);
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

// the page tensor as rows of head_dim elements; box = box_rows x 64 elements, 128-byte swizzle.
// Maps are kept per (pointer, rows, head_dim, box): the page tensors live as long as the engine.
int page_map(CUtensorMap* out, const void* base, long long rows, int head_dim, int box_rows) {
    static std::map<std::tuple<const void*, long long, int, int>, CUtensorMap> cache;
    static std::mutex lock;
    std::lock_guard<std::mutex> guard(lock);
    auto key = std::make_tuple(base, rows, head_dim, box_rows);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return TL_OK;
    }
    EncodeTiledFn fn = encode_tiled();
    if (fn == nullptr) return TL_BAD_SIZE;
    cuuint64_t dims[2] = {(cuuint64_t)head_dim, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)head_dim * 2};
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
    return (size_t)stages_for<HD>() * 2 * (HD / 64) * BN * 128 + 16 * (HD + 8) * 2 + 1024;
}

struct Plan {
    int ng, n_gchunks, tpw, n_q_tiles, n_splits;
};

bool takes(int n_heads, int n_kv_heads, int head_dim, int page_size, int max_q_len) {
    if (head_dim != 64 && head_dim != 128) return false;
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0) return false;
    if (page_size < 1 || (page_size & (page_size - 1)) != 0) return false;           // a power of two
    const int group = n_heads / n_kv_heads;
    const int ng = group < 16 ? group : 16;
    return max_q_len >= 1 && max_q_len <= 16 / ng;
}

Plan make_plan(int n_seqs, int n_heads, int n_kv_heads, int head_dim, int max_q_len, int max_kv_len, int allow_split) {
    Plan pl;
    const int group = n_heads / n_kv_heads;
    pl.ng = group < 16 ? group : 16;
    pl.n_gchunks = (group + pl.ng - 1) / pl.ng;
    pl.tpw = 16 / pl.ng;
    pl.n_q_tiles = (max_q_len + pl.tpw - 1) / pl.tpw;
    pl.n_splits = 1;
    if (allow_split > 1) {                       // a given number of splits (tests and measurements)
        pl.n_splits = allow_split < MERGE_MAX_SPLITS ? allow_split : MERGE_MAX_SPLITS;
    } else if (allow_split && max_kv_len >= 2 * MIN_SPLIT) {
        // CTAs run in waves; with s splits a CTA does 1/s of the keys.  Pick the s that makes
        // (waves / s), the time in units of one unsplit CTA, smallest.  While everything fits one
        // wave, more splits cost next to nothing (a CTA walks its tiles one after the other, so few
        // CTAs with long walks leave most of the memory system idle: one request of 8,192 keys
        // takes 21.8 us in 8 splits and 11.2 us in 32); beyond one wave each split is charged
        // for its partial results and the merge.
        const size_t per_cta = head_dim == 128 ? smem_for<128>() : smem_for<64>();
        int per_sm = (int)((size_t)224 * 1024 / (per_cta + 1024));
        if (per_sm > 6) per_sm = 6;
        const long long slots = 148LL * per_sm;
        const long long base = (long long)pl.n_q_tiles * n_kv_heads * pl.n_gchunks * n_seqs;
        int most = max_kv_len / MIN_SPLIT;
        if (most > MERGE_MAX_SPLITS) most = MERGE_MAX_SPLITS;
        double best = 1e30;
        for (int sp = 1; sp <= most; ++sp) {
            const long long waves = (base * sp + slots - 1) / slots;
            const double cost = (double)waves / sp + (waves == 1 ? 0.0005 : 0.01) * sp;
            if (cost < best - 1e-9) {
                best = cost;
                pl.n_splits = sp;
            }
        }
    }
    return pl;
}

template <int HD, int NT>
int launch(const CUtensorMap& mk, const CUtensorMap& mv, const DecodeParams& p, dim3 grid, cudaStream_t s) {
    constexpr size_t smem = smem_for<HD>();
    auto kern = attention_decode_kernel<HD, stages_for<HD>(), NT>;
    static bool raised = false;
    if (!raised) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        raised = true;
    }
    return (int)tl_launch(kern, grid, dim3(NTHREADS), smem, s, mk, mv, p);
}

}  // namespace

// 1 if this kernel takes the step: head_dim 64 or 128, a page size that is a power of two, and
// every request's rows (tokens x heads of a kv group) within one 16-row tile.
extern "C" int tl_attention_decode_supports(int n_heads, int n_kv_heads, int head_dim, int page_size, int max_q_len) {
    return takes(n_heads, n_kv_heads, head_dim, page_size, max_q_len) ? 1 : 0;
}

extern "C" int tl_attention_decode_plan(int n_tokens, int n_seqs, int n_heads, int n_kv_heads, int head_dim,
                                        int max_q_len, int max_kv_len, int allow_split,
                                        int* n_splits, long long* workspace_floats) {
    if (!takes(n_heads, n_kv_heads, head_dim, 16, max_q_len)) return TL_BAD_SIZE;
    const Plan pl = make_plan(n_seqs, n_heads, n_kv_heads, head_dim, max_q_len, max_kv_len, allow_split);
    *n_splits = pl.n_splits;
    *workspace_floats = pl.n_splits > 1 ? (long long)n_tokens * n_heads * pl.n_splits * (head_dim + 2) : 0;
    return TL_OK;
}

// Same arguments as tl_paged_attention_mma; n_pages is the first extent of the page tensors.
extern "C" int tl_paged_attention_decode(const void* q, const void* k_pages, const void* v_pages, void* out,
                                         const int* block_table, int table_stride, const int* q_start,
                                         const int* kv_len, float* workspace, int* status, int n_tokens, int n_seqs,
                                         int n_heads, int n_kv_heads, int head_dim, int page_size, long long n_pages,
                                         int max_q_len, int max_kv_len, int window, float scale, int allow_split,
                                         void* stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return TL_OK;
    if (!takes(n_heads, n_kv_heads, head_dim, page_size, max_q_len) || max_kv_len <= 0 || n_pages <= 0) return TL_BAD_SIZE;
    if (n_pages * n_kv_heads * page_size >= (1LL << 31)) return TL_BAD_SIZE;
    if (!aligned16(q) || !aligned16(k_pages) || !aligned16(v_pages) || !aligned16(out) || status == nullptr) return TL_BAD_ALIGN;
    const Plan pl = make_plan(n_seqs, n_heads, n_kv_heads, head_dim, max_q_len, max_kv_len, allow_split);
    if (pl.n_splits > 1 && workspace == nullptr) return TL_BAD_SIZE;
    if (n_seqs > 65535 || (long long)n_kv_heads * pl.n_gchunks > 65535) return TL_BAD_SIZE;

    DecodeParams p;
    p.q = (const __nv_bfloat16*)q; p.out = (__nv_bfloat16*)out;
    p.block_table = block_table; p.q_start = q_start; p.kv_len = kv_len; p.table_stride = table_stride;
    p.status = status;
    p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.page_size = page_size;
    p.page_shift = 0;
    while ((1 << p.page_shift) < page_size) ++p.page_shift;
    p.box_rows = page_size < BN ? page_size : BN;
    p.total_rows = (int)(n_pages * n_kv_heads * page_size);
    p.group = n_heads / n_kv_heads; p.ng = pl.ng; p.n_gchunks = pl.n_gchunks; p.tpw = pl.tpw;
    p.window = window > 0 ? window : 0;
    {
        // (an upper bound of what the call reads: every request's keys and values up to the longest context)
        const double kv_bytes = 2.0 * n_seqs * (double)max_kv_len * n_kv_heads * head_dim * 2;
        // (measured: with 64 requests of 2,048 tokens a step is 2.5 % shorter with the mark, with 32 requests 1 %,
        // with 8 requests of 2,048 tokens, whose keys and values L2 holds, 1 % longer; no difference elsewhere)
        p.streamed = kv_bytes > 96e6 ? 1 : 0;
    }
    p.n_splits = pl.n_splits;
    p.scale_log2 = scale * LOG2E;
    p.part_o = workspace;
    p.part_ml = workspace ? workspace + (size_t)n_tokens * n_heads * pl.n_splits * head_dim : nullptr;

    const long long rows = n_pages * n_kv_heads * page_size;
    CUtensorMap mk, mv;
    int rc = page_map(&mk, k_pages, rows, head_dim, p.box_rows);
    if (rc != TL_OK) return rc;
    rc = page_map(&mv, v_pages, rows, head_dim, p.box_rows);
    if (rc != TL_OK) return rc;

    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(pl.n_q_tiles * pl.n_splits, n_kv_heads * pl.n_gchunks, n_seqs);
    // query rows a CTA can meet: one 8-row block is enough for them, or two
    const int rows_used = (max_q_len < pl.tpw ? max_q_len : pl.tpw) * pl.ng;
    if (rows_used <= 8)
        rc = head_dim == 128 ? launch<128, 1>(mk, mv, p, grid, s) : launch<64, 1>(mk, mv, p, grid, s);
    else
        rc = head_dim == 128 ? launch<128, 2>(mk, mv, p, grid, s) : launch<64, 2>(mk, mv, p, grid, s);
    if (rc != TL_OK) return rc;
    if (pl.n_splits > 1) {
        cudaError_t e = tl_launch(merge_partials_kernel, dim3((unsigned)n_tokens * (unsigned)n_heads),
                                  dim3(head_dim >= 128 ? 128u : 64u), 0, s, (const float*)p.part_o, (const float*)p.part_ml,
                                  p.out, pl.n_splits, head_dim);
        if (e != cudaSuccess) return (int)e;
    }
    return TL_OK;
}
