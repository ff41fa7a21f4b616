// C[M, N] = A[M, K] . W[N, K]^T with float32 multiply-adds on the CUDA cores (no tensor cores,
// hence no reduced-precision matrix mode): the projection kernel of the true 32-bit path, and a
// fallback for bfloat16 operands.  Both operands are K-major as stored: activations row-major and
// weights in the [out, in] layout of nn.Linear (torchllms/models/networks.py:474-493, :600-602).
//
// 64 x 64 output tile per CTA, K walked 16 at a time through shared memory, 4 x 4 outputs per
// thread; every edge is guarded, so M, N and K may be anything.  The K loop order is the same
// for every row, so a row's result does not depend on which other rows share the launch.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, PAD = 4, NT = 256;

template <typename T, typename TO>
__global__ void __launch_bounds__(NT) gemm_simt_kernel(const T* __restrict__ A, const T* __restrict__ W,
                                                       TO* __restrict__ C, int M, int N, int K) {
    __shared__ float As[BK][BM + PAD];
    __shared__ float Ws[BK][BN + PAD];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int lrow = tid >> 2;         // 0..63: tile row this thread loads
    const int lk = (tid & 3) * 4;      // 0, 4, 8, 12: first of its four k
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        {
            const int gm = m0 + lrow, gn = n0 + lrow;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int gk = k0 + lk + e;
                As[lk + e][lrow] = (gm < M && gk < K) ? to_float(A[(size_t)gm * K + gk]) : 0.f;
                Ws[lk + e][lrow] = (gn < N && gk < K) ? to_float(W[(size_t)gn * K + gk]) : 0.f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            const float4 a4 = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
            const float4 w4 = *reinterpret_cast<const float4*>(&Ws[k][tx * 4]);
            const float a[4] = {a4.x, a4.y, a4.z, a4.w};
            const float w[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn < N) C[(size_t)gm * N + gn] = from_float<TO>(acc[i][j]);
        }
    }
}

template <typename T, typename TO>
int launch(const void* A, const void* W, void* C, int M, int N, int K, cudaStream_t s) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return TL_BAD_SIZE;
    gemm_simt_kernel<T, TO><<<grid, NT, 0, s>>>((const T*)A, (const T*)W, (TO*)C, M, N, K);
    TL_LAUNCH_CHECK();
    return TL_OK;
}

}  // namespace

extern "C" int tl_gemm_simt(const void* A, const void* W, void* C, int in_dtype, int out_dtype,
                            int M, int N, int K, void* stream) {
    if (M <= 0 || N <= 0) return TL_OK;
    if (K <= 0) return TL_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    if (in_dtype == TL_F32 && out_dtype == TL_F32) return launch<float, float>(A, W, C, M, N, K, s);
    if (in_dtype == TL_BF16 && out_dtype == TL_BF16) return launch<__nv_bfloat16, __nv_bfloat16>(A, W, C, M, N, K, s);
    if (in_dtype == TL_BF16 && out_dtype == TL_F32) return launch<__nv_bfloat16, float>(A, W, C, M, N, K, s);
    return TL_BAD_DTYPE;
}
