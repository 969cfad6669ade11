// out[M, N] = A[M, K] * W[N, K]^T with float32 multiply-adds on the CUDA cores.
//
// This is the matrix product of the true 32-bit path: no tensor cores and no
// reduced-precision mode.  Each output element is a plain float32 sum over k in
// ascending order, so its value does not depend on M, on the position of its row in
// the batch, or on which other rows are present.  A and W may be float32 or
// bfloat16 (read exactly, accumulated in float32); the output is float32 or the
// activation type.  Any M, N, K is accepted.
//
// The reference uses at::linear here (cuBLAS SGEMM in float32,
// pulsar-core/src/model/qwen3.cpp:82-84, 114, 117-119, 128).
#include "common.cuh"

namespace {

using namespace pb;

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;   // 256 threads, 4x4 outputs each

template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TA* __restrict__ A, const TW* __restrict__ W, TO* __restrict__ out, int M, int N, int K) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int row0 = blockIdx.y * BM, col0 = blockIdx.x * BN;
    const int tr = (tid / 16) * TM, tc = (tid % 16) * TN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 rows x 16 k per operand = 1024 elements, 4 per thread, k fastest for coalescing.
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int idx = tid + e * 256;
            const int r = idx / BK, kk = idx % BK;
            const int gr = row0 + r, gk = k0 + kk;
            As[kk][r] = (gr < M && gk < K) ? to_float(A[(size_t)gr * K + gk]) : 0.0f;
            const int gc = col0 + r;
            Ws[kk][r] = (gc < N && gk < K) ? to_float(W[(size_t)gc * K + gk]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], w[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][tr + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tc + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gr = row0 + tr + i;
        if (gr >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gc = col0 + tc + j;
            if (gc < N) out[(size_t)gr * N + gc] = from_float<TO>(acc[i][j]);
        }
    }
}

template <typename TA, typename TW, typename TO>
int launch(const void* A, const void* W, void* out, int M, int N, int K, cudaStream_t stream) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return PB_ERR_TOO_LARGE;
    gemm_simt_kernel<TA, TW, TO><<<grid, 256, 0, stream>>>((const TA*)A, (const TW*)W, (TO*)out, M, N, K);
    return launch_status();
}

}  // namespace

// a_dtype / w_dtype / out_dtype: PB_F32 or PB_BF16.
PB_EXPORT int pb_gemm_simt(int a_dtype, int w_dtype, int out_dtype, const void* A, const void* W, void* out,
                           int M, int N, int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return PB_ERR_BAD_SIZE;
    if ((a_dtype | w_dtype | out_dtype) & ~1) return PB_ERR_BAD_DTYPE;
    typedef __nv_bfloat16 bf;
    const int key = a_dtype * 4 + w_dtype * 2 + out_dtype;
    switch (key) {
        case 0: return launch<float, float, float>(A, W, out, M, N, K, stream);
        case 1: return launch<float, float, bf>(A, W, out, M, N, K, stream);
        case 2: return launch<float, bf, float>(A, W, out, M, N, K, stream);
        case 3: return launch<float, bf, bf>(A, W, out, M, N, K, stream);
        case 4: return launch<bf, float, float>(A, W, out, M, N, K, stream);
        case 5: return launch<bf, float, bf>(A, W, out, M, N, K, stream);
        case 6: return launch<bf, bf, float>(A, W, out, M, N, K, stream);
        case 7: return launch<bf, bf, bf>(A, W, out, M, N, K, stream);
    }
    return PB_ERR_BAD_DTYPE;
}
