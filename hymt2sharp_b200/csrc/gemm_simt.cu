// General matrix product on CUDA cores, any sizes: C = epilogue(A[M,K] · W[N,K]^T).
// Both operands are K-contiguous (W is stored [out][in], the layout of
// src/HyMT2Sharp/HunyuanDenseModel.cs:586-587).  Products and sums are float32
// FMAs in ascending K order, so an output element does not depend on M or on
// its row's place in the batch.  This is the whole of the 32-bit path and the
// fallback of the bfloat16 path for shapes that the tensor-core kernels refuse.
//
// Epilogues:
//   0 store      C = acc
//   1 accumulate C += acc                      (projection back into the residual stream)
//   2 swiglu     C = silu(acc_gate) * acc_up   (W holds N gate rows, then N up rows;
//                                               src/HyMT2Sharp/Ops.cs:1053)
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4, THREADS = 256;

enum { EPI_STORE = 0, EPI_ACCUMULATE = 1, EPI_SWIGLU = 2 };

template <typename T>
__device__ __forceinline__ void load4(const T* row, int k, int K, bool row_ok, bool vec, float out[4]) {
    if (row_ok && vec && k + 4 <= K) {
        if constexpr (sizeof(T) == 4) {
            float4 v = *reinterpret_cast<const float4*>(row + k);
            out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
        } else {
            uint2 v = *reinterpret_cast<const uint2*>(row + k);
            __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&v.x);
            __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162*>(&v.y);
            out[0] = __low2float(a); out[1] = __high2float(a); out[2] = __low2float(b); out[3] = __high2float(b);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 4; i++) out[i] = (row_ok && k + i < K) ? to_float(row[k + i]) : 0.f;
    }
}

template <typename TA, typename TW, typename TC, int EPI>
__global__ void __launch_bounds__(THREADS)
gemm_simt_kernel(TC* __restrict__ C, const TA* __restrict__ A, const TW* __restrict__ W, int M, int N, int K,
                 long lda, long ldw, long ldc, bool vec_a, bool vec_w) {
    constexpr int NB = EPI == EPI_SWIGLU ? 2 : 1;
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[NB][BK][BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int lrow = tid >> 2, lk = (tid & 3) * 4;  // loader: 64 rows x 4 groups of 4 k
    const int tm = (tid >> 4) * TM, tn = (tid & 15) * TN;

    float acc[NB][TM][TN];
#pragma unroll
    for (int b = 0; b < NB; b++)
#pragma unroll
        for (int i = 0; i < TM; i++)
#pragma unroll
            for (int j = 0; j < TN; j++) acc[b][i][j] = 0.f;

    const bool a_ok = m0 + lrow < M, w_ok = n0 + lrow < N;
    const TA* a_row = A + (size_t)(a_ok ? m0 + lrow : 0) * lda;
    const TW* w_row[NB];
#pragma unroll
    for (int b = 0; b < NB; b++) w_row[b] = W + ((size_t)b * N + (w_ok ? n0 + lrow : 0)) * ldw;

    for (int k0 = 0; k0 < K; k0 += BK) {
        float va[4], vw[NB][4];
        load4(a_row, k0 + lk, K, a_ok, vec_a, va);
#pragma unroll
        for (int b = 0; b < NB; b++) load4(w_row[b], k0 + lk, K, w_ok, vec_w, vw[b]);
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; i++) {
            As[lk + i][lrow] = va[i];
#pragma unroll
            for (int b = 0; b < NB; b++) Ws[b][lk + i][lrow] = vw[b][i];
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; kk++) {
            float a[TM], w[NB][TN];
#pragma unroll
            for (int i = 0; i < TM; i++) a[i] = As[kk][tm + i];
#pragma unroll
            for (int b = 0; b < NB; b++)
#pragma unroll
                for (int j = 0; j < TN; j++) w[b][j] = Ws[b][kk][tn + j];
#pragma unroll
            for (int b = 0; b < NB; b++)
#pragma unroll
                for (int i = 0; i < TM; i++)
#pragma unroll
                    for (int j = 0; j < TN; j++) acc[b][i][j] = fmaf(a[i], w[b][j], acc[b][i][j]);
        }
    }

#pragma unroll
    for (int i = 0; i < TM; i++) {
        const int m = m0 + tm + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; j++) {
            const int n = n0 + tn + j;
            if (n >= N) continue;
            TC* c = C + (size_t)m * ldc + n;
            if constexpr (EPI == EPI_STORE) {
                *c = from_float<TC>(acc[0][i][j]);
            } else if constexpr (EPI == EPI_ACCUMULATE) {
                *c = from_float<TC>(to_float(*c) + acc[0][i][j]);
            } else {
                const float g = acc[0][i][j], u = acc[NB - 1][i][j];
                *c = from_float<TC>(g / (1.0f + expf(-g)) * u);
            }
        }
    }
}

template <typename TA, typename TW, typename TC>
int launch(void* C, const void* A, const void* W, int M, int N, int K, long lda, long ldw, long ldc, int epi,
           cudaStream_t stream) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    const bool vec_a = (lda % 4 == 0) && ((uintptr_t)A % 16 == 0);
    const bool vec_w = (ldw % 4 == 0) && ((uintptr_t)W % 16 == 0);
#define HYMT2_GEMM_CASE(E)                                                                                  \
    gemm_simt_kernel<TA, TW, TC, E><<<grid, THREADS, 0, stream>>>((TC*)C, (const TA*)A, (const TW*)W, M, N, K, \
                                                                  lda, ldw, ldc, vec_a, vec_w)
    if (epi == EPI_STORE) HYMT2_GEMM_CASE(EPI_STORE);
    else if (epi == EPI_ACCUMULATE) HYMT2_GEMM_CASE(EPI_ACCUMULATE);
    else HYMT2_GEMM_CASE(EPI_SWIGLU);
#undef HYMT2_GEMM_CASE
    return hymt2_check_launch("gemm_simt");
}

}  // namespace

// C[M,N] (ldc) = epilogue(A[M,K] (lda) · W[N,K]^T (ldw)); for the swiglu epilogue W has 2N rows.
HYMT2_API int hymt2_gemm_simt(void* C, int c_dtype, const void* A, int a_dtype, const void* W, int w_dtype,
                              int M, int N, int K, long lda, long ldw, long ldc, int epilogue,
                              cudaStream_t stream) {
    if (M == 0 || N == 0) return HYMT2_OK;
    HYMT2_REQUIRE(M > 0 && N > 0 && K > 0, "gemm: bad sizes M=%d N=%d K=%d", M, N, K);
    HYMT2_REQUIRE(epilogue >= 0 && epilogue <= 2, "gemm: unknown epilogue %d", epilogue);
    HYMT2_REQUIRE(lda >= K && ldw >= K && ldc >= N, "gemm: a leading dimension is smaller than its row");
    HYMT2_REQUIRE((M + BM - 1) / BM <= 65535, "gemm: M=%d needs more than 65535 row tiles", M);
    HYMT2_DISPATCH_DTYPE(a_dtype, TA, HYMT2_DISPATCH_DTYPE(w_dtype, TW, HYMT2_DISPATCH_DTYPE(c_dtype, TC,
        return (launch<TA, TW, TC>(C, A, W, M, N, K, lda, ldw, ldc, epilogue, stream)))));
    return HYMT2_OK;
}
