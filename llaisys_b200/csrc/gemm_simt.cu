// Y[M,N] = X[M,K] * W[N,K]^T (+ bias[N]) with plain float32 FMA accumulation on the CUDA cores.
//
// This is the matrix product of the true 32-bit path (no tensor cores, so no reduced-precision
// matrix mode can slip in) and the fallback of the bfloat16 path for operands the tensor-core
// kernel does not take (a 32-bit weight under 16-bit activations, a reduction length that is
// not a multiple of 8).  Any M, N, K.  The formula is that of xsmccc/llaisys' linear operator
// (src/ops/linear/cpu/linear_cpu.cpp:21-40): accumulate over k in float32, add the bias, round once.
#include "common.cuh"

template <typename TX, typename TW, typename TO>
__global__ void __launch_bounds__(256)
gemm_tile_kernel(const TX* __restrict__ X, const TW* __restrict__ W, const void* __restrict__ bias,
                 int bias_dtype, TO* __restrict__ Y, int M, int N, int K, int ldx, int ldy) {
    constexpr int BM = 64, BN = 64, BK = 16;
    __shared__ float Xs[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    llb_grid_dependency_sync();
    int tid = threadIdx.x;
    int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    int ty = tid / 16, tx = tid % 16;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    int lr = tid / 4, lk = (tid % 4) * 4;      // this thread loads row lr, k = lk..lk+3
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            int k = k0 + lk + q;
            int m = m0 + lr, n = n0 + lr;
            Xs[lk + q][lr] = (m < M && k < K) ? to_f32(X[(size_t)m * ldx + k]) : 0.f;
            Ws[lk + q][lr] = (n < N && k < K) ? to_f32(W[(size_t)n * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = Xs[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias_dtype == LLB_F32 ? ((const float*)bias)[n] : to_f32(((const bf16*)bias)[n]);
            Y[(size_t)m * ldy + n] = from_f32<TO>(v);
        }
    }
}

// Few rows (decode): one warp per output column streams that weight row once for all rows.
template <typename TX, typename TW, typename TO, int MR>
__global__ void __launch_bounds__(256)
gemm_rows_kernel(const TX* __restrict__ X, const TW* __restrict__ W, const void* __restrict__ bias,
                 int bias_dtype, TO* __restrict__ Y, int M, int N, int K, int ldx, int ldy) {
    llb_grid_dependency_sync();
    int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= N) return;
    const TW* w = W + (size_t)warp * K;
    for (int m0 = 0; m0 < M; m0 += MR) {
        float acc[MR];
#pragma unroll
        for (int i = 0; i < MR; ++i) acc[i] = 0.f;
        for (int k = lane; k < K; k += 32) {
            float wv = to_f32(w[k]);
#pragma unroll
            for (int i = 0; i < MR; ++i)
                if (m0 + i < M) acc[i] = fmaf(to_f32(X[(size_t)(m0 + i) * ldx + k]), wv, acc[i]);
        }
#pragma unroll
        for (int i = 0; i < MR; ++i) {
            float v = warp_sum(acc[i]);
            if (lane == 0 && m0 + i < M) {
                if (bias) v += bias_dtype == LLB_F32 ? ((const float*)bias)[warp] : to_f32(((const bf16*)bias)[warp]);
                Y[(size_t)(m0 + i) * ldy + warp] = from_f32<TO>(v);
            }
        }
    }
}

template <typename TX, typename TW, typename TO>
static void launch(const void* X, const void* W, const void* bias, int bias_dtype, void* Y, int M,
                   int N, int K, int ldx, int ldy, cudaStream_t stream) {
    if (M <= 8) {
        int warps_per_block = 8;
        dim3 grid((N + warps_per_block - 1) / warps_per_block);
        llb_launch(gemm_rows_kernel<TX, TW, TO, 8>, grid, dim3(256), 0, stream,
                   (const TX*)X, (const TW*)W, bias, bias_dtype, (TO*)Y, M, N, K, ldx, ldy);
    } else {
        dim3 grid((N + 63) / 64, (M + 63) / 64);
        llb_launch(gemm_tile_kernel<TX, TW, TO>, grid, dim3(256), 0, stream,
                   (const TX*)X, (const TW*)W, bias, bias_dtype, (TO*)Y, M, N, K, ldx, ldy);
    }
}

// ldx, ldy: row strides of X and Y in elements (W is dense [N, K]).
LLB_API int llb_gemm_simt(const void* X, int x_dtype, const void* W, int w_dtype, const void* bias,
                          int bias_dtype, void* Y, int y_dtype, int M, int N, int K, int ldx,
                          int ldy, cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    if ((N + 63) / 64 > 2147483647 || (M + 63) / 64 > 65535) return (int)cudaErrorInvalidValue;
    LLB_DISPATCH_DTYPE(x_dtype, TX, {
        LLB_DISPATCH_DTYPE(w_dtype, TW, {
            LLB_DISPATCH_DTYPE(y_dtype, TO, {
                launch<TX, TW, TO>(X, W, bias, bias_dtype, Y, M, N, K, ldx, ldy, stream);
            });
        });
    });
    return llb_status();
}
