// Y[M, N] = X[M, K] . W[N, K]^T on the CUDA cores, any sizes, operands in
// float32 or bfloat16, accumulation in float32 with fused multiply-add.
//
// This is the matrix product of the true 32-bit path (no tensor-core mode is
// involved, so no reduced-precision matrix mode can slip in), and the product
// of last resort for shapes that the tensor-core kernels refuse.  It computes
// what the reference's matvec / matmul rows do
// (crates/mivi-quant/src/lib.rs:75-135, 143-245): out[b, n] = sum_d in[b, d] * W[n, d].
//
// Epilogues: 0 store float32, 1 store bfloat16, 2 add into a float32 matrix
// (the residual stream).  A bias [N] may be added in every mode.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename T>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const T* __restrict__ X, const T* __restrict__ W, const float* __restrict__ bias,
                 void* __restrict__ out, int mode, int M, int N, int K, int ldo) {
    mv_pdl_begin();
    __shared__ float Xs[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;          // 16 x 16 threads
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 x 16 elements of each operand, 4 per thread
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int idx = tid + e * 256;
            const int r = idx >> 4, c = idx & 15;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + c;
            Xs[c][r] = (gm < M && gk < K) ? mv_to_f32(X[(size_t)gm * K + gk]) : 0.f;
            Ws[c][r] = (gn < N && gk < K) ? mv_to_f32(W[(size_t)gn * K + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = Xs[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = Ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gm = m0 + ty * TM + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gn = n0 + tx * TN + j;
            if (gn >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias[gn];
            const size_t o = (size_t)gm * ldo + gn;
            if (mode == 0) ((float*)out)[o] = v;
            else if (mode == 1) ((__nv_bfloat16*)out)[o] = __float2bfloat16_rn(v);
            else ((float*)out)[o] += v;
        }
    }
}

}  // namespace

MV_API int mv_gemm_simt(const void* X, const void* W, int in_dtype, const float* bias, void* out,
                        int mode, int M, int N, int K, int ldo, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (in_dtype == MV_DT_BF16)
        mv_launch(gemm_simt_kernel<__nv_bfloat16>, grid, 256, 0, stream, (const __nv_bfloat16*)X, (const __nv_bfloat16*)W,
                                                   bias, out, mode, M, N, K, ldo);
    else
        mv_launch(gemm_simt_kernel<float>, grid, 256, 0, stream, (const float*)X, (const float*)W, bias, out, mode,
                                                   M, N, K, ldo);
    return mv_launch_status();
}
