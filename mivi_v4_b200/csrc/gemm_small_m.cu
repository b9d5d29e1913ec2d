// Y[M, N] = X[M, K] . W[N, K]^T for a handful of tokens (M <= 64), bfloat16
// operands, float32 accumulation: the matrix product of a decode step, whose
// cost is reading W once from HBM.
//
// The weight matrix takes the tensor core's M side ("swap-AB"): a warp owns 16
// (or 32) consecutive rows of W and a slice of K, and streams its rows straight
// from global memory into mma.sync fragments with 16-byte loads; the tokens
// are the N side, 8 per n-tile.  A thread's 16 bytes are 8 consecutive k of one
// row.  The fragment layout of mma.m16n8k16 wants k = {2t, 2t+1, 2t+8, 2t+9}
// from lane t of a group, but a dot product does not care in which order k is
// summed as long as both operands agree: the thread's first 4 values serve
// one mma as those four k, the last 4 the next mma, and X is loaded with the
// same rule, so no shuffle and no shared-memory staging of W is needed.
//
// The warps of a block split K and add their partial sums through shared
// memory in warp order, so the result is the same in every run.
//
// What it replaces in the reference: quantized_matvec, one output row per
// dot product over the input (crates/mivi-quant/src/lib.rs:75-135).
#include "common.cuh"

namespace {


__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                 "{%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// NT: n-tiles of 8 tokens; RT: tiles of 16 weight rows per warp; UNROLL: k-steps
// of 32 whose W loads are issued together (bytes in flight per warp).
template <int NT, int RT, int UNROLL>
__global__ void __launch_bounds__(512)
gemm_small_m_kernel(const __nv_bfloat16* __restrict__ W, const __nv_bfloat16* __restrict__ X,
                    const float* __restrict__ bias, void* __restrict__ out, int mode, int M, int N, int K,
                    int ldo) {
    extern __shared__ float red[];                      // [warps][RT*16][NT*8 + 1]
    constexpr int ROWS = RT * 16, COLS = NT * 8, LDR = COLS + 1;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * ROWS;

    float acc[RT][NT][4];
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[r][j][e] = 0.f;

    // rows this thread loads; rows past N are read from row N-1 and dropped at the end
    const __nv_bfloat16* wrow[RT][2];
#pragma unroll
    for (int r = 0; r < RT; ++r) {
        wrow[r][0] = W + (size_t)min(n0 + r * 16 + g, N - 1) * K;
        wrow[r][1] = W + (size_t)min(n0 + r * 16 + g + 8, N - 1) * K;
    }
    const __nv_bfloat16* xrow[NT];
    bool xok[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        xok[j] = j * 8 + g < M;
        xrow[j] = X + (size_t)min(j * 8 + g, M - 1) * K;
    }

    const int ksteps = (K + 31) >> 5;
    // contiguous run of k-steps for this warp
    const int per = (ksteps + nwarps - 1) / nwarps;
    const int ks_begin = warp * per, ks_end = min(ksteps, ks_begin + per);

    for (int ks = ks_begin; ks < ks_end; ks += UNROLL) {
        uint4 w[UNROLL][RT][2];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int k = ((ks + u) << 5) + 8 * t;
            const bool ok = (ks + u) < ks_end && k < K;
#pragma unroll
            for (int r = 0; r < RT; ++r)
#pragma unroll
                for (int h = 0; h < 2; ++h)
                    w[u][r][h] = ok ? ld_stream16(wrow[r][h] + k) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int k = ((ks + u) << 5) + 8 * t;
            const bool ok = (ks + u) < ks_end && k < K;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const uint4 x = (ok && xok[j]) ? *reinterpret_cast<const uint4*>(xrow[j] + k)
                                               : make_uint4(0, 0, 0, 0);
#pragma unroll
                for (int r = 0; r < RT; ++r) {
                    mma_bf16(acc[r][j], w[u][r][0].x, w[u][r][1].x, w[u][r][0].y, w[u][r][1].y, x.x, x.y);
                    mma_bf16(acc[r][j], w[u][r][0].z, w[u][r][1].z, w[u][r][0].w, w[u][r][1].w, x.z, x.w);
                }
            }
        }
    }

    // partial sums of all warps -> shared memory
    float* mine = red + (size_t)warp * ROWS * LDR;
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            const int row = r * 16 + g, col = j * 8 + 2 * t;
            mine[row * LDR + col] = acc[r][j][0];
            mine[row * LDR + col + 1] = acc[r][j][1];
            mine[(row + 8) * LDR + col] = acc[r][j][2];
            mine[(row + 8) * LDR + col + 1] = acc[r][j][3];
        }
    __syncthreads();
    for (int idx = threadIdx.x; idx < ROWS * M; idx += blockDim.x) {
        const int r = idx % ROWS, m = idx / ROWS;
        const int n = n0 + r;
        if (n >= N) continue;
        float v = 0.f;
        for (int wp = 0; wp < nwarps; ++wp) v += red[(size_t)wp * ROWS * LDR + r * LDR + m];
        if (bias) v += bias[n];
        const size_t o = (size_t)m * ldo + n;
        if (mode == 0) ((float*)out)[o] = v;
        else if (mode == 1) ((__nv_bfloat16*)out)[o] = __float2bfloat16_rn(v);
        else ((float*)out)[o] += v;
    }
}

template <int NT, int RT, int UNROLL>
int launch(const void* W, const void* X, const float* bias, void* out, int mode, int M, int N, int K, int ldo,
           cudaStream_t stream) {
    constexpr int ROWS = RT * 16, LDR = NT * 8 + 1;
    const int ksteps = (K + 31) / 32;
    int warps = ksteps / (2 * UNROLL);
    warps = warps < 1 ? 1 : (warps > 16 ? 16 : warps);
    const size_t smem = (size_t)warps * ROWS * LDR * sizeof(float);
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(gemm_small_m_kernel<NT, RT, UNROLL>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        attr_set = true;
    }
    const unsigned blocks = (unsigned)((N + ROWS - 1) / ROWS);
    gemm_small_m_kernel<NT, RT, UNROLL><<<blocks, warps * 32, smem, stream>>>(
        (const __nv_bfloat16*)W, (const __nv_bfloat16*)X, bias, out, mode, M, N, K, ldo);
    return mv_launch_status();
}

}  // namespace

// mode: 0 store float32, 1 store bfloat16, 2 add into float32.  Needs
// 1 <= M <= 64, K a multiple of 8, and 16-byte aligned operands.
MV_API int mv_gemm_small_m(const void* X, const void* W, const float* bias, void* out, int mode, int M,
                           int N, int K, int ldo, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 64 || K % 8 || ((uintptr_t)X & 15) || ((uintptr_t)W & 15)) return (int)cudaErrorInvalidValue;
    const int nt = (M + 7) / 8;
    // 32 rows per warp halve the re-reads of X; 16 rows keep enough blocks for a narrow matrix
    const bool wide = N >= 32 * 2 * 148;
#define MV_GO(NT, RT, U) return launch<NT, RT, U>(W, X, bias, out, mode, M, N, K, ldo, stream)
    switch (nt) {
        case 1: if (wide) MV_GO(1, 2, 4); else MV_GO(1, 1, 4);
        case 2: if (wide) MV_GO(2, 2, 4); else MV_GO(2, 1, 4);
        case 3: case 4: if (wide) MV_GO(4, 2, 4); else MV_GO(4, 1, 4);
        default: if (wide) MV_GO(8, 2, 2); else MV_GO(8, 1, 4);
    }
#undef MV_GO
}
