// Y[M, N] = X[M, K] . W[N, K]^T on the fifth-generation tensor cores:
// bfloat16 operands brought into shared memory by TMA, tcgen05.mma issued by
// one thread with the accumulator in tensor memory, read back with tcgen05.ld
// for the epilogue.  This is the matrix product of prefill (M > 64); the
// decode step's product is gemm_small_m.cu.
//
// Both operands are K-major (X rows and W rows are contiguous in K), so a
// 128 x 64 tile of either is 128 rows of 128 bytes: exactly the 128-byte
// swizzle atom that TMA writes and the MMA's shared-memory descriptor reads.
//
// Block = one 128 x BN tile of Y, 6 warps:
//   warp 0   one lane issues the TMA loads of the K blocks into a ring of
//            STAGES buffers (full/empty mbarriers);
//   warp 1   allocates BN columns of tensor memory; one lane issues four
//            128 x BN x 16 MMAs per K block and commits to the stage's
//            "empty" barrier, at the end to the "accumulator ready" barrier;
//   warps 2-5 wait for the accumulator, read their 32 lanes (rows) of tensor
//            memory 32 columns at a time and write Y (store float32, store
//            bfloat16, or add into float32; optional bias).
// Two blocks fit one SM (3 stages of 32 KB each), so one block's epilogue
// overlaps the other's main loop.
//
// Every wait on an mbarrier is bounded: after about two seconds it gives up,
// raises the error flag that the host passes in, and the block still runs to
// its end and frees its tensor memory.  Rows past M or N and the tail of K are
// zero-filled by TMA and masked in the epilogue, so any M, N and any K that is
// a multiple of 8 (16-byte rows) work.
//
// Reference counterpart: quantized_matmul_rows, out[b, n] = sum_d in[b, d] W[n, d]
// (crates/mivi-quant/src/lib.rs:143-245).
#include "tc_common.cuh"

namespace {

constexpr int THREADS = 192;

#include "gemm_tc_store.cuh"

// The consuming end of a norm carried by products (see gemm_small_m.cu; null when unused): the rows of X
// still lack their norm's scale, so every row of the result is multiplied by
// rsqrt(sum of the row's partial sums / dim + eps).
struct RowScale {
    const float* part;                 // [rows][stride], n sums of squares per row
    int n, stride;
    float inv_dim, eps;
};
__device__ __forceinline__ float row_sum(const RowScale& rs, int row, int M) {
    float ss = 0.f;
    if (rs.part && row < M)
        for (int p = 0; p < rs.n; ++p) ss += rs.part[(size_t)row * rs.stride + p];
    return ss;
}
__device__ __forceinline__ void scale_chunk(unsigned (&r)[32], float sc) {
#pragma unroll
    for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * sc);
}

template <int BN, int STAGES>
struct SmemLayout {
    static constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int TILE_BYTES = STAGES * STAGE_BYTES;
    static constexpr int BAR_BYTES = (2 * STAGES + 1) * 8 + 8;
    static constexpr int TOTAL = TILE_BYTES + BAR_BYTES + 1024;      // 1024 for the manual alignment
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const float* __restrict__ bias, void* __restrict__ out, int mode, int M, int N, int K, int ldo,
               const RowScale rs, int* __restrict__ err) {
    using L = SmemLayout<BN, STAGES>;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned long long* bars = (unsigned long long*)(smem + L::TILE_BYTES);
    unsigned* tmem_holder = (unsigned*)(bars + 2 * STAGES + 1);
    const unsigned full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES, acc_bar = full0 + 16 * STAGES;
    const unsigned tiles0 = smem_u32(smem);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int kblocks = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(acc_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_holder)), "r"((unsigned)BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_base = *tmem_holder;

    if (warp == 0) {
        if (lane == 0) {
            for (int kb = 0; kb < kblocks; ++kb) {
                const int s = kb % STAGES;
                const unsigned phase = (unsigned)(kb / STAGES) & 1u;
                if (!mbar_wait(empty0 + 8 * s, phase ^ 1u, err, 1)) break;
                mbar_expect_tx(full0 + 8 * s, L::STAGE_BYTES);
                const unsigned a_dst = tiles0 + s * L::STAGE_BYTES;
                tma_load_2d(a_dst, &map_a, kb * BK, m0, full0 + 8 * s);
                tma_load_2d(a_dst + L::A_BYTES, &map_b, kb * BK, n0, full0 + 8 * s);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const unsigned idesc = instr_desc(BM, BN);
            bool ok = true;
            for (int kb = 0; kb < kblocks && ok; ++kb) {
                const int s = kb % STAGES;
                const unsigned phase = (unsigned)(kb / STAGES) & 1u;
                ok = mbar_wait(full0 + 8 * s, phase, err, 2);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned a_addr = tiles0 + s * L::STAGE_BYTES;
                const unsigned b_addr = a_addr + L::A_BYTES;
#pragma unroll
                for (int k = 0; k < BK / 16; ++k) {
                    // 16 elements of K are 32 bytes further along the swizzled row
                    mma_f16(tmem_base, smem_desc(a_addr + k * 32), smem_desc(b_addr + k * 32), idesc,
                            (kb > 0 || k > 0) ? 1u : 0u);
                }
                mma_commit(empty0 + 8 * s);               // the stage is free once these MMAs have read it
            }
            mma_commit(acc_bar);                          // the accumulator is complete
        }
    } else {
        // epilogue: warp w reads tensor-memory lanes 32 * (w % 4) .. + 31
        const int quarter = warp & 3;
        const int row = m0 + quarter * 32 + lane;
        const float ss = row_sum(rs, row, M);            // asked for while the products still run
        if (mbar_wait(acc_bar, 0, err, 3)) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float sc = rs.part ? 1.0f / sqrtf(ss * rs.inv_dim + rs.eps) : 1.f;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                unsigned r[32];
                tmem_ld32(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)c0, r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (rs.part) scale_chunk(r, sc);
                if (row < M) store_chunk(r, row, n0 + c0, N, mode, bias, out, ldo);
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((unsigned)BN)
                     : "memory");
    }
}

// ---------------------------------------------------------------------------
// The same product for wide matrices: 128 x 256 tiles, one block per SM that
// walks over tiles (consecutive blocks share a tile of W, so W comes from HBM
// once and from L2 afterwards), and TWO accumulators of 256 columns in tensor
// memory: while the epilogue warps drain one, the MMA warp fills the other, and
// the TMA warp runs ahead across tile boundaries.  A 128 x 256 tile needs
// 48 KB of operands per 128 x 256 x 64 of MMA work, 96 bytes per clock at full
// tensor rate, which four stages of shared memory can keep in flight; the
// 128 x 128 tile needs 128.
// ---------------------------------------------------------------------------
template <int STAGES>
struct WideLayout {
    static constexpr int BN = 256;
    static constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int TILE_BYTES = STAGES * STAGE_BYTES;
    static constexpr int BAR_BYTES = (2 * STAGES + 4) * 8 + 8;
    static constexpr int TOTAL = TILE_BYTES + BAR_BYTES + 1024;
};

template <int STAGES>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_wide_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const float* __restrict__ bias, void* __restrict__ out, int mode, int M, int N, int K, int ldo,
                    const RowScale rs, int* __restrict__ err) {
    using L = WideLayout<STAGES>;
    constexpr int BN = L::BN;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned long long* bars = (unsigned long long*)(smem + L::TILE_BYTES);
    unsigned* tmem_holder = (unsigned*)(bars + 2 * STAGES + 4);
    const unsigned full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES;
    const unsigned acc_full0 = full0 + 16 * STAGES, acc_empty0 = acc_full0 + 16;
    const unsigned tiles0 = smem_u32(smem);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN;
    const int tiles = m_tiles * n_tiles;
    const int kblocks = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(acc_full0 + 8 * a, 1);
            mbar_init(acc_empty0 + 8 * a, 4);             // one arrival per epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_holder)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_base = *tmem_holder;

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;                                   // K blocks issued so far, over all tiles
            bool ok = true;
            for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
                const int m0 = (t % m_tiles) * BM, n0 = (t / m_tiles) * BN;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    const unsigned phase = (unsigned)(it / STAGES) & 1u;
                    ok = mbar_wait(empty0 + 8 * s, phase ^ 1u, err, 1);
                    if (!ok) break;
                    mbar_expect_tx(full0 + 8 * s, L::STAGE_BYTES);
                    const unsigned a_dst = tiles0 + s * L::STAGE_BYTES;
                    tma_load_2d(a_dst, &map_a, kb * BK, m0, full0 + 8 * s);
                    tma_load_2d(a_dst + L::A_BYTES, &map_b, kb * BK, n0, full0 + 8 * s);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const unsigned idesc = instr_desc(BM, BN);
            int it = 0, local = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++local) {
                const int acc = local & 1;
                const unsigned acc_phase = (unsigned)(local >> 1) & 1u;
                ok = mbar_wait(acc_empty0 + 8 * acc, acc_phase ^ 1u, err, 4);   // the epilogue has drained it
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned tmem_acc = tmem_base + (unsigned)(acc * BN);
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    const unsigned phase = (unsigned)(it / STAGES) & 1u;
                    ok = mbar_wait(full0 + 8 * s, phase, err, 2);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const unsigned a_addr = tiles0 + s * L::STAGE_BYTES;
                    const unsigned b_addr = a_addr + L::A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)
                        mma_f16(tmem_acc, smem_desc(a_addr + k * 32), smem_desc(b_addr + k * 32), idesc,
                                (kb > 0 || k > 0) ? 1u : 0u);
                    mma_commit(empty0 + 8 * s);
                }
                mma_commit(acc_full0 + 8 * acc);
            }
        }
    } else {
        const int quarter = warp & 3;
        int local = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++local) {
            const int m0 = (t % m_tiles) * BM, n0 = (t / m_tiles) * BN;
            const int acc = local & 1;
            const unsigned acc_phase = (unsigned)(local >> 1) & 1u;
            const int row = m0 + quarter * 32 + lane;
            const float ss = row_sum(rs, row, M);        // asked for while the tile's products still run
            ok = mbar_wait(acc_full0 + 8 * acc, acc_phase, err, 3);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float sc = rs.part ? 1.0f / sqrtf(ss * rs.inv_dim + rs.eps) : 1.f;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                if (n0 + c0 >= N) break;
                unsigned r[32];
                tmem_ld32(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(acc * BN + c0), r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (rs.part) scale_chunk(r, sc);
                if (row < M) store_chunk(r, row, n0 + c0, N, mode, bias, out, ldo);
            }
            // this warp has read its lanes of the accumulator: hand it back
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty0 + 8 * acc) : "memory");
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

int sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

template <int STAGES>
int launch_wide(const void* X, const void* W, const float* bias, void* out, int mode, int M, int N, int K, int ldo,
                const RowScale& rs, int* err, cudaStream_t stream) {
    using L = WideLayout<STAGES>;
    CUtensorMap ma, mb;
    if (!tensor_map(X, M, K, BM, &ma) || !tensor_map(W, N, K, L::BN, &mb)) return (int)cudaErrorInvalidValue;
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(gemm_tc_wide_kernel<STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        attr_set = true;
    }
    const int tiles = ((M + BM - 1) / BM) * ((N + L::BN - 1) / L::BN);
    const int blocks = tiles < sm_count() ? tiles : sm_count();
    gemm_tc_wide_kernel<STAGES><<<blocks, THREADS, L::TOTAL, stream>>>(ma, mb, bias, out, mode, M, N, K, ldo, rs, err);
    return mv_launch_status();
}

template <int BN, int STAGES>
int launch(const void* X, const void* W, const float* bias, void* out, int mode, int M, int N, int K, int ldo,
           const RowScale& rs, int* err, cudaStream_t stream) {
    using L = SmemLayout<BN, STAGES>;
    CUtensorMap ma, mb;
    if (!tensor_map(X, M, K, BM, &ma) || !tensor_map(W, N, K, BN, &mb)) return (int)cudaErrorInvalidValue;
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        attr_set = true;
    }
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    gemm_tc_kernel<BN, STAGES><<<grid, THREADS, L::TOTAL, stream>>>(ma, mb, bias, out, mode, M, N, K, ldo, rs, err);
    return mv_launch_status();
}

}  // namespace

// mode: 0 store float32, 1 store bfloat16, 2 add into float32, 3 SwiGLU (W rows in groups
// of 16 gate + 16 up; out is bfloat16 [M, N/2] with row stride ldo).  ``err`` points to a
// device int that a block sets (1 producer, 2 MMA, 3 epilogue) if a wait ran out.
// Needs K a multiple of 8 and 16-byte aligned operands.  scale_part (or null): the consuming end of a
// carried norm, [M][scale_stride] with n_scale_part sums of squares a row over ``dim`` elements.
MV_API int mv_gemm_tc(const void* X, const void* W, const float* bias, void* out, int mode, int M, int N,
                      int K, int ldo, const float* scale_part, int n_scale_part, int scale_stride, int dim, float eps,
                      int* err, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || ((uintptr_t)X & 15) || ((uintptr_t)W & 15)) return (int)cudaErrorInvalidValue;
    if (mode == 3 && (N % 32 || ldo % 2)) return (int)cudaErrorInvalidValue;
    if (scale_part && (n_scale_part <= 0 || n_scale_part > scale_stride || dim <= 0)) return (int)cudaErrorInvalidValue;
    RowScale rs = {};
    if (scale_part) rs = RowScale{scale_part, n_scale_part, scale_stride, 1.0f / (float)dim, eps};
    if (N <= 64) return launch<64, 4>(X, W, bias, out, mode, M, N, K, ldo, rs, err, stream);
    // wide enough for 128 x 256 tiles to give every SM work: the persistent kernel
    const long long wide_tiles = (long long)((M + BM - 1) / BM) * ((N + 255) / 256);
    if (N >= 256 && wide_tiles >= 96) return launch_wide<4>(X, W, bias, out, mode, M, N, K, ldo, rs, err, stream);
    return launch<128, 3>(X, W, bias, out, mode, M, N, K, ldo, rs, err, stream);
}
