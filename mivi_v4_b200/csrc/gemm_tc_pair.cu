// Y[M, N] = X[M, K] . W[N, K]^T for many rows, with TWO multiprocessors on one
// 256 x 256 tile of Y (tcgen05.mma.cta_group::2): the matrix product of prefill
// where the output is large enough to give every pair work.
//
// Why a pair.  A 128 x 256 tile on one multiprocessor needs 48 KB of operands per
// 128 x 256 x 64 of MMA work: 96 bytes a clock read by the tensor core at full
// rate, and as many again written by TMA, against the 128 bytes a clock that a
// multiprocessor's shared memory delivers; the one-SM kernel (gemm_tc.cu) is bound
// by that (tensor pipe 67 % busy on the widest product).  With cta_group::2 each
// block of a pair holds its own 128 rows of X and only HALF of the tile's 256 rows
// of W (the tensor cores of the pair read each other's half), so a block's operand
// traffic per K block drops from 48 KB to 32 KB for the same MMA work per SM.
//
// The pair (a cluster of two blocks; rank 0 leads):
//   warp 0   in BOTH blocks one lane issues the TMA loads of its block's operand
//            halves into its own ring of STAGES buffers; the bytes of both blocks
//            are counted on the LEADER's "full" barrier of the stage (the loads carry
//            .cta_group::2 and no multicast; each block reads global memory itself);
//   warp 1   allocates tensor memory in both blocks (one allocation of the pair);
//            in the leader one lane issues four 256 x 256 x 16 MMAs per K block and
//            commits them to the stage's "empty" barrier of BOTH blocks, at a tile's
//            end to the "accumulator full" barrier of both;
//   warps 2-5 in both blocks drain their block's 128 rows of the accumulator (two
//            accumulators of 256 columns alternate, so the drain of one tile runs
//            under the MMAs of the next) and arrive on the leader's "accumulator
//            empty" barrier.
// Every wait is bounded as in gemm_tc.cu; a block that gives up still reaches the
// pair's final barrier, so its peer is never left waiting for it.
//
// Reference counterpart: quantized_matmul_rows, out[b, n] = sum_d in[b, d] W[n, d]
// (crates/mivi-quant/src/lib.rs:143-245).
#include "tc_common.cuh"

namespace {

constexpr int PAIR_THREADS = 192;
constexpr int PAIR_BN = 256;          // columns of Y a pair's tile has; each block holds 128 rows of W for them

#include "gemm_tc_store.cuh"

// The two optional ends of a norm carried by products (as in gemm_small_m.cu and gemm_tc_swap.cu; all
// null / 0 when unused): a product that reads rows which still lack their norm's scale multiplies
// every row of its result by rsqrt(sum of the row's partial sums / dim + eps); a product that adds into
// the residual stream also writes bf16(x_new * g) and, per row and tile of 256 columns, the sum of x_new^2.
struct PairLink {
    const float* scale_part;           // consumer: [rows][scale_stride], n_scale_part sums of squares per row it reads
    int n_scale_part, scale_stride;
    float inv_dim, eps;
    const float* emit_g;               // producer (mode 2): the next norm's weight [N]
    __nv_bfloat16* emit_x;             // bf16(x_new * g) [M, N]
    float* emit_part;                  // [rows][emit_stride]
    int emit_stride;
    int by_rows;                       // float32 results in whole chunks of 32 columns: the epilogue stores by rows
};

template <int STAGES>
struct PairLayout {
    static constexpr int A_BYTES = BM * BK * 2, B_BYTES = (PAIR_BN / 2) * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;                 // of one block
    static constexpr int TILE_BYTES = STAGES * STAGE_BYTES;
    static constexpr int TURN_BYTES = 4 * 32 * 32 * 4;                    // each epilogue warp turns 32 x 32 floats
    static constexpr int BAR_BYTES = (2 * STAGES + 4) * 8 + 8;
    static constexpr int TOTAL = TILE_BYTES + TURN_BYTES + BAR_BYTES + 1024;
};

__device__ __forceinline__ unsigned cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// the address, in the cluster's shared window, of ``addr`` (an address of this block) in block ``rank``
__device__ __forceinline__ unsigned in_block(unsigned addr, unsigned rank) {
    unsigned out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
    return out;
}
__device__ __forceinline__ void pair_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(unsigned dst, const CUtensorMap* map, int x, int y, unsigned leader_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(leader_bar) : "memory");
}
__device__ __forceinline__ void mma_f16_pair(unsigned tmem_d, unsigned long long a, unsigned long long b, unsigned idesc,
                                             unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives on the barrier at this offset in both blocks of the pair once the MMAs issued so far are done
__device__ __forceinline__ void mma_commit_pair(unsigned bar) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(bar), "h"((unsigned short)3) : "memory");
}
__device__ __forceinline__ void arrive_remote(unsigned cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

template <int STAGES>
__global__ void __launch_bounds__(PAIR_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const float* __restrict__ bias, void* __restrict__ out, int mode, int M, int N, int K, int ldo,
                    const PairLink link, int* __restrict__ err) {
    using L = PairLayout<STAGES>;
    constexpr int BN = PAIR_BN;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned long long* bars = (unsigned long long*)(smem + L::TILE_BYTES + L::TURN_BYTES);
    unsigned* tmem_holder = (unsigned*)(bars + 2 * STAGES + 4);
    const unsigned full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES;
    const unsigned acc_full0 = full0 + 16 * STAGES, acc_empty0 = acc_full0 + 16;
    const unsigned tiles0 = smem_u32(smem);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned rank = cluster_rank();
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int m_tiles = (M + 2 * BM - 1) / (2 * BM), n_tiles = (N + BN - 1) / BN;
    const int tiles = m_tiles * n_tiles;
    const int kblocks = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);                  // the leader's: its producer's arrival, the bytes of both blocks
            mbar_init(empty0 + 8 * s, 1);                 // each block's own: the leader's commit reaches both
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(acc_full0 + 8 * a, 1);              // each block's own
            mbar_init(acc_empty0 + 8 * a, 8);             // the leader's: four epilogue warps of each block
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_holder)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    pair_sync();                                          // both blocks' barriers and tensor memory are there
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_base = *tmem_holder;
    mv_pdl_begin();                                       // X and Y belong to the kernel before until here

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;                                   // K blocks issued so far, over all tiles
            bool ok = true;
            for (int t = pair; t < tiles && ok; t += n_pairs) {
                const int m0 = (t % m_tiles) * 2 * BM + (int)rank * BM;
                const int n0 = (t / m_tiles) * BN + (int)rank * (BN / 2);
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    const unsigned phase = (unsigned)(it / STAGES) & 1u;
                    ok = mbar_wait(empty0 + 8 * s, phase ^ 1u, err, 1);
                    if (!ok) break;
                    if (leader) mbar_expect_tx(full0 + 8 * s, 2 * L::STAGE_BYTES);
                    const unsigned bar = in_block(full0 + 8 * s, 0);
                    const unsigned a_dst = tiles0 + s * L::STAGE_BYTES;
                    tma_load_2d_pair(a_dst, &map_a, kb * BK, m0, bar);
                    tma_load_2d_pair(a_dst + L::A_BYTES, &map_b, kb * BK, n0, bar);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            const unsigned idesc = instr_desc(2 * BM, BN);
            int it = 0, local = 0;
            bool ok = true;
            for (int t = pair; t < tiles && ok; t += n_pairs, ++local) {
                const int acc = local & 1;
                const unsigned acc_phase = (unsigned)(local >> 1) & 1u;
                ok = mbar_wait(acc_empty0 + 8 * acc, acc_phase ^ 1u, err, 4);   // both blocks have drained it
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
                        mma_f16_pair(tmem_acc, smem_desc(a_addr + k * 32), smem_desc(b_addr + k * 32), idesc,
                                     (kb > 0 || k > 0) ? 1u : 0u);
                    mma_commit_pair(empty0 + 8 * s);
                }
                mma_commit_pair(acc_full0 + 8 * acc);
            }
        }
    } else {
        const int quarter = warp & 3;
        float* turn = (float*)(smem + L::TILE_BYTES) + quarter * (32 * 32);
        const bool by_rows = link.by_rows != 0;
        int local = 0;
        bool ok = true;
        for (int t = pair; t < tiles && ok; t += n_pairs, ++local) {
            const int m0 = (t % m_tiles) * 2 * BM + (int)rank * BM, n0 = (t / m_tiles) * BN;
            const int acc = local & 1;
            const unsigned acc_phase = (unsigned)(local >> 1) & 1u;
            const int row = m0 + quarter * 32 + lane;
            // What the epilogue needs from memory is asked for before the wait for the accumulator, while
            // the tile's products still run: a carried norm's partial sums of this row, and the first old
            // values of the residual stream where the product hands the next norm on.
            float ss = 0.f;
            if (link.scale_part && row < M) {
                for (int p = 0; p < link.n_scale_part; ++p) ss += link.scale_part[(size_t)row * link.scale_stride + p];
            }
            // Float32 results in whole chunks of 32 columns go to memory by rows: a warp turns its 32 x 32
            // values in shared memory, so that one instruction covers 4 rows of 128 contiguous bytes instead
            // of 16 bytes of each of 32 rows.  There lane l has the columns 4 (l % 8) .. + 3 of the rows
            // l / 8 + 4 i.
            const int sub = lane >> 3, c4 = lane & 7;
            const int row0 = m0 + quarter * 32 + sub;
            float* op = (float*)out + (size_t)row0 * ldo + n0 + 4 * c4;
            float4 old[8], nxt[8];
            auto request = [&](int c, float4 (&dst)[8]) {
                if (n0 + 32 * c < N) {
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        if (row0 + 4 * i < M) dst[i] = *reinterpret_cast<const float4*>(op + (size_t)(4 * i) * ldo + 32 * c);
                }
            };
            if (link.emit_x) request(0, old);
            ok = mbar_wait(acc_full0 + 8 * acc, acc_phase, err, 3);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float sc = link.scale_part ? 1.0f / sqrtf(ss * link.inv_dim + link.eps) : 1.f;
            if (by_rows) {
                float sq[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) sq[i] = 0.f;
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    if (n0 + 32 * c >= N) break;
                    unsigned r[32];
                    tmem_ld32(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(acc * BN + 32 * c), r);
                    if (link.emit_x && c + 1 < BN / 32) request(c + 1, nxt);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    // 16-byte piece q of row ``lane`` lies at piece q ^ (lane % 8): no bank is asked twice, neither here nor below
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        *reinterpret_cast<float4*>(turn + lane * 32 + ((q ^ (lane & 7)) << 2)) =
                            make_float4(__uint_as_float(r[4 * q]) * sc, __uint_as_float(r[4 * q + 1]) * sc,
                                        __uint_as_float(r[4 * q + 2]) * sc, __uint_as_float(r[4 * q + 3]) * sc);
                    __syncwarp();
                    float4 b4 = make_float4(0.f, 0.f, 0.f, 0.f), g4 = b4;
                    if (bias) b4 = *reinterpret_cast<const float4*>(bias + n0 + 32 * c + 4 * c4);
                    if (link.emit_x) g4 = *reinterpret_cast<const float4*>(link.emit_g + n0 + 32 * c + 4 * c4);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int rl = sub + 4 * i;
                        float4 v = *reinterpret_cast<const float4*>(turn + rl * 32 + ((c4 ^ (rl & 7)) << 2));
                        v.x += b4.x; v.y += b4.y; v.z += b4.z; v.w += b4.w;
                        if (row0 + 4 * i < M) {
                            float4* p = reinterpret_cast<float4*>(op + (size_t)(4 * i) * ldo + 32 * c);
                            if (link.emit_x) {
                                // completes the residual stream and hands the next norm on
                                v.x += old[i].x; v.y += old[i].y; v.z += old[i].z; v.w += old[i].w;
                                *p = v;
                                const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x * g4.x, v.y * g4.y);
                                const __nv_bfloat162 hi = __floats2bfloat162_rn(v.z * g4.z, v.w * g4.w);
                                *reinterpret_cast<uint2*>(link.emit_x + (size_t)(row0 + 4 * i) * N + n0 + 32 * c + 4 * c4) =
                                    make_uint2(*reinterpret_cast<const unsigned*>(&lo), *reinterpret_cast<const unsigned*>(&hi));
                                sq[i] = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, sq[i]))));
                            } else if (mode == 2) {
                                // added in memory: nothing comes back, so the epilogue does not wait for a read
                                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                                             ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
                            } else {
                                *p = v;
                            }
                        }
                    }
                    __syncwarp();                         // the values are out before the next chunk is turned
                    if (link.emit_x) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) old[i] = nxt[i];
                    }
                }
                if (link.emit_x) {
                    // a row's sum of squares over the tile: its eight lanes' sums together
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        sq[i] += __shfl_xor_sync(0xffffffffu, sq[i], 1);
                        sq[i] += __shfl_xor_sync(0xffffffffu, sq[i], 2);
                        sq[i] += __shfl_xor_sync(0xffffffffu, sq[i], 4);
                        if (c4 == 0 && row0 + 4 * i < M)
                            link.emit_part[(size_t)(row0 + 4 * i) * link.emit_stride + n0 / BN] = sq[i];
                    }
                }
            } else {
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    if (n0 + c0 >= N) break;
                    unsigned r[32];
                    tmem_ld32(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(acc * BN + c0), r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (link.scale_part) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * sc);
                    }
                    if (row < M) store_chunk(r, row, n0 + c0, N, mode, bias, out, ldo);
                }
            }
            // this warp has read its lanes of the accumulator: tell the leader's MMA warp
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) arrive_remote(in_block(acc_empty0 + 8 * acc, 0));
        }
    }
    // nobody leaves while its peer may still read its shared memory or signal its barriers
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    pair_sync();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

template <int STAGES>
int launch_pair(const void* X, const void* W, const float* bias, void* out, int mode, int M, int N, int K, int ldo,
                const PairLink& link, int* err, cudaStream_t stream) {
    using L = PairLayout<STAGES>;
    CUtensorMap ma, mb;
    if (!tensor_map(X, M, K, BM, &ma) || !tensor_map(W, N, K, PAIR_BN / 2, &mb)) return (int)cudaErrorInvalidValue;
    static int max_pairs = 0;
    if (max_pairs == 0) {
        cudaFuncSetAttribute(gemm_tc_pair_kernel<STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        int dev = 0, sms = 148;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        // how many pairs the device runs at once (a pair needs two free multiprocessors of one group)
        cudaLaunchConfig_t probe = {};
        probe.gridDim = dim3((unsigned)sms);
        probe.blockDim = dim3(PAIR_THREADS);
        probe.dynamicSmemBytes = L::TOTAL;
        cudaLaunchAttribute pa[1];
        pa[0].id = cudaLaunchAttributeClusterDimension;
        pa[0].val.clusterDim.x = 2; pa[0].val.clusterDim.y = 1; pa[0].val.clusterDim.z = 1;
        probe.attrs = pa;
        probe.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_pair_kernel<STAGES>, &probe) != cudaSuccess || n <= 0) n = sms / 2;
        max_pairs = n < sms / 2 ? n : sms / 2;
        cudaGetLastError();
    }
    const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + PAIR_BN - 1) / PAIR_BN);
    const int pairs = tiles < max_pairs ? tiles : max_pairs;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * pairs));
    cfg.blockDim = dim3(PAIR_THREADS);
    cfg.dynamicSmemBytes = L::TOTAL;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = mv_pdl_enabled() ? 2 : 1;
    cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel<STAGES>, ma, mb, bias, out, mode, M, N, K, ldo, link, err);
    return mv_launch_status();
}

}  // namespace

// Same contract as mv_gemm_tc (gemm_tc.cu); for M > 128.  Returns cudaErrorInvalidValue for shapes it
// does not take (the caller then uses mv_gemm_tc).
MV_API int mv_gemm_tc_pair(const void* X, const void* W, const float* bias, void* out, int mode, int M, int N,
                           int K, int ldo, const float* scale_part, int n_scale_part, int scale_stride, int dim,
                           float eps, const float* emit_g, void* emit_x, float* emit_part, int emit_stride, int* err,
                           cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || ((uintptr_t)X & 15) || ((uintptr_t)W & 15)) return (int)cudaErrorInvalidValue;
    if (mode == 3 && (N % 32 || ldo % 2)) return (int)cudaErrorInvalidValue;
    if (M <= BM || N < PAIR_BN / 2) return (int)cudaErrorInvalidValue;
    // an emitting product writes rows of 32 columns in 16-byte pieces: N in steps of 32, aligned buffers
    if (emit_x && (mode != 2 || ldo != N || N % 32 || !emit_g || !emit_part || emit_stride < (N + PAIR_BN - 1) / PAIR_BN ||
                   (((uintptr_t)out | (uintptr_t)emit_x | (uintptr_t)emit_g | (uintptr_t)bias) & 15)))
        return (int)cudaErrorInvalidValue;
    if (scale_part && (n_scale_part <= 0 || n_scale_part > scale_stride || dim <= 0)) return (int)cudaErrorInvalidValue;
    PairLink link = {};
    if (scale_part) {
        link.scale_part = scale_part;
        link.n_scale_part = n_scale_part;
        link.scale_stride = scale_stride;
        link.inv_dim = 1.0f / (float)dim;
        link.eps = eps;
    }
    if (emit_x) {
        link.emit_g = emit_g;
        link.emit_x = (__nv_bfloat16*)emit_x;
        link.emit_part = emit_part;
        link.emit_stride = emit_stride;
    }
    link.by_rows = (mode == 0 || mode == 2) && N % 32 == 0 && ldo % 4 == 0 && !(((uintptr_t)out | (uintptr_t)bias) & 15);
    if (emit_x && !link.by_rows) return (int)cudaErrorInvalidValue;
    return launch_pair<6>(X, W, bias, out, mode, M, N, K, ldo, link, err, stream);
}
