// Y[M, N] = X[M, K] . W[N, K]^T for a decode step (M <= 64 tokens) on the
// fifth-generation tensor cores, with the roles of the operands swapped: a tile
// of 128 rows of W is the MMA's M side, the tokens are its N side (16, 32 or 64
// columns of tensor memory).  The cost of the step is reading W once, so the
// kernel is a pipeline that keeps TMA loads of W in flight: one lane issues the
// loads of 128 x 64 tiles into a ring of stages, one lane issues the MMAs and
// hands the stages back, and nothing passes through registers until the end.
//
// A block owns one row tile and one slice of K; the slices of a tile form a
// thread-block cluster.  Each block moves its accumulator from tensor memory to
// shared memory; the cluster's first block adds the slices in rank order through
// distributed shared memory and runs the epilogue (store float32 / bfloat16, add
// into float32, or SwiGLU over rows grouped 16 gate + 16 up; optional bias).
// Every sum has a fixed order.  Waits on mbarriers are bounded (see
// tc_common.cuh); the cluster barrier is the hardware's.
//
// Reference counterpart: quantized_matvec (crates/mivi-quant/src/lib.rs:75-135).
#include <cooperative_groups.h>

#include "tc_common.cuh"

namespace cg = cooperative_groups;

namespace {

constexpr int THREADS = 192;

// The two optional ends of a norm carried by products (see gemm_small_m.cu; all null / 0 when unused).
struct NormLink {
    const float* scale_part;           // consumer: [tokens][scale_stride], n_scale_part sums of squares per row it reads
    int n_scale_part, scale_stride;
    float inv_dim, eps;
    const float* emit_g;               // producer (mode 2): the next norm's weight [N]
    __nv_bfloat16* emit_x;             // bf16(x_new * g) [M, N]
    float* emit_part;                  // [tokens][emit_stride] sums of x_new^2 over each tile's 128 rows
    int emit_stride;
};

template <int BN, int STAGES>
struct SwapLayout {
    static constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int TILE_BYTES = STAGES * STAGE_BYTES;
    static constexpr int CSUM_BYTES = BM * BN * 4;   // [token][row]: a warp reads consecutive words
    static constexpr int BAR_BYTES = (2 * STAGES + 1) * 8 + 8;
    static constexpr int TOTAL = (TILE_BYTES > CSUM_BYTES ? TILE_BYTES : CSUM_BYTES) + BAR_BYTES + 1024;
    static constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(THREADS)
gemm_tc_swap_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    const float* __restrict__ bias, void* __restrict__ out, int mode, int M, int N, int K, int ldo,
                    const NormLink link, int* __restrict__ err) {
    using L = SwapLayout<BN, STAGES>;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    constexpr int DATA_BYTES = L::TILE_BYTES > L::CSUM_BYTES ? L::TILE_BYTES : L::CSUM_BYTES;
    unsigned long long* bars = (unsigned long long*)(smem + DATA_BYTES);
    unsigned* tmem_holder = (unsigned*)(bars + 2 * STAGES + 1);
    float* csum = reinterpret_cast<float*>(smem);       // reuses the ring once the MMAs are done
    const unsigned full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES, acc_bar = full0 + 16 * STAGES;
    const unsigned tiles0 = smem_u32(smem);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int slices = gridDim.x, slice = blockIdx.x;
    const int n0 = blockIdx.y * BM;
    const int kblocks = (K + BK - 1) / BK;
    const int per = (kblocks + slices - 1) / slices;
    const int kb0 = slice * per;
    const int nkb = max(0, min(kblocks, kb0 + per) - kb0);

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
                     ::"r"(smem_u32(tmem_holder)), "r"((unsigned)L::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_base = *tmem_holder;

    bool acc_ok = nkb > 0;
    // Under programmatic dependent launch this block may have started while the kernel before it is
    // still running.  The weights do not depend on that kernel: the ring's first round of W tiles is
    // requested at once; X, and everything the epilogue reads, only after the wait.
    mv_pdl_launch_dependents();
    if (warp == 0) {
        if (lane == 0) {
            const int first = nkb < STAGES ? nkb : STAGES;
            for (int i = 0; i < first; ++i) {
                mbar_expect_tx(full0 + 8 * i, L::STAGE_BYTES);
                tma_load_2d(tiles0 + i * L::STAGE_BYTES, &map_w, (kb0 + i) * BK, n0, full0 + 8 * i);
            }
            mv_pdl_wait();
            for (int i = 0; i < first; ++i)
                tma_load_2d(tiles0 + i * L::STAGE_BYTES + L::A_BYTES, &map_x, (kb0 + i) * BK, 0, full0 + 8 * i);
            for (int i = first; i < nkb; ++i) {
                const int s = i % STAGES;
                const unsigned phase = (unsigned)(i / STAGES) & 1u;
                if (!mbar_wait(empty0 + 8 * s, phase ^ 1u, err, 1)) break;
                mbar_expect_tx(full0 + 8 * s, L::STAGE_BYTES);
                const unsigned a_dst = tiles0 + s * L::STAGE_BYTES;
                tma_load_2d(a_dst, &map_w, (kb0 + i) * BK, n0, full0 + 8 * s);
                tma_load_2d(a_dst + L::A_BYTES, &map_x, (kb0 + i) * BK, 0, full0 + 8 * s);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && nkb > 0) {
            const unsigned idesc = instr_desc(BM, BN);
            for (int i = 0; i < nkb; ++i) {
                const int s = i % STAGES;
                const unsigned phase = (unsigned)(i / STAGES) & 1u;
                if (!mbar_wait(full0 + 8 * s, phase, err, 2)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned a_addr = tiles0 + s * L::STAGE_BYTES;
                const unsigned b_addr = a_addr + L::A_BYTES;
#pragma unroll
                for (int k = 0; k < BK / 16; ++k)
                    mma_f16(tmem_base, smem_desc(a_addr + k * 32), smem_desc(b_addr + k * 32), idesc,
                            (i > 0 || k > 0) ? 1u : 0u);
                mma_commit(empty0 + 8 * s);
            }
            mma_commit(acc_bar);
        }
    } else {
        // this block's accumulator: tensor memory -> shared memory, rows = rows of W, columns = tokens
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        if (acc_ok) acc_ok = mbar_wait(acc_bar, 0, err, 3);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
            unsigned v[32];
            if (acc_ok) {
                tmem_ld32(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)c0, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = 0u;
            }
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (c0 + j < BN) csum[(c0 + j) * BM + r] = __uint_as_float(v[j]);      // [token][row]
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");

    // The slices of this tile are added in rank order.  The work of adding is dealt out to all blocks
    // of the cluster: an item is 32 consecutive rows for one token (a warp, one row per lane), item i
    // belongs to block i mod slices.  A lane first requests its value from every slice, then adds.
    mv_pdl_wait();                 // the epilogue reads (and overwrites) what the kernel before may still use
    const float* share[8];
    if (slices > 1) {
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        for (int s = 0; s < slices; ++s) share[s] = cluster.map_shared_rank(csum, s);
    } else {
        __syncthreads();
        share[0] = csum;
    }
    {
        // An item is the tile's 128 rows for one token, four consecutive rows per lane (16-byte reads
        // through distributed shared memory, 16-byte stores).  A warp takes its items two at a time:
        // first every load of both (the slices' sums, and the old values where the product is added
        // to memory), then the arithmetic and the stores - so the round trips overlap.
        constexpr int CH = 2, WARPS_ALL = THREADS / 32;
        const int r = 4 * lane, n = n0 + r;
        const bool vec_ok = n + 3 < N && (ldo & 3) == 0 && ((uintptr_t)out & 15) == 0;   // else one by one
        for (int m0 = slice + slices * warp; m0 < M; m0 += CH * slices * WARPS_ALL) {
            float4 part[CH][8], old[CH];
            float ss[CH];
#pragma unroll
            for (int c = 0; c < CH; ++c) {
                const int m = m0 + c * slices * WARPS_ALL;
                // a carried norm's sums of this token: lane p holds sums p, p + 32, ...
                ss[c] = 0.f;
                if (link.scale_part && m < M)
                    for (int p = lane; p < link.n_scale_part; p += 32)
                        ss[c] += link.scale_part[(size_t)m * link.scale_stride + p];
#pragma unroll
                for (int s = 0; s < 8; ++s)
                    part[c][s] = (m < M && s < slices) ? *reinterpret_cast<const float4*>(share[s] + m * BM + r)
                                                       : make_float4(0.f, 0.f, 0.f, 0.f);
                old[c] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (mode == 2 && m < M) {
                    const float* o = (const float*)out + (size_t)m * ldo + n;
                    if (vec_ok) old[c] = *reinterpret_cast<const float4*>(o);
                    else {
                        if (n < N) old[c].x = o[0];
                        if (n + 1 < N) old[c].y = o[1];
                        if (n + 2 < N) old[c].z = o[2];
                        if (n + 3 < N) old[c].w = o[3];
                    }
                }
            }
#pragma unroll
            for (int c = 0; c < CH; ++c) {
                const int m = m0 + c * slices * WARPS_ALL;
                if (m >= M) break;
                float v[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int s = 0; s < 8; ++s) {
                    v[0] += part[c][s].x; v[1] += part[c][s].y; v[2] += part[c][s].z; v[3] += part[c][s].w;
                }
                if (link.scale_part) {
                    const float sc = 1.0f / sqrtf(mv_warp_sum(ss[c]) * link.inv_dim + link.eps);
#pragma unroll
                    for (int e = 0; e < 4; ++e) v[e] *= sc;
                }
                if (bias) {
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        if (n + e < N) v[e] += bias[n + e];
                }
                if (mode == 3) {
                    // rows in groups of 16 gate + 16 up: of every 8 lanes the first 4 hold gate rows,
                    // the next 4 the up rows of the same features
                    float up[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) up[e] = __shfl_down_sync(0xffffffffu, v[e], 4);
                    if ((lane & 4) == 0 && n + 16 < N) {
                        __nv_bfloat16* o = (__nv_bfloat16*)out + (size_t)m * ldo + (n >> 5) * 16 + (r & 15);
#pragma unroll
                        for (int e = 0; e < 4; ++e) o[e] = __float2bfloat16_rn(v[e] / (1.0f + expf(-v[e])) * up[e]);
                    }
                } else {
                    const size_t o = (size_t)m * ldo + n;
                    if (mode == 2) { v[0] += old[c].x; v[1] += old[c].y; v[2] += old[c].z; v[3] += old[c].w; }
                    if (mode == 1) {
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            if (n + e < N) ((__nv_bfloat16*)out)[o + e] = __float2bfloat16_rn(v[e]);
                    } else if (vec_ok) {
                        *reinterpret_cast<float4*>((float*)out + o) = make_float4(v[0], v[1], v[2], v[3]);
                    } else {
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            if (n + e < N) ((float*)out)[o + e] = v[e];
                    }
                    if (mode == 2 && link.emit_x) {
                        // the next norm's rows and this tile's share of the token's sum of squares
                        float sq = 0.f;
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            if (n + e < N) {
                                link.emit_x[(size_t)m * N + n + e] = __float2bfloat16_rn(v[e] * link.emit_g[n + e]);
                                sq = fmaf(v[e], v[e], sq);
                            }
                        sq = mv_warp_sum(sq);
                        if (lane == 0) link.emit_part[(size_t)m * link.emit_stride + blockIdx.y] = sq;
                    }
                }
            }
        }
    }
    // nobody leaves while another block may still read its shared memory
    if (slices > 1) mv_cluster_sync_relaxed();
    else __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"((unsigned)L::TMEM_COLS) : "memory");
    }
}

// Slices of K (at most 8, the portable cluster size): as many blocks as fit the GPU at two a
// multiprocessor, each with at least two K blocks.
int k_slices(int N, int K) {
    const int tiles = (N + BM - 1) / BM, kblocks = (K + BK - 1) / BK;
    int slices = 2 * 148 / tiles;
    slices = slices >= 8 ? 8 : (slices >= 4 ? 4 : (slices >= 2 ? 2 : 1));   // clusters of other sizes schedule worse
    while (slices > 1 && kblocks / slices < 2) slices >>= 1;
    return slices < 1 ? 1 : slices;
}

template <int BN, int STAGES>
int launch(const void* X, const void* W, const float* bias, void* out, int mode, int M, int N, int K, int ldo,
           const NormLink& link, int* err, cudaStream_t stream) {
    using L = SwapLayout<BN, STAGES>;
    CUtensorMap mw, mx;
    if (!tensor_map(W, N, K, BM, &mw) || !tensor_map(X, M, K, BN, &mx)) return (int)cudaErrorInvalidValue;
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(gemm_tc_swap_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        attr_set = true;
    }
    const int tiles = (N + BM - 1) / BM;
    const int slices = k_slices(N, K);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(slices, tiles);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = L::TOTAL;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (mv_pdl_enabled()) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    if (slices > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = slices;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    cudaLaunchKernelEx(&cfg, gemm_tc_swap_kernel<BN, STAGES>, mw, mx, bias, out, mode, M, N, K, ldo, link, err);
    return mv_launch_status();
}

}  // namespace

// Same contract as mv_gemm_small_m (modes 0-3, 1 <= M <= 64, K a multiple of 8,
// 16-byte aligned operands; scale_part / emit_x as there, with one sum per tile of 128 rows), plus
// the error flag of the bounded waits.
MV_API int mv_gemm_tc_swap(const void* X, const void* W, const float* bias, void* out, int mode, int M, int N,
                           int K, int ldo, const float* scale_part, int n_scale_part, int scale_stride, int dim,
                           float eps, const float* emit_g, void* emit_x, float* emit_part, int emit_stride,
                           int* err, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 64 || K <= 0 || K % 8 || ((uintptr_t)X & 15) || ((uintptr_t)W & 15)) return (int)cudaErrorInvalidValue;
    if (mode == 3 && N % 32) return (int)cudaErrorInvalidValue;
    if (emit_x && (mode != 2 || ldo != N || !emit_g || !emit_part || emit_stride < (N + BM - 1) / BM))
        return (int)cudaErrorInvalidValue;
    if (scale_part && (n_scale_part <= 0 || n_scale_part > scale_stride || dim <= 0)) return (int)cudaErrorInvalidValue;
    NormLink link = {};
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
    // A ring of 8 stages fills a multiprocessor's shared memory with one block.  Clusters of such
    // blocks need 8 free multiprocessors in one GPC each, and only 15 fit the GPU at a time: a
    // product that is cut along K takes 4 stages, so that two blocks share a multiprocessor.
    const bool deep = k_slices(N, K) == 1;
#define MV_GO(BN) return deep ? launch<BN, 8>(X, W, bias, out, mode, M, N, K, ldo, link, err, stream) \
                              : launch<BN, 4>(X, W, bias, out, mode, M, N, K, ldo, link, err, stream)
    if (M <= 16) MV_GO(16);
    if (M <= 32) MV_GO(32);
    MV_GO(64);
#undef MV_GO
}
