// Y[M, N] = X[M, K] . W[N, K]^T for a step of few tokens (a decode step, a short prompt) on the
// fifth-generation tensor cores, with the roles of the operands swapped: a tile
// of 128 rows of W is the MMA's M side, the tokens are its N side (16 to 128
// columns of tensor memory; more tokens than 128 are tiles of 128 along the grid's z, whose
// blocks find W in the L2 cache after the first).  The cost of the step is reading W once, so the
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

// The gated short convolution of a decode step as the epilogue of its input projection (TAIL 1;
// crates/mivi-model/src/ssm.rs:81-140).  The rows of W [3 H, K] come regrouped: 32 channels' B rows, then
// their C rows, then their x rows, group after group, so that a block's one tile of 96 rows (the MMA still
// works on 128: the last 32 rows of a stage are never loaded and their results never read) holds all three of
// its 32 channels.  The block count, the stage size and the two blocks a multiprocessor are those of the plain
// product.  After the slices are added a lane finishes one channel of a token: B * x, the k taps over the
// sequence's k-1 kept values, the shift of those, C *.
struct ConvTail {
    const float* taps;                 // [H][k]
    const float* conv_bias;            // [H] or null
    float* state;                      // [slots][k - 1][H], the last k-1 values of B * x per sequence
    const int* slots;                  // [M]: the slot of token m's sequence (one token a sequence)
    int k;
};

// The preparation of q, k and v as the epilogue of their fused projection (TAIL 2, head size 64, the
// pairs (2i, 2i+1); crates/mivi-model/src/transformer.rs:81-108): W is [(nh + 2 nkv) 64, K], query
// heads, then key heads, then value heads; a tile of 128 rows is two heads, a half-warp finishes one
// for a token with four elements a lane: RMSNorm over the head (q and k), rotation by the token's
// position (q and k), then q goes out in bfloat16 and k and v into the token's row of its cache page.
struct HeadTail {
    const float* wq;                   // [64] norm weight of the query heads, or null: no norm
    const float* wk;                   // the same for the key heads
    const float* inv_freq;             // [32] or null: no rotation
    const int* positions;              // [M]
    const int* seq_of;                 // [M] row of the page table
    const int* page_table;
    __nv_bfloat16* pool;               // [page][K, V][kv head][page_size][64]
    __nv_bfloat16* q_out;              // [M][nh * 64]
    long long page_stride;
    float eps;
    int table_stride, page_shift, nh, nkv;
};

// What the NEXT product of the step will read (or null): once a block's loads are all issued, the
// idle lanes of its loading warp ask the L2 cache for their share of these lines.
struct Ahead {
    const void* w;
    long long bytes;
};

template <int BN, int STAGES, int TAIL>
struct SwapLayout {
    static constexpr int W_ROWS = TAIL == 1 ? 96 : BM;   // rows of W that a tile loads (TAIL 1: 32 channels' B, C and x rows)
    static constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int TX_BYTES = W_ROWS * BK * 2 + B_BYTES;        // what the loads of a stage bring
    static constexpr int TILE_BYTES = STAGES * STAGE_BYTES;
    static constexpr int CSUM_BYTES = BM * BN * 4;        // [token][row]: a warp reads consecutive words
    static constexpr int BAR_BYTES = (2 * STAGES + 1) * 8 + 8;
    static constexpr int TOTAL = (TILE_BYTES > CSUM_BYTES ? TILE_BYTES : CSUM_BYTES) + BAR_BYTES + 1024;
    static constexpr int TMEM_COLS = BN <= 32 ? 32 : (BN <= 64 ? 64 : (BN <= 128 ? 128 : 256));
};

template <int BN, int STAGES, int TAIL>
__global__ void __launch_bounds__(THREADS)
gemm_tc_swap_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    const float* __restrict__ bias, void* __restrict__ out, int mode, int M, int N, int K, int ldo,
                    const NormLink link, const ConvTail tail, const HeadTail heads, const Ahead ahead,
                    int* __restrict__ err) {
    using L = SwapLayout<BN, STAGES, TAIL>;
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
    const int n0 = blockIdx.y * L::W_ROWS;
    const int mt0 = blockIdx.z * BN;                    // this block's first token (TAIL 1 and 2: always 0)
    const int m_end = min(M, mt0 + BN);
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
                mbar_expect_tx(full0 + 8 * i, L::TX_BYTES);
                tma_load_2d(tiles0 + i * L::STAGE_BYTES, &map_w, (kb0 + i) * BK, n0, full0 + 8 * i);
            }
            mv_pdl_wait();
            for (int i = 0; i < first; ++i)
                tma_load_2d(tiles0 + i * L::STAGE_BYTES + L::A_BYTES, &map_x, (kb0 + i) * BK, mt0, full0 + 8 * i);
            for (int i = first; i < nkb; ++i) {
                const int s = i % STAGES;
                const unsigned phase = (unsigned)(i / STAGES) & 1u;
                if (!mbar_wait(empty0 + 8 * s, phase ^ 1u, err, 1)) break;
                mbar_expect_tx(full0 + 8 * s, L::TX_BYTES);
                const unsigned a_dst = tiles0 + s * L::STAGE_BYTES;
                tma_load_2d(a_dst, &map_w, (kb0 + i) * BK, n0, full0 + 8 * s);
                tma_load_2d(a_dst + L::A_BYTES, &map_x, (kb0 + i) * BK, mt0, full0 + 8 * s);
            }
        }
        __syncwarp();
        if (ahead.w && ahead.bytes > 0 && blockIdx.z == 0) {
            // this block's own loads are on their way: ask L2 for the block's share of what comes next
            const long long lines = ahead.bytes >> 7;
            const long long nblk = (long long)gridDim.x * gridDim.y, me = (long long)blockIdx.y * gridDim.x + blockIdx.x;
            for (long long l = me * 32 + lane; l < lines; l += nblk * 32)
                asm volatile("prefetch.global.L2 [%0];" ::"l"((const char*)ahead.w + (l << 7)));
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
        for (int c0 = 0; c0 < BN; c0 += (BN < 32 ? BN : 32)) {
            unsigned v[32];
            if (acc_ok) {
                tmem_ld32(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)c0, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = 0u;
            }
#pragma unroll
            for (int j = 0; j < (BN < 32 ? BN : 32); ++j)
                csum[(c0 + j) * BM + r] = __uint_as_float(v[j]);      // [accumulator][token][row], column c0 + j
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
    constexpr int WARPS_ALL = THREADS / 32;
    if constexpr (TAIL == 1) {
        // An item is one token's 32 channels of this block, a channel a lane; N counts channels.
        const int d = 32 * (int)blockIdx.y + lane;
        const int k = tail.k;
        for (int m = slice + slices * warp; m < M; m += slices * WARPS_ALL) {
            float ss = 0.f;
            if (link.scale_part)
                for (int p = lane; p < link.n_scale_part; p += 32)
                    ss += link.scale_part[(size_t)m * link.scale_stride + p];
            float part[3][8];
#pragma unroll
            for (int t = 0; t < 3; ++t)
#pragma unroll
                for (int sl = 0; sl < 8; ++sl)
                    part[t][sl] = sl < slices ? share[sl][m * BM + 32 * t + lane] : 0.f;
            float v[3] = {0.f, 0.f, 0.f};
#pragma unroll
            for (int t = 0; t < 3; ++t)
#pragma unroll
                for (int sl = 0; sl < 8; ++sl) v[t] += part[t][sl];
            float sc = 1.f;
            if (link.scale_part) sc = 1.0f / sqrtf(mv_warp_sum(ss) * link.inv_dim + link.eps);
            if (d >= N) continue;
            float Bv = v[0] * sc, Cv = v[1] * sc, Xv = v[2] * sc;
            if (bias) { Bv += bias[d]; Cv += bias[N + d]; Xv += bias[2 * N + d]; }
            const float bx = Bv * Xv;
            float* st = tail.state + (size_t)tail.slots[m] * (k - 1) * N;
            float y = tail.conv_bias ? tail.conv_bias[d] : 0.f;
            for (int j = 0; j < k - 1; ++j) {
                const float old = st[(size_t)j * N + d];
                y = fmaf(tail.taps[d * k + j], old, y);
                if (j > 0) st[(size_t)(j - 1) * N + d] = old;        // shift towards the older end
            }
            if (k > 1) st[(size_t)(k - 2) * N + d] = bx;
            y = fmaf(tail.taps[d * k + (k - 1)], bx, y);
            ((__nv_bfloat16*)out)[(size_t)m * ldo + d] = __float2bfloat16_rn(Cv * y);
        }
    } else if constexpr (TAIL == 2) {
        // The heads: an item is the tile's two heads of one token; a half-warp holds a head, a lane four
        // consecutive elements of it, that is the pairs 2 sub and 2 sub + 1.
        const int sub = lane & 15, r = 4 * lane;
        const int hs = 2 * (int)blockIdx.y + (lane >> 4);
        const int n_slots = heads.nh + 2 * heads.nkv;
        const bool is_q = hs < heads.nh, is_k = !is_q && hs < heads.nh + heads.nkv;
        const float* w = is_q ? heads.wq : (is_k ? heads.wk : nullptr);
        float4 w4 = make_float4(1.f, 1.f, 1.f, 1.f);
        if (w) w4 = *reinterpret_cast<const float4*>(w + 4 * sub);
        const bool rotate = heads.inv_freq && (is_q || is_k);
        const float f0 = rotate ? heads.inv_freq[2 * sub] : 0.f, f1 = rotate ? heads.inv_freq[2 * sub + 1] : 0.f;
        for (int m = slice + slices * warp; m < M; m += slices * WARPS_ALL) {
            float ss = 0.f;
            if (link.scale_part)
                for (int p = lane; p < link.n_scale_part; p += 32)
                    ss += link.scale_part[(size_t)m * link.scale_stride + p];
            float4 part[8];
#pragma unroll
            for (int sl = 0; sl < 8; ++sl)
                part[sl] = sl < slices ? *reinterpret_cast<const float4*>(share[sl] + m * BM + r)
                                       : make_float4(0.f, 0.f, 0.f, 0.f);
            float v[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int sl = 0; sl < 8; ++sl) {
                v[0] += part[sl].x; v[1] += part[sl].y; v[2] += part[sl].z; v[3] += part[sl].w;
            }
            if (link.scale_part) {
                const float sc = 1.0f / sqrtf(mv_warp_sum(ss) * link.inv_dim + link.eps);
#pragma unroll
                for (int e = 0; e < 4; ++e) v[e] *= sc;
            }
            // the head's sum of squares: over the 16 lanes of the half-warp (every lane takes part)
            float hq = fmaf(v[0], v[0], fmaf(v[1], v[1], fmaf(v[2], v[2], v[3] * v[3])));
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) hq += __shfl_xor_sync(0xffffffffu, hq, o);
            if (hs >= n_slots) continue;
            const int pos = heads.positions[m];
            if (w) {
                const float scale = 1.0f / sqrtf(hq / 64.0f + heads.eps);
                v[0] *= scale * w4.x; v[1] *= scale * w4.y; v[2] *= scale * w4.z; v[3] *= scale * w4.w;
            }
            if (rotate) {
                float sn0, cs0, sn1, cs1;
                sincosf((float)pos * f0, &sn0, &cs0);
                sincosf((float)pos * f1, &sn1, &cs1);
                const float a0 = v[0] * cs0 - v[1] * sn0, b0 = v[0] * sn0 + v[1] * cs0;
                const float a1 = v[2] * cs1 - v[3] * sn1, b1 = v[2] * sn1 + v[3] * cs1;
                v[0] = a0; v[1] = b0; v[2] = a1; v[3] = b1;
            }
            __nv_bfloat16* dst;
            if (is_q) {
                dst = heads.q_out + ((size_t)m * heads.nh + hs) * 64;
            } else {
                const int page_size = 1 << heads.page_shift;
                const int page = heads.page_table[(size_t)heads.seq_of[m] * heads.table_stride + (pos >> heads.page_shift)];
                const int g2 = is_k ? hs - heads.nh : hs - heads.nh - heads.nkv;
                dst = heads.pool + (size_t)page * heads.page_stride + (size_t)(pos & (page_size - 1)) * 64 +
                      ((size_t)(is_k ? 0 : 1) * heads.nkv + g2) * page_size * 64;
            }
            mv_store4(dst + 4 * sub, v[0], v[1], v[2], v[3]);
        }
    } else
    {
        // An item is the tile's 128 rows for one token, four consecutive rows per lane (16-byte reads
        // through distributed shared memory, 16-byte stores).  A warp takes its items two at a time:
        // first every load of both (the slices' sums, and the old values where the product is added
        // to memory), then the arithmetic and the stores - so the round trips overlap.
        constexpr int CH = 2;
        const int r = 4 * lane, n = n0 + r;
        const bool vec_ok = n + 3 < N && (ldo & 3) == 0 && ((uintptr_t)out & 15) == 0;   // else one by one
        for (int m0 = mt0 + slice + slices * warp; m0 < m_end; m0 += CH * slices * WARPS_ALL) {
            float4 part[CH][8], old[CH];
            float ss[CH];
#pragma unroll
            for (int c = 0; c < CH; ++c) {
                const int m = m0 + c * slices * WARPS_ALL;
                // a carried norm's sums of this token: lane p holds sums p, p + 32, ...
                ss[c] = 0.f;
                if (link.scale_part && m < m_end)
                    for (int p = lane; p < link.n_scale_part; p += 32)
                        ss[c] += link.scale_part[(size_t)m * link.scale_stride + p];
#pragma unroll
                for (int s = 0; s < 8; ++s)
                    part[c][s] = (m < m_end && s < slices) ? *reinterpret_cast<const float4*>(share[s] + (m - mt0) * BM + r)
                                                       : make_float4(0.f, 0.f, 0.f, 0.f);
                old[c] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (mode == 2 && m < m_end) {
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
                if (m >= m_end) break;
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
int k_slices(int N, int K, int per_sm = 2, int token_tiles = 1) {
    const int tiles = ((N + BM - 1) / BM) * token_tiles, kblocks = (K + BK - 1) / BK;
    int slices = per_sm * 148 / tiles;
    slices = slices >= 8 ? 8 : (slices >= 4 ? 4 : (slices >= 2 ? 2 : 1));   // clusters of other sizes schedule worse
    // more tiles than the GPU holds at once: still two slices (measured at 64 tokens on [65536, 2048]:
    // 65 us against 73 with one; two blocks a multiprocessor overlap one's reduce with the other's loads)
    if (slices < 2 && kblocks >= 8) slices = 2;
    while (slices > 1 && kblocks / slices < 2) slices >>= 1;
    return slices < 1 ? 1 : slices;
}

template <int BN, int STAGES, int TAIL = 0>
int launch(const void* X, const void* W, const float* bias, void* out, int mode, int M, int N, int K, int ldo,
           const NormLink& link, const ConvTail& tail, const HeadTail& heads, const Ahead& ahead, int* err,
           cudaStream_t stream, int slices) {
    using L = SwapLayout<BN, STAGES, TAIL>;
    CUtensorMap mw, mx;
    // TAIL 1: W has three times N rows (B, C and x rows in groups of 32 channels), N counts channels
    if (!tensor_map(W, TAIL == 1 ? 3 * N : N, K, L::W_ROWS, &mw) || !tensor_map(X, M, K, BN, &mx))
        return (int)cudaErrorInvalidValue;
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(gemm_tc_swap_kernel<BN, STAGES, TAIL>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        attr_set = true;
    }
    const int tiles = TAIL == 1 ? (N + 31) / 32 : (N + BM - 1) / BM;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(slices, tiles, (M + BN - 1) / BN);
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
    cudaLaunchKernelEx(&cfg, gemm_tc_swap_kernel<BN, STAGES, TAIL>, mw, mx, bias, out, mode, M, N, K, ldo, link, tail, heads,
                       ahead, err);
    return mv_launch_status();
}

}  // namespace

// Same contract as mv_gemm_small_m (modes 0-3, K a multiple of 8, 16-byte aligned operands;
// scale_part / emit_x as there, with one sum per tile of 128 rows) for any M >= 1, plus the error
// flag of the bounded waits.
MV_API int mv_gemm_tc_swap(const void* X, const void* W, const float* bias, void* out, int mode, int M, int N,
                           int K, int ldo, const float* scale_part, int n_scale_part, int scale_stride, int dim,
                           float eps, const float* emit_g, void* emit_x, float* emit_part, int emit_stride,
                           const void* next_w, long long next_bytes, int* err, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || ((uintptr_t)X & 15) || ((uintptr_t)W & 15)) return (int)cudaErrorInvalidValue;
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
    const Ahead ahead = {next_w, next_bytes};
    if (M > 64) {
        // More tokens: tiles of 128 tokens along the grid's z (three stages of 32 KB, two blocks a
        // multiprocessor).  Tiles of 256 tokens (one block a multiprocessor) measured slower at every size:
        // each block reads its own copy of X from the L2 cache, and that traffic grows with the tile.
        return launch<128, 3>(X, W, bias, out, mode, M, N, K, ldo, link, ConvTail{}, HeadTail{}, ahead, err, stream,
                              k_slices(N, K, 2, (M + 127) / 128));
    }
    const int slices = k_slices(N, K);
    const bool deep = slices == 1;
#define MV_GO(BN) return deep ? launch<BN, 8>(X, W, bias, out, mode, M, N, K, ldo, link, ConvTail{}, HeadTail{}, ahead, err, stream, slices) \
                              : launch<BN, 4>(X, W, bias, out, mode, M, N, K, ldo, link, ConvTail{}, HeadTail{}, ahead, err, stream, slices)
    if (M <= 16) MV_GO(16);
    if (M <= 32) MV_GO(32);
    MV_GO(64);
#undef MV_GO
}

namespace {
NormLink scale_link(const float* scale_part, int n_scale_part, int scale_stride, int dim, float eps) {
    NormLink link = {};
    if (scale_part) {
        link.scale_part = scale_part;
        link.n_scale_part = n_scale_part;
        link.scale_stride = scale_stride;
        link.inv_dim = 1.0f / (float)dim;
        link.eps = eps;
    }
    return link;
}
}  // namespace

// A decode step's gated short convolution together with its input projection, for 1 <= M <= 64 rows
// (one a sequence): [B | C | x] = X W^T (+ bias[3 H]); z[m, c] = C * (conv_bias + sum_j taps[c][j] * value j of
// the sequence's kept B*x values followed by this token's); ``state`` [slots][k-1][H] is shifted and updated
// for slots[m].  ``z`` is bfloat16 [M, H].  W's rows come regrouped by 32 channels ([B of 32 | C of 32 | x of
// 32] group after group; H a multiple of 32); ``bias`` in the original order [3 H].  scale_part etc. as in
// mv_gemm_tc_swap.
MV_API int mv_gemm_tc_swap_shortconv(const void* X, const void* W, const float* bias, const float* taps,
                                             const float* conv_bias, float* state, const int* slots, void* z, int M,
                                             int H, int K, int k, const float* scale_part, int n_scale_part,
                                             int scale_stride, int dim, float eps, const void* next_w,
                                             long long next_bytes, int* err, cudaStream_t stream) {
    if (M <= 0 || H <= 0) return 0;
    if (M > 64 || H % 32 || K <= 0 || K % 8 || ((uintptr_t)X & 15) || ((uintptr_t)W & 15) || k < 1 || k > 16 || !taps ||
        (!state && k > 1) || !slots)
        return (int)cudaErrorInvalidValue;
    if (scale_part && (n_scale_part <= 0 || n_scale_part > scale_stride || dim <= 0)) return (int)cudaErrorInvalidValue;
    const NormLink link = scale_link(scale_part, n_scale_part, scale_stride, dim, eps);
    const ConvTail tail = {taps, conv_bias, state, slots, k};
    const Ahead ahead = {next_w, next_bytes};
    // blocks of 96 rows, two a multiprocessor: K is cut as for a plain product of as many tiles
    const int kblocks = (K + BK - 1) / BK;
    int slices = 2 * 148 / (H / 32);
    slices = slices >= 8 ? 8 : (slices >= 4 ? 4 : (slices >= 2 ? 2 : 1));
    while (slices > 1 && kblocks / slices < 2) slices >>= 1;
#define MV_GO(BN) return launch<BN, 4, 1>(X, W, bias, z, 1, M, H, K, H, link, tail, HeadTail{}, ahead, err, stream, slices)
    if (M <= 16) MV_GO(16);
    if (M <= 32) MV_GO(32);
    MV_GO(64);
#undef MV_GO
}

// The fused q/k/v projection of a step of 1 <= M <= 64 tokens together with the preparation of its heads
// (head size 64, pairs (2i, 2i+1), bfloat16 cache): W [(nh + 2 nkv) 64, K].
MV_API int mv_gemm_tc_swap_heads(const void* X, const void* W, const float* wq, const float* wk, float head_eps,
                                 const float* inv_freq, const int* positions, const int* seq_of,
                                 const int* page_table, int table_stride, int page_size, void* pool,
                                 long long page_stride, void* q_out, int M, int nh, int nkv, int K,
                                 const float* scale_part, int n_scale_part, int scale_stride, int dim, float eps,
                                 const void* next_w, long long next_bytes, int* err, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (M > 64 || K <= 0 || K % 8 || ((uintptr_t)X & 15) || ((uintptr_t)W & 15) || nh <= 0 || nkv <= 0 ||
        (page_size & (page_size - 1)) || !positions || !seq_of || !page_table || !pool || !q_out ||
        ((uintptr_t)q_out & 7) || ((uintptr_t)pool & 7))
        return (int)cudaErrorInvalidValue;
    if (scale_part && (n_scale_part <= 0 || n_scale_part > scale_stride || dim <= 0)) return (int)cudaErrorInvalidValue;
    const NormLink link = scale_link(scale_part, n_scale_part, scale_stride, dim, eps);
    HeadTail heads = {};
    heads.wq = wq; heads.wk = wk; heads.inv_freq = inv_freq; heads.positions = positions; heads.seq_of = seq_of;
    heads.page_table = page_table; heads.pool = (__nv_bfloat16*)pool; heads.q_out = (__nv_bfloat16*)q_out;
    heads.page_stride = page_stride; heads.eps = head_eps; heads.table_stride = table_stride;
    heads.page_shift = 0;
    while ((1 << heads.page_shift) < page_size) ++heads.page_shift;
    heads.nh = nh; heads.nkv = nkv;
    const int N = (nh + 2 * nkv) * 64;
    const Ahead ahead = {next_w, next_bytes};
    const int slices = k_slices(N, K);
    const bool deep = slices == 1;
#define MV_GO(BN) return deep ? launch<BN, 8, 2>(X, W, nullptr, q_out, 1, M, N, K, N, link, ConvTail{}, heads, ahead, err, stream, slices) \
                              : launch<BN, 4, 2>(X, W, nullptr, q_out, 1, M, N, K, N, link, ConvTail{}, heads, ahead, err, stream, slices)
    if (M <= 16) MV_GO(16);
    if (M <= 32) MV_GO(32);
    MV_GO(64);
#undef MV_GO
}
