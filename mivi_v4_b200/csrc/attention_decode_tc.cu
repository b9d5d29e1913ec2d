// Attention of a step's single tokens over long caches on the fifth-generation
// tensor cores (head size 64, pages of 64 tokens, bfloat16, no window): flash
// decoding whose two products are tcgen05.mma.
//
// Block = one query token, one kv head, one split of that token's keys.  The
// query heads that share the kv head are the rows of the MMA's M side: head i of
// the group sits at row (i mod 4) * 32 + i / 4 of a 128-row tile, so that the
// four softmax warps (tensor memory lets a warp read only its own quarter of the
// lanes) each own a quarter of the heads.  The other rows hold whatever the
// shared memory held; rows never mix in either product, and they are not written
// out.  Keys and values come in blocks of 128 (two pages) by TMA straight out of
// the paged pool, as in attention_prefill_tc.cu.
//
//   warp 0      TMA: the query rows once, then K and V of every key block of the
//               split into rings of two stages each;
//   warp 1      MMA: S = Q K^T (128 x 128 x 64), issued for block j + 1 as soon as
//               the softmax warps have taken S of block j into registers; then
//               O += P V (128 x 64 x 128), V taken MN-major as it lies in the cache;
//   warps 4-7   softmax, one row per lane: mask past the token's position, maximum,
//               P = exp2(...) as bfloat16 into shared memory in the swizzled K-major
//               layout, row sum in float32; O stays in tensor memory and is rescaled
//               only when a row's maximum outgrows its reference by more than 2^8.
//
// A split writes its unnormalised O rows with their reference maximum and sum; a
// second kernel (one warp per token and head) merges the splits in a fixed order.
// With one split the rows are written out directly.  Every mbarrier wait is
// bounded (tc_common.cuh).  Two blocks fit a multiprocessor (112 KB of shared
// memory, 256 columns of tensor memory each), so one block's set-up hides behind
// the other's stream.
//
// Same mathematics as attention_decode.cu (reference: crates/mivi-model/src/
// transformer.rs:114-167, 293-298).
#include "tc_common.cuh"

namespace {

constexpr int DT_THREADS = 256;
constexpr int BQ = 128, BKV = 128, HD = 64, PAGE = 64;
constexpr int Q_BYTES = BQ * HD * 2;               // 16 KB
constexpr int KV_BYTES = BKV * HD * 2;             // 16 KB per stage (two pages)
constexpr int P_BYTES = BQ * BKV * 2;              // 32 KB: two K-major sub-tiles of [128 x 64]
constexpr int STAGES_KV = 2;
constexpr int DT_SMEM = Q_BYTES + 2 * STAGES_KV * KV_BYTES + P_BYTES + 256;
constexpr unsigned S_COL0 = 0, O_COL0 = 128, TMEM_COLS = 256;
constexpr float RESCALE_ABOVE = 8.0f;

enum { B_Q = 0, B_KFULL = 1, B_KEMPTY = B_KFULL + STAGES_KV, B_VFULL = B_KEMPTY + STAGES_KV,
       B_VEMPTY = B_VFULL + STAGES_KV, B_SFULL = B_VEMPTY + STAGES_KV, B_SEMPTY, B_PFULL, B_PVDONE, B_COUNT };
static_assert(B_COUNT * 8 + 8 <= 256, "barrier area");

__device__ __forceinline__ unsigned long long smem_desc_mn(unsigned addr) {
    unsigned long long d = 0;
    d |= (unsigned long long)((addr & 0x3ffffu) >> 4);
    d |= (unsigned long long)1 << 16;
    d |= (unsigned long long)(1024 >> 4) << 32;
    d |= (unsigned long long)1 << 46;
    d |= (unsigned long long)2 << 61;
    return d;
}
__device__ __forceinline__ void mbar_arrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void tmem_st32(unsigned taddr, const unsigned (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

// Maximum of 32 values of a row, of those among them that exist; four chains, so that no instruction waits
// for the one before it.
template <bool MASK>
__device__ __forceinline__ float chunk_max(const unsigned (&s)[32], int c, int visible) {
    float a[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
    for (int i = 0; i < 32; i += 4)
#pragma unroll
        for (int e = 0; e < 4; ++e)
            if (!MASK || c + i + e < visible) a[e] = fmaxf(a[e], __uint_as_float(s[i + e]));
    return fmaxf(fmaxf(a[0], a[1]), fmaxf(a[2], a[3]));
}

// 32 keys of one row: P = exp2(s * scale - ref) as bfloat16 into the row's four 16-byte chunks; returns their sum.
template <bool MASK>
__device__ __forceinline__ float row_exp(const unsigned (&s)[32], int c, int visible, float scale_log2, float ref,
                                         unsigned char* p_tile, int r) {
    float sum0 = 0.f, sum1 = 0.f;
    unsigned packed[16];
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
        float p0 = ex2(fmaf(__uint_as_float(s[i]), scale_log2, -ref));
        float p1 = ex2(fmaf(__uint_as_float(s[i + 1]), scale_log2, -ref));
        if (MASK) {
            if (c + i >= visible) p0 = 0.f;
            if (c + i + 1 >= visible) p1 = 0.f;
        }
        sum0 += p0;
        sum1 += p1;
        const __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
        packed[i >> 1] = *reinterpret_cast<const unsigned*>(&pk);
    }
    unsigned char* sub = p_tile + (c >> 6) * (BQ * 128) + r * 128;
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) {
        const int chunk = ((c & 63) >> 3) + q4;
        *reinterpret_cast<uint4*>(sub + ((chunk ^ (r & 7)) << 4)) =
            make_uint4(packed[4 * q4], packed[4 * q4 + 1], packed[4 * q4 + 2], packed[4 * q4 + 3]);
    }
    return sum0 + sum1;
}

// grid (splits, nkv, N).  part_o [N, nh, splits, 64], part_ml [N, nh, splits, 2] (reference maximum times
// scale_log2, sum); with one split the rows go to o [N, nh * 64] directly.
__global__ void __launch_bounds__(DT_THREADS, 2)
attention_decode_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                           const int* __restrict__ page_table, int table_stride, const int* __restrict__ positions,
                           const int* __restrict__ seq_of, __nv_bfloat16* __restrict__ o,
                           float* __restrict__ part_o, float* __restrict__ part_ml, int nh, int nkv,
                           float scale_log2, int* __restrict__ err) {
    // No slack for aligning: with it two blocks would not fit a multiprocessor.  The kernel has no
    // static shared memory, so the dynamic part starts on a 1024-byte boundary; if it ever does not,
    // the block reports it and leaves.
    extern __shared__ __align__(1024) unsigned char smem[];
    const unsigned q_s = smem_u32(smem);
    if (q_s & 1023u) {
        if (threadIdx.x == 0) atomicExch(err, 30);
        return;
    }
    const unsigned k_s = q_s + Q_BYTES, v_s = k_s + STAGES_KV * KV_BYTES, p_s = v_s + STAGES_KV * KV_BYTES;
    unsigned char* p_ptr = smem + Q_BYTES + 2 * STAGES_KV * KV_BYTES;
    unsigned long long* bars = (unsigned long long*)(p_ptr + P_BYTES);
    unsigned* tmem_holder = (unsigned*)(bars + B_COUNT);
    const unsigned bar0 = smem_u32(bars);
    auto bar = [&](int i) { return bar0 + 8u * (unsigned)i; };

    const int splits = gridDim.x, split = blockIdx.x, g = blockIdx.y, n = blockIdx.z;
    const int G = nh / nkv;
    const int kv_len = positions[n] + 1;
    const int blocks_all = (kv_len + BKV - 1) / BKV;
    const int per = (blocks_all + splits - 1) / splits;
    const int j0 = split * per, n_blocks = max(0, min(blocks_all, j0 + per) - j0);
    const int* table = page_table + (size_t)seq_of[n] * table_stride;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int active_warps = min(4, G);                 // head i sits in quarter i mod 4

    if (threadIdx.x == 0) {
        mbar_init(bar(B_Q), 1);
        for (int s = 0; s < STAGES_KV; ++s) {
            mbar_init(bar(B_KFULL + s), 1);
            mbar_init(bar(B_KEMPTY + s), 1);
            mbar_init(bar(B_VFULL + s), 1);
            mbar_init(bar(B_VEMPTY + s), 1);
        }
        mbar_init(bar(B_SFULL), 1);
        mbar_init(bar(B_SEMPTY), active_warps);
        mbar_init(bar(B_PFULL), active_warps);
        mbar_init(bar(B_PVDONE), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_holder)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_base = *tmem_holder;
    // set-up done (it may have run under the tail of the kernel before): from here on the step's data
    mv_pdl_wait();

    if (warp < 4) {
        // registers move from this warpgroup to the softmax warps (128 each at launch)
        asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
        if (warp == 0) {
        if (lane == 0 && n_blocks > 0) {
            // head i of the group: one row of 128 bytes to row (i mod 4) * 32 + i / 4 of the Q tile
            mbar_expect_tx(bar(B_Q), (unsigned)G * HD * 2);
            for (int i = 0; i < G; ++i)
                tma_load_2d(q_s + (unsigned)(((i & 3) * 32 + (i >> 2)) * 128), &map_q, 0, n * nh + g * G + i, bar(B_Q));
            for (int j = 0; j < n_blocks; ++j) {
                const int s = j % STAGES_KV;
                const unsigned ph = (unsigned)(j / STAGES_KV) & 1u;
                const int jb = j0 + j;
                const int pg0 = table[min(2 * jb, table_stride - 1)], pg1 = table[min(2 * jb + 1, table_stride - 1)];
                if (!mbar_wait(bar(B_KEMPTY + s), ph ^ 1u, err, 31)) break;
                mbar_expect_tx(bar(B_KFULL + s), KV_BYTES);
                tma_load_2d(k_s + s * KV_BYTES, &map_kv, 0, ((pg0 * 2 + 0) * nkv + g) * PAGE, bar(B_KFULL + s));
                tma_load_2d(k_s + s * KV_BYTES + KV_BYTES / 2, &map_kv, 0, ((pg1 * 2 + 0) * nkv + g) * PAGE,
                            bar(B_KFULL + s));
                if (!mbar_wait(bar(B_VEMPTY + s), ph ^ 1u, err, 32)) break;
                mbar_expect_tx(bar(B_VFULL + s), KV_BYTES);
                tma_load_2d(v_s + s * KV_BYTES, &map_kv, 0, ((pg0 * 2 + 1) * nkv + g) * PAGE, bar(B_VFULL + s));
                tma_load_2d(v_s + s * KV_BYTES + KV_BYTES / 2, &map_kv, 0, ((pg1 * 2 + 1) * nkv + g) * PAGE,
                            bar(B_VFULL + s));
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && n_blocks > 0) {
            const unsigned idesc_qk = instr_desc(BQ, BKV);
            const unsigned idesc_pv = instr_desc(BQ, HD) | (1u << 16);          // B operand MN-major
            bool ok = mbar_wait(bar(B_Q), 0, err, 33);
            auto issue_qk = [&](int j) {
                const int s = j % STAGES_KV;
                if (!mbar_wait(bar(B_KFULL + s), (unsigned)(j / STAGES_KV) & 1u, err, 34)) return false;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int k = 0; k < HD / 16; ++k)
                    mma_f16(tmem_base + S_COL0, smem_desc(q_s + k * 32), smem_desc(k_s + s * KV_BYTES + k * 32),
                            idesc_qk, k > 0 ? 1u : 0u);
                mma_commit(bar(B_SFULL));
                mma_commit(bar(B_KEMPTY + s));
                return true;
            };
            if (ok) ok = issue_qk(0);
            for (int j = 0; j < n_blocks && ok; ++j) {
                const int s = j % STAGES_KV;
                if (j + 1 < n_blocks) {
                    // S of block j is in the softmax warps' registers: its columns are free for block j + 1
                    if (!(ok = mbar_wait(bar(B_SEMPTY), (unsigned)j & 1u, err, 35))) break;
                    if (!(ok = issue_qk(j + 1))) break;
                }
                if (!(ok = mbar_wait(bar(B_PFULL), (unsigned)j & 1u, err, 36))) break;
                if (!(ok = mbar_wait(bar(B_VFULL + s), (unsigned)(j / STAGES_KV) & 1u, err, 37))) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int k = 0; k < BKV / 16; ++k) {
                    const unsigned a_addr = p_s + (k >> 2) * (BQ * 128) + (k & 3) * 32;
                    const unsigned b_addr = v_s + s * KV_BYTES + k * 16 * 128;
                    mma_f16(tmem_base + O_COL0, smem_desc(a_addr), smem_desc_mn(b_addr), idesc_pv,
                            (j > 0 || k > 0) ? 1u : 0u);
                }
                mma_commit(bar(B_PVDONE));
                mma_commit(bar(B_VEMPTY + s));
            }
        }
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
        if ((warp & 3) < active_warps) {
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;                   // row of the tile = lane of tensor memory
        const int head_in_group = lane * 4 + quarter;
        const bool live = head_in_group < G;
        const int h = g * G + head_in_group;
        const unsigned lane_addr = (unsigned)(quarter * 32) << 16;
        const unsigned s_addr = tmem_base + lane_addr + S_COL0, o_addr = tmem_base + lane_addr + O_COL0;
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < n_blocks && ok; ++j) {
            ok = mbar_wait(bar(B_SFULL), (unsigned)j & 1u, err, 38);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            unsigned s0[32], s1[32], s2[32], s3[32];
            tmem_ld32(s_addr, s0);
            tmem_ld32(s_addr + 32, s1);
            tmem_ld32(s_addr + 64, s2);
            tmem_ld32(s_addr + 96, s3);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(B_SEMPTY));
            const int visible = kv_len - (j0 + j) * BKV;      // keys of this block that exist
            const bool mask = visible < BKV;                  // only a token's last block is ragged
            float mx = mask ? fmaxf(fmaxf(chunk_max<true>(s0, 0, visible), chunk_max<true>(s1, 32, visible)),
                                    fmaxf(chunk_max<true>(s2, 64, visible), chunk_max<true>(s3, 96, visible)))
                            : fmaxf(fmaxf(chunk_max<false>(s0, 0, visible), chunk_max<false>(s1, 32, visible)),
                                    fmaxf(chunk_max<false>(s2, 64, visible), chunk_max<false>(s3, 96, visible)));
            if (!live) mx = 0.f;                              // rows of no head: anything finite
            float corr = 1.0f;
            if (mx > m && (m == -INFINITY || (mx - m) * scale_log2 > RESCALE_ABOVE)) {
                corr = m == -INFINITY ? 0.f : ex2((m - mx) * scale_log2);
                m = mx;
            }
            // P of the block before and O are in use until its second product is done
            if (j > 0) {
                ok = mbar_wait(bar(B_PVDONE), (unsigned)(j - 1) & 1u, err, 39);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (__any_sync(0xffffffffu, corr != 1.0f)) {
#pragma unroll
                    for (int c = 0; c < HD; c += 32) {
                        unsigned v[32];
                        tmem_ld32(o_addr + (unsigned)c, v);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * corr);
                        tmem_st32(o_addr + (unsigned)c, v);
                    }
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                }
            }
            const float ref = m == -INFINITY ? 0.f : m * scale_log2;
            float sum;
            if (mask) {
                sum = (row_exp<true>(s0, 0, visible, scale_log2, ref, p_ptr, r) +
                       row_exp<true>(s1, 32, visible, scale_log2, ref, p_ptr, r)) +
                      (row_exp<true>(s2, 64, visible, scale_log2, ref, p_ptr, r) +
                       row_exp<true>(s3, 96, visible, scale_log2, ref, p_ptr, r));
            } else {
                sum = (row_exp<false>(s0, 0, visible, scale_log2, ref, p_ptr, r) +
                       row_exp<false>(s1, 32, visible, scale_log2, ref, p_ptr, r)) +
                      (row_exp<false>(s2, 64, visible, scale_log2, ref, p_ptr, r) +
                       row_exp<false>(s3, 96, visible, scale_log2, ref, p_ptr, r));
            }
            l = l * corr + sum;
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(B_PFULL));
        }
        if (ok && n_blocks > 0) ok = mbar_wait(bar(B_PVDONE), (unsigned)(n_blocks - 1) & 1u, err, 40);
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const bool direct = splits == 1;
            const float inv = direct && l > 0.f ? 1.0f / l : 1.0f;
            float* po = part_o + (((size_t)n * nh + h) * splits + split) * HD;
#pragma unroll
            for (int c = 0; c < HD; c += 32) {
                unsigned v[32];
                if (n_blocks > 0) {
                    tmem_ld32(o_addr + (unsigned)c, v);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = 0u;
                }
                if (live) {
                    if (direct) {
                        __nv_bfloat16* dst = o + ((size_t)n * nh + h) * HD + c;
#pragma unroll
                        for (int d = 0; d < 32; d += 8) {
                            unsigned w4[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const __nv_bfloat162 pk = __floats2bfloat162_rn(
                                    __uint_as_float(v[d + 2 * e]) * inv, __uint_as_float(v[d + 2 * e + 1]) * inv);
                                w4[e] = *reinterpret_cast<const unsigned*>(&pk);
                            }
                            *reinterpret_cast<uint4*>(dst + d) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
                        }
                    } else {
#pragma unroll
                        for (int d = 0; d < 32; d += 4)
                            *reinterpret_cast<float4*>(po + c + d) =
                                make_float4(__uint_as_float(v[d]), __uint_as_float(v[d + 1]), __uint_as_float(v[d + 2]),
                                            __uint_as_float(v[d + 3]));
                    }
                }
            }
            if (live && !direct) {
                float* pm = part_ml + (((size_t)n * nh + h) * splits + split) * 2;
                pm[0] = m == -INFINITY ? -INFINITY : m * scale_log2;
                pm[1] = l;
            }
        }
        }
    }
    // Only now may the next kernel's blocks be given multiprocessors: signalled earlier, they would take
    // the places of this grid's own later blocks and sit there waiting.
    mv_pdl_launch_dependents();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS)
                     : "memory");
    }
}

// One warp per (token, head): out = sum_s o_s 2^(m_s - M) / sum_s l_s 2^(m_s - M), splits in order.
__global__ void attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                       __nv_bfloat16* __restrict__ o, int rows, int splits) {
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float* ml = part_ml + (size_t)row * splits * 2;
    float M = -INFINITY;
    for (int s = 0; s < splits; ++s) M = fmaxf(M, ml[2 * s]);
    float a0 = 0.f, a1 = 0.f, L = 0.f;
    for (int s = 0; s < splits; ++s) {
        const float ms = ml[2 * s];
        if (ms == -INFINITY) continue;
        const float w = exp2f(ms - M);
        const float2 v = *reinterpret_cast<const float2*>(part_o + ((size_t)row * splits + s) * HD + 2 * lane);
        a0 = fmaf(v.x, w, a0);
        a1 = fmaf(v.y, w, a1);
        L = fmaf(ml[2 * s + 1], w, L);
    }
    const float inv = L > 0.f ? 1.0f / L : 0.f;
    *reinterpret_cast<__nv_bfloat162*>(o + (size_t)row * HD + 2 * lane) = __floats2bfloat162_rn(a0 * inv, a1 * inv);
}

}  // namespace

// bfloat16, head size 64, pages of 64 tokens, no window, at most 128 query heads per kv head.
// pool_rows = pages * 2 * nkv * 64.  part_o [N, nh, splits, 64] and part_ml [N, nh, splits, 2] float32.
MV_API int mv_attention_decode_tc(const void* q, const void* pool, long long pool_rows, const int* page_table,
                                  int table_stride, const int* positions, const int* seq_of, void* o, float* part_o,
                                  float* part_ml, int N, int nh, int nkv, float scale, int splits, int* err,
                                  cudaStream_t stream) {
    if (N <= 0) return 0;
    if (nh % nkv || nh / nkv > 128 || splits < 1 || ((uintptr_t)q & 15) || ((uintptr_t)pool & 15))
        return (int)cudaErrorInvalidValue;
    CUtensorMap mq, mkv;
    if (!tensor_map(q, N * nh, HD, 1, &mq) || !tensor_map(pool, (int)pool_rows, HD, PAGE, &mkv))
        return (int)cudaErrorInvalidValue;
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(attention_decode_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DT_SMEM);
        attr_set = true;
    }
    // A plain launch, not a programmatic one: started early, this grid's blocks (two fill a
    // multiprocessor) measured 12 us slower at 64 tokens; the kernel after it still starts under its tail.
    attention_decode_tc_kernel<<<dim3(splits, nkv, N), DT_THREADS, DT_SMEM, stream>>>(
        mq, mkv, page_table, table_stride, positions, seq_of, (__nv_bfloat16*)o, part_o, part_ml, nh, nkv,
        scale * 1.4426950408889634f, err);
    int rc = mv_launch_status();
    if (rc || splits == 1) return rc;
    const int rows = N * nh;
    attention_merge_kernel<<<(rows + 7) / 8, 256, 0, stream>>>(part_o, part_ml, (__nv_bfloat16*)o, rows, splits);
    return mv_launch_status();
}
