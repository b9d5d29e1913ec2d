// Attention of a step's single tokens over long caches on the fifth-generation
// tensor cores (head size 64, pages of 64 tokens, bfloat16, no window, at most
// 16 query heads a kv head): flash decoding whose two products are tcgen05.mma.
//
// Block = one query token, one kv head, one split of that token's keys.  Keys
// and values come in blocks of 128 (two pages) by TMA straight out of the paged
// pool, as in attention_prefill_tc.cu.
//
// The scores are computed TRANSPOSED, S^T = K Q^T: the 128 keys of a block are
// the MMA's M side (one lane of tensor memory each), the query heads that share
// the kv head its N side (16 columns).  Each of the 128 softmax threads then owns
// one key and all heads, so the exponentials of a block are a handful of
// instructions a warp (a thread per query row, the other way round, would issue
// 128 of them with one lane at work).  The maximum over the keys is taken by
// shuffles and one exchange through shared memory a block.  P goes to shared
// memory as [head row][key], the swizzled K-major A operand of O += P V with
// head i at row (i mod 4) * 32 + i / 4 of a 128-row tile; V is taken MN-major as
// it lies in the cache.  The rows of no head hold whatever the shared memory
// held; rows never mix in the product, and they are not written out.
//
//   warp 0      TMA: the query rows once, then K and V of every key block of the
//               split into rings of two stages each;
//   warp 1      MMA: S^T (128 x 16 x 64), issued for block j + 1 as soon as the
//               softmax warps have taken S^T of block j into registers; then
//               O += P V (128 x 64 x 128);
//   warps 4-7   softmax as above; O stays in tensor memory and is rescaled only
//               when a head's maximum outgrows its reference by more than 2^8.
//
// A split writes its unnormalised O rows with their reference maximum and sum; a
// second kernel (one warp per token and head) merges the splits in a fixed order.
// With one split the rows are written out directly.  Every mbarrier wait is
// bounded (tc_common.cuh).  Two blocks fit a multiprocessor, so one block's
// set-up hides behind the other's stream.
//
// Same mathematics as attention_decode.cu (reference: crates/mivi-model/src/
// transformer.rs:114-167, 293-298).
#include "tc_common.cuh"

namespace {

constexpr int DT_THREADS = 256;
constexpr int BQ = 128, BKV = 128, HD = 64, PAGE = 64, NQ = 16;
constexpr int Q_BYTES = NQ * HD * 2;               // 2 KB: 16 head rows
constexpr int KV_BYTES = BKV * HD * 2;             // 16 KB per stage (two pages)
constexpr int P_BYTES = BQ * BKV * 2;              // 32 KB: two K-major sub-tiles of [128 x 64]
constexpr int STAGES_KV = 2;
constexpr int X_BYTES = 3 * 4 * NQ * 4;            // maxima (two buffers) and sums exchanged between the warps
constexpr int DT_SMEM = Q_BYTES + 2 * STAGES_KV * KV_BYTES + P_BYTES + X_BYTES + 256;
constexpr unsigned S_COL0 = 0, O_COL0 = 64, TMEM_COLS = 128;
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
__device__ __forceinline__ void tmem_ld16(unsigned taddr, unsigned (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
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
// the 128 softmax threads meet (the other warps do not take part)
__device__ __forceinline__ void softmax_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// grid (splits, nkv, N).  part_o [N, nh, splits, 64], part_ml [N, nh, splits, 2] (reference maximum times
// scale_log2, sum); with one split the rows go to o [N, nh * 64] directly.  GP: heads a kv head, rounded up
// to 4, 8 or 16.
template <int GP>
__global__ void __launch_bounds__(DT_THREADS, 2)
attention_decode_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                           const int* __restrict__ page_table, int table_stride, const int* __restrict__ positions,
                           const int* __restrict__ seq_of, __nv_bfloat16* __restrict__ o,
                           float* __restrict__ part_o, float* __restrict__ part_ml, int nh, int nkv,
                           float scale_log2, int* __restrict__ err) {
    // No slack for aligning: the kernel has no static shared memory, so the dynamic part starts on a
    // 1024-byte boundary; if it ever does not, the block reports it and leaves.
    extern __shared__ __align__(1024) unsigned char smem[];
    const unsigned k_s = smem_u32(smem);
    if (k_s & 1023u) {
        if (threadIdx.x == 0) atomicExch(err, 30);
        return;
    }
    const unsigned v_s = k_s + STAGES_KV * KV_BYTES, p_s = v_s + STAGES_KV * KV_BYTES, q_s = p_s + P_BYTES;
    unsigned char* p_ptr = smem + 2 * STAGES_KV * KV_BYTES;
    float* xch = reinterpret_cast<float*>(p_ptr + P_BYTES + Q_BYTES);          // [3][4 warps][NQ]
    unsigned long long* bars = (unsigned long long*)(p_ptr + P_BYTES + Q_BYTES + X_BYTES);
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

    if (threadIdx.x == 0) {
        mbar_init(bar(B_Q), 1);
        for (int s = 0; s < STAGES_KV; ++s) {
            mbar_init(bar(B_KFULL + s), 1);
            mbar_init(bar(B_KEMPTY + s), 1);
            mbar_init(bar(B_VFULL + s), 1);
            mbar_init(bar(B_VEMPTY + s), 1);
        }
        mbar_init(bar(B_SFULL), 1);
        mbar_init(bar(B_SEMPTY), 4);
        mbar_init(bar(B_PFULL), 4);
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
    mv_pdl_wait();

    if (warp < 4) {
        // registers move from this warpgroup to the softmax warps (128 each at launch)
        asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
        if (warp == 0) {
            if (lane == 0 && n_blocks > 0) {
                // head i of the group: one row of 128 bytes, row i of the Q tile (the MMA's N side)
                mbar_expect_tx(bar(B_Q), (unsigned)G * HD * 2);
                for (int i = 0; i < G; ++i) tma_load_2d(q_s + (unsigned)(i * 128), &map_q, 0, n * nh + g * G + i, bar(B_Q));
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
                const unsigned idesc_qk = instr_desc(BKV, NQ);                      // keys x heads
                const unsigned idesc_pv = instr_desc(BQ, HD) | (1u << 16);          // B operand MN-major
                bool ok = mbar_wait(bar(B_Q), 0, err, 33);
                auto issue_qk = [&](int j) {
                    const int s = j % STAGES_KV;
                    if (!mbar_wait(bar(B_KFULL + s), (unsigned)(j / STAGES_KV) & 1u, err, 34)) return false;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                    for (int k = 0; k < HD / 16; ++k)
                        mma_f16(tmem_base + S_COL0, smem_desc(k_s + s * KV_BYTES + k * 32), smem_desc(q_s + k * 32),
                                idesc_qk, k > 0 ? 1u : 0u);
                    mma_commit(bar(B_SFULL));
                    mma_commit(bar(B_KEMPTY + s));
                    return true;
                };
                if (ok) ok = issue_qk(0);
                for (int j = 0; j < n_blocks && ok; ++j) {
                    const int s = j % STAGES_KV;
                    if (j + 1 < n_blocks) {
                        // S^T of block j is in the softmax warps' registers: its columns are free for block j + 1
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
        asm volatile("setmaxnreg.inc.sync.aligned.u32 200;");
        const int quarter = warp & 3;
        const int t = quarter * 32 + lane;                   // this thread's key within a block = its lane of tensor memory
        const unsigned lane_addr = (unsigned)(quarter * 32) << 16;
        const unsigned s_addr = tmem_base + lane_addr + S_COL0, o_addr = tmem_base + lane_addr + O_COL0;
        // the O row of lane t belongs to head own (if own < G): head i sits at row (i mod 4) * 32 + i / 4
        const int own = lane * 4 + quarter;
        float m[GP], l[GP];                                  // reference maxima (the same in every thread), this key's sums
#pragma unroll
        for (int h = 0; h < GP; ++h) { m[h] = -INFINITY; l[h] = 0.f; }
        bool ok = true;
        for (int j = 0; j < n_blocks && ok; ++j) {
            ok = mbar_wait(bar(B_SFULL), (unsigned)j & 1u, err, 38);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            unsigned sr[16];
            tmem_ld16(s_addr, sr);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(B_SEMPTY));
            const bool valid = t < kv_len - (j0 + j) * BKV;   // this key exists
            float sv[GP];
            float* wmax = xch + (j & 1) * 4 * NQ;             // two buffers: the next block writes the other one
#pragma unroll
            for (int h = 0; h < GP; ++h) {
                sv[h] = valid ? __uint_as_float(sr[h]) : -INFINITY;
                const float wm = mv_warp_max(sv[h]);
                if (lane == 0) wmax[quarter * NQ + h] = wm;
            }
            softmax_sync();
            float corr[GP];
            bool any = false;
#pragma unroll
            for (int h = 0; h < GP; ++h) {
                const float mx = fmaxf(fmaxf(wmax[h], wmax[NQ + h]), fmaxf(wmax[2 * NQ + h], wmax[3 * NQ + h]));
                corr[h] = 1.0f;
                if (h < G && mx > m[h] && (m[h] == -INFINITY || (mx - m[h]) * scale_log2 > RESCALE_ABOVE)) {
                    corr[h] = m[h] == -INFINITY ? 0.f : ex2((m[h] - mx) * scale_log2);
                    m[h] = mx;
                    any = true;
                }
            }
            // P of the block before and O are in use until its second product is done
            if (j > 0) {
                ok = mbar_wait(bar(B_PVDONE), (unsigned)(j - 1) & 1u, err, 39);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (any) {                                   // the same decision in every thread
                    float mine = 1.0f;
#pragma unroll
                    for (int h = 0; h < GP; ++h)
                        if (h == own) mine = corr[h];
#pragma unroll
                    for (int c = 0; c < HD; c += 32) {
                        unsigned v[32];
                        tmem_ld32(o_addr + (unsigned)c, v);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * mine);
                        tmem_st32(o_addr + (unsigned)c, v);
                    }
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                }
            }
            // this key's column of P, one bfloat16 a head, into the head's row of the swizzled K-major tile
            unsigned char* pcol = p_ptr + (t >> 6) * (BQ * 128) + (t & 7) * 2;
            const int chunk = (t & 63) >> 3;
#pragma unroll
            for (int h = 0; h < GP; ++h) {
                if (h < G) {
                    const float p = valid ? ex2(fmaf(sv[h], scale_log2, -m[h] * scale_log2)) : 0.f;
                    l[h] = l[h] * corr[h] + p;
                    const int row = (h & 3) * 32 + (h >> 2);
                    *reinterpret_cast<__nv_bfloat16*>(pcol + row * 128 + ((chunk ^ (row & 7)) << 4)) = __float2bfloat16_rn(p);
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(B_PFULL));
        }
        if (ok && n_blocks > 0) ok = mbar_wait(bar(B_PVDONE), (unsigned)(n_blocks - 1) & 1u, err, 40);
        // the heads' sums over all keys: by shuffles, then across the four warps
        float* wsum = xch + 2 * 4 * NQ;
#pragma unroll
        for (int h = 0; h < GP; ++h) {
            const float ws = mv_warp_sum(l[h]);
            if (lane == 0) wsum[quarter * NQ + h] = ws;
        }
        softmax_sync();
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const bool live = own < G;
            float m_own = -INFINITY, l_own = 0.f;
#pragma unroll
            for (int h = 0; h < GP; ++h)
                if (h == own) {
                    m_own = m[h];
                    l_own = (wsum[h] + wsum[NQ + h]) + (wsum[2 * NQ + h] + wsum[3 * NQ + h]);
                }
            const int hh = g * G + own;
            const bool direct = splits == 1;
            const float inv = direct && l_own > 0.f ? 1.0f / l_own : 1.0f;
            float* po = part_o + (((size_t)n * nh + hh) * splits + split) * HD;
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
                        __nv_bfloat16* dst = o + ((size_t)n * nh + hh) * HD + c;
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
                float* pm = part_ml + (((size_t)n * nh + hh) * splits + split) * 2;
                pm[0] = m_own == -INFINITY ? -INFINITY : m_own * scale_log2;
                pm[1] = l_own;
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

// bfloat16, head size 64, pages of 64 tokens, no window, at most 16 query heads per kv head.
// pool_rows = pages * 2 * nkv * 64.  part_o [N, nh, splits, 64] and part_ml [N, nh, splits, 2] float32.
MV_API int mv_attention_decode_tc(const void* q, const void* pool, long long pool_rows, const int* page_table,
                                  int table_stride, const int* positions, const int* seq_of, void* o, float* part_o,
                                  float* part_ml, int N, int nh, int nkv, float scale, int splits, int* err,
                                  cudaStream_t stream) {
    if (N <= 0) return 0;
    if (nh % nkv || nh / nkv > NQ || splits < 1 || ((uintptr_t)q & 15) || ((uintptr_t)pool & 15))
        return (int)cudaErrorInvalidValue;
    CUtensorMap mq, mkv;
    if (!tensor_map(q, N * nh, HD, 1, &mq) || !tensor_map(pool, (int)pool_rows, HD, PAGE, &mkv))
        return (int)cudaErrorInvalidValue;
    // A plain launch, not a programmatic one: started early, this grid's blocks (two fill a
    // multiprocessor) measured 12 us slower at 64 tokens; the kernel after it still starts under its tail.
    const int G = nh / nkv;
#define MV_GO(GP)                                                                                              \
    do {                                                                                                       \
        static bool attr_set = false;                                                                          \
        if (!attr_set) {                                                                                       \
            cudaFuncSetAttribute(attention_decode_tc_kernel<GP>, cudaFuncAttributeMaxDynamicSharedMemorySize,  \
                                 DT_SMEM);                                                                     \
            attr_set = true;                                                                                   \
        }                                                                                                      \
        attention_decode_tc_kernel<GP><<<dim3(splits, nkv, N), DT_THREADS, DT_SMEM, stream>>>(                 \
            mq, mkv, page_table, table_stride, positions, seq_of, (__nv_bfloat16*)o, part_o, part_ml, nh, nkv, \
            scale * 1.4426950408889634f, err);                                                                 \
    } while (0)
    if (G <= 4) MV_GO(4);
    else if (G <= 8) MV_GO(8);
    else MV_GO(16);
#undef MV_GO
    int rc = mv_launch_status();
    if (rc || splits == 1) return rc;
    const int rows = N * nh;
    attention_merge_kernel<<<(rows + 7) / 8, 256, 0, stream>>>(part_o, part_ml, (__nv_bfloat16*)o, rows, splits);
    return mv_launch_status();
}
