// Causal attention for prefill on the fifth-generation tensor cores, head size
// 64, pages of 64 tokens, bfloat16: both products of flash attention are
// tcgen05.mma with their results in tensor memory.
//
// Block = 256 consecutive query tokens of one sequence for one query head, as two
// tiles of 128 that share the key and value blocks.  The cached keys and values
// come in blocks of 128 (two pages), by TMA, straight out of the paged pool: a
// page of one kv head is a [64 rows x 128 bytes] tile, which is the 128-byte-
// swizzle atom that the MMA reads.
//
//   warp 0      TMA: the two Q tiles once, then the K and V pages of every key
//               block into rings of three stages each;
//   warp 1      MMA, for either tile: S = Q K^T (128 x 128 x 64) into the tile's S
//               columns of tensor memory, and O += P V (128 x 64 x 128) into the
//               tile's O columns, V taken MN-major as it lies in the cache.  S(tile, j + 1)
//               is issued as soon as the softmax warps have taken S(tile, j) into
//               registers, so both products run under the softmax arithmetic and a
//               tile's next row of S is there when its softmax comes back for it;
//   warps 4-11  softmax, four warps per tile, one query row per thread: the row of
//               S from tensor memory into registers (then the S columns are handed
//               back), mask, maximum, P = exp2(...), once PV of the block before is done,
//               as bfloat16 into shared memory in the swizzled K-major layout the
//               MMA wants, row sum in float32.  O stays in tensor memory; the
//               reference maximum of a row is only moved when the new maximum
//               exceeds it by more than 2^8 (P stays well inside bfloat16's range
//               and the sum in float32's), and only then the row of O is read,
//               scaled and written back.  At the end O / sum is written out.
//
// Every wait on an mbarrier is bounded (tc_common.cuh).  Keys past a sequence's
// end are masked; their pages may be any valid page (the page table's padding).
//
// Same mathematics as attention_prefill.cu (reference: crates/mivi-model/src/
// transformer.rs:114-167, 293-298).
#include "tc_common.cuh"

namespace {

constexpr int AT_THREADS = 384;                   // warps 0-3: TMA, MMA and two idle; warps 4-11: softmax
constexpr int BQ = 128, TILES = 2, BKV = 128, HD = 64, PAGE = 64;
constexpr int Q_BYTES = BQ * HD * 2;               // 16 KB per tile
constexpr int KV_BYTES = BKV * HD * 2;             // 16 KB per stage (two pages)
constexpr int P_BYTES = BQ * BKV * 2;              // 32 KB per tile: two K-major sub-tiles of [128 x 64]
constexpr int STAGES_KV = 3;
constexpr int AT_SMEM = TILES * Q_BYTES + 2 * STAGES_KV * KV_BYTES + TILES * P_BYTES + 256 + 1024;
constexpr unsigned S_COL0 = 0, O_COL0 = 256;       // tile t: S at 128 t, O at 256 + 64 t
constexpr float RESCALE_ABOVE = 8.0f;              // log2 of how far a row's maximum may outgrow its reference

// barriers, 8 bytes each
enum { B_Q = 0, B_KFULL = 1, B_KEMPTY = B_KFULL + STAGES_KV, B_VFULL = B_KEMPTY + STAGES_KV,
       B_VEMPTY = B_VFULL + STAGES_KV, B_SFULL = B_VEMPTY + STAGES_KV, B_PFULL = B_SFULL + TILES,
       B_PVDONE = B_PFULL + TILES, B_SFREE = B_PVDONE + TILES, B_COUNT = B_SFREE + TILES };
static_assert(B_COUNT * 8 + 8 <= 256, "barrier area");

// MN-major operand (V: rows are keys = K of the product, 128 bytes = 64 values of d per row), 128-byte swizzle:
// 8-row groups 1024 bytes apart (stride byte offset); one 64-wide chunk only, so the leading offset is unused.
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

// One row of S (128 values in registers): maximum over the keys the row may see; sixteen chains, so
// that no instruction waits for the one before it.
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
template <bool MASK>
__device__ __forceinline__ float row_max(const unsigned (&s0)[32], const unsigned (&s1)[32], const unsigned (&s2)[32],
                                         const unsigned (&s3)[32], int visible) {
    return fmaxf(fmaxf(chunk_max<MASK>(s0, 0, visible), chunk_max<MASK>(s1, 32, visible)),
                 fmaxf(chunk_max<MASK>(s2, 64, visible), chunk_max<MASK>(s3, 96, visible)));
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
    // sub-tile c / 64; 16-byte chunk index XOR (row % 8)
    unsigned char* sub = p_tile + (c >> 6) * (BQ * 128) + r * 128;
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) {
        const int chunk = ((c & 63) >> 3) + q4;
        *reinterpret_cast<uint4*>(sub + ((chunk ^ (r & 7)) << 4)) =
            make_uint4(packed[4 * q4], packed[4 * q4 + 1], packed[4 * q4 + 2], packed[4 * q4 + 3]);
    }
    return sum0 + sum1;
}

__global__ void __launch_bounds__(AT_THREADS, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                            const int* __restrict__ page_table, int table_stride, const int* __restrict__ cu,
                            const int* __restrict__ starts, __nv_bfloat16* __restrict__ o, int B, int nh, int nkv,
                            float scale_log2, int* __restrict__ err) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const unsigned q_s = smem_u32(smem);
    const unsigned k_s = q_s + TILES * Q_BYTES, v_s = k_s + STAGES_KV * KV_BYTES, p_s = v_s + STAGES_KV * KV_BYTES;
    unsigned char* p_ptr = smem + TILES * Q_BYTES + 2 * STAGES_KV * KV_BYTES;
    unsigned long long* bars = (unsigned long long*)(p_ptr + TILES * P_BYTES);
    unsigned* tmem_holder = (unsigned*)(bars + B_COUNT);
    const unsigned bar0 = smem_u32(bars);
    auto bar = [&](int i) { return bar0 + 8u * (unsigned)i; };

    // which sequence and which pair of tiles of it.  Blocks are handed out heads first, then pairs, and the
    // heavy (late) pairs come first: every head's longest pair starts in the first wave and the short ones fill
    // the gaps at the end (longest job first), instead of a head's long pairs starting when the grid is nearly done
    int b = 0, pair = (int)(gridDim.y - 1 - blockIdx.y);
    for (; b < B; ++b) {
        const int pairs = (cu[b + 1] - cu[b] + TILES * BQ - 1) / (TILES * BQ);
        if (pair < pairs) break;
        pair -= pairs;
    }
    if (b >= B) return;
    const int h = blockIdx.x, g = h / (nh / nkv);
    const int row0 = cu[b] + pair * TILES * BQ;
    const int nq = min(TILES * BQ, cu[b + 1] - row0);
    const int pos0 = starts[b] + pair * TILES * BQ;
    // key blocks of either tile: up to the block of its last query
    int nb[TILES];
#pragma unroll
    for (int t = 0; t < TILES; ++t) nb[t] = nq > t * BQ ? (pos0 + min(nq, (t + 1) * BQ) - 1) / BKV + 1 : 0;
    const int nb_max = max(nb[0], nb[1]);
    const int* table = page_table + (size_t)b * table_stride;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        mbar_init(bar(B_Q), 1);
        for (int s = 0; s < STAGES_KV; ++s) {
            mbar_init(bar(B_KFULL + s), 1);
            mbar_init(bar(B_KEMPTY + s), 1);
            mbar_init(bar(B_VFULL + s), 1);
            mbar_init(bar(B_VEMPTY + s), 1);
        }
        for (int t = 0; t < TILES; ++t) {
            mbar_init(bar(B_SFULL + t), 1);
            mbar_init(bar(B_PFULL + t), 4);
            mbar_init(bar(B_PVDONE + t), 1);
            mbar_init(bar(B_SFREE + t), 4);
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
    // set-up done (it may have run under the tail of the kernel before): from here on the step's data
    mv_pdl_wait();

    if (warp < 4) {
        // registers move from this warpgroup to the softmax warps (168 each at launch)
        asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
        if (warp == 0) {
            if (lane == 0) {
                mbar_expect_tx(bar(B_Q), TILES * Q_BYTES);
                for (int t = 0; t < TILES; ++t) tma_load_2d(q_s + t * Q_BYTES, &map_q, h * HD, row0 + t * BQ, bar(B_Q));
                for (int j = 0; j < nb_max; ++j) {
                    const int s = j % STAGES_KV;
                    const unsigned ph = (unsigned)(j / STAGES_KV) & 1u;
                    const int pg0 = table[min(2 * j, table_stride - 1)], pg1 = table[min(2 * j + 1, table_stride - 1)];
                    if (!mbar_wait(bar(B_KEMPTY + s), ph ^ 1u, err, 11)) break;
                    mbar_expect_tx(bar(B_KFULL + s), KV_BYTES);
                    tma_load_2d(k_s + s * KV_BYTES, &map_kv, 0, ((pg0 * 2 + 0) * nkv + g) * PAGE, bar(B_KFULL + s));
                    tma_load_2d(k_s + s * KV_BYTES + KV_BYTES / 2, &map_kv, 0, ((pg1 * 2 + 0) * nkv + g) * PAGE,
                                bar(B_KFULL + s));
                    if (!mbar_wait(bar(B_VEMPTY + s), ph ^ 1u, err, 12)) break;
                    mbar_expect_tx(bar(B_VFULL + s), KV_BYTES);
                    tma_load_2d(v_s + s * KV_BYTES, &map_kv, 0, ((pg0 * 2 + 1) * nkv + g) * PAGE, bar(B_VFULL + s));
                    tma_load_2d(v_s + s * KV_BYTES + KV_BYTES / 2, &map_kv, 0, ((pg1 * 2 + 1) * nkv + g) * PAGE,
                                bar(B_VFULL + s));
                }
            }
        } else if (warp == 1) {
            if (lane == 0) {
                const unsigned idesc_qk = instr_desc(BQ, BKV);
                const unsigned idesc_pv = instr_desc(BQ, HD) | (1u << 16);          // B operand MN-major
                bool ok = mbar_wait(bar(B_Q), 0, err, 13);
                // S(t, j) = Q_t K_j^T; the caller has waited for K_j
                auto issue_qk = [&](int t, int j) {
                    const int s = j % STAGES_KV;
    #pragma unroll
                    for (int k = 0; k < HD / 16; ++k)
                        mma_f16(tmem_base + S_COL0 + (unsigned)t * BKV, smem_desc(q_s + t * Q_BYTES + k * 32),
                                smem_desc(k_s + s * KV_BYTES + k * 32), idesc_qk, k > 0 ? 1u : 0u);
                    mma_commit(bar(B_SFULL + t));
                };
                if (ok) ok = mbar_wait(bar(B_KFULL), 0, err, 14);
                if (ok) {
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    #pragma unroll
                    for (int t = 0; t < TILES; ++t)
                        if (nb[t] > 0) issue_qk(t, 0);
                    mma_commit(bar(B_KEMPTY));
                }
                for (int j = 0; j < nb_max && ok; ++j) {
                    const int s = j % STAGES_KV, s1 = (j + 1) % STAGES_KV;
                    const unsigned ph = (unsigned)(j / STAGES_KV) & 1u, ph1 = (unsigned)((j + 1) / STAGES_KV) & 1u;
                    // S(t, j + 1) as soon as the tile's softmax warps hold S(t, j) in registers
                    if (j + 1 < nb_max) {
                        if (!(ok = mbar_wait(bar(B_KFULL + s1), ph1, err, 14))) break;
#pragma unroll
                        for (int t = 0; t < TILES; ++t) {
                            if (!ok || j + 1 >= nb[t]) continue;
                            if (!(ok = mbar_wait(bar(B_SFREE + t), (unsigned)j & 1u, err, 15))) break;
                            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                            issue_qk(t, j + 1);
                        }
                        if (!ok) break;
                        mma_commit(bar(B_KEMPTY + s1));
                    }
                    if (!(ok = mbar_wait(bar(B_VFULL + s), ph, err, 17))) break;
#pragma unroll
                    for (int t = 0; t < TILES; ++t) {
                        if (!ok || j >= nb[t]) continue;
                        if (!(ok = mbar_wait(bar(B_PFULL + t), (unsigned)j & 1u, err, 16))) break;
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                        for (int k = 0; k < BKV / 16; ++k) {
                            // A: P, K-major, sub-tile k / 4 (64 keys), 32 bytes per 16 keys within it
                            const unsigned a_addr = p_s + t * P_BYTES + (k >> 2) * (BQ * 128) + (k & 3) * 32;
                            // B: V, MN-major: 16 keys are 16 rows of 128 bytes
                            const unsigned b_addr = v_s + s * KV_BYTES + k * 16 * 128;
                            mma_f16(tmem_base + O_COL0 + (unsigned)t * HD, smem_desc(a_addr), smem_desc_mn(b_addr),
                                    idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
                        }
                        mma_commit(bar(B_PVDONE + t));         // P and O of this tile are free again once it is done
                    }
                    mma_commit(bar(B_VEMPTY + s));
                }
            }
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
        const int t = (warp - 4) >> 2, quarter = warp & 3;
        const int r = quarter * 32 + lane;                   // this thread's query row within the tile
        const int pos = pos0 + t * BQ + r;
        const unsigned lane_addr = (unsigned)(quarter * 32) << 16;
        const unsigned s_addr = tmem_base + lane_addr + S_COL0 + (unsigned)t * BKV;
        const unsigned o_addr = tmem_base + lane_addr + O_COL0 + (unsigned)t * HD;
        unsigned char* p_tile = p_ptr + t * P_BYTES;
        const int my_nb = t ? nb[1] : nb[0];
        float m = -INFINITY, l = 0.f;                        // m: the reference maximum of the row's exponentials
        bool ok = true;
        for (int j = 0; j < my_nb && ok; ++j) {
            ok = mbar_wait(bar(B_SFULL + t), (unsigned)j & 1u, err, 19);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            unsigned s0[32], s1[32], s2[32], s3[32];
            tmem_ld32(s_addr, s0);
            tmem_ld32(s_addr + 32, s1);
            tmem_ld32(s_addr + 64, s2);
            tmem_ld32(s_addr + 96, s3);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            // the row is in registers: the S columns go back to the MMA warp for the next key block
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(B_SFREE + t));
            const int key0 = j * BKV;
            const int visible = pos - key0 + 1;               // keys of this block that the row sees
            // warp-uniform: the block reaches past the tile's first query
            const bool mask = key0 + BKV - 1 > pos0 + t * BQ;
            const float mx = mask ? row_max<true>(s0, s1, s2, s3, visible) : row_max<false>(s0, s1, s2, s3, visible);
            float corr = 1.0f;
            if (mx > m && (m == -INFINITY || (mx - m) * scale_log2 > RESCALE_ABOVE)) {
                corr = m == -INFINITY ? 0.f : ex2((m - mx) * scale_log2);
                m = mx;
            }
            // P (shared memory) and O (tensor memory) are the block before's until its PV is done
            if (j > 0) {
                ok = mbar_wait(bar(B_PVDONE + t), (unsigned)(j - 1) & 1u, err, 20);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            }
            if (j > 0 && __any_sync(0xffffffffu, corr != 1.0f)) {
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
            const float ref = m == -INFINITY ? 0.f : m * scale_log2;
            float sum;
            if (mask) {
                sum = (row_exp<true>(s0, 0, visible, scale_log2, ref, p_tile, r) +
                       row_exp<true>(s1, 32, visible, scale_log2, ref, p_tile, r)) +
                      (row_exp<true>(s2, 64, visible, scale_log2, ref, p_tile, r) +
                       row_exp<true>(s3, 96, visible, scale_log2, ref, p_tile, r));
            } else {
                sum = (row_exp<false>(s0, 0, visible, scale_log2, ref, p_tile, r) +
                       row_exp<false>(s1, 32, visible, scale_log2, ref, p_tile, r)) +
                      (row_exp<false>(s2, 64, visible, scale_log2, ref, p_tile, r) +
                       row_exp<false>(s3, 96, visible, scale_log2, ref, p_tile, r));
            }
            l = l * corr + sum;
            // P written (and O rescaled): tell the MMA warp
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(B_PFULL + t));
        }
        if (ok && my_nb > 0) ok = mbar_wait(bar(B_PVDONE + t), (unsigned)(my_nb - 1) & 1u, err, 21);
        if (ok && my_nb > 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float inv = 1.0f / l;
            const bool live = t * BQ + r < nq;
            __nv_bfloat16* dst = o + ((size_t)(row0 + t * BQ + r) * nh + h) * HD;
#pragma unroll
            for (int c = 0; c < HD; c += 32) {
                unsigned v[32];
                tmem_ld32(o_addr + (unsigned)c, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (live) {
#pragma unroll
                    for (int d = 0; d < 32; d += 8) {
                        unsigned w4[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const __nv_bfloat162 pk = __floats2bfloat162_rn(__uint_as_float(v[d + 2 * e]) * inv,
                                                                            __uint_as_float(v[d + 2 * e + 1]) * inv);
                            w4[e] = *reinterpret_cast<const unsigned*>(&pk);
                        }
                        *reinterpret_cast<uint4*>(dst + c + d) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
                    }
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

}  // namespace

// bfloat16, head size 64, pages of 64 tokens, no window.  pool_rows = pages * 2 * nkv * 64.
MV_API int mv_attention_prefill_tc(const void* q, const void* pool, long long pool_rows, const int* page_table,
                                   int table_stride, const int* cu, const int* starts, void* o, int N, int B, int nh,
                                   int nkv, float scale, int* err, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (nh % nkv || ((uintptr_t)q & 15) || ((uintptr_t)pool & 15)) return (int)cudaErrorInvalidValue;
    CUtensorMap mq, mkv;
    if (!tensor_map(q, N, nh * HD, BQ, &mq) || !tensor_map(pool, (int)pool_rows, HD, PAGE, &mkv))
        return (int)cudaErrorInvalidValue;
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(attention_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_SMEM);
        attr_set = true;
    }
    dim3 grid(nh, (N + TILES * BQ - 1) / (TILES * BQ) + B);
    if (grid.y > 65535u) return (int)cudaErrorInvalidValue;
    // a plain launch, not a programmatic one (see attention_decode_tc.cu); the kernel after it still
    // starts under this one's tail
    attention_prefill_tc_kernel<<<grid, AT_THREADS, AT_SMEM, stream>>>(
        mq, mkv, page_table, table_stride, cu, starts, (__nv_bfloat16*)o, B, nh, nkv,
        scale * 1.4426950408889634f, err);
    return mv_launch_status();
}
