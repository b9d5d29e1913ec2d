// Causal attention for steps with many query tokens (prefill), bfloat16, over
// the paged cache: the work is split over the QUERIES.  Block = 64 consecutive
// query tokens of one sequence for one query head, 4 warps of 16 queries.  The
// keys and values the tile may see are streamed through shared memory in
// blocks of 64 (cp.async, double-buffered); scores and weighted sums run on the
// tensor cores (mma.sync m16n8k16, float32 accumulation) with the running-
// maximum softmax in float32 registers in between, the scores' accumulator
// fragments being reused as the left operand of the second product.
//
// Queries are the step's packed tokens; their positions are absolute, and the
// keys come from the cache (which already holds this step's own keys), so a
// prompt that arrives in several steps sees exactly the same keys as one that
// arrives whole.  A window > 0 keeps keys t > pos - window.
//
// Same formulas as attention.cu (reference: crates/mivi-model/src/
// transformer.rs:114-167, 293-298: scores q.k / sqrt(hd) over t <= pos,
// softmax in 32-bit with a running maximum, weighted sum of v, one division
// at the end).
#include "common.cuh"

namespace {

constexpr int QT = 64;          // queries per block
constexpr int KB = 64;          // keys per block of the stream
constexpr int NWARPS = 4;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                 "{%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&v);
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}

template <int HD>
__global__ void __launch_bounds__(NWARPS * 32)
attention_prefill_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ pool,
                         long long page_stride, const int* __restrict__ page_table, int table_stride,
                         int page_shift, const int* __restrict__ cu, const int* __restrict__ starts,
                         __nv_bfloat16* __restrict__ o, int B, int nh, int nkv, float scale_log2, int window) {
    constexpr int LDS = HD + 8;                       // padded row: conflict-free fragment loads
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* ks = reinterpret_cast<__nv_bfloat16*>(smem_raw);     // [2][KB][LDS]
    __nv_bfloat16* vs = ks + 2 * KB * LDS;                              // [2][KB][LDS]

    // which sequence and which tile of it
    int b = 0, tile = blockIdx.x;
    for (; b < B; ++b) {
        const int tiles = (cu[b + 1] - cu[b] + QT - 1) / QT;
        if (tile < tiles) break;
        tile -= tiles;
    }
    if (b >= B) return;
    const int h = blockIdx.y, g = h / (nh / nkv);
    const int row0 = cu[b] + tile * QT;               // first packed row of the tile
    const int rows_in_seq = cu[b + 1] - cu[b];
    const int nq = min(QT, rows_in_seq - tile * QT);  // queries of this tile that exist
    const int pos0 = starts[b] + tile * QT;           // position of the tile's first query
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gq = lane >> 2, t4 = lane & 3;
    const int page_size = 1 << page_shift;
    const int* table = page_table + (size_t)b * table_stride;
    const size_t v_off = (size_t)nkv * page_size * HD;

    // the two query rows of this thread (gq and gq + 8 of the warp's 16)
    const int qi0 = warp * 16 + gq, qi1 = qi0 + 8;
    const int p0 = pos0 + qi0, p1 = pos0 + qi1;       // their positions
    unsigned qf[HD / 16][4];
    {
        const __nv_bfloat16* r0 = q + ((size_t)(row0 + min(qi0, nq - 1)) * nh + h) * HD;
        const __nv_bfloat16* r1 = q + ((size_t)(row0 + min(qi1, nq - 1)) * nh + h) * HD;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
            qf[kk][0] = *reinterpret_cast<const unsigned*>(r0 + kk * 16 + 2 * t4);
            qf[kk][1] = *reinterpret_cast<const unsigned*>(r1 + kk * 16 + 2 * t4);
            qf[kk][2] = *reinterpret_cast<const unsigned*>(r0 + kk * 16 + 2 * t4 + 8);
            qf[kk][3] = *reinterpret_cast<const unsigned*>(r1 + kk * 16 + 2 * t4 + 8);
        }
    }

    float oacc[HD / 8][4];
#pragma unroll
    for (int j = 0; j < HD / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) oacc[j][e] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    // keys this tile can see: from the first query's window start to the last query's position
    const int last_pos = pos0 + nq - 1;
    const int first_key = window > 0 ? max(0, pos0 - window + 1) : 0;
    const int kb_begin = first_key / KB, kb_end = last_pos / KB + 1;

    auto load_block = [&](int kb, int buf) {
        // 64 rows of HD elements for K and for V, 16 bytes per copy
        constexpr int CHUNKS = HD / 8;
        for (int idx = threadIdx.x; idx < KB * CHUNKS; idx += NWARPS * 32) {
            const int r = idx / CHUNKS, c = idx - r * CHUNKS;
            const int t = min(kb * KB + r, last_pos);                    // rows past the end repeat the last key
            const int page = mv_read_page(table[t >> page_shift]);
            const __nv_bfloat16* src = pool + (size_t)page * page_stride +
                                       ((size_t)g * page_size + (t & (page_size - 1))) * HD + c * 8;
            cp_async16(ks + ((size_t)buf * KB + r) * LDS + c * 8, src);
            cp_async16(vs + ((size_t)buf * KB + r) * LDS + c * 8, src + v_off);
        }
    };

    load_block(kb_begin, 0);
    cp_async_commit();
    for (int kb = kb_begin; kb < kb_end; ++kb) {
        const int buf = (kb - kb_begin) & 1;
        if (kb + 1 < kb_end) load_block(kb + 1, buf ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();

        const __nv_bfloat16* kt = ks + (size_t)buf * KB * LDS;
        const __nv_bfloat16* vt = vs + (size_t)buf * KB * LDS;
        float s[KB / 8][4];
#pragma unroll
        for (int j = 0; j < KB / 8; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
            const __nv_bfloat16* krow = kt + (size_t)(j * 8 + gq) * LDS + 2 * t4;
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk) {
                const unsigned b0 = *reinterpret_cast<const unsigned*>(krow + kk * 16);
                const unsigned b1 = *reinterpret_cast<const unsigned*>(krow + kk * 16 + 8);
                mma_bf16(s[j], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], b0, b1);
            }
        }
        // mask, then the running maximum of the two rows
        const int key0 = kb * KB;
        const bool need_mask = key0 + KB - 1 > pos0 + warp * 16 || (window > 0 && key0 <= pos0 + warp * 16 + 15 - window);
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < KB / 8; ++j) {
            if (need_mask) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int t = key0 + j * 8 + 2 * t4 + (e & 1);
                    const int p = (e < 2) ? p0 : p1;
                    if (t > p || (window > 0 && t <= p - window)) s[j][e] = -INFINITY;
                }
            }
            mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
            mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        // a row whose keys are all masked so far keeps m = -inf; use 0 as its reference
        const float ref0 = mn0 == -INFINITY ? 0.f : mn0 * scale_log2;
        const float ref1 = mn1 == -INFINITY ? 0.f : mn1 * scale_log2;
        const float c0 = m0 == -INFINITY ? 0.f : exp2f(m0 * scale_log2 - ref0);
        const float c1 = m1 == -INFINITY ? 0.f : exp2f(m1 * scale_log2 - ref1);
        m0 = mn0; m1 = mn1;
        float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
        for (int j = 0; j < KB / 8; ++j) {
            s[j][0] = exp2f(s[j][0] * scale_log2 - ref0);
            s[j][1] = exp2f(s[j][1] * scale_log2 - ref0);
            s[j][2] = exp2f(s[j][2] * scale_log2 - ref1);
            s[j][3] = exp2f(s[j][3] * scale_log2 - ref1);
            sum0 += s[j][0] + s[j][1];
            sum1 += s[j][2] + s[j][3];
        }
        l0 = l0 * c0 + sum0;
        l1 = l1 * c1 + sum1;
#pragma unroll
        for (int j = 0; j < HD / 8; ++j) {
            oacc[j][0] *= c0; oacc[j][1] *= c0;
            oacc[j][2] *= c1; oacc[j][3] *= c1;
        }
        // O += P V, 16 keys at a time
#pragma unroll
        for (int kk = 0; kk < KB / 16; ++kk) {
            const unsigned a0 = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            const unsigned a1 = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            const unsigned a2 = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            const unsigned a3 = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int dj = 0; dj < HD / 16; ++dj) {
                // four 8x8 blocks of V: (keys 0-7, d 0-7), (keys 8-15, d 0-7), (keys 0-7, d 8-15), (keys 8-15, d 8-15)
                unsigned vb[4];
                const int mi = lane >> 3, r = lane & 7;
                ldmatrix_x4_trans(vb, vt + (size_t)(kk * 16 + (mi & 1) * 8 + r) * LDS + dj * 16 + (mi >> 1) * 8);
                mma_bf16(oacc[2 * dj], a0, a1, a2, a3, vb[0], vb[1]);
                mma_bf16(oacc[2 * dj + 1], a0, a1, a2, a3, vb[2], vb[3]);
            }
        }
        __syncthreads();
    }

    // row sums live in the four lanes of a quad
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float i0 = 1.f / l0, i1 = 1.f / l1;
    if (qi0 < nq) {
        __nv_bfloat16* dst = o + ((size_t)(row0 + qi0) * nh + h) * HD + 2 * t4;
#pragma unroll
        for (int j = 0; j < HD / 8; ++j)
            *reinterpret_cast<unsigned*>(dst + j * 8) = pack_bf16(oacc[j][0] * i0, oacc[j][1] * i0);
    }
    if (qi1 < nq) {
        __nv_bfloat16* dst = o + ((size_t)(row0 + qi1) * nh + h) * HD + 2 * t4;
#pragma unroll
        for (int j = 0; j < HD / 8; ++j)
            *reinterpret_cast<unsigned*>(dst + j * 8) = pack_bf16(oacc[j][2] * i1, oacc[j][3] * i1);
    }
}

template <int HD>
int launch(const void* q, const void* pool, long long page_stride, const int* page_table, int table_stride,
           int page_shift, const int* cu, const int* starts, void* o, int N, int B, int nh, int nkv, float scale,
           int window, cudaStream_t stream) {
    constexpr int LDS = HD + 8;
    const size_t smem = (size_t)4 * KB * LDS * sizeof(__nv_bfloat16);
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(attention_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        attr_set = true;
    }
    dim3 grid((N + QT - 1) / QT + B, nh);         // an upper bound of the tiles; spare blocks return at once
    attention_prefill_kernel<HD><<<grid, NWARPS * 32, smem, stream>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)pool, page_stride, page_table, table_stride, page_shift,
        cu, starts, (__nv_bfloat16*)o, B, nh, nkv, scale * 1.4426950408889634f, window);
    return mv_launch_status();
}

}  // namespace

// bfloat16 only; head sizes that are multiples of 16 up to 128.  Other sizes and
// float32 use the generic kernel.
MV_GUARD_SETTER(attention_prefill)

MV_API int mv_attention_prefill(const void* q, const void* pool, long long page_stride, const int* page_table,
                                int table_stride, int page_size, const int* cu, const int* starts, void* o,
                                int N, int B, int nh, int nkv, int hd, float scale, int window,
                                cudaStream_t stream) {
    if (N <= 0) return 0;
    if (nh % nkv || (page_size & (page_size - 1))) return (int)cudaErrorInvalidValue;
    int page_shift = 0;
    while ((1 << page_shift) < page_size) ++page_shift;
#define MV_HD(D)                                                                                              \
    case D: return launch<D>(q, pool, page_stride, page_table, table_stride, page_shift, cu, starts, o, N, B, \
                             nh, nkv, scale, window, stream);
    switch (hd) {
        MV_HD(16) MV_HD(32) MV_HD(48) MV_HD(64) MV_HD(80) MV_HD(96) MV_HD(112) MV_HD(128)
        default: return (int)cudaErrorInvalidValue;
    }
#undef MV_HD
}
