// Attention for steps with few query tokens (decoding): every query token reads
// the whole cache of its sequence, so the work is split over the KEYS, not the
// queries ("flash decoding"), and the query heads that share a kv head are
// served together so that each key and value is loaded once for all of them.
//
// Block = (query token, kv head x head tile, key split), 4 warps.  A block's
// share of the keys [lo, pos] is cut into runs of 32; the warps take the runs
// in turn.  In a run each lane scores one key against the GT query heads (the
// key's row is contiguous), the warp agrees on the running maximum of each
// head, then the lanes split the head's elements for the weighted sum of the
// values.  The warps' partial (max, sum, weighted values) are merged in shared
// memory; with more than one split the merged partials go to scratch memory,
// and the block that finishes last for a (token, kv head) merges the splits in
// split order and writes the output.  "Last" is decided by a ticket counter
// that the last block resets, so nobody waits and the scratch needs no
// clearing between launches.  All arithmetic is float32; the result does not
// depend on which block happened to be last.
//
// Cache layout and the formulas are those of attention.cu (reference:
// crates/mivi-model/src/transformer.rs:114-167, 293-298, which is already a
// one-query running-maximum loop over the cached keys).
#include "common.cuh"

namespace {

constexpr int WARPS = 4;

template <typename T, int GT, int R>   // GT query heads per block, R = ceil(hd / 32)
__global__ void __launch_bounds__(WARPS * 32)
attention_decode_kernel(const T* __restrict__ q, const T* __restrict__ pool, long long page_stride,
                        const int* __restrict__ page_table, int table_stride, int page_shift,
                        const int* __restrict__ positions, const int* __restrict__ seq_of, T* __restrict__ o,
                        float* __restrict__ part_o, float* __restrict__ part_ml, int* __restrict__ tickets,
                        int nh, int nkv, int hd, float scale, int window, int splits, int head_tiles) {
    mv_pdl_begin();
    extern __shared__ float sm[];
    // q heads [GT][hd] (scaled), then per warp: o [GT][hd], m [GT], l [GT]
    float* qs = sm;
    float* wo = qs + GT * hd;
    float* wm = wo + WARPS * GT * hd;
    float* wl = wm + WARPS * GT;
    __shared__ int is_last;

    const int n = blockIdx.x, split = blockIdx.z;
    const int g = blockIdx.y / head_tiles, tile = blockIdx.y - g * head_tiles;
    const int G = nh / nkv;
    const int h0 = g * G + tile * GT;                 // first query head of this block
    const int nheads = min(GT, G - tile * GT);        // heads of this tile that exist
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = positions[n];
    const int page_size = 1 << page_shift;
    const int* table = page_table + (size_t)seq_of[n] * table_stride;
    const size_t v_off = (size_t)nkv * page_size * hd;

    for (int i = threadIdx.x; i < GT * hd; i += WARPS * 32) {
        const int hh = i / hd, d = i - hh * hd;
        qs[i] = hh < nheads ? mv_to_f32(q[(size_t)n * nh * hd + (size_t)(h0 + hh) * hd + d]) * scale : 0.f;
    }
    __syncthreads();

    // this block's keys: runs of 32 from lo, dealt to the splits in equal contiguous shares
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int runs = (pos - lo + 32) >> 5;            // ceil((pos - lo + 1) / 32)
    const int per = (runs + splits - 1) / splits;
    const int run_begin = split * per, run_end = min(runs, run_begin + per);

    float acc[GT][R], m[GT], l[GT];
#pragma unroll
    for (int hh = 0; hh < GT; ++hh) {
        m[hh] = -INFINITY;
        l[hh] = 0.f;
#pragma unroll
        for (int r = 0; r < R; ++r) acc[hh][r] = 0.f;
    }

    for (int run = run_begin + warp; run < run_end; run += WARPS) {
        const int t = lo + (run << 5) + lane;
        const bool valid = t <= pos;
        const int cnt = min(32, pos - (lo + (run << 5)) + 1);
        // the row of this lane's key; lanes past the last key point at the run's first row
        const int tt = valid ? t : lo + (run << 5);
        const T* krow = pool + (size_t)mv_read_page(table[tt >> page_shift]) * page_stride +
                        ((size_t)g * page_size + (tt & (page_size - 1))) * hd;
        const unsigned long long kaddr = (unsigned long long)krow;
        float s[GT];
        constexpr int EPV = 16 / sizeof(T);                // elements per 16-byte load
        constexpr int VG = R <= 2 ? 16 : 8;                 // keys whose values are requested together
        float vv[VG][R];
        auto load_values = [&](int j0) {
#pragma unroll
            for (int jj = 0; jj < VG; ++jj) {
                const T* vrow = (const T*)__shfl_sync(0xffffffffu, kaddr, (j0 + jj) & 31) + v_off;
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const int d = lane + 32 * r;
                    vv[jj][r] = d < hd ? mv_to_f32(vrow[d]) : 0.f;
                }
            }
        };
        // Everything this run needs from memory is requested before any of it is used: a stretch of
        // this lane's key and the values of the first VG keys.  A lane then waits once, not per load.
        uint4 raw[8];
#pragma unroll
        for (int v = 0; v < 8; ++v)
            if (v * EPV < hd) raw[v] = *reinterpret_cast<const uint4*>(krow + v * EPV);
        load_values(0);
#pragma unroll
        for (int hh = 0; hh < GT; ++hh) s[hh] = 0.f;
        for (int d0 = 0; d0 < hd; d0 += 8 * EPV) {
            if (d0 > 0) {
#pragma unroll
                for (int v = 0; v < 8; ++v)
                    if (d0 + v * EPV < hd) raw[v] = *reinterpret_cast<const uint4*>(krow + d0 + v * EPV);
            }
#pragma unroll
            for (int v = 0; v < 8; ++v) {
                if (d0 + v * EPV < hd) {
                    float kv[EPV];
                    mv_unpack16(raw[v], kv, (const T*)nullptr);
#pragma unroll
                    for (int hh = 0; hh < GT; ++hh) {
                        const float* qh = qs + hh * hd + d0 + v * EPV;
#pragma unroll
                        for (int e = 0; e < EPV; ++e) s[hh] = fmaf(qh[e], kv[e], s[hh]);
                    }
                }
            }
        }
        float p[GT];
#pragma unroll
        for (int hh = 0; hh < GT; ++hh) {
            if (!valid) s[hh] = -INFINITY;
            const float m_new = fmaxf(m[hh], mv_warp_max(s[hh]));
            p[hh] = valid ? expf(s[hh] - m_new) : 0.f;
            const float corr = expf(m[hh] - m_new);
            l[hh] = l[hh] * corr + mv_warp_sum(p[hh]);
#pragma unroll
            for (int r = 0; r < R; ++r) acc[hh][r] *= corr;
            m[hh] = m_new;
        }
        // weighted sum of the values; lanes past the last key carry weight 0
        for (int j0 = 0; j0 < cnt; j0 += VG) {
            if (j0 > 0) load_values(j0);
#pragma unroll
            for (int jj = 0; jj < VG; ++jj) {
#pragma unroll
                for (int hh = 0; hh < GT; ++hh) {
                    const float pj = __shfl_sync(0xffffffffu, p[hh], (j0 + jj) & 31);
#pragma unroll
                    for (int r = 0; r < R; ++r) acc[hh][r] = fmaf(pj, vv[jj][r], acc[hh][r]);
                }
            }
        }
    }

    // merge the warps of this block
#pragma unroll
    for (int hh = 0; hh < GT; ++hh) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int d = lane + 32 * r;
            if (d < hd) wo[(warp * GT + hh) * hd + d] = acc[hh][r];
        }
        if (lane == 0) { wm[warp * GT + hh] = m[hh]; wl[warp * GT + hh] = l[hh]; }
    }
    __syncthreads();
    const size_t part_base = ((size_t)n * nh + h0) * splits;      // [(n, head), split]
    for (int i = threadIdx.x; i < nheads * hd; i += WARPS * 32) {
        const int hh = i / hd, d = i - hh * hd;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) mm = fmaxf(mm, wm[w * GT + hh]);
        float ll = 0.f, oo = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float c = wm[w * GT + hh] == -INFINITY ? 0.f : expf(wm[w * GT + hh] - mm);
            ll += wl[w * GT + hh] * c;
            oo += wo[(w * GT + hh) * hd + d] * c;
        }
        if (splits == 1) {
            o[(size_t)n * nh * hd + (size_t)(h0 + hh) * hd + d] = mv_from_f32<T>(oo / ll);
        } else {
            const size_t pi = part_base + (size_t)hh * splits + split;
            part_o[pi * hd + d] = oo;
            if (d == 0) { part_ml[pi * 2] = mm; part_ml[pi * 2 + 1] = ll; }
        }
    }
    if (splits == 1) return;

    // the block that arrives last for this (token, kv head, tile) merges the splits
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        int* ticket = tickets + (size_t)n * nkv * head_tiles + blockIdx.y;
        const int seen = atomicAdd(ticket, 1);
        is_last = seen == splits - 1;
        if (is_last) *ticket = 0;                     // ready for the next launch
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    for (int i = threadIdx.x; i < nheads * hd; i += WARPS * 32) {
        const int hh = i / hd, d = i - hh * hd;
        const size_t pb = part_base + (size_t)hh * splits;
        float mm = -INFINITY;
        // other blocks wrote these: read them past this SM's L1, which may hold a stale line
        for (int sp = 0; sp < splits; ++sp) mm = fmaxf(mm, __ldcg(&part_ml[(pb + sp) * 2]));
        float ll = 0.f, oo = 0.f;
        for (int sp = 0; sp < splits; ++sp) {
            const float ms = __ldcg(&part_ml[(pb + sp) * 2]);
            const float c = ms == -INFINITY ? 0.f : expf(ms - mm);
            ll += __ldcg(&part_ml[(pb + sp) * 2 + 1]) * c;
            oo += __ldcg(&part_o[(pb + sp) * hd + d]) * c;
        }
        o[(size_t)n * nh * hd + (size_t)(h0 + hh) * hd + d] = mv_from_f32<T>(oo / ll);
    }
}

template <typename T, int GT, int R>
int launch(const void* q, const void* pool, long long page_stride, const int* page_table, int table_stride,
           int page_shift, const int* positions, const int* seq_of, void* o, float* part_o, float* part_ml,
           int* tickets, int N, int nh, int nkv, int hd, float scale, int window, int splits, int head_tiles,
           cudaStream_t stream) {
    const size_t smem = (size_t)(GT * hd + WARPS * GT * hd + 2 * WARPS * GT) * sizeof(float);
    dim3 grid(N, nkv * head_tiles, splits);
    mv_launch(attention_decode_kernel<T, GT, R>, grid, WARPS * 32, smem, stream, 
        (const T*)q, (const T*)pool, page_stride, page_table, table_stride, page_shift, positions, seq_of,
        (T*)o, part_o, part_ml, tickets, nh, nkv, hd, scale, window, splits, head_tiles);
    return mv_launch_status();
}

template <typename T>
int dispatch(int gt, int r, const void* q, const void* pool, long long page_stride, const int* page_table,
             int table_stride, int page_shift, const int* positions, const int* seq_of, void* o, float* part_o,
             float* part_ml, int* tickets, int N, int nh, int nkv, int hd, float scale, int window, int splits,
             int head_tiles, cudaStream_t stream) {
#define MV_CASE(GT, R)                                                                                         \
    if (gt == GT && r == R)                                                                                    \
        return launch<T, GT, R>(q, pool, page_stride, page_table, table_stride, page_shift, positions, seq_of, \
                                o, part_o, part_ml, tickets, N, nh, nkv, hd, scale, window, splits, head_tiles, \
                                stream);
    MV_CASE(1, 1) MV_CASE(1, 2) MV_CASE(1, 4) MV_CASE(1, 8)
    MV_CASE(2, 1) MV_CASE(2, 2) MV_CASE(2, 4) MV_CASE(2, 8)
    MV_CASE(4, 1) MV_CASE(4, 2) MV_CASE(4, 4) MV_CASE(4, 8)
    MV_CASE(8, 1) MV_CASE(8, 2) MV_CASE(8, 4) MV_CASE(8, 8)
#undef MV_CASE
    return (int)cudaErrorInvalidValue;
}

}  // namespace

MV_GUARD_SETTER(attention_decode)

// Scratch: part_o [N * nh * splits * hd] floats, part_ml [N * nh * splits * 2]
// floats, tickets [N * nkv * head_tiles] ints that are zero before the first
// launch (the kernel leaves them zero).  gt = query heads per block (1, 2, 4, 8),
// head_tiles = ceil((nh / nkv) / gt).
MV_API int mv_attention_decode(const void* q, const void* pool, long long page_stride, const int* page_table,
                               int table_stride, int page_size, const int* positions, const int* seq_of,
                               void* o, int dtype, float* part_o, float* part_ml, int* tickets, int N, int nh,
                               int nkv, int hd, float scale, int window, int splits, int gt, int head_tiles,
                               cudaStream_t stream) {
    if (N <= 0) return 0;
    if (hd % 8 || hd > 256 || nh % nkv || (page_size & (page_size - 1)) || splits < 1 ||
        gt * head_tiles < nh / nkv)
        return (int)cudaErrorInvalidValue;
    int page_shift = 0;
    while ((1 << page_shift) < page_size) ++page_shift;
    const int r32 = (hd + 31) / 32;
    const int r = r32 <= 1 ? 1 : (r32 <= 2 ? 2 : (r32 <= 4 ? 4 : 8));
    if (dtype == MV_DT_BF16)
        return dispatch<__nv_bfloat16>(gt, r, q, pool, page_stride, page_table, table_stride, page_shift,
                                       positions, seq_of, o, part_o, part_ml, tickets, N, nh, nkv, hd, scale,
                                       window, splits, head_tiles, stream);
    return dispatch<float>(gt, r, q, pool, page_stride, page_table, table_stride, page_shift, positions, seq_of,
                           o, part_o, part_ml, tickets, N, nh, nkv, hd, scale, window, splits, head_tiles,
                           stream);
}

// ---------------------------------------------------------------------------
// mv_attention_decode_static: the same kernel for callers that cannot allocate.
// Declared and documented in attention_decode_static.h.
// ---------------------------------------------------------------------------
#include "attention_decode_static.h"

#include <stdio.h>

namespace {

// One array holds all three scratch regions.  It is part of the library's image:
// every GPU that loads the library keeps these bytes until the process exits.
constexpr size_t STATIC_TICKETS = MV_STATIC_ATTN_MAX_TICKETS;                  // ints, first
constexpr size_t STATIC_FLOATS = MV_STATIC_ATTN_MAX_FLOATS;                    // part_ml and part_o share these
static __device__ __align__(256) unsigned char g_static_attn_scratch[STATIC_TICKETS * sizeof(int) +
                                                                     STATIC_FLOATS * sizeof(float)];

constexpr int MAX_DEVICES = 64;
unsigned char* g_static_attn_ptr[MAX_DEVICES] = {nullptr};

int fail(char* errbuf, int errbuf_len, int code, const char* fmt, long long a = 0, long long b = 0) {
    if (errbuf && errbuf_len > 0) snprintf(errbuf, (size_t)errbuf_len, fmt, a, b);
    return code;
}

}  // namespace

MV_API int mv_attention_decode_static(const void* q, const void* pool, long long page_stride,
                                      const int* page_table, int table_stride, int page_size,
                                      const int* positions, const int* seq_of, void* o, int dtype, int N, int nh,
                                      int nkv, int hd, float scale, int window, int splits, cudaStream_t stream,
                                      char* errbuf, int errbuf_len) {
    if (errbuf && errbuf_len > 0) errbuf[0] = 0;
    if (N <= 0) return 0;
    // everything the kernel assumes is checked before the GPU is touched
    if (nkv <= 0 || nh <= 0 || nh % nkv)
        return fail(errbuf, errbuf_len, 1, "%lld heads are not a multiple of %lld kv heads", nh, nkv);
    if (splits < 1) return fail(errbuf, errbuf_len, 1, "splits must be at least 1, got %lld", splits);
    if (hd <= 0 || hd % 8 || hd > 256)
        return fail(errbuf, errbuf_len, 1, "head size %lld must be a multiple of 8 between 8 and 256", hd);
    if (page_size <= 0 || (page_size & (page_size - 1)))
        return fail(errbuf, errbuf_len, 1, "page size %lld is not a power of two", page_size);
    if (dtype != MV_DT_F32 && dtype != MV_DT_BF16)
        return fail(errbuf, errbuf_len, 1, "dtype %lld is neither 0 (float32) nor 1 (bfloat16)", dtype);
    if (!q || !pool || !page_table || !positions || !seq_of || !o)
        return fail(errbuf, errbuf_len, 1, "an input or output pointer is null");
    const int G = nh / nkv;
    const int gt = G <= 1 ? 1 : (G <= 2 ? 2 : (G <= 4 ? 4 : 8));
    const int head_tiles = (G + gt - 1) / gt;
    const size_t tickets = (size_t)N * nkv * head_tiles;
    const size_t ml_floats = (size_t)N * nh * splits * 2;
    const size_t o_floats = (size_t)N * nh * splits * hd;
    // the counters are used only when the keys are split
    if (splits > 1 && tickets > STATIC_TICKETS)
        return fail(errbuf, errbuf_len, 2,
                    "the built-in scratch holds %lld (token, kv head) counters, this call needs %lld; "
                    "use mv_attention_decode with scratch of your own", (long long)STATIC_TICKETS, (long long)tickets);
    if (splits > 1 && ml_floats + o_floats > STATIC_FLOATS)
        return fail(errbuf, errbuf_len, 2,
                    "the built-in scratch holds %lld floats of partial results, this call needs %lld; "
                    "use fewer splits or mv_attention_decode with scratch of your own",
                    (long long)STATIC_FLOATS, (long long)(ml_floats + o_floats));

    // Once per device, with that device current: the array's name is only a host-side stand-in
    // here; the device address has to be asked for.
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= MAX_DEVICES)
        return fail(errbuf, errbuf_len, 3, "cudaGetDevice failed or device ordinal out of range (error %lld, device %lld)",
                    (long long)e, dev);
    if (g_static_attn_ptr[dev] == nullptr) {
        unsigned char* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_static_attn_scratch);
        if (e != cudaSuccess || p == nullptr)
            return fail(errbuf, errbuf_len, 3, "cudaGetSymbolAddress failed on device %lld with error %lld", dev,
                        (long long)e);
        g_static_attn_ptr[dev] = p;
    }
    unsigned char* base = g_static_attn_ptr[dev];
    int* d_tickets = reinterpret_cast<int*>(base);
    float* d_ml = reinterpret_cast<float*>(base + STATIC_TICKETS * sizeof(int));
    float* d_o = d_ml + ml_floats;
    // The counters must start at zero; the array still holds whatever the last call left.
    if (splits > 1) {
        e = cudaMemsetAsync(d_tickets, 0, tickets * sizeof(int), stream);
        if (e != cudaSuccess) return fail(errbuf, errbuf_len, 3, "cudaMemsetAsync failed with error %lld", (long long)e);
    }
    const int rc = mv_attention_decode(q, pool, page_stride, page_table, table_stride, page_size, positions, seq_of,
                                       o, dtype, d_o, d_ml, d_tickets, N, nh, nkv, hd, scale, window, splits, gt,
                                       head_tiles, stream);
    if (rc != 0) return fail(errbuf, errbuf_len, 4, "the kernel launch failed with CUDA error %lld", rc);
    return 0;
}
