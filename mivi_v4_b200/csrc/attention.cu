// Grouped-query attention over the paged cache: the kernel that prepares q, k
// and v (per-head RMSNorm, rotation, append to the cache) and the generic
// attention kernel that serves every head size, dtype, window and cut of the
// token stream.
//
// Cache layout of one layer: pool[page][2 (K, V)][kv head][page_size][hd].
// A sequence's token t lies in page table[b][t / page_size] at row
// t % page_size.  page_size is a power of two.
//
// Reference: per-head norm of q and k with one [hd] weight and the layer
// norms' eps, before the rotation (crates/mivi-model/src/transformer.rs:81-96);
// rotation of pairs (2i, 2i+1) by pos * theta^(-2i/hd)
// (crates/mivi-core/src/rope.rs:59-61, 219-229); store k and v at pos
// (transformer.rs:108); head h reads kv head h / (nh / nkv); scores
// q.k / sqrt(hd) over t <= pos, running-maximum softmax in 32-bit, weighted
// sum of v, division by the sum at the end (transformer.rs:114-167, 293-298).
#include "common.cuh"

#define MV_MAX_HEAD_DIM 256

// ----------------------------------------------------- q/k norm, rope, append
// One warp per token and group of SLOTS head slots; head slots are nh query heads, then nkv key
// heads, then nkv value heads, as they lie in a row of the fused projection.  A head's row is read
// once, two neighbouring elements a lane (8 bytes), and stays in registers; the rows of all of a
// warp's slots are requested before any is used, so their round trips to memory overlap.
template <typename T, int SLOTS>
__global__ void qk_prepare_kernel(const float* __restrict__ qkv, const float* __restrict__ wq,
                                  const float* __restrict__ wk, float eps,
                                  const float* __restrict__ inv_freq, int half_split,
                                  const int* __restrict__ positions, const int* __restrict__ seq_of,
                                  const int* __restrict__ page_table, int table_stride, int page_shift,
                                  T* __restrict__ pool, long long page_stride, int append,
                                  T* __restrict__ q_out, int N, int nh, int nkv, int hd) {
    mv_pdl_begin();
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const int slots_per_tok = nh + 2 * nkv;
    const int groups = (slots_per_tok + SLOTS - 1) / SLOTS;
    if (warp >= N * groups) return;
    const int n = warp / groups, hs0 = (warp - n * groups) * SLOTS;
    const int half = hd >> 1;
    constexpr int MAXJ = MV_MAX_HEAD_DIM / 64;
    float2 x[SLOTS][MAXJ];
#pragma unroll
    for (int s = 0; s < SLOTS; ++s) {
        const float* row = qkv + ((size_t)n * slots_per_tok + hs0 + s) * hd;
#pragma unroll
        for (int j = 0; j < MAXJ; ++j) {
            const int i = lane + 32 * j;
            x[s][j] = (hs0 + s < slots_per_tok && i < half) ? *reinterpret_cast<const float2*>(row + 2 * i)
                                                            : make_float2(0.f, 0.f);
        }
    }
    const int pos = positions[n];
    const int page_size = 1 << page_shift;
    // the rotation of pair i at this position is the same for every head: worked out once a warp
    float sn[MAXJ], cs[MAXJ];
#pragma unroll
    for (int j = 0; j < MAXJ; ++j) {
        const int i = lane + 32 * j;
        sn[j] = 0.f;
        cs[j] = 1.f;
        if (inv_freq && !half_split && i < half && hs0 < nh + nkv) sincosf((float)pos * inv_freq[i], &sn[j], &cs[j]);
    }
    // where this token's keys and values go (only asked for if one of the slots is a key or value head)
    T* kv_row = nullptr;
    if (append && hs0 + SLOTS > nh) {
        const int page = page_table[(size_t)seq_of[n] * table_stride + (pos >> page_shift)];
        if (mv_page_ok(page)) kv_row = pool + (size_t)page * page_stride + (size_t)(pos & (page_size - 1)) * hd;
    }
#pragma unroll
    for (int s = 0; s < SLOTS; ++s) {
        const int hs = hs0 + s;
        if (hs >= slots_per_tok) break;
        const bool is_q = hs < nh, is_k = !is_q && hs < nh + nkv;
        T* dst;
        if (is_q) {
            dst = q_out + ((size_t)n * nh + hs) * hd;
        } else {
            if (!append || kv_row == nullptr) continue;
            const int g = is_k ? hs - nh : hs - nh - nkv;
            dst = kv_row + ((size_t)(is_k ? 0 : 1) * nkv + g) * page_size * hd;
        }
        if (!is_q && !is_k) {                       // value head: copy
#pragma unroll
            for (int j = 0; j < MAXJ; ++j) {
                const int i = lane + 32 * j;
                if (i < half) mv_store2(dst + 2 * i, x[s][j].x, x[s][j].y);
            }
            continue;
        }
        const float* w = is_q ? wq : wk;
        float scale = 1.f;
        if (w) {
            float ss = 0.f;
#pragma unroll
            for (int j = 0; j < MAXJ; ++j) ss = fmaf(x[s][j].x, x[s][j].x, fmaf(x[s][j].y, x[s][j].y, ss));
            ss = mv_warp_sum(ss);
            scale = 1.0f / sqrtf(ss / (float)hd + eps);
        }
        if (!half_split) {
            // pairs (2i, 2i+1): the two elements a lane holds
#pragma unroll
            for (int j = 0; j < MAXJ; ++j) {
                const int i = lane + 32 * j;
                if (i >= half) break;
                float a = x[s][j].x, b = x[s][j].y;
                if (w) {
                    const float2 ww = *reinterpret_cast<const float2*>(w + 2 * i);
                    a = a * scale * ww.x;
                    b = b * scale * ww.y;
                }
                if (inv_freq) {
                    const float ra = a * cs[j] - b * sn[j], rb = a * sn[j] + b * cs[j];
                    a = ra; b = rb;
                }
                mv_store2(dst + 2 * i, a, b);
            }
        } else {
            // pairs (i, i + half): the partner of an element lies half a row away; read by element
            const float* row = qkv + ((size_t)n * slots_per_tok + hs) * hd;
            for (int i = lane; i < half; i += 32) {
                float a = row[i], b = row[i + half];
                if (w) { a = a * scale * w[i]; b = b * scale * w[i + half]; }
                if (inv_freq) {
                    float sn1, cs1;
                    sincosf((float)pos * inv_freq[i], &sn1, &cs1);
                    const float ra = a * cs1 - b * sn1, rb = a * sn1 + b * cs1;
                    a = ra; b = rb;
                }
                dst[i] = mv_from_f32<T>(a);
                dst[i + half] = mv_from_f32<T>(b);
            }
        }
    }
}


// The same for heads of 64 with the pairs (2i, 2i+1), the shape of every LFM2 model, when a step has
// many tokens: one warp a token.  A lane holds four consecutive elements (two pairs) of a head, so
// a half-warp is one head and the warp takes two heads a round, eight heads' loads in flight before
// any is used.  The rotation of a lane's two pairs at this position is worked out once for all the
// token's heads, and the per-head sums of squares need four shuffles inside the half-warp.  With few
// tokens (a large decode batch, a short prompt) a token's heads are dealt out to ``split`` warps, eight
// head slots a round each, so that the step still fills the device.
template <typename T>
__global__ void __launch_bounds__(256)
qk_prepare_hd64_kernel(const float* __restrict__ qkv, const float* __restrict__ wq, const float* __restrict__ wk,
                       float eps, const float* __restrict__ inv_freq, const int* __restrict__ positions,
                       const int* __restrict__ seq_of, const int* __restrict__ page_table, int table_stride,
                       int page_shift, T* __restrict__ pool, long long page_stride, int append,
                       T* __restrict__ q_out, int N, int nh, int nkv, int split) {
    mv_pdl_begin();
    constexpr int HD = 64, U = 4;
    const int wid = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int n = wid / split, part = wid - n * split;
    if (n >= N) return;
    const int lane = threadIdx.x & 31, sub = lane & 15, hsel = lane >> 4;
    const int slots = nh + 2 * nkv;
    const int pos = positions[n];
    const int page_size = 1 << page_shift;
    float sn0 = 0.f, cs0 = 1.f, sn1 = 0.f, cs1 = 1.f;
    if (inv_freq) {
        sincosf((float)pos * inv_freq[2 * sub], &sn0, &cs0);
        sincosf((float)pos * inv_freq[2 * sub + 1], &sn1, &cs1);
    }
    const float4 one = make_float4(1.f, 1.f, 1.f, 1.f);
    const float4 wq4 = wq ? *reinterpret_cast<const float4*>(wq + 4 * sub) : one;
    const float4 wk4 = wk ? *reinterpret_cast<const float4*>(wk + 4 * sub) : one;
    T* kv_row = nullptr;
    if (append) {
        const int page = page_table[(size_t)seq_of[n] * table_stride + (pos >> page_shift)];
        if (mv_page_ok(page)) kv_row = pool + (size_t)page * page_stride + (size_t)(pos & (page_size - 1)) * HD;
    }
    const float* row = qkv + (size_t)n * slots * HD + 4 * sub;
    const int per = ((slots + split - 1) / split + 2 * U - 1) / (2 * U) * (2 * U);       // whole rounds a warp
    const int last = min(slots, (part + 1) * per);
    for (int base = part * per; base < last; base += 2 * U) {
        float4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int hs = base + 2 * u + hsel;
            v[u] = hs < slots ? *reinterpret_cast<const float4*>(row + (size_t)hs * HD) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int hs = base + 2 * u + hsel;
            const bool is_q = hs < nh, is_k = !is_q && hs < nh + nkv;
            float4 x = v[u];
            // every lane takes part in the shuffles; what a lane beyond the last head computes is not stored
            float ss = fmaf(x.x, x.x, fmaf(x.y, x.y, fmaf(x.z, x.z, x.w * x.w)));
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (hs >= slots) continue;
            if (is_q || is_k) {
                const float* w = is_q ? wq : wk;
                if (w) {
                    const float scale = 1.0f / sqrtf(ss / (float)HD + eps);
                    const float4 ww = is_q ? wq4 : wk4;
                    x.x *= scale * ww.x; x.y *= scale * ww.y; x.z *= scale * ww.z; x.w *= scale * ww.w;
                }
                if (inv_freq) {
                    const float a0 = x.x * cs0 - x.y * sn0, b0 = x.x * sn0 + x.y * cs0;
                    const float a1 = x.z * cs1 - x.w * sn1, b1 = x.z * sn1 + x.w * cs1;
                    x = make_float4(a0, b0, a1, b1);
                }
            }
            T* dst;
            if (is_q) {
                dst = q_out + ((size_t)n * nh + hs) * HD;
            } else {
                if (!append || kv_row == nullptr) continue;
                const int g = is_k ? hs - nh : hs - nh - nkv;
                dst = kv_row + ((size_t)(is_k ? 0 : 1) * nkv + g) * page_size * HD;
            }
            mv_store4(dst + 4 * sub, x.x, x.y, x.z, x.w);
        }
    }
}

MV_GUARD_SETTER(attention)

MV_API int mv_qk_prepare(const float* qkv, const float* wq, const float* wk, float eps,
                         const float* inv_freq, int half_split, const int* positions,
                         const int* seq_of, const int* page_table, int table_stride, int page_size,
                         void* pool, long long page_stride, int append, void* q_out, int dtype, int N,
                         int nh, int nkv, int hd, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (hd % 2 || hd > MV_MAX_HEAD_DIM || (page_size & (page_size - 1))) return (int)cudaErrorInvalidValue;
    int page_shift = 0;
    while ((1 << page_shift) < page_size) ++page_shift;
    if (hd == 64 && !half_split && N >= 65 && nkv > 0 &&
        ((((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)pool | (uintptr_t)wq | (uintptr_t)wk) & 15) == 0) &&
        (page_stride * (dtype == MV_DT_BF16 ? 2 : 4)) % 16 == 0) {
        // many tokens with heads of 64: a warp a token; fewer than fill the device: several warps a token
        const int rounds = (nh + 2 * nkv + 7) / 8;
        int split = (2 * 148 * 8 + N - 1) / N;
        split = split < 1 ? 1 : (split > rounds ? rounds : split);
        const unsigned tblocks = (unsigned)(((long long)N * split + 7) / 8);
        if (dtype == MV_DT_BF16)
            mv_launch(qk_prepare_hd64_kernel<__nv_bfloat16>, tblocks, 256, 0, stream, qkv, wq, wk, eps, inv_freq,
                      positions, seq_of, page_table, table_stride, page_shift, (__nv_bfloat16*)pool, page_stride,
                      append, (__nv_bfloat16*)q_out, N, nh, nkv, split);
        else
            mv_launch(qk_prepare_hd64_kernel<float>, tblocks, 256, 0, stream, qkv, wq, wk, eps, inv_freq, positions,
                      seq_of, page_table, table_stride, page_shift, (float*)pool, page_stride, append,
                      (float*)q_out, N, nh, nkv, split);
        return mv_launch_status();
    }
    // many tokens: four head slots a warp, whose loads overlap; few: one, for more warps
    const int slots = N >= 64 ? 4 : 1;
    const long long warps = (long long)N * ((nh + 2 * nkv + slots - 1) / slots);
    const int threads = 256;
    const unsigned blocks = (unsigned)((warps * 32 + threads - 1) / threads);
    if (slots == 4 && dtype == MV_DT_BF16)
        mv_launch(qk_prepare_kernel<__nv_bfloat16, 4>, blocks, threads, 0, stream,
            qkv, wq, wk, eps, inv_freq, half_split, positions, seq_of, page_table, table_stride,
            page_shift, (__nv_bfloat16*)pool, page_stride, append, (__nv_bfloat16*)q_out, N, nh, nkv, hd);
    else if (slots == 4)
        mv_launch(qk_prepare_kernel<float, 4>, blocks, threads, 0, stream,
            qkv, wq, wk, eps, inv_freq, half_split, positions, seq_of, page_table, table_stride,
            page_shift, (float*)pool, page_stride, append, (float*)q_out, N, nh, nkv, hd);
    else if (dtype == MV_DT_BF16)
        mv_launch(qk_prepare_kernel<__nv_bfloat16, 1>, blocks, threads, 0, stream, 
            qkv, wq, wk, eps, inv_freq, half_split, positions, seq_of, page_table, table_stride,
            page_shift, (__nv_bfloat16*)pool, page_stride, append, (__nv_bfloat16*)q_out, N, nh, nkv, hd);
    else
        mv_launch(qk_prepare_kernel<float, 1>, blocks, threads, 0, stream, 
            qkv, wq, wk, eps, inv_freq, half_split, positions, seq_of, page_table, table_stride,
            page_shift, (float*)pool, page_stride, append, (float*)q_out, N, nh, nkv, hd);
    return mv_launch_status();
}

// ------------------------------------------------------------------ attention
// One warp per (token, query head).  Keys are taken 32 at a time: each lane
// scores one key (its row of hd elements is contiguous), the warp agrees on the
// running maximum, then the lanes split the head's elements for the weighted
// sum of the values.  Works for every hd that is a multiple of 8 up to 256.
template <typename T>
__global__ void __launch_bounds__(128)
attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ pool, long long page_stride,
                         const int* __restrict__ page_table, int table_stride, int page_shift,
                         const int* __restrict__ positions, const int* __restrict__ seq_of,
                         T* __restrict__ o, int N, int nh, int nkv, int hd, float scale, int window) {
    mv_pdl_begin();
    __shared__ float qs[4][MV_MAX_HEAD_DIM];
    const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long warp = (long long)blockIdx.x * 4 + wib;
    if (warp >= (long long)N * nh) return;
    const int n = (int)(warp / nh), h = (int)(warp - (long long)n * nh);
    const int g = h / (nh / nkv);
    const int pos = positions[n];
    const int page_size = 1 << page_shift;
    const int* table = page_table + (size_t)seq_of[n] * table_stride;
    const size_t v_off = (size_t)nkv * page_size * hd;

    const T* qrow = q + (size_t)n * nh * hd + (size_t)h * hd;
    for (int d = lane; d < hd; d += 32) qs[wib][d] = mv_to_f32(qrow[d]) * scale;
    __syncwarp();

    float acc[MV_MAX_HEAD_DIM / 32];
#pragma unroll
    for (int r = 0; r < MV_MAX_HEAD_DIM / 32; ++r) acc[r] = 0.f;
    float m = -INFINITY, l = 0.f;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;

    for (int t0 = lo; t0 <= pos; t0 += 32) {
        const int t = t0 + lane;
        const bool valid = t <= pos;
        const T* krow = nullptr;
        float s = -INFINITY;
        if (valid) {
            const int page = mv_read_page(table[t >> page_shift]);
            krow = pool + (size_t)page * page_stride + ((size_t)g * page_size + (t & (page_size - 1))) * hd;
            float dot = 0.f;
            for (int d = 0; d < hd; d += 8) {
                float kv[8];
                mv_load8(krow + d, kv);
#pragma unroll
                for (int e = 0; e < 8; ++e) dot = fmaf(qs[wib][d + e], kv[e], dot);
            }
            s = dot;
        }
        const float m_new = fmaxf(m, mv_warp_max(s));
        const float p = valid ? expf(s - m_new) : 0.f;
        const float corr = expf(m - m_new);          // 0 on the first chunk (m = -inf)
        l = l * corr + mv_warp_sum(p);
#pragma unroll
        for (int r = 0; r < MV_MAX_HEAD_DIM / 32; ++r) acc[r] *= corr;
        m = m_new;
        const int cnt = min(32, pos - t0 + 1);
        const unsigned long long kaddr = (unsigned long long)krow;
        for (int j = 0; j < cnt; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const T* vrow = (const T*)__shfl_sync(0xffffffffu, kaddr, j) + v_off;
#pragma unroll
            for (int r = 0; r < MV_MAX_HEAD_DIM / 32; ++r) {
                const int d = lane + 32 * r;
                if (d < hd) acc[r] = fmaf(pj, mv_to_f32(vrow[d]), acc[r]);
            }
        }
    }
    const float inv = 1.0f / l;
    T* orow = o + (size_t)n * nh * hd + (size_t)h * hd;
#pragma unroll
    for (int r = 0; r < MV_MAX_HEAD_DIM / 32; ++r) {
        const int d = lane + 32 * r;
        if (d < hd) orow[d] = mv_from_f32<T>(acc[r] * inv);
    }
}

MV_API int mv_attention_generic(const void* q, const void* pool, long long page_stride,
                                const int* page_table, int table_stride, int page_size,
                                const int* positions, const int* seq_of, void* o, int dtype, int N,
                                int nh, int nkv, int hd, float scale, int window, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (hd % 8 || hd > MV_MAX_HEAD_DIM || nh % nkv || (page_size & (page_size - 1)))
        return (int)cudaErrorInvalidValue;
    int page_shift = 0;
    while ((1 << page_shift) < page_size) ++page_shift;
    const unsigned blocks = (unsigned)(((long long)N * nh + 3) / 4);
    if (dtype == MV_DT_BF16)
        mv_launch(attention_generic_kernel<__nv_bfloat16>, blocks, 128, 0, stream, 
            (const __nv_bfloat16*)q, (const __nv_bfloat16*)pool, page_stride, page_table, table_stride,
            page_shift, positions, seq_of, (__nv_bfloat16*)o, N, nh, nkv, hd, scale, window);
    else
        mv_launch(attention_generic_kernel<float>, blocks, 128, 0, stream, 
            (const float*)q, (const float*)pool, page_stride, page_table, table_stride, page_shift,
            positions, seq_of, (float*)o, N, nh, nkv, hd, scale, window);
    return mv_launch_status();
}
