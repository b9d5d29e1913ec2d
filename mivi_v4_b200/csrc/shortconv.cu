// The gated short convolution between its two projections, for any cut of the
// token stream: prompts of unequal lengths, chunks of a prompt, single tokens.
//
// p[n, 0:H] = B, p[n, H:2H] = C, p[n, 2H:3H] = X (the order is fixed by the
// reference: crates/mivi-model/src/ssm.rs:81-85); bx = B * X;
// y_t[d] = sum_j w[d, j] * bx_{t-(k-1)+j}[d], tap k-1 on the current token
// (ssm.rs:92-140); z = C * y (ssm.rs:110).  The reference keeps the last k
// values of bx per channel and shifts them each token; here a sequence's
// slot keeps the k-1 values BEFORE its next token, state[slot, j, d] =
// bx at position len-(k-1)+j, zero at the start of a sequence, so a step
// that begins in the middle of a sequence finds its left context there.
#include "common.cuh"

#define MV_MAX_CONV_K 16

// One thread per (token, channel).  Reads the old state only.
template <typename TO>
__global__ void shortconv_fwd_kernel(const float* __restrict__ p, const float* __restrict__ w,
                                     const float* __restrict__ bias, const float* __restrict__ state,
                                     const int* __restrict__ positions, const int* __restrict__ seq_of,
                                     const int* __restrict__ slots, const int* __restrict__ starts,
                                     TO* __restrict__ z, int N, int H, int k) {
    mv_pdl_begin();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)N * H) return;
    const int n = (int)(i / H), d = (int)(i - (long long)n * H);
    const int b = seq_of[n];
    const int pos = positions[n], start = starts[b];
    const float* st = state + (size_t)mv_read_slot(slots[b]) * (k - 1) * H;
    float y = bias ? bias[d] : 0.f;
    for (int j = 0; j < k; ++j) {
        const int src = pos - (k - 1) + j;
        float bx;
        if (src >= start) {
            const float* row = p + (size_t)(n - (pos - src)) * 3 * H;
            bx = row[d] * row[2 * H + d];
        } else {
            bx = st[(size_t)(src - start + (k - 1)) * H + d];
        }
        y = fmaf(w[d * k + j], bx, y);
    }
    z[i] = mv_from_f32<TO>(p[(size_t)n * 3 * H + H + d] * y);
}

// The same, four channels per thread with 16-byte loads (H a multiple of 4).
template <typename TO>
__global__ void shortconv_fwd_vec4_kernel(const float* __restrict__ p, const float* __restrict__ w,
                                          const float* __restrict__ bias, const float* __restrict__ state,
                                          const int* __restrict__ positions, const int* __restrict__ seq_of,
                                          const int* __restrict__ slots, const int* __restrict__ starts,
                                          TO* __restrict__ z, int N, int H, int k) {
    mv_pdl_begin();
    const int H4 = H >> 2;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)N * H4) return;
    const int n = (int)(i / H4), d = (int)(i - (long long)n * H4) * 4;
    const int b = seq_of[n];
    const int pos = positions[n], start = starts[b];
    const float* st = state + (size_t)mv_read_slot(slots[b]) * (k - 1) * H;
    float4 y = bias ? *reinterpret_cast<const float4*>(bias + d) : make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j < k; ++j) {
        const int src = pos - (k - 1) + j;
        float4 bx;
        if (src >= start) {
            const float* row = p + (size_t)(n - (pos - src)) * 3 * H;
            const float4 bb = *reinterpret_cast<const float4*>(row + d);
            const float4 xx = *reinterpret_cast<const float4*>(row + 2 * H + d);
            bx = make_float4(bb.x * xx.x, bb.y * xx.y, bb.z * xx.z, bb.w * xx.w);
        } else {
            bx = *reinterpret_cast<const float4*>(st + (size_t)(src - start + (k - 1)) * H + d);
        }
        y.x = fmaf(w[(d + 0) * k + j], bx.x, y.x);
        y.y = fmaf(w[(d + 1) * k + j], bx.y, y.y);
        y.z = fmaf(w[(d + 2) * k + j], bx.z, y.z);
        y.w = fmaf(w[(d + 3) * k + j], bx.w, y.w);
    }
    const float4 c = *reinterpret_cast<const float4*>(p + (size_t)n * 3 * H + H + d);
    mv_store4(z + (size_t)n * H + d, c.x * y.x, c.y * y.y, c.z * y.z, c.w * y.w);
}

// The same for a convolution of width KW (2 to 4) and steps of many tokens: a thread takes four
// channels of TOK consecutive tokens and carries the last KW-1 values of B*x in registers, so a
// token's B, C and x are read once (the kernel above reads B and x of the KW-1 tokens before it
// again for every token).  Where the tile crosses into another sequence the history is fetched anew.
template <typename TO, int KW, int TOK>
__global__ void shortconv_fwd_tile_kernel(const float* __restrict__ p, const float* __restrict__ w,
                                          const float* __restrict__ bias, const float* __restrict__ state,
                                          const int* __restrict__ positions, const int* __restrict__ seq_of,
                                          const int* __restrict__ slots, const int* __restrict__ starts,
                                          TO* __restrict__ z, int N, int H) {
    mv_pdl_begin();
    const int H4 = H >> 2;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int tiles = (N + TOK - 1) / TOK;
    if (i >= (long long)tiles * H4) return;
    const int tile = (int)(i / H4), d = (int)(i - (long long)tile * H4) * 4;
    float taps[4][KW];
#pragma unroll
    for (int e = 0; e < 4; ++e)
#pragma unroll
        for (int j = 0; j < KW; ++j) taps[e][j] = w[(d + e) * KW + j];
    const float4 bs = bias ? *reinterpret_cast<const float4*>(bias + d) : make_float4(0.f, 0.f, 0.f, 0.f);
    float4 hist[KW - 1];
    int prev_b = -1;
#pragma unroll
    for (int t = 0; t < TOK; ++t) {
        const int n = tile * TOK + t;
        if (n >= N) break;
        const int b = seq_of[n];
        const float* row = p + (size_t)n * 3 * H;
        if (b != prev_b) {
            // the KW-1 values before this token: from this step's rows or from the carried state
            const int pos = positions[n], start = starts[b];
            const float* st = state + (size_t)mv_read_slot(slots[b]) * (KW - 1) * H;
#pragma unroll
            for (int j = 0; j < KW - 1; ++j) {
                const int src = pos - (KW - 1) + j;
                if (src >= start) {
                    const float* r2 = p + (size_t)(n - (pos - src)) * 3 * H;
                    const float4 bb = *reinterpret_cast<const float4*>(r2 + d);
                    const float4 xx = *reinterpret_cast<const float4*>(r2 + 2 * H + d);
                    hist[j] = make_float4(bb.x * xx.x, bb.y * xx.y, bb.z * xx.z, bb.w * xx.w);
                } else {
                    hist[j] = *reinterpret_cast<const float4*>(st + (size_t)(src - start + (KW - 1)) * H + d);
                }
            }
            prev_b = b;
        }
        const float4 bb = *reinterpret_cast<const float4*>(row + d);
        const float4 c = *reinterpret_cast<const float4*>(row + H + d);
        const float4 xx = *reinterpret_cast<const float4*>(row + 2 * H + d);
        const float4 cur = make_float4(bb.x * xx.x, bb.y * xx.y, bb.z * xx.z, bb.w * xx.w);
        float4 y = bs;
#pragma unroll
        for (int j = 0; j < KW - 1; ++j) {
            y.x = fmaf(taps[0][j], hist[j].x, y.x);
            y.y = fmaf(taps[1][j], hist[j].y, y.y);
            y.z = fmaf(taps[2][j], hist[j].z, y.z);
            y.w = fmaf(taps[3][j], hist[j].w, y.w);
        }
        y.x = fmaf(taps[0][KW - 1], cur.x, y.x);
        y.y = fmaf(taps[1][KW - 1], cur.y, y.y);
        y.z = fmaf(taps[2][KW - 1], cur.z, y.z);
        y.w = fmaf(taps[3][KW - 1], cur.w, y.w);
        mv_store4(z + (size_t)n * H + d, c.x * y.x, c.y * y.y, c.z * y.z, c.w * y.w);
#pragma unroll
        for (int j = 0; j + 1 < KW - 1; ++j) hist[j] = hist[j + 1];
        hist[KW - 2] = cur;
    }
}

// One thread per (sequence, channel): the state after this step's tokens.
// New entry j holds position start+len-(k-1)+j: from this step's tokens if it
// lies in them, else old entry len+j.  Going up in j, every old entry is read
// before it is overwritten (len >= 1).
__global__ void shortconv_state_kernel(const float* __restrict__ p, float* __restrict__ state,
                                       const int* __restrict__ cu, const int* __restrict__ slots,
                                       const int* __restrict__ lens, int B, int H, int k) {
    mv_pdl_begin();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)B * H) return;
    const int b = (int)(i / H), d = (int)(i - (long long)b * H);
    const int len = lens[b];
    if (len <= 0 || !mv_slot_ok(slots[b])) return;
    float* st = state + (size_t)slots[b] * (k - 1) * H;
    const int first_row = cu[b];
    for (int j = 0; j < k - 1; ++j) {
        const int rel = len - (k - 1) + j;          // index among this step's tokens
        float v;
        if (rel >= 0) {
            const float* row = p + (size_t)(first_row + rel) * 3 * H;
            v = row[d] * row[2 * H + d];
        } else {
            v = st[(size_t)(len + j) * H + d];
        }
        st[(size_t)j * H + d] = v;
    }
}

// A step in which every sequence brings one token (decoding): one thread per
// (sequence, channel) does both, reading its k-1 state values once, writing z
// and the shifted state.  Nobody else reads or writes that thread's column.
template <typename TO>
__global__ void shortconv_decode_kernel(const float* __restrict__ p, const float* __restrict__ w,
                                        const float* __restrict__ bias, float* __restrict__ state,
                                        const int* __restrict__ slots, TO* __restrict__ z, int B, int H, int k) {
    mv_pdl_begin();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)B * H) return;
    const int b = (int)(i / H), d = (int)(i - (long long)b * H);
    if (!mv_slot_ok(slots[b])) return;
    float* st = state + (size_t)slots[b] * (k - 1) * H;
    const float* row = p + (size_t)b * 3 * H;
    const float bx = row[d] * row[2 * H + d];
    float y = bias ? bias[d] : 0.f;
    float prev = 0.f;
    for (int j = 0; j < k - 1; ++j) {
        const float v = st[(size_t)j * H + d];
        y = fmaf(w[d * k + j], v, y);
        if (j > 0) st[(size_t)(j - 1) * H + d] = v;         // shift towards the older end
        prev = v;
    }
    (void)prev;
    if (k > 1) st[(size_t)(k - 2) * H + d] = bx;
    y = fmaf(w[d * k + (k - 1)], bx, y);
    z[i] = mv_from_f32<TO>(row[H + d] * y);
}

// The same with four consecutive channels a thread, for widths up to 4 and 16-byte aligned rows: every
// load and store is 16 bytes (8 for bfloat16 z) and all of a thread's loads are requested before any is used.
template <typename TO, int KW>
__global__ void __launch_bounds__(256)
shortconv_decode_vec4_kernel(const float* __restrict__ p, const float* __restrict__ w, const float* __restrict__ bias,
                             float* __restrict__ state, const int* __restrict__ slots, TO* __restrict__ z, int B, int H) {
    mv_pdl_begin();
    const int hv = H >> 2;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)B * hv) return;
    const int b = (int)(i / hv), d = 4 * (int)(i - (long long)b * hv);
    if (!mv_slot_ok(slots[b])) return;
    float* st = state + (size_t)slots[b] * (KW - 1) * H + d;
    const float* row = p + (size_t)b * 3 * H + d;
    const float4 Bv = *reinterpret_cast<const float4*>(row), Cv = *reinterpret_cast<const float4*>(row + H),
                 Xv = *reinterpret_cast<const float4*>(row + 2 * H);
    float4 kept[KW > 1 ? KW - 1 : 1], tp[KW];
#pragma unroll
    for (int j = 0; j < KW - 1; ++j) kept[j] = *reinterpret_cast<const float4*>(st + (size_t)j * H);
#pragma unroll
    for (int j = 0; j < KW; ++j) tp[j] = *reinterpret_cast<const float4*>(w + (size_t)d * KW + 4 * j);   // 4 KW taps in a row
    float4 bb = make_float4(0.f, 0.f, 0.f, 0.f);
    if (bias) bb = *reinterpret_cast<const float4*>(bias + d);
    const float* tpf = reinterpret_cast<const float*>(tp);
    const float bx[4] = {Bv.x * Xv.x, Bv.y * Xv.y, Bv.z * Xv.z, Bv.w * Xv.w};
    const float cv[4] = {Cv.x, Cv.y, Cv.z, Cv.w};
    float y[4] = {bb.x, bb.y, bb.z, bb.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
#pragma unroll
        for (int j = 0; j < KW - 1; ++j) y[e] = fmaf(tpf[e * KW + j], reinterpret_cast<const float*>(&kept[j])[e], y[e]);
        y[e] = fmaf(tpf[e * KW + (KW - 1)], bx[e], y[e]);
    }
#pragma unroll
    for (int j = 1; j < KW - 1; ++j) *reinterpret_cast<float4*>(st + (size_t)(j - 1) * H) = kept[j];   // shift towards the older end
    if (KW > 1) *reinterpret_cast<float4*>(st + (size_t)(KW - 2) * H) = make_float4(bx[0], bx[1], bx[2], bx[3]);
    mv_store4(z + (size_t)b * H + d, cv[0] * y[0], cv[1] * y[1], cv[2] * y[2], cv[3] * y[3]);
}

MV_GUARD_SETTER(shortconv)

MV_API int mv_shortconv_decode(const float* p, const float* w, const float* bias, float* state,
                               const int* slots, void* z, int z_dtype, int B, int H, int k,
                               cudaStream_t stream) {
    if (B <= 0) return 0;
    if (k < 1 || k > MV_MAX_CONV_K) return (int)cudaErrorInvalidValue;
    const int threads = 256;
    const bool aligned = H % 4 == 0 && (((uintptr_t)p | (uintptr_t)w | (uintptr_t)state | (uintptr_t)bias | (uintptr_t)z) & 15) == 0;
    if (aligned && k <= 4) {
        const unsigned vblocks = (unsigned)(((long long)B * (H / 4) + threads - 1) / threads);
#define MV_DEC(TO_, KW_) mv_launch(shortconv_decode_vec4_kernel<TO_, KW_>, vblocks, threads, 0, stream, p, w, bias, state, \
                                   slots, (TO_*)z, B, H)
        if (z_dtype == MV_DT_BF16) {
            if (k == 1) MV_DEC(__nv_bfloat16, 1); else if (k == 2) MV_DEC(__nv_bfloat16, 2);
            else if (k == 3) MV_DEC(__nv_bfloat16, 3); else MV_DEC(__nv_bfloat16, 4);
        } else {
            if (k == 1) MV_DEC(float, 1); else if (k == 2) MV_DEC(float, 2); else if (k == 3) MV_DEC(float, 3); else MV_DEC(float, 4);
        }
#undef MV_DEC
        return mv_launch_status();
    }
    const unsigned blocks = (unsigned)(((long long)B * H + threads - 1) / threads);
    if (z_dtype == MV_DT_BF16)
        mv_launch(shortconv_decode_kernel<__nv_bfloat16>, blocks, threads, 0, stream, p, w, bias, state, slots,
                  (__nv_bfloat16*)z, B, H, k);
    else
        mv_launch(shortconv_decode_kernel<float>, blocks, threads, 0, stream, p, w, bias, state, slots, (float*)z,
                  B, H, k);
    return mv_launch_status();
}

MV_API int mv_shortconv(const float* p, const float* w, const float* bias, float* state,
                        const int* positions, const int* seq_of, const int* cu, const int* slots,
                        const int* starts, const int* lens, void* z, int z_dtype, int N, int B, int H,
                        int k, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (k < 1 || k > MV_MAX_CONV_K) return (int)cudaErrorInvalidValue;
    const int threads = 256;
    const unsigned blocks = (unsigned)(((long long)N * H + threads - 1) / threads);
    constexpr int TOK = 4;
    const bool aligned = H % 4 == 0 && (((uintptr_t)p | (uintptr_t)state | (uintptr_t)bias | (uintptr_t)z) & 15) == 0;
    if (aligned && N >= 64 && k >= 2 && k <= 4) {
        const unsigned tblocks = (unsigned)(((long long)((N + TOK - 1) / TOK) * (H / 4) + threads - 1) / threads);
#define MV_TILE(TO_, KW_) mv_launch(shortconv_fwd_tile_kernel<TO_, KW_, TOK>, tblocks, threads, 0, stream, p, w, bias, \
                                    state, positions, seq_of, slots, starts, (TO_*)z, N, H)
        if (z_dtype == MV_DT_BF16) {
            if (k == 2) MV_TILE(__nv_bfloat16, 2); else if (k == 3) MV_TILE(__nv_bfloat16, 3); else MV_TILE(__nv_bfloat16, 4);
        } else {
            if (k == 2) MV_TILE(float, 2); else if (k == 3) MV_TILE(float, 3); else MV_TILE(float, 4);
        }
#undef MV_TILE
    } else if (aligned) {
        const unsigned vblocks = (unsigned)(((long long)N * (H / 4) + threads - 1) / threads);
        if (z_dtype == MV_DT_BF16)
            mv_launch(shortconv_fwd_vec4_kernel<__nv_bfloat16>, vblocks, threads, 0, stream, p, w, bias, state, positions,
                      seq_of, slots, starts, (__nv_bfloat16*)z, N, H, k);
        else
            mv_launch(shortconv_fwd_vec4_kernel<float>, vblocks, threads, 0, stream, p, w, bias, state, positions, seq_of,
                      slots, starts, (float*)z, N, H, k);
    } else if (z_dtype == MV_DT_BF16)
        mv_launch(shortconv_fwd_kernel<__nv_bfloat16>, blocks, threads, 0, stream, p, w, bias, state, positions, seq_of, slots,
                                                            starts, (__nv_bfloat16*)z, N, H, k);
    else
        mv_launch(shortconv_fwd_kernel<float>, blocks, threads, 0, stream, p, w, bias, state, positions, seq_of, slots,
                                                            starts, (float*)z, N, H, k);
    if (k > 1) {
        const unsigned sblocks = (unsigned)(((long long)B * H + threads - 1) / threads);
        mv_launch(shortconv_state_kernel, sblocks, threads, 0, stream, p, state, cu, slots, lens, B, H, k);
    }
    return mv_launch_status();
}
