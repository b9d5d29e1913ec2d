// Y[M, N] = X[M, K] . W[N, K]^T for a handful of tokens (M <= 64), bfloat16
// operands, float32 accumulation: the matrix product of a decode step, whose
// cost is reading W once from HBM.
//
// The weight matrix takes the tensor core's M side ("swap-AB"): a warp owns 16
// (or 32) consecutive rows of W and a slice of K, and streams its rows straight
// from global memory into mma.sync fragments with 16-byte loads; the tokens
// are the N side, 8 per n-tile.  A thread's 16 bytes are 8 consecutive k of one
// row.  The fragment layout of mma.m16n8k16 wants k = {2t, 2t+1, 2t+8, 2t+9}
// from lane t of a group, but a dot product does not care in which order k is
// summed as long as both operands agree: the thread's first 4 values serve
// one mma as those four k, the last 4 the next mma, and X is loaded with the
// same rule, so no shuffle and no shared-memory staging of W is needed.
//
// Work is cut small so that many blocks are resident on every SM and their
// phases (load, multiply, reduce) overlap: a block is 4 warps on one tile of
// rows and one slice of K.  The slices of a tile form a thread-block cluster
// along K; each block adds its warps' partial sums in shared memory, then the
// cluster's first block reads the others' sums through distributed shared
// memory, adds them in rank order and runs the epilogue.  Every sum has a fixed
// order, so the result is the same in every run.
//
// The first loads of W are issued before the kernel waits for its predecessor
// (programmatic dependent launch): weights do not depend on it, and the stream
// of weights from HBM then does not pause at the kernel boundary.
//
// A norm between two products can ride on them (steps of few tokens pay more for a launch than for
// the norm's arithmetic).  The product that completes the residual stream (mode 2) may also write
// bf16(x_new * g), g the next norm's weight, and per row-tile sums of x_new^2 ("emit").  The product
// that consumes those rows then multiplies each token's results by rsqrt(sum / dim + eps), summing
// the tile sums in a fixed order ("scale"): W (x g s) = s W (x g), and the statistics stay float32.
//
// Two more epilogues finish a mixer's elementwise work where the values already are, which saves the
// step a launch a layer: the gated short convolution of a decode step after its input projection
// (ConvTail; crates/mivi-model/src/ssm.rs:81-140) and the preparation of q, k and v after their
// projection (HeadTail; crates/mivi-model/src/transformer.rs:81-108).  And a product can be told what
// the step's next product will read (Ahead): it then asks the L2 cache for the beginning of it.
//
// What it replaces in the reference: quantized_matvec, one output row per
// dot product over the input (crates/mivi-quant/src/lib.rs:75-135).
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace {


// The two optional ends of a norm carried by products (all null / 0 when unused).
struct NormLink {
    const float* scale_part;           // consumer: [tokens][scale_stride], n_scale_part sums of squares per row it reads
    int n_scale_part, scale_stride;
    float inv_dim, eps;
    const float* emit_g;               // producer (mode 2): the next norm's weight [N]
    __nv_bfloat16* emit_x;             // bf16(x_new * g) [M, N]
    float* emit_part;                  // [tokens][emit_stride] sums of x_new^2 over each tile's rows
    int emit_stride;
};

// The gated short convolution of a decode step as the epilogue of its input projection (the CONV
// kernels): W is [3 N, K] with the rows of B, C and x one after another; a block takes 16 channels,
// that is 16 rows out of each third, so that one lane ends up with B, C and x of one channel and
// can finish it: B * x, the k taps over the sequence's k-1 kept values, the shift of those, C *.
struct ConvTail {
    const float* taps;                 // [N][k]
    const float* conv_bias;            // [N] or null
    float* state;                      // [slots][k - 1][N], the last k-1 values of B * x per sequence
    const int* slots;                  // [M]: the slot of token m's sequence (one token a sequence)
    int k;
};

// The preparation of q, k and v as the epilogue of their fused projection (the HEADS kernels, head
// size 64): W is [(nh + 2 nkv) 64, K], query heads, then key heads, then value heads; a block takes
// one head, and a warp finishes it for one token with two elements a lane: RMSNorm over the head
// (q and k), rotation by the token's position (q and k), then q goes out in bfloat16 and k and v
// into the token's row of its sequence's cache page.
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
    int half_split, table_stride, page_shift, nh, nkv;
};

// What the NEXT product of the step will read (or null): once a block has its own weights, its
// threads ask the L2 cache for their share of these lines, so that HBM keeps streaming through
// this kernel's reduce, its tail and the next launch instead of pausing there.
struct Ahead {
    const void* w;
    long long bytes;
};

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                 "{%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// NT: n-tiles of 8 tokens; RT: tiles of 16 weight rows per warp; UNROLL: k-steps
// of 32 whose W loads are issued together.  gridDim.x = K slices (= cluster
// size), gridDim.y = row tiles.
// TAIL 1 (RT == 3): the three row tiles of a warp are N rows apart, N counts channels, see ConvTail.
// TAIL 2 (RT == 4): a tile is one head, see HeadTail.
template <int NT, int RT, int UNROLL, int WARPS, int TAIL>
__global__ void __launch_bounds__(WARPS * 32)
gemm_small_m_kernel(const __nv_bfloat16* __restrict__ W, const __nv_bfloat16* __restrict__ X,
                    const float* __restrict__ bias, void* __restrict__ out, int mode, int M, int N, int K,
                    int ldo, const NormLink link, const ConvTail tail, const HeadTail heads, const Ahead ahead) {
    constexpr bool CONV = TAIL == 1, HEADS = TAIL == 2;
    static_assert(!CONV || RT == 3, "the convolution epilogue takes B, C and x: three row tiles");
    static_assert(!HEADS || RT == 4, "the head epilogue takes heads of 64 rows");
    constexpr int ROWS = RT * 16, COLS = NT * 8, LDR = COLS + 1;
    extern __shared__ float sm[];
    float* red = sm;                                   // [WARPS][ROWS][LDR] partial sums of the warps
    float* csum = sm + WARPS * ROWS * LDR;             // [COLS][ROWS] their sum: this block's share
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.y * (CONV ? 16 : ROWS);
    const int slices = gridDim.x, slice = blockIdx.x;

    float acc[RT][NT][4];
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[r][j][e] = 0.f;

    // rows this thread loads; rows past N are read from row N-1 and dropped at the end
    const __nv_bfloat16* wrow[RT][2];
#pragma unroll
    for (int r = 0; r < RT; ++r) {
        if constexpr (CONV) {
            wrow[r][0] = W + ((size_t)r * N + min(n0 + g, N - 1)) * K;
            wrow[r][1] = W + ((size_t)r * N + min(n0 + g + 8, N - 1)) * K;
        } else {
            wrow[r][0] = W + (size_t)min(n0 + r * 16 + g, N - 1) * K;
            wrow[r][1] = W + (size_t)min(n0 + r * 16 + g + 8, N - 1) * K;
        }
    }
    const __nv_bfloat16* xrow[NT];
    bool xok[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        xok[j] = j * 8 + g < M;
        xrow[j] = X + (size_t)min(j * 8 + g, M - 1) * K;
    }

    // k-steps of 32: first cut into the cluster's slices, then into this block's warps
    const int ksteps = (K + 31) >> 5;
    const int per_slice = (ksteps + slices - 1) / slices;
    const int s_begin = slice * per_slice, s_end = min(ksteps, s_begin + per_slice);
    const int per = (max(0, s_end - s_begin) + WARPS - 1) / WARPS;
    const int ks_begin = s_begin + warp * per, ks_end = min(s_end, ks_begin + per);

    auto load_w = [&](uint4 (&w)[UNROLL][RT][2], int ks) {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int k = ((ks + u) << 5) + 8 * t;
            const bool ok = (ks + u) < ks_end && k < K;
#pragma unroll
            for (int r = 0; r < RT; ++r)
#pragma unroll
                for (int h = 0; h < 2; ++h)
                    w[u][r][h] = ok ? ld_stream16(wrow[r][h] + k) : make_uint4(0, 0, 0, 0);
        }
    };
    uint4 w[UNROLL][RT][2];
    load_w(w, ks_begin);              // weights do not depend on the kernel before this one
    mv_pdl_wait();
    for (int ks = ks_begin; ks < ks_end; ks += UNROLL) {
        uint4 x[UNROLL][NT];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int k = ((ks + u) << 5) + 8 * t;
            const bool ok = (ks + u) < ks_end && k < K;
#pragma unroll
            for (int j = 0; j < NT; ++j)
                x[u][j] = (ok && xok[j]) ? *reinterpret_cast<const uint4*>(xrow[j] + k) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u)
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int r = 0; r < RT; ++r) {
                    mma_bf16(acc[r][j], w[u][r][0].x, w[u][r][1].x, w[u][r][0].y, w[u][r][1].y, x[u][j].x, x[u][j].y);
                    mma_bf16(acc[r][j], w[u][r][0].z, w[u][r][1].z, w[u][r][0].w, w[u][r][1].w, x[u][j].z, x[u][j].w);
                }
        if (ks + UNROLL < ks_end) load_w(w, ks + UNROLL);
    }
    // From here on this block only adds up and writes: the next kernel may start to launch and
    // send out its own first loads.  (Earlier would let its blocks take the place of blocks of
    // this kernel that have not started yet.)
    mv_pdl_launch_dependents();
    if (ahead.w) {
        const unsigned n_lines = (unsigned)(ahead.bytes >> 7);
        const unsigned n_threads = gridDim.x * gridDim.y * blockDim.x;
        for (unsigned l = (blockIdx.y * gridDim.x + blockIdx.x) * blockDim.x + threadIdx.x; l < n_lines; l += n_threads)
            asm volatile("prefetch.global.L2 [%0];" ::"l"((const char*)ahead.w + ((size_t)l << 7)));
    }

    // What the epilogue's first item (most warps have at most one) will want from global memory is asked
    // for now and not touched until then: the answers arrive while the sums go through shared memory
    // and the cluster barrier.
    const int m_first = slice + slices * warp;
    const int n_lane = n0 + lane;
    const bool lane_ok = TAIL == 0 && lane < ROWS && n_lane < N;
    float early_old = 0.f, early_g = 0.f, early_part[4] = {0.f, 0.f, 0.f, 0.f};
    if (m_first < M) {
        if (mode == 2 && lane_ok) early_old = ((const float*)out)[(size_t)m_first * ldo + n_lane];
        if (link.scale_part) {
#pragma unroll
            for (int e = 0; e < 4; ++e)
                if (lane + 32 * e < link.n_scale_part)
                    early_part[e] = link.scale_part[(size_t)m_first * link.scale_stride + lane + 32 * e];
        }
    }
    if (link.emit_x && lane_ok) early_g = link.emit_g[n_lane];

    // the warps' partial sums -> shared memory -> their sum in warp order
    float* mine = red + (size_t)warp * ROWS * LDR;
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            const int row = r * 16 + g, col = j * 8 + 2 * t;
            mine[row * LDR + col] = acc[r][j][0];
            mine[row * LDR + col + 1] = acc[r][j][1];
            mine[(row + 8) * LDR + col] = acc[r][j][2];
            mine[(row + 8) * LDR + col + 1] = acc[r][j][3];
        }
    __syncthreads();
    // csum is laid out [token][row]: the lanes of a warp, one row each, then read consecutive words,
    // which is what a read through distributed shared memory wants (scattered words crawl there)
    for (int idx = threadIdx.x; idx < ROWS * COLS; idx += WARPS * 32) {
        const int c = idx / ROWS, r = idx - c * ROWS;
        float v = 0.f;
#pragma unroll
        for (int wp = 0; wp < WARPS; ++wp) v += red[(size_t)wp * ROWS * LDR + r * LDR + c];
        csum[c * ROWS + r] = v;
    }

    // The slices of this tile are added in rank order.  The work of adding is dealt out to all blocks
    // of the cluster: an item is the tile's rows for one token (one row per lane), item m belongs to
    // block m mod slices.  A lane first requests its value from every slice, then adds.
    const float* share[8];
    if (slices > 1) {
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        for (int s = 0; s < slices; ++s) share[s] = cluster.map_shared_rank(csum, s);
    } else {
        __syncthreads();
        share[0] = csum;
    }
    if constexpr (CONV) {
        // rows 0-15 of the tile are B, 16-31 C, 32-47 x of channels n0 .. n0+15.  Lanes 0-15 sum B and x
        // of their channel, lanes 16-31 C (and x once more, unused); C then crosses by a shuffle.
        const int c = n0 + (lane & 15);
        const bool c_ok = c < N;
        const int k = tail.k;
        for (int m = slice + slices * warp; m < M; m += slices * WARPS) {
            float part1[8], part2[8];
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                part1[s] = s < slices ? share[s][m * ROWS + lane] : 0.f;
                part2[s] = s < slices ? share[s][m * ROWS + 32 + (lane & 15)] : 0.f;
            }
            float v1 = 0.f, v2 = 0.f;
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                v1 += part1[s];
                v2 += part2[s];
            }
            if (link.scale_part) {
                float e[4] = {0.f, 0.f, 0.f, 0.f};
                if (m == m_first) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) e[q] = early_part[q];
                } else {
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        if (lane + 32 * q < link.n_scale_part)
                            e[q] = link.scale_part[(size_t)m * link.scale_stride + lane + 32 * q];
                }
                float ss = (e[0] + e[1]) + (e[2] + e[3]);
                for (int p = lane + 128; p < link.n_scale_part; p += 32)
                    ss += link.scale_part[(size_t)m * link.scale_stride + p];
                ss = mv_warp_sum(ss);
                const float rs = 1.0f / sqrtf(ss * link.inv_dim + link.eps);
                v1 *= rs;
                v2 *= rs;
            }
            if (bias && c_ok) {
                v1 += bias[(lane < 16 ? 0 : N) + c];
                v2 += bias[2 * N + c];
            }
            const float gate_c = __shfl_down_sync(0xffffffffu, v1, 16);
            if (lane < 16 && c_ok) {
                const float bx = v1 * v2;
                float* st = tail.state + (size_t)tail.slots[m] * (k - 1) * N;
                float y = tail.conv_bias ? tail.conv_bias[c] : 0.f;
                for (int j = 0; j < k - 1; ++j) {
                    const float v = st[(size_t)j * N + c];
                    y = fmaf(tail.taps[c * k + j], v, y);
                    if (j > 0) st[(size_t)(j - 1) * N + c] = v;         // shift towards the older end
                }
                if (k > 1) st[(size_t)(k - 2) * N + c] = bx;
                y = fmaf(tail.taps[c * k + (k - 1)], bx, y);
                ((__nv_bfloat16*)out)[(size_t)m * ldo + c] = __float2bfloat16_rn(gate_c * y);
            }
        }
    } else if constexpr (HEADS) {
        const int hs = blockIdx.y;                  // head slot: nh query heads, nkv key heads, nkv value heads
        const bool is_q = hs < heads.nh, is_k = !is_q && hs < heads.nh + heads.nkv;
        // the lane's two elements: neighbours, or half a head apart (the two ways of pairing for the rotation)
        const int r0 = heads.half_split ? lane : 2 * lane, r1 = heads.half_split ? lane + 32 : 2 * lane + 1;
        const float* w = is_q ? heads.wq : (is_k ? heads.wk : nullptr);
        float w0 = 1.f, w1 = 1.f, freq = 0.f;
        if (w) {
            w0 = w[r0];
            w1 = w[r1];
        }
        const bool rotate = heads.inv_freq && (is_q || is_k);
        if (rotate) freq = heads.inv_freq[lane];
        for (int m = slice + slices * warp; m < M; m += slices * WARPS) {
            float pa[8], pb[8];
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                pa[s] = s < slices ? share[s][m * ROWS + r0] : 0.f;
                pb[s] = s < slices ? share[s][m * ROWS + r1] : 0.f;
            }
            float a = 0.f, b = 0.f;
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                a += pa[s];
                b += pb[s];
            }
            const int pos = heads.positions[m];
            if (link.scale_part) {
                float e[4] = {0.f, 0.f, 0.f, 0.f};
                if (m == m_first) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) e[q] = early_part[q];
                } else {
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        if (lane + 32 * q < link.n_scale_part)
                            e[q] = link.scale_part[(size_t)m * link.scale_stride + lane + 32 * q];
                }
                float ss = (e[0] + e[1]) + (e[2] + e[3]);
                for (int p = lane + 128; p < link.n_scale_part; p += 32)
                    ss += link.scale_part[(size_t)m * link.scale_stride + p];
                ss = mv_warp_sum(ss);
                const float rs = 1.0f / sqrtf(ss * link.inv_dim + link.eps);
                a *= rs;
                b *= rs;
            }
            if (w) {
                float ss = fmaf(a, a, b * b);
                ss = mv_warp_sum(ss);
                const float scale = 1.0f / sqrtf(ss / (float)ROWS + heads.eps);
                a = a * scale * w0;
                b = b * scale * w1;
            }
            if (rotate) {
                float sn, cs;
                sincosf((float)pos * freq, &sn, &cs);
                const float ra = a * cs - b * sn, rb = a * sn + b * cs;
                a = ra;
                b = rb;
            }
            __nv_bfloat16* dst;
            if (is_q) {
                dst = heads.q_out + ((size_t)m * heads.nh + hs) * ROWS;
            } else {
                const int page_size = 1 << heads.page_shift;
                const int page = heads.page_table[(size_t)heads.seq_of[m] * heads.table_stride + (pos >> heads.page_shift)];
                const int g2 = is_k ? hs - heads.nh : hs - heads.nh - heads.nkv;
                dst = heads.pool + (size_t)page * heads.page_stride + (size_t)(pos & (page_size - 1)) * ROWS +
                      ((size_t)(is_k ? 0 : 1) * heads.nkv + g2) * page_size * ROWS;
            }
            if (heads.half_split) {
                dst[r0] = __float2bfloat16_rn(a);
                dst[r1] = __float2bfloat16_rn(b);
            } else {
                mv_store2(dst + r0, a, b);
            }
        }
    } else
    for (int m = slice + slices * warp; m < M; m += slices * WARPS) {
        const int r = lane;                         // ROWS is 16 or 32
        const int n = n0 + r;
        float part[8];
#pragma unroll
        for (int s = 0; s < 8; ++s) part[s] = (s < slices && r < ROWS) ? share[s][m * ROWS + r] : 0.f;
        float v = 0.f;
#pragma unroll
        for (int s = 0; s < 8; ++s) v += part[s];
        if (link.scale_part) {
            float ss = 0.f;
            if (m == m_first) {
                ss = (early_part[0] + early_part[1]) + (early_part[2] + early_part[3]);
                for (int p = lane + 128; p < link.n_scale_part; p += 32)
                    ss += link.scale_part[(size_t)m * link.scale_stride + p];
            } else {
                float e[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    if (lane + 32 * k < link.n_scale_part) e[k] = link.scale_part[(size_t)m * link.scale_stride + lane + 32 * k];
                ss = (e[0] + e[1]) + (e[2] + e[3]);
                for (int p = lane + 128; p < link.n_scale_part; p += 32)
                    ss += link.scale_part[(size_t)m * link.scale_stride + p];
            }
            ss = mv_warp_sum(ss);
            v *= 1.0f / sqrtf(ss * link.inv_dim + link.eps);
        }
        if (bias && r < ROWS && n < N) v += bias[n];
        if (mode == 3) {
            // ROWS == 32: lanes 0-15 hold gate rows, lanes 16-31 the up rows of the same features
            const float up = __shfl_down_sync(0xffffffffu, v, 16);
            if (lane < 16 && n + 16 < N)
                ((__nv_bfloat16*)out)[(size_t)m * ldo + (n >> 5) * 16 + lane] =
                    __float2bfloat16_rn(v / (1.0f + expf(-v)) * up);
        } else {
            float sq = 0.f;
            if (r < ROWS && n < N) {
                const size_t o = (size_t)m * ldo + n;
                if (mode == 0) ((float*)out)[o] = v;
                else if (mode == 1) ((__nv_bfloat16*)out)[o] = __float2bfloat16_rn(v);
                else {
                    const float x_new = (m == m_first ? early_old : ((float*)out)[o]) + v;
                    ((float*)out)[o] = x_new;
                    if (link.emit_x) {
                        link.emit_x[(size_t)m * N + n] = __float2bfloat16_rn(x_new * early_g);
                        sq = x_new * x_new;
                    }
                }
            }
            if (mode == 2 && link.emit_x) {
                sq = mv_warp_sum(sq);
                if (lane == 0) link.emit_part[(size_t)m * link.emit_stride + blockIdx.y] = sq;
            }
        }
    }
    // nobody leaves while another block may still read its shared memory
    if (slices > 1) mv_cluster_sync_relaxed();
}

template <int NT, int RT, int UNROLL, int WARPS, int TAIL = 0>
int launch(const void* W, const void* X, const float* bias, void* out, int mode, int M, int N, int K, int ldo,
           const NormLink& link, const ConvTail& tail, const HeadTail& heads, const Ahead& ahead, cudaStream_t stream) {
    constexpr bool CONV = TAIL == 1;
    constexpr int ROWS = RT * 16, LDR = NT * 8 + 1;
    const int ksteps = (K + 31) / 32;
    const int tiles = CONV ? (N + 15) / 16 : (N + ROWS - 1) / ROWS;
    // slices of K: every warp should still have UNROLL k-steps, and there is no point in many
    // more blocks than the GPU holds at once (about 8 per SM)
    int slices = ksteps / (WARPS * UNROLL);
    slices = slices < 1 ? 1 : (slices > 8 ? 8 : slices);
    // (the convolution kernel holds three row tiles a warp: its registers leave room for 5 blocks;
    // with more blocks than fit at once it measured 12.8 us on [3 x 2048, 2048] against 8.9 us)
    while (slices > 1 && (long long)tiles * slices > 148 * (TAIL == 1 ? 5 : TAIL == 2 ? 4 : 8)) slices >>= 1;
    const size_t smem = (size_t)(WARPS + 1) * ROWS * LDR * sizeof(float);
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(gemm_small_m_kernel<NT, RT, UNROLL, WARPS, TAIL>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             160 * 1024);
        attr_set = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(slices, tiles);
    cfg.blockDim = dim3(WARPS * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (mv_pdl_small_m_enabled()) {
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
    cudaLaunchKernelEx(&cfg, gemm_small_m_kernel<NT, RT, UNROLL, WARPS, TAIL>, (const __nv_bfloat16*)W,
                       (const __nv_bfloat16*)X, bias, out, mode, M, N, K, ldo, link, tail, heads, ahead);
    return mv_launch_status();
}

}  // namespace

// Rows of W per block for this shape: 32 halve the re-reads of X and are what the SwiGLU
// epilogue needs; 16 keep more blocks for a narrow matrix.  (Also the rows behind one tile sum.)
MV_API int mv_gemm_small_m_tile_rows(int N, int mode) { return (N >= 32 * 2 * 148 || mode == 3) ? 32 : 16; }

// mode: 0 store float32, 1 store bfloat16, 2 add into float32, 3 SwiGLU (W rows in
// groups of 16 gate + 16 up; out is bfloat16 [M, N/2] with row stride ldo).  Needs
// 1 <= M <= 64, K a multiple of 8, and 16-byte aligned operands.
// scale_part (or null): [M][scale_stride] of which n_scale_part sums of squares per token; every token's
// results are multiplied by rsqrt(sum / dim + eps) before bias and activation.  emit_x (or null, mode 2
// only, ldo == N): receives bf16(out_new * emit_g), and emit_part [M][emit_stride] the sums of out_new^2
// per tile of mv_gemm_small_m_tile_rows(N, 2) rows.  next_w (or null), next_bytes: memory that the
// step's next product will read, to be requested into L2 meanwhile.
MV_API int mv_gemm_small_m(const void* X, const void* W, const float* bias, void* out, int mode, int M,
                           int N, int K, int ldo, const float* scale_part, int n_scale_part, int scale_stride,
                           int dim, float eps, const float* emit_g, void* emit_x, float* emit_part,
                           int emit_stride, const void* next_w, long long next_bytes, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 64 || K % 8 || ((uintptr_t)X & 15) || ((uintptr_t)W & 15)) return (int)cudaErrorInvalidValue;
    if (mode == 3 && N % 32) return (int)cudaErrorInvalidValue;
    if (emit_x && (mode != 2 || ldo != N || !emit_g || !emit_part ||
                   emit_stride < (N + mv_gemm_small_m_tile_rows(N, 2) - 1) / mv_gemm_small_m_tile_rows(N, 2)))
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
    const int nt = (M + 7) / 8;
    const bool wide = mv_gemm_small_m_tile_rows(N, mode) == 32;
#define MV_GO(NT, RT, U, WARPS) return launch<NT, RT, U, WARPS>(W, X, bias, out, mode, M, N, K, ldo, link, ConvTail{}, HeadTail{}, Ahead{next_w, next_bytes}, stream)
    // few tokens: small blocks, many per SM; many tokens: large blocks, so that X is re-read less
    switch (nt) {
        case 1: if (wide) MV_GO(1, 2, 2, 4); else MV_GO(1, 1, 4, 4);
        case 2: if (wide) MV_GO(2, 2, 2, 4); else MV_GO(2, 1, 4, 4);
        case 3: case 4: if (wide) MV_GO(4, 2, 2, 8); else MV_GO(4, 1, 4, 8);
        default: if (wide) MV_GO(8, 2, 2, 16); else MV_GO(8, 1, 4, 16);
    }
#undef MV_GO
}

// The input projection of a gated short convolution and the convolution's decode step in one kernel,
// for steps in which each of M <= 8 sequences brings one token: W [3 H, K] (rows of B, then C, then x),
// bias [3 H] or null, taps [H][k], conv_bias [H] or null, state [slots][k - 1][H] (read, shifted and
// written for the M sequences in slots[0..M)), z bfloat16 [M, H] = C * conv(B * x).  scale_part as in
// mv_gemm_small_m.  Needs K a multiple of 8 and 16-byte aligned X and W.
MV_API int mv_gemm_small_m_shortconv(const void* X, const void* W, const float* bias, const float* taps,
                                     const float* conv_bias, float* state, const int* slots, void* z, int M,
                                     int H, int K, int k, const float* scale_part, int n_scale_part,
                                     int scale_stride, int dim, float eps, const void* next_w,
                                     long long next_bytes, cudaStream_t stream) {
    if (M <= 0 || H <= 0) return 0;
    if (M > 8 || K % 8 || ((uintptr_t)X & 15) || ((uintptr_t)W & 15) || k < 1 || !taps || !slots || (k > 1 && !state))
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
    ConvTail tail = {taps, conv_bias, state, slots, k};
    return launch<1, 3, 2, 4, 1>(W, X, bias, z, 1, M, H, K, H, link, tail, HeadTail{}, Ahead{next_w, next_bytes}, stream);
}

// The fused q/k/v projection of an attention layer and the preparation of its heads in one kernel, for
// steps of M <= 8 tokens and heads of 64: W [(nh + 2 nkv) 64, K]; wq, wk [64] or null (no norm);
// inv_freq [32] or null (no rotation); half_split: pairs (i, i + 32) instead of (2i, 2i + 1); the
// token's position and page-table row; pool bfloat16 [pages][2][nkv][page_size][64] with page_stride
// elements a page; q_out bfloat16 [M, nh 64].  scale_part and next_w as in mv_gemm_small_m.
MV_API int mv_gemm_small_m_heads(const void* X, const void* W, const float* wq, const float* wk, float eps,
                                 const float* inv_freq, int half_split, const int* positions, const int* seq_of,
                                 const int* page_table, int table_stride, int page_size, void* pool,
                                 long long page_stride, void* q_out, int M, int nh, int nkv, int K,
                                 const float* scale_part, int n_scale_part, int scale_stride, int dim, float eps_norm,
                                 const void* next_w, long long next_bytes, cudaStream_t stream) {
    if (M <= 0 || nh <= 0) return 0;
    if (M > 8 || K % 8 || ((uintptr_t)X & 15) || ((uintptr_t)W & 15) || nkv < 0 || !positions || !q_out ||
        (nkv > 0 && (!seq_of || !page_table || !pool || page_size <= 0 || (page_size & (page_size - 1)))))
        return (int)cudaErrorInvalidValue;
    if (scale_part && (n_scale_part <= 0 || n_scale_part > scale_stride || dim <= 0)) return (int)cudaErrorInvalidValue;
    NormLink link = {};
    if (scale_part) {
        link.scale_part = scale_part;
        link.n_scale_part = n_scale_part;
        link.scale_stride = scale_stride;
        link.inv_dim = 1.0f / (float)dim;
        link.eps = eps_norm;
    }
    HeadTail heads = {};
    heads.wq = wq;
    heads.wk = wk;
    heads.inv_freq = inv_freq;
    heads.positions = positions;
    heads.seq_of = seq_of;
    heads.page_table = page_table;
    heads.pool = (__nv_bfloat16*)pool;
    heads.q_out = (__nv_bfloat16*)q_out;
    heads.page_stride = page_stride;
    heads.eps = eps;
    heads.half_split = half_split;
    heads.table_stride = table_stride;
    while ((1 << heads.page_shift) < page_size) ++heads.page_shift;
    heads.nh = nh;
    heads.nkv = nkv;
    const int N = (nh + 2 * nkv) * 64;
    return launch<1, 4, 2, 4, 2>(W, X, nullptr, q_out, 1, M, N, K, N, link, ConvTail{}, heads,
                                 Ahead{next_w, next_bytes}, stream);
}
