// Sampling of one token for each row of logits, on the device, in the order of
// the reference's sampler (crates/mivi-model/src/sampler.rs:92-136):
// penalties over the recent tokens (222-260), greedy if temperature <= 0 (the
// first maximum wins, 305-315), temperature (282-287), min-p (263-279), top-k
// keeping ties at the k-th value (290-302), softmax, then the nucleus
// (150-218) or the plain categorical draw (138-148).
//
// One block of 1024 threads per row; the row is copied to scratch first, so the
// caller's logits stay as they are.  Thread t owns the run of indices
// [t * seg, (t + 1) * seg), seg = ceil(V / 1024): running sums in index order are
// then prefix sums in thread order.  In the scratch the k-th element of thread t
// lies at k * 1024 + t, so that every pass reads it coalesced (laid out by index,
// a thread's run would be 256 bytes away from its neighbour's).  The scratch of a
// row holds seg * 1024 values; the places past V hold -infinity.
//
// Two things are this library's own.  (1) The uniform number: the reference
// keeps one xorshift64* state for its single sequence (sampler.rs:70-76); a
// batch needs draws that do not depend on what else is in the batch, so the
// draw of a sequence at a decoding step is a splitmix64 hash of
// (seed, stream, step), top 24 bits as in the reference.  (2) Probability mass
// is summed as 40-bit fixed point in 64-bit integers: integer sums do not
// depend on the order of the additions, so the result is the same in every
// run and for every thread layout.  The nucleus is the shortest prefix in
// descending probability (ties: lower index first) whose mass reaches top_p;
// the draw walks the kept tokens in index order.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace {

constexpr int THREADS = 1024;
constexpr int RECENT_MAX = 64;
constexpr int RING = 128;              // places of a device-side ring of recent tokens: twice the window

__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__device__ __forceinline__ unsigned draw24(unsigned long long seed, unsigned long long stream,
                                           unsigned long long step) {
    unsigned long long z = mix64(seed);
    z = mix64(z ^ (stream * 0xD1342543DE82EF95ull));
    z = mix64(z ^ (step * 0xA24BAED4963EE407ull));
    return (unsigned)(z >> 40);
}
// floats -> unsigned keys with the same order
__device__ __forceinline__ unsigned order_key(float x) {
    const unsigned u = __float_as_uint(x);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ unsigned long long fixed40(float e) {
    return (unsigned long long)(e * 1099511627776.0f);       // e in [0, 1]
}

struct Shared {
    unsigned cnt[256];
    unsigned long long mass[256];
    float fred[33];
    int ired[33];
    unsigned long long wsum[33];
    unsigned sel_prefix;
    unsigned sel_remaining;
    unsigned long long sel_mass_above;
    int result;
    float cval[1024];                  // what top-k left, in index order, when it fits: values ...
    int cidx[1024];                    // ... and their indices
};

__device__ float block_max(float v, Shared& sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = mv_warp_max(v);
    __syncthreads();
    if (lane == 0) sh.fred[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = sh.fred[lane];
        t = mv_warp_max(t);
        if (lane == 0) sh.fred[32] = t;
    }
    __syncthreads();
    return sh.fred[32];
}

// exclusive prefix sum over the block in thread order; *total gets the sum
__device__ unsigned long long block_excl_scan(unsigned long long v, Shared& sh, unsigned long long* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned long long inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    __syncthreads();
    if (lane == 31) sh.wsum[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        unsigned long long w = sh.wsum[lane];
        unsigned long long winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned long long t = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += t;
        }
        sh.wsum[lane] = winc - w;
        if (lane == 31) sh.wsum[32] = winc;
    }
    __syncthreads();
    *total = sh.wsum[32];
    return sh.wsum[warp] + inc - v;
}

// Walking 256 radix bins from the top by ONE WARP (every lane calls these, lane l holds bins 8l ... 8l+7)
// instead of one thread: the sums of the bins above a lane come from a shuffle scan, each lane walks its own
// eight bins with them, and the highest lane that finds the bin wins - the bin a single thread would find.
//
// select_count: the highest bin b >= 1 with cnt[b] >= rem - (sum of the bins above b); bin 0 if there is none.
// rem_out: rem less the sum of the bins above the chosen one.
__device__ __forceinline__ void select_count(const unsigned* cnt, unsigned rem, unsigned& bin_out, unsigned& rem_out) {
    const int lane = threadIdx.x & 31;
    unsigned c[8], s = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) { c[i] = cnt[8 * lane + i]; s += c[i]; }
    unsigned t = s;                                       // sum over this lane and the lanes above it
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned u = __shfl_down_sync(0xffffffffu, t, o);
        if (lane + o < 32) t += u;
    }
    unsigned above = t - s;
    int found = -1;
    unsigned left = 0;
#pragma unroll
    for (int i = 7; i >= 0; --i) {
        const int b = 8 * lane + i;
        if (found < 0 && b > 0 && above < rem) {
            if (c[i] >= rem - above) { found = b; left = rem - above; }
            else above += c[i];
        }
    }
    const unsigned hits = __ballot_sync(0xffffffffu, found >= 0);
    if (hits) {
        const int src = 31 - __clz(hits);
        bin_out = (unsigned)__shfl_sync(0xffffffffu, found, src);
        rem_out = __shfl_sync(0xffffffffu, left, src);
    } else {
        const unsigned all = __shfl_sync(0xffffffffu, t, 0), c0 = __shfl_sync(0xffffffffu, c[0], 0);
        bin_out = 0;
        rem_out = rem - (all - c0);
    }
}
// select_mass: the highest bin b >= 1 that holds something (cnt[b] > 0) and whose mass brings the mass above
// it (above0 plus the bins above b) to the target; bin 0 if there is none.  above_out: the mass above it.
__device__ __forceinline__ void select_mass(const unsigned* cnt, const unsigned long long* mass,
                                            unsigned long long above0, unsigned long long target, unsigned& bin_out,
                                            unsigned long long& above_out) {
    const int lane = threadIdx.x & 31;
    unsigned long long m[8], s = 0;
    unsigned c[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { c[i] = cnt[8 * lane + i]; m[i] = mass[8 * lane + i]; s += m[i]; }
    unsigned long long t = s;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long u = __shfl_down_sync(0xffffffffu, t, o);
        if (lane + o < 32) t += u;
    }
    unsigned long long above = above0 + (t - s);
    int found = -1;
    unsigned long long at = 0;
#pragma unroll
    for (int i = 7; i >= 0; --i) {
        const int b = 8 * lane + i;
        if (found < 0 && b > 0) {
            if (c[i] && above + m[i] >= target) { found = b; at = above; }
            else above += m[i];
        }
    }
    const unsigned hits = __ballot_sync(0xffffffffu, found >= 0);
    if (hits) {
        const int src = 31 - __clz(hits);
        bin_out = (unsigned)__shfl_sync(0xffffffffu, found, src);
        above_out = __shfl_sync(0xffffffffu, at, src);
    } else {
        const unsigned long long all = __shfl_sync(0xffffffffu, t, 0), m0 = __shfl_sync(0xffffffffu, m[0], 0);
        bin_out = 0;
        above_out = above0 + (all - m0);
    }
}

// *p += x on a 64-bit word of shared memory by two native 32-bit atomics (the 64-bit one is a compare-and-swap
// loop): the add that wraps the low word carries into the high word.  Exact once all adds have been made.
__device__ __forceinline__ void add64(unsigned long long* p, unsigned long long x) {
    unsigned* w = reinterpret_cast<unsigned*>(p);
    const unsigned xl = (unsigned)x, xh = (unsigned)(x >> 32);
    const unsigned old = atomicAdd(w, xl);
    const unsigned up = xh + ((old + xl < old) ? 1u : 0u);
    if (up) atomicAdd(w + 1, up);
}
// mass[bin] += q and cnt[bin] += 1 where ``on``
__device__ __forceinline__ void hist_add(unsigned long long* mass, unsigned* cnt, bool on, unsigned bin,
                                         unsigned long long q) {
    if (on) {
        add64(&mass[bin], q);
        atomicAdd(&cnt[bin], 1u);
    }
}

// The largest value of the block and, among equal ones, its smallest index, to *dst.
__device__ __forceinline__ void block_argmax_first(float best, int besti, Shared& sh, int* dst) {
    const int tid = threadIdx.x;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
        if (ov > best || (ov == best && oi < besti)) { best = ov; besti = oi; }
    }
    if ((tid & 31) == 0) { sh.fred[tid >> 5] = best; sh.ired[tid >> 5] = besti; }
    __syncthreads();
    if (tid < 32) {
        best = sh.fred[tid]; besti = sh.ired[tid];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
            if (ov > best || (ov == best && oi < besti)) { best = ov; besti = oi; }
        }
        if (tid == 0) *dst = besti == 0x7fffffff ? 0 : besti;
    }
}

// The end of a row's sampling, from values that temperature, min-p and top-k have been through: softmax
// masses, nucleus, draw.  Thread t owns the run xr[k * THREADS], k < seg, of indices t * seg + k - or, with
// ``compact``, the one element sh.cval[t] of the list of what top-k left, whose index is sh.cidx[t].
__device__ void sample_tail(Shared& sh, float* xr, int seg, bool compact, float mx, float top_p,
                            unsigned long long seed, unsigned long long stream_id, int my_step,
                            const float* __restrict__ src, float inv_t, int V, int* out_b, int* my_ring) {
    const int tid = threadIdx.x;
    // 6. softmax masses in fixed point; each thread owns a run of indices (or one element of the list)
    unsigned long long mine = 0;
    for (int k = 0; k < seg; ++k) {
        const float v = xr[(size_t)k * THREADS];
        const float e = v == -INFINITY ? 0.f : expf(v - mx);
        xr[(size_t)k * THREADS] = e;
        mine += fixed40(e);
    }
    unsigned long long total;
    block_excl_scan(mine, sh, &total);

    // 7. nucleus: the value at which the descending mass reaches top_p
    float cut_e = 0.f;                    // keep e > cut_e, and the first n_take of e == cut_e
    unsigned long long n_take = ~0ull;
    unsigned long long kept = total;
    if (top_p < 1.0f) {
        const unsigned long long target = (unsigned long long)((double)top_p * (double)total);
        if (tid == 0) { sh.sel_prefix = 0; sh.sel_mass_above = 0; }
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            if (tid < 256) { sh.mass[tid] = 0; sh.cnt[tid] = 0; }
            __syncthreads();
            const unsigned prefix = sh.sel_prefix;
            const unsigned himask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
            for (int k = 0; k < seg; ++k) {
                const float e = xr[(size_t)k * THREADS];
                const unsigned key = __float_as_uint(e);          // e >= 0: bit order is value order
                hist_add(sh.mass, sh.cnt, e > 0.f && (key & himask) == prefix, (key >> shift) & 255u, fixed40(e));
            }
            __syncthreads();
            if (tid < 32) {
                unsigned bin;
                unsigned long long above;
                select_mass(sh.cnt, sh.mass, sh.sel_mass_above, target, bin, above);
                __syncwarp();
                if (tid == 0) {
                    sh.sel_prefix = prefix | (bin << shift);
                    sh.sel_mass_above = above;
                }
            }
            __syncthreads();
        }
        cut_e = __uint_as_float(sh.sel_prefix);
        const unsigned long long above = sh.sel_mass_above;
        const unsigned long long qc = fixed40(cut_e);
        if (qc == 0 || cut_e <= 0.f) {
            n_take = ~0ull;               // nothing left to cut: keep all
            cut_e = 0.f;
        } else {
            const unsigned long long need = target > above ? target - above : 1;
            n_take = (need + qc - 1) / qc;
            if (n_take == 0) n_take = 1;
        }
        // rank of this thread's first tie, in index order
        unsigned long long ties = 0;
        for (int k = 0; k < seg; ++k) ties += (xr[(size_t)k * THREADS] == cut_e && cut_e > 0.f) ? 1 : 0;
        unsigned long long tie_total;
        unsigned long long tie_rank = block_excl_scan(ties, sh, &tie_total);
        mine = 0;
        for (int k = 0; k < seg; ++k) {
            const float e = xr[(size_t)k * THREADS];
            bool keep = e > cut_e;
            if (e == cut_e && cut_e > 0.f) { keep = tie_rank < n_take; ++tie_rank; }
            if (!keep) xr[(size_t)k * THREADS] = 0.f;
            else mine += fixed40(e);
        }
        block_excl_scan(mine, sh, &kept);
    }

    // 8. the draw: first kept index whose running mass exceeds u * kept
    const unsigned k24 = draw24(seed, stream_id, (unsigned long long)my_step);
    const unsigned long long lo = kept * (unsigned long long)k24;
    const unsigned long long hi = __umul64hi(kept, (unsigned long long)k24);
    const unsigned long long r = (hi << 40) | (lo >> 24);
    unsigned long long dummy;
    const unsigned long long before = block_excl_scan(mine, sh, &dummy);
    if (tid == 0) sh.result = -1;
    __syncthreads();
    if (mine > 0 && before <= r && r < before + mine) {
        unsigned long long c = before;
        for (int k = 0; k < seg; ++k) {
            const unsigned long long qv = fixed40(xr[(size_t)k * THREADS]);
            if (qv == 0) continue;
            c += qv;
            if (r < c) { sh.result = compact ? sh.cidx[tid] : tid * seg + k; break; }
        }
    }
    __syncthreads();
    if (tid == 0) {
        int res = sh.result;
        if (res < 0) {                    // all mass below the fixed-point resolution: fall back to the maximum
            res = 0;
            for (int i = 0; i < V; ++i)
                if (src[i] * inv_t == mx) { res = i; break; }
        }
        *out_b = res;
        if (my_ring) my_ring[my_step & (RING - 1)] = res;
    }
}

// One row, by one block of 1024 threads: see the head of the file.  ``tiles``: 32 x 33 floats a warp.
__device__ void sample_row(const float* __restrict__ logits, long long ld, float* __restrict__ work, int V,
                           float temperature, int top_k, float top_p, float min_p, float rep_pen, float pres_pen,
                           float freq_pen, const int* __restrict__ recent, const int* __restrict__ n_recent,
                           unsigned long long seed, const int* __restrict__ streams, const int* __restrict__ steps,
                           int* __restrict__ ring, const int* __restrict__ ring_row, int* __restrict__ out, int b,
                           Shared& sh, float* tiles) {

    const int tid = threadIdx.x;
    const float* src = logits + (size_t)b * ld;
    int seg = (V + THREADS - 1) / THREADS;
    const int VP = seg * THREADS;
    bool compact = false;
    float* x = work + (size_t)b * VP;                  // element i at x[(i % seg) * THREADS + i / seg]

    // The recent tokens of a row come from the caller (recent, n_recent) or from a ring that this kernel
    // keeps itself on the device: ring [states, 128], state ring_row[b], the token sampled at step s at place
    // s mod 128.  Step s looks at the places of steps s-1 ... s-64; its own place lies outside them, so a
    // step that runs twice sees the same tokens and writes the same place both times.
    int* my_ring = ring ? ring + (size_t)ring_row[b] * RING : nullptr;
    const int my_step = steps ? steps[b] : 0;
    const int nr = my_ring ? min(my_step, RECENT_MAX) : (n_recent ? min(n_recent[b], RECENT_MAX) : 0);
    const bool pen = nr > 0 && ((rep_pen > 0.f && rep_pen != 1.f) || pres_pen != 0.f || freq_pen != 0.f);

    // 0. greedy without penalties: the first maximum of the logits as they are, read once, four at a time
    if (temperature <= 0.f && !pen) {
        float best = -INFINITY;
        int besti = 0x7fffffff;
        const bool vec = (((uintptr_t)src) & 15) == 0;
        const int V4 = vec ? V >> 2 : 0;
        for (int i = tid; i < V4; i += THREADS) {
            const float4 v = reinterpret_cast<const float4*>(src)[i];
            // within a thread the indices go up, so ">" keeps the first of equal values
            if (v.x > best) { best = v.x; besti = 4 * i; }
            if (v.y > best) { best = v.y; besti = 4 * i + 1; }
            if (v.z > best) { best = v.z; besti = 4 * i + 2; }
            if (v.w > best) { best = v.w; besti = 4 * i + 3; }
        }
        for (int i = 4 * V4 + tid; i < V; i += THREADS) {
            const float v = src[i];
            if (v > best) { best = v; besti = i; }
        }
        block_argmax_first(best, besti, sh, out + b);
        if (my_ring && tid == 0) my_ring[my_step & (RING - 1)] = out[b];
        return;
    }

    // The copy, read by index and written to its place, both coalesced: a warp moves tiles of 32 threads'
    // runs x 32 elements through a 32 x 33 tile of its own in shared memory.
    {
        const int warp = tid >> 5, lane = tid & 31;
        float* tile = tiles + warp * (32 * 33);
        const int t0 = warp * 32;                       // the warp's threads: t0 .. t0 + 31
        for (int k0 = 0; k0 < seg; k0 += 32) {
            // row a of the tile: the 32 elements k0 .. k0+31 of thread t0 + a's run, consecutive indices
#pragma unroll 4
            for (int a = 0; a < 32; ++a) {
                const int k = k0 + lane, i = (t0 + a) * seg + k;
                tile[a * 33 + lane] = (k < seg && i < V) ? src[i] : -INFINITY;
            }
            __syncwarp();
            // column b of the tile goes to place (k0 + b) * THREADS + t0 .. t0+31: consecutive places
#pragma unroll 4
            for (int bcol = 0; bcol < 32; ++bcol)
                if (k0 + bcol < seg) x[(size_t)(k0 + bcol) * THREADS + t0 + lane] = tile[lane * 33 + bcol];
            __syncwarp();
        }
    }
    __syncthreads();

    // 1. penalties, once per distinct recent token
    if (pen && tid < nr) {
        // recent token j (0 <= j < nr)
        auto rc_at = [&](int j) {
            return my_ring ? my_ring[(my_step - 1 - j) & (RING - 1)] : recent[(size_t)b * RECENT_MAX + j];
        };
        const int tok = rc_at(tid);
        bool first = tok >= 0 && tok < V;
        int count = 0;
        for (int j = 0; j < nr; ++j) {
            if (rc_at(j) == tok) {
                if (j < tid) first = false;
                ++count;
            }
        }
        if (first) {
            float& xt = x[(size_t)(tok % seg) * THREADS + tok / seg];
            float v = xt;
            if (rep_pen > 0.f && rep_pen != 1.f) v = v > 0.f ? v / rep_pen : v * rep_pen;
            if (pres_pen != 0.f) v -= pres_pen;
            if (freq_pen != 0.f) v -= freq_pen * (float)count;
            xt = v;
        }
    }
    __syncthreads();

    // 2. greedy: the first maximum wins
    if (temperature <= 0.f) {
        float best = -INFINITY;
        int besti = 0x7fffffff;
        for (int k = 0; k < seg; ++k) {
            const float v = x[(size_t)k * THREADS + tid];
            if (v > best) { best = v; besti = tid * seg + k; }
        }
        block_argmax_first(best, besti, sh, out + b);
        if (my_ring && tid == 0) my_ring[my_step & (RING - 1)] = out[b];      // thread 0 wrote out[b] itself
        return;
    }

    // 3. temperature, maximum
    const float inv_t = 1.0f / temperature;
    float mx = -INFINITY;
    for (int i = tid; i < VP; i += THREADS) {          // these passes do not care which index a place holds
        const float v = x[i] * inv_t;
        x[i] = v;
        mx = fmaxf(mx, v);
    }
    mx = block_max(mx, sh);

    // 4. min-p
    if (min_p > 0.f && min_p < 1.f) {
        const float thr = mx + logf(min_p);
        for (int i = tid; i < VP; i += THREADS)
            if (x[i] < thr) x[i] = -INFINITY;
        __syncthreads();
    }

    // 5. top-k: radix select of the k-th largest value, ties at it are kept
    if (top_k > 0 && top_k < V) {
        if (tid == 0) { sh.sel_prefix = 0; sh.sel_remaining = (unsigned)top_k; }
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            if (tid < 256) sh.cnt[tid] = 0;
            __syncthreads();
            const unsigned prefix = sh.sel_prefix;
            const unsigned himask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
            for (int i = tid; i < VP; i += THREADS) {
                const unsigned key = order_key(x[i]);
                if ((key & himask) == prefix) atomicAdd(&sh.cnt[(key >> shift) & 255u], 1u);
            }
            __syncthreads();
            if (tid < 32) {
                unsigned bin, rem;
                select_count(sh.cnt, sh.sel_remaining, bin, rem);
                __syncwarp();
                if (tid == 0) {
                    sh.sel_prefix = prefix | (bin << shift);
                    sh.sel_remaining = rem;
                }
            }
            __syncthreads();
        }
        const unsigned cut = sh.sel_prefix;
        // What is left (top_k values and their ties) usually fits one element a thread: each thread counts
        // the survivors of its run, a prefix sum gives their places in index order, and the rest of the
        // kernel walks a list of at most 1,024 elements in shared memory instead of the whole row.
        unsigned long long keepers = 0;
        for (int k = 0; k < seg; ++k) {
            float& v = x[(size_t)k * THREADS + tid];
            if (order_key(v) < cut) v = -INFINITY;
            else if (v != -INFINITY) ++keepers;
        }
        unsigned long long n_left;
        unsigned long long at = block_excl_scan(keepers, sh, &n_left);
        if (n_left <= THREADS) {
            sh.cval[tid] = -INFINITY;
            sh.cidx[tid] = 0;
            __syncthreads();
            for (int k = 0; k < seg && keepers; ++k) {
                const float v = x[(size_t)k * THREADS + tid];
                if (v != -INFINITY) {
                    sh.cval[at] = v;
                    sh.cidx[at] = tid * seg + k;
                    ++at;
                }
            }
            compact = true;
        }
        __syncthreads();
    }

    sample_tail(sh, compact ? sh.cval + tid : x + tid, compact ? 1 : seg, compact, mx, top_p, seed,
                (unsigned long long)(streams ? streams[b] : b), my_step, src, inv_t, V, out + b, my_ring);
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, long long ld, float* __restrict__ work, int V,
              float temperature, int top_k, float top_p, float min_p, float rep_pen, float pres_pen,
              float freq_pen, const int* __restrict__ recent, const int* __restrict__ n_recent,
              unsigned long long seed, const int* __restrict__ streams, const int* __restrict__ steps,
              int* __restrict__ ring, const int* __restrict__ ring_row, int* __restrict__ out,
              const int* __restrict__ flag_src, int* __restrict__ flag_dst) {
    mv_pdl_begin();
    // a word that travels with the tokens: the device's error flag as the step before this kernel left it
    if (flag_dst && blockIdx.x == 0 && threadIdx.x == 0) *flag_dst = *flag_src;
    __shared__ Shared sh;
    extern __shared__ float tiles[];
    sample_row(logits, ld, work, V, temperature, top_k, top_p, min_p, rep_pen, pres_pen, freq_pen, recent, n_recent,
               seed, streams, steps, ring, ring_row, out, (int)blockIdx.x, sh, tiles);
}


// ---------------------------------------------------------------------------
// The same for the usual case of a small top_k (1 ... 1024), by a CLUSTER of 8 blocks a row: the row's
// values are spread over the registers of 8,192 threads (8 each at a vocabulary of 65,536), so penalties,
// temperature, min-p and the four passes of the top-k radix select touch no memory at all; the blocks
// exchange a maximum, four histograms and their survivor counts through distributed shared memory.  What
// top-k leaves is gathered, in index order, into the first block's list, and that block runs sample_tail.
// Every block takes the same decisions from the same sums, so there is one cluster barrier a step.  If more
// than 1,024 values survive (a wall of ties at the k-th value) the first block does the whole row the slow way.
// Without top_k the row stays in the registers to the end (cluster_tail): masses, the nucleus' four passes
// and the draw exchange a block's sums and histograms the same way.
// ---------------------------------------------------------------------------
constexpr int CL_MAX = 8;             // blocks a row: 8, or 4 when more rows come than the GPU holds clusters of 8 at once
constexpr int VPT_MAX = 16;            // values a thread: vocabularies up to 8 * 1024 * 16

struct ClusterShared {
    unsigned cnt[2][256];              // this block's radix histogram; two buffers, used in turn
    unsigned tot[256];                 // the cluster's histogram, which every block sums for itself
    float bmax;                        // this block's maximum
    unsigned keep;                     // how many of this block's values top-k left
    unsigned sel_prefix, sel_remaining;
    // without top-k (cluster_tail)
    unsigned long long mass[2][256];   // this block's histogram of masses, as cnt
    unsigned long long mtot[256];      // the cluster's
    unsigned long long xch[3];         // this block's sums, one place for each exchange
    unsigned long long sel_above;
    int result;                        // the first block's: the drawn index, written by the block that finds it
    int rec[RECENT_MAX];               // the recent tokens, newest first
    int pen_tok[RECENT_MAX];           // each distinct one at its first place (-1 elsewhere) ...
    int pen_cnt[RECENT_MAX];           // ... and how often it occurs
};

// A sum over the cluster of one value a block (thread 0 of each block passes it on): the total, and in
// ``below`` the sum of the blocks before this one.  Each call has a place of its own, so none waits for the last.
template <int CL>
__device__ __forceinline__ unsigned long long cluster_sum(cg::cluster_group& cluster, ClusterShared& cs, int place,
                                                          unsigned long long mine, int rank,
                                                          unsigned long long& below) {
    if (threadIdx.x == 0) cs.xch[place] = mine;
    cluster.sync();
    unsigned long long total = 0;
    below = 0;
#pragma unroll
    for (int rr = 0; rr < CL; ++rr) {
        const unsigned long long c = *cluster.map_shared_rank(&cs.xch[place], rr);
        if (rr < rank) below += c;
        total += c;
    }
    return total;
}

// sample_tail for a row that lies in the registers of the cluster (no top-k): v holds this thread's values
// after temperature and min-p, indices i0 ... i0 + vpt - 1, in the order (block, thread, k).  The same sums
// in the same fixed point as sample_tail, so the same token.
template <int CL>
__device__ __forceinline__ void cluster_tail(cg::cluster_group& cluster, Shared& sh, ClusterShared& cs,
                                             float (&v)[VPT_MAX], int vpt, int i0, int rank, float mx, float top_p,
                                             unsigned long long seed, unsigned long long stream_id, int my_step,
                                             const float* __restrict__ src, float inv_t, int V, int* out_b,
                                             int* my_ring) {
    const int tid = threadIdx.x;
    unsigned long long mine = 0;
#pragma unroll
    for (int k = 0; k < VPT_MAX; ++k) {
        const float e = v[k] == -INFINITY ? 0.f : expf(v[k] - mx);
        v[k] = e;
        mine += fixed40(e);
    }
    if (rank == 0 && tid == 0) cs.result = -1;
    unsigned long long in_block, below;
    unsigned long long at = block_excl_scan(mine, sh, &in_block);
    const unsigned long long total = cluster_sum<CL>(cluster, cs, 0, in_block, rank, below);
    unsigned long long kept = total;

    if (top_p < 1.0f) {
        const unsigned long long target = (unsigned long long)((double)top_p * (double)total);
        unsigned prefix = 0;
        unsigned long long above = 0;
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass, buf = pass & 1;
            if (tid < 256) { cs.mass[buf][tid] = 0; cs.cnt[buf][tid] = 0; }
            __syncthreads();
            const unsigned himask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
#pragma unroll
            for (int k = 0; k < VPT_MAX; ++k) {
                if (k < vpt) {
                    const unsigned key = __float_as_uint(v[k]);
                    hist_add(cs.mass[buf], cs.cnt[buf], v[k] > 0.f && (key & himask) == prefix, (key >> shift) & 255u,
                             fixed40(v[k]));
                }
            }
            cluster.sync();
            if (tid < 256) {
                unsigned c = 0;
                unsigned long long m = 0;
#pragma unroll
                for (int rr = 0; rr < CL; ++rr) {
                    c += *cluster.map_shared_rank(&cs.cnt[buf][tid], rr);
                    m += *cluster.map_shared_rank(&cs.mass[buf][tid], rr);
                }
                cs.tot[tid] = c;
                cs.mtot[tid] = m;
            }
            __syncthreads();
            if (tid < 32) {
                unsigned bin;
                unsigned long long ab;
                select_mass(cs.tot, cs.mtot, above, target, bin, ab);
                if (tid == 0) {
                    cs.sel_prefix = prefix | (bin << shift);
                    cs.sel_above = ab;
                }
            }
            __syncthreads();
            prefix = cs.sel_prefix;
            above = cs.sel_above;
        }
        float cut_e = __uint_as_float(prefix);
        unsigned long long n_take;
        const unsigned long long qc = fixed40(cut_e);
        if (qc == 0 || cut_e <= 0.f) {
            n_take = ~0ull;
            cut_e = 0.f;
        } else {
            const unsigned long long need = target > above ? target - above : 1;
            n_take = (need + qc - 1) / qc;
            if (n_take == 0) n_take = 1;
        }
        unsigned long long ties = 0;
#pragma unroll
        for (int k = 0; k < VPT_MAX; ++k) ties += (v[k] == cut_e && cut_e > 0.f) ? 1 : 0;
        unsigned long long ties_block, ties_below;
        unsigned long long tie_rank = block_excl_scan(ties, sh, &ties_block);
        cluster_sum<CL>(cluster, cs, 1, ties_block, rank, ties_below);
        tie_rank += ties_below;
        mine = 0;
#pragma unroll
        for (int k = 0; k < VPT_MAX; ++k) {
            const float e = v[k];
            bool keep = e > cut_e;
            if (e == cut_e && cut_e > 0.f) { keep = tie_rank < n_take; ++tie_rank; }
            if (!keep) v[k] = 0.f;
            else mine += fixed40(e);
        }
        at = block_excl_scan(mine, sh, &in_block);
        kept = cluster_sum<CL>(cluster, cs, 2, in_block, rank, below);
    }

    const unsigned k24 = draw24(seed, stream_id, (unsigned long long)my_step);
    const unsigned long long lo = kept * (unsigned long long)k24;
    const unsigned long long hi = __umul64hi(kept, (unsigned long long)k24);
    const unsigned long long r = (hi << 40) | (lo >> 24);
    const unsigned long long before = below + at;
    if (mine > 0 && before <= r && r < before + mine) {
        unsigned long long c = before;
        int found = -1;
#pragma unroll
        for (int k = 0; k < VPT_MAX; ++k) {
            const unsigned long long qv = fixed40(v[k]);
            if (found < 0 && qv != 0) {
                c += qv;
                if (r < c) found = i0 + k;
            }
        }
        *cluster.map_shared_rank(&cs.result, 0) = found;
    }
    cluster.sync();                                       // after it nobody touches another block's memory
    if (rank == 0 && tid == 0) {
        int res = cs.result;
        if (res < 0) {                    // all mass below the fixed-point resolution: fall back to the maximum
            res = 0;
            for (int i = 0; i < V; ++i)
                if (src[i] * inv_t == mx) { res = i; break; }
        }
        *out_b = res;
        if (my_ring) my_ring[my_step & (RING - 1)] = res;
    }
}

template <int CL>
__global__ void __launch_bounds__(THREADS)
sample_cluster_kernel(const float* __restrict__ logits, long long ld, float* __restrict__ work, int V,
                      float temperature, int top_k, float top_p, float min_p, float rep_pen, float pres_pen,
                      float freq_pen, const int* __restrict__ recent, const int* __restrict__ n_recent,
                      unsigned long long seed, const int* __restrict__ streams, const int* __restrict__ steps,
                      int* __restrict__ ring, const int* __restrict__ ring_row, int* __restrict__ out,
                      const int* __restrict__ flag_src, int* __restrict__ flag_dst) {
    mv_pdl_begin();
    if (flag_dst && blockIdx.x == 0 && threadIdx.x == 0) *flag_dst = *flag_src;
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ Shared sh;
    __shared__ ClusterShared cs;
    extern __shared__ float tiles[];
    const int rank = (int)cluster.block_rank(), b = blockIdx.x / CL, tid = threadIdx.x;
    const float* src = logits + (size_t)b * ld;
    const int vpt = (V + CL * THREADS - 1) / (CL * THREADS);
    const int i0 = (rank * THREADS + tid) * vpt;          // this thread's indices: i0 ... i0 + vpt - 1

    float v[VPT_MAX];
#pragma unroll
    for (int k = 0; k < VPT_MAX; ++k) v[k] = (k < vpt && i0 + k < V) ? src[i0 + k] : -INFINITY;

    // 1. penalties, once per distinct recent token, by the thread that holds the token's logit
    int* my_ring = ring ? ring + (size_t)ring_row[b] * RING : nullptr;
    const int my_step = steps ? steps[b] : 0;
    const int nr = my_ring ? min(my_step, RECENT_MAX) : (n_recent ? min(n_recent[b], RECENT_MAX) : 0);
    const bool pen = nr > 0 && ((rep_pen > 0.f && rep_pen != 1.f) || pres_pen != 0.f || freq_pen != 0.f);
    if (pen) {                                            // (pen and nr are the same for the whole block)
        // the recent tokens into shared memory, each distinct one once with its count: 64 loads side by side
        // instead of 64 one after another in every thread
        if (tid < RECENT_MAX) cs.rec[tid] = tid < nr ? (my_ring ? my_ring[(my_step - 1 - tid) & (RING - 1)]
                                                                : recent[(size_t)b * RECENT_MAX + tid]) : -1;
        __syncthreads();
        if (tid < nr) {
            const int tok = cs.rec[tid];
            bool first = tok >= 0 && tok < V;
            int count = 0;
            for (int j = 0; j < nr; ++j) {
                if (cs.rec[j] == tok) {
                    if (j < tid) first = false;
                    ++count;
                }
            }
            cs.pen_tok[tid] = first ? tok : -1;
            cs.pen_cnt[tid] = count;
        }
        __syncthreads();
        for (int j = 0; j < nr; ++j) {
            const int tok = cs.pen_tok[j], k0 = tok - i0;
            if (tok < 0 || k0 < 0 || k0 >= vpt) continue;
            const int count = cs.pen_cnt[j];
#pragma unroll
            for (int k = 0; k < VPT_MAX; ++k) {
                if (k == k0) {
                    float x = v[k];
                    if (rep_pen > 0.f && rep_pen != 1.f) x = x > 0.f ? x / rep_pen : x * rep_pen;
                    if (pres_pen != 0.f) x -= pres_pen;
                    if (freq_pen != 0.f) x -= freq_pen * (float)count;
                    v[k] = x;
                }
            }
        }
    }

    // 3. temperature, maximum over the cluster
    const float inv_t = 1.0f / temperature;
    float mx = -INFINITY;
#pragma unroll
    for (int k = 0; k < VPT_MAX; ++k) {
        v[k] *= inv_t;
        mx = fmaxf(mx, v[k]);
    }
    mx = block_max(mx, sh);
    if (tid == 0) cs.bmax = mx;
    if (rank == 0) {                                      // the list that the survivors will be gathered into
        sh.cval[tid] = -INFINITY;
        sh.cidx[tid] = 0;
    }
    cluster.sync();
#pragma unroll
    for (int rr = 0; rr < CL; ++rr) mx = fmaxf(mx, *cluster.map_shared_rank(&cs.bmax, rr));

    // 4. min-p
    if (min_p > 0.f && min_p < 1.f) {
        const float thr = mx + logf(min_p);
#pragma unroll
        for (int k = 0; k < VPT_MAX; ++k)
            if (v[k] < thr) v[k] = -INFINITY;
    }

    if (top_k <= 0 || top_k >= V) {                       // no top-k: the row stays in the cluster's registers
        cluster_tail<CL>(cluster, sh, cs, v, vpt, i0, rank, mx, top_p, seed, (unsigned long long)(streams ? streams[b] : b),
                     my_step, src, inv_t, V, out + b, my_ring);
        return;
    }

    // 5. top-k: radix select of the k-th largest value over the cluster, ties at it are kept
    unsigned prefix = 0, remaining = (unsigned)top_k;
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass, buf = pass & 1;
        if (tid < 256) cs.cnt[buf][tid] = 0;
        __syncthreads();
        const unsigned himask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
#pragma unroll
        for (int k = 0; k < VPT_MAX; ++k) {
            if (k < vpt) {
                const unsigned key = order_key(v[k]);
                if ((key & himask) == prefix) atomicAdd(&cs.cnt[buf][(key >> shift) & 255u], 1u);
            }
        }
        cluster.sync();                                   // (a block barrier too)
        if (tid < 256) {
            unsigned t = 0;
#pragma unroll
            for (int rr = 0; rr < CL; ++rr) t += *cluster.map_shared_rank(&cs.cnt[buf][tid], rr);
            cs.tot[tid] = t;
        }
        __syncthreads();
        if (tid < 32) {
            unsigned bin, rem;
            select_count(cs.tot, remaining, bin, rem);
            if (tid == 0) {
                cs.sel_prefix = prefix | (bin << shift);
                cs.sel_remaining = rem;
            }
        }
        __syncthreads();
        prefix = cs.sel_prefix;
        remaining = cs.sel_remaining;
    }
    const unsigned cut = prefix;
    unsigned long long keepers = 0;
#pragma unroll
    for (int k = 0; k < VPT_MAX; ++k) {
        if (order_key(v[k]) < cut) v[k] = -INFINITY;
        else if (v[k] != -INFINITY) ++keepers;
    }
    unsigned long long n_block;
    unsigned long long at = block_excl_scan(keepers, sh, &n_block);
    if (tid == 0) cs.keep = (unsigned)n_block;
    cluster.sync();
    unsigned base = 0, n_left = 0;
#pragma unroll
    for (int rr = 0; rr < CL; ++rr) {
        const unsigned c = *cluster.map_shared_rank(&cs.keep, rr);
        if (rr < rank) base += c;
        n_left += c;
    }
    if (n_left <= (unsigned)THREADS) {
        // the survivors, in index order (blocks, then threads, then a thread's values), into the first block's list
        float* cval0 = cluster.map_shared_rank(sh.cval, 0);
        int* cidx0 = cluster.map_shared_rank(sh.cidx, 0);
        unsigned place = base + (unsigned)at;
#pragma unroll
        for (int k = 0; k < VPT_MAX; ++k) {
            if (v[k] != -INFINITY) {
                cval0[place] = v[k];
                cidx0[place] = i0 + k;
                ++place;
            }
        }
    }
    cluster.sync();                                       // after it nobody touches another block's memory
    if (rank != 0) return;
    if (n_left <= (unsigned)THREADS) {
        sample_tail(sh, sh.cval + tid, 1, true, mx, top_p, seed, (unsigned long long)(streams ? streams[b] : b), my_step,
                    src, inv_t, V, out + b, my_ring);
    } else {
        sample_row(logits, ld, work, V, temperature, top_k, top_p, min_p, rep_pen, pres_pen, freq_pen, recent, n_recent,
                   seed, streams, steps, ring, ring_row, out, b, sh, tiles);
    }
}

}  // namespace

MV_API int mv_sample(const float* logits, long long ld, float* work, int B, int V, float temperature,
                     int top_k, float top_p, float min_p, float rep_pen, float pres_pen, float freq_pen,
                     const int* recent, const int* n_recent, unsigned long long seed, const int* streams,
                     const int* steps, int* ring, const int* ring_row, int* out, const int* flag_src, int* flag_dst,
                     cudaStream_t stream) {
    if (B <= 0) return 0;
    if (!flag_src) flag_dst = nullptr;
    constexpr size_t TILES = (size_t)(THREADS / 32) * 32 * 33 * sizeof(float);   // a 32 x 33 tile a warp
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TILES);
        attr_set = true;
    }
    // no top_k, or a small one, over a vocabulary that the cluster's threads can hold: the cluster kernel.
    // Up to 16 rows take 8 blocks each; more rows than that would come in waves (measured at 24 rows of
    // 65,536: 50 us with 8 blocks a row, 31 us with 4), so they take 4 blocks each if the vocabulary fits
    // (MIVI_SAMPLE_CLUSTER forces 4 or 8).
    const bool no_k = top_k <= 0 || top_k >= V;
    if (temperature > 0.f && (no_k || top_k <= THREADS) && V <= CL_MAX * THREADS * VPT_MAX) {
        static const int forced = [] { const char* e = getenv("MIVI_SAMPLE_CLUSTER"); return e ? atoi(e) : 0; }();
        int cl = (B > 16 && V <= 4 * THREADS * VPT_MAX) ? 4 : 8;
        if ((forced == 4 && V <= 4 * THREADS * VPT_MAX) || forced == 8) cl = forced;
        auto kernel = cl == 4 ? sample_cluster_kernel<4> : sample_cluster_kernel<8>;
        static bool attr2_set[2] = {false, false};
        if (!attr2_set[cl == 4]) {
            cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TILES);
            attr2_set[cl == 4] = true;
        }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)B * cl);
        cfg.blockDim = dim3(THREADS);
        cfg.dynamicSmemBytes = TILES;
        cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        int na = 0;
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = cl;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
        if (mv_pdl_enabled()) {
            attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[na].val.programmaticStreamSerializationAllowed = 1;
            ++na;
        }
        cfg.attrs = attr;
        cfg.numAttrs = na;
        cudaLaunchKernelEx(&cfg, kernel, logits, ld, work, V, temperature, top_k, top_p, min_p, rep_pen,
                           pres_pen, freq_pen, recent, n_recent, seed, streams, steps, ring, ring_row, out, flag_src,
                           flag_dst);
        return mv_launch_status();
    }
    mv_launch(sample_kernel, B, THREADS, TILES, stream, logits, ld, work, V, temperature, top_k, top_p, min_p,
              rep_pen, pres_pen, freq_pen, recent, n_recent, seed, streams, steps, ring, ring_row, out, flag_src, flag_dst);
    return mv_launch_status();
}
