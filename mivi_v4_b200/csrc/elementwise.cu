// Embedding gather, RMSNorm and SwiGLU: the memory-bound row kernels.
//
// Each is the device form of a loop of the reference engine: the embedding
// row copy (crates/mivi-model/src/model.rs:355-366), rms_norm
// (crates/mivi-core/src/simd/norm.rs:38-72) and swiglu
// (crates/mivi-core/src/math.rs:94-98).
#include "common.cuh"

// ---------------------------------------------------------------- embedding
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ tok,
                             float* __restrict__ x, int H) {
    mv_pdl_begin();
    const int n = blockIdx.x;
    const T* row = table + (size_t)tok[n] * H;
    float* out = x + (size_t)n * H;
    for (int h = threadIdx.x; h < H; h += blockDim.x) out[h] = mv_to_f32(row[h]);
}

MV_API int mv_embed(const void* table, int table_dtype, const int* tok, float* x, int N, int H,
                    cudaStream_t stream) {
    if (N <= 0) return 0;
    const int threads = H >= 1024 ? 256 : 128;
    if (table_dtype == MV_DT_BF16)
        mv_launch(embed_kernel<__nv_bfloat16>, N, threads, 0, stream, (const __nv_bfloat16*)table, tok, x, H);
    else
        mv_launch(embed_kernel<float>, N, threads, 0, stream, (const float*)table, tok, x, H);
    return mv_launch_status();
}

// The same, and the first norm of the first layer handed to the product that follows (steps of few
// tokens): xg = bf16(x * g), and per warp the sum of its elements' squares, one partial sum a warp;
// the product multiplies its results by rsqrt(sum of the partials / H + eps).
template <typename T>
__global__ void embed_link_kernel(const T* __restrict__ table, const int* __restrict__ tok, float* __restrict__ x,
                                  int H, const float* __restrict__ g, __nv_bfloat16* __restrict__ xg,
                                  float* __restrict__ part, int part_stride) {
    mv_pdl_begin();
    const int n = blockIdx.x;
    const T* row = table + (size_t)tok[n] * H;
    float ss = 0.f;
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        const float v = mv_to_f32(row[h]);
        x[(size_t)n * H + h] = v;
        xg[(size_t)n * H + h] = __float2bfloat16_rn(v * g[h]);
        ss = fmaf(v, v, ss);
    }
    ss = mv_warp_sum(ss);
    if ((threadIdx.x & 31) == 0) part[(size_t)n * part_stride + (threadIdx.x >> 5)] = ss;
}

static inline int embed_threads(int H) { return H >= 1024 ? 256 : 128; }

// How many partial sums a row mv_embed_link writes.
MV_API int mv_embed_link_partials(int H) { return embed_threads(H) / 32; }

MV_API int mv_embed_link(const void* table, int table_dtype, const int* tok, float* x, int N, int H, const float* g,
                         void* xg, float* part, int part_stride, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (!g || !xg || !part || part_stride < embed_threads(H) / 32) return (int)cudaErrorInvalidValue;
    if (table_dtype == MV_DT_BF16)
        mv_launch(embed_link_kernel<__nv_bfloat16>, N, embed_threads(H), 0, stream, (const __nv_bfloat16*)table, tok, x, H,
                  g, (__nv_bfloat16*)xg, part, part_stride);
    else
        mv_launch(embed_link_kernel<float>, N, embed_threads(H), 0, stream, (const float*)table, tok, x, H, g,
                  (__nv_bfloat16*)xg, part, part_stride);
    return mv_launch_status();
}

// ------------------------------------------------------------------ rmsnorm
// y[i, :] = x[r, :] * rsqrt(mean(x[r, :]^2) + eps) * w, r = rows ? rows[i] : i.
// Statistics in 32-bit whatever the output type.
template <typename TO>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w,
                               TO* __restrict__ y, const int* __restrict__ rows, int H, float eps) {
    mv_pdl_begin();
    __shared__ float scratch[33];
    const int i = blockIdx.x;
    const int r = rows ? rows[i] : i;
    const float* xr = x + (size_t)r * H;
    float ss = 0.f;
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        const float v = xr[h];
        ss = fmaf(v, v, ss);
    }
    ss = mv_block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)H + eps);
    TO* yr = y + (size_t)i * H;
    for (int h = threadIdx.x; h < H; h += blockDim.x) yr[h] = mv_from_f32<TO>(xr[h] * scale * w[h]);
}

// The same for rows that fit the registers of one block (H a multiple of 4, at most
// 8192): each thread keeps its float4s, so the row is read once.
template <typename TO, int THREADS>
__global__ void __launch_bounds__(THREADS)
rmsnorm_regs_kernel(const float* __restrict__ x, const float* __restrict__ w, TO* __restrict__ y,
                    const int* __restrict__ rows, int H, float eps) {
    mv_pdl_begin();
    __shared__ float scratch[33];
    constexpr int MAXV = 8192 / 4 / THREADS;
    const int i = blockIdx.x;
    const int r = rows ? rows[i] : i;
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)r * H);
    const int nv = H >> 2;
    float4 v[MAXV];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
        const int c = threadIdx.x + j * THREADS;
        if (c < nv) {
            v[j] = xr[c];
            ss = fmaf(v[j].x, v[j].x, ss); ss = fmaf(v[j].y, v[j].y, ss);
            ss = fmaf(v[j].z, v[j].z, ss); ss = fmaf(v[j].w, v[j].w, ss);
        }
    }
    ss = mv_block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)H + eps);
    TO* yr = y + (size_t)i * H;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
        const int c = threadIdx.x + j * THREADS;
        if (c < nv) {
            const float4 ww = reinterpret_cast<const float4*>(w)[c];
            mv_store4(yr + 4 * c, v[j].x * scale * ww.x, v[j].y * scale * ww.y, v[j].z * scale * ww.z,
                      v[j].w * scale * ww.w);
        }
    }
}

// Many rows (a prefill): one WARP per row, each lane keeping up to 16 float4 of it in registers.  All
// of a row's loads are in flight at once and the sum needs shuffles only, no block barrier.  H a multiple
// of 4, at most 2048 (16 float4 a lane).
template <typename TO>
__global__ void __launch_bounds__(256)
rmsnorm_warp_kernel(const float* __restrict__ x, const float* __restrict__ w, TO* __restrict__ y,
                    const int* __restrict__ rows, int n_rows, int H, float eps) {
    mv_pdl_begin();
    constexpr int MAXV = 16;
    const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (i >= n_rows) return;
    const int r = rows ? rows[i] : i;
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)r * H);
    const int nv = H >> 2;
    float4 v[MAXV];
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
        const int c = lane + 32 * j;
        v[j] = c < nv ? xr[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
        ss = fmaf(v[j].x, v[j].x, ss); ss = fmaf(v[j].y, v[j].y, ss);
        ss = fmaf(v[j].z, v[j].z, ss); ss = fmaf(v[j].w, v[j].w, ss);
    }
    ss = mv_warp_sum(ss);
    const float scale = 1.0f / sqrtf(ss / (float)H + eps);
    TO* yr = y + (size_t)i * H;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
        const int c = lane + 32 * j;
        if (c < nv) {
            const float4 ww = reinterpret_cast<const float4*>(w)[c];
            mv_store4(yr + 4 * c, v[j].x * scale * ww.x, v[j].y * scale * ww.y, v[j].z * scale * ww.z,
                      v[j].w * scale * ww.w);
        }
    }
}

MV_API int mv_rmsnorm(const float* x, const float* w, void* y, int y_dtype, const int* rows,
                      int n_rows, int H, float eps, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    const bool aligned = H % 4 == 0 && (((uintptr_t)x | (uintptr_t)w | (uintptr_t)y) & 15) == 0;
    if (aligned && H <= 2048 && H >= 512 && n_rows >= 512) {
        const unsigned blocks = (unsigned)((n_rows + 7) / 8);
        if (y_dtype == MV_DT_BF16)
            mv_launch(rmsnorm_warp_kernel<__nv_bfloat16>, blocks, 256, 0, stream, x, w, (__nv_bfloat16*)y, rows, n_rows, H, eps);
        else
            mv_launch(rmsnorm_warp_kernel<float>, blocks, 256, 0, stream, x, w, (float*)y, rows, n_rows, H, eps);
        return mv_launch_status();
    }
    if (aligned && H <= 8192 && H >= 256) {
        if (y_dtype == MV_DT_BF16)
            mv_launch(rmsnorm_regs_kernel<__nv_bfloat16, 256>, n_rows, 256, 0, stream, x, w, (__nv_bfloat16*)y, rows, H, eps);
        else
            mv_launch(rmsnorm_regs_kernel<float, 256>, n_rows, 256, 0, stream, x, w, (float*)y, rows, H, eps);
        return mv_launch_status();
    }
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    if (y_dtype == MV_DT_BF16)
        mv_launch(rmsnorm_kernel<__nv_bfloat16>, n_rows, threads, 0, stream, x, w, (__nv_bfloat16*)y, rows, H, eps);
    else
        mv_launch(rmsnorm_kernel<float>, n_rows, threads, 0, stream, x, w, (float*)y, rows, H, eps);
    return mv_launch_status();
}

// ------------------------------------------------------------------- swiglu
// h[n, f] = silu(gate) * up, silu(a) = a / (1 + e^-a).  group == 0: gate = gu[n, f],
// up = gu[n, F + f] (the two halves end to end).  group == 16: the columns come in
// groups of 16 gate values followed by the 16 up values of the same features.
template <typename TO>
__global__ void swiglu_kernel(const float* __restrict__ gu, TO* __restrict__ h, long long total, int F, int group) {
    mv_pdl_begin();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long n = i / F;
    const int f = (int)(i - n * F);
    const int ga = group ? (f / group) * 2 * group + f % group : f;
    const int gb = group ? ga + group : F + f;
    const float a = gu[n * 2 * F + ga];
    const float b = gu[n * 2 * F + gb];
    h[i] = mv_from_f32<TO>(a / (1.0f + expf(-a)) * b);
}

MV_API int mv_swiglu(const float* gu, void* h, int h_dtype, int N, int F, int group, cudaStream_t stream) {
    const long long total = (long long)N * F;
    if (total <= 0) return 0;
    const int threads = 256;
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    if (h_dtype == MV_DT_BF16)
        mv_launch(swiglu_kernel<__nv_bfloat16>, blocks, threads, 0, stream, gu, (__nv_bfloat16*)h, total, F, group);
    else
        mv_launch(swiglu_kernel<float>, blocks, threads, 0, stream, gu, (float*)h, total, F, group);
    return mv_launch_status();
}

// ------------------------------------------------------------- small copies
// A few bytes from the device to pinned host memory on ``stream`` (the error flag's
// way to the host; recorded into a CUDA graph like any launch).
MV_API int mv_copy_to_host(void* dst, const void* src, long long bytes, cudaStream_t stream) {
    if (bytes <= 0) return 0;
    return (int)cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDeviceToHost, stream);
}

// ------------------------------------------------------------------- delay
// Keeps the stream busy for ``us`` microseconds (at most 50 ms): a profile of a step of
// many short kernels enqueues it first, so that the step's launches queue up behind it and
// run back to back instead of each waiting for the host.
__global__ void delay_kernel(unsigned long long ns) {
    unsigned long long t0, t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    do {
        __nanosleep(2000);
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    } while (t - t0 < ns);
}

MV_API int mv_delay(long long us, cudaStream_t stream) {
    if (us <= 0) return 0;
    if (us > 50000) us = 50000;
    delay_kernel<<<1, 1, 0, stream>>>((unsigned long long)us * 1000ull);
    return mv_launch_status();
}
