// Shared device helpers: element types, 32-bit conversions, reductions.
// Every kernel of this library computes in 32-bit floats whatever its
// operands' storage type is; only the storage differs between the bfloat16
// and the float32 path.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define MV_DT_F32 0
#define MV_DT_BF16 1

#define MV_API extern "C" __attribute__((visibility("default")))

__device__ __forceinline__ float mv_to_f32(float v) { return v; }
__device__ __forceinline__ float mv_to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T mv_from_f32(float v);
template <> __device__ __forceinline__ float mv_from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 mv_from_f32<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

// two or four consecutive values in one store
__device__ __forceinline__ void mv_store2(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
__device__ __forceinline__ void mv_store2(__nv_bfloat16* p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}
__device__ __forceinline__ void mv_store4(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void mv_store4(__nv_bfloat16* p, float a, float b, float c, float d) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const unsigned*>(&lo), *reinterpret_cast<const unsigned*>(&hi));
}

__device__ __forceinline__ float mv_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float mv_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.
// ``scratch`` holds 33 floats of shared memory.  The order of the additions
// depends only on the block size, so the result is reproducible.
__device__ __forceinline__ float mv_block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = mv_warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.f;
        t = mv_warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// Loads 8 consecutive elements (16-byte aligned for bf16, 32-byte span for
// f32) into floats.
__device__ __forceinline__ void mv_load8(const float* p, float* out) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
    out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
}
__device__ __forceinline__ void mv_load8(const __nv_bfloat16* p, float* out) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        out[2 * i] = __uint_as_float(w[i] << 16);
        out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

// ---- programmatic dependent launch -------------------------------------------
// The kernels of a decode step are many and short, and each waits for the one
// before it.  Launched with the "programmatic stream serialization" attribute, a
// kernel may become resident while its predecessor still runs; it must then call
// mv_pdl_wait() before it touches anything the predecessor wrote (or anything a
// predecessor may still read).  mv_pdl_launch_dependents() tells the runtime
// that the NEXT kernel may start to launch.  What a kernel does between the two
// (the matrix products prefetch their weights) overlaps with its predecessor.
__device__ __forceinline__ void mv_pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void mv_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void mv_pdl_begin() {
    mv_pdl_launch_dependents();
    mv_pdl_wait();
}

#ifndef __CUDACC_RTC__
#include <stdlib.h>
#include <utility>
// The attribute is on unless MIVI_PDL=0 is set in the environment.  Measured on decode steps of the
// 1.2B-parameter model it is worth 8 to 11 % from 16 tokens on, where the products run on the TMA
// pipeline of gemm_tc_swap.cu and request their first weight tiles before the wait, and 3 % on a
// prefill; the register-streaming gemm_small_m.cu gains nothing from it and has a switch of its own
// (MIVI_PDL_SMALL_M=1), off by default.
static inline bool mv_pdl_enabled() {
    static const bool on = [] {
        const char* e = getenv("MIVI_PDL");
        return !(e && e[0] == '0');
    }();
    return on;
}
static inline bool mv_pdl_small_m_enabled() {
    static const bool on = [] {
        const char* e = getenv("MIVI_PDL_SMALL_M");
        return mv_pdl_enabled() && e && e[0] == '1';
    }();
    return on;
}
template <typename... KArgs, typename... Args>
static inline void mv_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = mv_pdl_enabled() ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
#endif

// A cluster barrier that orders nothing in memory: for "nobody leaves before everybody is here".
__device__ __forceinline__ void mv_cluster_sync_relaxed() {
    asm volatile("barrier.cluster.arrive.relaxed.aligned;\n\tbarrier.cluster.wait.aligned;" ::: "memory");
}

// 16 bytes already in registers -> floats (4 of float32, 8 of bfloat16)
__device__ __forceinline__ void mv_unpack16(const uint4& r, float* out, const float*) {
    out[0] = __uint_as_float(r.x); out[1] = __uint_as_float(r.y);
    out[2] = __uint_as_float(r.z); out[3] = __uint_as_float(r.w);
}
__device__ __forceinline__ void mv_unpack16(const uint4& r, float* out, const __nv_bfloat16*) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        out[2 * i] = __uint_as_float(w[i] << 16);
        out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

// ---- index checks of a debug build -------------------------------------------------
// Built with -DMIVI_DEBUG_CHECKS (MIVI_DEBUG_CHECKS=1 in the environment of the process that
// loads the library), the kernels that turn a page-table entry or a slot number into an
// address compare it first with the bound that the launch wrapper declared for this file
// (mv_set_guard_<file>): an index outside it is never used for an access - a read takes
// page or slot 0 instead, a write is skipped - and the device's error flag is set to 4,
// which the host reports like a wait that ran out.  Nothing traps.  In an ordinary build
// the checks compile to nothing.
#ifdef MIVI_DEBUG_CHECKS
struct MvGuard {
    int n_pages, n_slots;
    int* err;
};
static __device__ MvGuard mv_guard = {0x7fffffff, 0x7fffffff, nullptr};
__device__ __forceinline__ bool mv_page_ok(int page) {
    if ((unsigned)page < (unsigned)mv_guard.n_pages) return true;
    if (mv_guard.err) atomicExch(mv_guard.err, 4);
    return false;
}
__device__ __forceinline__ bool mv_slot_ok(int slot) {
    if ((unsigned)slot < (unsigned)mv_guard.n_slots) return true;
    if (mv_guard.err) atomicExch(mv_guard.err, 4);
    return false;
}
#define MV_GUARD_SETTER(file)                                                                         \
    MV_API int mv_set_guard_##file(int n_pages, int n_slots, int* err, cudaStream_t stream) {            \
        const MvGuard g = {n_pages, n_slots, err};                                                    \
        return (int)cudaMemcpyToSymbolAsync(mv_guard, &g, sizeof(g), 0, cudaMemcpyHostToDevice, stream); \
    }
#else
__device__ __forceinline__ bool mv_page_ok(int) { return true; }
__device__ __forceinline__ bool mv_slot_ok(int) { return true; }
#define MV_GUARD_SETTER(file)
#endif
// an index for a read: itself, or 0 (always valid) where the debug build finds it out of bounds
__device__ __forceinline__ int mv_read_page(int page) { return mv_page_ok(page) ? page : 0; }
__device__ __forceinline__ int mv_read_slot(int slot) { return mv_slot_ok(slot) ? slot : 0; }

static inline int mv_launch_status() {
    return (int)cudaGetLastError();
}
