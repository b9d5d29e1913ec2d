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

static inline int mv_launch_status() {
    return (int)cudaGetLastError();
}
