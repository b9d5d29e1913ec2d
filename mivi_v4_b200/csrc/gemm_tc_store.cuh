// The epilogue of the tcgen05 matrix products: one row's 32 consecutive columns of the accumulator,
// from registers to Y, in the mode asked for (0 store float32, 1 store bfloat16, 2 add into float32,
// 3 SwiGLU over columns that alternate in groups of 16 gate and 16 up values).  Included inside the
// including file's own namespace.
// One row's 32 consecutive columns of the accumulator, from registers to Y, in the mode asked for.
__device__ __forceinline__ void store_chunk(const unsigned (&r)[32], int row, int n_base, int N, int mode,
                                            const float* __restrict__ bias, void* __restrict__ out, int ldo) {

        if (mode == 3) {
            // columns n_base .. +15 are gate, +16 .. +31 the up values of the same features
            if (n_base + 32 <= N) {
                __nv_bfloat16* dst = (__nv_bfloat16*)out + (size_t)row * ldo + (n_base >> 1);
                unsigned packed[8];
#pragma unroll
                for (int j = 0; j < 16; j += 2) {
                    float a0 = __uint_as_float(r[j]), a1 = __uint_as_float(r[j + 1]);
                    float b0 = __uint_as_float(r[j + 16]), b1 = __uint_as_float(r[j + 17]);
                    if (bias) {
                        a0 += bias[n_base + j]; a1 += bias[n_base + j + 1];
                        b0 += bias[n_base + j + 16]; b1 += bias[n_base + j + 17];
                    }
                    const __nv_bfloat162 v = __floats2bfloat162_rn(a0 / (1.0f + expf(-a0)) * b0,
                                                                   a1 / (1.0f + expf(-a1)) * b1);
                    packed[j >> 1] = *reinterpret_cast<const unsigned*>(&v);
                }
                if ((((uintptr_t)dst) & 15) == 0) {
                    reinterpret_cast<uint4*>(dst)[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                    reinterpret_cast<uint4*>(dst)[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j) reinterpret_cast<unsigned*>(dst)[j] = packed[j];
                }
            }
        } else if (mode == 1) {
            __nv_bfloat16* dst = (__nv_bfloat16*)out + (size_t)row * ldo + n_base;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                if (n_base + j < N) {
                    float v = __uint_as_float(r[j]);
                    if (bias) v += bias[n_base + j];
                    dst[j] = __float2bfloat16_rn(v);
                }
            }
        } else {
            float* dst = (float*)out + (size_t)row * ldo + n_base;
            const bool vec = n_base + 32 <= N && (((uintptr_t)dst) & 15) == 0;
            if (vec) {
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                           __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                    if (bias) {
                        const float4 bb = *reinterpret_cast<const float4*>(bias + n_base + j);
                        v.x += bb.x; v.y += bb.y; v.z += bb.z; v.w += bb.w;
                    }
                    float4* p = reinterpret_cast<float4*>(dst + j);
                    if (mode == 2) {
                        // added in memory: nothing comes back, so the epilogue does not wait for a read
                        // (one add an element a product: the same sum as load, add, store)
                        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                                     ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
                    } else {
                        *p = v;
                    }
                }
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    if (n_base + j < N) {
                        float v = __uint_as_float(r[j]);
                        if (bias) v += bias[n_base + j];
                        if (mode == 2) v += dst[j];
                        dst[j] = v;
                    }
                }
            }
        }

}

