// Y[M, N] = X[M, K] . W[N, K]^T on the fifth-generation tensor cores:
// bfloat16 operands brought into shared memory by TMA, tcgen05.mma issued by
// one thread with the accumulator in tensor memory, read back with tcgen05.ld
// for the epilogue.  This is the matrix product of prefill (M > 64); the
// decode step's product is gemm_small_m.cu.
//
// Both operands are K-major (X rows and W rows are contiguous in K), so a
// 128 x 64 tile of either is 128 rows of 128 bytes: exactly the 128-byte
// swizzle atom that TMA writes and the MMA's shared-memory descriptor reads.
//
// Block = one 128 x BN tile of Y, 6 warps:
//   warp 0   one lane issues the TMA loads of the K blocks into a ring of
//            STAGES buffers (full/empty mbarriers);
//   warp 1   allocates BN columns of tensor memory; one lane issues four
//            128 x BN x 16 MMAs per K block and commits to the stage's
//            "empty" barrier, at the end to the "accumulator ready" barrier;
//   warps 2-5 wait for the accumulator, read their 32 lanes (rows) of tensor
//            memory 32 columns at a time and write Y (store float32, store
//            bfloat16, or add into float32; optional bias).
// Two blocks fit one SM (3 stages of 32 KB each), so one block's epilogue
// overlaps the other's main loop.
//
// Every wait on an mbarrier is bounded: after about two seconds it gives up,
// raises the error flag that the host passes in, and the block still runs to
// its end and frees its tensor memory.  Rows past M or N and the tail of K are
// zero-filled by TMA and masked in the epilogue, so any M, N and any K that is
// a multiple of 8 (16-byte rows) work.
//
// Reference counterpart: quantized_matmul_rows, out[b, n] = sum_d in[b, d] W[n, d]
// (crates/mivi-quant/src/lib.rs:143-245).
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace {

constexpr int BM = 128, BK = 64;
constexpr int THREADS = 192;
constexpr unsigned long long WAIT_NS = 2000000000ull;

__device__ __forceinline__ unsigned smem_u32(const void* p) {
    return (unsigned)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ unsigned long long globaltimer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: false (and the error flag set) if the phase did not complete in time.
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, int* err, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = globaltimer();
    for (;;) {
        for (int i = 0; i < 256; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (globaltimer() - t0 > WAIT_NS) {
            atomicExch(err, code);
            return false;
        }
    }
}
__device__ __forceinline__ void tma_load_2d(unsigned dst, const CUtensorMap* map, int x, int y, unsigned bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
// Shared-memory matrix descriptor: K-major tile, 128-byte swizzle; 8-row groups are 1024 bytes apart.
__device__ __forceinline__ unsigned long long smem_desc(unsigned addr) {
    unsigned long long d = 0;
    d |= (unsigned long long)((addr & 0x3ffffu) >> 4);          // start address
    d |= (unsigned long long)1 << 16;                            // leading byte offset (unused with swizzle)
    d |= (unsigned long long)(1024 >> 4) << 32;                  // stride byte offset
    d |= (unsigned long long)1 << 46;                            // descriptor version of sm_100
    d |= (unsigned long long)2 << 61;                            // SWIZZLE_128B
    return d;
}
// Instruction descriptor of kind::f16: bf16 x bf16 -> f32, both operands K-major.
__device__ __forceinline__ unsigned instr_desc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(m >> 4) << 24);
}
__device__ __forceinline__ void mma_f16(unsigned tmem_d, unsigned long long a, unsigned long long b, unsigned idesc,
                                        unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mma_commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(unsigned taddr, unsigned (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}

template <int BN, int STAGES>
struct SmemLayout {
    static constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int TILE_BYTES = STAGES * STAGE_BYTES;
    static constexpr int BAR_BYTES = (2 * STAGES + 1) * 8 + 8;
    static constexpr int TOTAL = TILE_BYTES + BAR_BYTES + 1024;      // 1024 for the manual alignment
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const float* __restrict__ bias, void* __restrict__ out, int mode, int M, int N, int K, int ldo,
               int* __restrict__ err) {
    using L = SmemLayout<BN, STAGES>;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned long long* bars = (unsigned long long*)(smem + L::TILE_BYTES);
    unsigned* tmem_holder = (unsigned*)(bars + 2 * STAGES + 1);
    const unsigned full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES, acc_bar = full0 + 16 * STAGES;
    const unsigned tiles0 = smem_u32(smem);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int kblocks = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(acc_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_holder)), "r"((unsigned)BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_base = *tmem_holder;

    if (warp == 0) {
        if (lane == 0) {
            for (int kb = 0; kb < kblocks; ++kb) {
                const int s = kb % STAGES;
                const unsigned phase = (unsigned)(kb / STAGES) & 1u;
                if (!mbar_wait(empty0 + 8 * s, phase ^ 1u, err, 1)) break;
                mbar_expect_tx(full0 + 8 * s, L::STAGE_BYTES);
                const unsigned a_dst = tiles0 + s * L::STAGE_BYTES;
                tma_load_2d(a_dst, &map_a, kb * BK, m0, full0 + 8 * s);
                tma_load_2d(a_dst + L::A_BYTES, &map_b, kb * BK, n0, full0 + 8 * s);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const unsigned idesc = instr_desc(BM, BN);
            bool ok = true;
            for (int kb = 0; kb < kblocks && ok; ++kb) {
                const int s = kb % STAGES;
                const unsigned phase = (unsigned)(kb / STAGES) & 1u;
                ok = mbar_wait(full0 + 8 * s, phase, err, 2);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned a_addr = tiles0 + s * L::STAGE_BYTES;
                const unsigned b_addr = a_addr + L::A_BYTES;
#pragma unroll
                for (int k = 0; k < BK / 16; ++k) {
                    // 16 elements of K are 32 bytes further along the swizzled row
                    mma_f16(tmem_base, smem_desc(a_addr + k * 32), smem_desc(b_addr + k * 32), idesc,
                            (kb > 0 || k > 0) ? 1u : 0u);
                }
                mma_commit(empty0 + 8 * s);               // the stage is free once these MMAs have read it
            }
            mma_commit(acc_bar);                          // the accumulator is complete
        }
    } else {
        // epilogue: warp w reads tensor-memory lanes 32 * (w % 4) .. + 31
        const int quarter = warp & 3;
        const int row = m0 + quarter * 32 + lane;
        if (mbar_wait(acc_bar, 0, err, 3)) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                unsigned r[32];
                tmem_ld32(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)c0, r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (row < M) {
                    const int n_base = n0 + c0;
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
                                    const float4 old = *p;
                                    v.x += old.x; v.y += old.y; v.z += old.z; v.w += old.w;
                                }
                                *p = v;
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
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((unsigned)BN)
                     : "memory");
    }
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encoder() {
    static EncodeTiled fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiled)p;
    });
    return fn;
}

struct MapKey {
    const void* ptr; int rows, cols, box_rows;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && rows == o.rows && cols == o.cols && box_rows == o.box_rows;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        return std::hash<const void*>()(k.ptr) ^ ((size_t)k.rows * 1000003u) ^ ((size_t)k.cols * 7919u) ^
               ((size_t)k.box_rows << 20);
    }
};

// A row-major [rows, cols] bfloat16 matrix read in boxes of box_rows x 64 with the 128-byte swizzle.
bool tensor_map(const void* ptr, int rows, int cols, int box_rows, CUtensorMap* out) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    const MapKey key{ptr, rows, cols, box_rows};
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return true; }
    EncodeTiled enc = encoder();
    if (!enc) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    CUtensorMap m;
    if (enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, m);
    *out = m;
    return true;
}

template <int BN, int STAGES>
int launch(const void* X, const void* W, const float* bias, void* out, int mode, int M, int N, int K, int ldo,
           int* err, cudaStream_t stream) {
    using L = SmemLayout<BN, STAGES>;
    CUtensorMap ma, mb;
    if (!tensor_map(X, M, K, BM, &ma) || !tensor_map(W, N, K, BN, &mb)) return (int)cudaErrorInvalidValue;
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        attr_set = true;
    }
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    gemm_tc_kernel<BN, STAGES><<<grid, THREADS, L::TOTAL, stream>>>(ma, mb, bias, out, mode, M, N, K, ldo, err);
    return mv_launch_status();
}

}  // namespace

// mode: 0 store float32, 1 store bfloat16, 2 add into float32, 3 SwiGLU (W rows in groups
// of 16 gate + 16 up; out is bfloat16 [M, N/2] with row stride ldo).  ``err`` points to a
// device int that a block sets (1 producer, 2 MMA, 3 epilogue) if a wait ran out.
// Needs K a multiple of 8 and 16-byte aligned operands.
MV_API int mv_gemm_tc(const void* X, const void* W, const float* bias, void* out, int mode, int M, int N,
                      int K, int ldo, int* err, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || ((uintptr_t)X & 15) || ((uintptr_t)W & 15)) return (int)cudaErrorInvalidValue;
    if (mode == 3 && (N % 32 || ldo % 2)) return (int)cudaErrorInvalidValue;
    if (N <= 64) return launch<64, 4>(X, W, bias, out, mode, M, N, K, ldo, err, stream);
    return launch<128, 3>(X, W, bias, out, mode, M, N, K, ldo, err, stream);
}
