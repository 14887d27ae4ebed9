// Matrix product for steps with many rows (prompts) on Blackwell's fifth-generation tensor
// cores: out[M, N] = x[M, K] @ W[N, K]^T, bfloat16 operands, float32 accumulation in tensor
// memory.  The reference calls a library product here (engine/engine.py:341-350); this is
// the library-free path, and the only place where the gate/up product and the SwiGLU that
// follows it (engine/kernels/torch_ref.py:74-88) are one kernel.
//
// A block computes 128 x 256 tiles of the output, one after another (one block per SM).  Operand tiles of 64 k (128 bytes per
// row) are brought to shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle) through
// a ring of stages guarded by mbarriers; one thread issues tcgen05.mma (M 128, N 256, K 16,
// four per stage) with the accumulator in 256 columns of tensor memory; tcgen05.commit
// releases a stage when the products that read it are done.  Four warps then read the
// accumulator (tcgen05.ld, one lane quarter each), round once to bfloat16 and store.
//
// SwiGLU mode: the 256 accumulator columns are 128 gate columns and the 128 up columns that
// belong to them (two TMA boxes of 128 weight rows each, from the two halves of the
// concatenated weight); the epilogue stores rnd(rnd(silu(g)) * u), where g and u are first
// rounded to bfloat16 as the separate product would have stored them.
//
// Every wait on an mbarrier is bounded: after kWaitLimitNs by the global timer the waiter sets
// THN_ERR_WAIT_TIMEOUT in the caller's error word and goes on to the common exit, where
// tensor memory is given back.  No wait depends on another block.
#include <cuda.h>

#include "common.cuh"

namespace {

constexpr int BM = 128, BN = 256, BK = 64, UMMA_K = 16;
constexpr int kStages = 4;
constexpr int kThreads = 192;                         // warp 0: TMA, warp 1: MMA + TMEM, warps 2-5: epilogue
constexpr int kTmemCols = 512;                        // two accumulators of 256 columns
constexpr uint32_t kABytes = BM * BK * 2, kBBytes = BN * BK * 2;
constexpr uint32_t kStageBytes = kABytes + kBBytes;
constexpr size_t kSmemBytes = (size_t)kStages * kStageBytes + 1024 /* alignment */ + 256 /* barriers */;
constexpr unsigned long long kWaitLimitNs = 20ull * 1000 * 1000;   // a wait gives up after 20 ms

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
// Bounded wait for the phase with the given parity.  Returns false when it gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_addr(bar);
    unsigned long long start = 0;
    for (int spin = 0;; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
        if ((spin & 63) == 63) {                  // look at the clock now and then
            unsigned long long now;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
            if (start == 0) start = now;
            else if (now - start > kWaitLimitNs) return false;
            __nanosleep(64);
        }
    }
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_addr(dst)), "l"(map), "r"(smem_addr(bar)), "r"(x), "r"(y)
        : "memory");
}

// Shared-memory matrix descriptor for a K-major tile with 128-byte rows and 128-byte swizzle:
// start address / 16 in bits 0-13, leading byte offset (unused here) 16-29, stride byte
// offset (8 rows = 1024 bytes) / 16 in bits 32-45, descriptor version 1 in bits 46-47,
// swizzle mode 2 (128 bytes) in bits 61-63.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    uint64_t desc = 0;
    desc |= (uint64_t)((addr & 0x3FFFF) >> 4);
    desc |= (uint64_t)1 << 16;
    desc |= (uint64_t)(1024 >> 4) << 32;
    desc |= (uint64_t)1 << 46;
    desc |= (uint64_t)2 << 61;
    return desc;
}

// Instruction descriptor, kind::f16: D float32 (bits 4-5 = 1), A and B bfloat16 (bits 7-9 and
// 10-12 = 1), both K-major (bits 15, 16 = 0), N / 8 in bits 17-22, M / 16 in bits 24-28.
constexpr uint32_t kInstrDesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(kInstrDesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void tmem_load_32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// SWIGLU == 0: out [M, N] = x W^T, tile columns [n0, n0 + 256).
// SWIGLU == 1: W is [2 * N, K] = cat(gate, up); out [M, N] = silu(x gate^T) * (x up^T), tile
// columns [n0, n0 + 128); accumulator columns 0-127 are gate, 128-255 the matching up.
//
// A block walks tiles blockIdx.x, blockIdx.x + gridDim.x, ...  The accumulator is double
// buffered in tensor memory (2 x 256 columns): while the epilogue warps drain one tile, the
// MMA thread is already multiplying the next one into the other half.
template <int SWIGLU>
__global__ void __launch_bounds__(kThreads, 1) gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                   const __grid_constant__ CUtensorMap map_b,
                                                                   __nv_bfloat16* __restrict__ out, int M, int N,
                                                                   int K, int tiles_n, int n_tiles,
                                                                   int* __restrict__ err) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + (size_t)kStages * kStageBytes);
    uint64_t* empty = full + kStages;
    uint64_t* acc_full = empty + kStages;      // [2] accumulator ready for the epilogue
    uint64_t* acc_empty = acc_full + 2;        // [2] accumulator drained
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* give_up = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int kTileCols = SWIGLU ? BN / 2 : BN;           // output columns of a tile
    const int n_k = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(acc_full + i, 1);
            mbar_init(acc_empty + i, 4);       // one arrival per epilogue warp
        }
        *give_up = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {   // one warp allocates both accumulators' columns of tensor memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)),
                     "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // ---- TMA producer
        int it = 0;
        for (int tile = blockIdx.x; tile < n_tiles && !*give_up; tile += gridDim.x) {
            const int m0 = (tile / tiles_n) * BM, n0 = (tile % tiles_n) * kTileCols;
            for (int kb = 0; kb < n_k; ++kb, ++it) {
                const int s = it % kStages;
                if (!mbar_wait(empty + s, ((it / kStages) & 1) ^ 1)) {
                    if (err) atomicOr(err, THN_ERR_WAIT_TIMEOUT);
                    *give_up = 1;
                    break;
                }
                unsigned char* a_dst = tiles + (size_t)s * kStageBytes;
                unsigned char* b_dst = a_dst + kABytes;
                mbar_expect_tx(full + s, kStageBytes);
                tma_load_2d(a_dst, &map_a, full + s, kb * BK, m0);
                if (SWIGLU) {
                    tma_load_2d(b_dst, &map_b, full + s, kb * BK, n0);                    // 128 gate rows
                    tma_load_2d(b_dst + kBBytes / 2, &map_b, full + s, kb * BK, N + n0);  // 128 up rows
                } else {
                    tma_load_2d(b_dst, &map_b, full + s, kb * BK, n0);
                }
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer
        int it = 0, local = 0;
        for (int tile = blockIdx.x; tile < n_tiles && !*give_up; tile += gridDim.x, ++local) {
            const int buf = local & 1;
            bool ok = mbar_wait(acc_empty + buf, ((local >> 1) & 1) ^ 1);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t tmem_d = tmem_base + buf * BN;
            for (int kb = 0; kb < n_k && ok; ++kb, ++it) {
                const int s = it % kStages;
                ok = mbar_wait(full + s, (it / kStages) & 1);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_addr = smem_addr(tiles + (size_t)s * kStageBytes);
                const uint64_t a_desc = smem_desc(a_addr), b_desc = smem_desc(a_addr + kABytes);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)      // 32 bytes further along K: + 2 in the address field
                    umma(tmem_d, a_desc + 2 * k, b_desc + 2 * k, (kb | k) != 0);
                umma_commit(empty + s);                    // the stage is free when these products are done
            }
            umma_commit(acc_full + buf);
            if (!ok) {
                if (err) atomicOr(err, THN_ERR_WAIT_TIMEOUT);
                *give_up = 1;
            }
        }
    } else if (warp >= 2) {
        // ---- epilogue: warp w reads tensor-memory lanes 32 * (w % 4) .. + 31 (= tile rows)
        const int quarter = warp & 3;
        int local = 0;
        for (int tile = blockIdx.x; tile < n_tiles && !*give_up; tile += gridDim.x, ++local) {
            const int buf = local & 1;
            const int m0 = (tile / tiles_n) * BM, n0 = (tile % tiles_n) * kTileCols;
            const int row = m0 + quarter * 32 + lane;
            if (!__all_sync(0xffffffffu, mbar_wait(acc_full + buf, (local >> 1) & 1))) {      // all lanes together before tcgen05.ld
                if (lane == 0 && err) atomicOr(err, THN_ERR_WAIT_TIMEOUT);
                *give_up = 1;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t taddr = tmem_base + buf * BN + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < kTileCols; c += 32) {
                uint32_t v[32], u[32];
                tmem_load_32(taddr + c, v);
                if (SWIGLU) tmem_load_32(taddr + BN / 2 + c, u);
                if (row < M) {
                    __nv_bfloat16* dst = out + (size_t)row * N + n0 + c;
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        uint4 packed;
                        __nv_bfloat16* pb = reinterpret_cast<__nv_bfloat16*>(&packed);
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            float x = __uint_as_float(v[j + e]);
                            if (SWIGLU) {
                                const float g = rnd<__nv_bfloat16>(x);
                                const float up = rnd<__nv_bfloat16>(__uint_as_float(u[j + e]));
                                x = rnd<__nv_bfloat16>(g / (1.0f + expf(-g))) * up;
                            }
                            pb[e] = __float2bfloat16_rn(x);
                        }
                        if (n0 + c + j + 8 <= N) {
                            *reinterpret_cast<uint4*>(dst + j) = packed;
                        } else {
                            for (int e = 0; e < 8; ++e)
                                if (n0 + c + j + e < N) dst[j + e] = pb[e];
                        }
                    }
                }
            }
            // this warp has read its quarter of the accumulator: hand it back
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0)
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(acc_empty + buf)) : "memory");
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
    static EncodeTiled fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &result) == cudaSuccess &&
            result == cudaDriverEntryPointSuccess)
            fn = (EncodeTiled)p;
    }
    return fn;
}

// A row-major [rows, K] bfloat16 matrix as a 2-D tensor map with boxes of 64 k x box_rows.
bool make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
    EncodeTiled encode = encode_tiled();
    if (encode == nullptr) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

// 1 if thn_gemm_tcgen05_bf16 takes this shape: K a multiple of 8 (TMA wants 16-byte row
// strides), N a multiple of 8 (16-byte stores).
THN_API int thn_gemm_tcgen05_supported(int M, int N, int K) {
    return M >= 1 && N >= 8 && N % 8 == 0 && K >= 8 && K % 8 == 0;
}

// out [M, N] bfloat16 = x [M, K] @ w [N, K]^T; with swiglu != 0, w is [2 * N, K] (gate rows,
// then up rows) and out [M, N] = silu(x gate^T) * (x up^T).  All pointers 16-byte aligned.
// err: device error word (THN_ERR_WAIT_TIMEOUT if a pipeline wait gave up).
THN_API int thn_gemm_tcgen05_bf16(void* out, const void* x, const void* w, int M, int N, int K, int swiglu, int* err,
                                  cudaStream_t stream) {
    THN_UNSUPPORTED_IF(!thn_gemm_tcgen05_supported(M, N, K), "gemm_tcgen05: shape M=%d N=%d K=%d not supported "
                       "(N and K multiples of 8)", M, N, K);
    THN_CHECK_ARG((((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15) == 0,
                  "gemm_tcgen05: operands must be 16-byte aligned");
    THN_UNSUPPORTED_IF(swiglu && N % (BN / 2) != 0, "gemm_tcgen05: fused SwiGLU needs N (%d) to be a multiple of %d",
                       N, BN / 2);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)kSmemBytes);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(gemm_tcgen05_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)kSmemBytes);
        if (e != cudaSuccess) {
            thn_set_error("gemm_tcgen05: cannot reserve %zu bytes of shared memory: %s", kSmemBytes,
                          cudaGetErrorString(e));
            return (int)e;
        }
        configured = true;
    }
    CUtensorMap map_a, map_b;
    if (!make_map(&map_a, x, M, K, BM) || !make_map(&map_b, w, swiglu ? 2 * N : N, K, swiglu ? BN / 2 : BN)) {
        thn_set_error("gemm_tcgen05: cuTensorMapEncodeTiled failed for M=%d N=%d K=%d", M, N, K);
        return THN_BAD_ARGUMENT;
    }
    const int tile_cols = swiglu ? BN / 2 : BN;
    const int tiles_n = (N + tile_cols - 1) / tile_cols;
    const long long n_tiles = (long long)tiles_n * ((M + BM - 1) / BM);
    THN_UNSUPPORTED_IF(n_tiles > 0x7fffffff, "gemm_tcgen05: too many tiles");
    static int n_sms = 0;
    if (n_sms == 0) {
        int device = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, device);
        if (n_sms <= 0) n_sms = 1;
    }
    const unsigned grid = (unsigned)(n_tiles < n_sms ? n_tiles : n_sms);
    if (swiglu)
        thn_launch(gemm_tcgen05_kernel<1>, grid, kThreads, kSmemBytes, stream, map_a, map_b, (__nv_bfloat16*)out, M, N,
                   K, tiles_n, (int)n_tiles, err);
    else
        thn_launch(gemm_tcgen05_kernel<0>, grid, kThreads, kSmemBytes, stream, map_a, map_b, (__nv_bfloat16*)out, M, N,
                   K, tiles_n, (int)n_tiles, err);
    return thn_launch_status("gemm_tcgen05");
}
