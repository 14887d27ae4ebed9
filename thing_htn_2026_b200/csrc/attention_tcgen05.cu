// Causal grouped-query flash attention for prompts on Blackwell's fifth-generation tensor
// cores, over the paged cache (bfloat16, head size 128, pages of 64 keys).  The reference
// calls a library's flash attention here (engine/engine.py:1123-1131, :1165-1179); the
// arithmetic is engine/kernels/torch_ref.py:168-227: scores and softmax in float32, the
// un-normalised probabilities rounded to bfloat16 before they multiply V, one division by
// the float32 row sum at the end.
//
// One block: 128 consecutive rows of one sequence, one query head.  Row r of the tile is
// lane r of tensor memory and is owned by one thread of the four softmax warps, so a row's
// maximum and sum need no shuffles.  Per tile of 64 keys (one page):
//   S = Q K^T      tcgen05.mma, M 128, N 64, K 16 x 8; Q and K tiles in shared memory (TMA,
//                  128-byte swizzle, K-major), S in 64 columns of tensor memory;
//   softmax        each thread reads its row of S (tcgen05.ld), masks, takes the running
//                  maximum, rescales the output accumulator in tensor memory when the
//                  maximum moved, and writes exp2 of its row as bfloat16 pairs back into the
//                  first 32 columns of the S buffer it came from (tcgen05.st): that is P;
//   O += P V       tcgen05.mma, M 128, N 128, K 16 x 4; P as the operand from tensor memory,
//                  the V page as it lies in the cache ([key][d]: the N index contiguous, an
//                  MN-major operand), O in 128 columns of tensor memory.
// K and V pages come through a two-stage ring filled by TMA from a tensor map over the
// cache entry.  S has two buffers, so S of tile t + 1 is multiplied while the softmax warps
// work on tile t, and since P lives in its own S buffer nothing but the tensor core's own
// order stands between one tile's O += P V and the next tile's softmax.  Two blocks per SM.
//
// Every wait on an mbarrier is bounded (see gemm_tcgen05.cu); a waiter that gives up sets
// THN_ERR_WAIT_TIMEOUT and all roles leave through the common exit.
#include <cuda.h>
#include <math.h>

#include "common.cuh"

namespace {

constexpr int kRows = 128, kKeys = 64, D = 128;
constexpr int kThreads = 192;                     // warp 0: TMA, warp 1: MMA + TMEM, warps 2-5: softmax
constexpr int kStages = 2;
constexpr int kTmemCols = 256;                    // S (two buffers): columns 0-63 and 64-127, O: columns 128-255
constexpr int kColS = 0, kColO = 128;
constexpr uint32_t kQBytes = kRows * D * 2;       // 32 KB: two [128 x 64] swizzled blocks
constexpr uint32_t kKBytes = kKeys * D * 2;       // 16 KB: two [64 x 64] blocks
constexpr uint32_t kVBytes = kKeys * D * 2;       // 16 KB: two [64 keys x 64 d] blocks
constexpr uint32_t kStageBytes = kKBytes + kVBytes;
constexpr size_t kSmemBytes = kQBytes + kStages * kStageBytes + 256;   // two blocks fit one SM
constexpr unsigned long long kWaitLimitNs = 20ull * 1000 * 1000;   // a wait gives up after 20 ms
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
// Bounded wait: try_wait parks the thread in hardware for a short while instead of spinning
// (spinning warps would take issue slots from the softmax warps); the global timer bounds
// the whole wait.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_addr(bar);
    unsigned long long start = 0;
    for (;;) {
        uint32_t done;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, 1000;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
        unsigned long long now;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
        if (start == 0) start = now;
        else if (now - start > kWaitLimitNs) return false;
    }
}
// The same without parking: for the one thread that issues the products, whose every wait stands
// between the softmax warps and the tensor core.
__device__ __forceinline__ bool mbar_wait_spin(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_addr(bar);
    unsigned long long start = 0;
    for (int spins = 0;; ++spins) {
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
        if ((spins & 63) == 63) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
            if (start == 0) start = now;
            else if (now - start > kWaitLimitNs) return false;
        }
    }
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_addr(dst)), "l"(map), "r"(smem_addr(bar)), "r"(x), "r"(y)
        : "memory");
}

// Shared-memory matrix descriptors, 128-byte swizzle, version 1 (see gemm_tcgen05.cu).
// K-major (rows of 64 k = 128 bytes; 8 rows = 1024 bytes apart): Q, K and P.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// MN-major (rows of 64 n = 128 bytes, one row per k; 8 k = 1024 bytes apart; the next 64 n
// lie `next_n_block` bytes further): the V page, n = d, k = key.
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr, uint32_t next_n_block) {
    return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)(next_n_block >> 4) << 16) |
           ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// Instruction descriptors, kind::f16, float32 accumulator, bfloat16 operands.
constexpr uint32_t instr_desc(int m, int n, int b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}
constexpr uint32_t kDescS = instr_desc(kRows, kKeys, 0);   // S = Q K^T: both K-major
constexpr uint32_t kDescO = instr_desc(kRows, D, 1);       // O += P V: V MN-major

__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                     uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The same with the 128-row operand read from tensor memory: lane = row, a 32-bit column holds
// two consecutive k.
__device__ __forceinline__ void umma_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
        "}\n"
        ::"r"(tmem_d), "r"(tmem_a), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void tmem_load_32(uint32_t taddr, float (&r)[32]) {
    uint32_t v[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) r[i] = __uint_as_float(v[i]);
}
__device__ __forceinline__ void tmem_store_32(uint32_t taddr, const float (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(__float_as_uint(r[0])), "r"(__float_as_uint(r[1])), "r"(__float_as_uint(r[2])),
          "r"(__float_as_uint(r[3])), "r"(__float_as_uint(r[4])), "r"(__float_as_uint(r[5])),
          "r"(__float_as_uint(r[6])), "r"(__float_as_uint(r[7])), "r"(__float_as_uint(r[8])),
          "r"(__float_as_uint(r[9])), "r"(__float_as_uint(r[10])), "r"(__float_as_uint(r[11])),
          "r"(__float_as_uint(r[12])), "r"(__float_as_uint(r[13])), "r"(__float_as_uint(r[14])),
          "r"(__float_as_uint(r[15])), "r"(__float_as_uint(r[16])), "r"(__float_as_uint(r[17])),
          "r"(__float_as_uint(r[18])), "r"(__float_as_uint(r[19])), "r"(__float_as_uint(r[20])),
          "r"(__float_as_uint(r[21])), "r"(__float_as_uint(r[22])), "r"(__float_as_uint(r[23])),
          "r"(__float_as_uint(r[24])), "r"(__float_as_uint(r[25])), "r"(__float_as_uint(r[26])),
          "r"(__float_as_uint(r[27])), "r"(__float_as_uint(r[28])), "r"(__float_as_uint(r[29])),
          "r"(__float_as_uint(r[30])), "r"(__float_as_uint(r[31]))
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// For the test of the bounded waits only: when set, the loader brings Q and then no key or value
// page at all, so that the waits for them run out, say so in the error word, and the block leaves
// through its common exit.
__device__ int g_test_skip_kv_loads = 0;

// map_q: q as [rows, n_q * 128], boxes of 64 x 128 rows.  map_kv: the cache entry as
// [pages * 2 * n_kv * 64, 128], boxes of 64 x 64 rows (one half of one head's page).
__global__ void __launch_bounds__(kThreads, 2) attention_tcgen05_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
    __nv_bfloat16* __restrict__ out, const int* __restrict__ tile_row0, const int* __restrict__ tile_rows,
    const int* __restrict__ row_slot, const int* __restrict__ row_pos, const int* __restrict__ block_table,
    int bt_stride, int n_kv, int n_q, float scale_log2, int window, int* __restrict__ err) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(1024) unsigned char smem_raw[];      // swizzled tiles want 1024-byte alignment
    unsigned char* q_smem = smem_raw;
    unsigned char* kv_smem = q_smem + kQBytes;                         // [stage][K 16 KB | V 16 KB]
    uint64_t* q_full = reinterpret_cast<uint64_t*>(kv_smem + kStages * kStageBytes);
    uint64_t* k_full = q_full + 1;               // [kStages] the K page of a tile is in shared memory
    uint64_t* k_empty = k_full + kStages;        // [kStages] ... and has been multiplied (free after S = Q K^T)
    uint64_t* v_full = k_empty + kStages;        // [kStages] the same for the V page
    uint64_t* v_empty = v_full + kStages;        // [kStages] (free after O += P V)
    uint64_t* s_full = v_empty + kStages;        // [2] S = Q K^T of a tile is in tensor memory (two buffers)
    uint64_t* p_ready = s_full + 2;              // [2] P of a tile is in its S buffer (4 arrivals).  One per buffer: a
                                                 // warp that is a tile ahead of the others arrives on the other one
    uint64_t* o_full = p_ready + 2;              // O += P V of this tile is done
    uint64_t* o_done = o_full + 1;               // the block's last O += P V is done
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_done + 1);
    volatile int* give_up = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = gridDim.y - 1 - blockIdx.y, h = blockIdx.x;     // heads fastest; the list ends with the long tiles
    const int row0 = tile_row0[tile], n_rows = tile_rows[tile];
    const int kvh = h / (n_q / n_kv);
    const int pos0 = row_pos[row0], pos_last = pos0 + n_rows - 1;
    int first_key = 0;
    if (window > 0 && pos0 - window + 1 > 0) first_key = pos0 - window + 1;
    const int t_first = first_key / kKeys, t_last = pos_last / kKeys;
    const int* pages = block_table + (size_t)row_slot[row0] * bt_stride;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < kStages; ++s) {
            mbar_init(k_full + s, 1);
            mbar_init(k_empty + s, 1);
            mbar_init(v_full + s, 1);
            mbar_init(v_empty + s, 1);
        }
        mbar_init(s_full, 1);
        mbar_init(s_full + 1, 1);
        mbar_init(p_ready, 4);
        mbar_init(p_ready + 1, 4);
        mbar_init(o_full, 1);
        mbar_init(o_done, 1);
        *give_up = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)),
                     "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // ---- TMA producer: Q once, then one K page and one V page per tile
        mbar_expect_tx(q_full, kQBytes);
        tma_load_2d(q_smem, &map_q, q_full, h * D, row0);
        tma_load_2d(q_smem + kQBytes / 2, &map_q, q_full, h * D + 64, row0);
        // K pages and V pages have rings of their own: a K page is free again once S = Q K^T has
        // read it, long before the tile's V page, so K runs one tile further ahead: K(0), K(1),
        // V(0), K(2), V(1), ...
        const int n_it = g_test_skip_kv_loads ? 0 : t_last - t_first + 1;
        auto load = [&](int it, int which) {        // which: 0 = K, 1 = V
            const int s = it % kStages;
            uint64_t* empty = which ? v_empty : k_empty;
            uint64_t* full = which ? v_full : k_full;
            if (!mbar_wait(empty + s, ((it / kStages) & 1) ^ 1)) {
                if (err) atomicOr(err, THN_ERR_WAIT_TIMEOUT);
                return false;
            }
            const int page = pages[t_first + it];
            if (page < 0) {
                if (err) atomicOr(err, THN_ERR_PAGE_UNMAPPED);
                return false;
            }
            unsigned char* dst = kv_smem + (size_t)s * kStageBytes + (which ? kKBytes : 0);
            const int row = ((page * 2 + which) * n_kv + kvh) * kKeys;
            mbar_expect_tx(full + s, kKBytes);
            tma_load_2d(dst, &map_kv, full + s, 0, row);
            tma_load_2d(dst + kKBytes / 2, &map_kv, full + s, 64, row);
            return true;
        };
        bool ok = n_it <= 0 || load(0, 0);
        for (int it = 0; it < n_it && ok && !*give_up; ++it) {
            if (it + 1 < n_it) ok = load(it + 1, 0);
            if (ok) ok = load(it, 1);
        }
        if (!ok) *give_up = 1;
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer.  S of tile it + 1 is multiplied while the softmax warps work on
        // tile it; O += P V of tile it follows as soon as its P is ready.
        bool ok = mbar_wait_spin(q_full, 0);
        const int n_it = t_last - t_first + 1;
        const uint32_t q_addr = smem_addr(q_smem);
        auto qk = [&](int it) {          // S[it & 1] = Q K(it)^T
            const int s = it % kStages;
            if (!mbar_wait_spin(k_full + s, (it / kStages) & 1)) return false;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t k_addr = smem_addr(kv_smem + (size_t)s * kStageBytes);
            // eight k steps of 16 d; d 0-63 in the first swizzled block, 64-127 in the second
#pragma unroll
            for (int k = 0; k < D / 16; ++k) {
                const uint64_t a = desc_k_major(q_addr + (k / 4) * (kQBytes / 2) + (k % 4) * 32);
                const uint64_t b = desc_k_major(k_addr + (k / 4) * (kKBytes / 2) + (k % 4) * 32);
                umma(tmem_base + kColS + (it & 1) * kKeys, a, b, kDescS, k != 0);
            }
            umma_commit(k_empty + s);             // the K page is free when these products are done
            umma_commit(s_full + (it & 1));
            return true;
        };
        if (ok && n_it > 0) ok = qk(0);
        for (int it = 0; it < n_it && ok && !*give_up; ++it) {
            if (it + 1 < n_it) {
                ok = qk(it + 1);
                if (!ok) break;
            }
            ok = mbar_wait_spin(p_ready + (it & 1), (it >> 1) & 1);      // P is in tensor memory; O has been rescaled
            if (!ok) break;
            const int s = it % kStages;
            ok = mbar_wait_spin(v_full + s, (it / kStages) & 1);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t v_addr = smem_addr(kv_smem + (size_t)s * kStageBytes) + kKBytes;
            // O += P V: four k steps of 16 keys; P: 8 columns of bfloat16 pairs per step, in the
            // S buffer of this tile; V rows are keys, 16 keys = 2048 bytes further
#pragma unroll
            for (int k = 0; k < kKeys / 16; ++k) {
                const uint64_t b = desc_mn_major(v_addr + k * 2048, kVBytes / 2);
                umma_a_tmem(tmem_base + kColO, tmem_base + kColS + (it & 1) * kKeys + k * 8, b, kDescO, (it | k) != 0);
            }
            umma_commit(v_empty + s);             // the V page is free when these products are done
            umma_commit(o_full);
            if (it + 1 == n_it) umma_commit(o_done);
        }
        if (!ok) {
            if (err) atomicOr(err, THN_ERR_WAIT_TIMEOUT);
            *give_up = 1;
        }
    } else if (warp >= 2) {
        // ---- softmax: thread = row.  Warp w owns tensor-memory lanes 32 * (w % 4) .. + 31.
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;                   // row of the tile
        const int pos = pos0 + r;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
        float run_max = -INFINITY, run_sum = 0.f;
        bool ok = true;
        int it = 0;
        for (int t = t_first; t <= t_last && !*give_up; ++t, ++it) {
            ok = mbar_wait(s_full + (it & 1), (it >> 1) & 1);
            ok = __all_sync(0xffffffffu, ok);        // the lanes leave a wait one by one; tcgen05.ld wants the warp together
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float s[64];
            {
                float part[32];
                tmem_load_32(lane_base + kColS + (it & 1) * kKeys, part);
#pragma unroll
                for (int i = 0; i < 32; ++i) s[i] = part[i];
                tmem_load_32(lane_base + kColS + (it & 1) * kKeys + 32, part);
#pragma unroll
                for (int i = 0; i < 32; ++i) s[32 + i] = part[i];
            }
            const int key0 = t * kKeys;
            float tile_max = -INFINITY;
            // a tile that every row of this warp sees whole needs no mask
            const int warp_first = pos0 + quarter * 32, warp_last = warp_first + 31;
            const bool whole = key0 + kKeys - 1 <= warp_first && (window <= 0 || key0 > warp_last - window);
            if (!whole) {
#pragma unroll
                for (int i = 0; i < 64; ++i) {
                    const int key = key0 + i;
                    const bool visible = key <= pos && (window <= 0 || key > pos - window);
                    s[i] = visible ? s[i] : -INFINITY;
                }
            }
#pragma unroll
            for (int i = 0; i < 64; i += 2) tile_max = fmaxf(tile_max, fmaxf(s[i], s[i + 1]));
            tile_max *= scale_log2;                                        // scale > 0: the maximum scales with it
            // The reference point of the exponentials follows the maximum only when the maximum
            // has moved by more than 2^8 (softmax does not depend on the reference point; P stays
            // below 2^8, far inside bfloat16 and float32 range), so that the output accumulator
            // in tensor memory is rescaled a few times per row instead of at nearly every tile.
            float new_max = run_max;
            if (tile_max > run_max + 8.0f) new_max = tile_max;
            const float base = new_max == -INFINITY ? 0.f : new_max;      // no visible key yet
            const float corr = fast_exp2(run_max - base);                  // 1 when unchanged, 0 on the first tile
            run_max = new_max;
            // P, rounded to bfloat16, in registers first: the exponentials run while the
            // previous O += P V is still in the tensor core.
            float sum = 0.f;
            uint4 packed[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                __nv_bfloat162* pb = reinterpret_cast<__nv_bfloat162*>(&packed[c]);
#pragma unroll
                for (int e = 0; e < 8; e += 2) {
                    const float p0 = fast_exp2(fmaf(s[c * 8 + e], scale_log2, -base));
                    const float p1 = fast_exp2(fmaf(s[c * 8 + e + 1], scale_log2, -base));
                    sum += p0 + p1;
                    pb[e / 2] = __floats2bfloat162_rn(p0, p1);
                }
            }
            // O is rescaled only when some row of the warp moved its reference point; then the
            // previous O += P V must be complete first (S of this tile says that the one before
            // that is, so the parity is unambiguous).  tcgen05.ld/st are warp-wide, so the whole
            // warp goes if any of its rows must.
            if (it > 0 && __any_sync(0xffffffffu, corr != 1.0f)) {
                ok = __all_sync(0xffffffffu, mbar_wait(o_full, (it - 1) & 1));
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
                for (int c = 0; c < D; c += 32) {
                    float o[32];
                    tmem_load_32(lane_base + kColO + c, o);
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] *= corr;
                    tmem_store_32(lane_base + kColO + c, o);
                }
            }
            // P over the first 32 columns of this tile's S (the row's S is in registers by now):
            // column j holds keys 2j and 2j + 1.
            {
                float words[32];
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    words[4 * c] = __uint_as_float(packed[c].x);
                    words[4 * c + 1] = __uint_as_float(packed[c].y);
                    words[4 * c + 2] = __uint_as_float(packed[c].z);
                    words[4 * c + 3] = __uint_as_float(packed[c].w);
                }
                tmem_store_32(lane_base + kColS + (it & 1) * kKeys, words);
            }
            run_sum = run_sum * corr + sum;
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(p_ready + (it & 1));
        }
        if (ok && !*give_up && it > 0) {             // (ok is the same in every lane: see the waits above)
            ok = __all_sync(0xffffffffu, mbar_wait(o_done, 0));
            if (ok) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const float inv = 1.0f / run_sum;
                __nv_bfloat16* dst = out + ((size_t)(row0 + r) * n_q + h) * D;
#pragma unroll 1
                for (int c = 0; c < D; c += 32) {
                    float o[32];
                    tmem_load_32(lane_base + kColO + c, o);
                    if (r < n_rows) {
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            uint4 packed;
                            __nv_bfloat16* pb = reinterpret_cast<__nv_bfloat16*>(&packed);
#pragma unroll
                            for (int e = 0; e < 8; ++e) pb[e] = __float2bfloat16_rn(o[j + e] * inv);
                            *reinterpret_cast<uint4*>(dst + c + j) = packed;
                        }
                    }
                }
            }
        }
        if (!ok) {
            if (lane == 0 && err) atomicOr(err, THN_ERR_WAIT_TIMEOUT);
            *give_up = 1;
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

// A row-major [rows, cols] bfloat16 matrix with boxes of 64 columns x box_rows rows.
bool make_map(CUtensorMap* map, const void* base, long long rows, long long cols, int box_rows) {
    EncodeTiled encode = encode_tiled();
    if (encode == nullptr) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

// Test switch (see g_test_skip_kv_loads): nonzero makes every later launch on the current device
// run into its wait limit.  Returns a status.
THN_API int thn_attention_tcgen05_test_skip_loads(int on) {
    const int value = on ? 1 : 0;
    cudaError_t e = cudaMemcpyToSymbol(g_test_skip_kv_loads, &value, sizeof(int));
    if (e != cudaSuccess) {
        thn_set_error("attention_tcgen05 test switch: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return THN_OK;
}

// 1 if thn_attention_prefill_tcgen05 takes this shape.
THN_API int thn_attention_tcgen05_supported(int head_dim, int page_size, int n_q, int n_kv) {
    return head_dim == D && page_size == kKeys && n_kv > 0 && n_q % n_kv == 0;
}

// Same contract as thn_attention_prefill_bf16 with row tiles of 128 rows (tile_rows 1..128);
// n_rows_total is the number of packed rows of q and out, n_pages the pages of the cache entry.
THN_API int thn_attention_prefill_tcgen05(void* out, const void* q, const int* tile_row0, const int* tile_rows,
                                          int n_tiles, int n_rows_total, const int* row_slot, const int* row_pos,
                                          const void* kv_base, long long n_pages, const int* block_table,
                                          int bt_stride, int n_kv, int page_size, int head_dim, int n_q, float scale,
                                          int window, int* err, cudaStream_t stream) {
    THN_CHECK_ARG(n_tiles >= 0 && n_q > 0 && n_rows_total >= 0 && n_pages > 0, "attention_tcgen05: bad sizes");
    THN_UNSUPPORTED_IF(!thn_attention_tcgen05_supported(head_dim, page_size, n_q, n_kv),
                       "attention_tcgen05: head_dim %d, page %d, heads %d/%d not supported", head_dim, page_size, n_q,
                       n_kv);
    THN_CHECK_ARG((((uintptr_t)q | (uintptr_t)out | (uintptr_t)kv_base) & 15) == 0,
                  "attention_tcgen05: operands must be 16-byte aligned");
    if (n_tiles == 0) return THN_OK;
    THN_UNSUPPORTED_IF(n_tiles > 65535, "attention_tcgen05: %d row tiles in one step (at most 65535)", n_tiles);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)kSmemBytes);
        if (e != cudaSuccess) {
            thn_set_error("attention_tcgen05: cannot reserve %zu bytes of shared memory: %s", kSmemBytes,
                          cudaGetErrorString(e));
            return (int)e;
        }
        configured = true;
    }
    CUtensorMap map_q, map_kv;
    if (!make_map(&map_q, q, n_rows_total, (long long)n_q * D, kRows) ||
        !make_map(&map_kv, kv_base, n_pages * 2 * n_kv * kKeys, D, kKeys)) {
        thn_set_error("attention_tcgen05: cuTensorMapEncodeTiled failed");
        return THN_BAD_ARGUMENT;
    }
    dim3 grid(n_q, n_tiles);
    thn_launch(attention_tcgen05_kernel, grid, kThreads, kSmemBytes, stream, map_q, map_kv, (__nv_bfloat16*)out,
               tile_row0, tile_rows, row_slot, row_pos, block_table, bt_stride, n_kv, n_q, scale * kLog2e, window, err);
    return thn_launch_status("attention_tcgen05");
}
