// Weight-streaming matrix product for single-token steps on Blackwell's TMA and fifth-generation
// tensor cores: out[M, N] = x[M, K] @ W[N, K]^T with few rows (M <= 64), bfloat16 operands,
// float32 accumulation in tensor memory.  The reference calls a library product here
// (engine/engine.py:341-350) and closed its own attempt at this kernel
// (engine/kernels/gemm.py:49-136).
//
// At these sizes the product is bound by reading W once from HBM and lasts a few
// microseconds, so everything serves to have many bytes of W in flight early:
//
//  * The operands are swapped: 128 rows of W are the 128-row operand of tcgen05.mma and the
//    few rows of x its narrow one (N = 16, 32 or 64), so no tensor-core row is padding.
//  * The work is the tile-major sequence of (128 rows of W) x (64 of K) units, cut into one
//    equal run per block, one block per SM: every SM streams the same number of bytes whatever
//    the shape.  A tile that several blocks share gets float32 partials in scratch memory; the
//    warp that arrives last (one counter per tile and lane quarter) adds them in ascending k
//    order and stores.  Nobody waits for anybody.
//  * One thread feeds a ring of stages by TMA (128-byte swizzle); the loads of W for the
//    first stages are issued before the kernel waits for its predecessor in the stream (the
//    weights do not depend on it), only x waits.  One thread issues the products; four warps
//    read the accumulator (thread = row of W) and store it transposed, coalesced along N.
//
// SwiGLU mode: W is [2 * N, K] = cat(gate, up).  A stage holds the gate tile and the up tile
// of the same output features; they accumulate side by side in tensor memory, and the
// epilogue stores rnd(rnd(silu(g)) * u) with g and u first rounded to bfloat16, as the
// separate product and engine/kernels/torch_ref.py:74-88 would have done.
//
// Every wait on an mbarrier is bounded by the global timer; on expiry the block sets
// THN_ERR_WAIT_TIMEOUT in the caller's error word, stops its other warps, frees its tensor
// memory and returns.  No wait depends on another block.
#include <cuda.h>

#include "common.cuh"

namespace {

constexpr int BW = 128, BK = 64, UMMA_K = 16;
constexpr int kThreads = 192;                         // warp 0: TMA, warp 1: MMA + TMEM, warps 2-5: epilogue
constexpr uint32_t kWBytes = BW * BK * 2;
constexpr size_t kSmemBudget = 200 * 1024;
constexpr int kMaxStages = 12;
constexpr unsigned long long kWaitLimitNs = 20ull * 1000 * 1000;   // a wait gives up after 20 ms

template <int NX, int SWIGLU>
struct Shape {
    static constexpr uint32_t kXBytes = NX * BK * 2;
    static constexpr uint32_t kStageBytes = kWBytes * (1 + SWIGLU) + kXBytes;
    static constexpr int kStages =
        (int)(kSmemBudget / kStageBytes) < kMaxStages ? (int)(kSmemBudget / kStageBytes) : kMaxStages;
    static constexpr int kAccCols = NX * (1 + SWIGLU);          // one accumulator
    static constexpr int kTmemCols = 2 * kAccCols < 32 ? 32 : 2 * kAccCols;   // two of them; a power of two
    static constexpr size_t kSmemBytes = (size_t)kStages * kStageBytes + 1024 /* alignment */ + 512 /* barriers */;
    // kind::f16: D float32 (bit 4), A and B bfloat16 (bits 7, 10), both K-major, N / 8 at bit 17, M / 16 at bit 24
    static constexpr uint32_t kInstrDesc =
        (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NX >> 3) << 17) | ((uint32_t)(BW >> 4) << 24);
};

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
// Bounded wait for the phase with the given parity: the thread is parked by the hardware for
// up to a microsecond per attempt, and the global timer ends the wait.  False: gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_addr(bar);
    unsigned long long start = 0;
    for (int spin = 0;; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(done)
            : "r"(addr), "r"(parity), "r"(1000)
            : "memory");
        if (done) return true;
        if ((spin & 7) == 7) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
            if (start == 0) start = now;
            else if (now - start > kWaitLimitNs) return false;
        }
    }
}
// The same without parking: for the two single threads that feed the ring and issue the
// products, whose every wait stands between HBM and the tensor core.
__device__ __forceinline__ bool mbar_wait_spin(uint64_t* bar, uint32_t parity) {
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
        if ((spin & 63) == 63) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
            if (start == 0) start = now;
            else if (now - start > kWaitLimitNs) return false;
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
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}
// 16 consecutive columns of this warp's 32 lanes; the caller waits with tmem_wait_load().
__device__ __forceinline__ void tmem_load_16(uint32_t taddr, float* r) {
    uint32_t v[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) r[i] = __uint_as_float(v[i]);
}
__device__ __forceinline__ void tmem_wait_load() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// A block's run [u_begin, u_end) of the tile-major unit sequence, as segments: the part of the
// run that lies in one tile, chunks [c0, c1) of it.  The run is worked through in the order
// last tile, first tile, tiles between: the two ends are the tiles that other blocks may
// share, and taking them first puts the exchange of partial sums into the middle of the
// kernel instead of its tail.
struct Segment {
    int tile, c0, c1;
};
struct Run {
    long long u_begin, u_end;
    int chunks, t0, n_seg;
    __device__ __forceinline__ Run(long long b, long long e, int ch) : u_begin(b), u_end(e), chunks(ch) {
        t0 = (int)(b / ch);
        n_seg = (int)((e - 1) / ch) - t0 + 1;
    }
    __device__ __forceinline__ Segment at(int k) const {      // k-th segment in working order
        const int i = n_seg < 3 ? k : (k == 0 ? n_seg - 1 : k - 1);
        Segment s;
        s.tile = t0 + i;
        s.c0 = i == 0 ? (int)(u_begin - (long long)t0 * chunks) : 0;
        s.c1 = i == n_seg - 1 ? (int)(u_end - (long long)s.tile * chunks) : chunks;
        return s;
    }
};

// Block b takes units [b * span, (b + 1) * span) of the tile-major sequence.  The partial of a
// shared tile goes to scratch slot 2 b (the tile holds the start of b's run) or 2 b + 1 (the
// run started in an earlier tile): [accumulator column][row of the tile] floats.
// counters: 4 ints per tile (one per lane quarter), zero before the first call and after every call.
template <int NX, int SWIGLU, typename OutT>
__global__ void __launch_bounds__(kThreads, 1) gemm_stream_kernel(
    const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, OutT* __restrict__ out,
    float* __restrict__ scratch, int* __restrict__ counters, int M, int N, int chunks, int span,
    long long total_units, int early_limit, int* __restrict__ err) {
    using S = Shape<NX, SWIGLU>;
    pdl_launch_dependents();
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + (size_t)S::kStages * S::kStageBytes);
    uint64_t* empty = full + S::kStages;
    uint64_t* acc_full = empty + S::kStages;   // [2] accumulator ready for the epilogue
    uint64_t* acc_empty = acc_full + 2;        // [2] accumulator read out
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* give_up = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long u_begin = (long long)blockIdx.x * span;
    const long long u_end = min(u_begin + span, total_units);

    if (warp == 0) {                           // one barrier per lane
        if (lane < S::kStages) mbar_init(full + lane, 1);
        else if (lane < 2 * S::kStages) mbar_init(empty + (lane - S::kStages), 1);
        else if (lane < 2 * S::kStages + 2) mbar_init(acc_full + (lane - 2 * S::kStages), 1);
        else if (lane < 2 * S::kStages + 4) mbar_init(acc_empty + (lane - 2 * S::kStages - 2), 4);   // one arrival per epilogue warp
        if (lane == 0) *give_up = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)),
                     "r"(S::kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
        // ---- TMA producer.  W of the first stages goes out before the wait for the kernel
        // that produces x; x follows after it.
        auto load_w = [&](int s, int tile, int c) {
            unsigned char* dst = tiles + (size_t)s * S::kStageBytes;
            mbar_expect_tx(full + s, S::kStageBytes);
            tma_load_2d(dst, &map_w, full + s, c * BK, tile * BW);
            if (SWIGLU) tma_load_2d(dst + kWBytes, &map_w, full + s, c * BK, N + tile * BW);
        };
        auto load_x = [&](int s, int c) {
            tma_load_2d(tiles + (size_t)s * S::kStageBytes + kWBytes * (1 + SWIGLU), &map_x, full + s, c * BK, 0);
        };
        const Run run(u_begin, u_end, chunks);
        int early_chunk[kMaxStages];
        const int early = min(S::kStages, early_limit);     // W tiles requested before the dependency wait
        int it = 0;
        bool waited = false, ok = true;
        for (int k = 0; k < run.n_seg && ok && !*give_up; ++k) {
            const Segment seg = run.at(k);
            for (int c = seg.c0; c < seg.c1; ++c, ++it) {
                const int s = it % S::kStages;
                if (it < early) {                          // the stage has never been used: no wait
                    load_w(s, seg.tile, c);
                    early_chunk[it] = c;
                    continue;
                }
                if (!waited) {
                    pdl_wait();
                    for (int i = 0; i < early; ++i) load_x(i, early_chunk[i]);
                    waited = true;
                }
                if (!mbar_wait_spin(empty + s, ((it / S::kStages) & 1) ^ 1)) {
                    if (err) atomicOr(err, THN_ERR_WAIT_TIMEOUT);
                    *give_up = 1;
                    ok = false;
                    break;
                }
                load_w(s, seg.tile, c);
                load_x(s, c);
            }
        }
        if (!waited) {
            pdl_wait();
            for (int i = 0; i < it && i < early; ++i) load_x(i, early_chunk[i]);
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer
        pdl_wait();
        int it = 0, local = 0;
        bool ok = true;
        const Run run(u_begin, u_end, chunks);
        for (; local < run.n_seg && ok && !*give_up; ++local) {
            const Segment seg = run.at(local);
            const int buf = local & 1;
            ok = mbar_wait(acc_empty + buf, ((local >> 1) & 1) ^ 1);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t tmem_d = tmem_base + buf * S::kAccCols;
            for (int c = seg.c0; c < seg.c1 && ok; ++c, ++it) {
                const int s = it % S::kStages;
                ok = mbar_wait_spin(full + s, (it / S::kStages) & 1);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t w_addr = smem_addr(tiles + (size_t)s * S::kStageBytes);
                const uint64_t w_desc = smem_desc(w_addr);
                const uint64_t x_desc = smem_desc(w_addr + kWBytes * (1 + SWIGLU));
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k) {    // 32 bytes further along K: + 2 in the address field
                    umma(tmem_d, w_desc + 2 * k, x_desc + 2 * k, S::kInstrDesc, (c != seg.c0) | (k != 0));
                    if (SWIGLU)
                        umma(tmem_d + NX, smem_desc(w_addr + kWBytes) + 2 * k, x_desc + 2 * k, S::kInstrDesc,
                             (c != seg.c0) | (k != 0));
                }
                umma_commit(empty + s);                    // the stage is free when these products are done
            }
            umma_commit(acc_full + buf);
        }
        if (!ok) {
            if (err) atomicOr(err, THN_ERR_WAIT_TIMEOUT);
            *give_up = 1;
        }
    } else if (warp >= 2) {
        // ---- epilogue: warp w owns tensor-memory lanes 32 * (w % 4) .. + 31 = rows of the W tile
        pdl_wait();
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const Run run(u_begin, u_end, chunks);
        for (int local = 0; local < run.n_seg && !*give_up; ++local) {
            const Segment seg = run.at(local);
            const int buf = local & 1;
            if (!__all_sync(0xffffffffu, mbar_wait(acc_full + buf, (local >> 1) & 1))) {      // all lanes together before tcgen05.ld
                if (lane == 0 && err) atomicOr(err, THN_ERR_WAIT_TIMEOUT);
                *give_up = 1;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float acc[S::kAccCols];
            const uint32_t taddr = tmem_base + buf * S::kAccCols + ((uint32_t)(quarter * 32) << 16);
#pragma unroll
            for (int c = 0; c < S::kAccCols; c += 16) tmem_load_16(taddr + c, acc + c);
            tmem_wait_load();
            // the accumulator is in registers: hand it back to the MMA thread
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty + buf);

            const long long tile_first = (long long)seg.tile * chunks;
            const int first_block = (int)(tile_first / span);
            const int touching = (int)((tile_first + chunks - 1) / span) - first_block + 1;
            bool finish = touching == 1;
            if (!finish) {
                const size_t slot_floats = (size_t)S::kAccCols * BW;
                const bool head = u_begin >= tile_first;
                float* mine = scratch + ((size_t)blockIdx.x * 2 + (head ? 0 : 1)) * slot_floats;
#pragma unroll
                for (int j = 0; j < S::kAccCols; ++j)
                    if ((j % NX) < M) __stcg(mine + (size_t)j * BW + r, acc[j]);
                __threadfence();
                __syncwarp();
                int arrived = 0;
                if (lane == 0) arrived = atomicAdd(counters + seg.tile * 4 + quarter, 1);
                arrived = __shfl_sync(0xffffffffu, arrived, 0);
                if (arrived == touching - 1) {             // every other partial of these rows is complete
                    __threadfence();
                    if (lane == 0) counters[seg.tile * 4 + quarter] = 0;     // ready for the next call
                    // ascending block = ascending k, sixteen columns at a time
#pragma unroll
                    for (int j0 = 0; j0 < S::kAccCols; j0 += 16) {
                        float sum[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) sum[j] = 0.f;
#pragma unroll 2
                        for (int b = first_block; b < first_block + touching; ++b) {
                            const bool b_head = (long long)b * span >= tile_first;
                            const float* part = scratch + ((size_t)b * 2 + (b_head ? 0 : 1)) * slot_floats;
                            float v[16];
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                v[j] = ((j0 + j) % NX) < M ? __ldcg(part + (size_t)(j0 + j) * BW + r) : 0.f;
#pragma unroll
                            for (int j = 0; j < 16; ++j) sum[j] += v[j];
                        }
#pragma unroll
                        for (int j = 0; j < 16; ++j) acc[j0 + j] = sum[j];
                    }
                    finish = true;
                }
            }
            if (finish) {
                const int n = seg.tile * BW + r;
                if (n < N) {
#pragma unroll
                    for (int j = 0; j < NX; ++j) {
                        if (j < M) {
                            float v = acc[j];
                            if (SWIGLU) {
                                const float g = rnd<__nv_bfloat16>(v);
                                const float up = rnd<__nv_bfloat16>(acc[NX + j]);
                                v = rnd<__nv_bfloat16>(g / (1.0f + expf(-g))) * up;
                            }
                            out[(size_t)j * N + n] = from_f32<OutT>(v);
                        }
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(S::kTmemCols) : "memory");
    }
}

// Few tiles (N small against the number of SMs): every tile is cut along K among the blocks
// of one thread-block cluster, one tile per cluster, and the partial sums meet in distributed
// shared memory instead of global memory: block q of the cluster owns the columns j = q,
// q + cluster size, ...; every block writes its partial of a column into the owner's shared
// memory (a region of its own, beside the stages, since the owner may still be streaming),
// the cluster's hardware barrier orders it, and the owner adds the partials in ascending k
// order and stores.  After the barrier nobody touches another block's memory, so a block
// may leave as soon as it has stored.
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_size() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}
// *mine as it lies in block `rank` of the cluster <- v
__device__ __forceinline__ void store_to_block(float* mine, uint32_t rank, float v) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_addr(mine)), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}

// Stages of the cluster kernel: the shared-memory budget less the region that receives the
// other blocks' partials, [own column][sending block][row], at most NX + 8 x 128 floats.
template <int NX>
struct ClusterShape {
    static constexpr int kRecvFloats = (NX + 8) * BW;
    static constexpr int kStages =
        (int)((kSmemBudget - kRecvFloats * 4) / Shape<NX, 0>::kStageBytes) < kMaxStages
            ? (int)((kSmemBudget - kRecvFloats * 4) / Shape<NX, 0>::kStageBytes) : kMaxStages;
    static constexpr size_t kSmemBytes =
        (size_t)kStages * Shape<NX, 0>::kStageBytes + kRecvFloats * 4 + 1024 /* alignment */ + 512 /* barriers */;
};

template <int NX, typename OutT>
__global__ void __launch_bounds__(kThreads, 1) gemm_stream_cluster_kernel(
    const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, OutT* __restrict__ out,
    int M, int N, int chunks, int early_limit, int* __restrict__ err) {
    using S = Shape<NX, 0>;
    constexpr int kStages = ClusterShape<NX>::kStages;
    pdl_launch_dependents();
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    float* recv = reinterpret_cast<float*>(tiles + (size_t)kStages * S::kStageBytes);
    uint64_t* full = reinterpret_cast<uint64_t*>(recv + ClusterShape<NX>::kRecvFloats);
    uint64_t* empty = full + kStages;
    uint64_t* acc_full = empty + kStages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
    volatile int* give_up = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = (int)cluster_rank(), n_ranks = (int)cluster_size();
    const int tile = blockIdx.x / n_ranks;
    const int c0 = (int)((long long)chunks * rank / n_ranks), c1 = (int)((long long)chunks * (rank + 1) / n_ranks);

    if (warp == 0) {                           // one barrier per lane
        if (lane < kStages) mbar_init(full + lane, 1);
        else if (lane < 2 * kStages) mbar_init(empty + (lane - kStages), 1);
        else if (lane == 2 * kStages) mbar_init(acc_full, 1);
        if (lane == 0) *give_up = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)),
                     "r"(S::kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
        // ---- TMA producer: W of the first stages before the wait for the kernel that makes x
        auto load_w = [&](int s, int c) {
            mbar_expect_tx(full + s, S::kStageBytes);
            tma_load_2d(tiles + (size_t)s * S::kStageBytes, &map_w, full + s, c * BK, tile * BW);
        };
        auto load_x = [&](int s, int c) {
            tma_load_2d(tiles + (size_t)s * S::kStageBytes + kWBytes, &map_x, full + s, c * BK, 0);
        };
        // (not all stages: the TMA unit works its queue in order, about 32 bytes a clock, and the
        // first x tile would wait behind every W tile requested here)
        const int early = min(min(kStages, early_limit), c1 - c0);
        for (int i = 0; i < early; ++i) load_w(i, c0 + i);
        pdl_wait();
        for (int i = 0; i < early; ++i) load_x(i, c0 + i);
        int it = early;
        for (int c = c0 + early; c < c1 && !*give_up; ++c, ++it) {
            const int s = it % kStages;
            if (!mbar_wait_spin(empty + s, ((it / kStages) & 1) ^ 1)) {
                if (err) atomicOr(err, THN_ERR_WAIT_TIMEOUT);
                *give_up = 1;
                break;
            }
            load_w(s, c);
            load_x(s, c);
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer
        bool ok = true;
        int it = 0;
        for (int c = c0; c < c1 && ok && !*give_up; ++c, ++it) {
            const int s = it % kStages;
            ok = mbar_wait_spin(full + s, (it / kStages) & 1);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t w_addr = smem_addr(tiles + (size_t)s * S::kStageBytes);
            const uint64_t w_desc = smem_desc(w_addr), x_desc = smem_desc(w_addr + kWBytes);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)
                umma(tmem_base, w_desc + 2 * k, x_desc + 2 * k, S::kInstrDesc, (c != c0) | (k != 0));
            umma_commit(empty + s);
        }
        umma_commit(acc_full);
        if (!ok) {
            if (err) atomicOr(err, THN_ERR_WAIT_TIMEOUT);
            *give_up = 1;
        }
    } else if (warp >= 2) {
        // ---- epilogue, first half: this block's partial, column by column, to the columns' owners
        pdl_wait();
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        float acc[NX];
#pragma unroll
        for (int j = 0; j < NX; ++j) acc[j] = 0.f;
        if (c1 > c0) {
            if (__all_sync(0xffffffffu, mbar_wait(acc_full, 0))) {      // all lanes together before tcgen05.ld
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16);
#pragma unroll
                for (int c = 0; c < NX; c += 16) tmem_load_16(taddr + c, acc + c);
                tmem_wait_load();
            } else {
                if (lane == 0 && err) atomicOr(err, THN_ERR_WAIT_TIMEOUT);
                *give_up = 1;
            }
        }
        // column j goes to block j % n_ranks, as that block's column j / n_ranks, sender `rank`
        int owner = 0, slot = rank;                 // slot = (j / n_ranks) * n_ranks + rank, kept without divisions
#pragma unroll
        for (int j = 0; j < NX; ++j) {
            if (j < M) store_to_block(recv + slot * BW + r, (uint32_t)owner, acc[j]);
            if (++owner == n_ranks) {
                owner = 0;
                slot += n_ranks;
            }
        }
    }
    cluster_sync();
    if (warp >= 2) {
        // ---- epilogue, second half: this block's columns, partials added in ascending k order
        const int r = (warp & 3) * 32 + lane;
        const int n = tile * BW + r;
        for (int j = rank, jl = 0; j < M; j += n_ranks, ++jl) {
            float v[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) v[q] = q < n_ranks ? recv[(jl * n_ranks + q) * BW + r] : 0.f;
            float sum = 0.f;
#pragma unroll
            for (int q = 0; q < 8; ++q) sum += v[q];
            if (n < N) out[(size_t)j * N + n] = from_f32<OutT>(sum);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(S::kTmemCols) : "memory");
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

// A row-major [rows, K] bfloat16 matrix as a 2-D tensor map with boxes of 64 k x box_rows;
// what a box covers beyond the matrix reads as zero.
bool make_map(CUtensorMap* map, const void* base, long long rows, int K, int box_rows) {
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

// Measured on the decode step (2.378 ms with all 11 stages requested early, 2.313 ms with 2 or 3).
int g_stream_early = 3;

int sm_count() {
    static int n_sms = 0;
    if (n_sms == 0) {
        int device = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, device);
        if (n_sms <= 0) n_sms = 1;
    }
    return n_sms;
}

int padded_rows(int M) { return M <= 16 ? 16 : M <= 32 ? 32 : 64; }

struct Plan {
    int chunks, span, blocks;
    long long units;
};

Plan plan_for(int N, int K, int n_blocks) {
    Plan p;
    p.chunks = (K + BK - 1) / BK;
    p.units = (long long)((N + BW - 1) / BW) * p.chunks;
    if (n_blocks <= 0) n_blocks = sm_count();
    p.span = (int)((p.units + n_blocks - 1) / n_blocks);
    if (p.span < 1) p.span = 1;
    p.blocks = (int)((p.units + p.span - 1) / p.span);
    return p;
}

template <int NX, int SWIGLU, typename OutT>
int launch(const CUtensorMap& map_w, const CUtensorMap& map_x, void* out, float* scratch, int* counters, int M, int N,
           const Plan& p, int* err, cudaStream_t stream) {
    using S = Shape<NX, SWIGLU>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_stream_kernel<NX, SWIGLU, OutT>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)S::kSmemBytes);
        if (e != cudaSuccess) {
            thn_set_error("gemm_stream: cannot reserve %zu bytes of shared memory: %s", S::kSmemBytes,
                          cudaGetErrorString(e));
            return (int)e;
        }
        configured = true;
    }
    thn_launch(gemm_stream_kernel<NX, SWIGLU, OutT>, (unsigned)p.blocks, kThreads, S::kSmemBytes, stream, map_w, map_x,
               (OutT*)out, scratch, counters, M, N, p.chunks, p.span, p.units, g_stream_early, err);
    return thn_launch_status("gemm_stream");
}

// The largest cluster size (2 to 8) of which n_tiles clusters are resident at once, or 0.
template <int NX, typename OutT>
int cluster_size_for(int n_tiles) {
    using S = Shape<NX, 0>;
    static int resident[9] = {-1, -1, -1, -1, -1, -1, -1, -1, -1};     // clusters of each size that fit
    if (resident[0] < 0) {
        resident[0] = 0;
        if (cudaFuncSetAttribute(gemm_stream_cluster_kernel<NX, OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)ClusterShape<NX>::kSmemBytes) != cudaSuccess) {
            cudaGetLastError();
            for (int c = 1; c <= 8; ++c) resident[c] = 0;
        }
    }
    for (int c = 8; c >= 2; --c) {
        if (resident[c] < 0) {
            cudaLaunchConfig_t config = {};
            config.gridDim = dim3((unsigned)(c * 64));
            config.blockDim = dim3(kThreads);
            config.dynamicSmemBytes = ClusterShape<NX>::kSmemBytes;
            cudaLaunchAttribute attribute[1];
            attribute[0].id = cudaLaunchAttributeClusterDimension;
            attribute[0].val.clusterDim.x = (unsigned)c;
            attribute[0].val.clusterDim.y = 1;
            attribute[0].val.clusterDim.z = 1;
            config.attrs = attribute;
            config.numAttrs = 1;
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, gemm_stream_cluster_kernel<NX, OutT>, &config) != cudaSuccess) {
                cudaGetLastError();
                n = 0;
            }
            resident[c] = n;
        }
        if (resident[c] >= n_tiles) return c;
    }
    return 0;
}

template <int NX, typename OutT>
int launch_cluster(const CUtensorMap& map_w, const CUtensorMap& map_x, void* out, int M, int N, int chunks, int n_tiles,
                   int c, int* err, cudaStream_t stream) {
    using S = Shape<NX, 0>;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((unsigned)(n_tiles * c));
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = ClusterShape<NX>::kSmemBytes;
    config.stream = stream;
    cudaLaunchAttribute attribute[2];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = (unsigned)c;
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = 1;
    attribute[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = g_thn_pdl ? 2 : 1;
    cudaLaunchKernelEx(&config, gemm_stream_cluster_kernel<NX, OutT>, map_w, map_x, (OutT*)out, M, N, chunks,
                       g_stream_early, err);
    return thn_launch_status("gemm_stream (cluster)");
}

// The cluster size to use for a shape: n_blocks < 0 asks for exactly -n_blocks (tests);
// n_blocks == 0 takes the largest that keeps every tile's cluster resident, if the tiles are
// few enough to need the split (fewer than half the SMs) and the blocks many enough to
// stream at full rate; 0: the balanced runs through global memory.
template <int NX, typename OutT>
int choose_cluster(int n_tiles, int chunks, int n_blocks) {
    if (n_blocks > 0) return 0;
    const int best = cluster_size_for<NX, OutT>(n_tiles);
    if (n_blocks < 0) return (-n_blocks >= 2 && -n_blocks <= best) ? -n_blocks : 0;
    if (best < 2 || n_tiles * 2 > sm_count() || n_tiles * best * 3 < sm_count() * 2 || chunks < best) return 0;
    return best;
}

}  // namespace

// How many stages of W a block requests before it waits for the kernel that produces x.
THN_API void thn_set_stream_early(int stages) { g_stream_early = stages < 1 ? 1 : stages; }

// 1 if thn_gemm_stream_bf16 takes this shape: at most 64 rows, K a multiple of 8 (TMA wants
// 16-byte row strides).
THN_API int thn_gemm_stream_supported(int M, int N, int K) { return M >= 1 && M <= 64 && N >= 1 && K >= 8 && K % 8 == 0; }

// What a call needs: *scratch_floats of float32 scratch and *n_counters ints (zero before the
// first call; the kernel leaves them zero).  n_blocks <= 0: one block per SM.
THN_API int thn_gemm_stream_scratch(int M, int N, int K, int swiglu, int n_blocks, long long* scratch_floats,
                                    int* n_counters) {
    const Plan p = plan_for(N, K, n_blocks > 0 ? n_blocks : 0);
    *scratch_floats = (long long)p.blocks * 2 * padded_rows(M) * (swiglu ? 2 : 1) * BW;
    *n_counters = 4 * ((N + BW - 1) / BW);
    return THN_OK;
}

// out [M, N] (bfloat16, or float32 with out_dtype THN_F32) = x [M, K] @ w [N, K]^T; with
// swiglu != 0, w is [2 * N, K] (gate rows, then up rows) and out = silu(x gate^T) * (x up^T).
// scratch and counters as thn_gemm_stream_scratch says.  All pointers 16-byte aligned.
// n_blocks: 0 lets the library choose between balanced runs on every SM and one cluster per
// tile; > 0 cuts balanced runs for that many blocks; < 0 asks for clusters of -n_blocks.
// err: device error word (THN_ERR_WAIT_TIMEOUT if a pipeline wait gave up).
THN_API int thn_gemm_stream_bf16(void* out, int out_dtype, float* scratch, int* counters, const void* x, const void* w,
                                 int M, int N, int K, int swiglu, int n_blocks, int* err, cudaStream_t stream) {
    THN_UNSUPPORTED_IF(!thn_gemm_stream_supported(M, N, K), "gemm_stream: shape M=%d N=%d K=%d not supported "
                       "(1 <= M <= 64, K a multiple of 8)", M, N, K);
    THN_CHECK_ARG((((uintptr_t)x | (uintptr_t)w | (uintptr_t)out | (uintptr_t)scratch) & 15) == 0,
                  "gemm_stream: operands must be 16-byte aligned");
    THN_CHECK_ARG(out_dtype == THN_F32 || out_dtype == THN_BF16, "gemm_stream: unknown output dtype %d", out_dtype);
    THN_CHECK_ARG(scratch != nullptr && counters != nullptr, "gemm_stream: scratch and counters, please");
    THN_UNSUPPORTED_IF(swiglu && out_dtype != THN_BF16, "gemm_stream: fused SwiGLU stores bfloat16 only");
    const Plan p = plan_for(N, K, n_blocks > 0 ? n_blocks : 0);
    const int nx = padded_rows(M);
    CUtensorMap map_w, map_x;
    if (!make_map(&map_w, w, swiglu ? 2LL * N : N, K, BW) || !make_map(&map_x, x, M, K, nx)) {
        thn_set_error("gemm_stream: cuTensorMapEncodeTiled failed for M=%d N=%d K=%d", M, N, K);
        return THN_BAD_ARGUMENT;
    }
    const int n_tiles = (N + BW - 1) / BW;
#define CLUSTER(NX, OutT)                                                                                           \
    do {                                                                                                            \
        const int c = choose_cluster<NX, OutT>(n_tiles, p.chunks, n_blocks);                                        \
        if (c) return launch_cluster<NX, OutT>(map_w, map_x, out, M, N, p.chunks, n_tiles, c, err, stream);         \
    } while (0)
#define GO(NX)                                                                                                      \
    do {                                                                                                            \
        if (swiglu) return launch<NX, 1, __nv_bfloat16>(map_w, map_x, out, scratch, counters, M, N, p, err, stream); \
        if (out_dtype == THN_BF16) CLUSTER(NX, __nv_bfloat16);                                                      \
        else CLUSTER(NX, float);                                                                                    \
        if (out_dtype == THN_BF16)                                                                                  \
            return launch<NX, 0, __nv_bfloat16>(map_w, map_x, out, scratch, counters, M, N, p, err, stream);        \
        return launch<NX, 0, float>(map_w, map_x, out, scratch, counters, M, N, p, err, stream);                    \
    } while (0)
    if (nx == 16) GO(16);
    if (nx == 32) GO(32);
    GO(64);
#undef GO
#undef CLUSTER
}
