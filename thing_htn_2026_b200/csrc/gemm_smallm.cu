// Weight-streaming matrix product for decode steps: out[M, N] = x[M, K] @ W[N, K]^T with
// few rows (M <= 16), bfloat16 operands, float32 accumulation.  At these sizes the product
// is bound by reading W once from HBM and a call lasts only a few microseconds, so the
// kernel is built to get every byte in flight at once: the work is cut into (16 rows of W)
// x (slice of K) items, one per warp, about as many as the GPU has warp slots; a warp reads
// whole 128-byte lines of its rows straight into tensor-core fragments (no shared memory,
// no block-wide synchronisation) with several lines per row in flight.  The items are cut
// from the tile-major sequence of (tile, K chunk) units in equal runs, so every warp of the
// one resident wave carries the same load whatever the shape.
//
// The tensor-core shape is m16n8k16 with W as the 16-row operand and x^T as the 8-column
// operand (out^T = W x^T).  The k index inside a fragment is a free permutation as long
// as both operands use the same one, so a lane takes 8 consecutive k (16 bytes) of its
// row per load instead of the scattered pairs of the canonical layout, and the four lanes
// of a row cover 64 contiguous bytes.
//
// A tile whose chunks are shared by several warps gets one float32 partial slab per warp in
// scratch memory.  Each warp counts itself in on the tile when its slab is written; the warp
// that arrives last adds the slabs in ascending k order (so the result does not depend on
// who was last) and stores the tile, rounded once to bfloat16 where the reference's library
// product would have rounded (engine/engine.py:341-350), or as float32 for logits.  Nobody
// waits for anybody.
//
// The reference's own attempt at this kernel is engine/kernels/gemm.py:49-136 (closed
// there); its library call is what this replaces on the decode path.
#include "common.cuh"

namespace {

constexpr int kWarps = 4;
constexpr int kChunk = 64;   // k per row per step: one 128-byte line
constexpr int kUnroll = 4;   // lines per row in flight
constexpr int kMaxSlabs = 8;    // at most this many warps share a tile
constexpr int kMinBlocks = 4;   // register budget: ptxas keeps every load of a group in flight only if told so

__device__ __forceinline__ uint4 load_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t word(const uint4 (&v)[2], int i) {
    const uint4& q = v[i >> 2];
    switch (i & 3) {
        case 0: return q.x;
        case 1: return q.y;
        case 2: return q.z;
        default: return q.w;
    }
}

// U chunks of one tile: every load is issued before the first product, without
// predicates (rows past N or M read a valid row instead and are dropped at the store).
template <int MT, int U>
__device__ __forceinline__ void run_chunks(float (&acc)[MT][4], const __nv_bfloat16* w0, const __nv_bfloat16* w1,
                                           const __nv_bfloat16* const (&xr)[MT], int k0) {
    uint4 wv[U][2][2];
    uint4 xv[U][MT][2];
#pragma unroll
    for (int v = 0; v < U; ++v) {
        wv[v][0][0] = load_stream(w0 + k0 + v * kChunk);
        wv[v][0][1] = load_stream(w0 + k0 + v * kChunk + 32);
        wv[v][1][0] = load_stream(w1 + k0 + v * kChunk);
        wv[v][1][1] = load_stream(w1 + k0 + v * kChunk + 32);
    }
#pragma unroll
    for (int v = 0; v < U; ++v)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            xv[v][mt][0] = __ldg(reinterpret_cast<const uint4*>(xr[mt] + k0 + v * kChunk));
            xv[v][mt][1] = __ldg(reinterpret_cast<const uint4*>(xr[mt] + k0 + v * kChunk + 32));
        }
#pragma unroll
    for (int v = 0; v < U; ++v)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
                mma_bf16(acc[mt], word(wv[v][0], 2 * j), word(wv[v][1], 2 * j), word(wv[v][0], 2 * j + 1),
                         word(wv[v][1], 2 * j + 1), word(xv[v][mt], 2 * j), word(xv[v][mt], 2 * j + 1));
}

// MT: 8-row tiles of x (M <= 8 * MT).  The work is the sequence of (tile of 16 W rows,
// 64-wide chunk of K) units, tile-major; warp i of the grid takes units [i * span,
// (i + 1) * span), so all warps carry the same load whatever the shape.
// Within a chunk lane t of a row holds k = 8t .. 8t+7 and 32+8t .. 32+8t+7.
template <int MT, typename OutT>
__global__ void __launch_bounds__(kWarps * 32, MT == 1 ? kMinBlocks : kMinBlocks - 1) gemm_smallm_kernel(
    OutT* __restrict__ out, float* __restrict__ slabs, int* __restrict__ counters,
    const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, int M, int N, int K, int chunks,
    int span, long long total_units, int prefetch) {
    const int lane = threadIdx.x & 31;
    const long long warp_global = (long long)blockIdx.x * kWarps + (threadIdx.x >> 5);
    long long u = warp_global * span;
    const long long u_end = min(u + span, total_units);
    const int g = lane >> 2, t = lane & 3;
    const size_t slab_stride = (size_t)M * N;

    // While the kernel that produces x is still running, pull this warp's stretch of W
    // towards L2: one 128-byte line per instruction, 16 rows x 2 lines per warp step.
    pdl_launch_dependents();
    for (long long pu = u; prefetch && pu < u_end;) {
        const int tile = (int)(pu / chunks);
        const int c0 = (int)(pu - (long long)tile * chunks);
        const int c1 = (int)min((long long)chunks, c0 + (u_end - pu));
        const int row = tile * 16 + (lane & 15);
        if (row < N)
            for (int c = c0 + (lane >> 4); c < c1; c += 2)
                asm volatile("prefetch.global.L2 [%0];" ::"l"(w + (size_t)row * K + (size_t)c * kChunk));
        pu += c1 - c0;
    }
    pdl_wait();

    const __nv_bfloat16* xr[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) xr[mt] = x + (size_t)(mt * 8 + g < M ? mt * 8 + g : 0) * K + 8 * t;

    while (u < u_end) {
        const int tile = (int)(u / chunks);
        const int c0 = (int)(u - (long long)tile * chunks);
        const int c1 = (int)min((long long)chunks, c0 + (u_end - u));
        const int n0 = tile * 16;
        const bool live0 = n0 + g < N, live1 = n0 + g + 8 < N;
        const __nv_bfloat16* w0 = w + (size_t)(live0 ? n0 + g : 0) * K + 8 * t;
        const __nv_bfloat16* w1 = w + (size_t)(live1 ? n0 + g + 8 : 0) * K + 8 * t;

        float acc[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[mt][i] = 0.f;

        int chunk = c0;
        for (; chunk + kUnroll <= c1; chunk += kUnroll) run_chunks<MT, kUnroll>(acc, w0, w1, xr, chunk * kChunk);
        for (; chunk < c1; ++chunk) run_chunks<MT, 1>(acc, w0, w1, xr, chunk * kChunk);

        // Fragment element i of x-tile mt: W row n0 + g + 8 * (i / 2), x row mt * 8 + 2t + (i % 2).
        const long long tile_first = (long long)tile * chunks;
        const int first_warp = (int)(tile_first / span);
        const int touching = (int)((tile_first + chunks - 1) / span) - first_warp + 1;
        bool finish = touching == 1;
        if (!finish) {
            float* mine = slabs + (size_t)(warp_global - first_warp) * slab_stride;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int m = mt * 8 + 2 * t + (i & 1), n = n0 + g + 8 * (i >> 1);
                    if (m < M && n < N) __stcg(mine + (size_t)m * N + n, acc[mt][i]);
                }
            __threadfence();
            __syncwarp();
            int arrived = 0;
            if (lane == 0) arrived = atomicAdd(counters + tile, 1);
            arrived = __shfl_sync(0xffffffffu, arrived, 0);
            if (arrived == touching - 1) {          // every other slab of this tile is complete
                __threadfence();
                if (lane == 0) counters[tile] = 0;  // ready for the next call
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int m = mt * 8 + 2 * t + (i & 1), n = n0 + g + 8 * (i >> 1);
                        float v[kMaxSlabs];
#pragma unroll
                        for (int sl = 0; sl < kMaxSlabs; ++sl)
                            v[sl] = (sl < touching && m < M && n < N)
                                        ? __ldcg(slabs + (size_t)sl * slab_stride + (size_t)m * N + n) : 0.f;
                        float sum = 0.f;
#pragma unroll
                        for (int sl = 0; sl < kMaxSlabs; ++sl) sum += v[sl];
                        acc[mt][i] = sum;
                    }
                finish = true;
            }
        }
        if (finish) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int m = mt * 8 + 2 * t + (i & 1), n = n0 + g + 8 * (i >> 1);
                    if (m < M && n < N) out[(size_t)m * N + n] = from_f32<OutT>(acc[mt][i]);
                }
        }
        u += c1 - c0;
    }
}

template <int MT>
int resident_warps(int n_sms) {
    int blocks = 0;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, gemm_smallm_kernel<MT, __nv_bfloat16>,
                                                                  kWarps * 32, 0);
    if (e != cudaSuccess || blocks < 1) blocks = 1;
    return blocks * kWarps * n_sms;
}

}  // namespace

constexpr int kSmallMMax = 16;
int g_thn_prefetch = 1;

// 1 (default): the product prefetches its weights towards L2 before it waits for its input.
THN_API void thn_set_weight_prefetch(int enabled) { g_thn_prefetch = enabled ? 1 : 0; }


// 1 if thn_gemm_smallm_bf16 takes this shape.
THN_API int thn_gemm_smallm_supported(int M, int N, int K) {
    return M >= 1 && M <= kSmallMMax && N >= 1 && K >= kChunk && K % kChunk == 0;
}

// The schedule for a shape: units per warp (*span_out) and, as the return value, the number
// of float32 slabs [M, N] of scratch the call needs (0: no tile is shared, no scratch).
// n_warps <= 0 asks for as many warps as the GPU holds at once for this kernel.
THN_API int thn_gemm_smallm_plan(int M, int N, int K, int n_sms, int n_warps, int* span_out) {
    const int chunks = K / kChunk;
    const long long tiles = (N + 15) / 16;
    const long long units = tiles * chunks;
    if (n_warps <= 0) n_warps = M <= 8 ? resident_warps<1>(n_sms) : resident_warps<2>(n_sms);
    long long span = (units + n_warps - 1) / n_warps;
    if (span < 2 && chunks >= 2) span = 2;
    // at most kMaxSlabs warps share a tile
    if (span < (chunks + kMaxSlabs - 2) / (kMaxSlabs - 1)) span = (chunks + kMaxSlabs - 2) / (kMaxSlabs - 1);
    int slabs = 1;
    for (long long j = 0; j < tiles; ++j) {
        const long long first = (j * chunks) / span, last = ((j + 1) * chunks - 1) / span;
        if (last - first + 1 > slabs) slabs = (int)(last - first + 1);
    }
    *span_out = (int)span;
    return slabs > 1 ? slabs : 0;
}

// out [M, N] (bfloat16, or float32 with out_dtype THN_F32) = x [M, K] @ w [N, K]^T.  span
// and n_slabs come from thn_gemm_smallm_plan.  slabs: n_slabs * M * N floats of scratch
// (may be null when n_slabs == 0).  counters: one int per 16 rows of w, zero before the
// first call; the kernel leaves them zero.  Operands 16-byte aligned, K a multiple of 64.
THN_API int thn_gemm_smallm_bf16(void* out, int out_dtype, float* slabs, int* counters, const void* x, const void* w,
                                 int M, int N, int K, int span, int n_slabs, cudaStream_t stream) {
    THN_UNSUPPORTED_IF(!thn_gemm_smallm_supported(M, N, K), "gemm_smallm: shape M=%d N=%d K=%d not supported "
                       "(1 <= M <= %d, K a multiple of %d)", M, N, K, kSmallMMax, kChunk);
    THN_CHECK_ARG(span >= 1 && n_slabs >= 0 && n_slabs <= kMaxSlabs, "gemm_smallm: bad schedule span=%d slabs=%d",
                  span, n_slabs);
    THN_CHECK_ARG(n_slabs == 0 || (slabs != nullptr && counters != nullptr),
                  "gemm_smallm: a schedule with shared tiles needs scratch and counters");
    THN_CHECK_ARG((((uintptr_t)x | (uintptr_t)w) & 15) == 0, "gemm_smallm: operands must be 16-byte aligned");
    THN_CHECK_ARG(out_dtype == THN_F32 || out_dtype == THN_BF16, "gemm_smallm: unknown output dtype %d", out_dtype);
    const int chunks = K / kChunk;
    const long long units = (long long)((N + 15) / 16) * chunks;
    {   // the schedule must not let more warps share a tile than the scratch has slabs
        const long long worst = (chunks + span - 1) / span + 1;
        THN_CHECK_ARG(span >= chunks || worst <= (n_slabs > 0 ? kMaxSlabs : 1) + 1,
                      "gemm_smallm: span %d shares a tile among too many warps", span);
    }
    const long long warps = (units + span - 1) / span;
    const unsigned blocks = (unsigned)((warps + kWarps - 1) / kWarps);
    const __nv_bfloat16* xp = (const __nv_bfloat16*)x;
    const __nv_bfloat16* wp = (const __nv_bfloat16*)w;
#define LAUNCH(MT, OutT)                                                                                      \
    thn_launch(gemm_smallm_kernel<MT, OutT>, blocks, kWarps * 32, 0, stream, (OutT*)out, slabs, counters, xp, wp, M, \
                                                                    N, K, chunks, span, units, g_thn_prefetch)
    if (M <= 8 && out_dtype == THN_BF16) LAUNCH(1, __nv_bfloat16);
    else if (M <= 8) LAUNCH(1, float);
    else if (out_dtype == THN_BF16) LAUNCH(2, __nv_bfloat16);
    else LAUNCH(2, float);
#undef LAUNCH
    return thn_launch_status("gemm_smallm");
}
