// Tensor-core attention over the paged cache for bfloat16: a flash kernel for steps that
// bring several tokens per sequence (prompts), and a split-KV kernel with a merge pass for
// single-token steps (flash decoding).  Scores, softmax and the output accumulate in
// float32; the un-normalised probabilities are rounded to bfloat16 before they multiply V
// (engine/kernels/torch_ref.py:219-225).  The reference's counterparts: flash SDPA for
// prompts (engine/engine.py:1123-1131) and engine/kernels/attention.py:115-275 for decode.
//
// Both kernels work on tiles of 64 keys, which is the cache's page size: a tile of one
// head is 64 * head_dim contiguous values.  Tiles reach shared memory with 16-byte
// cp.async copies; rows are padded by 16 bytes so that ldmatrix reads do not collide.
// Instantiated for head sizes 64 and 128; other sizes use the generic kernel.
#include <cuda.h>
#include <math.h>

#include <algorithm>

#include "common.cuh"

namespace {

constexpr int kTile = 64;        // keys per tile == page size
constexpr int kThreads = 128;    // 4 warps (decode)
constexpr int kPrefillRows = 128;                          // query rows per block in the prompt kernel
constexpr int kPrefillThreads = kPrefillRows / 16 * 32;    // one warp per 16 rows
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(smem)), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(smem)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(smem)));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Copies a [rows_total=64][D] tile (contiguous in global memory) into padded shared rows.
template <int D, int THREADS = kThreads>
__device__ __forceinline__ void load_tile_async(__nv_bfloat16* smem, const __nv_bfloat16* gmem) {
    constexpr int kChunksPerRow = D / 8, kPitch = D + 8;
#pragma unroll
    for (int c = threadIdx.x; c < kTile * kChunksPerRow; c += THREADS) {
        const int row = c / kChunksPerRow, col = (c % kChunksPerRow) * 8;
        cp_async16(smem + row * kPitch + col, gmem + row * D + col);
    }
}

// One warp: S[16 x NK*8] = Q[16 x D] K^T for NK key blocks of 8 starting at key_block0.
template <int D, int NK>
__device__ __forceinline__ void qk_tile(float (&s)[NK][4], const uint32_t (&qf)[D / 16][4], const __nv_bfloat16* k_smem,
                                        int key_block0, int lane) {
    constexpr int kPitch = D + 8;
#pragma unroll
    for (int n = 0; n < NK; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) s[n][i] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
        for (int n = 0; n < NK; n += 2) {
            uint32_t b[4];
            const int key = (key_block0 + n + (lane >> 4)) * 8 + (lane & 7);
            ldmatrix_x4(b, k_smem + key * kPitch + kk * 16 + ((lane >> 3) & 1) * 8);
            mma_bf16(s[n], qf[kk], b[0], b[1]);
            mma_bf16(s[n + 1], qf[kk], b[2], b[3]);
        }
    }
}

// One warp: O[16 x D] += P[16 x NK*8] V for the same key blocks.  P comes as bf16 A fragments.
template <int D, int NK>
__device__ __forceinline__ void pv_tile(float (&o)[D / 8][4], const uint32_t (&pf)[NK / 2][4],
                                        const __nv_bfloat16* v_smem, int key_block0, int lane) {
    constexpr int kPitch = D + 8;
#pragma unroll
    for (int kk = 0; kk < NK / 2; ++kk) {
#pragma unroll
        for (int nd = 0; nd < D / 8; nd += 2) {
            uint32_t b[4];
            const int key = (key_block0 + 2 * kk) * 8 + ((lane >> 3) & 1) * 8 + (lane & 7);
            ldmatrix_x4_trans(b, v_smem + key * kPitch + (nd + (lane >> 4)) * 8);
            mma_bf16(o[nd], pf[kk], b[0], b[1]);
            mma_bf16(o[nd + 1], pf[kk], b[2], b[3]);
        }
    }
}

// Online-softmax state of the two rows a thread owns (row g = lane / 4 and row g + 8), in
// the log2 domain.  l holds this thread's share of the row sum until finish().
struct RowState {
    float m[2], l[2];
    __device__ __forceinline__ void init() {
        m[0] = m[1] = -INFINITY;
        l[0] = l[1] = 0.f;
    }
};

// Masks (done by the caller), rescales and exponentiates one S tile in place, produces P
// fragments and rescales O.
template <int D, int NK>
__device__ __forceinline__ void softmax_tile(float (&s)[NK][4], RowState& st, float (&o)[D / 8][4],
                                             uint32_t (&pf)[NK / 2][4]) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float mx = -INFINITY;
#pragma unroll
        for (int n = 0; n < NK; ++n) mx = fmaxf(mx, fmaxf(s[n][2 * r], s[n][2 * r + 1]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(st.m[r], mx);
        const float base = m_new == -INFINITY ? 0.f : m_new;       // a row with no visible key yet
        const float corr = exp2f(st.m[r] - base);                    // exp2(-inf) = 0 on first use
        st.m[r] = m_new;
        float sum = 0.f;
#pragma unroll
        for (int n = 0; n < NK; ++n) {
            s[n][2 * r] = exp2f(s[n][2 * r] - base);
            s[n][2 * r + 1] = exp2f(s[n][2 * r + 1] - base);
            sum += s[n][2 * r] + s[n][2 * r + 1];
        }
        st.l[r] = st.l[r] * corr + sum;
#pragma unroll
        for (int nd = 0; nd < D / 8; ++nd) {
            o[nd][2 * r] *= corr;
            o[nd][2 * r + 1] *= corr;
        }
    }
#pragma unroll
    for (int kk = 0; kk < NK / 2; ++kk) {
        pf[kk][0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        pf[kk][1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        pf[kk][2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        pf[kk][3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
    }
}

// ------------------------------------------------------------------ several tokens per sequence

// One block: kPrefillRows consecutive rows of one sequence (tile_row0 .., clipped to the sequence)
// for one query head; warp w owns rows 16w .. 16w+15.
template <int D>
__global__ void __launch_bounds__(kPrefillThreads) attention_prefill_kernel(
    __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ q, const int* __restrict__ tile_row0,
    const int* __restrict__ tile_rows, const int* __restrict__ row_slot, const int* __restrict__ row_pos, PagedKV kv,
    int n_q, float scale_log2, int window, int* __restrict__ err) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int kPitch = D + 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* q_smem = reinterpret_cast<__nv_bfloat16*>(smem_raw);            // [rows][kPitch]
    __nv_bfloat16* k_smem = q_smem + kPrefillRows * kPitch;                        // [2][64][kPitch]
    __nv_bfloat16* v_smem = k_smem + 2 * kTile * kPitch;                           // [2][64][kPitch]

    // Later tiles of a sequence see more keys and run longer: start them first, so that the
    // short ones fill the end of the grid.
    const int tile = gridDim.y - 1 - blockIdx.y, h = blockIdx.x;
    const int row0 = tile_row0[tile], n_rows = tile_rows[tile];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int kvh = h / (n_q / kv.n_kv);
    const int pos0 = row_pos[row0];                   // rows of a tile are consecutive positions
    const int pos_last = pos0 + n_rows - 1;
    const int* pages = kv.block_table + (size_t)row_slot[row0] * kv.bt_stride;

    // Q tile -> shared (rows past the sequence are zero)
    for (int c = threadIdx.x; c < kPrefillRows * (D / 8); c += kPrefillThreads) {
        const int r = c / (D / 8), col = (c % (D / 8)) * 8;
        if (r < n_rows)
            cp_async16(q_smem + r * kPitch + col, q + ((size_t)(row0 + r) * n_q + h) * D + col);
        else
            *reinterpret_cast<uint4*>(q_smem + r * kPitch + col) = make_uint4(0, 0, 0, 0);
    }
    cp_async_commit();

    int first_key = 0;
    if (window > 0 && pos0 - window + 1 > 0) first_key = pos0 - window + 1;
    const int t_first = first_key / kTile, t_last = pos_last / kTile;

    auto issue = [&](int t, int stage) {
        const int page = pages[t];
        if (page < 0) {
            if (threadIdx.x == 0 && err) atomicOr(err, THN_ERR_PAGE_UNMAPPED);
        } else {
            const __nv_bfloat16* base = (const __nv_bfloat16*)kv.base;
            load_tile_async<D, kPrefillThreads>(k_smem + stage * kTile * kPitch, base + kv_offset(kv, page, 0, kvh, 0));
            load_tile_async<D, kPrefillThreads>(v_smem + stage * kTile * kPitch, base + kv_offset(kv, page, 1, kvh, 0));
        }
        cp_async_commit();
    };
    issue(t_first, 0);

    cp_async_wait<1>();          // Q has landed
    __syncthreads();
    uint32_t qf[D / 16][4];
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk)
        ldmatrix_x4(qf[kk], q_smem + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * kPitch + kk * 16 + (lane >> 4) * 8);

    float o[D / 8][4];
#pragma unroll
    for (int nd = 0; nd < D / 8; ++nd)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[nd][i] = 0.f;
    RowState st;
    st.init();
    const int g = lane >> 2, tq = lane & 3;
    const int my_pos[2] = {pos0 + warp * 16 + g, pos0 + warp * 16 + g + 8};

    for (int t = t_first; t <= t_last; ++t) {
        const int stage = (t - t_first) & 1;
        if (t < t_last) issue(t + 1, stage ^ 1); else cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const int key0 = t * kTile;
        // A warp whose rows all lie before this tile has nothing to see in it.
        const bool warp_active = key0 <= pos0 + warp * 16 + 15;
        if (warp_active) {
            float s[8][4];
            qk_tile<D, 8>(s, qf, k_smem + stage * kTile * kPitch, 0, lane);
            const bool need_mask = key0 + kTile - 1 > pos0 + warp * 16 || (window > 0 && key0 < pos0 + warp * 16 + 15 - window + 1);
#pragma unroll
            for (int n = 0; n < 8; ++n)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float v = s[n][i] * scale_log2;
                    if (need_mask) {
                        const int key = key0 + n * 8 + tq * 2 + (i & 1);
                        const int p = my_pos[i >> 1];
                        if (key > p || (window > 0 && key <= p - window)) v = -INFINITY;
                    }
                    s[n][i] = v;
                }
            uint32_t pf[4][4];
            softmax_tile<D, 8>(s, st, o, pf);
            pv_tile<D, 8>(o, pf, v_smem + stage * kTile * kPitch, 0, lane);
        }
        __syncthreads();
    }

#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float l = st.l[r];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        const int row = warp * 16 + g + 8 * r;
        if (row < n_rows) {
            const float inv = 1.0f / l;
            __nv_bfloat16* dst = out + ((size_t)(row0 + row) * n_q + h) * D;
#pragma unroll
            for (int nd = 0; nd < D / 8; ++nd)
                *reinterpret_cast<uint32_t*>(dst + nd * 8 + tq * 2) = pack_bf16(o[nd][2 * r] * inv, o[nd][2 * r + 1] * inv);
        }
    }
}

// ------------------------------------------------------------------ one token per sequence

// One block: (sequence b, kv head, split).  The G query heads of the kv head are the rows
// of one 16-row tile.  The block walks the 64-key tiles of its split; warp w takes keys
// 16w .. 16w+15 of every tile and keeps its own running state; the four states are merged
// at the end.  With n_splits == 1 the block writes the output; otherwise it writes its
// partial (max, sum, un-normalised output) to scratch.  With counters, each block then counts
// itself in on its (sequence, kv head), and the block that arrives last combines the
// partials in split order (so the result does not depend on who was last) and writes the
// output; nobody waits.  Without counters the merge kernel does it.
// STAGES: tile buffers (2 when a block has few tiles and more blocks per SM matter, 3 when
// one block walks a whole sequence).
//
// FUSED: q is not given; the block takes the step's raw q/k/v rows (the output of the fused
// q/k/v product) and does what the separate kernel of rope_cache.cu does, with the same
// arithmetic (engine/kernels/torch_ref.py:47-58 and :100-117): its query heads are
// normalised and rotated on the way into shared memory, and the block whose keys end with the
// sequence's new position normalises and rotates the new key, copies the new value, writes
// both to the cache and into its own tile.  One kernel less per layer and step.
struct FusedInput {
    const __nv_bfloat16* qkv;    // [n_seqs, (n_q + 2 n_kv) * D]
    const void* q_gain;          // [D] bfloat16, or float32 when gain_f32
    const void* k_gain;
    const float* cos_tab;        // [table_len, D / 2]
    const float* sin_tab;
    float eps;
    int table_len, gain_f32, write_cache;
};

__device__ __forceinline__ float gain_at(const void* gain, int f32, int i) {
    return f32 ? reinterpret_cast<const float*>(gain)[i] : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(gain)[i]);
}

// One head of D values, a lane holding [d0, d0 + E) and [D/2 + d0, ..) of it in registers:
// RMSNorm with gain, then the rotation by the row's angles; every product rounded to bfloat16
// as the reference does.
template <int D>
__device__ __forceinline__ void norm_rotate_head(const __nv_bfloat16 (&in_lo)[D / 64], const __nv_bfloat16 (&in_hi)[D / 64],
                                                 const float (&g_lo)[D / 64], const float (&g_hi)[D / 64], float eps,
                                                 const float (&c)[D / 64], const float (&sn)[D / 64],
                                                 __nv_bfloat16 (&lo)[D / 64], __nv_bfloat16 (&hi)[D / 64]) {
    using B = __nv_bfloat16;
    constexpr int E = D / 64;
    float a[E], b[E], ss = 0.f;
#pragma unroll
    for (int e = 0; e < E; ++e) {
        a[e] = __bfloat162float(in_lo[e]);
        b[e] = __bfloat162float(in_hi[e]);
        ss += a[e] * a[e] + b[e] * b[e];
    }
    ss = warp_sum(ss);
    const float rstd = 1.0f / sqrtf(ss / (float)D + eps);
#pragma unroll
    for (int e = 0; e < E; ++e) {
        const float x0 = rnd<B>(g_lo[e] * rnd<B>(a[e] * rstd));
        const float x1 = rnd<B>(g_hi[e] * rnd<B>(b[e] * rstd));
        lo[e] = __float2bfloat16_rn(rnd<B>(x0 * c[e]) + rnd<B>(-x1 * sn[e]));
        hi[e] = __float2bfloat16_rn(rnd<B>(x1 * c[e]) + rnd<B>(x0 * sn[e]));
    }
}

// CLUSTER: the splits of one (sequence, kv head) are the blocks of one thread-block cluster,
// and their partial results meet in distributed shared memory instead of global memory: after
// a first barrier (every block is done with its tile buffers) each block writes its partial
// into block 0's tile buffers, a second barrier orders that, and block 0 combines the
// partials in split order from its own shared memory and writes the output.
// 2^x on the special-function unit (about two float32 ulp).  Used for the weights with which
// partial results are merged: the same weight scales a partial's sum and its output.
__device__ __forceinline__ float merge_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}
// *mine as it lies in block `rank` of the cluster <- v
__device__ __forceinline__ void store_to_block(float* mine, uint32_t rank, float v) {
    uint32_t local = (uint32_t)__cvta_generic_to_shared(mine), remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}

template <int D, int STAGES, bool FUSED, bool CLUSTER>
__global__ void __launch_bounds__(kThreads) attention_decode_kernel(
    __nv_bfloat16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
    const __nv_bfloat16* __restrict__ q, const int* __restrict__ row_slot, const int* __restrict__ row_pos,
    PagedKV kv, int n_q, int n_splits, float scale_log2, int window, int* __restrict__ counters,
    int* __restrict__ err, FusedInput fused) {
    pdl_launch_dependents();
    pdl_wait();
    static_assert(!FUSED || D % 64 == 0, "the fused prologue deals D / 64 values of each half of a head to a lane");
    constexpr int kPitch = D + 8, kStages = STAGES;
    constexpr int E = D >= 64 ? D / 64 : 1, kHalf = D / 2;
    // FUSED: the step's raw rows and the gains are requested first, so that they travel while
    // the block finds its pages (position -> page -> tile is a chain of dependent loads).
    __nv_bfloat16 raw_lo[E], raw_hi[E];                    // query head `warp` of the group (heads warp + 4, .. are read later)
    __nv_bfloat16 raw_k_lo[E], raw_k_hi[E], new_v_lo[E], new_v_hi[E];   // warp 0: the step's own key and value
    float qg_lo[E], qg_hi[E], kg_lo[E], kg_hi[E];
    if constexpr (FUSED) {
        const int lane_ = threadIdx.x & 31, warp_ = threadIdx.x >> 5, d0 = lane_ * E;
        const int G_ = n_q / kv.n_kv;
        const __nv_bfloat16* row = fused.qkv + (size_t)blockIdx.x * (n_q + 2 * kv.n_kv) * D;
#pragma unroll
        for (int e = 0; e < E; ++e) {
            raw_lo[e] = warp_ < G_ ? row[(size_t)(blockIdx.y * G_ + warp_) * D + d0 + e] : __float2bfloat16_rn(0.f);
            raw_hi[e] = warp_ < G_ ? row[(size_t)(blockIdx.y * G_ + warp_) * D + kHalf + d0 + e] : __float2bfloat16_rn(0.f);
        }
#pragma unroll
        for (int e = 0; e < E; ++e) {
            qg_lo[e] = gain_at(fused.q_gain, fused.gain_f32, d0 + e);
            qg_hi[e] = gain_at(fused.q_gain, fused.gain_f32, kHalf + d0 + e);
        }
        if (warp_ == 0 && fused.write_cache) {
            const __nv_bfloat16* k_row = row + (size_t)(n_q + blockIdx.y) * D;
            const __nv_bfloat16* v_row = row + (size_t)(n_q + kv.n_kv + blockIdx.y) * D;
#pragma unroll
            for (int e = 0; e < E; ++e) {
                raw_k_lo[e] = k_row[d0 + e];
                raw_k_hi[e] = k_row[kHalf + d0 + e];
                new_v_lo[e] = v_row[d0 + e];
                new_v_hi[e] = v_row[kHalf + d0 + e];
                kg_lo[e] = gain_at(fused.k_gain, fused.gain_f32, d0 + e);
                kg_hi[e] = gain_at(fused.k_gain, fused.gain_f32, kHalf + d0 + e);
            }
        }
    }
    __shared__ int is_last;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* q_smem = reinterpret_cast<__nv_bfloat16*>(smem_raw);            // [16][kPitch]
    __nv_bfloat16* k_smem = q_smem + 16 * kPitch;                                   // [kStages][64][kPitch]
    __nv_bfloat16* v_smem = k_smem + kStages * kTile * kPitch;

    const int b = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int G = n_q / kv.n_kv;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pos = row_pos[b];
    const int* pages = kv.block_table + (size_t)row_slot[b] * kv.bt_stride;

    int first_key = 0;
    if (window > 0 && pos - window + 1 > 0) first_key = pos - window + 1;
    const int t_first = first_key / kTile, t_last = pos / kTile;
    const int n_tiles = t_last - t_first + 1;
    // as even as it goes: the first n_tiles % n_splits splits take one tile more than the others
    const int per_split = n_tiles / n_splits, longer = n_tiles - per_split * n_splits;
    const int t_begin = t_first + split * per_split + min(split, longer);
    const int t_end = t_begin + per_split + (split < longer ? 1 : 0);      // exclusive; == t_begin for an empty split

    __nv_bfloat16 new_k_lo[E], new_k_hi[E];
    const bool patches = FUSED && fused.write_cache && t_begin <= t_last && t_last < t_end;
    if (!FUSED) {
        for (int c = threadIdx.x; c < 16 * (D / 8); c += kThreads) {
            const int r = c / (D / 8), col = (c % (D / 8)) * 8;
            if (r < G)
                cp_async16(q_smem + r * kPitch + col, q + ((size_t)b * n_q + kvh * G + r) * D + col);
            else
                *reinterpret_cast<uint4*>(q_smem + r * kPitch + col) = make_uint4(0, 0, 0, 0);
        }
    }
    cp_async_commit();

    // (the page of a tile is looked up a tile before its loads are issued: the loads' addresses
    // wait for it, and a lookup per tile in the loop would stall the block once per tile)
    auto page_of = [&](int t) { return t < t_end ? pages[t] : 0; };
    auto issue = [&](int t, int stage, int page) {
        if (t < t_end) {
            if (page < 0) {
                if (threadIdx.x == 0 && err) atomicOr(err, THN_ERR_PAGE_UNMAPPED);
            } else {
                const __nv_bfloat16* base = (const __nv_bfloat16*)kv.base;
                load_tile_async<D>(k_smem + stage * kTile * kPitch, base + kv_offset(kv, page, 0, kvh, 0));
                load_tile_async<D>(v_smem + stage * kTile * kPitch, base + kv_offset(kv, page, 1, kvh, 0));
            }
        }
        cp_async_commit();
    };
    // FUSED: the row's angles are requested before the page of the first tile is looked up
    float angle_c[E], angle_s[E];
    if constexpr (FUSED) {
        const int at = pos < fused.table_len ? pos : 0;
#pragma unroll
        for (int e = 0; e < E; ++e) {
            angle_c[e] = fused.cos_tab[(size_t)at * kHalf + lane * E + e];
            angle_s[e] = fused.sin_tab[(size_t)at * kHalf + lane * E + e];
        }
    }
#pragma unroll
    for (int ahead = 0; ahead < kStages - 1; ++ahead)                                   // kStages - 1 tiles in flight
        issue(t_begin + ahead, ahead, page_of(t_begin + ahead));
    int page_next = page_of(t_begin + kStages - 1);

    // the first tiles are on their way while the block prepares its queries
    if constexpr (FUSED) {
        if (pos >= fused.table_len) {
            if (threadIdx.x == 0 && err) atomicOr(err, THN_ERR_POSITION_RANGE);
            cp_async_wait<0>();
            return;
        }
        const int d0 = lane * E;
        float c[E], sn[E];
#pragma unroll
        for (int e = 0; e < E; ++e) {
            c[e] = rnd<__nv_bfloat16>(angle_c[e]);
            sn[e] = rnd<__nv_bfloat16>(angle_s[e]);
        }
        const __nv_bfloat16* qkv_row = fused.qkv + (size_t)b * (n_q + 2 * kv.n_kv) * D;
#pragma unroll 1
        for (int r = warp; r < 16; r += 4) {              // rolled: one pass per warp when G <= 4
            __nv_bfloat16 lo[E], hi[E];
            if (r < G) {                                   // the same for the whole warp
                if (r != warp) {
#pragma unroll
                    for (int e = 0; e < E; ++e) {
                        raw_lo[e] = qkv_row[(size_t)(kvh * G + r) * D + d0 + e];
                        raw_hi[e] = qkv_row[(size_t)(kvh * G + r) * D + kHalf + d0 + e];
                    }
                }
                norm_rotate_head<D>(raw_lo, raw_hi, qg_lo, qg_hi, fused.eps, c, sn, lo, hi);
            } else {
#pragma unroll
                for (int e = 0; e < E; ++e) lo[e] = hi[e] = __float2bfloat16_rn(0.f);
            }
#pragma unroll
            for (int e = 0; e < E; ++e) {
                q_smem[r * kPitch + d0 + e] = lo[e];
                q_smem[r * kPitch + kHalf + d0 + e] = hi[e];
            }
        }
        if (patches && warp == 0) norm_rotate_head<D>(raw_k_lo, raw_k_hi, kg_lo, kg_hi, fused.eps, c, sn, new_k_lo, new_k_hi);
    }
    cp_async_wait<kStages - 1>();                                           // Q has landed
    __syncthreads();
    uint32_t qf[D / 16][4];
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk)
        ldmatrix_x4(qf[kk], q_smem + ((lane & 7) + ((lane >> 3) & 1) * 8) * kPitch + kk * 16 + (lane >> 4) * 8);

    float o[D / 8][4];
#pragma unroll
    for (int nd = 0; nd < D / 8; ++nd)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[nd][i] = 0.f;
    RowState st;
    st.init();
    const int tq = lane & 3;

    for (int t = t_begin, stage = 0; t < t_end; ++t, stage = stage + 1 == kStages ? 0 : stage + 1) {
        const int page_now = page_next;
        page_next = page_of(t + kStages);
        issue(t + kStages - 1, stage == 0 ? kStages - 1 : stage - 1, page_now);     // into the buffer the last tile left
        cp_async_wait<kStages - 1>();
        __syncthreads();
        if constexpr (FUSED) if (patches && t == t_last) {
            // the tile came from the cache without this step's token: put it in, here and there
            if (warp == 0) {
                const int page = pages[t], in_page = pos % kTile, d0 = lane * E;
                if (page >= 0) {
                    __nv_bfloat16* k_dst = (__nv_bfloat16*)kv.base + kv_offset(kv, page, 0, kvh, in_page);
                    __nv_bfloat16* v_dst = (__nv_bfloat16*)kv.base + kv_offset(kv, page, 1, kvh, in_page);
                    __nv_bfloat16* k_row = k_smem + stage * kTile * kPitch + in_page * kPitch;
                    __nv_bfloat16* v_row = v_smem + stage * kTile * kPitch + in_page * kPitch;
#pragma unroll
                    for (int e = 0; e < E; ++e) {
                        k_dst[d0 + e] = k_row[d0 + e] = new_k_lo[e];
                        k_dst[kHalf + d0 + e] = k_row[kHalf + d0 + e] = new_k_hi[e];
                        v_dst[d0 + e] = v_row[d0 + e] = new_v_lo[e];
                        v_dst[kHalf + d0 + e] = v_row[kHalf + d0 + e] = new_v_hi[e];
                    }
                }
            }
            __syncthreads();
        }
        const int key0 = t * kTile + warp * 16;
        float s[2][4];
        qk_tile<D, 2>(s, qf, k_smem + stage * kTile * kPitch, warp * 2, lane);
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int key = key0 + n * 8 + tq * 2 + (i & 1);
                const bool visible = key <= pos && key >= first_key;
                s[n][i] = visible ? s[n][i] * scale_log2 : -INFINITY;
            }
        uint32_t pf[1][4];
        softmax_tile<D, 2>(s, st, o, pf);
        pv_tile<D, 2>(o, pf, v_smem + stage * kTile * kPitch, warp * 2, lane);
        __syncthreads();
    }
    cp_async_wait<0>();
    __syncthreads();

    // Merge the four warps through shared memory (the tile buffers are free now).  Only the G
    // rows that are query heads are kept; a row takes D + 8 floats so that the rows a warp
    // stores together fall into different banks.
    constexpr int kOPitch = D + 8;
    constexpr int kKeep = 16 * D / kThreads;                    // merged values a thread holds (G <= 16)
    float* m_smem = reinterpret_cast<float*>(k_smem);           // [4][16]
    float* l_smem = m_smem + 64;                                // [4][16]
    float* o_smem = l_smem + 64;                                // [4][G][kOPitch]
    const int g = lane >> 2;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float l = st.l[r];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        const int row = g + 8 * r;
        if (row < G) {
            if (tq == 0) {
                m_smem[warp * 16 + row] = st.m[r];
                l_smem[warp * 16 + row] = l;
            }
#pragma unroll
            for (int nd = 0; nd < D / 8; ++nd)
                *reinterpret_cast<float2*>(o_smem + (warp * G + row) * kOPitch + nd * 8 + tq * 2) =
                    make_float2(o[nd][2 * r], o[nd][2 * r + 1]);
        }
    }
    __syncthreads();
    // weight of warp w in row r, and the row's (max, sum), once: threads 0 .. 4 G - 1
    float* wgt_smem = o_smem + 4 * 16 * kOPitch;                // [16][4]; then (max, sum) [16][2]
    float* ml_smem = wgt_smem + 64;
    if ((threadIdx.x & ~31) < 4 * G) {                          // whole warps: the shuffles below take all 32 lanes
        const bool live = threadIdx.x < 4 * G;
        const int row = min((int)threadIdx.x >> 2, 15), w = threadIdx.x & 3;
        const float mine = m_smem[w * 16 + row];
        float m = mine;
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
        const float wgt = m == -INFINITY ? 0.f : merge_exp2(mine - m);
        float l = l_smem[w * 16 + row] * wgt;
        const float l1 = l + __shfl_xor_sync(0xffffffffu, l, 1);          // (w0 + w1), (w2 + w3): the order is fixed
        l = l1 + __shfl_xor_sync(0xffffffffu, l1, 2);
        if (live) {
            wgt_smem[row * 4 + w] = wgt;
            if (w == 0) {
                ml_smem[row * 2] = m;
                ml_smem[row * 2 + 1] = l;
            }
        }
    }
    __syncthreads();
    // (These loops run once per block and are left rolled on purpose: unrolled, their
    // instructions cost more to fetch than to execute.)
    float keep[kKeep];
#pragma unroll 1
    for (int i = 0; i < kKeep; ++i) {
        const int e = threadIdx.x + i * kThreads;
        if (e >= G * D) break;
        const int row = e / D, d = e % D;
        const float4 wgt = *reinterpret_cast<const float4*>(wgt_smem + row * 4);
        const float acc = (o_smem[(0 * G + row) * kOPitch + d] * wgt.x + o_smem[(1 * G + row) * kOPitch + d] * wgt.y) +
                          (o_smem[(2 * G + row) * kOPitch + d] * wgt.z + o_smem[(3 * G + row) * kOPitch + d] * wgt.w);
        const size_t head = (size_t)b * n_q + kvh * G + row;
        if (n_splits == 1) {
            out[head * D + d] = __float2bfloat16_rn(acc / ml_smem[row * 2 + 1]);
        } else if (CLUSTER) {
            keep[i] = acc;
        } else {
            __stcg(part_o + (head * n_splits + split) * D + d, acc);
            if (d == 0) {
                __stcg(part_ml + (head * n_splits + split) * 2, ml_smem[row * 2]);
                __stcg(part_ml + (head * n_splits + split) * 2 + 1, ml_smem[row * 2 + 1]);
            }
        }
    }
    if (CLUSTER) {
        // No early return above in this mode: every thread of every block reaches both barriers.
        // In block 0, over the tile buffers: after each block's own (max, sum) of its warps, the
        // partial outputs [split][G * D]; near the end (max, sum) [8 splits][16 rows][2] and the
        // weights of the splits.
        constexpr int kTileFloats = 2 * kStages * kTile * kPitch / 2;
        float* recv_o = reinterpret_cast<float*>(k_smem) + 128;
        float* w_smem = reinterpret_cast<float*>(k_smem) + kTileFloats - (16 * 32 + 16);     // [16][32]
        float* l_total = w_smem + 16 * 32;                       // [16]
        float* recv_ml = w_smem - 8 * 32;
        // (the row's (max, sum) leave this block's buffers before block 0's copy of them may be overwritten)
        const float ml_held = threadIdx.x < 2 * G ? ml_smem[threadIdx.x] : 0.f;
        cluster_sync_all();                                      // every block is done with its tile buffers
#pragma unroll 1
        for (int i = 0; i < kKeep; ++i) {
            const int e = threadIdx.x + i * kThreads;
            if (e >= G * D) break;
            store_to_block(recv_o + split * G * D + e, 0, keep[i]);
        }
        if (threadIdx.x < 2 * G) store_to_block(recv_ml + split * 32 + threadIdx.x, 0, ml_held);
        cluster_sync_all();                                      // every partial is in block 0
        if (split != 0) return;
        for (int row = warp; row < G; row += 4) {
            const float ms = lane < n_splits ? recv_ml[lane * 32 + row * 2] : -INFINITY;
            const float ls = lane < n_splits ? recv_ml[lane * 32 + row * 2 + 1] : 0.f;
            const float m = warp_max(ms);
            const float wgt = ms == -INFINITY ? 0.f : merge_exp2(ms - m);
            const float l = warp_sum(ls * wgt);
            w_smem[row * 32 + lane] = wgt;
            if (lane == 0) l_total[row] = 1.0f / l;
        }
        __syncthreads();
#pragma unroll 1
        for (int e = threadIdx.x; e < G * D; e += kThreads) {
            const int row = e / D, d = e % D;
            const size_t head = (size_t)b * n_q + kvh * G + row;
            float v[8];                                          // at most 8 splits in a cluster
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = j < n_splits ? recv_o[j * G * D + e] : 0.f;
            float acc = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) acc += v[j] * w_smem[row * 32 + j];                 // split order
            out[head * D + d] = __float2bfloat16_rn(acc * l_total[row]);
        }
        return;
    }
    if (n_splits == 1 || counters == nullptr) return;

    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) is_last = atomicAdd(counters + b * kv.n_kv + kvh, 1) == n_splits - 1;
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (threadIdx.x == 0) counters[b * kv.n_kv + kvh] = 0;        // ready for the next call
    // Weights of the splits, one warp per head: lane = split (n_splits <= 32).
    float* w_smem = reinterpret_cast<float*>(v_smem);            // [16][32]
    float* l_total = w_smem + 16 * 32;                           // [16]
    for (int row = warp; row < G; row += 4) {
        const size_t head = (size_t)b * n_q + kvh * G + row;
        const float ms = lane < n_splits ? __ldcg(part_ml + (head * n_splits + lane) * 2) : -INFINITY;
        const float ls = lane < n_splits ? __ldcg(part_ml + (head * n_splits + lane) * 2 + 1) : 0.f;
        const float m = warp_max(ms);
        const float wgt = ms == -INFINITY ? 0.f : exp2f(ms - m);
        const float l = warp_sum(ls * wgt);
        w_smem[row * 32 + lane] = wgt;
        if (lane == 0) l_total[row] = l;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < G * D; e += kThreads) {
        const int row = e / D, d = e % D;
        const size_t head = (size_t)b * n_q + kvh * G + row;
        const float* src = part_o + head * n_splits * D + d;
        float acc = 0.f;
        for (int s0 = 0; s0 < n_splits; s0 += 8) {               // eight loads in flight, added in split order
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = s0 + j < n_splits ? __ldcg(src + (size_t)(s0 + j) * D) : 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) acc += v[j] * w_smem[row * 32 + ((s0 + j) & 31)];
        }
        out[head * D + d] = __float2bfloat16_rn(acc / l_total[row]);
    }
}

// out[head] = sum_s o_s * 2^(m_s - m) / sum_s l_s * 2^(m_s - m); splits are combined in
// ascending order.
__global__ void attention_merge_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ part_o,
                                       const float* __restrict__ part_ml, int n_splits, int D) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t head = blockIdx.x;
    float m = -INFINITY;
    for (int s = 0; s < n_splits; ++s) m = fmaxf(m, part_ml[(head * n_splits + s) * 2]);
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float l = 0.f, acc = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const float ms = part_ml[(head * n_splits + s) * 2];
            if (ms == -INFINITY) continue;
            const float wgt = exp2f(ms - m);
            l += part_ml[(head * n_splits + s) * 2 + 1] * wgt;
            acc += part_o[(head * n_splits + s) * D + d] * wgt;
        }
        out[head * D + d] = __float2bfloat16_rn(acc / l);
    }
}

// ------------------------------------------------------------------ single tokens, many sequences
//
// When a step brings more (sequence, kv head) pairs than the GPU holds clusters, the key range
// of a pair is not split and the kernel below takes over.  It is built for bandwidth: a fixed
// number of blocks, as many as are resident at once, each of which works through several
// pairs, one after the other, without letting its loads run dry in between.
//
//   * Warp 4 is the loader.  It walks the block's pairs and their pages (32 page numbers per
//     lookup, the next pair's position and slot requested a pair ahead) and one lane fetches
//     every K tile and V tile with `cp.async.bulk.tensor` from a tensor map over the cache
//     entry ([pages * 2 * n_kv * 64 rows, head_dim], boxes of 64 values x 64 rows, 128-byte
//     swizzle, so that ldmatrix reads no bank twice without padded rows) onto the tile
//     buffer's mbarrier.  It runs up to STAGES tiles ahead of the arithmetic, across pair
//     boundaries.
//   * Warp 5 prepares the queries of the NEXT pair while the arithmetic works on this one: it
//     copies the pair's query heads into shared memory, or (FUSED) normalises and rotates
//     them from the step's raw q/k/v rows, and normalises and rotates the step's own key,
//     writes it and the value to the cache and leaves both in shared memory for the tile.
//   * Warps 0-3 are the arithmetic of attention_decode_kernel (16 keys of every tile each,
//     the same fragments, masks and rounding), reading the swizzled tiles.  They give a tile
//     buffer back with one arrival per warp on its second mbarrier and meet among
//     themselves on a named barrier only where a pair ends (the merge of their four partial
//     results, in scratch of its own, as the tile buffers are in use).
//
// Every wait on an mbarrier is bounded by the clock (20 ms); a waiter that gives up sets
// THN_ERR_WAIT_TIMEOUT, tells the others, and the loader waits (bounded again) for the
// copies it still has in flight before it returns.

constexpr int kStreamThreads = 192;            // four arithmetic warps, the loader, the preparer
constexpr unsigned long long kStreamWaitNs = 20ull * 1000 * 1000;

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
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
        else if (now - start > kStreamWaitNs) return false;
    }
}
__device__ __forceinline__ void tma_tile(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
// The four arithmetic warps among themselves (barrier 0 is __syncthreads).  The warps come here
// from branches that only some of their lanes took, and unlike __syncthreads an asm statement
// does not make the compiler bring them together first: so the warp converges explicitly, and
// the barrier is the form that counts threads, not the one that wants whole warps.
__device__ __forceinline__ void sync_arithmetic() {
    __syncwarp();
    asm volatile("barrier.sync 1, 128;" ::: "memory");
}

// Byte offset of the 16 bytes that hold values [d, d + 8) of row `row` in a tile that came as
// boxes of 64 values x 64 rows with the 128-byte swizzle: a row of a box is 128 bytes, its eight
// 16-byte pieces are exchanged by the row's low three bits, the second box follows the first.
__device__ __forceinline__ uint32_t swizzled(int row, int d) {
    return (uint32_t)((d >> 6) * (kTile * 128) + row * 128 + ((((d & 63) >> 3) ^ (row & 7)) << 4));
}

// qk_tile and pv_tile on swizzled tiles.
template <int D, int NK>
__device__ __forceinline__ void qk_tile_swizzled(float (&s)[NK][4], const uint32_t (&qf)[D / 16][4],
                                                 const unsigned char* k_tile, int key_block0, int lane) {
#pragma unroll
    for (int n = 0; n < NK; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) s[n][i] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
        for (int n = 0; n < NK; n += 2) {
            uint32_t b[4];
            const int key = (key_block0 + n + (lane >> 4)) * 8 + (lane & 7);
            ldmatrix_x4(b, k_tile + swizzled(key, kk * 16 + ((lane >> 3) & 1) * 8));
            mma_bf16(s[n], qf[kk], b[0], b[1]);
            mma_bf16(s[n + 1], qf[kk], b[2], b[3]);
        }
    }
}
template <int D, int NK>
__device__ __forceinline__ void pv_tile_swizzled(float (&o)[D / 8][4], const uint32_t (&pf)[NK / 2][4],
                                                 const unsigned char* v_tile, int key_block0, int lane) {
#pragma unroll
    for (int kk = 0; kk < NK / 2; ++kk) {
#pragma unroll
        for (int nd = 0; nd < D / 8; nd += 2) {
            uint32_t b[4];
            const int key = (key_block0 + 2 * kk) * 8 + ((lane >> 3) & 1) * 8 + (lane & 7);
            ldmatrix_x4_trans(b, v_tile + swizzled(key, (nd + (lane >> 4)) * 8));
            mma_bf16(o[nd], pf[kk], b[0], b[1]);
            mma_bf16(o[nd + 1], pf[kk], b[2], b[3]);
        }
    }
}

// Shared memory of the streaming kernel for groups of G query heads: tile buffers (each K tile
// and V tile 64 * D * 2 bytes; the buffers start the block's shared memory, 1024-byte aligned
// for the swizzle), q [16][D], the step's own key and value for two pairs [2][2][D], the merge
// scratch ((max, sum) of four warps, their outputs [4][G][D + 8], weights), flags and barriers.
template <int D>
constexpr size_t stream_smem(int stages, int G) {
    return (size_t)stages * 2 * kTile * D * 2 + 16 * D * 2 + 4 * D * 2 + (size_t)(128 + 4 * G * (D + 8) + 64 + 32) * 4 +
           (size_t)(2 * stages + 2) * 8 + 16;
}
constexpr int kStreamRankedSeqs = 256;      // sequences up to which the pairs are dealt out by length (6 bytes each)

template <int D, int STAGES, bool FUSED>
__global__ void __launch_bounds__(kStreamThreads, D == 128 ? 2 : 3) attention_decode_stream_kernel(
    const __grid_constant__ CUtensorMap map_kv, __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ q,
    const int* __restrict__ row_slot, const int* __restrict__ row_pos, PagedKV kv, int n_seqs, int n_q,
    float scale_log2, int window, int* __restrict__ err, FusedInput fused, int by_length) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int kOPitch = D + 8;
    constexpr int E = D / 64, kHalf = D / 2;
    constexpr uint32_t kTileBytes = kTile * D * 2;
    extern __shared__ __align__(1024) unsigned char tiles[];
    __nv_bfloat16* q_smem = reinterpret_cast<__nv_bfloat16*>(tiles + (size_t)STAGES * 2 * kTileBytes);   // [16][D]
    __nv_bfloat16* own_smem = q_smem + 16 * D;                          // [2 pairs][key, value][D]
    const int G = n_q / kv.n_kv;
    float* m_smem = reinterpret_cast<float*>(own_smem + 4 * D);         // [4][16]
    float* l_smem = m_smem + 64;                                        // [4][16]
    float* o_smem = l_smem + 64;                                        // [4][G][kOPitch]
    float* wgt_smem = o_smem + 4 * G * kOPitch;                         // [16][4]
    float* ml_smem = wgt_smem + 64;                                     // [16][2]
    uint64_t* full = reinterpret_cast<uint64_t*>(ml_smem + 32);         // [STAGES] a tile pair has landed
    uint64_t* empty = full + STAGES;                                    // [STAGES] the four warps are done with it
    uint64_t* q_full = empty + STAGES;                                  // the next pair's q (and own key, value) are ready
    uint64_t* q_empty = q_full + 1;                                     // the four warps hold q in registers
    volatile int* give_up = reinterpret_cast<volatile int*>(q_empty + 1);
    volatile int* position_bad = give_up + 1;                           // [2] by pair parity
    unsigned short* by_rank = reinterpret_cast<unsigned short*>(const_cast<int*>(position_bad + 2) + 1);   // [n_seqs] (by_length)

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n_pairs = n_seqs * kv.n_kv;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, 4);
        }
        mbar_init(q_full, 1);
        mbar_init(q_empty, 4);
        *give_up = (smem_u32(tiles) & 1023u) ? 1 : 0;      // the swizzle's arithmetic needs the alignment
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // by_length: the sequences ranked by their length, longest first (ties by index), every
    // block for itself: by_rank[rank] = sequence.  The pairs are then dealt out in that order,
    // forwards in even rounds and backwards in odd ones, so that a block's pairs add up to about
    // the same number of keys whatever the lengths are.
    if (by_length) {
        int* lengths = reinterpret_cast<int*>(by_rank + ((n_seqs + 1) & ~1));       // [n_seqs], read once from global memory
        for (int b = threadIdx.x; b < n_seqs; b += kStreamThreads) lengths[b] = row_pos[b];
        __syncthreads();
        for (int b = threadIdx.x; b < n_seqs; b += kStreamThreads) {
            const int mine = lengths[b];
            int rank = 0;
            for (int other = 0; other < n_seqs; ++other) {
                const int theirs = lengths[other];
                rank += (theirs > mine || (theirs == mine && other < b)) ? 1 : 0;
            }
            by_rank[rank] = (unsigned short)b;
        }
    }
    __syncthreads();
    // The k-th pair of this block: (sequence, kv head), or sequence -1 when the block has no k-th pair.
    const int n_rounds = (n_pairs + (int)gridDim.x - 1) / (int)gridDim.x;
    auto pair_of = [&](int k, int& b, int& kvh) {
        int item = k * (int)gridDim.x + ((k & 1) && by_length ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x);
        if (k >= n_rounds || item >= n_pairs) {
            b = -1;
            kvh = 0;
            return;
        }
        kvh = item % kv.n_kv;
        b = by_length ? (int)by_rank[item / kv.n_kv] : item / kv.n_kv;
    };
    if (*give_up) {
        if (threadIdx.x == 0 && err) atomicOr(err, THN_ERR_WAIT_TIMEOUT);
        return;
    }

    if (warp == 4) {
        // ---------------------------------------------------------------- the loader
        int it = 0;                                        // tiles requested so far by this block
        bool ok = true;
        int b_next, kvh_next, pos_next = 0, slot_next = 0;
        pair_of(0, b_next, kvh_next);
        if (b_next >= 0) {
            pos_next = row_pos[b_next];
            slot_next = row_slot[b_next];
        }
        for (int k = 0; k < n_rounds && ok && !*give_up; ++k) {
            const int b = b_next, kvh = kvh_next;
            const int pos = pos_next, slot = slot_next;
            pair_of(k + 1, b_next, kvh_next);
            if (b_next >= 0) {                              // a pair ahead: on its way while this pair's tiles are requested
                pos_next = row_pos[b_next];
                slot_next = row_slot[b_next];
            }
            if (b < 0) continue;
            int first_key = 0;
            if (window > 0 && pos - window + 1 > 0) first_key = pos - window + 1;
            const int t_first = first_key / kTile, t_last = pos / kTile;
            const int* pages = kv.block_table + (size_t)slot * kv.bt_stride;
            for (int t0 = t_first; t0 <= t_last && ok; t0 += 32) {
                const int mine = t0 + lane <= t_last ? pages[t0 + lane] : 0;
                const int n = min(32, t_last - t0 + 1);
                for (int j = 0; j < n && ok; ++j, ++it) {
                    const int page = __shfl_sync(0xffffffffu, mine, j);
                    const int s = it % STAGES;
                    if (lane == 0) {
                        ok = mbar_wait(empty + s, ((it / STAGES) & 1) ^ 1);
                        if (!ok) {
                            if (err) atomicOr(err, THN_ERR_WAIT_TIMEOUT);
                        } else if (page < 0) {
                            if (err) atomicOr(err, THN_ERR_PAGE_UNMAPPED);
                            mbar_arrive(full + s);          // nothing is fetched; the arithmetic goes on over what lies there
                        } else {
                            unsigned char* dst = tiles + (size_t)s * 2 * kTileBytes;
                            mbar_expect_tx(full + s, 2 * kTileBytes);
                            const int k_row = ((page * 2 + 0) * kv.n_kv + kvh) * kTile;
                            const int v_row = ((page * 2 + 1) * kv.n_kv + kvh) * kTile;
#pragma unroll
                            for (int half = 0; half < D / 64; ++half) {
                                tma_tile(dst + half * (kTile * 128), &map_kv, full + s, half * 64, k_row);
                                tma_tile(dst + kTileBytes + half * (kTile * 128), &map_kv, full + s, half * 64, v_row);
                            }
                        }
                    }
                    ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
                }
            }
        }
        if (!ok) *give_up = 1;
        // Copies still in flight must land before the block's shared memory is given up: wait
        // for the last STAGES tiles requested (a tile the arithmetic has taken is complete).
        if (lane == 0) {
            for (int back = 1; back <= STAGES && back <= it; ++back) {
                const int j = it - back;
                mbar_wait(full + j % STAGES, (j / STAGES) & 1);
            }
        }
        return;
    }

    if (warp == 5) {
        // ---------------------------------------------------------------- the preparer
        const int d0 = lane * E;
        for (int c = lane; c < 16 * (D / 8); c += 32)                   // rows beyond the group stay zero
            *reinterpret_cast<uint4*>(q_smem + c * 8) = make_uint4(0, 0, 0, 0);
        float qg_lo[E], qg_hi[E], kg_lo[E], kg_hi[E];
        if (FUSED) {
#pragma unroll
            for (int e = 0; e < E; ++e) {
                qg_lo[e] = gain_at(fused.q_gain, fused.gain_f32, d0 + e);
                qg_hi[e] = gain_at(fused.q_gain, fused.gain_f32, kHalf + d0 + e);
                kg_lo[e] = gain_at(fused.k_gain, fused.gain_f32, d0 + e);
                kg_hi[e] = gain_at(fused.k_gain, fused.gain_f32, kHalf + d0 + e);
            }
        }
        __syncwarp();
        bool ok = true;
        for (int round = 0, k = 0; round < n_rounds && ok && !*give_up; ++round) {
            int b, kvh;
            pair_of(round, b, kvh);
            if (b < 0) continue;
            const int k_now = k++;
            // what the pair needs from global memory is requested before the wait for q's buffer
            __nv_bfloat16 raw_lo[4][E], raw_hi[4][E];                     // up to four heads in flight
            const int pos = FUSED ? row_pos[b] : 0;
            const bool position_ok = !FUSED || pos < fused.table_len;
            if (lane == 0) ok = mbar_wait(q_empty, (k_now & 1) ^ 1);
            ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
            if (!ok) {
                if (lane == 0 && err) atomicOr(err, THN_ERR_WAIT_TIMEOUT);
                break;
            }
            if (!FUSED) {
                for (int c = lane; c < G * (D / 8); c += 32)
                    *reinterpret_cast<uint4*>(q_smem + c * 8) =
                        *reinterpret_cast<const uint4*>(q + ((size_t)b * n_q + kvh * G) * D + c * 8);
            } else {
                const int at = position_ok ? pos : 0;
                float c[E], sn[E];
#pragma unroll
                for (int e = 0; e < E; ++e) {
                    c[e] = rnd<__nv_bfloat16>(fused.cos_tab[(size_t)at * kHalf + d0 + e]);
                    sn[e] = rnd<__nv_bfloat16>(fused.sin_tab[(size_t)at * kHalf + d0 + e]);
                }
                const __nv_bfloat16* qkv_row = fused.qkv + (size_t)b * (n_q + 2 * kv.n_kv) * D;
                for (int r0 = 0; r0 < G; r0 += 4) {                     // four heads' loads in flight at a time
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int r = min(r0 + i, G - 1);
#pragma unroll
                        for (int e = 0; e < E; ++e) {
                            raw_lo[i][e] = qkv_row[(size_t)(kvh * G + r) * D + d0 + e];
                            raw_hi[i][e] = qkv_row[(size_t)(kvh * G + r) * D + kHalf + d0 + e];
                        }
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        if (r0 + i >= G) break;
                        __nv_bfloat16 lo[E], hi[E];
                        norm_rotate_head<D>(raw_lo[i], raw_hi[i], qg_lo, qg_hi, fused.eps, c, sn, lo, hi);
#pragma unroll
                        for (int e = 0; e < E; ++e) {
                            q_smem[(r0 + i) * D + d0 + e] = lo[e];
                            q_smem[(r0 + i) * D + kHalf + d0 + e] = hi[e];
                        }
                    }
                }
                if (fused.write_cache) {
                    // the step's own key (normalised, rotated) and value: into the cache now, and
                    // kept for the last tile, which may have been fetched without them
                    const __nv_bfloat16* k_row = qkv_row + (size_t)(n_q + kvh) * D;
                    const __nv_bfloat16* v_row = qkv_row + (size_t)(n_q + kv.n_kv + kvh) * D;
                    __nv_bfloat16 raw_k_lo[E], raw_k_hi[E], new_k_lo[E], new_k_hi[E], new_v_lo[E], new_v_hi[E];
#pragma unroll
                    for (int e = 0; e < E; ++e) {
                        raw_k_lo[e] = k_row[d0 + e];
                        raw_k_hi[e] = k_row[kHalf + d0 + e];
                        new_v_lo[e] = v_row[d0 + e];
                        new_v_hi[e] = v_row[kHalf + d0 + e];
                    }
                    const int page = position_ok ? (kv.block_table + (size_t)row_slot[b] * kv.bt_stride)[pos / kTile] : -1;
                    norm_rotate_head<D>(raw_k_lo, raw_k_hi, kg_lo, kg_hi, fused.eps, c, sn, new_k_lo, new_k_hi);
                    __nv_bfloat16* own = own_smem + (k_now & 1) * 2 * D;
#pragma unroll
                    for (int e = 0; e < E; ++e) {
                        own[d0 + e] = new_k_lo[e];
                        own[kHalf + d0 + e] = new_k_hi[e];
                        own[D + d0 + e] = new_v_lo[e];
                        own[D + kHalf + d0 + e] = new_v_hi[e];
                    }
                    if (page >= 0) {
                        __nv_bfloat16* k_dst = (__nv_bfloat16*)kv.base + kv_offset(kv, page, 0, kvh, pos % kTile);
                        __nv_bfloat16* v_dst = (__nv_bfloat16*)kv.base + kv_offset(kv, page, 1, kvh, pos % kTile);
#pragma unroll
                        for (int e = 0; e < E; ++e) {
                            k_dst[d0 + e] = new_k_lo[e];
                            k_dst[kHalf + d0 + e] = new_k_hi[e];
                            v_dst[d0 + e] = new_v_lo[e];
                            v_dst[kHalf + d0 + e] = new_v_hi[e];
                        }
                    }
                }
                if (lane == 0) {
                    position_bad[k_now & 1] = position_ok ? 0 : 1;
                    if (!position_ok && err) atomicOr(err, THN_ERR_POSITION_RANGE);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(q_full);              // (release: the warp's stores above are visible to the waiters)
        }
        return;
    }

    // -------------------------------------------------------------------- the arithmetic
    const int tq = lane & 3, g = lane >> 2;
    int it = 0, k = 0;
    bool ok = true;
    int b_next, kvh_next;
    pair_of(0, b_next, kvh_next);
    int pos_next = b_next >= 0 ? row_pos[b_next] : 0;
    for (int round = 0; round < n_rounds; ++round) {
        const int b = b_next, kvh = kvh_next;
        const int pos = pos_next;
        pair_of(round + 1, b_next, kvh_next);
        if (b_next >= 0) pos_next = row_pos[b_next];
        if (b < 0) continue;
        int first_key = 0;
        if (window > 0 && pos - window + 1 > 0) first_key = pos - window + 1;
        const int t_first = first_key / kTile, t_last = pos / kTile;

        // ---- q from the preparer
        // (The lanes of a warp leave a wait one by one; what follows, ldmatrix and mma.sync, must
        // be executed by the whole warp together, and an asm statement does not make the compiler
        // bring the lanes together: hence the __syncwarp after every wait.)
        if (ok && !*give_up) ok = mbar_wait(q_full, k & 1);
        __syncwarp();
        const bool alive = ok && !*give_up;
        uint32_t qf[D / 16][4];
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
            ldmatrix_x4(qf[kk], q_smem + ((lane & 7) + ((lane >> 3) & 1) * 8) * D + kk * 16 + (lane >> 4) * 8);
        const bool position_ok = !FUSED || position_bad[k & 1] == 0;
        __syncwarp();
        if (lane == 0 && alive) mbar_arrive(q_empty);     // (the preparer writes q with plain stores: the same proxy)
        // FUSED: the warp whose sixteen keys of the last tile include the step's own position
        // puts that token's key and value into the tile.
        const bool patches = FUSED && fused.write_cache && warp == (pos % kTile) / 16 && position_ok;

        float o[D / 8][4];
#pragma unroll
        for (int nd = 0; nd < D / 8; ++nd)
#pragma unroll
            for (int i = 0; i < 4; ++i) o[nd][i] = 0.f;
        RowState st;
        st.init();

        for (int t = t_first; t <= t_last; ++t, ++it) {
            const int s = it % STAGES;
            if (ok && !*give_up) ok = mbar_wait(full + s, (it / STAGES) & 1);
            ok = __all_sync(0xffffffffu, ok);         // one decision for the warp, and the lanes together again
            if (!ok || *give_up) continue;            // keep counting tiles; nothing more is computed
            unsigned char* k_tile = tiles + (size_t)s * 2 * kTileBytes;
            unsigned char* v_tile = k_tile + kTileBytes;
            if (patches && t == t_last) {
                // the tile may have come from the cache without this step's token (no other warp
                // reads these rows of the tile)
                const int in_page = pos % kTile, d0 = lane * E;
                const __nv_bfloat16* own = own_smem + (k & 1) * 2 * D;
#pragma unroll
                for (int e = 0; e < E; ++e) {
                    const uint32_t lo_at = swizzled(in_page, d0 + e) + ((d0 + e) & 7) * 2;
                    const uint32_t hi_at = swizzled(in_page, kHalf + d0 + e) + ((kHalf + d0 + e) & 7) * 2;
                    *reinterpret_cast<__nv_bfloat16*>(k_tile + lo_at) = own[d0 + e];
                    *reinterpret_cast<__nv_bfloat16*>(k_tile + hi_at) = own[kHalf + d0 + e];
                    *reinterpret_cast<__nv_bfloat16*>(v_tile + lo_at) = own[D + d0 + e];
                    *reinterpret_cast<__nv_bfloat16*>(v_tile + hi_at) = own[D + kHalf + d0 + e];
                }
                // the next fetch into this buffer comes through the asynchronous proxy
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
            }
            const int key0 = t * kTile + warp * 16;
            float sc[2][4];
            qk_tile_swizzled<D, 2>(sc, qf, k_tile, warp * 2, lane);
#pragma unroll
            for (int n = 0; n < 2; ++n)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int key = key0 + n * 8 + tq * 2 + (i & 1);
                    const bool visible = key <= pos && key >= first_key;
                    sc[n][i] = visible ? sc[n][i] * scale_log2 : -INFINITY;
                }
            uint32_t pf[1][4];
            softmax_tile<D, 2>(sc, st, o, pf);
            pv_tile_swizzled<D, 2>(o, pf, v_tile, warp * 2, lane);
            // The buffer goes back to the loader, whose next copy into it is made by the
            // asynchronous proxy, while these reads were made by the generic one: the barrier
            // alone does not order the two, the proxy fence does.  (Without it one run in four of
            // a 48-sequence step read sixteen columns of a V tile that the next copy had already
            // reached, with two blocks on an SM.)
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(empty + s);
        }

        // ---- merge the four warps (as attention_decode_kernel does, in scratch of its own)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float l = st.l[r];
            l += __shfl_xor_sync(0xffffffffu, l, 1);
            l += __shfl_xor_sync(0xffffffffu, l, 2);
            const int row = g + 8 * r;
            if (row < G) {
                if (tq == 0) {
                    m_smem[warp * 16 + row] = st.m[r];
                    l_smem[warp * 16 + row] = l;
                }
#pragma unroll
                for (int nd = 0; nd < D / 8; ++nd)
                    *reinterpret_cast<float2*>(o_smem + (warp * G + row) * kOPitch + nd * 8 + tq * 2) =
                        make_float2(o[nd][2 * r], o[nd][2 * r + 1]);
            }
        }
        sync_arithmetic();
        if ((threadIdx.x & ~31) < 4 * G) {                          // whole warps: the shuffles below take all 32 lanes
            const bool live = threadIdx.x < 4 * G;
            const int row = min((int)threadIdx.x >> 2, 15), w = threadIdx.x & 3;
            const float mine = m_smem[w * 16 + row];
            float m = mine;
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
            const float wgt = m == -INFINITY ? 0.f : merge_exp2(mine - m);
            float l = l_smem[w * 16 + row] * wgt;
            const float l1 = l + __shfl_xor_sync(0xffffffffu, l, 1);          // (w0 + w1), (w2 + w3): the order is fixed
            l = l1 + __shfl_xor_sync(0xffffffffu, l1, 2);
            if (live) {
                wgt_smem[row * 4 + w] = wgt;
                if (w == 0) {
                    ml_smem[row * 2] = m;
                    ml_smem[row * 2 + 1] = l;
                }
            }
        }
        sync_arithmetic();
        if (ok && !*give_up && position_ok) {
#pragma unroll 1
            for (int e = threadIdx.x; e < G * D; e += 128) {
                const int row = e / D, d = e % D;
                const float4 wgt = *reinterpret_cast<const float4*>(wgt_smem + row * 4);
                const float acc = (o_smem[(0 * G + row) * kOPitch + d] * wgt.x + o_smem[(1 * G + row) * kOPitch + d] * wgt.y) +
                                  (o_smem[(2 * G + row) * kOPitch + d] * wgt.z + o_smem[(3 * G + row) * kOPitch + d] * wgt.w);
                out[((size_t)b * n_q + kvh * G + row) * D + d] = __float2bfloat16_rn(acc / ml_smem[row * 2 + 1]);
            }
        }
        sync_arithmetic();                                  // the scratch is free for the next pair
        ++k;
    }
    if (!ok) {
        if (lane == 0 && err) atomicOr(err, THN_ERR_WAIT_TIMEOUT);
        *give_up = 1;
    }
}

template <int D> constexpr size_t prefill_smem() { return (size_t)(kPrefillRows + 4 * kTile) * (D + 8) * 2; }
template <int D, int STAGES> constexpr size_t decode_smem() { return (size_t)(16 + 2 * STAGES * kTile) * (D + 8) * 2; }

template <int D>
int launch_prefill(void* out, const void* q, const int* tile_row0, const int* tile_rows, int n_tiles,
                   const int* row_slot, const int* row_pos, PagedKV kv, int n_q, float scale, int window, int* err,
                   cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)prefill_smem<D>());
        if (e != cudaSuccess) {
            thn_set_error("attention_prefill: cannot reserve %zu bytes of shared memory: %s", prefill_smem<D>(),
                          cudaGetErrorString(e));
            return (int)e;
        }
        configured = true;
    }
    THN_UNSUPPORTED_IF(n_tiles > 65535, "attention_prefill: %d row tiles in one step (at most 65535)", n_tiles);
    dim3 grid(n_q, n_tiles);
    thn_launch(attention_prefill_kernel<D>, grid, kPrefillThreads, prefill_smem<D>(), stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)q, tile_row0, tile_rows, row_slot, row_pos, kv, n_q,
        scale * kLog2e, window, err);
    return thn_launch_status("attention_prefill");
}

template <int D, int STAGES, bool FUSED, bool CLUSTER>
int configure_decode() {
    static bool configured = false;
    if (!configured) {

        cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<D, STAGES, FUSED, CLUSTER>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)decode_smem<D, STAGES>());
        if (e != cudaSuccess) {
            thn_set_error("attention_decode: cannot reserve %zu bytes of shared memory: %s",
                          decode_smem<D, STAGES>(), cudaGetErrorString(e));
            return (int)e;
        }
        configured = true;
    }
    return THN_OK;
}

// What the last launch of a decode kernel was built with: tile buffers * 10, + 1 if the splits
// met in a cluster, + 2 for the streaming kernel.  Tests read it to see that they reached the
// variant they mean to check.
int g_last_decode_variant = 0;

constexpr int kMaxClusterSplits = 8;      // the portable cluster size; clusters of 16 measured slower than 8 (12.1 -> 14.1 us at batch 1, 4,096 keys)
int g_decode_cluster = 1;

// Blocks of the single-token kernel with STAGES tile buffers that one SM holds at a time.
template <int D, int STAGES>
int decode_blocks_per_sm() {
    static int blocks = 0;
    if (blocks == 0) {
        blocks = -1;
        if (configure_decode<D, STAGES, false, false>() == THN_OK) {
            int n = 0;
            cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(
                &n, attention_decode_kernel<D, STAGES, false, false>, kThreads, decode_smem<D, STAGES>());
            if (e == cudaSuccess && n > 0) blocks = n; else cudaGetLastError();
        }
    }
    return blocks > 0 ? blocks : 1;
}

int sm_count() {
    static int sms = 0;
    if (sms == 0) {
        int device = 0;
        cudaGetDevice(&device);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) sms = 1;
    }
    return sms;
}

// How many clusters of c blocks of the single-token kernel (STAGES tile buffers, fused or not) the
// GPU holds at once.
template <int D, int STAGES, bool FUSED>
int decode_clusters_resident(int c) {
    static int resident[kMaxClusterSplits + 1] = {0};
    static bool known[kMaxClusterSplits + 1] = {false};
    if (c < 2 || c > kMaxClusterSplits) return 0;
    if (!known[c]) {
        known[c] = true;
        if (configure_decode<D, STAGES, FUSED, true>() != THN_OK) return 0;
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3(1, 64, (unsigned)c);
        config.blockDim = dim3(kThreads);
        config.dynamicSmemBytes = decode_smem<D, STAGES>();
        cudaLaunchAttribute attribute[1];
        attribute[0].id = cudaLaunchAttributeClusterDimension;
        attribute[0].val.clusterDim.x = 1;
        attribute[0].val.clusterDim.y = 1;
        attribute[0].val.clusterDim.z = (unsigned)c;
        config.attrs = attribute;
        config.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, attention_decode_kernel<D, STAGES, FUSED, true>, &config) != cudaSuccess) {
            cudaGetLastError();
            n = 0;
        }
        resident[c] = n;
    }
    return resident[c];
}

template <int D, int STAGES, bool FUSED, bool CLUSTER>
int launch_decode_with(void* out, float* part_o, float* part_ml, const void* q, const int* row_slot, const int* row_pos,
                       PagedKV kv, int n_seqs, int n_q, int n_splits, float scale, int window, int* counters, int* err,
                       cudaStream_t stream, const FusedInput& fused) {
    int configured = configure_decode<D, STAGES, FUSED, CLUSTER>();
    if (configured != THN_OK) return configured;
    g_last_decode_variant = STAGES * 10 + (CLUSTER ? 1 : 0);
    dim3 grid(n_seqs, kv.n_kv, n_splits);
    if (CLUSTER)      // the splits of a (sequence, kv head) as one cluster along z
        thn_launch_cluster(attention_decode_kernel<D, STAGES, FUSED, CLUSTER>, grid, kThreads, decode_smem<D, STAGES>(),
                           stream, dim3(1, 1, n_splits), (__nv_bfloat16*)out, part_o, part_ml, (const __nv_bfloat16*)q,
                           row_slot, row_pos, kv, n_q, n_splits, scale * kLog2e, window, counters, err, fused);
    else
        thn_launch(attention_decode_kernel<D, STAGES, FUSED, CLUSTER>, grid, kThreads, decode_smem<D, STAGES>(), stream,
                   (__nv_bfloat16*)out, part_o, part_ml, (const __nv_bfloat16*)q, row_slot, row_pos, kv, n_q, n_splits,
                   scale * kLog2e, window, counters, err, fused);
    return thn_launch_status(CLUSTER ? "attention_decode (cluster)" : "attention_decode");
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The cache entry as [pages * 2 * n_kv * 64 rows, head_dim] bfloat16 with boxes of 64 values x 64
// rows and the 128-byte swizzle.
bool make_kv_map(CUtensorMap* map, const void* base, long long n_pages, int n_kv, int head_dim) {
    static EncodeTiledFn encode = nullptr;
    if (encode == nullptr) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &result) != cudaSuccess ||
            result != cudaDriverEntryPointSuccess)
            return false;
        encode = (EncodeTiledFn)fn;
    }
    const cuuint64_t dims[2] = {(cuuint64_t)head_dim, (cuuint64_t)(n_pages * 2 * n_kv * kTile)};
    const cuuint64_t strides[1] = {(cuuint64_t)head_dim * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)kTile};
    const cuuint32_t elem[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int g_decode_stream = 1;           // 0: never; 1: when the pairs are more than its resident blocks; 2: whenever one split is asked for
int g_decode_stream_stages = 3;    // tile buffers of the streaming kernel: 3 or 6
int g_decode_stream_by_length = 1; // its pairs dealt out by length (0: in index order)
constexpr int kNotTaken = -1;      // launch_decode_stream leaves the step to the caller

template <int D, int STAGES, bool FUSED>
int launch_decode_stream(void* out, const void* q, const int* row_slot, const int* row_pos, PagedKV kv,
                         long long n_pages, int n_seqs, int n_q, float scale, int window, int* err, cudaStream_t stream,
                         const FusedInput& fused, int hints) {
    const int lengths_differ = hints & 1;
    const int G = n_q / kv.n_kv;
    // Ranking costs each block about a microsecond at its start and gains 9 % on lengths spread
    // over 64 to 2,048 keys: it is done where the caller says that the lengths differ.
    const int by_length = g_decode_stream_by_length && lengths_differ && n_seqs <= kStreamRankedSeqs;
    const size_t smem = stream_smem<D>(STAGES, G) + (by_length ? (size_t)((n_seqs + 1) & ~1) * 2 + (size_t)n_seqs * 4 : 0);
    static size_t reserved = 0;
    static int per_sm_for[17] = {0};
    auto kernel = attention_decode_stream_kernel<D, STAGES, FUSED>;
    if (smem > reserved) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            thn_set_error("attention_decode (streaming): cannot reserve %zu bytes of shared memory: %s", smem,
                          cudaGetErrorString(e));
            return (int)e;
        }
        reserved = smem;
    }
    if (per_sm_for[G] == 0) {
        int n = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, kStreamThreads, smem) != cudaSuccess || n < 1) {
            cudaGetLastError();
            n = 1;
        }
        per_sm_for[G] = n;
    }
    CUtensorMap map;
    if (!make_kv_map(&map, kv.base, n_pages, kv.n_kv, D)) {
        thn_set_error("attention_decode (streaming): cannot describe the cache entry to the copy engine");
        return THN_BAD_ARGUMENT;
    }
    // As many blocks as are resident at once, fewer if that spreads the pairs more evenly.
    const long long n_pairs = (long long)n_seqs * kv.n_kv, resident = (long long)sm_count() * per_sm_for[G];
    if (n_pairs <= resident && g_decode_stream < 2 && !(hints & 2)) return kNotTaken;     // nothing to stream across
    const long long rounds = (n_pairs + resident - 1) / resident;
    const int grid = (int)((n_pairs + rounds - 1) / rounds);
    g_last_decode_variant = STAGES * 10 + 2;
    thn_launch(kernel, dim3(grid), kStreamThreads, smem, stream, map, (__nv_bfloat16*)out, (const __nv_bfloat16*)q,
               row_slot, row_pos, kv, n_seqs, n_q, scale * kLog2e, window, err, fused, by_length);
    return thn_launch_status("attention_decode (streaming)");
}

// A block keeps STAGES - 1 tiles on their way while it works on one.  A block that has an SM to
// itself needs about five in flight for its share of the memory bandwidth; with more blocks on an
// SM each has less shared memory and needs less.  The deepest pipeline with which the whole grid
// is still resident at once is taken: it depends on the batch only, not on the lengths.
template <int D, bool FUSED = false>
int launch_decode(void* out, float* part_o, float* part_ml, const void* q, const int* row_slot, const int* row_pos,
                  PagedKV kv, int n_seqs, int n_q, int n_splits, float scale, int window, int* counters, int* err,
                  cudaStream_t stream, FusedInput fused = FusedInput{}, long long n_pages = 0, int hints = 1) {
#define THN_DECODE_ARGS out, part_o, part_ml, q, row_slot, row_pos, kv, n_seqs, n_q, n_splits, scale, window, counters, err, stream, fused
    const int n_pairs = n_seqs * kv.n_kv;
    if (counters != nullptr && n_splits >= 2 && n_splits <= kMaxClusterSplits && g_decode_cluster) {
        if (decode_clusters_resident<D, 6, FUSED>(n_splits) >= n_pairs) return launch_decode_with<D, 6, FUSED, true>(THN_DECODE_ARGS);
        if (decode_clusters_resident<D, 3, FUSED>(n_splits) >= n_pairs) return launch_decode_with<D, 3, FUSED, true>(THN_DECODE_ARGS);
        return launch_decode_with<D, 2, FUSED, true>(THN_DECODE_ARGS);
    }
    // One block per pair would be next.  With the cache entry's size known, the kernel that
    // streams several pairs through each resident block takes the step instead.
    // It pays where one block per pair would need a second pass (more pairs than the GPU holds
    // such blocks with two tile buffers each); below that, one block per pair was as fast or
    // faster: 2.74 / 2.93 / 3.09 against 2.77 / 3.04 / 3.14 ms per step at batch 32 / 40 / 48,
    // and 3.43 / 3.47 against 3.24 / 3.34 ms at batch 56 / 64 (Qwen3-4B sizes, 8 kv heads).
    // The caller may know better (hint 2: long sequences, where streaming won from about 128
    // pairs of 1,024 keys on: 4.38 against 4.76 ms per step at batch 24 with 4,096 keys).
    const bool second_pass = (long long)n_pairs > (long long)sm_count() * decode_blocks_per_sm<D, 2>();
    const bool asked_for = (hints & 2) != 0;
    if (n_splits == 1 && n_pages > 0 && (g_decode_stream == 2 || (g_decode_stream == 1 && (second_pass || asked_for)))) {
        const int taken = g_decode_stream_stages >= 6
            ? launch_decode_stream<D, 6, FUSED>(out, q, row_slot, row_pos, kv, n_pages, n_seqs, n_q, scale, window, err,
                                                stream, fused, hints)
            : launch_decode_stream<D, 3, FUSED>(out, q, row_slot, row_pos, kv, n_pages, n_seqs, n_q, scale, window, err,
                                                stream, fused, hints);
        if (taken != kNotTaken) return taken;
    }
    const long long n_blocks = (long long)n_pairs * n_splits, sms = sm_count();
    int status;
    // (One block per pair and more blocks than the GPU holds even with two buffers each: the step
    // takes a second pass anyway, and three buffers were faster then, 3.47 against 3.73 ms per step
    // at batch 64; with 40 and 48 sequences, one pass with two buffers, 3.00 and 3.13 against 3.23
    // and 3.41 ms.)
    if (n_blocks <= sms * decode_blocks_per_sm<D, 6>()) status = launch_decode_with<D, 6, FUSED, false>(THN_DECODE_ARGS);
    else if (n_blocks <= sms * decode_blocks_per_sm<D, 3>()) status = launch_decode_with<D, 3, FUSED, false>(THN_DECODE_ARGS);
    else if (n_blocks <= sms * decode_blocks_per_sm<D, 2>() || n_splits > 1) status = launch_decode_with<D, 2, FUSED, false>(THN_DECODE_ARGS);
    else status = launch_decode_with<D, 3, FUSED, false>(THN_DECODE_ARGS);
#undef THN_DECODE_ARGS
    if (status != THN_OK || n_splits == 1 || counters != nullptr) return status;
    thn_launch(attention_merge_kernel, n_seqs * n_q, D <= 64 ? 64 : 128, 0, stream, (__nv_bfloat16*)out, part_o, part_ml,
                                                                            n_splits, D);
    return thn_launch_status("attention_merge");
}

// Head sizes other than 64 and 128: the same single-token kernel with two tile buffers, the
// query prepared by the separate kernel; the splits meet in a cluster where all clusters of
// the step are resident, else through scratch memory.
template <int D>
int launch_decode_lite(void* out, float* part_o, float* part_ml, const void* q, const int* row_slot, const int* row_pos,
                       PagedKV kv, int n_seqs, int n_q, int n_splits, float scale, int window, int* counters, int* err,
                       cudaStream_t stream) {
    const FusedInput fused{};
#define THN_DECODE_ARGS out, part_o, part_ml, q, row_slot, row_pos, kv, n_seqs, n_q, n_splits, scale, window, counters, err, stream, fused
    if (counters != nullptr && n_splits >= 2 && n_splits <= kMaxClusterSplits && g_decode_cluster &&
        decode_clusters_resident<D, 2, false>(n_splits) >= n_seqs * kv.n_kv)
        return launch_decode_with<D, 2, false, true>(THN_DECODE_ARGS);
    const int status = launch_decode_with<D, 2, false, false>(THN_DECODE_ARGS);
#undef THN_DECODE_ARGS
    if (status != THN_OK || n_splits == 1 || counters != nullptr) return status;
    thn_launch(attention_merge_kernel, n_seqs * n_q, D <= 64 ? 64 : 128, 0, stream, (__nv_bfloat16*)out, part_o, part_ml,
               n_splits, D);
    return thn_launch_status("attention_merge");
}

// CALL(D) for the head size at hand.  64 and 128 have every variant; the other multiples of 16
// from 32 to 128 have the plain ones.
#define THN_FOR_HEAD_DIM(head_dim, CALL) \
    switch (head_dim) {                  \
        case 32: CALL(32);               \
        case 48: CALL(48);               \
        case 64: CALL(64);               \
        case 80: CALL(80);               \
        case 96: CALL(96);               \
        case 112: CALL(112);             \
        default: CALL(128);              \
    }

}  // namespace

// 1 if the tensor-core kernels take this shape (bfloat16 only), else 0: head sizes in steps of
// 16 from 32 to 128, pages of 64 tokens, at most 16 query heads per kv head.
THN_API int thn_attention_mma_supported(int head_dim, int page_size, int n_q, int n_kv) {
    return head_dim >= 32 && head_dim <= 128 && head_dim % 16 == 0 && page_size == kTile && n_kv > 0 &&
           n_q % n_kv == 0 && n_q / n_kv <= 16;
}

// 1 if thn_attention_decode_fused_bf16 takes this shape: as above, with a head size of 64 or 128.
THN_API int thn_attention_fused_supported(int head_dim, int page_size, int n_q, int n_kv) {
    return (head_dim == 64 || head_dim == 128) && thn_attention_mma_supported(head_dim, page_size, n_q, n_kv);
}

// Tile buffers * 10 + (1: cluster, 2: streaming) of the most recent decode attention launch of this process.
THN_API int thn_attention_decode_last_variant() { return g_last_decode_variant; }

// Rows of a row tile of the prompt kernel (see thn_attention_prefill_bf16).
THN_API int thn_attention_prefill_tile_rows() { return kPrefillRows; }

// Rows of a step that brings one or more tokens per sequence.  tile_row0[i] is the first
// packed row of tile i, tile_rows[i] (1..thn_attention_prefill_tile_rows()) the number of its rows; the rows of a tile are
// consecutive tokens of one sequence.  q, out [rows, n_q * head_dim] bfloat16.
THN_API int thn_attention_prefill_bf16(void* out, const void* q, const int* tile_row0, const int* tile_rows,
                                       int n_tiles, const int* row_slot, const int* row_pos, const void* kv_base,
                                       const int* block_table, int bt_stride, int n_kv, int page_size, int head_dim,
                                       int n_q, float scale, int window, int* err, cudaStream_t stream) {
    THN_CHECK_ARG(n_tiles >= 0 && n_q > 0, "attention_prefill: bad sizes");
    THN_UNSUPPORTED_IF(!thn_attention_mma_supported(head_dim, page_size, n_q, n_kv),
                       "attention_prefill: head_dim %d, page %d, heads %d/%d not supported by the tensor-core kernel",
                       head_dim, page_size, n_q, n_kv);
    if (n_tiles == 0) return THN_OK;
    PagedKV kv{kv_base, block_table, bt_stride, n_kv, page_size, head_dim};
#define CALL(D) return launch_prefill<D>(out, q, tile_row0, tile_rows, n_tiles, row_slot, row_pos, kv, n_q, scale, window, err, stream)
    THN_FOR_HEAD_DIM(head_dim, CALL)
#undef CALL
}

// Scratch floats needed by thn_attention_decode_bf16 for n_splits > 1: partial outputs
// [n_seqs * n_q * n_splits * head_dim] followed by (max, sum) pairs [n_seqs * n_q * n_splits * 2].
THN_API long long thn_attention_decode_scratch_floats(int n_seqs, int n_q, int n_splits, int head_dim) {
    if (n_splits <= 1) return 0;
    return (long long)n_seqs * n_q * n_splits * (head_dim + 2);
}

// Blocks of the decode kernel that one SM holds at a time (for choosing n_splits so that
// the grid is one wave).
THN_API int thn_attention_decode_blocks_per_sm(int head_dim) {
#define CALL(D) return decode_blocks_per_sm<D, 2>()
    THN_FOR_HEAD_DIM(head_dim, CALL)
#undef CALL
}

// 0: the splits of a sequence always meet in global memory; 1 (default): in a thread-block
// cluster's shared memory when there are at most thn_attention_decode_cluster_splits() of them.
THN_API void thn_set_decode_cluster(int enabled) { g_decode_cluster = enabled ? 1 : 0; }
THN_API int thn_attention_decode_cluster_splits() { return g_decode_cluster ? kMaxClusterSplits : 0; }

// Splits (2 .. 8, the blocks of one cluster) per (sequence, kv head) for a single-token step of
// n_pairs such pairs; 0: one block per pair.  As many as fill the SMs once with every cluster of
// the step resident (a cluster that has to wait for the first ones to end costs a whole second
// pass: 2.49 against 2.31 ms per step with 7 instead of 6 at batch 8), but clusters of more than
// six blocks only where they are so few that each block has an SM to itself.  Measured inside the
// decode step of the Qwen3-4B sizes on B200 (ms per step, 512-640 keys): batch 2: 2.245 / 2.187 /
// 2.205 with 4 / 6 / 8; batch 4: 2.236 / 2.227 / 2.240; batch 8: 2.327 / 2.294 / 2.306 with 4 / 5
// / 6; batch 16: 2.492 / 2.466 / 2.461 with 1 / 2 / 3.  (Timed alone, back to back, fewer and
// larger blocks look better than they are in the step: there the next launch overlaps them.)
THN_API int thn_attention_decode_one_wave_splits(int head_dim, int fused, int n_pairs) {
    if (!g_decode_cluster || n_pairs <= 0) return 0;
    const int sms = sm_count();
    const int per_sm = thn_attention_decode_blocks_per_sm(head_dim);
    const int most = n_pairs * kMaxClusterSplits * 2 <= sms ? kMaxClusterSplits : 6;
    auto resident = [&](int c) {
        if (fused && head_dim == 64) return decode_clusters_resident<64, 2, true>(c);
        if (fused && head_dim == 128) return decode_clusters_resident<128, 2, true>(c);
#define CALL(D) return decode_clusters_resident<D, 2, false>(c)
        THN_FOR_HEAD_DIM(head_dim, CALL)
#undef CALL
    };
    for (int c = std::min(most, per_sm * sms / n_pairs); c >= 2; --c)
        if (resident(c) >= n_pairs) return c;
    return 0;
}

// Which unsplit single-token steps the streaming kernel takes: 0: none (one block per pair);
// 1 (default): those with more (sequence, kv head) pairs than it has resident blocks; 2: all.
// stages: its tile buffers, 3 or 6.
// 1 unless the streaming kernel has been switched off.
THN_API int thn_attention_decode_streams() { return g_decode_stream != 0; }
THN_API void thn_set_decode_stream_order(int by_length) { g_decode_stream_by_length = by_length ? 1 : 0; }
THN_API void thn_set_decode_stream(int mode, int stages) {
    g_decode_stream = mode < 0 ? 0 : mode > 2 ? 2 : mode;
    g_decode_stream_stages = stages >= 6 ? 6 : 3;
}

// One token per sequence: row b is sequence b.  scratch may be null when n_splits == 1.
// n_pages: pages of the cache entry (0 if unknown: the kernels that need a map of it are left out).
// hints: what the caller knows of the step, as bits; no result depends on them.  1: the sequences
// differ in length (0: about equally long, and a kernel may skip what it would do to balance
// them).  2: the sequences are long and many enough for the streaming kernel (see launch_decode).
// counters: n_seqs * n_kv ints, zero before the first call and left zero, with which the
// last block of each (sequence, kv head) combines the splits itself; null: a second kernel
// combines them.
THN_API int thn_attention_decode_bf16(void* out, const void* q, const int* row_slot, const int* row_pos,
                                      const void* kv_base, const int* block_table, int bt_stride, int n_kv,
                                      int page_size, int head_dim, int n_seqs, int n_q, int n_splits, float scale,
                                      int window, float* scratch, int* counters, long long n_pages, int hints,
                                      int* err, cudaStream_t stream) {
    THN_CHECK_ARG(n_seqs >= 0 && n_q > 0 && n_splits >= 1 && n_splits <= 65535, "attention_decode: bad sizes");
    THN_CHECK_ARG(counters == nullptr || n_splits <= 32, "attention_decode: at most 32 splits with counters, got %d",
                  n_splits);
    THN_UNSUPPORTED_IF(!thn_attention_mma_supported(head_dim, page_size, n_q, n_kv),
                       "attention_decode: head_dim %d, page %d, heads %d/%d not supported by the tensor-core kernel",
                       head_dim, page_size, n_q, n_kv);
    THN_CHECK_ARG(n_splits == 1 || scratch != nullptr, "attention_decode: %d splits need scratch memory", n_splits);
    if (n_seqs == 0) return THN_OK;
    PagedKV kv{kv_base, block_table, bt_stride, n_kv, page_size, head_dim};
    float* part_o = scratch;
    float* part_ml = scratch ? scratch + (size_t)n_seqs * n_q * n_splits * head_dim : nullptr;
    if (head_dim == 64)
        return launch_decode<64>(out, part_o, part_ml, q, row_slot, row_pos, kv, n_seqs, n_q, n_splits, scale, window,
                                 counters, err, stream, FusedInput{}, n_pages, hints);
    if (head_dim == 128)
        return launch_decode<128>(out, part_o, part_ml, q, row_slot, row_pos, kv, n_seqs, n_q, n_splits, scale, window,
                                  counters, err, stream, FusedInput{}, n_pages, hints);
#define CALL(D) return launch_decode_lite<D>(out, part_o, part_ml, q, row_slot, row_pos, kv, n_seqs, n_q, n_splits, scale, window, counters, err, stream)
    THN_FOR_HEAD_DIM(head_dim, CALL)
#undef CALL
}

// The same with the q/k norm, the rotation and the cache write of the step's token inside the
// kernel: qkv [n_seqs, (n_q + 2 n_kv) * head_dim] bfloat16 is the raw output of the q/k/v
// product; gains [head_dim] bfloat16 (w_dtype THN_BF16) or float32; cos/sin [table_len,
// head_dim / 2].  With write_cache == 0 the cache already holds the step's token (a layer that
// reads another layer's cache) and only q is prepared.
THN_API int thn_attention_decode_fused_bf16(void* out, const void* qkv, const void* q_gain, const void* k_gain,
                                            int w_dtype, float eps, const float* cos_tab, const float* sin_tab,
                                            int table_len, int write_cache, const int* row_slot, const int* row_pos,
                                            void* kv_base, const int* block_table, int bt_stride, int n_kv,
                                            int page_size, int head_dim, int n_seqs, int n_q, int n_splits, float scale,
                                            int window, float* scratch, int* counters, long long n_pages,
                                            int hints, int* err, cudaStream_t stream) {
    THN_CHECK_ARG(n_seqs >= 0 && n_q > 0 && n_splits >= 1 && n_splits <= 65535, "attention_decode_fused: bad sizes");
    THN_CHECK_ARG(counters == nullptr || n_splits <= 32, "attention_decode_fused: at most 32 splits with counters, got %d",
                  n_splits);
    THN_UNSUPPORTED_IF(!thn_attention_fused_supported(head_dim, page_size, n_q, n_kv),
                       "attention_decode_fused: head_dim %d, page %d, heads %d/%d not supported by the fused kernel",
                       head_dim, page_size, n_q, n_kv);
    THN_CHECK_ARG(qkv && q_gain && k_gain && cos_tab && sin_tab, "attention_decode_fused: gains and angles, please");
    THN_CHECK_ARG(w_dtype == THN_BF16 || w_dtype == THN_F32, "attention_decode_fused: unknown gain dtype %d", w_dtype);
    THN_CHECK_ARG(n_splits == 1 || scratch != nullptr, "attention_decode_fused: %d splits need scratch memory", n_splits);
    if (n_seqs == 0) return THN_OK;
    PagedKV kv{kv_base, block_table, bt_stride, n_kv, page_size, head_dim};
    float* part_o = scratch;
    float* part_ml = scratch ? scratch + (size_t)n_seqs * n_q * n_splits * head_dim : nullptr;
    FusedInput fused{(const __nv_bfloat16*)qkv, q_gain, k_gain, cos_tab, sin_tab, eps, table_len, w_dtype == THN_F32,
                     write_cache};
    if (head_dim == 64)
        return launch_decode<64, true>(out, part_o, part_ml, nullptr, row_slot, row_pos, kv, n_seqs, n_q, n_splits, scale,
                                       window, counters, err, stream, fused, n_pages, hints);
    return launch_decode<128, true>(out, part_o, part_ml, nullptr, row_slot, row_pos, kv, n_seqs, n_q, n_splits, scale,
                                    window, counters, err, stream, fused, n_pages, hints);
}

// ------------------------------------------------------------------ no device allocation

#include <mutex>

#include "attention_no_alloc.h"

namespace {

// Scratch of thn_attention_decode_bf16_no_alloc.  In host code this name is only a handle
// for cudaGetSymbolAddress; the address a kernel can use is looked up once per device.
static __device__ __align__(256) float g_no_alloc_scratch[THN_NO_ALLOC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
float* g_no_alloc_address[kMaxDevices] = {};
std::mutex g_no_alloc_mutex;

// The device address of the scratch array on the current device, or null with the error set.
float* no_alloc_scratch_address() {
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess || device < 0 || device >= kMaxDevices) {
        thn_set_error("attention_decode_no_alloc: cannot tell the current device (%s)",
                      e == cudaSuccess ? "index out of range" : cudaGetErrorString(e));
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(g_no_alloc_mutex);
    if (g_no_alloc_address[device] == nullptr) {
        float* address = nullptr;
        e = cudaGetSymbolAddress((void**)&address, g_no_alloc_scratch);
        if (e != cudaSuccess || address == nullptr) {
            thn_set_error("attention_decode_no_alloc: cudaGetSymbolAddress failed on device %d: %s", device,
                          cudaGetErrorString(e));
            return nullptr;
        }
        g_no_alloc_address[device] = address;
    }
    return g_no_alloc_address[device];
}

}  // namespace

THN_API int thn_attention_decode_bf16_no_alloc(void* out, const void* q, const int* row_slot, const int* row_pos,
                                               const void* kv_base, const int* block_table, int bt_stride, int n_kv,
                                               int page_size, int head_dim, int n_seqs, int n_q, int n_splits,
                                               float scale, int window, int* err, cudaStream_t stream) {
    THN_CHECK_ARG(n_seqs >= 0 && n_q > 0 && n_splits >= 1 && n_splits <= 65535 && head_dim > 0,
                  "attention_decode_no_alloc: bad sizes");
    const long long need = thn_attention_decode_scratch_floats(n_seqs, n_q, n_splits, head_dim);
    THN_CHECK_ARG(need <= THN_NO_ALLOC_SCRATCH_FLOATS,
                  "attention_decode_no_alloc: %d sequences x %d heads x %d splits x head size %d need %lld floats of "
                  "scratch, the built-in array holds %d; use fewer splits, or thn_attention_decode_bf16 with "
                  "scratch of your own", n_seqs, n_q, n_splits, head_dim, need, THN_NO_ALLOC_SCRATCH_FLOATS);
    float* scratch = nullptr;
    if (need > 0) {
        scratch = no_alloc_scratch_address();
        if (scratch == nullptr) return THN_BAD_ARGUMENT;
    }
    return thn_attention_decode_bf16(out, q, row_slot, row_pos, kv_base, block_table, bt_stride, n_kv, page_size,
                                     head_dim, n_seqs, n_q, n_splits, scale, window, scratch, nullptr, /*n_pages=*/0, /*hints=*/1, err,
                                     stream);
}
