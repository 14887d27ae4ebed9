// Fused per-head RMSNorm of q and k, rotary position encoding, and the write of K and V
// into the paged cache.  One warp per (row, head).
//
// Formulas: engine/kernels/torch_ref.py:141-162 (column layout Nq q heads, Nkv k heads,
// Nkv v heads; norm before rotation; V copied untouched) and :94-104 (rotation:
// out = rnd(rnd(x*cos) + rnd(rotate_half(x)*sin)), rotate_half(x) = cat(-x[D/2:], x[:D/2])).
// The angle tables are float32 (engine/engine.py:238-247); with bfloat16 activations
// cos and sin are rounded to bfloat16 as the reference's tables are (:246-247).
#include "common.cuh"

constexpr int kMaxHeadDim = 512;

template <typename T, typename WT>
__global__ void qk_norm_rope_cache_kernel(
    T* __restrict__ q_out, const T* __restrict__ qkv, const WT* __restrict__ q_gain, const WT* __restrict__ k_gain,
    float eps, const float* __restrict__ cos_tab, const float* __restrict__ sin_tab, int table_len, int rotary_dim,
    const int* __restrict__ row_slot, const int* __restrict__ row_pos, PagedKV kv, int n_rows, int n_q, int write_cache,
    int* __restrict__ err) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float smem[];
    const int lane = threadIdx.x & 31, warp_in_block = threadIdx.x >> 5;
    const int n_heads_total = n_q + 2 * kv.n_kv;
    const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + warp_in_block;
    if (unit >= (long long)n_rows * n_heads_total) return;
    const int m = (int)(unit / n_heads_total), head = (int)(unit - (long long)m * n_heads_total);
    const int D = kv.head_dim;
    const bool is_q = head < n_q, is_k = !is_q && head < n_q + kv.n_kv;
    if (!is_q && !write_cache) return;
    float* buf = smem + warp_in_block * D;
    const long long src = (long long)m * n_heads_total * D + (long long)head * D;
    const int pos = row_pos[m];

    T* dst;
    if (is_q) {
        dst = q_out + (size_t)m * n_q * D + (size_t)head * D;
    } else {
        const int kvh = is_k ? head - n_q : head - n_q - kv.n_kv;
        const int page = kv.block_table[(size_t)row_slot[m] * kv.bt_stride + pos / kv.page_size];
        if (page < 0) {
            if (lane == 0 && err) atomicOr(err, THN_ERR_PAGE_UNMAPPED);
            return;
        }
        dst = (T*)kv.base + kv_offset(kv, page, is_k ? 0 : 1, kvh, pos % kv.page_size);
    }

    if (!is_q && !is_k) {  // V: plain copy
        for (int d = lane; d < D; d += 32) dst[d] = from_f32<T>(to_f32<T>(qkv[src + d]));
        return;
    }

    const WT* gain = is_q ? q_gain : k_gain;
    float ss = 0.f;
    for (int d = lane; d < D; d += 32) {
        const float v = to_f32<T>(qkv[src + d]);
        buf[d] = v;
        ss += v * v;
    }
    if (gain) {
        ss = warp_sum(ss);
        const float rstd = 1.0f / sqrtf(ss / (float)D + eps);
        for (int d = lane; d < D; d += 32) buf[d] = rnd<T>(to_f32<WT>(gain[d]) * rnd<T>(buf[d] * rstd));
    }
    __syncwarp();
    if (cos_tab == nullptr) {
        for (int d = lane; d < D; d += 32) dst[d] = from_f32<T>(buf[d]);
        return;
    }
    if (pos >= table_len) {
        if (lane == 0 && err) atomicOr(err, THN_ERR_POSITION_RANGE);
        return;
    }
    const int half = rotary_dim / 2;
    const float* c_row = cos_tab + (size_t)pos * half;
    const float* s_row = sin_tab + (size_t)pos * half;
    for (int d = lane; d < D; d += 32) {
        float out = buf[d];
        if (d < rotary_dim) {
            const int i = d < half ? d : d - half;
            const float c = rnd<T>(c_row[i]), s = rnd<T>(s_row[i]);
            const float rotated = d < half ? -buf[d + half] : buf[d - half];
            out = rnd<T>(rnd<T>(out * c) + rnd<T>(rotated * s));
        }
        dst[d] = from_f32<T>(out);
    }
}

// The serving case: bfloat16 tensor input, head sizes 64, 128 and 256, full rotation.  A lane
// owns E = D / 64 consecutive values in each half of the head, so the partner of every value
// it rotates is its own: no shared memory, 4-byte or wider accesses, same arithmetic.  A warp
// takes H consecutive heads of one row (their loads all in flight before the first is used);
// single-token steps use H = 1, so that every head has a warp of its own, and steps of more
// than kFewRows rows use the 16-byte kernel further down.
constexpr int kFewRows = 64;

template <typename WT, int D, int H>
__global__ void qk_norm_rope_cache_bf16_kernel(
    __nv_bfloat16* __restrict__ q_out, const __nv_bfloat16* __restrict__ qkv, const WT* __restrict__ q_gain,
    const WT* __restrict__ k_gain, float eps, const float* __restrict__ cos_tab, const float* __restrict__ sin_tab,
    int table_len, const int* __restrict__ row_slot, const int* __restrict__ row_pos, PagedKV kv, int n_rows, int n_q,
    int write_cache, int* __restrict__ err) {
    pdl_launch_dependents();
    pdl_wait();
    using B = __nv_bfloat16;
    constexpr int E = D / 64, kHalf = D / 2;
    const int lane = threadIdx.x & 31;
    const int n_heads_total = n_q + 2 * kv.n_kv;
    const int groups = (n_heads_total + H - 1) / H;
    const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= (long long)n_rows * groups) return;
    const int m = (int)(unit / groups), head0 = (int)(unit - (long long)m * groups) * H;
    const int n_here = min(H, (write_cache ? n_heads_total : n_q) - head0);
    if (n_here <= 0) return;
    const __nv_bfloat16* src = qkv + (size_t)m * n_heads_total * D + (size_t)head0 * D;
    const int d0 = lane * E;                       // this lane's values: [d0, d0 + E) and [kHalf + d0, ...)
    __nv_bfloat16 lo[H][E], hi[H][E];
#pragma unroll
    for (int i = 0; i < H; ++i) {
        if (i < n_here) {
#pragma unroll
            for (int e = 0; e < E; ++e) {
                lo[i][e] = src[(size_t)i * D + d0 + e];
                hi[i][e] = src[(size_t)i * D + kHalf + d0 + e];
            }
        }
    }
    const int pos = row_pos[m];
    if (pos >= table_len) {
        if (lane == 0 && err) atomicOr(err, THN_ERR_POSITION_RANGE);
        return;
    }
    float c[E], sn[E];
#pragma unroll
    for (int e = 0; e < E; ++e) {
        c[e] = rnd<B>(cos_tab[(size_t)pos * kHalf + d0 + e]);
        sn[e] = rnd<B>(sin_tab[(size_t)pos * kHalf + d0 + e]);
    }
    int page = 0;
    if (head0 + n_here > n_q) {
        page = kv.block_table[(size_t)row_slot[m] * kv.bt_stride + pos / kv.page_size];
        if (page < 0) {
            if (lane == 0 && err) atomicOr(err, THN_ERR_PAGE_UNMAPPED);
            return;
        }
    }
#pragma unroll
    for (int i = 0; i < H; ++i) {
        if (i >= n_here) break;
        const int head = head0 + i;                // the same for the whole warp
        const bool is_q = head < n_q, is_k = !is_q && head < n_q + kv.n_kv;
        __nv_bfloat16* dst;
        if (is_q) {
            dst = q_out + (size_t)m * n_q * D + (size_t)head * D;
        } else {
            const int kvh = is_k ? head - n_q : head - n_q - kv.n_kv;
            dst = (__nv_bfloat16*)kv.base + kv_offset(kv, page, is_k ? 0 : 1, kvh, pos % kv.page_size);
        }
        if (!is_q && !is_k) {                      // V: plain copy
#pragma unroll
            for (int e = 0; e < E; ++e) {
                dst[d0 + e] = lo[i][e];
                dst[kHalf + d0 + e] = hi[i][e];
            }
            continue;
        }
        const WT* gain = is_q ? q_gain : k_gain;
        float a[E], b[E], ss = 0.f;
#pragma unroll
        for (int e = 0; e < E; ++e) {
            a[e] = __bfloat162float(lo[i][e]);
            b[e] = __bfloat162float(hi[i][e]);
            ss += a[e] * a[e] + b[e] * b[e];
        }
        ss = warp_sum(ss);
        const float rstd = 1.0f / sqrtf(ss / (float)D + eps);
#pragma unroll
        for (int e = 0; e < E; ++e) {
            const float x0 = rnd<B>(to_f32<WT>(gain[d0 + e]) * rnd<B>(a[e] * rstd));
            const float x1 = rnd<B>(to_f32<WT>(gain[kHalf + d0 + e]) * rnd<B>(b[e] * rstd));
            dst[d0 + e] = __float2bfloat16_rn(rnd<B>(x0 * c[e]) + rnd<B>(-x1 * sn[e]));
            dst[kHalf + d0 + e] = __float2bfloat16_rn(rnd<B>(x1 * c[e]) + rnd<B>(x0 * sn[e]));
        }
    }
}

// Steps of many rows (prompts): the same arithmetic with 16-byte accesses.  A head is spread
// over L = D / 8 lanes, eight consecutive values each, so a warp takes 32 / L heads per pass
// and kVecPasses passes whose loads are all in flight together; the value a lane rotates with
// lives L / 2 lanes away and comes by shuffle; the sum of squares is reduced over the L
// lanes of the head.
constexpr int kVecPasses = 4;

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __bfloat1622float2(p[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}

template <typename WT>
__device__ __forceinline__ void load_gain8(const WT* gain, int d, float (&g)[8]);
template <>
__device__ __forceinline__ void load_gain8<__nv_bfloat16>(const __nv_bfloat16* gain, int d, float (&g)[8]) {
    unpack8(*reinterpret_cast<const uint4*>(gain + d), g);
}
template <>
__device__ __forceinline__ void load_gain8<float>(const float* gain, int d, float (&g)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(gain + d), b = *reinterpret_cast<const float4*>(gain + d + 4);
    g[0] = a.x; g[1] = a.y; g[2] = a.z; g[3] = a.w; g[4] = b.x; g[5] = b.y; g[6] = b.z; g[7] = b.w;
}

template <typename WT, int D>
__global__ void qk_norm_rope_cache_bf16_vec_kernel(
    __nv_bfloat16* __restrict__ q_out, const __nv_bfloat16* __restrict__ qkv, const WT* __restrict__ q_gain,
    const WT* __restrict__ k_gain, float eps, const float* __restrict__ cos_tab, const float* __restrict__ sin_tab,
    int table_len, const int* __restrict__ row_slot, const int* __restrict__ row_pos, PagedKV kv, int n_rows, int n_q,
    int write_cache, int* __restrict__ err) {
    pdl_launch_dependents();
    pdl_wait();
    using B = __nv_bfloat16;
    constexpr int L = D / 8, kHalf = D / 2, kPerPass = 32 / L, kPerWarp = kPerPass * kVecPasses;
    const int lane = threadIdx.x & 31;
    const int n_heads_total = n_q + 2 * kv.n_kv;
    const int n_used = write_cache ? n_heads_total : n_q;
    const int groups = (n_used + kPerWarp - 1) / kPerWarp;
    const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= (long long)n_rows * groups) return;
    const int m = (int)(unit / groups), head0 = (int)(unit - (long long)m * groups) * kPerWarp;
    const int sub = lane / L, l = lane % L;            // which head of the pass, which eighth of it
    const int d = 8 * l;                               // this lane's values: [d, d + 8)
    const __nv_bfloat16* row = qkv + (size_t)m * n_heads_total * D;

    uint4 raw[kVecPasses];
#pragma unroll
    for (int p = 0; p < kVecPasses; ++p) {
        const int head = head0 + p * kPerPass + sub;
        raw[p] = head < n_used ? *reinterpret_cast<const uint4*>(row + (size_t)head * D + d) : make_uint4(0, 0, 0, 0);
    }
    const int pos = row_pos[m];
    if (pos >= table_len) {
        if (lane == 0 && err) atomicOr(err, THN_ERR_POSITION_RANGE);
        return;
    }
    // angles of this lane's values: index d mod D/2 in the row's table
    // (a bfloat16 product of two bfloat16 values is their exact product rounded once, which
    // is what rounding the float32 product gives: the paired instructions do four roundings of
    // the reference's formula at a quarter of the instructions)
    __nv_bfloat162 c2[4], s2[4];
    {
        const float* cr = cos_tab + (size_t)pos * kHalf + (d % kHalf);
        const float* sr = sin_tab + (size_t)pos * kHalf + (d % kHalf);
        const float4 c0 = *reinterpret_cast<const float4*>(cr), c1 = *reinterpret_cast<const float4*>(cr + 4);
        const float4 s0 = *reinterpret_cast<const float4*>(sr), s1 = *reinterpret_cast<const float4*>(sr + 4);
        const float cc[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        const float ss[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            c2[i] = __floats2bfloat162_rn(cc[2 * i], cc[2 * i + 1]);
            s2[i] = __floats2bfloat162_rn(ss[2 * i], ss[2 * i + 1]);
        }
    }
    int page = 0;
    if (head0 + kPerWarp > n_q && write_cache) {
        page = kv.block_table[(size_t)row_slot[m] * kv.bt_stride + pos / kv.page_size];
        if (page < 0) {
            if (lane == 0 && err) atomicOr(err, THN_ERR_PAGE_UNMAPPED);
            return;
        }
    }
    const bool upper = d >= kHalf;                     // this lane holds the second half of the head
#pragma unroll
    for (int p = 0; p < kVecPasses; ++p) {
        const int head = head0 + p * kPerPass + sub;   // may differ between the lanes of a warp
        const bool live = head < n_used;
        const bool is_q = head < n_q, is_k = !is_q && head < n_q + kv.n_kv;
        float x[8];
        unpack8(raw[p], x);
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += x[i] * x[i];
#pragma unroll
        for (int off = 1; off < L; off <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
        const float rstd = 1.0f / sqrtf(ss / (float)D + eps);
        float g[8];
        load_gain8<WT>(is_q ? q_gain : k_gain, d, g);
        uint4 mine;                                    // gain * normalised value, rounded, as bfloat16 pairs
        {
            __nv_bfloat162* mp = reinterpret_cast<__nv_bfloat162*>(&mine);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const __nv_bfloat162 normed = __floats2bfloat162_rn(x[2 * i] * rstd, x[2 * i + 1] * rstd);
                if (sizeof(WT) == 2) {
                    mp[i] = __hmul2(__floats2bfloat162_rn(g[2 * i], g[2 * i + 1]), normed);
                } else {                               // float32 gains: the product is rounded from float32
                    const float2 nf = __bfloat1622float2(normed);
                    mp[i] = __floats2bfloat162_rn(g[2 * i] * nf.x, g[2 * i + 1] * nf.y);
                }
            }
        }
        uint4 other;                                   // the same of the lane L / 2 away
        other.x = __shfl_xor_sync(0xffffffffu, mine.x, L / 2);
        other.y = __shfl_xor_sync(0xffffffffu, mine.y, L / 2);
        other.z = __shfl_xor_sync(0xffffffffu, mine.z, L / 2);
        other.w = __shfl_xor_sync(0xffffffffu, mine.w, L / 2);
        if (!live) continue;
        __nv_bfloat16* dst;
        if (is_q) {
            dst = q_out + (size_t)m * n_q * D + (size_t)head * D + d;
        } else {
            const int kvh = is_k ? head - n_q : head - n_q - kv.n_kv;
            dst = (__nv_bfloat16*)kv.base + kv_offset(kv, page, is_k ? 0 : 1, kvh, pos % kv.page_size) + d;
        }
        if (!is_q && !is_k) {                          // V: plain copy
            *reinterpret_cast<uint4*>(dst) = raw[p];
            continue;
        }
        const __nv_bfloat162* ap = reinterpret_cast<const __nv_bfloat162*>(&mine);
        const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&other);
        uint4 res;
        __nv_bfloat162* rp = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            // first half: x0 * c - x1 * s with x1 from the partner; second half: x1 * c + x0 * s
            const float2 p1 = __bfloat1622float2(__hmul2(ap[i], c2[i]));
            const float2 p2 = __bfloat1622float2(__hmul2(upper ? bp[i] : __hneg2(bp[i]), s2[i]));
            rp[i] = __floats2bfloat162_rn(p1.x + p2.x, p1.y + p2.y);       // the sum in float32, rounded once
        }
        *reinterpret_cast<uint4*>(dst) = res;
    }
}

// qkv [n_rows, (n_q + 2*n_kv) * head_dim] -> q_out [n_rows, n_q * head_dim]; K and V of
// every row go to (slot, position) of the cache entry unless write_cache == 0.
// q_gain/k_gain may be null (no head norm); cos_tab may be null (no rotation).
THN_API int thn_qk_norm_rope_cache(void* q_out, const void* qkv,
                                   const void* q_gain, const void* k_gain, int w_dtype,
                                   float eps, const float* cos_tab, const float* sin_tab, int table_len,
                                   int rotary_dim, const int* row_slot, const int* row_pos, void* kv_base,
                                   const int* block_table, int bt_stride, int n_kv, int page_size, int head_dim,
                                   int n_rows, int n_q, int write_cache, int dtype, int* err, cudaStream_t stream) {
    THN_CHECK_ARG(n_rows >= 0 && n_q > 0 && n_kv > 0 && page_size > 0, "qk_norm_rope_cache: bad sizes");
    THN_UNSUPPORTED_IF(head_dim <= 0 || head_dim > kMaxHeadDim, "qk_norm_rope_cache: head_dim %d not in [1, %d]",
                       head_dim, kMaxHeadDim);
    THN_CHECK_ARG(rotary_dim >= 0 && rotary_dim <= head_dim && rotary_dim % 2 == 0,
                  "qk_norm_rope_cache: rotary_dim %d must be even and <= head_dim %d", rotary_dim, head_dim);
    THN_CHECK_ARG((q_gain == nullptr) == (k_gain == nullptr), "qk_norm_rope_cache: q and k gains come together");
    THN_CHECK_ARG(qkv != nullptr, "qk_norm_rope_cache: no q/k/v rows");
    if (n_rows == 0) return THN_OK;
    PagedKV kv{kv_base, block_table, bt_stride, n_kv, page_size, head_dim};
    const int warps = 4;
    const long long units = (long long)n_rows * (n_q + 2 * n_kv);
    const unsigned blocks = (unsigned)((units + warps - 1) / warps);
    const size_t smem = (size_t)warps * head_dim * sizeof(float);
    if (dtype == THN_BF16 && q_gain && cos_tab && rotary_dim == head_dim &&
        (head_dim == 64 || head_dim == 128 || head_dim == 256)) {
        const bool many = n_rows > kFewRows && (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)kv_base |
                                                  (uintptr_t)q_gain | (uintptr_t)k_gain | (uintptr_t)cos_tab |
                                                  (uintptr_t)sin_tab) & 15) == 0;
        const int per_pass = 32 / (head_dim / 8);
        const int n_used = write_cache ? n_q + 2 * n_kv : n_q;
        const long long fast_units = many ? (long long)n_rows * ((n_used + per_pass * kVecPasses - 1) / (per_pass * kVecPasses))
                                          : (long long)n_rows * (n_q + 2 * n_kv);
        const unsigned fast_blocks = (unsigned)((fast_units + warps - 1) / warps);
#define FAST_ARGS(WT)                                                                                               \
    (__nv_bfloat16*)q_out, (const __nv_bfloat16*)qkv, (const WT*)q_gain, (const WT*)k_gain, eps, cos_tab, sin_tab,  \
        table_len, row_slot, row_pos, kv, n_rows, n_q, write_cache, err
#define FAST(WT, D)                                                                                                 \
    do {                                                                                                            \
        if (many) thn_launch(qk_norm_rope_cache_bf16_vec_kernel<WT, D>, fast_blocks, warps * 32, 0, stream, FAST_ARGS(WT)); \
        else thn_launch(qk_norm_rope_cache_bf16_kernel<WT, D, 1>, fast_blocks, warps * 32, 0, stream, FAST_ARGS(WT)); \
    } while (0)
        bool done = true;
        if (w_dtype == THN_BF16 && head_dim == 64) FAST(__nv_bfloat16, 64);
        else if (w_dtype == THN_BF16 && head_dim == 128) FAST(__nv_bfloat16, 128);
        else if (w_dtype == THN_BF16 && head_dim == 256) FAST(__nv_bfloat16, 256);
        else if (w_dtype == THN_F32 && head_dim == 64) FAST(float, 64);
        else if (w_dtype == THN_F32 && head_dim == 128) FAST(float, 128);
        else if (w_dtype == THN_F32 && head_dim == 256) FAST(float, 256);
        else done = false;
#undef FAST
#undef FAST_ARGS
        if (done) return thn_launch_status("qk_norm_rope_cache");
    }
#define LAUNCH(T, WT)                                                                                              \
    thn_launch(qk_norm_rope_cache_kernel<T, WT>, blocks, warps * 32, smem, stream, \
        (T*)q_out, (const T*)qkv, (const WT*)q_gain,                                                                \
        (const WT*)k_gain, eps, cos_tab, sin_tab, table_len,                                                       \
        rotary_dim, row_slot, row_pos, kv, n_rows, n_q, write_cache, err)
    if (dtype == THN_F32 && w_dtype == THN_F32) LAUNCH(float, float);
    else if (dtype == THN_BF16 && w_dtype == THN_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else if (dtype == THN_BF16 && w_dtype == THN_F32) LAUNCH(__nv_bfloat16, float);
    else THN_CHECK_ARG(false, "qk_norm_rope_cache: unsupported dtypes activation=%d gain=%d", dtype, w_dtype);
#undef LAUNCH
    return thn_launch_status("qk_norm_rope_cache");
}
