// Row gather (embedding), RMSNorm with and without the residual add, SwiGLU, and the
// small kernels that turn a step's batch description into per-row indices.
//
// Formulas and rounding points: engine/kernels/torch_ref.py:47-58 (RMSNorm: the
// normalised value is rounded before the gain), :61-68 (residual add rounded once),
// :74-88 (silu rounded, product rounded).  Reductions are float32 with an order fixed
// by the block size, so a row's result does not depend on the batch it is in.
#include <cstdarg>
#include <cstdio>

#include "common.cuh"

static thread_local char g_error[512] = "";

void thn_set_error(const char* fmt, ...) {
    va_list args;
    va_start(args, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, args);
    va_end(args);
}

int g_thn_pdl = 1;

// 0: plain launches; 1 (default): kernels may be scheduled while their predecessor drains.
THN_API void thn_set_pdl(int enabled) { g_thn_pdl = enabled ? 1 : 0; }

THN_API const char* thn_last_error() { return g_error; }
THN_API int thn_abi_version() { return 1; }

// ------------------------------------------------------------------ gather rows

template <typename T>
__global__ void gather_rows_kernel(T* __restrict__ out, const T* __restrict__ table, const int* __restrict__ index,
                                   int width, int n_table_rows, int* __restrict__ err) {
    pdl_launch_dependents();
    pdl_wait();
    const int m = blockIdx.x;
    int row = index[m];
    if (row < 0 || row >= n_table_rows) {
        if (threadIdx.x == 0 && err) atomicOr(err, THN_ERR_TOKEN_RANGE);
        row = 0;
    }
    const T* src = table + (size_t)row * width;
    T* dst = out + (size_t)m * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = src[i];
}

THN_API int thn_gather_rows(void* out, const void* table, const int* index, int n_rows, int width,
                            int n_table_rows, int dtype, int* err, cudaStream_t stream) {
    THN_CHECK_ARG(n_rows >= 0 && width > 0 && n_table_rows > 0, "gather_rows: bad sizes rows=%d width=%d table=%d",
                  n_rows, width, n_table_rows);
    if (n_rows == 0) return THN_OK;
    if (dtype == THN_F32)
        thn_launch(gather_rows_kernel<float>, n_rows, 256, 0, stream, (float*)out, (const float*)table, index, width,
                                                              n_table_rows, err);
    else if (dtype == THN_BF16)
        thn_launch(gather_rows_kernel<__nv_bfloat16>, n_rows, 256, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)table, index, width, n_table_rows, err);
    else
        THN_CHECK_ARG(false, "gather_rows: unknown dtype %d", dtype);
    return thn_launch_status("gather_rows");
}

// ------------------------------------------------------------------ RMSNorm

constexpr int kNormThreads = 256;
constexpr int kNormKeep = 16;   // values a thread keeps in registers between the two passes

// y = w * rnd(v * rstd), rstd = 1/sqrt(mean(v^2) + eps).  v = h, or with a branch output d:
// v = rnd(h + d), stored back to h first.  One block per row.
template <typename T, typename WT, bool ADD>
__global__ void __launch_bounds__(kNormThreads) rmsnorm_kernel(T* __restrict__ y, T* __restrict__ h,
                                                               const T* __restrict__ d, const WT* __restrict__ w, int width,
                                                               float eps) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[33];
    const size_t base = (size_t)blockIdx.x * width;
    float keep[kNormKeep];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < kNormKeep; ++j) {
        const int i = threadIdx.x + j * kNormThreads;
        float v = 0.f;
        if (i < width) {
            v = to_f32<T>(h[base + i]);
            if (ADD) {
                v = rnd<T>(v + to_f32<T>(d[base + i]));
                h[base + i] = from_f32<T>(v);
            }
        }
        keep[j] = v;
        ss += v * v;
    }
    for (int i = threadIdx.x + kNormKeep * kNormThreads; i < width; i += kNormThreads) {
        float v = to_f32<T>(h[base + i]);
        if (ADD) {
            v = rnd<T>(v + to_f32<T>(d[base + i]));
            h[base + i] = from_f32<T>(v);
        }
        ss += v * v;
    }
    const float total = block_sum(ss, scratch);
    const float rstd = 1.0f / sqrtf(total / (float)width + eps);
#pragma unroll
    for (int j = 0; j < kNormKeep; ++j) {
        const int i = threadIdx.x + j * kNormThreads;
        if (i < width) y[base + i] = from_f32<T>(to_f32<WT>(w[i]) * rnd<T>(keep[j] * rstd));
    }
    for (int i = threadIdx.x + kNormKeep * kNormThreads; i < width; i += kNormThreads) {
        const float v = to_f32<T>(h[base + i]);
        y[base + i] = from_f32<T>(to_f32<WT>(w[i]) * rnd<T>(v * rstd));
    }
}

// The common serving case, bfloat16 rows of up to 8192 values with width % 8 == 0: one
// 16-byte vector per thread, every load issued before the first use, same arithmetic and
// rounding as the kernel above.  blockDim depends on the width only.
template <typename WT, bool ADD>
__global__ void __launch_bounds__(1024) rmsnorm_bf16_vec_kernel(__nv_bfloat16* __restrict__ y,
                                                                __nv_bfloat16* __restrict__ h,
                                                                const __nv_bfloat16* __restrict__ d,
                                                                const WT* __restrict__ w, int width, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[33];
    const size_t base = (size_t)blockIdx.x * width;
    const int i0 = threadIdx.x * 8;
    const bool live = i0 < width;
    uint4 hv = make_uint4(0, 0, 0, 0), dv = make_uint4(0, 0, 0, 0);
    float gain[8];
    if (live) {
        hv = *reinterpret_cast<const uint4*>(h + base + i0);
        if (ADD) dv = *reinterpret_cast<const uint4*>(d + base + i0);
        if (sizeof(WT) == 2) {
            const uint4 wv = *reinterpret_cast<const uint4*>(w + i0);
            const __nv_bfloat16* wb = reinterpret_cast<const __nv_bfloat16*>(&wv);
#pragma unroll
            for (int j = 0; j < 8; ++j) gain[j] = __bfloat162float(wb[j]);
        } else {
            const float4 w0 = *reinterpret_cast<const float4*>(w + i0);
            const float4 w1 = *reinterpret_cast<const float4*>(w + i0 + 4);
            gain[0] = w0.x; gain[1] = w0.y; gain[2] = w0.z; gain[3] = w0.w;
            gain[4] = w1.x; gain[5] = w1.y; gain[6] = w1.z; gain[7] = w1.w;
        }
    }
    const __nv_bfloat16* hb = reinterpret_cast<const __nv_bfloat16*>(&hv);
    const __nv_bfloat16* db = reinterpret_cast<const __nv_bfloat16*>(&dv);
    float v[8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        v[j] = __bfloat162float(hb[j]);
        if (ADD) v[j] = rnd<__nv_bfloat16>(v[j] + __bfloat162float(db[j]));
        ss += v[j] * v[j];
    }
    if (ADD && live) {
        uint4 out;
        __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(&out);
#pragma unroll
        for (int j = 0; j < 8; ++j) ob[j] = __float2bfloat16_rn(v[j]);
        *reinterpret_cast<uint4*>(h + base + i0) = out;
    }
    const float total = block_sum(ss, scratch);
    const float rstd = 1.0f / sqrtf(total / (float)width + eps);
    if (live) {
        uint4 out;
        __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(&out);
#pragma unroll
        for (int j = 0; j < 8; ++j) ob[j] = __float2bfloat16_rn(gain[j] * rnd<__nv_bfloat16>(v[j] * rstd));
        *reinterpret_cast<uint4*>(y + base + i0) = out;
    }
}

template <typename WT>
static bool launch_rmsnorm_vec(void* y, void* h, const void* d, const void* w, int rows,
                               int width, float eps, cudaStream_t stream) {
    if (width % 8 || width > 8192 || (((uintptr_t)y | (uintptr_t)h | (uintptr_t)d | (uintptr_t)w) & 15))
        return false;
    const int threads = ((width / 8 + 31) / 32) * 32;
    if (d)
        thn_launch(rmsnorm_bf16_vec_kernel<WT, true>, rows, threads, 0, stream, (__nv_bfloat16*)y, (__nv_bfloat16*)h, (const __nv_bfloat16*)d, (const WT*)w, width, eps);
    else
        thn_launch(rmsnorm_bf16_vec_kernel<WT, false>, rows, threads, 0, stream, (__nv_bfloat16*)y, (__nv_bfloat16*)h, nullptr, (const WT*)w, width, eps);
    return true;
}

template <typename T, typename WT>
static void launch_rmsnorm(void* y, void* h, const T* d, const void* w, int rows, int width, float eps,
                           cudaStream_t stream) {
    if (d)
        thn_launch(rmsnorm_kernel<T, WT, true>, rows, kNormThreads, 0, stream, (T*)y, (T*)h, d, (const WT*)w, width, eps);
    else
        thn_launch(rmsnorm_kernel<T, WT, false>, rows, kNormThreads, 0, stream, (T*)y, (T*)h, d, (const WT*)w, width, eps);
}

// y = RMSNorm(h).  With d (a tensor of h's type): h is updated in place to rnd(h + d) first.
THN_API int thn_rmsnorm(void* y, void* h, const void* d, const void* w, int rows, int width, float eps, int dtype,
                        int w_dtype, cudaStream_t stream) {
    THN_CHECK_ARG(rows >= 0 && width > 0, "rmsnorm: bad sizes rows=%d width=%d", rows, width);
    THN_CHECK_ARG(eps > 0.f, "rmsnorm: eps must be positive, got %g", (double)eps);
    if (rows == 0) return THN_OK;
    if (dtype == THN_F32 && w_dtype == THN_F32)
        launch_rmsnorm<float, float>(y, h, (const float*)d, w, rows, width, eps, stream);
    else if (dtype == THN_BF16 && w_dtype == THN_BF16 &&
             launch_rmsnorm_vec<__nv_bfloat16>(y, h, d, w, rows, width, eps, stream)) {
    } else if (dtype == THN_BF16 && w_dtype == THN_F32 && launch_rmsnorm_vec<float>(y, h, d, w, rows, width, eps, stream)) {
    } else if (dtype == THN_BF16 && w_dtype == THN_BF16)
        launch_rmsnorm<__nv_bfloat16, __nv_bfloat16>(y, h, (const __nv_bfloat16*)d, w, rows, width, eps, stream);
    else if (dtype == THN_BF16 && w_dtype == THN_F32)
        launch_rmsnorm<__nv_bfloat16, float>(y, h, (const __nv_bfloat16*)d, w, rows, width, eps, stream);
    else
        THN_CHECK_ARG(false, "rmsnorm: unsupported dtypes activation=%d gain=%d", dtype, w_dtype);
    return thn_launch_status("rmsnorm");
}

// ------------------------------------------------------------------ SwiGLU

// out[m, i] = rnd(rnd(g / (1 + exp(-g))) * u), g = gu[m, i], u = gu[m, inter + i].
template <typename T>
__global__ void swiglu_kernel(T* __restrict__ out, const T* __restrict__ gu, long long total, int inter) {
    pdl_launch_dependents();
    pdl_wait();
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
        const long long m = e / inter;
        const int i = (int)(e - m * inter);
        const float g = to_f32<T>(gu[m * 2 * inter + i]);
        const float u = to_f32<T>(gu[m * 2 * inter + inter + i]);
        const float s = rnd<T>(g / (1.0f + expf(-g)));
        out[e] = from_f32<T>(s * u);
    }
}

// bfloat16 tensor input with inter % 8 == 0: eight values per thread, 16-byte accesses.
__global__ void swiglu_bf16_vec_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ gu,
                                       long long total_vecs, int inter_vecs) {
    pdl_launch_dependents();
    pdl_wait();
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total_vecs; e += stride) {
        const long long m = e / inter_vecs;
        const int i = (int)(e - m * inter_vecs);
        const uint4 gv = *reinterpret_cast<const uint4*>(gu + (m * 2 * inter_vecs + i) * 8);
        const uint4 uv = *reinterpret_cast<const uint4*>(gu + (m * 2 * inter_vecs + inter_vecs + i) * 8);
        const __nv_bfloat16* gb = reinterpret_cast<const __nv_bfloat16*>(&gv);
        const __nv_bfloat16* ub = reinterpret_cast<const __nv_bfloat16*>(&uv);
        // silu in float32 with the fast exponential and reciprocal (a few float32 ulp, far below
        // the bfloat16 rounding that follows); the product of the two bfloat16 values with the
        // paired instruction, which rounds the exact product once as the reference's does.
        uint4 ov;
        __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&ov);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(gb);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(ub);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 g = __bfloat1622float2(g2[j]);
            const float s0 = __fdividef(g.x, 1.0f + __expf(-g.x)), s1 = __fdividef(g.y, 1.0f + __expf(-g.y));
            ob[j] = __hmul2(__floats2bfloat162_rn(s0, s1), u2[j]);
        }
        *reinterpret_cast<uint4*>(out + e * 8) = ov;
    }
}

// gu [rows, 2 * inter] (gate columns, then up columns) -> out [rows, inter].
THN_API int thn_swiglu(void* out, const void* gu, int rows, int inter, int dtype, cudaStream_t stream) {
    THN_CHECK_ARG(rows >= 0 && inter > 0, "swiglu: bad sizes rows=%d inter=%d", rows, inter);
    const long long total = (long long)rows * inter;
    if (total == 0) return THN_OK;
    const int threads = 256;
    const long long want = (total + threads - 1) / threads;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    if (dtype == THN_BF16 && inter % 8 == 0 && (((uintptr_t)gu | (uintptr_t)out) & 15) == 0) {
        const long long vecs = total / 8;
        const long long want_vec = (vecs + threads - 1) / threads;
        thn_launch(swiglu_bf16_vec_kernel, (unsigned)(want_vec < 148 * 32 ? want_vec : 148 * 32), threads, 0, stream,
                   (__nv_bfloat16*)out, (const __nv_bfloat16*)gu, vecs, inter / 8);
        return thn_launch_status("swiglu");
    }
    if (dtype == THN_F32)
        thn_launch(swiglu_kernel<float>, blocks, threads, 0, stream, (float*)out, (const float*)gu, total, inter);
    else if (dtype == THN_BF16)
        thn_launch(swiglu_kernel<__nv_bfloat16>, blocks, threads, 0, stream, (__nv_bfloat16*)out,
                   (const __nv_bfloat16*)gu, total, inter);
    else
        THN_CHECK_ARG(false, "swiglu: unknown dtype %d", dtype);
    return thn_launch_status("swiglu");
}

// ------------------------------------------------------------------ step bookkeeping

// Row m of a packed step belongs to sequence b with cu[b] <= m < cu[b+1]; its slot is
// slots[b] and its absolute position is seq_lens[slot] + (m - cu[b]).
__global__ void step_rows_kernel(int* __restrict__ row_slot, int* __restrict__ row_pos,
                                 const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
                                 const int* __restrict__ seq_lens, int n_seqs) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x;
    if (b >= n_seqs) return;
    const int r0 = cu_seqlens[b], r1 = cu_seqlens[b + 1];
    const int slot = slots[b];
    const int start = seq_lens[slot];
    for (int r = r0 + threadIdx.x; r < r1; r += blockDim.x) {
        row_slot[r] = slot;
        row_pos[r] = start + (r - r0);
    }
}

THN_API int thn_step_rows(int* row_slot, int* row_pos, const int* cu_seqlens, const int* slots, const int* seq_lens,
                          int n_seqs, cudaStream_t stream) {
    THN_CHECK_ARG(n_seqs >= 0, "step_rows: bad batch %d", n_seqs);
    if (n_seqs == 0) return THN_OK;
    thn_launch(step_rows_kernel, n_seqs, 128, 0, stream, row_slot, row_pos, cu_seqlens, slots, seq_lens, n_seqs);
    return thn_launch_status("step_rows");
}

// seq_lens[slots[b]] += cu[b+1] - cu[b]: the step's tokens are now part of the sequences.
__global__ void advance_kernel(int* __restrict__ seq_lens, const int* __restrict__ slots,
                               const int* __restrict__ cu_seqlens, int n_seqs) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < n_seqs) seq_lens[slots[b]] += cu_seqlens[b + 1] - cu_seqlens[b];
}

THN_API int thn_advance(int* seq_lens, const int* slots, const int* cu_seqlens, int n_seqs, cudaStream_t stream) {
    THN_CHECK_ARG(n_seqs >= 0, "advance: bad batch %d", n_seqs);
    if (n_seqs == 0) return THN_OK;
    thn_launch(advance_kernel, (n_seqs + 127) / 128, 128, 0, stream, seq_lens, slots, cu_seqlens, n_seqs);
    return thn_launch_status("advance");
}

// ------------------------------------------------------------------ rotary table

// cos/sin of angle = position * inv_freq[i], all float32 (engine/engine.py:238-247).
__global__ void rope_table_kernel(float* __restrict__ cos_out, float* __restrict__ sin_out,
                                  const float* __restrict__ inv_freq, int first, int n_positions, int half) {
    pdl_launch_dependents();
    pdl_wait();
    const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= (long long)n_positions * half) return;
    const int p = (int)(e / half), i = (int)(e - (long long)p * half);
    const float angle = (float)(first + p) * inv_freq[i];
    cos_out[(size_t)(first + p) * half + i] = cosf(angle);
    sin_out[(size_t)(first + p) * half + i] = sinf(angle);
}

// Fills rows [first, first + n_positions) of tables [*, half].
THN_API int thn_rope_table(float* cos_out, float* sin_out, const float* inv_freq, int first, int n_positions,
                           int half, cudaStream_t stream) {
    THN_CHECK_ARG(first >= 0 && n_positions >= 0 && half > 0, "rope_table: bad sizes");
    const long long total = (long long)n_positions * half;
    if (total == 0) return THN_OK;
    thn_launch(rope_table_kernel, (unsigned)((total + 255) / 256), 256, 0, stream, cos_out, sin_out, inv_freq, first,
                                                                           n_positions, half);
    return thn_launch_status("rope_table");
}

// ------------------------------------------------------------------ int32 scatter and gather

// dst[index[i]] = value[i]: block-table cells and per-sequence counters changed by the host.
__global__ void scatter_i32_kernel(int* __restrict__ dst, const long long* __restrict__ index,
                                   const int* __restrict__ value, int n, long long dst_size) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n && index[i] >= 0 && index[i] < dst_size) dst[index[i]] = value[i];
}

THN_API int thn_scatter_i32(int* dst, const long long* index, const int* value, int n, long long dst_size,
                            cudaStream_t stream) {
    THN_CHECK_ARG(n >= 0 && dst_size >= 0, "scatter_i32: bad sizes");
    if (n == 0) return THN_OK;
    thn_launch(scatter_i32_kernel, (n + 127) / 128, 128, 0, stream, dst, index, value, n, dst_size);
    return thn_launch_status("scatter_i32");
}

// out[i] = src[index[i]]: the tokens that the sequences of a decode step feed next.
__global__ void gather_i32_kernel(int* __restrict__ out, const int* __restrict__ src, const int* __restrict__ index,
                                  int n) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = src[index[i]];
}

THN_API int thn_gather_i32(int* out, const int* src, const int* index, int n, cudaStream_t stream) {
    THN_CHECK_ARG(n >= 0, "gather_i32: bad size %d", n);
    if (n == 0) return THN_OK;
    thn_launch(gather_i32_kernel, (n + 127) / 128, 128, 0, stream, out, src, index, n);
    return thn_launch_status("gather_i32");
}
