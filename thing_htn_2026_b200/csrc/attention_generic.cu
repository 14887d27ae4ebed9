// Causal grouped-query attention over the paged cache for any head size: one warp per
// (row, query head), keys visited one by one in ascending position with a running
// maximum.  It serves the true 32-bit path and every bfloat16 shape that the tensor-core
// kernels do not take.  A row's arithmetic is a fixed sequence that depends only on that
// row's own keys, so its result is the same in a whole prompt, in a single-token step and
// in any batch.
//
// Formula: engine/kernels/torch_ref.py:168-227: scores = (q . k) * scale in float32;
// e = exp(s - max); the un-normalised e is rounded to the activation type before it
// multiplies V; the float32 sum of e divides at the end; query head h reads kv head
// h / (n_q / n_kv).  Row at position p sees keys j <= p, and j > p - window when a
// window is set (the reference has no window).
#include <math.h>

#include "common.cuh"

constexpr int kGenericMaxPerLane = 16;  // head_dim <= 512

template <typename T, int PER_LANE>
__global__ void attention_generic_kernel(T* __restrict__ out, const T* __restrict__ q,
                                         const int* __restrict__ row_slot, const int* __restrict__ row_pos,
                                         PagedKV kv, int n_rows, int n_q, float scale, int window,
                                         int* __restrict__ err) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= (long long)n_rows * n_q) return;
    const int m = (int)(unit / n_q), h = (int)(unit - (long long)m * n_q);
    const int D = kv.head_dim;
    const int kvh = h / (n_q / kv.n_kv);
    const int pos = row_pos[m];
    const int* pages = kv.block_table + (size_t)row_slot[m] * kv.bt_stride;

    float qv[PER_LANE], acc[PER_LANE];
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
        const int d = lane + 32 * i;
        qv[i] = d < D ? to_f32<T>(q[(size_t)m * n_q * D + (size_t)h * D + d]) : 0.f;
        acc[i] = 0.f;
    }
    float run_max = -INFINITY, run_sum = 0.f;
    int first = 0;
    if (window > 0 && pos - window + 1 > 0) first = pos - window + 1;

    int page_index = -1;
    const T* k_page = nullptr;
    const T* v_page = nullptr;
    for (int j = first; j <= pos; ++j) {
        if (j / kv.page_size != page_index) {
            page_index = j / kv.page_size;
            const int page = pages[page_index];
            if (page < 0) {
                if (lane == 0 && err) atomicOr(err, THN_ERR_PAGE_UNMAPPED);
                return;
            }
            k_page = (const T*)kv.base + kv_offset(kv, page, 0, kvh, 0);
            v_page = (const T*)kv.base + kv_offset(kv, page, 1, kvh, 0);
        }
        const size_t in_page = (size_t)(j % kv.page_size) * D;
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i) {
            const int d = lane + 32 * i;
            if (d < D) dot += qv[i] * to_f32<T>(k_page[in_page + d]);
        }
        const float s = warp_sum(dot) * scale;
        const float new_max = fmaxf(run_max, s);
        const float correction = expf(run_max - new_max);  // 0 on the first key
        const float e = expf(s - new_max);
        run_sum = run_sum * correction + e;
        const float p = rnd<T>(e);
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i) {
            const int d = lane + 32 * i;
            if (d < D) acc[i] = acc[i] * correction + p * to_f32<T>(v_page[in_page + d]);
        }
        run_max = new_max;
    }
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
        const int d = lane + 32 * i;
        if (d < D) out[(size_t)m * n_q * D + (size_t)h * D + d] = from_f32<T>(acc[i] / run_sum);
    }
}

template <typename T>
static int launch_generic(void* out, const void* q, const int* row_slot, const int* row_pos, PagedKV kv, int n_rows,
                          int n_q, float scale, int window, int* err, cudaStream_t stream) {
    const int warps = 4;
    const long long units = (long long)n_rows * n_q;
    const unsigned blocks = (unsigned)((units + warps - 1) / warps);
    const int per_lane = (kv.head_dim + 31) / 32;
#define LAUNCH(N)                                                                                                  \
    thn_launch(attention_generic_kernel<T, N>, blocks, warps * 32, 0, stream, (T*)out, (const T*)q, row_slot, row_pos, kv, \
                                                                      n_rows, n_q, scale, window, err)
    if (per_lane <= 1) LAUNCH(1);
    else if (per_lane <= 2) LAUNCH(2);
    else if (per_lane <= 4) LAUNCH(4);
    else if (per_lane <= 8) LAUNCH(8);
    else LAUNCH(16);
#undef LAUNCH
    return thn_launch_status("attention_generic");
}

// q, out [n_rows, n_q * head_dim]; the keys of a row are positions [.., row_pos] of the
// sequence in row_slot, already in the cache.  window <= 0 means all keys.
THN_API int thn_attention_generic(void* out, const void* q, const int* row_slot, const int* row_pos,
                                  const void* kv_base, const int* block_table, int bt_stride, int n_kv,
                                  int page_size, int head_dim, int n_rows, int n_q, float scale, int window,
                                  int dtype, int* err, cudaStream_t stream) {
    THN_CHECK_ARG(n_rows >= 0 && n_q > 0 && n_kv > 0 && page_size > 0, "attention_generic: bad sizes");
    THN_CHECK_ARG(n_q % n_kv == 0, "attention_generic: %d query heads are not a multiple of %d kv heads", n_q, n_kv);
    THN_UNSUPPORTED_IF(head_dim <= 0 || head_dim > 32 * kGenericMaxPerLane,
                       "attention_generic: head_dim %d not in [1, %d]", head_dim, 32 * kGenericMaxPerLane);
    if (n_rows == 0) return THN_OK;
    PagedKV kv{kv_base, block_table, bt_stride, n_kv, page_size, head_dim};
    if (dtype == THN_F32) return launch_generic<float>(out, q, row_slot, row_pos, kv, n_rows, n_q, scale, window, err, stream);
    if (dtype == THN_BF16)
        return launch_generic<__nv_bfloat16>(out, q, row_slot, row_pos, kv, n_rows, n_q, scale, window, err, stream);
    THN_CHECK_ARG(false, "attention_generic: unknown dtype %d", dtype);
    return THN_OK;
}
