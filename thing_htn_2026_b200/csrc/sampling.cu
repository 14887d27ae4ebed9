// Token choice from float32 logits: greedy argmax and temperature sampling.
//
// Greedy: the lowest index among exact ties (engine/engine.py:1121;
// OPTIMIZATION_GUIDE.md:213).  The reference samples with nothing else.  Temperature
// sampling uses the Gumbel-max rule: argmax(logit / T + noise) is a draw from
// softmax(logit / T).  The noise of vocabulary entry i is word i % 4 of
// Philox-4x32-10(counter = (i / 4, step, stream, 0), key = seed), u = ((word >> 9) + 0.5)
// * 2^-23, noise = -log(-log(u)); a sequence's draws depend on its own (seed, stream,
// step) only, never on its batch mates.
#include <math.h>

#include "common.cuh"

namespace {
struct Best {
    float value;
    int index;
};

__device__ __forceinline__ Best better(Best a, Best b) {
    if (b.value > a.value || (b.value == a.value && b.index < a.index)) return b;
    return a;
}

__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0,
                                              uint32_t k1, uint32_t out[4]) {
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
        const uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
        c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

// Best (score, index) over entries [begin, end) of one row, as seen by this thread; scores
// are logits, or logits / temperature + noise.
__device__ __forceinline__ Best scan_row(const float* __restrict__ x, int begin, int end, int vocab, float temp,
                                         unsigned long long s, uint32_t c1, uint32_t c2) {
    Best best{-INFINITY, 0x7fffffff};
    if (temp == 0.f) {
        for (int i = begin + threadIdx.x; i < end; i += blockDim.x) best = better(best, Best{x[i], i});
        return best;
    }
    const uint32_t k0 = (uint32_t)s, k1 = (uint32_t)(s >> 32);
    for (int b = begin / 4 + threadIdx.x; b < (end + 3) / 4; b += blockDim.x) {
        uint32_t words[4];
        philox4x32_10((uint32_t)b, c1, c2, 0u, k0, k1, words);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = 4 * b + j;
            if (i >= begin && i < end && i < vocab) {
                const float u = ((float)(words[j] >> 9) + 0.5f) * 1.1920928955078125e-07f;  // 2^-23
                const float noise = -logf(-logf(u));
                best = better(best, Best{x[i] / temp + noise, i});
            }
        }
    }
    return best;
}

__device__ __forceinline__ Best block_best(Best best, Best* partial /* [32] shared */) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best other{__shfl_xor_sync(0xffffffffu, best.value, o), __shfl_xor_sync(0xffffffffu, best.index, o)};
        best = better(best, other);
    }
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x < 32) {
        const int n_warps = (blockDim.x + 31) >> 5;
        best = threadIdx.x < n_warps ? partial[threadIdx.x] : Best{-INFINITY, 0x7fffffff};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            Best other{__shfl_xor_sync(0xffffffffu, best.value, o), __shfl_xor_sync(0xffffffffu, best.index, o)};
            best = better(best, other);
        }
    }
    return best;      // valid in thread 0
}

// Large vocabularies: blockIdx.y cuts the row into slices; each block leaves its slice's best
// (score, index) in part[row][slice]; choose_kernel then runs over the partials.
__global__ void __launch_bounds__(256) choose_slices_kernel(float* __restrict__ part_value, int* __restrict__ part_index,
                                                            const float* __restrict__ logits, int vocab,
                                                            long long row_stride, const float* __restrict__ temperature,
                                                            const unsigned long long* __restrict__ seed,
                                                            const int* __restrict__ stream_id,
                                                            const int* __restrict__ step,
                                                            const int* __restrict__ slots) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ Best partial[32];
    const int row = blockIdx.x, slice = blockIdx.y, n_slices = gridDim.y;
    const int who = slots ? slots[row] : row;
    const float temp = temperature ? temperature[who] : 0.f;
    const int per = ((vocab + n_slices - 1) / n_slices + 3) / 4 * 4;      // slices start at multiples of 4
    const int begin = min(vocab, slice * per), end = min(vocab, begin + per);
    const Best best = block_best(scan_row(logits + (size_t)row * row_stride, begin, end, vocab, temp,
                                          temp != 0.f ? seed[who] : 0ull, temp != 0.f ? (uint32_t)step[who] : 0u,
                                          temp != 0.f ? (uint32_t)stream_id[who] : 0u), partial);
    if (threadIdx.x == 0) {
        part_value[row * n_slices + slice] = best.value;
        part_index[row * n_slices + slice] = best.index;
    }
}

// One block per row.  temperature == nullptr or temperature[row] == 0: greedy.  With
// part_value the row's candidates are the n_slices partial results instead of the logits.
__global__ void __launch_bounds__(1024) choose_kernel(int* __restrict__ out, const float* __restrict__ logits,
                                                      int vocab, long long row_stride,
                                                      const float* __restrict__ temperature,
                                                      const unsigned long long* __restrict__ seed,
                                                      const int* __restrict__ stream_id, int* __restrict__ step,
                                                      const int* __restrict__ slots, int* __restrict__ last_token,
                                                      int bump_step, const float* __restrict__ part_value,
                                                      const int* __restrict__ part_index, int n_slices) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ Best partial[32];
    const int row = blockIdx.x;
    const int who = slots ? slots[row] : row;  // index of this row's per-sequence values
    const float temp = temperature ? temperature[who] : 0.f;
    Best best{-INFINITY, 0x7fffffff};
    if (part_value) {
        for (int i = threadIdx.x; i < n_slices; i += blockDim.x)
            best = better(best, Best{part_value[row * n_slices + i], part_index[row * n_slices + i]});
    } else {
        best = scan_row(logits + (size_t)row * row_stride, 0, vocab, vocab, temp, temp != 0.f ? seed[who] : 0ull,
                        temp != 0.f ? (uint32_t)step[who] : 0u, temp != 0.f ? (uint32_t)stream_id[who] : 0u);
    }
    best = block_best(best, partial);
    if (threadIdx.x == 0) {
        const int token = best.index == 0x7fffffff ? 0 : best.index;
        out[row] = token;
        if (last_token) last_token[who] = token;
        if (bump_step && step) step[who] += 1;
    }
}
}  // namespace

constexpr int kChooseSlices = 32;

// Floats of scratch thn_choose_tokens wants for this vocabulary (0: none).
THN_API long long thn_choose_tokens_scratch_floats(int rows, int vocab) {
    return vocab >= 32768 ? 2LL * rows * kChooseSlices : 0;
}

// logits [rows, vocab] float32 with row stride row_stride elements -> out [rows] int32.
// temperature, seed, stream_id, step are device arrays indexed by row, or by slots[row]
// when slots is given (per-sequence state); temperature may be null (all greedy), in which
// case seed and stream_id are not read.  With last_token the choice is also stored at the
// same index (the token the sequence feeds next); with bump_step the step counter at that
// index grows by one after it was used.  scratch (thn_choose_tokens_scratch_floats floats,
// or null) lets large vocabularies be scanned by many blocks per row.
THN_API int thn_choose_tokens(int* out, const float* logits, int rows, int vocab, long long row_stride,
                              const float* temperature, const unsigned long long* seed, const int* stream_id,
                              int* step, const int* slots, int* last_token, int bump_step, float* scratch,
                              cudaStream_t stream) {
    THN_CHECK_ARG(rows >= 0 && vocab > 0 && row_stride >= vocab, "choose_tokens: bad sizes rows=%d vocab=%d", rows,
                  vocab);
    THN_CHECK_ARG(temperature == nullptr || (seed && stream_id && step),
                  "choose_tokens: sampling needs seed, stream and step arrays");
    if (rows == 0) return THN_OK;
    if (scratch != nullptr && thn_choose_tokens_scratch_floats(rows, vocab) > 0) {
        float* part_value = scratch;
        int* part_index = reinterpret_cast<int*>(scratch + (size_t)rows * kChooseSlices);
        thn_launch(choose_slices_kernel, dim3(rows, kChooseSlices), 256, 0, stream, part_value, part_index, logits,
                   vocab, row_stride, temperature, seed, stream_id, (const int*)step, slots);
        int status = thn_launch_status("choose_tokens");
        if (status != THN_OK) return status;
        thn_launch(choose_kernel, rows, 32, 0, stream, out, logits, vocab, row_stride, temperature, seed, stream_id,
                   step, slots, last_token, bump_step, (const float*)part_value, (const int*)part_index,
                   kChooseSlices);
        return thn_launch_status("choose_tokens");
    }
    const int threads = vocab >= 4096 ? 1024 : 256;
    thn_launch(choose_kernel, rows, threads, 0, stream, out, logits, vocab, row_stride, temperature, seed, stream_id,
               step, slots, last_token, bump_step, (const float*)nullptr, (const int*)nullptr, 0);
    return thn_launch_status("choose_tokens");
}
