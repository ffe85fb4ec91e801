// What the attention kernels of both families share.
#pragma once
#include "common.cuh"

// Which token the z-th "small" token of the batch is: tokens of entries that bring at most
// dec_max tokens, in batch order (direct != 0: every token of the batch is one).  -1 if there is none.
__device__ __forceinline__ int small_token(int z, const int* __restrict__ q_start, int num_entries, int dec_max, int direct) {
    if (direct) return z < q_start[num_entries] ? z : -1;
    int acc = 0;
    for (int b = 0; b < num_entries; ++b) {
        const int n = q_start[b + 1] - q_start[b];
        if (n > 0 && n <= dec_max) {
            if (z < acc + n) return q_start[b] + z - acc;
            acc += n;
        }
    }
    return -1;
}

// The mask of a causal attention as one number: 0, every earlier key; w > 0, a sliding window of w keys (the
// query's own and the w - 1 before it); -c < 0, chunks of c positions counted from position 0 of the sequence
// (a query sees the earlier keys of its own chunk).  The first key that a query at `pos` sees:
__host__ __device__ __forceinline__ int first_visible(int pos, int mask) {
    if (mask > 0) return pos - mask + 1 > 0 ? pos - mask + 1 : 0;
    if (mask < 0) return pos / (-mask) * (-mask);
    return 0;
}

// Scores that are changed before the softmax: s <- cap * tanh(s / cap) (cap > 0), then s <- s - slope * dist for a
// key dist positions back.  tanh through one exponential and one quotient (absolute error about 1e-7).
__device__ __forceinline__ float capped_score(float s, float cap, float inv_cap) {
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(s * inv_cap * 2.8853900817779268f));   // e^(2 s / cap)
    return cap * (1.f - __fdividef(2.f, e + 1.f));
}
// slope of head h of nh: 2^(-x (h + 1) / nh)
__device__ __forceinline__ float head_slope(float x, int h, int nh) { return x > 0.f ? exp2f(-x * (float)(h + 1) / (float)nh) : 0.f; }
