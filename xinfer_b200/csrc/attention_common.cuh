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
// key dist positions back.  With e = exp(2 s / cap), cap * tanh(s / cap) = cap - 2 cap / (e + 1): one exponential, one
// reciprocal and one multiply-add that also takes whatever is added to the score (absolute error about 1e-7 of the
// cap).  raw: the unscaled score; k1 = scale * 2 log2(e) / cap; base: cap plus what is added.
__device__ __forceinline__ float capped_score(float raw, float k1, float neg2cap, float base) {
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(raw * k1));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(e + 1.f));     // e = inf gives 0: the score is the cap
    return fmaf(neg2cap, r, base);
}
// slope of head h of nh: 2^(-x (h + 1) / nh)
__device__ __forceinline__ float head_slope(float x, int h, int nh) { return x > 0.f ? exp2f(-x * (float)(h + 1) / (float)nh) : 0.f; }
