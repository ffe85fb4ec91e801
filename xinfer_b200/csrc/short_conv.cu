// Short causal convolution over time, one filter per channel, followed by SiLU:
//
//   y[t, c] = silu( bias[c] + sum_j taps[c, j] * u[t - (K-1) + j, c] )          u = 0 before a sequence's start
//
// u is a column range of the rows of a wider float32 matrix (a packed projection).  The K-1 inputs before a
// step's first token of a request are the request's state, state[slot, K-1, C] (oldest first, zero when a request
// opens); conv_state_kernel leaves the step's last K-1 inputs there afterwards (a separate launch, since the
// first tokens of the step read the old ones).  A thread per (token, channel); arithmetic float32, the taps are
// added in order j = 0 .. K-1 whatever the cut, so a token's result does not depend on the step it ran in.
#include "common.cuh"

constexpr int SC_MAX_TAPS = 16;

template <typename TO>
__global__ void conv_silu_kernel(TO* __restrict__ y, const float* __restrict__ u, long long u_ld, int u_off,
                                 const float* __restrict__ taps, const float* __restrict__ bias,
                                 const float* __restrict__ state, const int* __restrict__ req_of_token,
                                 const int* __restrict__ q_start, const int* __restrict__ slots, int C, int K) {
    const int t = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int b = req_of_token[t];
    if (b < 0) {
        y[(size_t)t * C + c] = from_f32<TO>(0.f);
        return;
    }
    const int t0 = q_start[b], slot = slots[b];
    float acc = bias ? bias[c] : 0.f;
    for (int j = 0; j < K; ++j) {
        const int src = t - (K - 1) + j;
        float v;
        if (src >= t0)
            v = u[(size_t)src * u_ld + u_off + c];
        else
            v = slot >= 0 ? state[((size_t)slot * (K - 1) + (K - 1 + src - t0)) * C + c] : 0.f;
        acc = fmaf(taps[(size_t)c * K + j], v, acc);
    }
    y[(size_t)t * C + c] = from_f32<TO>(acc / (1.f + expf(-acc)));
}

__global__ void conv_state_kernel(float* __restrict__ state, const float* __restrict__ u, long long u_ld, int u_off,
                                  const int* __restrict__ q_start, const int* __restrict__ slots, int C, int K) {
    const int b = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int slot = slots[b];
    if (c >= C || slot < 0) return;
    const int t0 = q_start[b], n = q_start[b + 1] - t0;
    if (n <= 0) return;
    float keep[SC_MAX_TAPS];
    float* st = state + (size_t)slot * (K - 1) * C + c;
#pragma unroll
    for (int k = 0; k < SC_MAX_TAPS; ++k) {
        if (k >= K - 1) break;
        const int rel = n - (K - 1) + k;       // index among this step's inputs; negative: still one of the old ones
        keep[k] = rel >= 0 ? u[(size_t)(t0 + rel) * u_ld + u_off + c] : st[(size_t)(K - 1 + rel) * C];
    }
#pragma unroll
    for (int k = 0; k < SC_MAX_TAPS; ++k) {
        if (k >= K - 1) break;
        st[(size_t)k * C] = keep[k];
    }
}

XB_EXPORT int xb_conv_silu(int out_dtype, void* y, const float* u, long long u_ld, int u_off, const float* taps,
                           const float* bias, const float* state, const int* req_of_token, const int* q_start,
                           const int* slots, int tokens, int C, int K, cudaStream_t stream) {
    if (tokens <= 0 || C <= 0) return 0;
    if (K < 1 || K > SC_MAX_TAPS) return (int)cudaErrorInvalidValue;
    const dim3 grid(tokens, (C + 127) / 128);
    if (out_dtype == XB_F32)
        conv_silu_kernel<float><<<grid, 128, 0, stream>>>((float*)y, u, u_ld, u_off, taps, bias, state, req_of_token, q_start, slots, C, K);
    else
        conv_silu_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>((__nv_bfloat16*)y, u, u_ld, u_off, taps, bias, state,
                                                                 req_of_token, q_start, slots, C, K);
    return xb_launch_status();
}

XB_EXPORT int xb_conv_state(float* state, const float* u, long long u_ld, int u_off, const int* q_start, const int* slots,
                            int entries, int C, int K, cudaStream_t stream) {
    if (entries <= 0 || C <= 0 || K <= 1) return 0;
    if (K > SC_MAX_TAPS) return (int)cudaErrorInvalidValue;
    const dim3 grid((C + 127) / 128, entries);
    conv_state_kernel<<<grid, 128, 0, stream>>>(state, u, u_ld, u_off, q_start, slots, C, K);
    return xb_launch_status();
}
