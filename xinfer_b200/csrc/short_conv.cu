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

template <typename TO, int V>
__device__ __forceinline__ void store_run(TO* dst, const float* r) {
#pragma unroll
    for (int v = 0; v < V; ++v) dst[v] = from_f32<TO>(r[v]);
}
template <>
__device__ __forceinline__ void store_run<float, 4>(float* dst, const float* r) {
    *reinterpret_cast<float4*>(dst) = make_float4(r[0], r[1], r[2], r[3]);
}
template <>
__device__ __forceinline__ void store_run<__nv_bfloat16, 4>(__nv_bfloat16* dst, const float* r) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(r[0], r[1]), b = __floats2bfloat162_rn(r[2], r[3]);
    uint2 q;
    q.x = *reinterpret_cast<const unsigned*>(&a);
    q.y = *reinterpret_cast<const unsigned*>(&b);
    *reinterpret_cast<uint2*>(dst) = q;
}

// The same sum for a run of `run` tokens and V neighbouring channels per thread: the K-1 inputs before a token stay in
// registers and move along, so every input crosses memory once per run (plus K-1 at the run's start) and the taps once
// per thread.  Where a run meets another request's first token the registers are filled again as above.  Taps are added
// in the same order as in conv_silu_kernel, so both give the same bits.
template <typename TO, int K, int V>
__global__ void __launch_bounds__(128) conv_silu_run_kernel(TO* __restrict__ y, const float* __restrict__ u, long long u_ld,
                                                            int u_off, const float* __restrict__ taps,
                                                            const float* __restrict__ bias, const float* __restrict__ state,
                                                            const int* __restrict__ req_of_token,
                                                            const int* __restrict__ q_start, const int* __restrict__ slots,
                                                            int C, int tokens, int run) {
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * V;
    if (c >= C) return;
    float tap[K][V], b0[V], win[K > 1 ? K - 1 : 1][V];
#pragma unroll
    for (int v = 0; v < V; ++v) {
        b0[v] = bias ? bias[c + v] : 0.f;
#pragma unroll
        for (int j = 0; j < K; ++j) tap[j][v] = taps[(size_t)(c + v) * K + j];
    }
    const int first = blockIdx.x * run, last = min(first + run, tokens);
    constexpr int U = 4;    // tokens whose inputs are asked for together, before the first of them is used
    int held = -1;          // the request whose inputs the registers hold
    for (int tu = first; tu < last; tu += U) {
        float x[U][V];
        int bs[U];
#pragma unroll
        for (int i = 0; i < U; ++i) {
            const int t = min(tu + i, last - 1);
            bs[i] = req_of_token[t];
            const float* p = u + (size_t)t * u_ld + u_off + c;
            if (V == 4) {
                const float4 q = *reinterpret_cast<const float4*>(p);
                x[i][0] = q.x, x[i][1 % V] = q.y, x[i][2 % V] = q.z, x[i][3 % V] = q.w;
            } else {
#pragma unroll
                for (int v = 0; v < V; ++v) x[i][v] = p[v];
            }
        }
#pragma unroll
        for (int i = 0; i < U; ++i) {
            const int t = tu + i;
            if (t >= last) break;
            const int b = bs[i];
            if (b < 0) {
                held = -1;
#pragma unroll
                for (int v = 0; v < V; ++v) y[(size_t)t * C + c + v] = from_f32<TO>(0.f);
                continue;
            }
            if (b != held) {    // the run's first token, or another request's first token of this step
                held = b;
                const int t0 = q_start[b], slot = slots[b];
#pragma unroll
                for (int j = 0; j < K - 1; ++j) {
                    const int src = t - (K - 1) + j;
#pragma unroll
                    for (int v = 0; v < V; ++v) {
                        if (src >= t0)
                            win[j][v] = u[(size_t)src * u_ld + u_off + c + v];
                        else
                            win[j][v] = slot >= 0 ? state[((size_t)slot * (K - 1) + (K - 1 + src - t0)) * C + c + v] : 0.f;
                    }
                }
            }
            float r[V];
#pragma unroll
            for (int v = 0; v < V; ++v) {
                float acc = b0[v];
#pragma unroll
                for (int j = 0; j < K - 1; ++j) acc = fmaf(tap[j][v], win[j][v], acc);
                acc = fmaf(tap[K - 1][v], x[i][v], acc);
                r[v] = acc / (1.f + expf(-acc));
#pragma unroll
                for (int j = 0; j + 1 < K - 1; ++j) win[j][v] = win[j + 1][v];
                if (K > 1) win[K - 2 < 0 ? 0 : K - 2][v] = x[i][v];
            }
            store_run<TO, V>(y + (size_t)t * C + c, r);
        }
    }
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

template <typename TO, int V>
static int conv_silu_runs(TO* y, const float* u, long long u_ld, int u_off, const float* taps, const float* bias,
                          const float* state, const int* req_of_token, const int* q_start, const int* slots, int tokens, int C,
                          int K, cudaStream_t stream) {
    // long enough runs to pay for the K-1 inputs read again at a run's start, short enough to fill the machine
    const int per_block = 128 * V, cols = (C + per_block - 1) / per_block;
    int run = 16;
    while (run > 1 && (long long)((tokens + run - 1) / run) * cols < 2 * 148) run /= 2;
    const dim3 grid((tokens + run - 1) / run, cols);
#define XB_CONV_K(KV)                                                                                                     \
    case KV:                                                                                                              \
        conv_silu_run_kernel<TO, KV, V><<<grid, 128, 0, stream>>>(y, u, u_ld, u_off, taps, bias, state, req_of_token,    \
                                                                  q_start, slots, C, tokens, run);                       \
        return 1;
    switch (K) {
        XB_CONV_K(1) XB_CONV_K(2) XB_CONV_K(3) XB_CONV_K(4) XB_CONV_K(5) XB_CONV_K(6) XB_CONV_K(7) XB_CONV_K(8)
        default: return 0;      // more taps than registers are kept for: a thread per token and channel
    }
#undef XB_CONV_K
}

template <typename TO>
static void conv_silu_launch(TO* y, const float* u, long long u_ld, int u_off, const float* taps, const float* bias,
                             const float* state, const int* req_of_token, const int* q_start, const int* slots, int tokens,
                             int C, int K, cudaStream_t stream) {
    const bool vec = C % 4 == 0 && u_ld % 4 == 0 && u_off % 4 == 0 && ((uintptr_t)u & 15) == 0 &&
                     ((uintptr_t)y & (4 * sizeof(TO) - 1)) == 0;
    const int done = vec ? conv_silu_runs<TO, 4>(y, u, u_ld, u_off, taps, bias, state, req_of_token, q_start, slots, tokens, C,
                                                 K, stream)
                         : conv_silu_runs<TO, 1>(y, u, u_ld, u_off, taps, bias, state, req_of_token, q_start, slots, tokens, C,
                                                 K, stream);
    if (done) return;
    const dim3 grid(tokens, (C + 127) / 128);
    conv_silu_kernel<TO><<<grid, 128, 0, stream>>>(y, u, u_ld, u_off, taps, bias, state, req_of_token, q_start, slots, C, K);
}

XB_EXPORT int xb_conv_silu(int out_dtype, void* y, const float* u, long long u_ld, int u_off, const float* taps,
                           const float* bias, const float* state, const int* req_of_token, const int* q_start,
                           const int* slots, int tokens, int C, int K, cudaStream_t stream) {
    if (tokens <= 0 || C <= 0) return 0;
    if (K < 1 || K > SC_MAX_TAPS) return (int)cudaErrorInvalidValue;
    if (out_dtype == XB_F32)
        conv_silu_launch<float>((float*)y, u, u_ld, u_off, taps, bias, state, req_of_token, q_start, slots, tokens, C, K, stream);
    else
        conv_silu_launch<__nv_bfloat16>((__nv_bfloat16*)y, u, u_ld, u_off, taps, bias, state, req_of_token, q_start, slots,
                                        tokens, C, K, stream);
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
