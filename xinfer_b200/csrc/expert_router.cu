// A learned router over experts with a per-expert score and a choice among groups of experts.
//
//   z_e      = W_r[e, :] . h                      float32 (h may arrive in the engine's type)
//   s_e      = sigmoid(z_e)                       the score, also the chosen expert's weight
//   c_e      = s_e + correction_e                 the choice score (correction absent: c = s)
//   group g  = experts g * E/groups .. (g + 1) * E/groups - 1; its score: the sum of its `group_best` largest c
//   allowed  = the experts of the `keep` groups with the largest scores (the others count as minus infinity)
//   chosen   = the `top` allowed experts with the largest c; weight of a chosen expert: s_e (not renormalized),
//              or s_e / sum of the chosen s where `renorm` is set
//
// One block of four warps per token.  Ties go to the lower index.  choice[t, k] and weight[t, k] come out in
// the order of falling choice score.  Padding tokens (request -1) get expert 0 with weight 0.
#include "common.cuh"

#include <math_constants.h>

template <typename T>
__global__ void __launch_bounds__(128)
expert_router_kernel(int* __restrict__ choice, float* __restrict__ weight, const T* __restrict__ h,
                     const float* __restrict__ w_r, const float* __restrict__ correction,
                     const int* __restrict__ req_of_token, int E, int K, int top, int groups, int keep, int group_best,
                     int renorm) {
    extern __shared__ float sm[];
    float* s = sm;              // [E] scores
    float* c = sm + E;          // [E] choice scores (minus infinity once taken or not allowed)
    float* gs = sm + 2 * E;     // [groups]
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    if (req_of_token[t] < 0) {
        for (int k = threadIdx.x; k < top; k += blockDim.x) {
            choice[(size_t)t * top + k] = 0;
            weight[(size_t)t * top + k] = 0.f;
        }
        return;
    }
    const T* x = h + (size_t)t * K;
    for (int e = warp; e < E; e += nwarps) {
        const float* wr = w_r + (size_t)e * K;
        float z = 0.f;
        for (int i = lane; i < K; i += 32) z = fmaf(wr[i], to_f32<T>(x[i]), z);
        z = warp_sum(z);
        if (lane == 0) {
            const float v = 1.f / (1.f + expf(-z));
            s[e] = v;
            c[e] = v + (correction != nullptr ? correction[e] : 0.f);
        }
    }
    __syncthreads();
    const int per = E / groups;
    if (groups > 1 && keep < groups) {
        // a group's score: the sum of its group_best largest choice scores
        for (int g = threadIdx.x; g < groups; g += blockDim.x) {
            float sum = 0.f;
            int taken[8];
            const int nb = min(min(group_best, per), 8);
            for (int b = 0; b < nb; ++b) {
                float best = -CUDART_INF_F;
                int at = -1;
                for (int i = 0; i < per; ++i) {
                    bool used = false;
                    for (int u = 0; u < b; ++u) used |= taken[u] == i;
                    if (!used && (at < 0 || c[g * per + i] > best)) {
                        best = c[g * per + i];
                        at = i;
                    }
                }
                taken[b] = at;
                sum += best;
            }
            gs[g] = sum;
        }
        __syncthreads();
        // a group is kept when fewer than `keep` groups beat it (a tie goes to the lower index)
        for (int g = threadIdx.x; g < groups; g += blockDim.x) {
            int ahead = 0;
            for (int o = 0; o < groups; ++o) ahead += (gs[o] > gs[g]) || (gs[o] == gs[g] && o < g);
            if (ahead >= keep)
                for (int i = 0; i < per; ++i) c[g * per + i] = -CUDART_INF_F;
        }
        __syncthreads();
    }
    if (warp == 0) {
        float total = 0.f;
        for (int k = 0; k < top; ++k) {
            float best = -CUDART_INF_F;
            int at = 0x7fffffff;
            for (int e = lane; e < E; e += 32)
                if (c[e] > best) {          // (a lane walks upwards, so it keeps its lowest index on a tie)
                    best = c[e];
                    at = e;
                }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                if (ob > best || (ob == best && oa < at)) {
                    best = ob;
                    at = oa;
                }
            }
            if (at >= E) at = 0;      // fewer allowed experts than `top`: nothing is left
            const float wv = best == -CUDART_INF_F ? 0.f : s[at];
            total += wv;
            if (lane == 0) {
                choice[(size_t)t * top + k] = at;
                weight[(size_t)t * top + k] = wv;
                c[at] = -CUDART_INF_F;
            }
            __syncwarp();
        }
        if (renorm && total > 0.f)
            for (int k = lane; k < top; k += 32) weight[(size_t)t * top + k] /= total;
    }
}

XB_EXPORT int xb_expert_router(int dtype, int* choice, float* weight, const void* h, const float* w_r, const float* correction,
                               const int* req_of_token, int tokens, int experts, int K, int top, int groups, int keep,
                               int group_best, int renorm, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (experts <= 0 || top <= 0 || top > experts || groups <= 0 || experts % groups || keep <= 0 || keep > groups ||
        group_best <= 0 || group_best > 8)
        return (int)cudaErrorInvalidValue;
    const size_t smem = (2 * (size_t)experts + groups) * sizeof(float);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    if (dtype == XB_F32)
        expert_router_kernel<float><<<tokens, 128, smem, stream>>>(choice, weight, (const float*)h, w_r, correction, req_of_token,
                                                                   experts, K, top, groups, keep, group_best, renorm);
    else
        expert_router_kernel<__nv_bfloat16><<<tokens, 128, smem, stream>>>(choice, weight, (const __nv_bfloat16*)h, w_r, correction,
                                                                           req_of_token, experts, K, top, groups, keep,
                                                                           group_best, renorm);
    return xb_launch_status();
}
