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
// One block of four warps takes ROUTER_TOKENS consecutive tokens: one, so that a step of few tokens still spreads over
// the machine (blocks that run on one SM at the same time find the matrix in its L1), or two for steps of thousands
// of tokens.  First the logits: a warp takes an expert's row of W_r once for the block's tokens, lanes over the
// channels, four at a time where the rows allow it.  Then the choice: a warp per token.  A token's sums run in an
// order fixed by the lane layout, whatever shares its block.  Ties go to the lower index.  choice[t, k] and
// weight[t, k] come out in the order of falling choice score.  Padding tokens (request -1) get expert 0 with weight 0.
#include "common.cuh"

#include <math_constants.h>

constexpr int ROUTER_THREADS = 128;

template <typename T>
__device__ __forceinline__ void router_load4(const T* p, float (&v)[4]);
template <>
__device__ __forceinline__ void router_load4<float>(const float* p, float (&v)[4]) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
template <>
__device__ __forceinline__ void router_load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}

template <typename T, int ROUTER_TOKENS>
__global__ void __launch_bounds__(ROUTER_THREADS)
expert_router_kernel(int* __restrict__ choice, float* __restrict__ weight, const T* __restrict__ h,
                     const float* __restrict__ w_r, const float* __restrict__ correction,
                     const int* __restrict__ req_of_token, int tokens, int E, int K, int top, int groups, int keep,
                     int group_best, int renorm, int vec4) {
    extern __shared__ float sm[];
    float* s_all = sm;                                   // [tokens of the block][E] logits, then scores
    float* c_all = sm + ROUTER_TOKENS * E;               // [..][E] choice scores (minus infinity once taken or not allowed)
    float* g_all = sm + 2 * ROUTER_TOKENS * E;           // [..][groups]
    const int t0 = blockIdx.x * ROUTER_TOKENS, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int nt = min(ROUTER_TOKENS, tokens - t0);
    // a warp takes two experts at a time (e and e + nwarps): twice the loads in flight for the same chain of sums
    for (int e = warp; e < E; e += 2 * nwarps) {
        const int e2 = e + nwarps;
        const bool two = e2 < E;
        const float* wa = w_r + (size_t)e * K;
        const float* wb = w_r + (size_t)(two ? e2 : e) * K;
        float acc[ROUTER_TOKENS], acc2[ROUTER_TOKENS];
#pragma unroll
        for (int j = 0; j < ROUTER_TOKENS; ++j) acc[j] = acc2[j] = 0.f;
        if (vec4) {
#pragma unroll 4
            for (int i = lane * 4; i < K; i += 128) {
                const float4 a4 = *reinterpret_cast<const float4*>(wa + i);
                const float4 b4 = *reinterpret_cast<const float4*>(wb + i);
#pragma unroll
                for (int j = 0; j < ROUTER_TOKENS; ++j) {
                    if (j < nt) {
                        float x[4];
                        router_load4<T>(h + (size_t)(t0 + j) * K + i, x);
                        acc[j] = fmaf(a4.x, x[0], acc[j]);
                        acc[j] = fmaf(a4.y, x[1], acc[j]);
                        acc[j] = fmaf(a4.z, x[2], acc[j]);
                        acc[j] = fmaf(a4.w, x[3], acc[j]);
                        acc2[j] = fmaf(b4.x, x[0], acc2[j]);
                        acc2[j] = fmaf(b4.y, x[1], acc2[j]);
                        acc2[j] = fmaf(b4.z, x[2], acc2[j]);
                        acc2[j] = fmaf(b4.w, x[3], acc2[j]);
                    }
                }
            }
        } else {
            for (int i = lane; i < K; i += 32) {
                const float av = wa[i], bv = wb[i];
#pragma unroll
                for (int j = 0; j < ROUTER_TOKENS; ++j)
                    if (j < nt) {
                        const float xv = to_f32<T>(h[(size_t)(t0 + j) * K + i]);
                        acc[j] = fmaf(av, xv, acc[j]);
                        acc2[j] = fmaf(bv, xv, acc2[j]);
                    }
            }
        }
#pragma unroll
        for (int j = 0; j < ROUTER_TOKENS; ++j) {
            const float z = warp_sum(acc[j]), z2 = warp_sum(acc2[j]);
            if (lane == 0) {
                s_all[j * E + e] = z;
                if (two) s_all[j * E + e2] = z2;
            }
        }
    }
    __syncthreads();
    const int per = E / groups;
    for (int j = warp; j < nt; j += nwarps) {
        const int t = t0 + j;
        float* s = s_all + j * E;
        float* c = c_all + j * E;
        float* gs = g_all + j * groups;
        if (req_of_token[t] < 0) {
            for (int k = lane; k < top; k += 32) {
                choice[(size_t)t * top + k] = 0;
                weight[(size_t)t * top + k] = 0.f;
            }
            continue;
        }
        for (int e = lane; e < E; e += 32) {
            const float v = 1.f / (1.f + expf(-s[e]));
            s[e] = v;
            c[e] = v + (correction != nullptr ? correction[e] : 0.f);
        }
        __syncwarp();
        if (groups > 1 && keep < groups) {
            // a group's score: the sum of its group_best largest choice scores
            for (int g = lane; g < groups; g += 32) {
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
            __syncwarp();
            // a group is kept when fewer than `keep` groups beat it (a tie goes to the lower index)
            for (int g = lane; g < groups; g += 32) {
                int ahead = 0;
                for (int o = 0; o < groups; ++o) ahead += (gs[o] > gs[g]) || (gs[o] == gs[g] && o < g);
                if (ahead >= keep)
                    for (int i = 0; i < per; ++i) c[g * per + i] = -CUDART_INF_F;
            }
            __syncwarp();
        }
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
    const int per_block = tokens >= 4096 ? 2 : 1;
    const size_t smem = (size_t)per_block * (2 * (size_t)experts + groups) * sizeof(float);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    const size_t esz = dtype == XB_F32 ? 4 : 2;
    const int vec4 = (K % 4 == 0 && !((uintptr_t)h & (4 * esz - 1)) && !((uintptr_t)w_r & 15)) ? 1 : 0;
    const unsigned blocks = (unsigned)((tokens + per_block - 1) / per_block);
#define XB_ROUTER(T, N)                                                                                                   \
    expert_router_kernel<T, N><<<blocks, ROUTER_THREADS, smem, stream>>>(choice, weight, (const T*)h, w_r, correction,    \
                                                                         req_of_token, tokens, experts, K, top, groups,   \
                                                                         keep, group_best, renorm, vec4)
    if (dtype == XB_F32) {
        if (per_block == 2) XB_ROUTER(float, 2); else XB_ROUTER(float, 1);
    } else {
        if (per_block == 2) XB_ROUTER(__nv_bfloat16, 2); else XB_ROUTER(__nv_bfloat16, 1);
    }
#undef XB_ROUTER
    return xb_launch_status();
}
