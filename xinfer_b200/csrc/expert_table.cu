// Mixture of small gated experts chosen by a table over token ids (no router).
//
//   experts of token t:  table[id_t, 0..top)        each with weight 1 / top
//   expert e:            down_e( silu(gate_e h) * (up_e h) )
//
// Three kernels per layer:
//  1. route: the (token, choice) pairs are grouped by expert: counts, offsets and a permutation;
//  2. grouped products: a block takes a tile of rows of ONE expert and a tile of output columns, with that
//     expert's matrix (rows are gathered through the permutation for the gate/up product, whose tile holds
//     the same columns of gate and up and finishes with silu(gate) * up);
//  3. combine: out[t] = (1 / top) * sum_k y[row of (t, k)], summed in the order of k.
// A row's products are reduced in an order that depends only on the row, so a token's result does not
// depend on which other tokens share its expert.  Accumulation is float32.
#include "common.cuh"

// ------------------------------------------------------------------------------------------
// 1. route.  One block.  offsets[E + 1]; perm[r] = t * top + k for grouped row r; inv[t * top + k] = r.
// The experts of token t are row id_t of the table, or row t where no ids are given (a router's choices).
// Padding tokens (request -1) take part in nothing: their pairs get inv = -1.
// ------------------------------------------------------------------------------------------
__global__ void expert_route_kernel(int* __restrict__ offsets, int* __restrict__ perm, int* __restrict__ inv,
                                    const int* __restrict__ table, const int* __restrict__ ids,
                                    const int* __restrict__ sampled, int num_sampled, const int* __restrict__ req_of_token,
                                    int T, int top, int E, int vocab, int* err) {
    extern __shared__ int sh[];      // counts[E], cursor[E]
    int* counts = sh;
    int* cursor = sh + E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    const int n = T * top;
    for (int p = threadIdx.x; p < n; p += blockDim.x) {
        const int t = p / top, k = p - t * top;
        int id = ids != nullptr ? ids[t] : t;     // no ids: the table has a row per token of the step
        if (id < 0 && sampled != nullptr && -1 - id < num_sampled) id = sampled[-1 - id];
        int e = -1;
        if (req_of_token[t] >= 0) {
            if (id < 0 || id >= vocab) {
                atomicOr(err, XB_ERR_BAD_TOKEN);
            } else {
                e = table[(size_t)id * top + k];
                if (e < 0 || e >= E) {
                    atomicOr(err, XB_ERR_BAD_ROW);
                    e = -1;
                }
            }
        }
        inv[p] = e;          // the expert for now; the row below
        if (e >= 0) atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < E; ++e) {
            offsets[e] = at;
            cursor[e] = at;
            at += counts[e];
        }
        offsets[E] = at;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < n; p += blockDim.x) {
        const int e = inv[p];
        if (e < 0) continue;
        const int r = atomicAdd(&cursor[e], 1);
        perm[r] = p;
        inv[p] = r;
    }
}

XB_EXPORT int xb_expert_route(int* offsets, int* perm, int* inv, const int* table, const int* ids, const int* sampled,
                              int num_sampled, const int* req_of_token, int tokens, int top, int experts, int vocab, int* err,
                              cudaStream_t stream) {
    if (tokens <= 0) return 0;
    const size_t smem = 2 * (size_t)experts * sizeof(int);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    expert_route_kernel<<<1, 1024, smem, stream>>>(offsets, perm, inv, table, ids, sampled, num_sampled, req_of_token, tokens,
                                                   top, experts, vocab, err);
    return xb_launch_status();
}

// ------------------------------------------------------------------------------------------
// 2. grouped product on FMA units.  y[r, n] = sum_k a[src(r), k] * w[e(r), n, k]
//    gather: src(r) = perm[r] / top, else src(r) = r.
//    gated:  w[e] is [2 * N, K] (gate rows, then up rows), y[r, n] = act(gate) * f(up), the activation by code.
// 32 x 64 tile, 16-deep panels, 256 threads with 2 x 4 outputs each (x 2 accumulators when gated).
// Block (x, y): column tile x; row tile y is found by walking over the experts' counts.
// ------------------------------------------------------------------------------------------
template <typename TA, typename TW, typename TO, bool GATED>
__global__ void expert_gemm_kernel(TO* __restrict__ y, const TA* __restrict__ a, const TW* __restrict__ w,
                                   const int* __restrict__ offsets, const int* __restrict__ perm, int gather, int top,
                                   int E, int N, int K, long long ldw, long long estride, int act, float p0, float p1) {
    constexpr int BM = 32, BN = 64, BK = 16;
    __shared__ float sa[BK][BM + 1];
    __shared__ float sw[GATED ? 2 : 1][BK][BN + 1];
    __shared__ int s_e, s_row0, s_rows;
    __shared__ int src[BM];
    if (threadIdx.x == 0) {
        int tile = blockIdx.y, found = -1, row0 = 0, rows = 0;
        for (int e = 0; e < E; ++e) {
            const int cnt = offsets[e + 1] - offsets[e];
            const int nt = (cnt + BM - 1) / BM;
            if (tile < nt) {
                found = e;
                row0 = offsets[e] + tile * BM;
                rows = min(BM, cnt - tile * BM);
                break;
            }
            tile -= nt;
        }
        s_e = found; s_row0 = row0; s_rows = rows;
    }
    __syncthreads();
    const int e = s_e;
    if (e < 0) return;
    const int row0 = s_row0, rows = s_rows;
    if (threadIdx.x < BM) {
        const int i = (int)threadIdx.x;
        src[i] = i < rows ? (gather ? perm[row0 + i] / top : row0 + i) : -1;
    }
    __syncthreads();
    const int n0 = blockIdx.x * BN;
    const TW* we = w + (size_t)e * estride;     // row n of this expert's matrix starts at we + n * ldw
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;     // 16 x 16 threads: 4 columns x 2 rows each
    float acc[2][4], acc2[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = acc2[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int idx = threadIdx.x; idx < BM * BK; idx += 256) {
            const int r = idx / BK, c = idx % BK;
            const int s = src[r], gk = k0 + c;
            sa[c][r] = (s >= 0 && gk < K) ? to_f32<TA>(a[(size_t)s * K + gk]) : 0.f;
        }
        for (int idx = threadIdx.x; idx < BN * BK; idx += 256) {
            const int r = idx / BK, c = idx % BK;
            const int gn = n0 + r, gk = k0 + c;
            const bool ok = gn < N && gk < K;
            sw[0][c][r] = ok ? to_f32<TW>(we[(size_t)gn * ldw + gk]) : 0.f;
            if (GATED) sw[GATED ? 1 : 0][c][r] = ok ? to_f32<TW>(we[(size_t)(N + gn) * ldw + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float av[2], wv[4], uv[4];
#pragma unroll
            for (int i = 0; i < 2; ++i) av[i] = sa[kk][ty * 2 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                wv[j] = sw[0][kk][tx * 4 + j];
                if (GATED) uv[j] = sw[GATED ? 1 : 0][kk][tx * 4 + j];
            }
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
                    if (GATED) acc2[i][j] = fmaf(av[i], uv[j], acc2[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = ty * 2 + i;
        if (r >= rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            float v = acc[i][j];
            if (GATED) {
                v = gate_mul_any(act, v, acc2[i][j], p0, p1);
            }
            y[(size_t)(row0 + r) * N + gn] = from_f32<TO>(v);
        }
    }
}

template <typename TA, typename TW, typename TO>
static int expert_gemm_launch(void* y, const void* a, const void* w, const int* offsets, const int* perm, int gather, int top,
                              int E, int rows_max, int N, int K, int gated, long long ldw, long long estride, int act, float p0,
                              float p1, cudaStream_t stream) {
    const dim3 grid((N + 63) / 64, (rows_max + 31) / 32 + E);
    if (gated)
        expert_gemm_kernel<TA, TW, TO, true><<<grid, 256, 0, stream>>>((TO*)y, (const TA*)a, (const TW*)w, offsets, perm, gather, top, E, N, K, ldw, estride, act, p0, p1);
    else
        expert_gemm_kernel<TA, TW, TO, false><<<grid, 256, 0, stream>>>((TO*)y, (const TA*)a, (const TW*)w, offsets, perm, gather, top, E, N, K, ldw, estride, act, p0, p1);
    return xb_launch_status();
}

// in_dtype: type of a and w; out_dtype: type of y.  rows_max: tokens * top.  Row n of expert e's matrix starts
// at w + e * estride + n * ldw (elements): [experts, rows, K] blocks, or matrices side by side along K.
XB_EXPORT int xb_expert_gemm(int in_dtype, int out_dtype, void* y, const void* a, const void* w, const int* offsets,
                             const int* perm, int gather, int top, int experts, int rows_max, int N, int K, int gated,
                             long long ldw, long long estride, int act, float p0, float p1, cudaStream_t stream) {
    if (rows_max <= 0 || N <= 0) return 0;
    typedef __nv_bfloat16 bf;
#define XB_ARGS y, a, w, offsets, perm, gather, top, experts, rows_max, N, K, gated, ldw, estride, act, p0, p1, stream
    if (in_dtype == XB_F32) return out_dtype == XB_F32 ? expert_gemm_launch<float, float, float>(XB_ARGS) : (int)cudaErrorInvalidValue;
    return out_dtype == XB_F32 ? expert_gemm_launch<bf, bf, float>(XB_ARGS) : expert_gemm_launch<bf, bf, bf>(XB_ARGS);
#undef XB_ARGS
}

// ------------------------------------------------------------------------------------------
// For steps of few tokens: every expert's gate/up values of every token come from ONE dense product with the
// experts' matrices stacked (weights are read once, as they would be anyway once most experts are in use).
//   act[t, e * F + f] = weight * silu(gu[t, e*2F + f]) * gu[t, e*2F + F + f]   if e is one of token t's experts
//                     = 0                                                       otherwise
// so that ONE product with the down matrices side by side along K sums the token's experts.
// ------------------------------------------------------------------------------------------
// `weights` [T, top] (absent: every chosen expert weighs 1 / top); no ids: the table has a row per token.
template <typename T>
__global__ void expert_select_gate_kernel(T* __restrict__ act, const T* __restrict__ gu, const int* __restrict__ table,
                                          const int* __restrict__ ids, const int* __restrict__ sampled, int num_sampled,
                                          const int* __restrict__ req_of_token, int top, int E, int F, int vocab,
                                          float weight, const float* __restrict__ weights, int code, float p0, float p1,
                                          int* err) {
    const int t = blockIdx.x, e = blockIdx.y;
    int id = ids != nullptr ? ids[t] : t;
    if (id < 0 && sampled != nullptr && -1 - id < num_sampled) id = sampled[-1 - id];
    bool chosen = false;
    if (req_of_token[t] >= 0) {
        if (id < 0 || id >= vocab) {
            if (threadIdx.x == 0 && e == 0) atomicOr(err, XB_ERR_BAD_TOKEN);
        } else {
            for (int k = 0; k < top; ++k)
                if (table[(size_t)id * top + k] == e) {
                    chosen = true;
                    if (weights != nullptr) weight = weights[(size_t)id * top + k];
                }
        }
    }
    const T* g = gu + ((size_t)t * E + e) * 2 * F;
    T* o = act + ((size_t)t * E + e) * F;
    for (int f = threadIdx.x; f < F; f += blockDim.x) {
        float v = 0.f;
        if (chosen) v = gate_mul_any(code, to_f32<T>(g[f]), to_f32<T>(g[F + f]), p0, p1) * weight;
        o[f] = from_f32<T>(v);
    }
}

XB_EXPORT int xb_expert_select_gate(int dtype, void* act, const void* gu, const int* table, const int* ids, const int* sampled,
                                    int num_sampled, const int* req_of_token, int tokens, int top, int experts, int F, int vocab,
                                    const float* weights, int code, float p0, float p1, int* err, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    const dim3 grid(tokens, experts);
    const float weight = 1.f / (float)top;
    if (dtype == XB_F32)
        expert_select_gate_kernel<float><<<grid, 256, 0, stream>>>((float*)act, (const float*)gu, table, ids, sampled, num_sampled,
                                                                   req_of_token, top, experts, F, vocab, weight, weights, code,
                                                                   p0, p1, err);
    else
        expert_select_gate_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((__nv_bfloat16*)act, (const __nv_bfloat16*)gu, table, ids,
                                                                           sampled, num_sampled, req_of_token, top, experts, F,
                                                                           vocab, weight, weights, code, p0, p1, err);
    return xb_launch_status();
}

// ------------------------------------------------------------------------------------------
// Rows in grouped order, for products that want each expert's rows as one contiguous matrix:
//   out[r, :] = x[perm[r] / top, :]   for r < offsets[E]
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void expert_gather_kernel(T* __restrict__ out, const T* __restrict__ x, const int* __restrict__ perm,
                                     const int* __restrict__ offsets, int top, int E, int K) {
    const int r = blockIdx.x;
    if (r >= offsets[E]) return;
    const T* src = x + (size_t)(perm[r] / top) * K;
    T* dst = out + (size_t)r * K;
    if ((K * sizeof(T)) % 16 == 0) {
        const int n16 = K * sizeof(T) / 16;
        for (int i = threadIdx.x; i < n16; i += blockDim.x) reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
    } else {
        for (int i = threadIdx.x; i < K; i += blockDim.x) dst[i] = src[i];
    }
}

XB_EXPORT int xb_expert_gather(int dtype, void* out, const void* x, const int* perm, const int* offsets, int rows_max, int top,
                               int experts, int K, cudaStream_t stream) {
    if (rows_max <= 0) return 0;
    if (dtype == XB_F32)
        expert_gather_kernel<float><<<rows_max, 128, 0, stream>>>((float*)out, (const float*)x, perm, offsets, top, experts, K);
    else
        expert_gather_kernel<__nv_bfloat16><<<rows_max, 128, 0, stream>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)x, perm, offsets,
                                                                         top, experts, K);
    return xb_launch_status();
}

// ------------------------------------------------------------------------------------------
// 3. combine.  out[t, :] = base[t, :] + sum_k w(t, k) * y[inv[t * top + k], :]   (a pair without a row adds nothing)
// w(t, k) = weights[t * top + k], or 1 / top for all where no weights are given; base may be absent.
// ------------------------------------------------------------------------------------------
template <typename TO>
__global__ void expert_combine_kernel(TO* __restrict__ out, const float* __restrict__ y, const int* __restrict__ inv, int top,
                                      int N, float weight, const float* __restrict__ weights, const TO* __restrict__ base) {
    const int t = blockIdx.x;
    for (int c = threadIdx.x; c < N; c += blockDim.x) {
        float s = 0.f;
        for (int k = 0; k < top; ++k) {
            const int r = inv[t * top + k];
            if (r >= 0) s += (weights != nullptr ? weights[t * top + k] : 1.f) * y[(size_t)r * N + c];
        }
        s *= weight;
        if (base != nullptr) s += to_f32<TO>(base[(size_t)t * N + c]);
        out[(size_t)t * N + c] = from_f32<TO>(s);
    }
}

// the same with four columns per thread (N a multiple of 4, float32 out and base, 16-byte aligned rows): the same sums
// in the same order
__global__ void expert_combine4_kernel(float4* __restrict__ out, const float4* __restrict__ y, const int* __restrict__ inv,
                                       int top, int N4, float weight, const float* __restrict__ weights,
                                       const float4* __restrict__ base) {
    const int t = blockIdx.x;
    for (int c = threadIdx.x; c < N4; c += blockDim.x) {
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int k = 0; k < top; ++k) {
            const int r = inv[t * top + k];
            if (r < 0) continue;
            const float w = weights != nullptr ? weights[t * top + k] : 1.f;
            const float4 v = y[(size_t)r * N4 + c];
            s.x += w * v.x; s.y += w * v.y; s.z += w * v.z; s.w += w * v.w;
        }
        s.x *= weight; s.y *= weight; s.z *= weight; s.w *= weight;
        if (base != nullptr) {
            const float4 bv = base[(size_t)t * N4 + c];
            s.x += bv.x; s.y += bv.y; s.z += bv.z; s.w += bv.w;
        }
        out[(size_t)t * N4 + c] = s;
    }
}

XB_EXPORT int xb_expert_combine(int out_dtype, void* out, const float* y, const int* inv, int tokens, int top, int N,
                                const float* weights, const void* base, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    const float weight = weights != nullptr ? 1.f : 1.f / (float)top;
    if (out_dtype == XB_F32 && N % 4 == 0 && !(((uintptr_t)out | (uintptr_t)y | (uintptr_t)base) & 15))
        expert_combine4_kernel<<<tokens, 256, 0, stream>>>((float4*)out, (const float4*)y, inv, top, N / 4, weight, weights,
                                                           (const float4*)base);
    else if (out_dtype == XB_F32)
        expert_combine_kernel<float><<<tokens, 256, 0, stream>>>((float*)out, y, inv, top, N, weight, weights, (const float*)base);
    else
        expert_combine_kernel<__nv_bfloat16><<<tokens, 256, 0, stream>>>((__nv_bfloat16*)out, y, inv, top, N, weight, weights,
                                                                         (const __nv_bfloat16*)base);
    return xb_launch_status();
}
