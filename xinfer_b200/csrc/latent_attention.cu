// Attention over a cached latent: every token leaves one vector c (kv_rank channels, RMS-normed) and one rotated
// key part k_r (rot_dim channels) that all heads share; a head's keys and values are linear maps of c,
//   k_h[j] = [W_uk,h c_j | k_r,j],   v_h[j] = W_uv,h c_j.
// The score of head h is q_h . k_h[j] = (W_uk,h^T q_h,plain) . c_j + q_h,rot . k_r,j, and the output
// W_uv,h (sum_j p_j c_j): with the query carried into the latent space and the value map applied after the
// sum, attention runs over the cached rows [c | k_r] directly, as one key/value head of kv_rank + rot_dim key
// channels whose first kv_rank channels are also the value.  Here are the kernels around that attention:
//
//   latent_prepare_kernel   norms c, rotates k_r and writes the row [c | k_r] to its page; puts the query of
//                           every head together as [q carried into the latent space | rotated q part]
//   gate_sigmoid_kernel     heads' outputs times sigmoid(gate), laid out token by token
//   gemm_batched_plain      the per-head maps as a batch of small matrix products on FMA units (float32 path)
#include "common.cuh"

// proj[t] holds the step's packed projection of token t: the queries at q_off (heads x (d + rd), a head as
// [d plain | rd to rotate]) and, at kv_off, [kv_rank latent | rd key part] (kv_off < 0: this layer reads the
// rows another layer wrote).  q_lat[t, h] (strides given) is the head's query already carried into the latent
// space; absent: the latent part of q_abs has been written already (by the product that formed it) and stays.  The first `rot` channels of a rotated part turn by position * inv_freq[pair] (pairs 2i, 2i+1), cos
// and sin times rot_mag; the others pass.
template <typename T>
__global__ void latent_prepare_kernel(T* __restrict__ q_abs, T* __restrict__ cache, const T* __restrict__ proj,
                                      long long row_len, int q_off, int kv_off, const T* __restrict__ q_lat,
                                      long long ql_ts, long long ql_hs, const float* __restrict__ norm_w,
                                      const float* __restrict__ inv_freq, const int* __restrict__ positions,
                                      const int* __restrict__ req_of_token, const int* __restrict__ block_table,
                                      int table_stride, int nh, int d, int rd, int rank, int rot, int page_size,
                                      int num_pages, float eps, float rot_mag, int pairs, int* err) {
    extern __shared__ float sm[];
    __shared__ float scratch[33];
    const int half = rot / 2;
    float* cs = sm;          // [half]
    float* sn = sm + half;   // [half]
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int b = req_of_token[t];
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        float s, c;
        sincosf((float)pos * inv_freq[j], &s, &c);
        cs[j] = c * rot_mag;
        sn[j] = s * rot_mag;
    }
    __syncthreads();
    const T* row = proj + (size_t)t * row_len;
    const int dk = rank + rd;
    // queries: [latent part | rotated part]
    if (q_lat != nullptr) {
        for (int i = threadIdx.x; i < nh * rank; i += blockDim.x) {
            const int h = i / rank, c = i % rank;
            q_abs[((size_t)t * nh + h) * dk + c] = q_lat[(size_t)t * ql_ts + (size_t)h * ql_hs + c];
        }
    }
    if (pairs) {
        // bfloat16 rows whose rotated parts start on 4-byte boundaries: a pair of neighbours per access
        const int hp = rd / 2;
        for (int i = threadIdx.x; i < nh * hp; i += blockDim.x) {
            const int h = i / hp, pr = i % hp;
            const __nv_bfloat162 in = *reinterpret_cast<const __nv_bfloat162*>(
                reinterpret_cast<const __nv_bfloat16*>(row) + q_off + (size_t)h * (d + rd) + d + 2 * pr);
            float2 v = __bfloat1622float2(in);
            if (2 * pr < rot) v = make_float2(fmaf(v.x, cs[pr], -v.y * sn[pr]), fmaf(v.y, cs[pr], v.x * sn[pr]));
            *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<__nv_bfloat16*>(q_abs) + ((size_t)t * nh + h) * dk + rank + 2 * pr) =
                __floats2bfloat162_rn(v.x, v.y);
        }
    } else {
        for (int i = threadIdx.x; i < nh * rd; i += blockDim.x) {
            const int h = i / rd, e = i % rd;
            const T* qr = row + q_off + (size_t)h * (d + rd) + d;
            float v = to_f32<T>(qr[e]);
            if (e < rot) {
                const float o = to_f32<T>(qr[e ^ 1]);
                v = (e & 1) ? fmaf(v, cs[e >> 1], o * sn[e >> 1]) : fmaf(v, cs[e >> 1], -o * sn[e >> 1]);
            }
            q_abs[((size_t)t * nh + h) * dk + rank + e] = from_f32<T>(v);
        }
    }
    if (kv_off < 0 || b < 0) return;
    const int page = block_table[(size_t)b * table_stride + pos / page_size];
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0) atomicOr(err, XB_ERR_BAD_PAGE);
        return;
    }
    const T* kv = row + kv_off;
    float ss = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) {
        const float v = to_f32<T>(kv[i]);
        ss += v * v;
    }
    const float inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)rank + eps);
    T* dst = cache + ((size_t)page * page_size + (pos % page_size)) * dk;
    for (int i = threadIdx.x; i < dk; i += blockDim.x) {
        float v = to_f32<T>(kv[i]);
        if (i < rank) {
            v = v * inv * norm_w[i];
        } else {
            const int e = i - rank;
            if (e < rot) {
                const float o = to_f32<T>(kv[rank + (e ^ 1)]);
                v = (e & 1) ? fmaf(v, cs[e >> 1], o * sn[e >> 1]) : fmaf(v, cs[e >> 1], -o * sn[e >> 1]);
            }
        }
        dst[i] = from_f32<T>(v);
    }
}

XB_EXPORT int xb_latent_prepare(int dtype, void* q_abs, void* cache, const void* proj, long long row_len, int q_off,
                                int kv_off, const void* q_lat, long long ql_ts, long long ql_hs, const float* norm_w,
                                const float* inv_freq, const int* positions, const int* req_of_token,
                                const int* block_table, int table_stride, int tokens, int nh, int d, int rd, int rank,
                                int rot, int page_size, int num_pages, float eps, float rot_mag, int* err,
                                cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (rot % 2 || rot > rd) return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)rot * sizeof(float);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    const int work = q_lat != nullptr ? nh * (rank + rd) : (nh * rd > rank + rd ? nh * rd : rank + rd);
    // small blocks: a token's work is a few thousand elements behind a chain of dependent steps (angles, a block-wide
    // sum), so many resident blocks hide more than many threads per block
    const int threads = work >= 16384 ? 256 : 128;
#define XB_GO(T)                                                                                                        \
    latent_prepare_kernel<T><<<tokens, threads, smem, stream>>>((T*)q_abs, (T*)cache, (const T*)proj, row_len, q_off,  \
        kv_off, (const T*)q_lat, ql_ts, ql_hs, norm_w, inv_freq, positions, req_of_token, block_table, table_stride,   \
        nh, d, rd, rank, rot, page_size, num_pages, eps, rot_mag, pairs, err)
    const int pairs = (dtype == XB_BF16 && !((row_len | q_off | d | rd | rank) & 1) &&
                       !(((uintptr_t)proj | (uintptr_t)q_abs) & 3)) ? 1 : 0;
    if (dtype == XB_F32) XB_GO(float);
    else XB_GO(__nv_bfloat16);
#undef XB_GO
    return xb_launch_status();
}

// out[t, h * dv + v] = heads[t * h_ts + h * h_hs + v] * sigmoid(gate[t * g_ts + h * dv + v])   (float32 arithmetic);
// `heads` may be `out` itself laid out the same way (in place).  per_head: the gate is one number per head,
// gate[t * g_ts + h]
template <typename T>
__global__ void gate_sigmoid_kernel(T* out, const T* heads, long long h_ts, long long h_hs,
                                    const T* __restrict__ gate, long long g_ts, int nh, int dv, size_t n, int per_head) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const size_t w = (size_t)nh * dv;
    const size_t t = i / w, c = i % w;
    const int h = (int)(c / dv), v = (int)(c % dv);
    const float g = to_f32<T>(gate[t * g_ts + (per_head ? (size_t)h : c)]);
    const float o = to_f32<T>(heads[t * h_ts + (size_t)h * h_hs + v]);
    out[i] = from_f32<T>(o / (1.f + expf(-g)));
}

// eight bfloat16 elements per thread with 16-byte accesses (dv and every stride a multiple of 8, pointers aligned);
// grid (pieces of a token's row, tokens)
__global__ void gate_sigmoid_bf16x8_kernel(__nv_bfloat16* out, const __nv_bfloat16* heads, long long h_ts,
                                           long long h_hs, const __nv_bfloat16* __restrict__ gate, long long g_ts, int nh,
                                           int dv, int tokens, int per_head) {
    const int w = nh * dv;
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (c >= w) return;
    const int h = c / dv, v = c - h * dv;
    for (int t = blockIdx.y; t < tokens; t += gridDim.y) {
        uint4 pg;
        if (per_head) {     // one number for the head's eight channels
            const unsigned short one = *reinterpret_cast<const unsigned short*>(gate + (size_t)t * g_ts + h);
            const uint32_t two = (uint32_t)one | ((uint32_t)one << 16);
            pg = make_uint4(two, two, two, two);
        } else {
            pg = *reinterpret_cast<const uint4*>(gate + (size_t)t * g_ts + c);
        }
        const uint4 po = *reinterpret_cast<const uint4*>(heads + (size_t)t * h_ts + (size_t)h * h_hs + v);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&pg);
        const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(&po);
        uint4 res;
        __nv_bfloat162* r2 = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 g = __bfloat1622float2(g2[k]), o = __bfloat1622float2(o2[k]);
            r2[k] = __floats2bfloat162_rn(o.x / (1.f + expf(-g.x)), o.y / (1.f + expf(-g.y)));
        }
        *reinterpret_cast<uint4*>(out + (size_t)t * w + c) = res;
    }
}

XB_EXPORT int xb_gate_sigmoid(int dtype, void* out, const void* heads, long long h_ts, long long h_hs, const void* gate,
                              long long g_ts, int tokens, int nh, int dv, int per_head, cudaStream_t stream) {
    const size_t n = (size_t)tokens * nh * dv;
    if (n == 0) return 0;
    if (dtype == XB_BF16 && dv % 8 == 0 && h_ts % 8 == 0 && h_hs % 8 == 0 &&
        !(((uintptr_t)out | (uintptr_t)heads) & 15) && (per_head || (g_ts % 8 == 0 && !((uintptr_t)gate & 15)))) {
        const int vecs = nh * dv / 8;
        const int threads = vecs >= 256 ? 256 : 64;
        const dim3 grid((unsigned)((vecs + threads - 1) / threads), (unsigned)(tokens < 65535 ? tokens : 65535));
        gate_sigmoid_bf16x8_kernel<<<grid, threads, 0, stream>>>(
            (__nv_bfloat16*)out, (const __nv_bfloat16*)heads, h_ts, h_hs, (const __nv_bfloat16*)gate, g_ts, nh, dv, tokens, per_head);
        return xb_launch_status();
    }
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (dtype == XB_F32)
        gate_sigmoid_kernel<float><<<blocks, 256, 0, stream>>>((float*)out, (const float*)heads, h_ts, h_hs, (const float*)gate, g_ts, nh, dv, n, per_head);
    else
        gate_sigmoid_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)heads, h_ts, h_hs,
                                                                      (const __nv_bfloat16*)gate, g_ts, nh, dv, n, per_head);
    return xb_launch_status();
}

// c[b, m, n] = sum_k a[b, m, k] * w[b, n, k] with float32 FMA accumulation, k in order for every output (a row's
// result does not depend on M).  Strides in elements: a (sab, sam, 1), w (swb, swn, swk), c (scb, scm, 1).
// 32 x 32 tile, 16-deep panels, 256 threads with 2 x 2 outputs each.
template <typename T>
__global__ void gemm_batched_plain_kernel(T* __restrict__ c, const T* __restrict__ a, const T* __restrict__ w, int M, int N,
                                          int K, long long sab, long long sam, long long swb, long long swn, long long swk,
                                          long long scb, long long scm) {
    __shared__ float As[16][33];
    __shared__ float Ws[16][33];
    const int bz = blockIdx.z, m0 = blockIdx.y * 32, n0 = blockIdx.x * 32;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const T* ab = a + (size_t)bz * sab;
    const T* wb = w + (size_t)bz * swb;
    float acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
    for (int k0 = 0; k0 < K; k0 += 16) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int idx = threadIdx.x + r * 256;
            const int mm = idx >> 4, kk = idx & 15;
            As[kk][mm] = (m0 + mm < M && k0 + kk < K) ? to_f32<T>(ab[(size_t)(m0 + mm) * sam + k0 + kk]) : 0.f;
            // consecutive threads follow whichever of w's two strides is 1
            const int nn = swk == 1 ? idx >> 4 : idx & 31, kw = swk == 1 ? idx & 15 : idx >> 5;
            Ws[kw][nn] = (n0 + nn < N && k0 + kw < K) ? to_f32<T>(wb[(size_t)(n0 + nn) * swn + (size_t)(k0 + kw) * swk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) {
            const float a0 = As[kk][ty * 2], a1 = As[kk][ty * 2 + 1];
            const float w0 = Ws[kk][tx * 2], w1 = Ws[kk][tx * 2 + 1];
            acc[0][0] = fmaf(a0, w0, acc[0][0]);
            acc[0][1] = fmaf(a0, w1, acc[0][1]);
            acc[1][0] = fmaf(a1, w0, acc[1][0]);
            acc[1][1] = fmaf(a1, w1, acc[1][1]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int m = m0 + ty * 2 + i, n = n0 + tx * 2 + j;
            if (m < M && n < N) c[(size_t)bz * scb + (size_t)m * scm + n] = from_f32<T>(acc[i][j]);
        }
}

XB_EXPORT int xb_gemm_batched_plain(int dtype, void* c, const void* a, const void* w, int batch, int M, int N, int K,
                                    long long sab, long long sam, long long swb, long long swn, long long swk,
                                    long long scb, long long scm, cudaStream_t stream) {
    if (batch <= 0 || M <= 0 || N <= 0) return 0;
    if (batch > 65535 || (M + 31) / 32 > 65535) return (int)cudaErrorInvalidValue;
    dim3 grid((N + 31) / 32, (M + 31) / 32, batch);
    if (dtype == XB_F32)
        gemm_batched_plain_kernel<float><<<grid, 256, 0, stream>>>((float*)c, (const float*)a, (const float*)w, M, N, K, sab, sam,
                                                                   swb, swn, swk, scb, scm);
    else
        gemm_batched_plain_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((__nv_bfloat16*)c, (const __nv_bfloat16*)a,
                                                                           (const __nv_bfloat16*)w, M, N, K, sab, sam, swb,
                                                                           swn, swk, scb, scm);
    return xb_launch_status();
}
