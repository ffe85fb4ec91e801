// Attention whose heads talk to each other before the softmax, over the paged cache.
//
//   raw_g[i, j]  = scale * q_g[i] . k_kv(g)[j]                    every query head g
//   s_h[i, j]    = sum_g talk[h, g] * raw_g[i, j]                 (talk absent: s = raw)
//   p_h[i, j]    = exp(s_h[i, j]) / (sink + sum_j' exp(s_h[i, j']))   sink = 1 with a silent extra entry of
//                                                                 score 0, else 0;  j' over the keys i sees
//   o_h[i]       = out_scale * sum_j p_h[i, j] v_kv(h)[j]
//
// A key is seen by the query at position p when max(0, p - window + 1) <= j <= p (window <= 0: from 0).
// Because every head's score of a (query, key) pair enters every head's softmax, a block takes all
// heads of a tile of queries.  Scores, the mix, the softmax and the value sum are float32 in both
// storage types.  Also here: the kernel that prepares a step's queries, keys and values (rotation,
// per-head norm before or after it, page write) with heads of different key and value sizes.
#include "common.cuh"

// ------------------------------------------------------------------------------------------
// qkv[t] = [heads x d | kv_heads x d | kv_heads x dv].  Per q/k head, in this order:
//   norm_mode 1: x <- x / rms(x) * w      (w absent: 1)
//   rotation of the first `rot` channels by position * inv_freq[pair]  (inv_freq absent: none);
//     cos and sin are multiplied by rot_mag (1: a pure rotation)
//   norm_mode 2: x <- x / rms(x) * w
//   norm_mode 3: like 1, but ONE root mean square over all of a token's q channels (and one over all of its k
//     channels), with weights of heads x d (kv_heads x d) channels
// The values are read at v_off of the row (the default lies behind q and k; the offset of k makes the keys as
// projected, before norm and rotation, double as values; the bias is read at the same offset).
// `bias` (float32, laid out like a qkv row; absent: none) is added to q, k and v first.  With temp_every > 0 a
// query at position p is multiplied, last of all, by 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1).
// q goes to q_out[t, h], k and v into their pages ([page, kv_head, slot, d] and [.., dv]).
// One block per token, one warp per head at a time; the angles' cos/sin are formed once per token.
// ------------------------------------------------------------------------------------------
// Four consecutive elements at once where the row allows it (bfloat16: 8-byte accesses; float32: 16-byte).
template <typename T>
__device__ __forceinline__ void load4(const T* p, float (&v)[4]);
template <>
__device__ __forceinline__ void load4<float>(const float* p, float (&v)[4]) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
template <>
__device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
template <typename T>
__device__ __forceinline__ void store4(T* p, const float (&v)[4]);
template <>
__device__ __forceinline__ void store4<float>(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[4]) {
    uint2 t;
    *reinterpret_cast<__nv_bfloat162*>(&t.x) = __floats2bfloat162_rn(v[0], v[1]);
    *reinterpret_cast<__nv_bfloat162*>(&t.y) = __floats2bfloat162_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = t;
}

template <typename T>
__global__ void qkv_prepare_kernel(T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                   const T* __restrict__ qkv, const float* __restrict__ q_w, const float* __restrict__ k_w,
                                   const float* __restrict__ inv_freq, const int* __restrict__ positions,
                                   const int* __restrict__ req_of_token, const int* __restrict__ block_table,
                                   int table_stride, int nh, int nkv, int d, int dv, int rot, int interleaved, int norm_mode,
                                   int page_size, int num_pages, float eps, int write_kv, int vec4, float rot_mag,
                                   const float* __restrict__ bias, float temp_coef, int temp_every, long long row_len,
                                   long long v_off, int* err) {
    extern __shared__ float sm[];
    __shared__ float red2[2][32];
    const int half = rot / 2;
    float* cs = sm;                 // [half]
    float* sn = sm + half;          // [half]
    const int nwarps = blockDim.x >> 5, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* xs = sm + 2 * half + (size_t)warp * d;   // this warp's head
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int b = req_of_token[t];
    if (inv_freq) {
        for (int j = threadIdx.x; j < half; j += blockDim.x) {
            const float a = (float)pos * inv_freq[j];
            float s, c;
            sincosf(a, &s, &c);
            cs[j] = c * rot_mag;
            sn[j] = s * rot_mag;
        }
    }
    __syncthreads();
    long long kv_row = -1;
    if (write_kv && b >= 0) {
        const int page = block_table[(size_t)b * table_stride + pos / page_size];
        if (page < 0 || page >= num_pages) {
            if (threadIdx.x == 0) atomicOr(err, XB_ERR_BAD_PAGE);
        } else {
            kv_row = (long long)page * nkv * page_size + (pos % page_size);
        }
    }
    const T* row = qkv + (size_t)t * row_len;     // (a row may hold more behind its q, k and v)
    float inv_q = 1.f, inv_k = 1.f;
    if (norm_mode == 3) {     // one root mean square over the whole q projection, one over the whole k projection
        float sq = 0.f, sk = 0.f;
        const int nq = nh * d, nqk = (nh + nkv) * d;
        if (vec4) {           // (d a multiple of 4: a group of four never straddles q and k)
            for (int i = threadIdx.x * 4; i < nqk; i += blockDim.x * 4) {
                float v[4];
                load4<T>(row + i, v);
                float s4 = 0.f;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    if (bias) v[k] += bias[i + k];
                    s4 += v[k] * v[k];
                }
                if (i < nq) sq += s4; else sk += s4;
            }
        } else {
            for (int i = threadIdx.x; i < nqk; i += blockDim.x) {
                const float v = to_f32<T>(row[i]) + (bias ? bias[i] : 0.f);
                if (i < nq) sq += v * v; else sk += v * v;
            }
        }
        // both sums through one pass over the block: an order fixed by the thread layout
        sq = warp_sum(sq);
        sk = warp_sum(sk);
        if (lane == 0) {
            red2[0][warp] = sq;
            red2[1][warp] = sk;
        }
        __syncthreads();
        float tq = lane < nwarps ? red2[0][lane] : 0.f, tk = lane < nwarps ? red2[1][lane] : 0.f;
        tq = warp_sum(tq);
        tk = warp_sum(tk);
        inv_q = 1.f / sqrtf(tq / (float)nq + eps);
        inv_k = 1.f / sqrtf(tk / (float)(nkv * d) + eps);
    }
    // the query's temperature: it grows with the logarithm of the number of whole periods the sequence has seen
    const float q_mul = temp_every > 0 ? 1.f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.f) : 1.f;
    for (int h = warp; h < nh + 2 * nkv; h += nwarps) {
        if (h >= nh + nkv) {      // a value head: copy (plus its bias)
            if (kv_row < 0) continue;
            const int g = h - nh - nkv;
            const T* x = row + v_off + (size_t)g * dv;
            const float* bv = bias ? bias + v_off + (size_t)g * dv : nullptr;
            T* dst = v_cache + (size_t)(kv_row + (long long)g * page_size) * dv;
            if (vec4) {
                for (int i = lane * 4; i < dv; i += 128) {
                    float v[4];
                    load4<T>(x + i, v);
                    if (bv) {
#pragma unroll
                        for (int k = 0; k < 4; ++k) v[k] += bv[i + k];
                    }
                    store4<T>(dst + i, v);
                }
            } else if (bv) {
                for (int i = lane; i < dv; i += 32) dst[i] = from_f32<T>(to_f32<T>(x[i]) + bv[i]);
            } else {
                for (int i = lane; i < dv; i += 32) dst[i] = x[i];
            }
            continue;
        }
        const bool is_q = h < nh;
        if (!is_q && kv_row < 0) continue;
        const T* x = row + (size_t)h * d;
        const float* bh = bias ? bias + (size_t)h * d : nullptr;
        const float om = is_q ? q_mul : 1.f;
        T* dst = is_q ? q_out + ((size_t)t * nh + h) * d
                      : k_cache + (size_t)(kv_row + (long long)(h - nh) * page_size) * d;
        const float* nw = is_q ? q_w : k_w;
        if (norm_mode == 3 && nw) nw += (size_t)(is_q ? h : h - nh) * d;     // weights over the whole projection
        if (vec4 && (norm_mode == 0 || norm_mode == 3) && (!inv_freq || (interleaved && rot % 4 == 0))) {
            // nothing of a head is needed before its own elements can be finished (no norm over the head; pairs of
            // neighbours lie in one group of four): load, bias, norm and weight, rotation, store - no shared memory
            const float inv = norm_mode == 3 ? (is_q ? inv_q : inv_k) : 1.f;
            for (int i = lane * 4; i < d; i += 128) {
                float v[4];
                load4<T>(x + i, v);
                if (bh) {
                    const float4 b4 = *reinterpret_cast<const float4*>(bh + i);
                    v[0] += b4.x; v[1] += b4.y; v[2] += b4.z; v[3] += b4.w;
                }
                if (norm_mode == 3) {
                    float4 w4 = make_float4(1.f, 1.f, 1.f, 1.f);
                    if (nw) w4 = *reinterpret_cast<const float4*>(nw + i);
                    v[0] = v[0] * inv * w4.x; v[1] = v[1] * inv * w4.y; v[2] = v[2] * inv * w4.z; v[3] = v[3] * inv * w4.w;
                }
                if (inv_freq && i < rot) {
                    const int j = i >> 1;
                    const float u0 = v[0], w0 = v[1], u1 = v[2], w1 = v[3];
                    v[0] = u0 * cs[j] - w0 * sn[j];
                    v[1] = w0 * cs[j] + u0 * sn[j];
                    v[2] = u1 * cs[j + 1] - w1 * sn[j + 1];
                    v[3] = w1 * cs[j + 1] + u1 * sn[j + 1];
                }
#pragma unroll
                for (int k = 0; k < 4; ++k) v[k] *= om;
                store4<T>(dst + i, v);
            }
            continue;
        }
        float ss = 0.f;
        if (vec4 && norm_mode == 3) {     // the root mean square is known already: norm and weight while loading
            const float inv = is_q ? inv_q : inv_k;
            for (int i = lane * 4; i < d; i += 128) {
                float v[4];
                load4<T>(x + i, v);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    if (bh) v[k] += bh[i + k];
                    xs[i + k] = v[k] * inv * (nw ? nw[i + k] : 1.f);
                }
            }
        } else if (vec4) {
            for (int i = lane * 4; i < d; i += 128) {
                float v[4];
                load4<T>(x + i, v);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    if (bh) v[k] += bh[i + k];
                    xs[i + k] = v[k];
                    ss += v[k] * v[k];
                }
            }
        } else {
            for (int i = lane; i < d; i += 32) {
                const float v = to_f32<T>(x[i]) + (bh ? bh[i] : 0.f);
                xs[i] = v;
                ss += v * v;
            }
        }
        __syncwarp();
        if (norm_mode == 1 || (norm_mode == 3 && !vec4)) {
            const float inv = norm_mode == 3 ? (is_q ? inv_q : inv_k) : 1.f / sqrtf(warp_sum(ss) / (float)d + eps);
            for (int i = lane; i < d; i += 32) xs[i] = xs[i] * inv * (nw ? nw[i] : 1.f);
            __syncwarp();
        }
        if (inv_freq) {
            for (int j = lane; j < half; j += 32) {
                const int i0 = interleaved ? 2 * j : j, i1 = interleaved ? 2 * j + 1 : j + half;
                const float u = xs[i0], v = xs[i1];
                xs[i0] = u * cs[j] - v * sn[j];
                xs[i1] = v * cs[j] + u * sn[j];
            }
            __syncwarp();
        }
        float inv = 1.f;
        if (norm_mode == 2) {
            ss = 0.f;
            for (int i = lane; i < d; i += 32) ss += xs[i] * xs[i];
            inv = 1.f / sqrtf(warp_sum(ss) / (float)d + eps);
        }
        if (vec4) {
            for (int i = lane * 4; i < d; i += 128) {
                float v[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) v[k] = (norm_mode == 2 ? xs[i + k] * inv * (nw ? nw[i + k] : 1.f) : xs[i + k]) * om;
                store4<T>(dst + i, v);
            }
        } else if (norm_mode == 2) {
            for (int i = lane; i < d; i += 32) dst[i] = from_f32<T>(xs[i] * inv * (nw ? nw[i] : 1.f) * om);
        } else {
            for (int i = lane; i < d; i += 32) dst[i] = from_f32<T>(xs[i] * om);
        }
        __syncwarp();
    }
}

XB_EXPORT int xb_qkv_prepare(int dtype, void* q_out, void* k_cache, void* v_cache, const void* qkv, const float* q_w,
                             const float* k_w, const float* inv_freq, const int* positions, const int* req_of_token,
                             const int* block_table, int table_stride, int tokens, int nh, int nkv, int d, int dv, int rot,
                             int interleaved, int norm_mode, int page_size, int num_pages, float eps, int write_kv, float rot_mag,
                             const float* bias, float temp_coef, int temp_every, long long row_len, long long v_off,
                             int* err, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (v_off < 0) v_off = (long long)(nh + nkv) * d;
    // a warp per head at a time: as many warps as a token has heads, up to 16
    const int heads = nh + 2 * nkv;
    int threads = heads >= 16 ? 512 : (heads >= 8 ? 256 : 128);
    size_t smem = ((size_t)rot + (size_t)(threads / 32) * d) * sizeof(float);
    while (smem > 48 * 1024 && threads > 32) {     // very wide heads: fewer warps, each still with room for its head
        threads /= 2;
        smem = ((size_t)rot + (size_t)(threads / 32) * d) * sizeof(float);
    }
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    // four elements per access where every head starts on such a boundary, in the rows and in the pages
    const size_t esz = dtype == XB_F32 ? 4 : 2;
    const int vec4 = (d % 4 == 0 && dv % 4 == 0 && row_len % 4 == 0 && v_off % 4 == 0 &&
                      !(((uintptr_t)bias | (uintptr_t)q_w | (uintptr_t)k_w) & 15) &&
                      !(((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_cache | (uintptr_t)v_cache) & (4 * esz - 1))) ? 1 : 0;
    if (dtype == XB_F32)
        qkv_prepare_kernel<float><<<tokens, threads, smem, stream>>>(
            (float*)q_out, (float*)k_cache, (float*)v_cache, (const float*)qkv, q_w, k_w, inv_freq, positions, req_of_token,
            block_table, table_stride, nh, nkv, d, dv, rot, interleaved, norm_mode, page_size, num_pages, eps, write_kv, vec4, rot_mag,
            bias, temp_coef, temp_every, row_len, v_off, err);
    else
        qkv_prepare_kernel<__nv_bfloat16><<<tokens, threads, smem, stream>>>(
            (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, (const __nv_bfloat16*)qkv, q_w, k_w,
            inv_freq, positions, req_of_token, block_table, table_stride, nh, nkv, d, dv, rot, interleaved, norm_mode,
            page_size, num_pages, eps, write_kv, vec4, rot_mag, bias, temp_coef, temp_every, row_len, v_off, err);
    return xb_launch_status();
}

// ------------------------------------------------------------------------------------------
// The attention itself on FMA units.  A block takes `bq` consecutive queries of one entry (a query
// tile) with all heads and walks over the keys in tiles of BK:
//   1. per kv head: its keys to shared memory, raw scores of the group's query heads;
//   2. the mix across heads, the causal / window mask;
//   3. per (head, query) row the running maximum (it starts at 0 with a sink, whose entry is always
//      there), the weights exp(s - max) and the factor that brings earlier sums to the new maximum;
//   4. per kv head: its values to shared memory, the value sums of the group's heads (each thread
//      keeps its share of the tile's outputs in registers).
// Block x of the grid finds its (entry, tile) by walking over q_start; blocks beyond the last tile
// leave.  `parts` > 1 (single-token entries with long contexts): the keys of an entry are cut into
// `parts` ranges, block (x, y) takes range y and leaves its maximum, sum and unnormalised output in
// scratch; attn_talking_merge_kernel puts the ranges together.
// ------------------------------------------------------------------------------------------
constexpr int TA_THREADS = 256;
constexpr int TA_BK = 32;
constexpr int TA_OPT = 64;     // most outputs a thread keeps

struct TalkArgs {
    const int* q_start;
    const int* start_pos;
    const int* block_table;
    const float* talk;
    float* part_o;     // [tokens, parts, heads, dv]   (parts > 1)
    float* part_ml;    // [tokens, parts, heads, 2]
    int num_entries, table_stride, nh, nkv, d, dv, page_size, num_pages, window, sink, bq, parts, ldo;
    float scale, out_scale;
    int* err;
};

template <typename T>
__global__ void __launch_bounds__(TA_THREADS) attn_talking_kernel(T* __restrict__ out, const T* __restrict__ q,
                                                                  const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                                                                  TalkArgs a) {
    extern __shared__ float sm[];
    __shared__ int s_entry, s_tile;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int H = a.nh, G = a.nkv, d = a.d, dv = a.dv, BQ = a.bq, rep = H / G;
    if (tid == 0) {
        int tile = blockIdx.x, found = -1;
        for (int b = 0; b < a.num_entries; ++b) {
            const int n = a.q_start[b + 1] - a.q_start[b];
            const int nt = (n + BQ - 1) / BQ;
            if (tile < nt) { found = b; break; }
            tile -= nt;
        }
        s_entry = found;
        s_tile = tile;
    }
    __syncthreads();
    const int b = s_entry;
    if (b < 0) return;
    const int n_b = a.q_start[b + 1] - a.q_start[b];
    const int i0 = s_tile * BQ;
    const int nq = min(BQ, n_b - i0);
    const int t0 = a.q_start[b] + i0;
    const int p0 = a.start_pos[b] + i0;           // position of the tile's first query
    const int* table = a.block_table + (size_t)b * a.table_stride;

    const int ldk = (d > dv ? d : dv) + 1;
    float* qs = sm;                                   // [BQ][H][d]
    float* kv = qs + (size_t)BQ * H * d;              // [BK][ldk]
    float* S = kv + (size_t)TA_BK * ldk;              // [H][BQ][BK] raw
    float* P = S + (size_t)H * BQ * TA_BK;            // [H][BQ][BK] mixed, then weights
    float* tk = P + (size_t)H * BQ * TA_BK;           // [H][H]
    float* rm = tk + (size_t)H * H;                   // [H*BQ] running maximum
    float* rl = rm + H * BQ;                          // running sum
    float* rc = rl + H * BQ;                          // this tile's correction factor

    for (int e = tid; e < BQ * H * d; e += TA_THREADS) {
        const int i = e / (H * d);
        qs[e] = i < nq ? to_f32<T>(q[(size_t)(t0 + i) * H * d + (e - i * H * d)]) * a.scale : 0.f;
    }
    if (a.talk)
        for (int e = tid; e < H * H; e += TA_THREADS) tk[e] = a.talk[e];
    for (int e = tid; e < H * BQ; e += TA_THREADS) {
        rm[e] = a.sink && blockIdx.y == 0 ? 0.f : -INFINITY;
        rl[e] = a.sink && blockIdx.y == 0 ? 1.f : 0.f;
    }
    float o[TA_OPT];
#pragma unroll
    for (int k = 0; k < TA_OPT; ++k) o[k] = 0.f;
    const int n_out = BQ * H * dv;    // element e = (i * H + h) * dv + c

    // the keys this block walks over
    const int last = p0 + nq - 1;
    int lo = (a.window > 0 && p0 - a.window + 1 > 0) ? p0 - a.window + 1 : 0;
    int hi = last + 1;
    if (a.parts > 1) {
        const int tiles = (hi - lo / TA_BK * TA_BK + TA_BK - 1) / TA_BK;
        const int per = (tiles + a.parts - 1) / a.parts;
        const int first = lo / TA_BK * TA_BK + (int)blockIdx.y * per * TA_BK;
        lo = max(lo, first);
        hi = min(hi, first + per * TA_BK);
    }
    for (int k0 = lo / TA_BK * TA_BK; k0 < hi; k0 += TA_BK) {
        // 1. raw scores
        for (int g = 0; g < G; ++g) {
            __syncthreads();
            for (int e = tid; e < TA_BK * d; e += TA_THREADS) {
                const int j = e / d, c = e - j * d;
                const int key = k0 + j;
                float v = 0.f;
                if (key >= lo && key < hi) {
                    const int page = table[key / a.page_size];
                    if (page < 0 || page >= a.num_pages) {
                        if (c == 0) atomicOr(a.err, XB_ERR_BAD_PAGE);
                    } else {
                        v = to_f32<T>(k_cache[(((size_t)page * G + g) * a.page_size + key % a.page_size) * d + c]);
                    }
                }
                kv[j * ldk + c] = v;
            }
            __syncthreads();
            for (int e = tid; e < rep * BQ * TA_BK; e += TA_THREADS) {
                const int j = e % TA_BK, i = (e / TA_BK) % BQ, h = g * rep + e / (TA_BK * BQ);
                const float* qr = qs + ((size_t)i * H + h) * d;
                const float* kr = kv + j * ldk;
                float s = 0.f;
                for (int c = 0; c < d; ++c) s = fmaf(qr[c], kr[c], s);
                S[((size_t)h * BQ + i) * TA_BK + j] = s;
            }
        }
        __syncthreads();
        // 2. mix and mask
        for (int e = tid; e < H * BQ * TA_BK; e += TA_THREADS) {
            const int j = e % TA_BK, i = (e / TA_BK) % BQ, h = e / (TA_BK * BQ);
            const int key = k0 + j, p = p0 + i;
            float s;
            if (a.talk) {
                s = 0.f;
                const float* tr = tk + (size_t)h * H;
                for (int g = 0; g < H; ++g) s = fmaf(tr[g], S[((size_t)g * BQ + i) * TA_BK + j], s);
            } else {
                s = S[e];
            }
            const bool seen = i < nq && key >= lo && key < hi && key <= p && (a.window <= 0 || key > p - a.window);
            P[e] = seen ? s : -INFINITY;
        }
        __syncthreads();
        // 3. rows of the softmax
        for (int r = warp; r < H * BQ; r += TA_THREADS / 32) {
            float* pr = P + (size_t)r * TA_BK;
            const float s = pr[lane];
            const float m_old = rm[r];
            const float m_new = fmaxf(m_old, warp_max(s));
            const float w = m_new == -INFINITY ? 0.f : expf(s - m_new);
            const float sum = warp_sum(w);
            pr[lane] = w;
            if (lane == 0) {
                const float corr = m_new == -INFINITY ? 1.f : expf(m_old - m_new);
                rc[r] = corr;
                rl[r] = rl[r] * corr + sum;
                rm[r] = m_new;
            }
        }
        // 4. value sums
        for (int g = 0; g < G; ++g) {
            __syncthreads();
            for (int e = tid; e < TA_BK * dv; e += TA_THREADS) {
                const int j = e / dv, c = e - j * dv;
                const int key = k0 + j;
                float v = 0.f;
                if (key >= lo && key < hi) {
                    const int page = table[key / a.page_size];
                    if (page >= 0 && page < a.num_pages)
                        v = to_f32<T>(v_cache[(((size_t)page * G + g) * a.page_size + key % a.page_size) * dv + c]);
                }
                kv[j * ldk + c] = v;
            }
            __syncthreads();
#pragma unroll
            for (int k = 0; k < TA_OPT; ++k) {
                const int e = tid + k * TA_THREADS;
                if (e >= n_out) break;
                const int c = e % dv, ih = e / dv, h = ih % H, i = ih / H;
                if (h / rep != g) continue;
                const int r = h * BQ + i;
                const float* pr = P + (size_t)r * TA_BK;
                float acc = o[k] * rc[r];
#pragma unroll 8
                for (int j = 0; j < TA_BK; ++j) acc = fmaf(pr[j], kv[j * ldk + c], acc);
                o[k] = acc;
            }
        }
    }
    __syncthreads();
    if (a.parts > 1) {
        // one query per block here (bq == 1): leave this range's maximum, sum and output
        float* po = a.part_o + ((size_t)t0 * a.parts + blockIdx.y) * H * dv;
        float* pml = a.part_ml + ((size_t)t0 * a.parts + blockIdx.y) * H * 2;
#pragma unroll
        for (int k = 0; k < TA_OPT; ++k) {
            const int e = tid + k * TA_THREADS;
            if (e >= n_out) break;
            po[e] = o[k];
        }
        for (int h = tid; h < H; h += TA_THREADS) {
            pml[2 * h] = rm[h];
            pml[2 * h + 1] = rl[h];
        }
        return;
    }
#pragma unroll
    for (int k = 0; k < TA_OPT; ++k) {
        const int e = tid + k * TA_THREADS;
        if (e >= n_out) break;
        const int c = e % dv, ih = e / dv, h = ih % H, i = ih / H;
        if (i >= nq) continue;
        const float l = rl[h * BQ + i];
        out[(size_t)(t0 + i) * a.ldo + (size_t)h * dv + c] = from_f32<T>(l > 0.f ? o[k] / l * a.out_scale : 0.f);
    }
}

// out[t, h] = out_scale * sum_y e^(m_y - m) o_y / sum_y e^(m_y - m) l_y  over the `parts` key ranges of token t.
// One block per (token, head): the ranges' factors once into shared memory, then a thread per column.
template <typename T>
__global__ void attn_talking_merge_kernel(T* __restrict__ out, const float* __restrict__ part_o,
                                          const float* __restrict__ part_ml, int H, int dv, int parts, int ldo,
                                          float out_scale) {
    extern __shared__ float fy[];          // [parts] factors, then the sum
    const int t = blockIdx.x, h = blockIdx.y;
    const float* ml = part_ml + (size_t)t * parts * H * 2 + 2 * h;
    if (threadIdx.x < 32) {
        float m = -INFINITY;
        for (int y = threadIdx.x; y < parts; y += 32) m = fmaxf(m, ml[(size_t)y * H * 2]);
        m = warp_max(m);
        float l = 0.f;
        for (int y = threadIdx.x; y < parts; y += 32) {
            const float my = ml[(size_t)y * H * 2];
            const float f = my == -INFINITY ? 0.f : expf(my - m);
            fy[y] = f;
            l += f * ml[(size_t)y * H * 2 + 1];
        }
        l = warp_sum(l);
        if (threadIdx.x == 0) fy[parts] = l;
    }
    __syncthreads();
    const float l = fy[parts];
    const float scale = l > 0.f ? out_scale / l : 0.f;
    for (int c = threadIdx.x; c < dv; c += blockDim.x) {
        float acc = 0.f;
        for (int y = 0; y < parts; ++y) {
            const float f = fy[y];
            if (f != 0.f) acc = fmaf(f, part_o[(((size_t)t * parts + y) * H + h) * dv + c], acc);
        }
        out[(size_t)t * ldo + (size_t)h * dv + c] = from_f32<T>(acc * scale);
    }
}

template <typename T>
static int talking_merge_launch(void* out, const float* part_o, const float* part_ml, int tokens, int H, int dv, int parts,
                                int ldo, float out_scale, cudaStream_t stream) {
    const int threads = dv >= 128 ? 128 : (dv >= 64 ? 64 : 32);
    attn_talking_merge_kernel<T><<<dim3(tokens, H), threads, (parts + 1) * sizeof(float), stream>>>((T*)out, part_o, part_ml, H, dv,
                                                                                                  parts, ldo, out_scale);
    return xb_launch_status();
}

// the merge alone, for the tensor-core form of the kernel (talking_attention_mma.cu)
extern "C" int xb_attn_talking_merge_bf16(void* out, const float* part_o, const float* part_ml, int tokens, int H, int dv,
                                          int parts, int ldo, float out_scale, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    return talking_merge_launch<__nv_bfloat16>(out, part_o, part_ml, tokens, H, dv, parts, ldo, out_scale, stream);
}

static size_t talking_smem(int H, int d, int dv, int bq) {
    const int ldk = (d > dv ? d : dv) + 1;
    return ((size_t)bq * H * d + (size_t)TA_BK * ldk + 2 * (size_t)H * bq * TA_BK + (size_t)H * H + 3 * (size_t)H * bq) * sizeof(float);
}

// Largest query tile (a power of two up to `want`) whose outputs fit the threads' registers and whose
// tiles fit shared memory; 0: the sizes do not fit at all.
XB_EXPORT int xb_attn_talking_tile(int nh, int d, int dv, int want) {
    for (int bq = 16; bq >= 1; bq >>= 1) {
        if (bq > want && bq > 1) continue;
        if ((long long)bq * nh * dv <= (long long)TA_THREADS * TA_OPT && talking_smem(nh, d, dv, bq) <= 200 * 1024) return bq;
    }
    return 0;
}

XB_EXPORT int xb_attn_talking(int dtype, void* out, int ldo, const void* q, const void* k_cache, const void* v_cache,
                              const float* talk, const int* q_start, const int* start_pos, int num_entries,
                              const int* block_table, int table_stride, int tokens, int nh, int nkv, int d, int dv,
                              int page_size, int num_pages, int window, float scale, int sink, float out_scale, int bq,
                              int parts, float* part_o, float* part_ml, int* err, cudaStream_t stream) {
    if (tokens <= 0 || num_entries <= 0) return 0;
    if (bq <= 0 || (long long)bq * nh * dv > (long long)TA_THREADS * TA_OPT || nh % nkv) return (int)cudaErrorInvalidValue;
    if (parts > 1 && (bq != 1 || !part_o || !part_ml)) return (int)cudaErrorInvalidValue;
    const size_t smem = talking_smem(nh, d, dv, bq);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    TalkArgs a;
    a.q_start = q_start; a.start_pos = start_pos; a.block_table = block_table; a.talk = talk;
    a.part_o = part_o; a.part_ml = part_ml;
    a.num_entries = num_entries; a.table_stride = table_stride; a.nh = nh; a.nkv = nkv; a.d = d; a.dv = dv;
    a.page_size = page_size; a.num_pages = num_pages; a.window = window; a.sink = sink; a.bq = bq;
    a.parts = parts < 1 ? 1 : parts; a.ldo = ldo; a.scale = scale; a.out_scale = out_scale; a.err = err;
    const dim3 grid((tokens + bq - 1) / bq + num_entries, a.parts);
    int rc;
    if (dtype == XB_F32) {
        cudaFuncSetAttribute(attn_talking_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        attn_talking_kernel<float><<<grid, TA_THREADS, smem, stream>>>((float*)out, (const float*)q, (const float*)k_cache,
                                                                      (const float*)v_cache, a);
        rc = xb_launch_status();
        if (rc == 0 && a.parts > 1) {
            rc = talking_merge_launch<float>(out, part_o, part_ml, tokens, nh, dv, a.parts, ldo, out_scale, stream);
        }
    } else {
        typedef __nv_bfloat16 bf;
        cudaFuncSetAttribute(attn_talking_kernel<bf>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        attn_talking_kernel<bf><<<grid, TA_THREADS, smem, stream>>>((bf*)out, (const bf*)q, (const bf*)k_cache,
                                                                   (const bf*)v_cache, a);
        rc = xb_launch_status();
        if (rc == 0 && a.parts > 1) {
            rc = talking_merge_launch<bf>(out, part_o, part_ml, tokens, nh, dv, a.parts, ldo, out_scale, stream);
        }
    }
    return rc;
}
