// What a model adds to a token's embedding row, and what a layer reads from a table over token ids.
//
//   embed_sum_kernel     x[t] = E[id] * scale + Pair[row(prev, id)] + Pos[position]          (float32 out)
//                        row = (prev * mul_prev + id * mul_cur) mod buckets; the first token of a sequence, which has
//                        no predecessor, takes row `buckets`.  The predecessor of a step's first token of a request is
//                        the request's state (prev_state[slot]); prev_store_kernel leaves a step's last token there.
//   token_gate_kernel    g[t, j] = gelu_tanh(u[t, j]) * Table[id, col0 + j]
//
// A token id -1 - i stands for sampled[i], an id that a sampler left on the device.
#include "common.cuh"

__device__ __forceinline__ int resolve_id(const int* __restrict__ ids, int t, const int* __restrict__ sampled, int num_sampled) {
    int id = ids[t];
    if (id < 0 && sampled != nullptr && -1 - id < num_sampled) id = sampled[-1 - id];
    return id;
}

template <typename T>
__global__ void embed_sum_kernel(float* __restrict__ out, const T* __restrict__ table, const T* __restrict__ pair,
                                 const T* __restrict__ pos_table, const int* __restrict__ ids, const int* __restrict__ sampled,
                                 int num_sampled, const int* __restrict__ positions, const int* __restrict__ req_of_token,
                                 const int* __restrict__ q_start, const int* __restrict__ slots,
                                 const int* __restrict__ prev_state, int hidden, int vocab, int buckets, long long mul_prev,
                                 long long mul_cur, int max_pos, float scale, int* err) {
    const int t = blockIdx.x;
    float* o = out + (size_t)t * hidden;
    const int b = req_of_token[t];
    const int id = resolve_id(ids, t, sampled, num_sampled);
    const int p = positions[t];
    bool bad = false;
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicOr(err, XB_ERR_BAD_TOKEN);
        bad = true;
    }
    if (pos_table != nullptr && (p < 0 || p >= max_pos)) {
        if (threadIdx.x == 0 && b >= 0) atomicOr(err, XB_ERR_BAD_POSITION);
        bad = true;
    }
    if (b < 0 || bad) {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = 0.f;
        return;
    }
    const T* pr = nullptr;
    if (pair != nullptr) {
        long long row = buckets;
        if (p > 0) {
            int prev;
            if (t > q_start[b]) {
                prev = resolve_id(ids, t - 1, sampled, num_sampled);
            } else {
                const int slot = slots[b];
                prev = slot >= 0 ? prev_state[slot] : 0;
            }
            if (prev < 0 || prev >= vocab) {
                if (threadIdx.x == 0) atomicOr(err, XB_ERR_BAD_TOKEN);
                prev = 0;
            }
            row = ((long long)prev * mul_prev + (long long)id * mul_cur) % (long long)buckets;
            if (row < 0) row += buckets;
        }
        pr = pair + (size_t)row * hidden;
    }
    const T* r = table + (size_t)id * hidden;
    const T* ps = pos_table ? pos_table + (size_t)p * hidden : nullptr;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = to_f32<T>(r[i]) * scale;
        if (pr) v += to_f32<T>(pr[i]);
        if (ps) v += to_f32<T>(ps[i]);
        o[i] = v;
    }
}

XB_EXPORT int xb_embed_sum(int table_dtype, float* out, const void* table, const void* pair, const void* pos_table,
                           const int* ids, const int* sampled, int num_sampled, const int* positions, const int* req_of_token,
                           const int* q_start, const int* slots, const int* prev_state, int tokens, int hidden, int vocab,
                           int buckets, long long mul_prev, long long mul_cur, int max_pos, float scale, int* err,
                           cudaStream_t stream) {
    if (tokens <= 0) return 0;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (table_dtype == XB_F32)
        embed_sum_kernel<float><<<tokens, threads, 0, stream>>>(out, (const float*)table, (const float*)pair, (const float*)pos_table,
                                                               ids, sampled, num_sampled, positions, req_of_token, q_start, slots,
                                                               prev_state, hidden, vocab, buckets, mul_prev, mul_cur, max_pos, scale, err);
    else
        embed_sum_kernel<__nv_bfloat16><<<tokens, threads, 0, stream>>>(
            out, (const __nv_bfloat16*)table, (const __nv_bfloat16*)pair, (const __nv_bfloat16*)pos_table, ids, sampled,
            num_sampled, positions, req_of_token, q_start, slots, prev_state, hidden, vocab, buckets, mul_prev, mul_cur, max_pos,
            scale, err);
    return xb_launch_status();
}

// prev_state[slot of entry b] = the entry's last token of this step
__global__ void prev_store_kernel(int* __restrict__ prev_state, const int* __restrict__ ids, const int* __restrict__ sampled,
                                  int num_sampled, const int* __restrict__ q_start, const int* __restrict__ slots, int entries) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= entries) return;
    const int slot = slots[b];
    const int t0 = q_start[b], t1 = q_start[b + 1];
    if (slot < 0 || t1 <= t0) return;
    prev_state[slot] = resolve_id(ids, t1 - 1, sampled, num_sampled);
}

XB_EXPORT int xb_prev_store(int* prev_state, const int* ids, const int* sampled, int num_sampled, const int* q_start,
                            const int* slots, int entries, cudaStream_t stream) {
    if (entries <= 0) return 0;
    prev_store_kernel<<<(entries + 127) / 128, 128, 0, stream>>>(prev_state, ids, sampled, num_sampled, q_start, slots, entries);
    return xb_launch_status();
}

template <typename T>
__global__ void token_gate_kernel(T* __restrict__ out, const T* __restrict__ u, const T* __restrict__ table, int table_ld,
                                  int col0, const int* __restrict__ ids, const int* __restrict__ sampled, int num_sampled,
                                  const int* __restrict__ req_of_token, int dim, int vocab, size_t n, int* err) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int t = (int)(i / dim), j = (int)(i % dim);
    const int id = resolve_id(ids, t, sampled, num_sampled);
    if (req_of_token[t] < 0 || id < 0 || id >= vocab) {
        if (req_of_token[t] >= 0 && j == 0) atomicOr(err, XB_ERR_BAD_TOKEN);
        out[i] = from_f32<T>(0.f);
        return;
    }
    const float e = to_f32<T>(table[(size_t)id * table_ld + col0 + j]);
    out[i] = from_f32<T>(gelu_tanh_f32(to_f32<T>(u[i])) * e);
}

XB_EXPORT int xb_token_gate(int dtype, void* out, const void* u, const void* table, int table_ld, int col0, const int* ids,
                            const int* sampled, int num_sampled, const int* req_of_token, int tokens, int dim, int vocab,
                            int* err, cudaStream_t stream) {
    const size_t n = (size_t)tokens * dim;
    if (n == 0) return 0;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (dtype == XB_F32)
        token_gate_kernel<float><<<blocks, 256, 0, stream>>>((float*)out, (const float*)u, (const float*)table, table_ld, col0, ids,
                                                            sampled, num_sampled, req_of_token, dim, vocab, n, err);
    else
        token_gate_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)u,
                                                                    (const __nv_bfloat16*)table, table_ld, col0, ids, sampled,
                                                                    num_sampled, req_of_token, dim, vocab, n, err);
    return xb_launch_status();
}
