// Recurrences whose state is a matrix per head, carried per request in float32:
//
//   selective_scan_kernel   (state-space duality)   S[N, P]:  S <- exp(-A dt) S + dt B x^T,   y = S^T C + D x
//   delta_rule_kernel       (gated delta rule)      S[d, dv]: S <- diag(g) S,  u = beta (v - S^T k),  S <- S + k u^T,
//                                                             o = S^T q      (the read-out sees the token's own write)
//   gated_head_norm_kernel  the gate and the RMS norm over a head (or a group of channels) behind either
//
// Layout of both scans: a block takes one (request, head) and a tile of the state's columns (columns never mix);
// a column's rows are dealt out to DS neighbouring lanes, each keeping R of them in registers, and sums over
// rows are folded with shuffles.  Tokens of a request are walked in order; the state is read from state[slot] at
// the step's first token and left there after its last, so a cut between steps changes nothing but when the
// state crosses memory.  Everything is float32: decays, softplus, exponentials, step sizes, unit norms, gates.
#include "common.cuh"

__device__ __forceinline__ float softplus_f32(float v) { return v > 20.f ? v : log1pf(expf(v)); }
__device__ __forceinline__ float sigmoid_exact(float v) { return 1.f / (1.f + expf(-v)); }

template <int DS>
__device__ __forceinline__ float fold(float v) {
#pragma unroll
    for (int o = DS / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// xbc[t] = [x: H*P | B: G*N | C: G*N] after the short convolution; dt is column dt_off + h of proj[t] (before
// the bias and the softplus).  state [slots, H, N, P].  y [T, H*P].
template <int DS, int R>
__global__ void selective_scan_kernel(float* __restrict__ y, const float* __restrict__ xbc, int C,
                                      const float* __restrict__ proj, long long ldp, int dt_off,
                                      const float* __restrict__ dt_bias, const float* __restrict__ A_log,
                                      const float* __restrict__ Dv, float* __restrict__ state,
                                      const int* __restrict__ q_start, const int* __restrict__ slots, int H, int P, int N,
                                      int G) {
    const int b = blockIdx.x, h = blockIdx.y;
    const int VT = blockDim.x / DS;
    const int col = threadIdx.x / DS, ds = threadIdx.x % DS;
    const int p = blockIdx.z * VT + col;
    const int slot = slots[b];
    const int t0 = q_start[b], t1 = q_start[b + 1];
    if (slot < 0 || t1 <= t0) return;
    const bool active = p < P;
    const int inner = H * P, g = h / (H / G);
    const float A = expf(A_log[h]), dtb = dt_bias[h], Dh = Dv[h];
    float S[R];
    float* st = state + ((size_t)slot * H + h) * N * P;
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int n = ds + r * DS;
        S[r] = (active && n < N) ? st[(size_t)n * P + p] : 0.f;
    }
    for (int t = t0; t < t1; ++t) {
        const float dt = softplus_f32(proj[(size_t)t * ldp + dt_off + h] + dtb);
        const float dec = expf(-A * dt);
        const float* row = xbc + (size_t)t * C;
        const float xv = active ? row[h * P + p] : 0.f;
        const float* Bp = row + inner + g * N;
        const float* Cp = Bp + G * N;
        const float dx = dt * xv;
        float acc = 0.f;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int n = ds + r * DS;
            if (n < N) {
                S[r] = fmaf(dec, S[r], Bp[n] * dx);
                acc = fmaf(S[r], Cp[n], acc);
            }
        }
        acc = fold<DS>(acc);
        if (active && ds == 0) y[(size_t)t * inner + h * P + p] = fmaf(Dh, xv, acc);
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int n = ds + r * DS;
        if (active && n < N) st[(size_t)n * P + p] = S[r];
    }
}

// qkv[t] = [q: G*d | k: G*d | v: H*dv] after the short convolution; beta is column beta_off + h of proj[t] before
// the sigmoid; ag[t] holds the decay's pre-activation for (head, key channel) at its front.  q and k become unit
// vectors over a head (q also times d^-1/2); g = exp(-exp(A_log_h) softplus(a + dt_bias)) per (head, key channel).
// state [slots, H, d, dv].  o [T, H*dv].
template <int DS, int R>
__global__ void delta_rule_kernel(float* __restrict__ o, const float* __restrict__ qkv, int Cq,
                                  const float* __restrict__ proj, long long ldp, int beta_off,
                                  const float* __restrict__ ag, long long ldag, const float* __restrict__ dt_bias,
                                  const float* __restrict__ A_log, float* __restrict__ state,
                                  const int* __restrict__ q_start, const int* __restrict__ slots, int H, int G, int d, int dv,
                                  float unit_eps) {
    const int b = blockIdx.x, h = blockIdx.y;
    const int VT = blockDim.x / DS;
    const int col = threadIdx.x / DS, ds = threadIdx.x % DS;
    const int vc = blockIdx.z * VT + col;
    const int slot = slots[b];
    const int t0 = q_start[b], t1 = q_start[b + 1];
    if (slot < 0 || t1 <= t0) return;
    const bool active = vc < dv;
    const int kvh = h / (H / G);
    const float A = expf(A_log[h]);
    const float qk_scale = 1.f / sqrtf((float)d);
    float S[R], qr[R], kr[R], bias[R];
    float* st = state + ((size_t)slot * H + h) * d * dv;
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int j = ds + r * DS;
        S[r] = (active && j < d) ? st[(size_t)j * dv + vc] : 0.f;
        bias[r] = j < d ? dt_bias[h * d + j] : 0.f;
    }
    for (int t = t0; t < t1; ++t) {
        const float* row = qkv + (size_t)t * Cq;
        const float* qp = row + kvh * d;
        const float* kp = row + (G + kvh) * d;
        const float* ap = ag + (size_t)t * ldag + h * d;
        float sq = 0.f, sk = 0.f;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int j = ds + r * DS;
            qr[r] = j < d ? qp[j] : 0.f;
            kr[r] = j < d ? kp[j] : 0.f;
            sq = fmaf(qr[r], qr[r], sq);
            sk = fmaf(kr[r], kr[r], sk);
        }
        sq = fold<DS>(sq);
        sk = fold<DS>(sk);
        const float qs = qk_scale / sqrtf(sq + unit_eps), ks = 1.f / sqrtf(sk + unit_eps);
        const float beta = sigmoid_exact(proj[(size_t)t * ldp + beta_off + h]);
        const float vv = active ? row[2 * G * d + h * dv + vc] : 0.f;
        float a1 = 0.f, a2 = 0.f, kq = 0.f;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int j = ds + r * DS;
            if (j < d) {
                const float dec = expf(-A * softplus_f32(ap[j] + bias[r]));
                const float kn = kr[r] * ks, qn = qr[r] * qs;
                S[r] *= dec;
                a1 = fmaf(S[r], kn, a1);
                a2 = fmaf(S[r], qn, a2);
                kq = fmaf(kn, qn, kq);
                kr[r] = kn;
            }
        }
        a1 = fold<DS>(a1);
        a2 = fold<DS>(a2);
        kq = fold<DS>(kq);
        const float u = beta * (vv - a1);
#pragma unroll
        for (int r = 0; r < R; ++r) S[r] = fmaf(kr[r], u, S[r]);
        if (active && ds == 0) o[(size_t)t * H * dv + h * dv + vc] = fmaf(u, kq, a2);
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int j = ds + r * DS;
        if (active && j < d) st[(size_t)j * dv + vc] = S[r];
    }
}

// rows: the smallest (DS, R) with DS * R >= rows; columns per block so that a block has up to 256 threads
struct ScanShape {
    int ds, r;
};
static inline bool scan_shape(int rows, ScanShape& s) {
    static const ScanShape shapes[] = {{4, 4}, {4, 8}, {4, 16}, {4, 32}, {8, 32}, {16, 32}, {32, 32}};
    for (const ScanShape& c : shapes)
        if (c.ds * c.r >= rows) {
            s = c;
            return true;
        }
    return false;
}

#define XB_SCAN_DISPATCH(KERNEL, ...)                                                           \
    switch (s.ds * 100 + s.r) {                                                                \
        case 404: KERNEL<4, 4><<<grid, threads, 0, stream>>>(__VA_ARGS__); break;              \
        case 408: KERNEL<4, 8><<<grid, threads, 0, stream>>>(__VA_ARGS__); break;              \
        case 416: KERNEL<4, 16><<<grid, threads, 0, stream>>>(__VA_ARGS__); break;             \
        case 432: KERNEL<4, 32><<<grid, threads, 0, stream>>>(__VA_ARGS__); break;             \
        case 832: KERNEL<8, 32><<<grid, threads, 0, stream>>>(__VA_ARGS__); break;             \
        case 1632: KERNEL<16, 32><<<grid, threads, 0, stream>>>(__VA_ARGS__); break;           \
        default: KERNEL<32, 32><<<grid, threads, 0, stream>>>(__VA_ARGS__); break;             \
    }

static inline int scan_columns(int cols, int ds) {
    // a whole number of warps; as many columns as fit 256 threads, or all of them
    int vt = 256 / ds;
    while (vt / 2 >= cols && vt * ds > 32) vt /= 2;
    return vt;
}

XB_EXPORT int xb_selective_scan(float* y, const float* xbc, int C, const float* proj, long long ldp, int dt_off,
                                const float* dt_bias, const float* A_log, const float* Dv, float* state, const int* q_start,
                                const int* slots, int entries, int H, int P, int N, int G, cudaStream_t stream) {
    if (entries <= 0) return 0;
    ScanShape s;
    if (!scan_shape(N, s) || H % G || entries > 2147483647 || H > 65535) return (int)cudaErrorInvalidValue;
    const int vt = scan_columns(P, s.ds);
    const dim3 grid(entries, H, (P + vt - 1) / vt);
    const int threads = vt * s.ds;
    XB_SCAN_DISPATCH(selective_scan_kernel, y, xbc, C, proj, ldp, dt_off, dt_bias, A_log, Dv, state, q_start, slots, H, P, N, G)
    return xb_launch_status();
}

XB_EXPORT int xb_delta_rule(float* o, const float* qkv, int Cq, const float* proj, long long ldp, int beta_off, const float* ag,
                            long long ldag, const float* dt_bias, const float* A_log, float* state, const int* q_start,
                            const int* slots, int entries, int H, int G, int d, int dv, float unit_eps, cudaStream_t stream) {
    if (entries <= 0) return 0;
    ScanShape s;
    if (!scan_shape(d, s) || H % G || H > 65535) return (int)cudaErrorInvalidValue;
    const int vt = scan_columns(dv, s.ds);
    const dim3 grid(entries, H, (dv + vt - 1) / vt);
    const int threads = vt * s.ds;
    XB_SCAN_DISPATCH(delta_rule_kernel, o, qkv, Cq, proj, ldp, beta_off, ag, ldag, dt_bias, A_log, state, q_start, slots, H, G, d,
                     dv, unit_eps)
    return xb_launch_status();
}

// One block per (token, group of `part` consecutive channels of the W):
//   mode 0:  v = y * silu(gate);  out = v * rsqrt(mean(v^2) + eps) * w[c mod w_len]          (gate before the norm)
//   mode 1:  out = y * rsqrt(mean(y^2) + eps) * w[c mod w_len] * sigmoid(gate)               (gate behind it)
// gate is column g_off + c of a wider float32 row.
template <typename TO>
__global__ void gated_head_norm_kernel(TO* __restrict__ out, const float* __restrict__ y, const float* __restrict__ gate,
                                       long long ldg, int g_off, const float* __restrict__ w, int w_len, int W, int part,
                                       float eps, int mode) {
    __shared__ float scratch[33];
    const int t = blockIdx.x, c0 = blockIdx.y * part;
    const float* yr = y + (size_t)t * W + c0;
    const float* gr = gate + (size_t)t * ldg + g_off + c0;
    float ss = 0.f;
    for (int i = threadIdx.x; i < part; i += blockDim.x) {
        float v = yr[i];
        if (mode == 0) {
            const float z = gr[i];
            v *= z / (1.f + expf(-z));
        }
        ss = fmaf(v, v, ss);
    }
    const float inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)part + eps);
    TO* o = out + (size_t)t * W + c0;
    for (int i = threadIdx.x; i < part; i += blockDim.x) {
        const float z = gr[i];
        float v = yr[i];
        if (mode == 0)
            v = v * (z / (1.f + expf(-z))) * inv * w[(c0 + i) % w_len];
        else
            v = v * inv * w[(c0 + i) % w_len] * sigmoid_exact(z);
        o[i] = from_f32<TO>(v);
    }
}

XB_EXPORT int xb_gated_head_norm(int out_dtype, void* out, const float* y, const float* gate, long long ldg, int g_off,
                                 const float* w, int w_len, int tokens, int W, int part, float eps, int mode,
                                 cudaStream_t stream) {
    if (tokens <= 0 || W <= 0) return 0;
    if (part <= 0 || W % part || W / part > 65535) return (int)cudaErrorInvalidValue;
    const dim3 grid(tokens, W / part);
    const int threads = part >= 1024 ? 256 : (part >= 128 ? 128 : (part > 32 ? 64 : 32));
    if (out_dtype == XB_F32)
        gated_head_norm_kernel<float><<<grid, threads, 0, stream>>>((float*)out, y, gate, ldg, g_off, w, w_len, W, part, eps, mode);
    else
        gated_head_norm_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>((__nv_bfloat16*)out, y, gate, ldg, g_off, w, w_len,
                                                                           W, part, eps, mode);
    return xb_launch_status();
}
