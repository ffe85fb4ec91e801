// Recurrences whose state is a matrix per head, carried per request in float32:
//
//   selective_scan_kernel   (state-space duality)   S[N, P]:  S <- exp(-A dt) S + dt B x^T,   y = S^T C + D x
//   delta_rule_kernel       (gated delta rule)      S[d, dv]: S <- diag(g) S,  u = beta (v - S^T k),  S <- S + k u^T,
//                                                             o = S^T q      (read after the token's own update)    
//   gated_head_norm_kernel  the gate and the RMS norm over a head (or a group of channels) behind either
//
// Layout of both scans: a block takes one (request, head) and a tile of the state's columns (columns never mix).
// Its first warps compute: a lane keeps kRows rows of two neighbouring columns in registers; DS lanes of a warp
// share a column pair and fold their sums over rows with shuffles.  Its last warps feed them: tokens of a request
// are walked in order, a tile of TT tokens at a time, and while the computing warps work on one tile the feeding
// warps bring the next one into shared memory with asynchronous copies, work out what every column needs alike
// (step sizes, decays, unit vectors, beta) once per token, and write the tile before to memory.  The step loop
// reads broadcast vectors from shared memory only.  One block barrier per tile hands the buffers over.  The state
// is read from state[slot] at the step's first token and left there after its last, so a cut between steps changes
// nothing but when the state crosses memory.  Everything is float32: decays, softplus, exponentials, step sizes,
// unit norms, gates.
#include "common.cuh"

__device__ __forceinline__ float softplus_f32(float v) { return v > 20.f ? v : log1pf(expf(v)); }
__device__ __forceinline__ float sigmoid_exact(float v) { return 1.f / (1.f + expf(-v)); }

namespace {
constexpr int kRows = 16;            // state rows a lane keeps per column
constexpr int kRowsPad = kRows + 4;  // the same rows in shared memory, spaced so that row groups fall on different banks
constexpr int kScanTile = 16;        // tokens per tile, at most

__device__ __forceinline__ void scan_cp4(float* dst, const float* src) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(s), "l"(src) : "memory");
}
__device__ __forceinline__ void scan_cp16(float* dst, const float* src) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(src) : "memory");
}
__device__ __forceinline__ void scan_cp_land() {
    asm volatile("cp.async.commit_group;\n" ::: "memory");
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncwarp();
}

// lanes of a warp are laid out [DS row groups][32 / DS column pairs]; the sum runs over the row groups
template <int DS>
__device__ __forceinline__ float fold_rows(float v) {
#pragma unroll
    for (int o = 16; o >= 32 / DS; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_total(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ int padded_row(int j) { return (j / kRows) * kRowsPad + (j % kRows); }

// A row vector of `len` floats (rows up to `padded` are zero) into the padded layout; `vec` says that source and
// length allow 16-byte copies.
__device__ __forceinline__ void stage_rows(float* dst, const float* src, int len, int padded, int lane, bool vec) {
    if (vec) {
        for (int j = lane * 4; j < padded; j += 128) {
            if (j < len)
                scan_cp16(dst + padded_row(j), src + j);
            else
                *reinterpret_cast<float4*>(dst + padded_row(j)) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    } else {
        for (int j = lane; j < padded; j += 32) {
            if (j < len)
                scan_cp4(dst + padded_row(j), src + j);
            else
                dst[padded_row(j)] = 0.f;
        }
    }
}
// The block's columns [c_base, c_base + VT) of a row of `cols` columns; the ones past the end are zero.
__device__ __forceinline__ void stage_cols(float* dst, const float* src, int c_base, int cols, int VT, int lane, bool vec) {
    if (vec) {
        for (int c = lane * 4; c < VT; c += 128) {
            if (c_base + c < cols)
                scan_cp16(dst + c, src + c_base + c);
            else
                *reinterpret_cast<float4*>(dst + c) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    } else {
        for (int c = lane; c < VT; c += 32) {
            if (c_base + c < cols)
                scan_cp4(dst + c, src + c_base + c);
            else
                dst[c] = 0.f;
        }
    }
}
}  // namespace

// xbc[t] = [x: H*P | B: G*N | C: G*N] after the short convolution; dt is column dt_off + h of proj[t] (before
// the bias and the softplus).  state [slots, H, N, P].  y [T, H*P].  Shared memory: two stages of
// B[TT][NP] C[TT][NP] x[TT][VT] dt[TT] dec[TT], then two tiles y[TT][VT].  `cw` of the block's warps compute.
template <int DS>
__global__ void __launch_bounds__(384, 1) selective_scan_kernel(float* __restrict__ y, const float* __restrict__ xbc, int C,
                                                             const float* __restrict__ proj, long long ldp, int dt_off,
                                                             const float* __restrict__ dt_bias,
                                                             const float* __restrict__ A_log, const float* __restrict__ Dv,
                                                             float* __restrict__ state, const int* __restrict__ q_start,
                                                             const int* __restrict__ slots, int H, int P, int N, int G,
                                                             int TT, int stage, int cw, int vec) {
    extern __shared__ __align__(16) float scan_smem[];
    constexpr int CGW = 32 / DS, NP = DS * kRowsPad, NR = DS * kRows;
    const int b = blockIdx.x, h = blockIdx.y;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int VT = cw * CGW * 2, c_base = blockIdx.z * VT;
    const int slot = slots[b];
    const int t0 = q_start[b], t1 = q_start[b + 1];
    if (slot < 0 || t1 <= t0) return;
    const int inner = H * P, g = h / (H / G);
    const int ntiles = (t1 - t0 + TT - 1) / TT;
    float* sy = scan_smem + 2 * stage;
    if (w >= cw) {
        // feeding warps: warp `pi` of `pw` takes tokens pi, pi + pw, ... of every tile
        const int pi = w - cw, pw = (blockDim.x >> 5) - cw;
        const float A = expf(A_log[h]), dtb = dt_bias[h];
        auto bring = [&](int tile) {
            float* sB = scan_smem + (tile & 1) * stage;
            float* sC = sB + TT * NP;
            float* sx = sC + TT * NP;
            float* sdt = sx + TT * VT;
            const int tb = t0 + tile * TT, nt = min(TT, t1 - tb);
            for (int tt = pi; tt < nt; tt += pw) {
                const float* row = xbc + (size_t)(tb + tt) * C;
                stage_rows(sB + tt * NP, row + inner + g * N, N, NR, lane, vec);
                stage_rows(sC + tt * NP, row + inner + (G + g) * N, N, NR, lane, vec);
                stage_cols(sx + tt * VT, row + h * P, c_base, P, VT, lane, vec);
            }
            const int mine = pi + lane * pw;
            if (mine < nt) scan_cp4(sdt + mine, proj + (size_t)(tb + mine) * ldp + dt_off + h);
            scan_cp_land();
            if (mine < nt) {
                const float dt = softplus_f32(sdt[mine] + dtb);
                sdt[mine] = dt;
                sdt[TT + mine] = expf(-A * dt);
            }
        };
        auto leave = [&](int tile) {
            const float* src = sy + (tile & 1) * TT * VT;
            const int tb = t0 + tile * TT, nt = min(TT, t1 - tb);
            for (int tt = pi; tt < nt; tt += pw)
                for (int c = lane; c < VT; c += 32)
                    if (c_base + c < P) y[(size_t)(tb + tt) * inner + h * P + c_base + c] = src[tt * VT + c];
        };
        bring(0);
        __syncthreads();
        for (int tile = 0; tile < ntiles; ++tile) {
            if (tile + 1 < ntiles) bring(tile + 1);
            if (tile > 0) leave(tile - 1);
            __syncthreads();
        }
        leave(ntiles - 1);
        return;
    }
    const int ds = lane / CGW, cl = (w * CGW + lane % CGW) * 2, p0 = c_base + cl;
    const float Dh = Dv[h];
    float S0[kRows], S1[kRows];
    float* st = state + ((size_t)slot * H + h) * N * P;
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
        const int n = ds * kRows + r;
        S0[r] = (n < N && p0 < P) ? st[(size_t)n * P + p0] : 0.f;
        S1[r] = (n < N && p0 + 1 < P) ? st[(size_t)n * P + p0 + 1] : 0.f;
    }
    __syncthreads();
    for (int tile = 0; tile < ntiles; ++tile) {
        const float* sB = scan_smem + (tile & 1) * stage + ds * kRowsPad;
        const float* sC = sB + TT * NP;
        const float* sx = scan_smem + (tile & 1) * stage + 2 * TT * NP;
        const float* sdt = sx + TT * VT;
        sx += cl;
        float* out = sy + (tile & 1) * TT * VT + cl;
        const int nt = min(TT, t1 - t0 - tile * TT);
        for (int tt = 0; tt < nt; ++tt, sB += NP, sC += NP, sx += VT, out += VT) {
            const float dt = sdt[tt], dec = sdt[TT + tt];
            const float2 xv = *reinterpret_cast<const float2*>(sx);
            const float dx0 = dt * xv.x, dx1 = dt * xv.y;
            const float4* Bp = reinterpret_cast<const float4*>(sB);
            const float4* Cp = reinterpret_cast<const float4*>(sC);
            float a0 = 0.f, a1 = 0.f;
#pragma unroll
            for (int i = 0; i < kRows / 4; ++i) {
                const float4 bv = Bp[i], cv = Cp[i];
                const float bq[4] = {bv.x, bv.y, bv.z, bv.w}, cq[4] = {cv.x, cv.y, cv.z, cv.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    S0[4 * i + e] = fmaf(dec, S0[4 * i + e], bq[e] * dx0);
                    S1[4 * i + e] = fmaf(dec, S1[4 * i + e], bq[e] * dx1);
                    a0 = fmaf(S0[4 * i + e], cq[e], a0);
                    a1 = fmaf(S1[4 * i + e], cq[e], a1);
                }
            }
            a0 = fold_rows<DS>(a0);
            a1 = fold_rows<DS>(a1);
            if (ds == 0) *reinterpret_cast<float2*>(out) = make_float2(fmaf(Dh, xv.x, a0), fmaf(Dh, xv.y, a1));
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
        const int n = ds * kRows + r;
        if (n < N && p0 < P) st[(size_t)n * P + p0] = S0[r];
        if (n < N && p0 + 1 < P) st[(size_t)n * P + p0 + 1] = S1[r];
    }
}

// qkv[t] = [q: G*d | k: G*d | v: H*dv] after the short convolution; beta is column beta_off + h of proj[t] before
// the sigmoid; ag[t] holds the decay's pre-activation for (head, key channel) at its front.  q and k become unit
// vectors over a head (q also times d^-1/2); g = exp(-exp(A_log_h) softplus(a + dt_bias)) per (head, key channel).
// state [slots, H, d, dv].  o [T, H*dv].  Shared memory: two stages of q[TT][DP] k[TT][DP] g[TT][DP] v[TT][VT]
// beta[TT] kq[TT], then two tiles o[TT][VT].  With gS the decayed state, o = (gS)^T q + u (k . q).
template <int DS>
__global__ void __launch_bounds__(384, 1) delta_rule_kernel(float* __restrict__ o, const float* __restrict__ qkv, int Cq,
                                                         const float* __restrict__ proj, long long ldp, int beta_off,
                                                         const float* __restrict__ ag, long long ldag,
                                                         const float* __restrict__ dt_bias, const float* __restrict__ A_log,
                                                         float* __restrict__ state, const int* __restrict__ q_start,
                                                         const int* __restrict__ slots, int H, int G, int d, int dv,
                                                         float unit_eps, int TT, int stage, int cw, int vec) {
    extern __shared__ __align__(16) float scan_smem[];
    constexpr int CGW = 32 / DS, DP = DS * kRowsPad, NR = DS * kRows;
    const int b = blockIdx.x, h = blockIdx.y;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int VT = cw * CGW * 2, c_base = blockIdx.z * VT;
    const int slot = slots[b];
    const int t0 = q_start[b], t1 = q_start[b + 1];
    if (slot < 0 || t1 <= t0) return;
    const int kvh = h / (H / G);
    const int ntiles = (t1 - t0 + TT - 1) / TT;
    float* so = scan_smem + 2 * stage;
    if (w >= cw) {
        // feeding warps: warp `pi` of `pw` takes tokens pi, pi + pw, ... of every tile
        const int pi = w - cw, pw = (blockDim.x >> 5) - cw;
        const float A = expf(A_log[h]);
        const float qk_scale = 1.f / sqrtf((float)d);
        const float* bias = dt_bias + (size_t)h * d;
        auto bring = [&](int tile) {
            float* sq = scan_smem + (tile & 1) * stage;
            float* sk = sq + TT * DP;
            float* sg = sk + TT * DP;
            float* sv = sg + TT * DP;
            float* sbeta = sv + TT * VT;
            const int tb = t0 + tile * TT, nt = min(TT, t1 - tb);
            for (int tt = pi; tt < nt; tt += pw) {
                const float* row = qkv + (size_t)(tb + tt) * Cq;
                stage_rows(sq + tt * DP, row + kvh * d, d, NR, lane, vec);
                stage_rows(sk + tt * DP, row + (G + kvh) * d, d, NR, lane, vec);
                stage_rows(sg + tt * DP, ag + (size_t)(tb + tt) * ldag + h * d, d, NR, lane, vec);
                stage_cols(sv + tt * VT, row + 2 * G * d + h * dv, c_base, dv, VT, lane, vec);
                if (lane == 0) scan_cp4(sbeta + tt, proj + (size_t)(tb + tt) * ldp + beta_off + h);
            }
            scan_cp_land();
            for (int tt = pi; tt < nt; tt += pw) {
                float* q = sq + tt * DP;
                float* k = sk + tt * DP;
                float* gd = sg + tt * DP;
                float qq = 0.f, kk = 0.f;
                for (int j = lane; j < d; j += 32) {
                    const int at = padded_row(j);
                    qq = fmaf(q[at], q[at], qq);
                    kk = fmaf(k[at], k[at], kk);
                }
                qq = warp_total(qq);
                kk = warp_total(kk);
                const float qs = qk_scale / sqrtf(qq + unit_eps), ks = 1.f / sqrtf(kk + unit_eps);
                float kq = 0.f;
                for (int j = lane; j < d; j += 32) {
                    const int at = padded_row(j);
                    const float qn = q[at] * qs, kn = k[at] * ks;
                    q[at] = qn;
                    k[at] = kn;
                    kq = fmaf(kn, qn, kq);
                    gd[at] = expf(-A * softplus_f32(gd[at] + bias[j]));
                }
                kq = warp_total(kq);
                if (lane == 0) {
                    sbeta[TT + tt] = kq;
                    sbeta[tt] = sigmoid_exact(sbeta[tt]);
                }
            }
        };
        auto leave = [&](int tile) {
            const float* src = so + (tile & 1) * TT * VT;
            const int tb = t0 + tile * TT, nt = min(TT, t1 - tb);
            for (int tt = pi; tt < nt; tt += pw)
                for (int c = lane; c < VT; c += 32)
                    if (c_base + c < dv) o[((size_t)(tb + tt) * H + h) * dv + c_base + c] = src[tt * VT + c];
        };
        bring(0);
        __syncthreads();
        for (int tile = 0; tile < ntiles; ++tile) {
            if (tile + 1 < ntiles) bring(tile + 1);
            if (tile > 0) leave(tile - 1);
            __syncthreads();
        }
        leave(ntiles - 1);
        return;
    }
    const int ds = lane / CGW, cl = (w * CGW + lane % CGW) * 2, v0 = c_base + cl;
    float S0[kRows], S1[kRows];
    float* st = state + ((size_t)slot * H + h) * d * dv;
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
        const int j = ds * kRows + r;
        S0[r] = (j < d && v0 < dv) ? st[(size_t)j * dv + v0] : 0.f;
        S1[r] = (j < d && v0 + 1 < dv) ? st[(size_t)j * dv + v0 + 1] : 0.f;
    }
    __syncthreads();
    for (int tile = 0; tile < ntiles; ++tile) {
        const float* sq = scan_smem + (tile & 1) * stage + ds * kRowsPad;
        const float* sk = sq + TT * DP;
        const float* sg = sk + TT * DP;
        const float* sv = scan_smem + (tile & 1) * stage + 3 * TT * DP;
        const float* sbeta = sv + TT * VT;
        sv += cl;
        float* out = so + (tile & 1) * TT * VT + cl;
        const int nt = min(TT, t1 - t0 - tile * TT);
        for (int tt = 0; tt < nt; ++tt, sq += DP, sk += DP, sg += DP, sv += VT, out += VT) {
            const float beta = sbeta[tt], kq = sbeta[TT + tt];
            const float2 vv = *reinterpret_cast<const float2*>(sv);
            const float4* qp = reinterpret_cast<const float4*>(sq);
            const float4* kp = reinterpret_cast<const float4*>(sk);
            const float4* gp = reinterpret_cast<const float4*>(sg);
            float kr[kRows];
            float a10 = 0.f, a11 = 0.f, a20 = 0.f, a21 = 0.f;
#pragma unroll
            for (int i = 0; i < kRows / 4; ++i) {
                const float4 g4 = gp[i], k4 = kp[i], q4 = qp[i];
                const float gq[4] = {g4.x, g4.y, g4.z, g4.w}, kq4[4] = {k4.x, k4.y, k4.z, k4.w};
                const float qq4[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int r = 4 * i + e;
                    S0[r] *= gq[e];
                    S1[r] *= gq[e];
                    a10 = fmaf(S0[r], kq4[e], a10);
                    a11 = fmaf(S1[r], kq4[e], a11);
                    a20 = fmaf(S0[r], qq4[e], a20);
                    a21 = fmaf(S1[r], qq4[e], a21);
                    kr[r] = kq4[e];
                }
            }
            a10 = fold_rows<DS>(a10);
            a11 = fold_rows<DS>(a11);
            a20 = fold_rows<DS>(a20);
            a21 = fold_rows<DS>(a21);
            const float u0 = beta * (vv.x - a10), u1 = beta * (vv.y - a11);
#pragma unroll
            for (int r = 0; r < kRows; ++r) {
                S0[r] = fmaf(kr[r], u0, S0[r]);
                S1[r] = fmaf(kr[r], u1, S1[r]);
            }
            if (ds == 0) *reinterpret_cast<float2*>(out) = make_float2(fmaf(u0, kq, a20), fmaf(u1, kq, a21));
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
        const int j = ds * kRows + r;
        if (j < d && v0 < dv) st[(size_t)j * dv + v0] = S0[r];
        if (j < d && v0 + 1 < dv) st[(size_t)j * dv + v0 + 1] = S1[r];
    }
}

// Row groups per column pair: the smallest power of two with DS * kRows >= rows.
static inline int scan_row_groups(int rows) {
    int ds = 1;
    while (ds * kRows < rows) ds *= 2;
    return ds;
}

// Computing warps per block: enough to cover the columns (at most 8), fewer (down to 2) while the grid would
// leave a third of the processors idle.  Every block of a head repeats the feeding warps' work, so column tiles
// are not cut finer than that.
static inline int scan_warps(int cols, int ds, long long heads_total) {
    const int per_warp = (32 / ds) * 2;
    int warps = 1;
    while (warps < 8 && warps * per_warp < cols) warps *= 2;
    while (warps > 2 && heads_total * ((cols + warps * per_warp - 1) / (warps * per_warp)) < 100) warps /= 2;
    return warps;
}

static inline bool scan_aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

// Floats of one stage (`vectors` row vectors and two scalars per token beside the column tile), rounded so that
// the second stage stays 16-byte aligned; the tile shrinks until two stages and two output tiles fit.
static inline void scan_tile(int vectors, int ds, int vt, int& tt, int& stage, size_t& bytes) {
    for (tt = kScanTile;; tt /= 2) {
        stage = (tt * (vectors * ds * kRowsPad + vt + 2) + 3) & ~3;
        bytes = ((size_t)2 * stage + (size_t)2 * tt * vt) * sizeof(float);
        if (bytes <= 200 * 1024 || tt == 1) return;
    }
}

template <typename K>
static inline int scan_smem_opt_in(K kernel, size_t bytes) {
    if (bytes <= 48 * 1024) return 0;
    return (int)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

#define XB_SCAN_DISPATCH(KERNEL, DSV, ...)                                                       \
    switch (DSV) {                                                                              \
        case 1: XB_SCAN_LAUNCH(KERNEL<1>, __VA_ARGS__) break;                                   \
        case 2: XB_SCAN_LAUNCH(KERNEL<2>, __VA_ARGS__) break;                                   \
        case 4: XB_SCAN_LAUNCH(KERNEL<4>, __VA_ARGS__) break;                                   \
        case 8: XB_SCAN_LAUNCH(KERNEL<8>, __VA_ARGS__) break;                                   \
        case 16: XB_SCAN_LAUNCH(KERNEL<16>, __VA_ARGS__) break;                                 \
        default: XB_SCAN_LAUNCH(KERNEL<32>, __VA_ARGS__) break;                                 \
    }
#define XB_SCAN_LAUNCH(K, ...)                                  \
    {                                                           \
        const int rc = scan_smem_opt_in(K, bytes);              \
        if (rc) return rc;                                      \
        K<<<grid, threads, bytes, stream>>>(__VA_ARGS__);       \
    }

XB_EXPORT int xb_selective_scan(float* y, const float* xbc, int C, const float* proj, long long ldp, int dt_off,
                                const float* dt_bias, const float* A_log, const float* Dv, float* state, const int* q_start,
                                const int* slots, int entries, int H, int P, int N, int G, cudaStream_t stream) {
    if (entries <= 0) return 0;
    if (N < 1 || N > 32 * kRows || P < 1 || G < 1 || H % G || H > 65535) return (int)cudaErrorInvalidValue;
    const int ds = scan_row_groups(N);
    const int warps = scan_warps(P, ds, (long long)entries * H);
    const int vt = warps * (32 / ds) * 2;
    int tt, stage;
    size_t bytes;
    scan_tile(2, ds, vt, tt, stage, bytes);
    const dim3 grid(entries, H, (P + vt - 1) / vt);
    const int threads = (warps + 4) * 32;  // four feeding warps
    const int vec = scan_aligned16(xbc) && C % 4 == 0 && P % 4 == 0 && N % 4 == 0 && vt % 4 == 0;
    XB_SCAN_DISPATCH(selective_scan_kernel, ds, y, xbc, C, proj, ldp, dt_off, dt_bias, A_log, Dv, state, q_start, slots, H, P, N,
                     G, tt, stage, warps, vec)
    return xb_launch_status();
}

XB_EXPORT int xb_delta_rule(float* o, const float* qkv, int Cq, const float* proj, long long ldp, int beta_off, const float* ag,
                            long long ldag, const float* dt_bias, const float* A_log, float* state, const int* q_start,
                            const int* slots, int entries, int H, int G, int d, int dv, float unit_eps, cudaStream_t stream) {
    if (entries <= 0) return 0;
    if (d < 1 || d > 32 * kRows || dv < 1 || G < 1 || H % G || H > 65535) return (int)cudaErrorInvalidValue;
    const int ds = scan_row_groups(d);
    const int warps = scan_warps(dv, ds, (long long)entries * H);
    const int vt = warps * (32 / ds) * 2;
    int tt, stage;
    size_t bytes;
    scan_tile(3, ds, vt, tt, stage, bytes);
    const dim3 grid(entries, H, (dv + vt - 1) / vt);
    // the unit vectors and decays are the feeding warps' work: eight of them where the block has room, else four
    const int threads = (warps + (warps <= 4 ? 8 : 4)) * 32;
    const int vec = scan_aligned16(qkv) && scan_aligned16(ag) && Cq % 4 == 0 && ldag % 4 == 0 && d % 4 == 0 && dv % 4 == 0 &&
                    vt % 4 == 0;
    XB_SCAN_DISPATCH(delta_rule_kernel, ds, o, qkv, Cq, proj, ldp, beta_off, ag, ldag, dt_bias, A_log, state, q_start, slots, H,
                     G, d, dv, unit_eps, tt, stage, warps, vec)
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

// The same for parts of at most 32 * NV channels: a warp per (token, part) keeps its channels in registers, one pass
// over memory, sums by shuffles; a block's warps take neighbouring parts of a token.
template <typename TO, int NV>
__global__ void __launch_bounds__(256) gated_head_norm_warp_kernel(TO* __restrict__ out, const float* __restrict__ y,
                                                                   const float* __restrict__ gate, long long ldg, int g_off,
                                                                   const float* __restrict__ w, int w_len, int W, int part,
                                                                   float eps, int mode, long long units) {
    const int lane = threadIdx.x & 31;
    const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= units) return;
    const int parts = W / part;
    const long long t = unit / parts;
    const int c0 = (int)(unit % parts) * part;
    const float* yr = y + (size_t)t * W + c0;
    const float* gr = gate + (size_t)t * ldg + g_off + c0;
    float v[NV], z[NV];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int i = lane + 32 * k;
        v[k] = i < part ? yr[i] : 0.f;
        z[k] = i < part ? gr[i] : 0.f;
        if (mode == 0) v[k] *= z[k] / (1.f + expf(-z[k]));
        ss = fmaf(v[k], v[k], ss);
    }
    const float inv = 1.f / sqrtf(warp_total(ss) / (float)part + eps);
    TO* o = out + (size_t)t * W + c0;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int i = lane + 32 * k;
        if (i >= part) continue;
        float r = v[k] * inv * w[(c0 + i) % w_len];
        if (mode != 0) r *= sigmoid_exact(z[k]);
        o[i] = from_f32<TO>(r);
    }
}

template <typename TO>
static void gated_head_norm_launch(TO* out, const float* y, const float* gate, long long ldg, int g_off, const float* w,
                                   int w_len, int tokens, int W, int part, float eps, int mode, cudaStream_t stream) {
    const long long units = (long long)tokens * (W / part);
    const int warps = 8;
    const unsigned blocks = (unsigned)((units + warps - 1) / warps);
#define XB_HEAD_NORM_NV(NVV)                                                                                              \
    gated_head_norm_warp_kernel<TO, NVV><<<blocks, warps * 32, 0, stream>>>(out, y, gate, ldg, g_off, w, w_len, W, part, \
                                                                            eps, mode, units)
    if (part <= 32) XB_HEAD_NORM_NV(1);
    else if (part <= 64) XB_HEAD_NORM_NV(2);
    else if (part <= 128) XB_HEAD_NORM_NV(4);
    else if (part <= 256) XB_HEAD_NORM_NV(8);
    else if (part <= 512) XB_HEAD_NORM_NV(16);
    else {
        const dim3 grid(tokens, W / part);
        const int threads = part >= 1024 ? 256 : 128;
        gated_head_norm_kernel<TO><<<grid, threads, 0, stream>>>(out, y, gate, ldg, g_off, w, w_len, W, part, eps, mode);
    }
#undef XB_HEAD_NORM_NV
}

XB_EXPORT int xb_gated_head_norm(int out_dtype, void* out, const float* y, const float* gate, long long ldg, int g_off,
                                 const float* w, int w_len, int tokens, int W, int part, float eps, int mode,
                                 cudaStream_t stream) {
    if (tokens <= 0 || W <= 0) return 0;
    if (part <= 0 || W % part || W / part > 65535) return (int)cudaErrorInvalidValue;
    if (out_dtype == XB_F32)
        gated_head_norm_launch<float>((float*)out, y, gate, ldg, g_off, w, w_len, tokens, W, part, eps, mode, stream);
    else
        gated_head_norm_launch<__nv_bfloat16>((__nv_bfloat16*)out, y, gate, ldg, g_off, w, w_len, tokens, W, part, eps, mode,
                                              stream);
    return xb_launch_status();
}
