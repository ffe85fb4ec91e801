// The grouped product of the table-routed experts (see expert_table.cu) for bfloat16 on tensor cores:
// y[r] = a[src(r)] . w[e(r)]^T over rows grouped by expert, mma.sync m16n8k16 tiles with float32 accumulators.
// A block takes 128 rows of ONE expert and 128 rows of that expert's matrix (gated: 64 columns of gate and the
// same 64 of up, finished as act(gate) * f(up) in the accumulators, the activation by code); K runs in panels of 32 through three
// shared-memory stages filled by 16-byte asynchronous copies.  A row's sum runs over K in the same order
// whatever shares its tile, so a token's result does not depend on its company.
#include "common.cuh"
#include "mma_sync.cuh"

using namespace xbmma;

constexpr int EG_BM = 128, EG_BN = 128, EG_BK = 32, EG_LD = EG_BK + 8, EG_THREADS = 256, EG_STAGES = 3;
constexpr size_t EG_SMEM = (size_t)EG_STAGES * (EG_BM + EG_BN) * EG_LD * sizeof(__nv_bfloat16);

__device__ __forceinline__ void eg_wait_but_one() { asm volatile("cp.async.wait_group 1;\n" ::: "memory"); }

template <typename TO, bool GATED>
__global__ void __launch_bounds__(EG_THREADS) expert_gemm_mma_kernel(TO* __restrict__ y, const __nv_bfloat16* __restrict__ a,
                                                                     const __nv_bfloat16* __restrict__ w,
                                                                     const int* __restrict__ offsets,
                                                                     const int* __restrict__ perm, int gather, int top, int E,
                                                                     int N, int K, long long ldw, long long estride, int act,
                                                                     float p0, float p1) {
    extern __shared__ __align__(16) unsigned char eg_smem[];
    typedef __nv_bfloat16 (*Tile)[EG_BM][EG_LD];            // EG_BM == EG_BN
    Tile As = reinterpret_cast<Tile>(eg_smem);
    Tile Bs = reinterpret_cast<Tile>(eg_smem + (size_t)EG_STAGES * EG_BM * EG_LD * sizeof(__nv_bfloat16));
    __shared__ int s_e, s_row0, s_rows;
    __shared__ int src[EG_BM];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        int tile = blockIdx.y, found = -1, row0 = 0, rows = 0;
        for (int e = 0; e < E; ++e) {
            const int cnt = offsets[e + 1] - offsets[e];
            const int nt = (cnt + EG_BM - 1) / EG_BM;
            if (tile < nt) {
                found = e;
                row0 = offsets[e] + tile * EG_BM;
                rows = min(EG_BM, cnt - tile * EG_BM);
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
    if (tid < EG_BM) src[tid] = tid < rows ? (gather ? perm[row0 + tid] / top : row0 + tid) : -1;
    __syncthreads();
    constexpr int COLS = GATED ? EG_BN / 2 : EG_BN;           // output columns of a block
    const int n0 = blockIdx.x * COLS;
    const __nv_bfloat16* we = w + (size_t)e * estride;       // row n of this expert's matrix starts at we + n * ldw
    const int wm = warp >> 1, wn = warp & 1;                  // 4 x 2 warps: 32 rows x 64 matrix rows each

    auto load = [&](int stage, int k0) {
        // A: 128 rows x 4 pieces of 8; B: 128 rows x 4 pieces
        for (int idx = tid; idx < (EG_BM + EG_BN) * 4; idx += EG_THREADS) {
            const int r = idx >> 2, c = (idx & 3) * 8;
            const int gk = k0 + c;
            if (r < EG_BM) {
                const int s = src[r];
                const bool ok = s >= 0 && gk < K;
                cp_async16(smem_addr(&As[stage][r][c]), ok ? (const void*)(a + (size_t)s * K + gk) : (const void*)a, ok ? 16 : 0);
            } else {
                const int br = r - EG_BM;
                // gated: matrix rows 0..63 are gate columns n0.., rows 64..127 the same columns of up
                const int gn = GATED ? (br < 64 ? n0 + br : N + n0 + (br - 64)) : n0 + br;
                const bool ok = (GATED ? (n0 + (br & 63)) < N : gn < N) && gk < K;
                cp_async16(smem_addr(&Bs[stage][br][c]), ok ? (const void*)(we + (size_t)gn * ldw + gk) : (const void*)w, ok ? 16 : 0);
            }
        }
        cp_async_commit();
    };

    float acc[2][8][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[i][j][c] = 0.f;
    const int panels = (K + EG_BK - 1) / EG_BK;
    load(0, 0);
    if (panels > 1) load(1, EG_BK); else cp_async_commit();
    for (int p = 0; p < panels; ++p) {
        const int st = p % EG_STAGES;
        eg_wait_but_one();                                    // panel p has landed (panel p + 1 may still be on its way)
        __syncthreads();                                      // ... for everyone, and everyone is done with panel p - 1
        if (p + 2 < panels) load((p + 2) % EG_STAGES, (p + 2) * EG_BK); else cp_async_commit();
#pragma unroll
        for (int ks = 0; ks < EG_BK / 16; ++ks) {
            uint32_t af[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i)
                ldmatrix_x4(af[i], smem_addr(&As[st][wm * 32 + i * 16 + (lane & 15)][ks * 16 + (lane >> 4) * 8]));
#pragma unroll
            for (int jp = 0; jp < 4; ++jp) {                  // a pair of 8-row tiles of the matrix
                // gated: pairs 0, 1 are gate columns wn * 32 .., pairs 2, 3 the same columns of up
                const int base = GATED ? (jp >> 1) * 64 + wn * 32 + (jp & 1) * 16 : wn * 64 + jp * 16;
                uint32_t bf[4];
                ldmatrix_x4(bf, smem_addr(&Bs[st][base + (lane & 7) + ((lane >> 4) << 3)][ks * 16 + ((lane >> 3) & 1) * 8]));
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    mma_bf16(acc[i][jp * 2], af[i], bf[0], bf[1]);
                    mma_bf16(acc[i][jp * 2 + 1], af[i], bf[2], bf[3]);
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = wm * 32 + i * 16 + (lane >> 2) + half * 8;
            if (r >= rows) continue;
            TO* yr = y + (size_t)(row0 + r) * N;
            if (GATED) {
#pragma unroll
                for (int j = 0; j < 4; ++j)
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        const int col = n0 + wn * 32 + j * 8 + (lane & 3) * 2 + c;
                        if (col < N) {
                            const float g = acc[i][j][half * 2 + c], u = acc[i][4 + j][half * 2 + c];
                            yr[col] = from_f32<TO>(gate_mul_any(act, g, u, p0, p1));
                        }
                    }
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j)
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        const int col = n0 + wn * 64 + j * 8 + (lane & 3) * 2 + c;
                        if (col < N) yr[col] = from_f32<TO>(acc[i][j][half * 2 + c]);
                    }
            }
        }
}

// bfloat16 operands, K a multiple of 8 (16-byte copies); returns cudaErrorNotSupported for other sizes.
XB_EXPORT int xb_expert_gemm_mma(int out_dtype, void* y, const void* a, const void* w, const int* offsets, const int* perm,
                                 int gather, int top, int experts, int rows_max, int N, int K, int gated, long long ldw,
                                 long long estride, int act, float p0, float p1, cudaStream_t stream) {
    if (rows_max <= 0 || N <= 0) return 0;
    if (K % 8 || ldw % 8 || estride % 8 || ((uintptr_t)a & 15) || ((uintptr_t)w & 15)) return (int)cudaErrorNotSupported;
    typedef __nv_bfloat16 bf;
    const int cols = gated ? EG_BN / 2 : EG_BN;
    const dim3 grid((N + cols - 1) / cols, (rows_max + EG_BM - 1) / EG_BM + experts);
#define XB_EG(TO, G)                                                                                                          \
    do {                                                                                                                      \
        cudaFuncSetAttribute(expert_gemm_mma_kernel<TO, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)EG_SMEM);       \
        expert_gemm_mma_kernel<TO, G><<<grid, EG_THREADS, EG_SMEM, stream>>>((TO*)y, (const bf*)a, (const bf*)w, offsets, perm, \
                                                                            gather, top, experts, N, K, ldw, estride, act,    \
                                                                            p0, p1);                                          \
    } while (0)
    if (out_dtype == XB_F32) {
        if (gated) XB_EG(float, true); else XB_EG(float, false);
    } else {
        if (gated) XB_EG(bf, true); else XB_EG(bf, false);
    }
#undef XB_EG
    return xb_launch_status();
}
