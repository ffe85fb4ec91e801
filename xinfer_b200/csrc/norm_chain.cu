// RMS norm that takes the residual arithmetic around it into one pass over a row of the float32 stream:
//
//   br  = branch[src]                                      (either type; absent: no addition)
//   br' = bw ? br * rsqrt(mean(br^2) + beps) * (boffset + bw) : br        the branch's own RMS norm
//   s   = x[src] + bscale * gain * br'                      gain: a learned vector (absent: ones)
//   out = w ? s * rsqrt(mean(s^2) + eps) * (offset + w) : s                in TO; out absent: only the sum
//
// sum_out (float32, nullable) receives s; it may be x itself when no rows are gathered.  Sums and statistics are
// float32; a row is reduced in an order fixed by the thread layout, so a row's result does not depend on the batch.
// Also here: the sum of two RMS-normed branches, a bias added to rows, and the gated activation with biases.
#include "common.cuh"

template <typename TB, typename TO>
__global__ void rms_chain_kernel(TO* __restrict__ out, float* sum_out, const float* x, const TB* __restrict__ branch,
                                 const int* __restrict__ rows, const float* __restrict__ w, const float* __restrict__ bw,
                                 const float* __restrict__ gain, int dim, int src_rows, float eps, float offset, float beps,
                                 float boffset, float bscale, int* err) {
    __shared__ float scratch[33];
    extern __shared__ float srow[];
    const int r = blockIdx.x;
    int src = rows ? rows[r] : r;
    if (src < 0 || src >= src_rows) {
        if (threadIdx.x == 0) atomicOr(err, XB_ERR_BAD_ROW);
        src = 0;
    }
    const float* xr = x + (size_t)src * dim;
    const TB* br = branch ? branch + (size_t)src * dim : nullptr;
    float binv = 1.f;
    if (br && bw) {
        float sb = 0.f;
        for (int i = threadIdx.x; i < dim; i += blockDim.x) {
            const float v = to_f32<TB>(br[i]);
            srow[i] = v;
            sb += v * v;
        }
        binv = 1.f / sqrtf(block_sum(sb, scratch) / (float)dim + beps);
    }
    float ss = 0.f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        float v = xr[i];
        if (br) {
            float b = bw ? srow[i] * binv * (boffset + bw[i]) : to_f32<TB>(br[i]);
            if (gain) b *= gain[i];
            v = bscale == 1.f ? v + b : fmaf(bscale, b, v);
        }
        srow[i] = v;
        ss += v * v;
    }
    float inv = 1.f;
    if (out && w) inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)dim + eps);
    TO* o = out ? out + (size_t)r * dim : nullptr;
    float* so = sum_out ? sum_out + (size_t)r * dim : nullptr;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float v = srow[i];
        if (so) so[i] = v;
        if (o) o[i] = from_f32<TO>(w ? v * inv * (offset + w[i]) : v);
    }
}

template <typename TB, typename TO>
static int rms_chain_launch(void* out, float* sum_out, const float* x, const void* branch, const int* rows, const float* w,
                            const float* bw, const float* gain, int nrows, int dim, int src_rows, float eps, float offset,
                            float beps, float boffset, float bscale, int* err, cudaStream_t stream) {
    const size_t smem = (size_t)dim * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    if (smem > 48 * 1024) cudaFuncSetAttribute(rms_chain_kernel<TB, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    const int threads = dim >= 2048 ? 512 : (dim >= 512 ? 256 : 128);
    rms_chain_kernel<TB, TO><<<nrows, threads, smem, stream>>>((TO*)out, sum_out, x, (const TB*)branch, rows, w, bw, gain, dim,
                                                              src_rows, eps, offset, beps, boffset, bscale, err);
    return xb_launch_status();
}

XB_EXPORT int xb_rms_chain(int branch_dtype, int out_dtype, void* out, float* sum_out, const float* x, const void* branch,
                           const int* rows, const float* w, const float* bw, const float* gain, int nrows, int dim,
                           int src_rows, float eps, float offset, float beps, float boffset, float bscale, int* err,
                           cudaStream_t stream) {
    if (nrows <= 0) return 0;
    typedef __nv_bfloat16 bf;
#define XB_ARGS out, sum_out, x, branch, rows, w, bw, gain, nrows, dim, src_rows, eps, offset, beps, boffset, bscale, err, stream
    if (branch_dtype == XB_F32) return out_dtype == XB_F32 ? rms_chain_launch<float, float>(XB_ARGS) : rms_chain_launch<float, bf>(XB_ARGS);
    return out_dtype == XB_F32 ? rms_chain_launch<bf, float>(XB_ARGS) : rms_chain_launch<bf, bf>(XB_ARGS);
#undef XB_ARGS
}

// out = sl * l * rsqrt(mean(l^2) + eps) * (offset + wl) + sr * r * rsqrt(mean(r^2) + eps) * (offset + wr), row by row
template <typename T>
__global__ void dual_rms_sum_kernel(T* __restrict__ out, const T* __restrict__ l, const T* __restrict__ r,
                                    const float* __restrict__ wl, const float* __restrict__ wr, int dim, float eps,
                                    float offset, float sl, float sr) {
    __shared__ float scratch[33];
    const size_t base = (size_t)blockIdx.x * dim;
    float a = 0.f, b = 0.f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float u = to_f32<T>(l[base + i]), v = to_f32<T>(r[base + i]);
        a += u * u;
        b += v * v;
    }
    const float il = 1.f / sqrtf(block_sum(a, scratch) / (float)dim + eps);
    const float ir = 1.f / sqrtf(block_sum(b, scratch) / (float)dim + eps);
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float u = to_f32<T>(l[base + i]) * il * (offset + wl[i]);
        const float v = to_f32<T>(r[base + i]) * ir * (offset + wr[i]);
        out[base + i] = from_f32<T>(sl * u + sr * v);
    }
}

XB_EXPORT int xb_dual_rms_sum(int dtype, void* out, const void* l, const void* r, const float* wl, const float* wr, int rows,
                              int dim, float eps, float offset, float sl, float sr, cudaStream_t stream) {
    if (rows <= 0) return 0;
    const int threads = dim >= 2048 ? 512 : (dim >= 512 ? 256 : 128);
    if (dtype == XB_F32)
        dual_rms_sum_kernel<float><<<rows, threads, 0, stream>>>((float*)out, (const float*)l, (const float*)r, wl, wr, dim, eps, offset, sl, sr);
    else
        dual_rms_sum_kernel<__nv_bfloat16><<<rows, threads, 0, stream>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)l,
                                                                        (const __nv_bfloat16*)r, wl, wr, dim, eps, offset, sl, sr);
    return xb_launch_status();
}

// x[t, i] += bias[i]
template <typename T>
__global__ void add_bias_kernel(T* x, const float* __restrict__ bias, size_t n, int dim) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = from_f32<T>(to_f32<T>(x[i]) + bias[i % dim]);
}

XB_EXPORT int xb_add_bias(int dtype, void* x, const float* bias, int rows, int dim, cudaStream_t stream) {
    const size_t n = (size_t)rows * dim;
    if (n == 0) return 0;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (dtype == XB_F32)
        add_bias_kernel<float><<<blocks, 256, 0, stream>>>((float*)x, bias, n, dim);
    else
        add_bias_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((__nv_bfloat16*)x, bias, n, dim);
    return xb_launch_status();
}

// out[t, i] = act(gu[t, i] + bias[i]) * (gu[t, I + i] + bias[I + i])    (float32 arithmetic, exact exponential)
template <typename TI, typename TO, int ACT>
__global__ void swiglu_bias_kernel(TO* __restrict__ out, const TI* __restrict__ gu, const float* __restrict__ bias, int I,
                                   size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const size_t t = i / I;
    const int c = (int)(i % I);
    const float g = to_f32<TI>(gu[t * 2 * I + c]) + bias[c];
    const float u = to_f32<TI>(gu[t * 2 * I + I + c]) + bias[I + c];
    out[i] = from_f32<TO>(gate_mul_f32<ACT>(g, u));
}

template <typename TI, typename TO>
static int swiglu_bias_launch(void* out, const void* gu, const float* bias, int rows, int I, int act, cudaStream_t stream) {
    const size_t n = (size_t)rows * I;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (act == XB_ACT_GELU_TANH)
        swiglu_bias_kernel<TI, TO, XB_ACT_GELU_TANH><<<blocks, 256, 0, stream>>>((TO*)out, (const TI*)gu, bias, I, n);
    else
        swiglu_bias_kernel<TI, TO, XB_ACT_SILU><<<blocks, 256, 0, stream>>>((TO*)out, (const TI*)gu, bias, I, n);
    return xb_launch_status();
}

XB_EXPORT int xb_swiglu_bias(int in_dtype, int out_dtype, void* out, const void* gu, const float* bias, int rows, int I, int act,
                             cudaStream_t stream) {
    if (rows <= 0 || I <= 0) return 0;
    typedef __nv_bfloat16 bf;
    if (in_dtype == XB_F32)
        return out_dtype == XB_F32 ? swiglu_bias_launch<float, float>(out, gu, bias, rows, I, act, stream)
                                   : swiglu_bias_launch<float, bf>(out, gu, bias, rows, I, act, stream);
    return out_dtype == XB_F32 ? swiglu_bias_launch<bf, float>(out, gu, bias, rows, I, act, stream)
                               : swiglu_bias_launch<bf, bf>(out, gu, bias, rows, I, act, stream);
}
