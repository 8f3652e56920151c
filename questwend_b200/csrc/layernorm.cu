// Layer norm with a weight and no bias, y = (v - mean(v)) / sqrt(mean((v - mean(v))^2) + eps) * w, everything 32-bit,
// in the three forms a block with norms before AND after each sublayer needs, as one kernel:
//
//   plain      out = LN(x) * w
//   onto       x += LN(a) * wa                      (the norm on a sublayer's output, added onto the stream in place)
//   both       x += LN(a) * wa;  out = LN(x) * w    (that, and the norm in front of the next sublayer, in one pass:
//                                                    the stream's row is read once and never re-read)
//
// One block per row.  The row is kept in registers (rows of up to 4 x ITERS x 256 values in 16-byte pieces) or passed through
// shared memory (any width).  The variance is the mean of the squared deviations from the mean (two passes over the kept
// row), not E[v^2] - E[v]^2.  `rows`, if given, names the rows of x that are normed (out then has one row per entry).
#include "common.cuh"

template <typename TOut> struct LnPack4;
template <> struct LnPack4<float> {
    static __device__ __forceinline__ void store(float* p, float a, float b, float c, float d) { *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d); }
};
template <> struct LnPack4<bf16> {
    static __device__ __forceinline__ void store(bf16* p, float a, float b, float c, float d) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
        uint2 u;
        u.x = *reinterpret_cast<uint32_t*>(&lo);
        u.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(p) = u;
    }
};

template <typename TOut>
__global__ void layernorm_kernel(float* x, const float* a, const float* __restrict__ wa, float eps_a, int write_sum,
                                 const float* __restrict__ w, TOut* __restrict__ out, const int* __restrict__ rows, int D, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ __align__(16) float row_cache[];
    __shared__ float red[32];
    const size_t at = (size_t)(rows ? rows[blockIdx.x] : blockIdx.x) * D;
    const float inv_d = 1.f / (float)D;
    if (a) {
        float s = 0.f;
        for (int i = threadIdx.x; i < D; i += blockDim.x) { const float v = a[at + i]; row_cache[i] = v; s += v; }
        const float mean = block_sum(s, red) * inv_d;
        float q = 0.f;
        for (int i = threadIdx.x; i < D; i += blockDim.x) { const float d = row_cache[i] - mean; q += d * d; }
        const float rstd = rsqrtf(block_sum(q, red) * inv_d + eps_a);
        for (int i = threadIdx.x; i < D; i += blockDim.x) {
            const float v = x[at + i] + (row_cache[i] - mean) * rstd * wa[i];
            row_cache[i] = v;
            if (write_sum) x[at + i] = v;
        }
    } else {
        for (int i = threadIdx.x; i < D; i += blockDim.x) row_cache[i] = x[at + i];
    }
    if (!out) return;
    float s = 0.f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) s += row_cache[i];
    const float mean = block_sum(s, red) * inv_d;
    float q = 0.f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) { const float d = row_cache[i] - mean; q += d * d; }
    const float rstd = rsqrtf(block_sum(q, red) * inv_d + eps);
    const size_t to = (size_t)blockIdx.x * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) out[to + i] = from_f32<TOut>((row_cache[i] - mean) * rstd * w[i]);
}

__device__ __forceinline__ float sum4(const float4& v) { return (v.x + v.y) + (v.z + v.w); }
__device__ __forceinline__ float dev4(const float4& v, float m) {
    const float a = v.x - m, b = v.y - m, c = v.z - m, d = v.w - m;
    return (a * a + b * b) + (c * c + d * d);
}

// Rows in registers: a thread holds ITERS pieces of 4 values; all of its loads are issued together.
template <typename TOut, int ITERS>
__global__ void __launch_bounds__(256)
layernorm_rows_kernel(float* x, const float* a, const float* __restrict__ wa, float eps_a, int write_sum,
                      const float* __restrict__ w, TOut* __restrict__ out, const int* __restrict__ rows, int D, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float red[32];
    const size_t at = (size_t)(rows ? rows[blockIdx.x] : blockIdx.x) * D;
    const int n4 = D / 4;
    const float inv_d = 1.f / (float)D;
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    float4* x4 = reinterpret_cast<float4*>(x + at);
    float4 v[ITERS];
#pragma unroll
    for (int k = 0; k < ITERS; ++k) { const int i = threadIdx.x + k * 256; v[k] = i < n4 ? x4[i] : zero; }
    if (a) {
        const float4* a4 = reinterpret_cast<const float4*>(a + at);
        float4 y[ITERS], g[ITERS];
        float s = 0.f;
#pragma unroll
        for (int k = 0; k < ITERS; ++k) {
            const int i = threadIdx.x + k * 256;
            y[k] = i < n4 ? a4[i] : zero;
            g[k] = i < n4 ? reinterpret_cast<const float4*>(wa)[i] : zero;
            s += sum4(y[k]);
        }
        const float mean = block_sum(s, red) * inv_d;
        float q = 0.f;
#pragma unroll
        for (int k = 0; k < ITERS; ++k) if (threadIdx.x + k * 256 < n4) q += dev4(y[k], mean);
        const float rstd = rsqrtf(block_sum(q, red) * inv_d + eps_a);
#pragma unroll
        for (int k = 0; k < ITERS; ++k) {
            const int i = threadIdx.x + k * 256;
            if (i < n4) {
                v[k].x += (y[k].x - mean) * rstd * g[k].x;
                v[k].y += (y[k].y - mean) * rstd * g[k].y;
                v[k].z += (y[k].z - mean) * rstd * g[k].z;
                v[k].w += (y[k].w - mean) * rstd * g[k].w;
                if (write_sum) x4[i] = v[k];
            }
        }
    }
    if (!out) return;
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < ITERS; ++k) s += sum4(v[k]);
    const float mean = block_sum(s, red) * inv_d;
    float q = 0.f;
#pragma unroll
    for (int k = 0; k < ITERS; ++k) if (threadIdx.x + k * 256 < n4) q += dev4(v[k], mean);
    const float rstd = rsqrtf(block_sum(q, red) * inv_d + eps);
    const size_t to = (size_t)blockIdx.x * D;
#pragma unroll
    for (int k = 0; k < ITERS; ++k) {
        const int i = threadIdx.x + k * 256;
        if (i < n4) {
            const float4 g = reinterpret_cast<const float4*>(w)[i];
            LnPack4<TOut>::store(out + to + 4 * (size_t)i, (v[k].x - mean) * rstd * g.x, (v[k].y - mean) * rstd * g.y,
                                 (v[k].z - mean) * rstd * g.z, (v[k].w - mean) * rstd * g.w);
        }
    }
}

template <typename TOut>
static int launch_layernorm(float* x, const float* a, const float* wa, float eps_a, int write_sum, const float* w, void* out,
                            const int* rows, int n_rows, int D, float eps, cudaStream_t stream) {
    auto aligned = [](const void* p) { return (uintptr_t)p % 16 == 0; };
    const bool vec = D % 4 == 0 && aligned(x) && aligned(a) && aligned(wa) && aligned(w) && aligned(out);
    if (vec && D / 4 <= 4 * 256) {
        if (D / 4 <= 256) qwb_launch(layernorm_rows_kernel<TOut, 1>, n_rows, 256, 0, stream, x, a, wa, eps_a, write_sum, w, (TOut*)out, rows, D, eps);
        else if (D / 4 <= 2 * 256) qwb_launch(layernorm_rows_kernel<TOut, 2>, n_rows, 256, 0, stream, x, a, wa, eps_a, write_sum, w, (TOut*)out, rows, D, eps);
        else qwb_launch(layernorm_rows_kernel<TOut, 4>, n_rows, 256, 0, stream, x, a, wa, eps_a, write_sum, w, (TOut*)out, rows, D, eps);
        return qwb_check_launch("layernorm");
    }
    const size_t smem = (size_t)D * sizeof(float);
    if (smem > 200 * 1024) return qwb_fail(QWB_ERR_ARG, "layernorm: width %d does not fit in shared memory", D);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(layernorm_kernel<TOut>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return qwb_fail(QWB_ERR_CUDA, "layernorm: %s", cudaGetErrorString(e));
    }
    qwb_launch(layernorm_kernel<TOut>, n_rows, D >= 1024 ? 256 : 128, smem, stream, x, a, wa, eps_a, write_sum, w, (TOut*)out, rows, D, eps);
    return qwb_check_launch("layernorm");
}

// x [T, D] float (rows of it if `rows`); a [T, D] float or null with its weight wa; w, out may be null together (onto only).
extern "C" int qwb_layernorm(float* x, const float* a, const float* wa, float eps_a, int write_sum, const float* w, void* out,
                             int out_dtype, const int* rows, int n_rows, int D, float eps, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (D <= 0) return qwb_fail(QWB_ERR_ARG, "layernorm: bad width %d", D);
    if ((a == nullptr) != (wa == nullptr)) return qwb_fail(QWB_ERR_ARG, "layernorm: a sublayer output needs its norm's weight and the other way round");
    if ((w == nullptr) != (out == nullptr)) return qwb_fail(QWB_ERR_ARG, "layernorm: an output needs a weight and the other way round");
    if (!a && !out) return 0;
    if (rows && a && write_sum) return qwb_fail(QWB_ERR_ARG, "layernorm: the sum is written back for whole tensors only");
    if (out && out_dtype == QWB_DT_BF16) return launch_layernorm<bf16>(x, a, wa, eps_a, write_sum, w, out, rows, n_rows, D, eps, stream);
    if (!out || out_dtype == QWB_DT_F32) return launch_layernorm<float>(x, a, wa, eps_a, write_sum, w, out, rows, n_rows, D, eps, stream);
    return qwb_fail(QWB_ERR_ARG, "layernorm: unknown dtype %d", out_dtype);
}
