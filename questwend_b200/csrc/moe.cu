// Routed experts: the router's choice and the experts' gated feed-forward for the tokens that chose them.
//
//   moe_route     scores = softmax(logits) over all experts (32-bit); the `top` largest, ties to the lower index;
//                 weights = the chosen scores, divided by their sum only if `renorm`
//   moe_gate_up   act[t, k, :] = silu(Wg[e] x_t) * (Wu[e] x_t), e = the k-th choice of token t
//   moe_down      out[t, :] = sum_k weight[t, k] * Wd[e_k] act[t, k, :]
//
// The products read each chosen expert's rows straight from the stacked weights (Wgu [E, 2F, D]: gate rows, then up
// rows; Wd [E, D, F]): a warp per output feature, 32-bit sums.  This is the form for a step of few tokens, where every
// token's experts are streamed once, and for the 32-bit engine.  Many bfloat16 tokens are sorted by expert instead
// and go through a library grouped product; moe_gated_act and moe_combine are the kernels around it.
#include "common.cuh"

#define QWB_MOE_MAX_TOP 16

__global__ void moe_route_kernel(const float* __restrict__ logits, int* __restrict__ chosen, float* __restrict__ weight,
                                 int T, int E, int top, int renorm) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= T) return;
    const float* z = logits + (size_t)t * E;
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) sum += expf(z[e] - mx);
    sum = warp_sum(sum);
    int picked[QWB_MOE_MAX_TOP];
    float score[QWB_MOE_MAX_TOP];
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int at = E;
        for (int e = lane; e < E; e += 32) {
            bool taken = false;
            for (int j = 0; j < k; ++j) taken |= picked[j] == e;
            if (!taken && (z[e] > best)) { best = z[e]; at = e; }
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        picked[k] = at;
        score[k] = expf(best - mx) / sum;
        total += score[k];
    }
    if (lane == 0)
        for (int k = 0; k < top; ++k) {
            chosen[(size_t)t * top + k] = picked[k];
            weight[(size_t)t * top + k] = renorm ? score[k] / total : score[k];
        }
}

extern "C" int qwb_moe_route(const float* logits, int* chosen, float* weight, int T, int E, int top, int renorm, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (E <= 0 || top <= 0 || top > E || top > QWB_MOE_MAX_TOP)
        return qwb_fail(QWB_ERR_ARG, "moe_route: %d of %d experts (at most %d)", top, E, QWB_MOE_MAX_TOP);
    qwb_launch(moe_route_kernel, (T + 3) / 4, 128, 0, stream, logits, chosen, weight, T, E, top, renorm);
    return qwb_check_launch("moe_route");
}

template <typename T>
__device__ __forceinline__ float warp_dot(const T* __restrict__ w, const T* __restrict__ x, int n, int lane) {
    constexpr int VEC = Vec16<T>::N;
    float acc = 0.f;
    if (n % VEC == 0 && (uintptr_t)w % 16 == 0 && (uintptr_t)x % 16 == 0) {
        const Vec16<T>* w16 = reinterpret_cast<const Vec16<T>*>(w);
        const Vec16<T>* x16 = reinterpret_cast<const Vec16<T>*>(x);
        for (int i = lane; i < n / VEC; i += 32) {
            float a[VEC], b[VEC];
            w16[i].get(a);
            x16[i].get(b);
#pragma unroll
            for (int e = 0; e < VEC; ++e) acc += a[e] * b[e];
        }
    } else {
        for (int i = lane; i < n; i += 32) acc += to_f32(w[i]) * to_f32(x[i]);
    }
    return warp_sum(acc);
}

// grid (ceil(F / 8), T * top); 8 warps, a feature each
template <typename T>
__global__ void moe_gate_up_kernel(const T* __restrict__ x, const T* __restrict__ wgu, const int* __restrict__ chosen,
                                   T* __restrict__ act, int D, int F, int top) {
    pdl_wait();
    pdl_launch_dependents();
    const int slot = blockIdx.y, t = slot / top;
    const int f = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (f >= F) return;
    const T* w = wgu + (size_t)chosen[slot] * 2 * F * D;
    const T* xr = x + (size_t)t * D;
    const float g = warp_dot(w + (size_t)f * D, xr, D, lane);
    const float u = warp_dot(w + (size_t)(F + f) * D, xr, D, lane);
    if (lane == 0) act[(size_t)slot * F + f] = from_f32<T>(g / (1.f + expf(-g)) * u);
}

// grid (ceil(D / 8), T); 8 warps, an output each
template <typename T>
__global__ void moe_down_kernel(const T* __restrict__ act, const T* __restrict__ wd, const int* __restrict__ chosen,
                                const float* __restrict__ weight, float* __restrict__ out, int D, int F, int top) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.y;
    const int d = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (d >= D) return;
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        const size_t slot = (size_t)t * top + k;
        const T* w = wd + ((size_t)chosen[slot] * D + d) * F;
        total += weight[slot] * warp_dot(w, act + slot * F, F, lane);
    }
    if (lane == 0) out[(size_t)t * D + d] = total;
}

extern "C" int qwb_moe_experts(const void* x, const void* wgu, const void* wd, const int* chosen, const float* weight,
                               void* act, float* out, int dtype, int T, int D, int F, int top, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (D <= 0 || F <= 0 || top <= 0) return qwb_fail(QWB_ERR_ARG, "moe_experts: width %d, expert width %d, %d choices", D, F, top);
    if ((long long)T * top > 65535 || T > 65535) return qwb_fail(QWB_ERR_ARG, "moe_experts: %d tokens x %d choices are too many for one launch", T, top);
    const dim3 g1((F + 7) / 8, T * top), g2((D + 7) / 8, T);
    if (dtype == QWB_DT_F32) {
        qwb_launch(moe_gate_up_kernel<float>, g1, 256, 0, stream, (const float*)x, (const float*)wgu, chosen, (float*)act, D, F, top);
        qwb_launch(moe_down_kernel<float>, g2, 256, 0, stream, (const float*)act, (const float*)wd, chosen, weight, out, D, F, top);
    } else if (dtype == QWB_DT_BF16) {
        qwb_launch(moe_gate_up_kernel<bf16>, g1, 256, 0, stream, (const bf16*)x, (const bf16*)wgu, chosen, (bf16*)act, D, F, top);
        qwb_launch(moe_down_kernel<bf16>, g2, 256, 0, stream, (const bf16*)act, (const bf16*)wd, chosen, weight, out, D, F, top);
    } else {
        return qwb_fail(QWB_ERR_ARG, "moe_experts: unknown dtype %d", dtype);
    }
    return qwb_check_launch("moe_experts");
}

// ---------------------------------------------------------------------------------
// Around a grouped product over token copies sorted by expert (bfloat16):
//   moe_gated_act  act[s, f] = silu(gu[s, f]) * gu[s, F + f]           gu [S, 2F] -> act [S, F]
//   moe_combine    out[t, :] = sum_k weight[t, k] * y[place[t, k], :]   y [S, D] -> out float [T, D]
// place[t, k] is the row of token t's k-th copy in the sorted order.
// ---------------------------------------------------------------------------------
__global__ void moe_gated_act_kernel(const bf16* __restrict__ gu, bf16* __restrict__ act, size_t n, int F) {
    pdl_wait();
    pdl_launch_dependents();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / F, f = i - r * F;
        const float g = to_f32(gu[r * 2 * F + f]), u = to_f32(gu[r * 2 * F + F + f]);
        act[i] = from_f32<bf16>(g / (1.f + expf(-g)) * u);
    }
}

extern "C" int qwb_moe_gated_act(const void* gu, void* act, int S, int F, cudaStream_t stream) {
    if (S <= 0 || F <= 0) return 0;
    const size_t n = (size_t)S * F;
    const int block = 256, grid = (int)((n + block - 1) / block < 148 * 16 ? (n + block - 1) / block : 148 * 16);
    qwb_launch(moe_gated_act_kernel, grid, block, 0, stream, (const bf16*)gu, (bf16*)act, n, F);
    return qwb_check_launch("moe_gated_act");
}

__global__ void moe_combine_kernel(const bf16* __restrict__ y, const long long* __restrict__ place, const float* __restrict__ weight,
                                   float* __restrict__ out, int D, int top) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float total = 0.f;
        for (int k = 0; k < top; ++k)
            total += weight[(size_t)t * top + k] * to_f32(y[(size_t)place[(size_t)t * top + k] * D + d]);
        out[(size_t)t * D + d] = total;
    }
}

extern "C" int qwb_moe_combine(const void* y, const long long* place, const float* weight, float* out, int T, int D, int top,
                               cudaStream_t stream) {
    if (T <= 0 || D <= 0) return 0;
    qwb_launch(moe_combine_kernel, T, D >= 1024 ? 256 : 128, 0, stream, (const bf16*)y, place, weight, out, D, top);
    return qwb_check_launch("moe_combine");
}
