// Latent attention for prompts that start a sequence, on the tensor cores (bfloat16, mma.sync m16n8k16).
//
// A prompt's keys and values per head are made once from its latents by two library products (k_plain = c W_uk^T,
// v = c W_uv^T), so a head's key is [k_plain_h | rotated part shared by the heads] and the attention is the usual one
// over DQ = dim + rot_dim query/key values and DV value values: cheaper for many tokens than scoring against the
// latents themselves (csrc/attention_latent.cu does that, for single tokens, continued prompts and the 32-bit engine).
// Causal, optional window (key j visible from position p when p - window < j <= p), optional sink per head (one more
// term exp(sink) in the denominator).  Scores, maxima, sums and the output accumulator are 32-bit; probabilities are
// rounded to bfloat16 for the second product, as in every tensor-core attention.
//
// Block = 64 queries of one (sequence, head), 4 warps of 16 rows; keys in tiles of 64.  Q, K and V tiles sit in shared
// memory with rows padded by 16 bytes (conflict-free ldmatrix); K and V have two buffers, and the next tile is copied
// in (cp.async) while this one is multiplied.
#include "common.cuh"

#define LM_BQ 64
#define LM_BK 64
#define LM_PAD 8

__device__ __forceinline__ void ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const bf16* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const bf16* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// 16 bytes from global to shared memory without passing through registers; `bytes` 0 writes zeros (src must still be valid)
__device__ __forceinline__ void cp_async16(bf16* dst, const bf16* src, int bytes) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// q [T, H, DQ]; k_plain [T, H, K]; k_rot: R values at kr + t * ld_kr; v [T, H, DV]; out [T, H * DV].  All bfloat16.
// K, R, DV multiples of 8; DQ = K + R a multiple of 16; DV <= 8 * NV.
template <int NV>       // n-tiles of 8 value columns the accumulator has room for
__global__ void __launch_bounds__(128)
latent_prefill_mma_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_plain, const bf16* __restrict__ kr, int ld_kr,
                          const bf16* __restrict__ v, const int* __restrict__ cu_seqlens, const float* __restrict__ sink,
                          bf16* __restrict__ out, int H, int K, int R, int DV, float scale, int window) {
    pdl_wait();
    pdl_launch_dependents();
    const int DQ = K + R;
    const int ldq = DQ + LM_PAD, ldv = DV + LM_PAD;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);           // [64][ldq]
    bf16* Kbuf = Qs + LM_BQ * ldq;                          // [2][64][ldq]
    bf16* Vbuf = Kbuf + 2 * LM_BK * ldq;                    // [2][64][ldv]

    const int b = blockIdx.z, h = blockIdx.y, q0 = blockIdx.x * LM_BQ;
    const int t0 = cu_seqlens[b], n = cu_seqlens[b + 1] - t0;
    if (q0 >= n) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // the queries of the tile (rows beyond the sequence: zeros), in the first copy group
    for (int idx = tid; idx < LM_BQ * (DQ / 8); idx += blockDim.x) {
        const int r = idx / (DQ / 8), c = (idx - r * (DQ / 8)) * 8;
        const bool in = q0 + r < n;
        cp_async16(Qs + r * ldq + c, q + ((size_t)(t0 + (in ? q0 + r : 0)) * H + h) * DQ + c, in ? 16 : 0);
    }

    float o[NV][4];
#pragma unroll
    for (int j = 0; j < NV; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;      // rows g and g + 8 of the warp's 16
    const int g = lane >> 2, tq = lane & 3;
    const int row0 = q0 + warp * 16 + g, row1 = row0 + 8;           // positions in the sequence (it starts at 0)

    const int k_hi = min(n, q0 + LM_BQ) - 1;
    const int k_lo = window > 0 ? max(0, q0 - window + 1) : 0;
    const int nv_used = DV / 8;
    const int kt0 = (k_lo / LM_BK) * LM_BK;

    auto copy_tile = [&](int kt, int stage) {                       // one commit group a tile
        bf16* Kd = Kbuf + stage * LM_BK * ldq;
        bf16* Vd = Vbuf + stage * LM_BK * ldv;
        for (int idx = tid; idx < LM_BK * (DQ / 8); idx += blockDim.x) {
            const int r = idx / (DQ / 8), c = (idx - r * (DQ / 8)) * 8;
            const bool in = kt + r < n;
            const size_t t = (size_t)(t0 + (in ? kt + r : 0));
            cp_async16(Kd + r * ldq + c, c < K ? k_plain + (t * H + h) * K + c : kr + t * ld_kr + (c - K), in ? 16 : 0);
        }
        for (int idx = tid; idx < LM_BK * (DV / 8); idx += blockDim.x) {
            const int r = idx / (DV / 8), c = (idx - r * (DV / 8)) * 8;
            const bool in = kt + r < n;
            cp_async16(Vd + r * ldv + c, v + ((size_t)(t0 + (in ? kt + r : 0)) * H + h) * DV + c, in ? 16 : 0);
        }
        cp_async_commit();
    };
    copy_tile(kt0, 0);

    for (int kt = kt0, it = 0; kt <= k_hi; kt += LM_BK, ++it) {
        const bf16* Ks = Kbuf + (it & 1) * LM_BK * ldq;
        const bf16* Vs = Vbuf + (it & 1) * LM_BK * ldv;
        if (kt + LM_BK <= k_hi) {                                   // the next tile into the other buffer (its last readers
            copy_tile(kt + LM_BK, (it + 1) & 1);                    // passed the barrier at the end of the round before)
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();

        // S = Q K^T for the warp's 16 rows and the tile's 64 keys
        float s[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
        for (int d = 0; d < DQ; d += 16) {
            uint32_t a0, a1, a2, a3;
            ldsm_x4(a0, a1, a2, a3, Qs + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldq + d + (lane >> 4) * 8);
#pragma unroll
            for (int j = 0; j < 8; j += 2) {                        // two tiles of 8 keys a load
                uint32_t b0, b1, b2, b3;
                ldsm_x4(b0, b1, b2, b3, Ks + (j * 8 + (lane & 7) + (lane >> 4) * 8) * ldq + d + ((lane >> 3) & 1) * 8);
                mma_bf16(s[j], a0, a1, a2, a3, b0, b1);
                mma_bf16(s[j + 1], a0, a1, a2, a3, b2, b3);
            }
        }
        // scale, mask, running maximum and sum
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = kt + j * 8 + tq * 2 + (e & 1);
                const int row = e < 2 ? row0 : row1;
                const bool ok = key <= row && key < n && (window <= 0 || key > row - window);
                s[j][e] = ok ? s[j][e] * scale : -INFINITY;
            }
            mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
            mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float base0 = mn0 == -INFINITY ? 0.f : mn0, base1 = mn1 == -INFINITY ? 0.f : mn1;
        const float alpha0 = expf(m0 - base0), alpha1 = expf(m1 - base1);      // m = -inf gives 0
        float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            s[j][0] = expf(s[j][0] - base0); s[j][1] = expf(s[j][1] - base0);
            s[j][2] = expf(s[j][2] - base1); s[j][3] = expf(s[j][3] - base1);
            sum0 += s[j][0] + s[j][1];
            sum1 += s[j][2] + s[j][3];
        }
        sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1); sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
        sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1); sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
        l0 = l0 * alpha0 + sum0; l1 = l1 * alpha1 + sum1;
        m0 = mn0; m1 = mn1;
#pragma unroll
        for (int j = 0; j < NV; ++j) { o[j][0] *= alpha0; o[j][1] *= alpha0; o[j][2] *= alpha1; o[j][3] *= alpha1; }

        // O += P V, 16 keys a step
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            const uint32_t a0 = pack_bf16(s[2 * ks][0], s[2 * ks][1]), a1 = pack_bf16(s[2 * ks][2], s[2 * ks][3]);
            const uint32_t a2 = pack_bf16(s[2 * ks + 1][0], s[2 * ks + 1][1]), a3 = pack_bf16(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
            for (int j = 0; j < NV; j += 2) {
                if (j < nv_used) {                                  // DV / 8 may be odd: the second tile of a pair reads padding
                    uint32_t b0, b1, b2, b3;                        // or the next row's start, and its result is never stored
                    ldsm_x4_trans(b0, b1, b2, b3, Vs + (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldv + j * 8 + (lane >> 4) * 8);
                    mma_bf16(o[j], a0, a1, a2, a3, b0, b1);
                    if (j + 1 < NV) mma_bf16(o[j + 1], a0, a1, a2, a3, b2, b3);
                }
            }
        }
        __syncthreads();                                            // this buffer may be copied into again
    }

    if (sink) {                                                     // one more term in the denominator, with no value
        const float sk = sink[h];
        const float mn0 = fmaxf(m0, sk), mn1 = fmaxf(m1, sk);
        const float r0 = expf(m0 - mn0), r1 = expf(m1 - mn1);
        l0 = l0 * r0 + expf(sk - mn0); l1 = l1 * r1 + expf(sk - mn1);
#pragma unroll
        for (int j = 0; j < NV; ++j) { o[j][0] *= r0; o[j][1] *= r0; o[j][2] *= r1; o[j][3] *= r1; }
    }
    const float inv0 = 1.f / l0, inv1 = 1.f / l1;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        if (j < nv_used) {
            const int col = j * 8 + tq * 2;
            if (row0 < n) *reinterpret_cast<uint32_t*>(out + ((size_t)(t0 + row0) * H + h) * DV + col) = pack_bf16(o[j][0] * inv0, o[j][1] * inv0);
            if (row1 < n) *reinterpret_cast<uint32_t*>(out + ((size_t)(t0 + row1) * H + h) * DV + col) = pack_bf16(o[j][2] * inv1, o[j][3] * inv1);
        }
    }
}

extern "C" int qwb_latent_prefill_mma(const void* q, const void* k_plain, const void* kr, int ld_kr, const void* v,
                                      const int* cu_seqlens, const float* sink, void* out, int B, int max_new, int H, int K,
                                      int R, int DV, float scale, int window, cudaStream_t stream) {
    if (B <= 0 || max_new <= 0) return 0;
    if (H <= 0 || K <= 0 || R < 0 || DV <= 0 || K % 8 || R % 8 || DV % 8 || (K + R) % 16 || DV > 256 || ld_kr % 8)
        return qwb_fail(QWB_ERR_ARG, "latent_prefill_mma: heads %d of %d + %d and %d values: parts in multiples of 8, %d + %d a multiple "
                        "of 16, up to 256 values", H, K, R, DV, K, R);
    if (B > 65535 || H > 65535) return qwb_fail(QWB_ERR_ARG, "latent_prefill_mma: batch %d or heads %d are too many", B, H);
    for (const void* p : {q, k_plain, kr, v, (const void*)out})
        if ((uintptr_t)p % 16) return qwb_fail(QWB_ERR_ARG, "latent_prefill_mma: a tensor is not 16-byte aligned");
    const size_t smem = ((size_t)3 * LM_BQ * (K + R + LM_PAD) + (size_t)2 * LM_BK * (DV + LM_PAD)) * sizeof(bf16);
    if (smem > 220 * 1024) return qwb_fail(QWB_ERR_ARG, "latent_prefill_mma: %d + %d query values do not fit in shared memory", K, R);
    const dim3 grid((max_new + LM_BQ - 1) / LM_BQ, H, B);
#define QWB_LM(NV)                                                                                                              \
    do {                                                                                                                        \
        if (smem > 48 * 1024) {                                                                                                 \
            cudaError_t e = cudaFuncSetAttribute(latent_prefill_mma_kernel<NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return qwb_fail(QWB_ERR_CUDA, "latent_prefill_mma: %s", cudaGetErrorString(e));               \
        }                                                                                                                       \
        qwb_launch(latent_prefill_mma_kernel<NV>, grid, 128, smem, stream, (const bf16*)q, (const bf16*)k_plain, (const bf16*)kr, ld_kr, \
                   (const bf16*)v, cu_seqlens, sink, (bf16*)out, H, K, R, DV, scale, window);                                   \
    } while (0)
    if (DV <= 32) QWB_LM(4); else if (DV <= 64) QWB_LM(8); else if (DV <= 128) QWB_LM(16); else QWB_LM(32);
#undef QWB_LM
    return qwb_check_launch("latent_prefill_mma");
}
