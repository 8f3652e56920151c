// Latent attention: every head reads the same cached row per token, [latent c (L values) | rotated key part
// (R values)], and that row's first L values are the value too.  A query head brings its query already taken
// into the latent space (W_uk^T q, L values) and its rotated part (R values); the score is their dot product
// with the cached row, times a scale; the output is the weighted sum of latents, which the caller takes through
// W_uv.  Causal, with an optional window (key j is visible from position p when p - window < j <= p) and an
// optional sink per head: one more term exp(sink) in the softmax's denominator that has no value.
// Scores, maxima, sums and the accumulator are 32-bit; the queries come in 32-bit; the cache is float or bfloat16.
//
// Cache layout: pool [n_pages, page_size, L + R]; page_table [B, table_width].
#include "common.cuh"

// ---------------------------------------------------------------------------------
// Preparation, one block per token:
//   c = dkv[:L] / rms(dkv[:L]) * c_weight          -> cache row [:L]
//   rotated key part: pairs (2i, 2i + 1) of dkv[L:] -> cache row [L:]  (values beyond 2 * half pass unchanged)
//   q_rot[t, h, :] = the same rotation of q[t, h, K:]; q_plain[h, t, :] = q[t, h, :K] in the products' dtype
//   or, for the tensor-core prompt kernel (q_full given): q_full[t, h, :] = [q[t, h, :K] | rotated part] and
//   row_new[t, :] = the cache row again, token by token, both in the products' dtype
// cos, sin [T, half] already hold any factor on them.
// ---------------------------------------------------------------------------------
template <typename T>
__global__ void latent_prep_kernel(const float* __restrict__ q, const float* __restrict__ dkv, const float* __restrict__ c_weight,
                                   const float* __restrict__ cosv, const float* __restrict__ sinv, const int* __restrict__ tok_seq,
                                   const int* __restrict__ tok_pos, const int* __restrict__ page_table, T* __restrict__ pool,
                                   T* __restrict__ q_plain, float* __restrict__ q_rot, T* __restrict__ q_full, T* __restrict__ row_new,
                                   int n_tok, int H, int K, int R, int L,
                                   int half, float eps, int page_size, int table_width, int store) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float red[32];
    const int t = blockIdx.x;
    const float* drow = dkv + (size_t)t * (L + R);
    const float* cs = cosv + (size_t)t * half;
    const float* sn = sinv + (size_t)t * half;
    if (store || row_new) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < L; i += blockDim.x) ss += drow[i] * drow[i];
        const float scale = rsqrtf(block_sum(ss, red) / (float)L + eps);
        const int b = tok_seq[t], pos = tok_pos[t];
        T* dst = store ? pool + ((size_t)page_table[(size_t)b * table_width + pos / page_size] * page_size + pos % page_size) * (L + R) : nullptr;
        T* again = row_new ? row_new + (size_t)t * (L + R) : nullptr;
        for (int i = threadIdx.x; i < L; i += blockDim.x) {
            const T c = from_f32<T>(drow[i] * scale * c_weight[i]);
            if (dst) dst[i] = c;
            if (again) again[i] = c;
        }
        for (int i = threadIdx.x; i < R; i += blockDim.x) {
            float v = drow[L + i];
            if (i < 2 * half) {
                const float other = drow[L + (i ^ 1)], c = cs[i >> 1], s = sn[i >> 1];
                v = (i & 1) ? v * c + other * s : v * c - other * s;
            }
            if (dst) dst[L + i] = from_f32<T>(v);
            if (again) again[L + i] = from_f32<T>(v);
        }
    }
    const float* qrow = q + (size_t)t * H * (K + R);
    if (q_full) {
        for (int idx = threadIdx.x; idx < H * (K + R); idx += blockDim.x) {
            const int h = idx / (K + R), i = idx - h * (K + R) - K;       // i >= 0: the rotated part
            float v = qrow[idx];
            if (i >= 0 && i < 2 * half) {
                const float other = qrow[h * (K + R) + K + (i ^ 1)], c = cs[i >> 1], s = sn[i >> 1];
                v = (i & 1) ? v * c + other * s : v * c - other * s;
            }
            q_full[(size_t)t * H * (K + R) + idx] = from_f32<T>(v);
        }
        return;
    }
    for (int idx = threadIdx.x; idx < H * K; idx += blockDim.x) {
        const int h = idx / K, d = idx - h * K;
        q_plain[((size_t)h * n_tok + t) * K + d] = from_f32<T>(qrow[h * (K + R) + d]);
    }
    for (int idx = threadIdx.x; idx < H * R; idx += blockDim.x) {
        const int h = idx / R, i = idx - h * R;
        const float* src = qrow + h * (K + R) + K;
        float v = src[i];
        if (i < 2 * half) {
            const float other = src[i ^ 1], c = cs[i >> 1], s = sn[i >> 1];
            v = (i & 1) ? v * c + other * s : v * c - other * s;
        }
        q_rot[(size_t)t * H * R + idx] = v;
    }
}

extern "C" int qwb_latent_prep(const float* q, const float* dkv, const float* c_weight, const float* cosv, const float* sinv,
                               const int* tok_seq, const int* tok_pos, const int* page_table, void* pool, int dtype,
                               void* q_plain, float* q_rot, void* q_full, void* row_new, int T, int H, int K, int R, int L,
                               int half, float eps, int page_size, int table_width, int store, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || K <= 0 || R < 0 || L <= 0 || half < 0 || 2 * half > R)
        return qwb_fail(QWB_ERR_ARG, "latent_prep: %d heads of %d + %d, latent %d, %d rotated pairs", H, K, R, L, half);
    if (dtype == QWB_DT_F32)
        qwb_launch(latent_prep_kernel<float>, T, 128, 0, stream, q, dkv, c_weight, cosv, sinv, tok_seq, tok_pos, page_table,
                   (float*)pool, (float*)q_plain, q_rot, (float*)q_full, (float*)row_new, T, H, K, R, L, half, eps, page_size,
                   table_width, store);
    else if (dtype == QWB_DT_BF16)
        qwb_launch(latent_prep_kernel<bf16>, T, 128, 0, stream, q, dkv, c_weight, cosv, sinv, tok_seq, tok_pos, page_table,
                   (bf16*)pool, (bf16*)q_plain, q_rot, (bf16*)q_full, (bf16*)row_new, T, H, K, R, L, half, eps, page_size,
                   table_width, store);
    else
        return qwb_fail(QWB_ERR_ARG, "latent_prep: unknown dtype %d", dtype);
    return qwb_check_launch("latent_prep");
}

// ---------------------------------------------------------------------------------
// Attention.  A block takes 16 rows, a row being a (token, head) pair: HB = min(H, 16) heads of TQ = 16 / HB
// consecutive tokens of one sequence, so that the rows share the key tiles.  4 warps, 4 rows each; keys in tiles
// of 32, one key per lane.  Prompts and single tokens are the same code (a single token is a tile of one token).
// A single-token step of few sequences takes 4 rows a block instead (a row a warp): four times the blocks.
//   q_abs [H, T, L] float, q_rot [T, H, R] float;  out [H, T, L] in the cache's dtype
// ---------------------------------------------------------------------------------
template <typename T, int NC, int RPW>      // NC * 32 >= L; RPW rows a warp: 4, or 1 to spread a small step over more blocks
__global__ void latent_attn_kernel(const float* __restrict__ q_abs, const float* __restrict__ q_rot, const T* __restrict__ pool,
                                   const int* __restrict__ page_table, const int* __restrict__ cu_seqlens,
                                   const int* __restrict__ pos0, const float* __restrict__ sink, T* __restrict__ out, int n_tok,
                                   int H, int L, int R, int page_size, int table_width, float scale, int window,
                                   int run_keys, int max_runs, float* __restrict__ part_acc, float* __restrict__ part_ml) {
    pdl_wait();
    pdl_launch_dependents();
    constexpr int ROWS = 4 * RPW, BK = 32;
    const int dk = L + R;
    extern __shared__ float smem[];
    float* Qs = smem;                       // [ROWS][dk], scaled
    float* Ks = Qs + ROWS * dk;             // [BK][dk + 1]

    // run_keys > 0: a step of one token per sequence, the keys cut into runs of run_keys; blockIdx.x is the run, and the
    // block leaves its running maximum, sum and unnormalised accumulator for latent_combine_kernel
    const int HB = min(H, ROWS), TQ = run_keys > 0 ? 1 : ROWS / HB;
    const int b = blockIdx.z, h0 = blockIdx.y * HB, q0 = run_keys > 0 ? 0 : blockIdx.x * TQ;
    const int t0 = cu_seqlens[b], n_new = cu_seqlens[b + 1] - t0;
    if (q0 >= n_new) return;
    const int nq = min(TQ, n_new - q0), nh = min(HB, H - h0);
    const int p0 = pos0[b];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (L % 4 == 0 && R % 4 == 0 && (uintptr_t)q_abs % 16 == 0 && (uintptr_t)q_rot % 16 == 0) {      // four values a load
        const int pieces = dk / 4;
#pragma unroll 2
        for (int idx = threadIdx.x; idx < ROWS * pieces; idx += blockDim.x) {
            const int r = idx / pieces, d = (idx - r * pieces) * 4;
            const int qi = r / HB, hi = r - qi * HB;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (qi < nq && hi < nh) {
                const int t = t0 + q0 + qi, h = h0 + hi;
                v = *reinterpret_cast<const float4*>(d < L ? q_abs + ((size_t)h * n_tok + t) * L + d
                                                           : q_rot + ((size_t)t * H + h) * R + (d - L));
            }
            float* dst = Qs + r * dk + d;
            dst[0] = v.x * scale; dst[1] = v.y * scale; dst[2] = v.z * scale; dst[3] = v.w * scale;
        }
    } else {
        for (int idx = threadIdx.x; idx < ROWS * dk; idx += blockDim.x) {
            const int r = idx / dk, d = idx - r * dk;
            const int qi = r / HB, hi = r - qi * HB;
            float v = 0.f;
            if (qi < nq && hi < nh) {
                const int t = t0 + q0 + qi, h = h0 + hi;
                v = d < L ? q_abs[((size_t)h * n_tok + t) * L + d] : q_rot[((size_t)t * H + h) * R + (d - L)];
            }
            Qs[idx] = v * scale;
        }
    }

    float m[RPW], l[RPW], acc[RPW][NC];
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
        m[i] = -INFINITY; l[i] = 0.f;
#pragma unroll
        for (int c = 0; c < NC; ++c) acc[i][c] = 0.f;
    }
    int k_last = p0 + q0 + nq - 1;
    int k_first = window > 0 ? max(0, p0 + q0 - window + 1) : 0;
    if (run_keys > 0) {
        k_first = max(k_first, (int)blockIdx.x * run_keys);
        k_last = min(k_last, ((int)blockIdx.x + 1) * run_keys - 1);
        if (k_first > k_last || (int)blockIdx.x >= max_runs) return;         // no visible key in this run (whole block)
    }
    const int* pages = page_table + (size_t)b * table_width;

    for (int kt = (k_first / BK) * BK; kt <= k_last; kt += BK) {
        __syncthreads();
        constexpr int VEC = Vec16<T>::N;
        if (dk % VEC == 0 && (uintptr_t)pool % 16 == 0) {           // a cached row is whole 16-byte pieces: one load a piece
            const int pieces = dk / VEC;
#pragma unroll 2
            for (int idx = threadIdx.x; idx < BK * pieces; idx += blockDim.x) {
                const int j = idx / pieces, d = (idx - j * pieces) * VEC, key = kt + j;
                float vals[VEC];
                if (key <= k_last) {
                    const Vec16<T> piece = *reinterpret_cast<const Vec16<T>*>(
                        pool + ((size_t)pages[key / page_size] * page_size + key % page_size) * dk + d);
                    piece.get(vals);
                } else {
#pragma unroll
                    for (int e = 0; e < VEC; ++e) vals[e] = 0.f;
                }
#pragma unroll
                for (int e = 0; e < VEC; ++e) Ks[j * (dk + 1) + d + e] = vals[e];
            }
        } else {
            for (int idx = threadIdx.x; idx < BK * dk; idx += blockDim.x) {
                const int j = idx / dk, d = idx - j * dk, key = kt + j;
                float kv = 0.f;
                if (key <= k_last) kv = to_f32(pool[((size_t)pages[key / page_size] * page_size + key % page_size) * dk + d]);
                Ks[j * (dk + 1) + d] = kv;
            }
        }
        __syncthreads();
        float s[RPW];
#pragma unroll
        for (int i = 0; i < RPW; ++i) s[i] = 0.f;
        const float* krow = Ks + lane * (dk + 1);
        for (int d = 0; d < dk; ++d) {
            const float kd = krow[d];
#pragma unroll
            for (int i = 0; i < RPW; ++i) s[i] += Qs[(warp * RPW + i) * dk + d] * kd;
        }
        const int key = kt + lane;
        float p[RPW];
#pragma unroll
        for (int i = 0; i < RPW; ++i) {
            const int r = warp * RPW + i;
            const int qi = r / HB, hi = r - qi * HB;
            const int qp = p0 + q0 + qi;
            const bool ok = qi < nq && hi < nh && key <= qp && (window <= 0 || key > qp - window);
            const float si = ok ? s[i] : -INFINITY;
            const float m_new = fmaxf(m[i], warp_max(si));
            if (m_new == -INFINITY) { p[i] = 0.f; continue; }
            const float alpha = expf(m[i] - m_new);
            p[i] = ok ? expf(si - m_new) : 0.f;
            l[i] = l[i] * alpha + warp_sum(p[i]);
            m[i] = m_new;
#pragma unroll
            for (int c = 0; c < NC; ++c) acc[i][c] *= alpha;
        }
        for (int j = 0; j < BK; ++j) {
            float pj[RPW];
#pragma unroll
            for (int i = 0; i < RPW; ++i) pj[i] = __shfl_sync(0xffffffffu, p[i], j);
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                const int d = lane + 32 * c;
                if (d < L) {
                    const float v = Ks[j * (dk + 1) + d];
#pragma unroll
                    for (int i = 0; i < RPW; ++i) acc[i][c] += pj[i] * v;
                }
            }
        }
    }

#pragma unroll
    for (int i = 0; i < RPW; ++i) {
        const int r = warp * RPW + i;
        const int qi = r / HB, hi = r - qi * HB;
        if (qi >= nq || hi >= nh) continue;
        const int h = h0 + hi;
        if (run_keys > 0) {
            const size_t at = ((size_t)b * H + h) * max_runs + blockIdx.x;
            if (lane == 0) { part_ml[2 * at] = m[i]; part_ml[2 * at + 1] = l[i]; }
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                const int d = lane + 32 * c;
                if (d < L) part_acc[at * L + d] = acc[i][c];
            }
            continue;
        }
        float mi = m[i], li = l[i], rescale = 1.f;
        if (sink) {                                             // one more term in the denominator, with no value
            const float sk = sink[h];
            const float m_new = fmaxf(mi, sk);
            rescale = expf(mi - m_new);
            li = li * rescale + expf(sk - m_new);
        }
        const float inv = rescale / li;
        T* o = out + ((size_t)h * n_tok + t0 + q0 + qi) * L;
#pragma unroll
        for (int c = 0; c < NC; ++c) {
            const int d = lane + 32 * c;
            if (d < L) o[d] = from_f32<T>(acc[i][c] * inv);
        }
    }
}

#define QWB_LATENT_MAX_L 512
#define QWB_LATENT_MAX_ROW 1024

// The runs of one (sequence, head) merged: out = sum_r acc_r e^(m_r - M) / (sum_r l_r e^(m_r - M) + e^(sink - M)),
// M = max(m_r, sink), over the runs that hold a visible key, in their order.  grid (H, B).
template <typename T>
__global__ void latent_combine_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                      const int* __restrict__ pos0, const float* __restrict__ sink, T* __restrict__ out,
                                      int n_tok, int H, int L, int window, int run_keys, int max_runs) {
    pdl_wait();
    pdl_launch_dependents();
    const int h = blockIdx.x, b = blockIdx.y;
    const int len = pos0[b] + 1;
    const int k_lo = window > 0 ? max(0, len - window) : 0;
    const int r0 = k_lo / run_keys, r1 = min((len - 1) / run_keys, max_runs - 1);
    const size_t base = ((size_t)b * H + h) * max_runs;
    float M = sink ? sink[h] : -INFINITY;
    for (int r = r0; r <= r1; ++r) M = fmaxf(M, part_ml[2 * (base + r)]);
    float denom = sink ? expf(sink[h] - M) : 0.f;
    for (int r = r0; r <= r1; ++r) denom += part_ml[2 * (base + r) + 1] * expf(part_ml[2 * (base + r)] - M);
    const float inv = 1.f / denom;
    __shared__ float wts[128];                                      // the runs' factors e^(m_r - M), 128 runs at a time
    float v[QWB_LATENT_MAX_L / 128];
#pragma unroll
    for (int i = 0; i < QWB_LATENT_MAX_L / 128; ++i) v[i] = 0.f;
    for (int first = r0; first <= r1; first += 128) {
        const int count = min(128, r1 - first + 1);
        __syncthreads();
        if ((int)threadIdx.x < count) wts[threadIdx.x] = expf(part_ml[2 * (base + first + threadIdx.x)] - M);
        __syncthreads();
#pragma unroll
        for (int i = 0; i < QWB_LATENT_MAX_L / 128; ++i) {
            const int d = threadIdx.x + i * 128;
            if (d < L)
                for (int r = 0; r < count; ++r) v[i] += part_acc[(base + first + r) * L + d] * wts[r];
        }
    }
#pragma unroll
    for (int i = 0; i < QWB_LATENT_MAX_L / 128; ++i) {
        const int d = threadIdx.x + i * 128;
        if (d < L) out[((size_t)h * n_tok + b) * L + d] = from_f32<T>(v[i] * inv);
    }
}

#define QWB_LATENT_RUN_KEYS 64

template <typename T>
static int launch_latent_attn(const float* q_abs, const float* q_rot, const void* pool, const int* page_table,
                              const int* cu_seqlens, const int* pos0, const float* sink, void* out, int B, int n_tok,
                              int max_new, int H, int L, int R, int page_size, int table_width, float scale, int window,
                              int max_runs, float* part_acc, float* part_ml, cudaStream_t stream) {
    const int dk = L + R;
    const int run_keys = max_runs > 0 ? QWB_LATENT_RUN_KEYS : 0;
    // few blocks (a single-token step of few sequences): a row a warp, so that four times as many blocks share the work
    const bool narrow = max_runs > 0 && (long long)B * max_runs * ((H + 15) / 16) < 120;
    const int rows = narrow ? 4 : 16;
    const size_t smem = ((size_t)rows * dk + 32 * (dk + 1)) * sizeof(float);
    const int HB = H < rows ? H : rows, TQ = rows / HB;
    dim3 grid(max_runs > 0 ? max_runs : (max_new + TQ - 1) / TQ, (H + HB - 1) / HB, B);
    const int nc = (L + 31) / 32;
#define QWB_LAUNCH_LATENT1(NC, RPW)                                                                                    \
    do {                                                                                                               \
        if (smem > 48 * 1024) {                                                                                        \
            cudaError_t e = cudaFuncSetAttribute(latent_attn_kernel<T, NC, RPW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return qwb_fail(QWB_ERR_CUDA, "latent_attn: %s", cudaGetErrorString(e));             \
        }                                                                                                              \
        qwb_launch(latent_attn_kernel<T, NC, RPW>, grid, 128, smem, stream, q_abs, q_rot, (const T*)pool, page_table,  \
                   cu_seqlens, pos0, sink, (T*)out, n_tok, H, L, R, page_size, table_width, scale, window, run_keys,   \
                   max_runs, part_acc, part_ml);                                                                      \
    } while (0)
#define QWB_LAUNCH_LATENT(NC) do { if (narrow) QWB_LAUNCH_LATENT1(NC, 1); else QWB_LAUNCH_LATENT1(NC, 4); } while (0)
    if (nc <= 2) QWB_LAUNCH_LATENT(2);
    else if (nc <= 4) QWB_LAUNCH_LATENT(4);
    else if (nc <= 8) QWB_LAUNCH_LATENT(8);
    else QWB_LAUNCH_LATENT(16);
#undef QWB_LAUNCH_LATENT1
#undef QWB_LAUNCH_LATENT
    if (int rc = qwb_check_launch("latent_attn")) return rc;
    if (max_runs > 0) {
        qwb_launch(latent_combine_kernel<T>, dim3(H, B), 128, 0, stream, (const float*)part_acc, (const float*)part_ml, pos0, sink,
                   (T*)out, n_tok, H, L, window, run_keys, max_runs);
        return qwb_check_launch("latent_combine");
    }
    return 0;
}


// max_runs > 0: every sequence brings one token (n_tok = B) and no sequence holds more than max_runs * 64 keys after the
// step; the keys are cut into runs of 64 (by the key's index, whatever else is in the batch), a block a run, and merged.
// scratch: max_runs * B * H * (L + 2) floats.
extern "C" int qwb_latent_run_keys() { return QWB_LATENT_RUN_KEYS; }

extern "C" int qwb_latent_attn(const float* q_abs, const float* q_rot, const void* pool, const int* page_table,
                               const int* cu_seqlens, const int* pos0, const float* sink, void* out, int dtype, int B,
                               int n_tok, int max_new, int H, int L, int R, int page_size, int table_width, float scale,
                               int window, int max_runs, float* scratch, cudaStream_t stream) {
    if (B <= 0 || n_tok <= 0 || max_new <= 0) return 0;
    if (H <= 0 || L <= 0 || R < 0 || L > QWB_LATENT_MAX_L || L + R > QWB_LATENT_MAX_ROW)
        return qwb_fail(QWB_ERR_ARG, "latent_attn: %d heads, latent %d (up to %d) + rotated %d (row up to %d)", H, L, QWB_LATENT_MAX_L, R, QWB_LATENT_MAX_ROW);
    if (page_size <= 0 || table_width <= 0) return qwb_fail(QWB_ERR_ARG, "latent_attn: bad page size %d or table width %d", page_size, table_width);
    if (B > 65535 || H > 65535) return qwb_fail(QWB_ERR_ARG, "latent_attn: batch %d or heads %d are too many", B, H);
    if (max_runs > 0 && (max_new != 1 || n_tok != B || !scratch))
        return qwb_fail(QWB_ERR_ARG, "latent_attn: runs of keys are for steps of one token per sequence, with scratch memory");
    float* part_acc = scratch;
    float* part_ml = max_runs > 0 ? scratch + (size_t)max_runs * B * H * L : nullptr;
    if (dtype == QWB_DT_F32)
        return launch_latent_attn<float>(q_abs, q_rot, pool, page_table, cu_seqlens, pos0, sink, out, B, n_tok, max_new, H, L, R,
                                         page_size, table_width, scale, window, max_runs, part_acc, part_ml, stream);
    if (dtype == QWB_DT_BF16)
        return launch_latent_attn<bf16>(q_abs, q_rot, pool, page_table, cu_seqlens, pos0, sink, out, B, n_tok, max_new, H, L, R,
                                        page_size, table_width, scale, window, max_runs, part_acc, part_ml, stream);
    return qwb_fail(QWB_ERR_ARG, "latent_attn: unknown dtype %d", dtype);
}
