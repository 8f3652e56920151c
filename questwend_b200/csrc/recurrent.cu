// Recurrent mixers: a short causal convolution over time with a tail kept per sequence, the state-space
// recurrence of Mamba-2 and the gated delta rule with one decay per key channel, and the gated norms that
// follow them.  Everything here is 32-bit: inputs are the 32-bit results of the projections, the states are
// float, and so are decays, step sizes, gates and unit norms.
//
// A step brings T packed tokens of B sequences (cu_seqlens [B + 1]); sequence b's state lives in row
// slots[b] of the state tensors.  One token per sequence (a decode step) is the same code with one token.
#include "common.cuh"

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }

#define QWB_CONV_MAX_TAPS 8

// ---------------------------------------------------------------------------------
// out[t, c] = act( bias[c] + sum_j w[c, j] * in(i - (taps - 1 - j), c) ),  i = the token's index in this step,
// in(i < 0) = the tail: tail[slot, taps - 1 + i, c] (the last taps - 1 inputs of the sequence before this step,
// zero for a new sequence).  x [T, ld] is read at column c (the caller offsets the pointer), out is [T, C].
// ---------------------------------------------------------------------------------
__global__ void short_conv_kernel(const float* __restrict__ x, int ld, const float* __restrict__ w, const float* __restrict__ bias,
                                  const float* tail, const int* __restrict__ tok_seq, const int* __restrict__ cu_seqlens,
                                  const int* __restrict__ slots, float* __restrict__ out, int T, int C, int taps, int act) {
    pdl_wait();
    pdl_launch_dependents();
    const int c = blockIdx.y * blockDim.x + threadIdx.x, t = blockIdx.x;
    if (c >= C || t >= T) return;
    const int b = tok_seq[t];
    const int i = t - cu_seqlens[b];
    float acc = bias ? bias[c] : 0.f;
    const float* tl = tail + (size_t)slots[b] * (taps - 1) * C;
    for (int j = 0; j < taps; ++j) {
        const int src = i - (taps - 1 - j);
        const float v = src >= 0 ? x[(size_t)(t - (taps - 1 - j)) * ld + c] : tl[(size_t)(taps - 1 + src) * C + c];
        acc += w[c * taps + j] * v;
    }
    out[(size_t)t * C + c] = act ? silu_f(acc) : acc;
}

// The tail after the step: the last taps - 1 inputs of each sequence (new ones, then what is left of the old tail).
__global__ void conv_tail_kernel(const float* __restrict__ x, int ld, float* tail, const int* __restrict__ cu_seqlens,
                                 const int* __restrict__ slots, int B, int C, int taps) {
    pdl_wait();
    pdl_launch_dependents();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, b = blockIdx.y;
    if (c >= C || b >= B) return;
    const int t0 = cu_seqlens[b], n_new = cu_seqlens[b + 1] - t0;
    float* tl = tail + (size_t)slots[b] * (taps - 1) * C;
    float keep[QWB_CONV_MAX_TAPS];
    for (int r = 0; r < taps - 1; ++r) {
        const int idx = n_new - (taps - 1) + r;
        keep[r] = idx >= 0 ? x[(size_t)(t0 + idx) * ld + c] : tl[(size_t)(r + n_new) * C + c];
    }
    for (int r = 0; r < taps - 1; ++r) tl[(size_t)r * C + c] = keep[r];
}

extern "C" int qwb_short_conv(const float* x, int ld, const float* w, const float* bias, float* tail, const int* tok_seq,
                              const int* cu_seqlens, const int* slots, float* out, int T, int B, int C, int taps, int act,
                              int update_tail, cudaStream_t stream) {
    if (T <= 0 || B <= 0) return 0;
    if (C <= 0 || taps < 1 || taps > QWB_CONV_MAX_TAPS || ld < C)
        return qwb_fail(QWB_ERR_ARG, "short_conv: %d channels, %d taps (1 to %d), row stride %d", C, taps, QWB_CONV_MAX_TAPS, ld);
    if (B > 65535 || C > 65535 * 128) return qwb_fail(QWB_ERR_ARG, "short_conv: %d sequences or %d channels are too many", B, C);
    const int block = C >= 256 ? 256 : 128;
    qwb_launch(short_conv_kernel, dim3(T, (C + block - 1) / block), block, 0, stream, x, ld, w, bias, (const float*)tail, tok_seq, cu_seqlens, slots, out, T, C, taps, act);
    if (int rc = qwb_check_launch("short_conv")) return rc;
    if (update_tail && taps > 1) {
        qwb_launch(conv_tail_kernel, dim3((C + block - 1) / block, B), block, 0, stream, x, ld, tail, cu_seqlens, slots, B, C, taps);
        return qwb_check_launch("conv_tail");
    }
    return 0;
}

// ---------------------------------------------------------------------------------
// Mamba-2 recurrence.  Per head h (group g = h / (H / G)), per token:
//     dt = softplus(dt_raw + dt_bias[h]);  S = exp(-exp(A_log[h]) dt) S + dt B x^T;  y = S^T C + D[h] x
// S is N x P (state x value size).  One block per (head, sequence); thread (part, p) keeps PER rows of column p
// of S in registers: rows part * PER .. part * PER + PER - 1.  The parts' sums meet in shared memory.
//   xbc [T, ldx] float: x [H * P] | B [G * N] | C [G * N] (after convolution and SiLU)
//   dt_raw: column h of a [T, ld_dt] matrix;  state [slots, H, N, P];  y [T, H * P]
// ---------------------------------------------------------------------------------
template <int PER>
__global__ void ssm_scan_kernel(const float* __restrict__ xbc, int ldx, const float* __restrict__ dt_raw, int ld_dt,
                                const float* __restrict__ dt_bias, const float* __restrict__ A_log, const float* __restrict__ Dskip,
                                float* state, const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
                                float* __restrict__ y, int H, int P, int N, int G, int write_state) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ float red[];                      // [2][parts][P]
    const int h = blockIdx.x, b = blockIdx.y;
    const int parts = (N + PER - 1) / PER;
    const int p = threadIdx.x % P, part = threadIdx.x / P;
    const int g = h / (H / G);
    const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
    const int n0 = part * PER;
    float* S = state + (((size_t)slots[b] * H + h) * N) * P;
    float s[PER];
#pragma unroll
    for (int k = 0; k < PER; ++k) s[k] = n0 + k < N ? S[(size_t)(n0 + k) * P + p] : 0.f;
    const float a = -expf(A_log[h]), dskip = Dskip[h], bias = dt_bias[h];
    const int inner = H * P;
    int buf = 0;
    for (int t = t0; t < t1; ++t) {
        const float* row = xbc + (size_t)t * ldx;
        const float dt = softplus_f(dt_raw[(size_t)t * ld_dt + h] + bias);
        const float decay = expf(a * dt);
        const float xv = row[h * P + p];
        const float dtx = dt * xv;
        const float* Bt = row + inner + g * N + n0;
        const float* Ct = Bt + G * N;
        float acc = 0.f;
#pragma unroll
        for (int k = 0; k < PER; ++k) {
            if (n0 + k < N) {
                s[k] = decay * s[k] + dtx * Bt[k];
                acc += s[k] * Ct[k];
            }
        }
        red[(buf * parts + part) * P + p] = acc;
        __syncthreads();
        if (part == 0) {
            float total = 0.f;
            for (int q = 0; q < parts; ++q) total += red[(buf * parts + q) * P + p];
            y[(size_t)t * inner + h * P + p] = total + dskip * xv;
        }
        buf ^= 1;
    }
    if (write_state) {
#pragma unroll
        for (int k = 0; k < PER; ++k)
            if (n0 + k < N) S[(size_t)(n0 + k) * P + p] = s[k];
    }
}

static int scan_rows_per_thread(int rows, int cols) {      // 16, 32 or 64 rows of the state per thread; 0: too large
    for (int per = 16; per <= 64; per *= 2)
        if ((size_t)cols * ((rows + per - 1) / per) <= 1024) return per;
    return 0;
}

extern "C" int qwb_ssm_scan(const float* xbc, int ldx, const float* dt_raw, int ld_dt, const float* dt_bias, const float* A_log,
                            const float* Dskip, float* state, const int* cu_seqlens, const int* slots, float* y, int B,
                            int H, int P, int N, int G, int write_state, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (H <= 0 || P <= 0 || N <= 0 || G <= 0 || H % G) return qwb_fail(QWB_ERR_ARG, "ssm_scan: %d heads, %d groups, state %d x %d", H, G, N, P);
    const int per = scan_rows_per_thread(N, P);
    if (!per) return qwb_fail(QWB_ERR_ARG, "ssm_scan: a state of %d x %d per head is too large (value size x ceil(state / 64) <= 1024)", N, P);
    if (B > 65535) return qwb_fail(QWB_ERR_ARG, "ssm_scan: %d sequences are too many", B);
    const int parts = (N + per - 1) / per;
    const size_t smem = (size_t)2 * parts * P * sizeof(float);
    const dim3 grid(H, B);
#define QWB_SSM(PER) qwb_launch(ssm_scan_kernel<PER>, grid, P * parts, smem, stream, xbc, ldx, dt_raw, ld_dt, dt_bias, A_log, Dskip, state, cu_seqlens, slots, y, H, P, N, G, write_state)
    if (per == 16) QWB_SSM(16); else if (per == 32) QWB_SSM(32); else QWB_SSM(64);
#undef QWB_SSM
    return qwb_check_launch("ssm_scan");
}

// ---------------------------------------------------------------------------------
// Gated delta rule, one decay per head and key channel.
// Preparation, one block per token: q and k (after convolution and SiLU) become unit vectors per head,
// x / sqrt(sum x^2 + unit_eps), q times q_scale; kq = k . q; beta = sigmoid(b_raw); decay[h, n] =
// exp(-exp(A_log[h]) softplus(a_raw[h, n] + dt_bias[h, n])).  b_raw: H columns of a matrix with rows of ld_b values.
//   qkv [T, ld]: q [Hk * K] | k [Hk * K] | v [H * P], q and k normalised in place
// ---------------------------------------------------------------------------------
__global__ void delta_prep_kernel(float* qkv, int ld, float* __restrict__ kq, const float* __restrict__ b_raw, int ld_b, float* __restrict__ beta,
                                  const float* __restrict__ a_raw, const float* __restrict__ dt_bias, const float* __restrict__ A_log,
                                  float* __restrict__ decay, int H, int Hk, int K, float unit_eps, float q_scale) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
    float* row = qkv + (size_t)t * ld;
    for (int kh = warp; kh < Hk; kh += nwarp) {
        float* q = row + kh * K;
        float* k = row + (Hk + kh) * K;
        float sq = 0.f, sk = 0.f;
        for (int i = lane; i < K; i += 32) { sq += q[i] * q[i]; sk += k[i] * k[i]; }
        sq = warp_sum(sq); sk = warp_sum(sk);
        const float rq = q_scale / sqrtf(sq + unit_eps), rk = 1.f / sqrtf(sk + unit_eps);
        float dot = 0.f;
        for (int i = lane; i < K; i += 32) {
            const float qn = q[i] * rq, kn = k[i] * rk;
            q[i] = qn; k[i] = kn;
            dot += qn * kn;
        }
        dot = warp_sum(dot);
        if (lane == 0) kq[(size_t)t * Hk + kh] = dot;
    }
    for (int i = threadIdx.x; i < H; i += blockDim.x) beta[(size_t)t * H + i] = sigmoid_f(b_raw[(size_t)t * ld_b + i]);
    for (int i = threadIdx.x; i < H * K; i += blockDim.x)
        decay[(size_t)t * H * K + i] = expf(-expf(A_log[i / K]) * softplus_f(a_raw[(size_t)t * H * K + i] + dt_bias[i]));
}

extern "C" int qwb_delta_prep(float* qkv, int ld, float* kq, const float* b_raw, int ld_b, float* beta, const float* a_raw,
                              const float* dt_bias, const float* A_log, float* decay, int T, int H, int Hk, int K,
                              float unit_eps, float q_scale, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || Hk <= 0 || K <= 0 || H % Hk) return qwb_fail(QWB_ERR_ARG, "delta_prep: %d heads, %d key heads of %d", H, Hk, K);
    qwb_launch(delta_prep_kernel, T, 128, 0, stream, qkv, ld, kq, b_raw, ld_b, beta, a_raw, dt_bias, A_log, decay, H, Hk, K, unit_eps, q_scale);
    return qwb_check_launch("delta_prep");
}

// The recurrence, per head h (key head kh = h / (H / Hk)), per token, S is K x P:
//     S = decay[:, None] * S;  u = beta (v - S^T k);  S = S + k u^T;  o = S^T q
// o is formed as (decayed S)^T q + u (k . q), so that one meeting of the parts' sums per token is enough.
// Threads as in ssm_scan_kernel: (part, p) keeps PER rows of column p.
template <int PER>
__global__ void delta_scan_kernel(const float* __restrict__ qkv, int ld, const float* __restrict__ kq, const float* __restrict__ beta,
                                  const float* __restrict__ decay, float* state, const int* __restrict__ cu_seqlens,
                                  const int* __restrict__ slots, float* __restrict__ o, int H, int Hk, int K, int P, int write_state) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ float red[];                      // [2][2][parts][P]
    const int h = blockIdx.x, b = blockIdx.y;
    const int parts = (K + PER - 1) / PER;
    const int p = threadIdx.x % P, part = threadIdx.x / P;
    const int kh = h / (H / Hk);
    const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
    const int n0 = part * PER;
    float* S = state + (((size_t)slots[b] * H + h) * K) * P;
    float s[PER];
#pragma unroll
    for (int k = 0; k < PER; ++k) s[k] = n0 + k < K ? S[(size_t)(n0 + k) * P + p] : 0.f;
    int buf = 0;
    for (int t = t0; t < t1; ++t) {
        const float* row = qkv + (size_t)t * ld;
        const float* qt = row + kh * K + n0;
        const float* kt = row + (Hk + kh) * K + n0;
        const float* gt = decay + ((size_t)t * H + h) * K + n0;
        const float v = row[2 * Hk * K + h * P + p];
        float kk[PER];
        float sk = 0.f, sq = 0.f;
#pragma unroll
        for (int k = 0; k < PER; ++k) {
            if (n0 + k < K) {
                kk[k] = kt[k];
                s[k] *= gt[k];
                sk += s[k] * kk[k];
                sq += s[k] * qt[k];
            }
        }
        float* r = red + (size_t)buf * 2 * parts * P;
        r[part * P + p] = sk;
        r[(parts + part) * P + p] = sq;
        __syncthreads();
        float tk = 0.f;
        for (int q = 0; q < parts; ++q) tk += r[q * P + p];
        const float u = beta[(size_t)t * H + h] * (v - tk);
#pragma unroll
        for (int k = 0; k < PER; ++k)
            if (n0 + k < K) s[k] += kk[k] * u;
        if (part == 0) {
            float tq = 0.f;
            for (int q = 0; q < parts; ++q) tq += r[(parts + q) * P + p];
            o[((size_t)t * H + h) * P + p] = tq + u * kq[(size_t)t * Hk + kh];
        }
        buf ^= 1;
    }
    if (write_state) {
#pragma unroll
        for (int k = 0; k < PER; ++k)
            if (n0 + k < K) S[(size_t)(n0 + k) * P + p] = s[k];
    }
}

extern "C" int qwb_delta_scan(const float* qkv, int ld, const float* kq, const float* beta, const float* decay, float* state,
                              const int* cu_seqlens, const int* slots, float* o, int B, int H, int Hk, int K, int P,
                              int write_state, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (H <= 0 || Hk <= 0 || K <= 0 || P <= 0 || H % Hk) return qwb_fail(QWB_ERR_ARG, "delta_scan: %d heads, %d key heads, state %d x %d", H, Hk, K, P);
    const int per = scan_rows_per_thread(K, P);
    if (!per) return qwb_fail(QWB_ERR_ARG, "delta_scan: a state of %d x %d per head is too large (value size x ceil(key size / 64) <= 1024)", K, P);
    if (B > 65535) return qwb_fail(QWB_ERR_ARG, "delta_scan: %d sequences are too many", B);
    const int parts = (K + per - 1) / per;
    const size_t smem = (size_t)4 * parts * P * sizeof(float);
    const dim3 grid(H, B);
#define QWB_DELTA(PER) qwb_launch(delta_scan_kernel<PER>, grid, P * parts, smem, stream, qkv, ld, kq, beta, decay, state, cu_seqlens, slots, o, H, Hk, K, P, write_state)
    if (per == 16) QWB_DELTA(16); else if (per == 32) QWB_DELTA(32); else QWB_DELTA(64);
#undef QWB_DELTA
    return qwb_check_launch("delta_scan");
}

// ---------------------------------------------------------------------------------
// Gated norm over equal parts of a row.  y [T, n_parts * part] float, gate: column slice of a [T, ld_gate] matrix.
//   mode 0: v = y * silu(gate); out = v / rms(v over the part) * w      (the gate before the norm)
//   mode 1: out = y / rms(y over the part) * w * sigmoid(gate)          (the gate after the norm)
// w has w_len entries and is indexed by column % w_len (the whole row, or one part shared by all parts).
// One warp per (token, part).
// ---------------------------------------------------------------------------------
template <typename TOut>
__global__ void gated_part_norm_kernel(const float* __restrict__ y, const float* __restrict__ gate, int ld_gate,
                                       const float* __restrict__ w, int w_len, TOut* __restrict__ out, int T, int n_parts,
                                       int part, float eps, int mode) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= (long long)T * n_parts) return;
    const int t = (int)(unit / n_parts), g = (int)(unit % n_parts);
    const int D = n_parts * part;
    const float* yr = y + (size_t)t * D + g * part;
    const float* gr = gate + (size_t)t * ld_gate + g * part;
    float ss = 0.f;
    for (int i = lane; i < part; i += 32) {
        const float v = mode == 0 ? yr[i] * silu_f(gr[i]) : yr[i];
        ss += v * v;
    }
    const float scale = rsqrtf(warp_sum(ss) / (float)part + eps);
    TOut* orow = out + (size_t)t * D + g * part;
    for (int i = lane; i < part; i += 32) {
        const float wi = w[(g * part + i) % w_len];
        const float v = mode == 0 ? yr[i] * silu_f(gr[i]) * scale * wi : yr[i] * scale * wi * sigmoid_f(gr[i]);
        orow[i] = from_f32<TOut>(v);
    }
}

extern "C" int qwb_gated_part_norm(const float* y, const float* gate, int ld_gate, const float* w, int w_len, void* out,
                                   int out_dtype, int T, int n_parts, int part, float eps, int mode, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (n_parts <= 0 || part <= 0 || w_len <= 0 || (mode != 0 && mode != 1))
        return qwb_fail(QWB_ERR_ARG, "gated_part_norm: %d parts of %d, weight of %d, mode %d", n_parts, part, w_len, mode);
    const long long units = (long long)T * n_parts;
    const unsigned blocks = (unsigned)((units + 3) / 4);
    if (out_dtype == QWB_DT_F32)
        qwb_launch(gated_part_norm_kernel<float>, blocks, 128, 0, stream, y, gate, ld_gate, w, w_len, (float*)out, T, n_parts, part, eps, mode);
    else if (out_dtype == QWB_DT_BF16)
        qwb_launch(gated_part_norm_kernel<bf16>, blocks, 128, 0, stream, y, gate, ld_gate, w, w_len, (bf16*)out, T, n_parts, part, eps, mode);
    else
        return qwb_fail(QWB_ERR_ARG, "gated_part_norm: unknown dtype %d", out_dtype);
    return qwb_check_launch("gated_part_norm");
}
