// The real-gated linear recurrent unit: per channel c, with gates r and i in (0, 1),
//
//   log a_t = -sharpness * r_t * softplus(lam_c),   S_t = a_t S_(t-1) + sqrt(1 - a_t^2) * i_t * u_t,
//
// from S = 0 at a sequence's start (the first token is no special case), the state S kept per sequence in 32-bit.
// The gates come from the recurrence's own input u through block-diagonal matrices: the channels are cut into equal
// blocks and block b of r is sigmoid(Wa[b] u_b + ba[b]), the same for i with Wi, bi.  Everything here is 32-bit: u is the
// 32-bit result of the convolution, the gate matrices are read in the engine's dtype and multiplied in float, and so are
// the logarithm of the decay, the exponential and the root (1 - a^2 is formed as -expm1(2 log a), which keeps its
// digits when a is close to 1).  The read-out multiplies S by a second branch, gelu(y + bias) (tanh form), and is written in the
// dtype of the product that follows.
//
//   block_gates      r and i for all tokens of a step: a tiled float product per (64 tokens, 64 outputs of one block), or,
//                    for up to 16 tokens, a warp per output channel that streams its row of the matrix
//   rglru_scan       one thread per (sequence, channel) walks the sequence's tokens in order
//   rglru_chunk_*    the same for long prompts in three passes: per chunk of tokens the product of its decays and its
//                    sum from a zero state; the chunks' carries in order; the chunks again from their carries
#include "common.cuh"

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float gelu_tanh_f(float v) { return 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v))); }

// ---------------------------------------------------------------------------------
// gates: grid (ceil(T / 64), blocks * ceil(n / 64), 2); z = 0: r from Wa, z = 1: i from Wi.  256 threads; thread (ty, tx)
// holds tokens 4 ty .. 4 ty + 3 and outputs tx, tx + 16, tx + 32, tx + 48 of the tile (neighbouring lanes read neighbouring
// rows of the weight tile: no bank conflicts); k goes in steps of 32 through shared memory.
// ---------------------------------------------------------------------------------
#define QWB_GATE_TILE_TOKENS 64
template <typename TW>
__global__ void __launch_bounds__(256)
block_gates_kernel(const float* __restrict__ u, const TW* __restrict__ wa, const float* __restrict__ ba, const TW* __restrict__ wi,
                   const float* __restrict__ bi, float* __restrict__ r_out, float* __restrict__ i_out, int T, int C, int n) {
    pdl_wait();
    pdl_launch_dependents();
    constexpr int TT = QWB_GATE_TILE_TOKENS;
    __shared__ float Us[TT][33];
    __shared__ float Ws[64][33];
    const int tiles = (n + 63) / 64;
    const int blk = blockIdx.y / tiles, o0 = (blockIdx.y % tiles) * 64, t0 = blockIdx.x * TT;
    const TW* W = (blockIdx.z ? wi : wa) + (size_t)blk * n * n;
    const float* bias = (blockIdx.z ? bi : ba) + (size_t)blk * n;
    float* out = blockIdx.z ? i_out : r_out;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < n; k0 += 32) {
        __syncthreads();
        for (int idx = tid; idx < TT * 32; idx += 256) {
            const int tt = idx >> 5, kk = idx & 31;
            Us[tt][kk] = (t0 + tt < T && k0 + kk < n) ? u[(size_t)(t0 + tt) * C + blk * n + k0 + kk] : 0.f;
        }
        for (int idx = tid; idx < 64 * 32; idx += 256) {
            const int oo = idx >> 5, kk = idx & 31;
            Ws[oo][kk] = (o0 + oo < n && k0 + kk < n) ? to_f32(W[(size_t)(o0 + oo) * n + k0 + kk]) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < 32; ++kk) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { a[i] = Us[4 * ty + i][kk]; w[i] = Ws[tx + 16 * i][kk]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] += a[i] * w[j];
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int t = t0 + 4 * ty + i;
        if (t >= T) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int o = o0 + tx + 16 * j;
            if (o < n) out[(size_t)t * C + blk * n + o] = sigmoid_f(acc[i][j] + bias[o]);
        }
    }
}

// A step of a few tokens (up to 16 rows: decode steps): a block takes 8 output channels of one gate block, a warp each.
// The tokens' inputs of that gate block pass through shared memory once per block (512 values of k at a time); a warp
// streams its channel's row of the gate's matrix once, the lanes stride over k, and the tokens' sums are reduced over the
// warp in a fixed order.  grid (blocks * ceil(n / 8), 2), 8 warps.
#define QWB_GATE_ROWS 16
#define QWB_GATE_ROWS_K 512
template <typename TW>
__global__ void __launch_bounds__(256)
block_gates_rows_kernel(const float* __restrict__ u, const TW* __restrict__ wa, const float* __restrict__ ba, const TW* __restrict__ wi,
                        const float* __restrict__ bi, float* __restrict__ r_out, float* __restrict__ i_out, int T, int C, int n) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float us[QWB_GATE_ROWS][QWB_GATE_ROWS_K];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int groups = (n + 7) / 8;
    const int blk = blockIdx.x / groups, o = (blockIdx.x % groups) * 8 + warp;
    const TW* W = (blockIdx.y ? wi : wa) + ((size_t)blk * n + min(o, n - 1)) * n;
    const float* ub = u + (size_t)blk * n;
    float acc[QWB_GATE_ROWS];
#pragma unroll
    for (int t = 0; t < QWB_GATE_ROWS; ++t) acc[t] = 0.f;
    for (int k0 = 0; k0 < n; k0 += QWB_GATE_ROWS_K) {
        const int kn = min(QWB_GATE_ROWS_K, n - k0);
        __syncthreads();
        for (int idx = threadIdx.x; idx < T * kn; idx += 256) {
            const int t = idx / kn, kk = idx - t * kn;
            us[t][kk] = ub[(size_t)t * C + k0 + kk];
        }
        __syncthreads();
        if (o < n) {
            for (int kk = lane; kk < kn; kk += 32) {
                const float w = to_f32(W[k0 + kk]);
#pragma unroll
                for (int t = 0; t < QWB_GATE_ROWS; ++t)
                    if (t < T) acc[t] += w * us[t][kk];
            }
        }
    }
    if (o >= n) return;
    const int c = blk * n + o;
    const float bias = (blockIdx.y ? bi : ba)[c];
    float* out = blockIdx.y ? i_out : r_out;
#pragma unroll
    for (int t = 0; t < QWB_GATE_ROWS; ++t) {
        if (t < T) {
            const float v = warp_sum(acc[t]);
            if (lane == 0) out[(size_t)t * C + c] = sigmoid_f(v + bias);
        }
    }
}

extern "C" int qwb_block_gates(const float* u, const void* wa, const float* ba, const void* wi, const float* bi, float* r_out,
                               float* i_out, int w_dtype, int T, int C, int blocks, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (C <= 0 || blocks <= 0 || C % blocks) return qwb_fail(QWB_ERR_ARG, "block_gates: %d channels in %d equal blocks", C, blocks);
    const int n = C / blocks;
    const long long gy = (long long)blocks * ((n + 63) / 64);
    if (gy > 65535) return qwb_fail(QWB_ERR_ARG, "block_gates: %d channels are too many", C);
    if (w_dtype != QWB_DT_BF16 && w_dtype != QWB_DT_F32) return qwb_fail(QWB_ERR_ARG, "block_gates: unknown dtype %d", w_dtype);
    if (T <= QWB_GATE_ROWS) {
        dim3 grid_rows((unsigned)(blocks * ((n + 7) / 8)), 2);
        if (w_dtype == QWB_DT_BF16) qwb_launch(block_gates_rows_kernel<bf16>, grid_rows, 256, 0, stream, u, (const bf16*)wa, ba, (const bf16*)wi, bi, r_out, i_out, T, C, n);
        else qwb_launch(block_gates_rows_kernel<float>, grid_rows, 256, 0, stream, u, (const float*)wa, ba, (const float*)wi, bi, r_out, i_out, T, C, n);
        return qwb_check_launch("block_gates_rows");
    }
    dim3 grid((T + QWB_GATE_TILE_TOKENS - 1) / QWB_GATE_TILE_TOKENS, (unsigned)gy, 2);
    if (w_dtype == QWB_DT_BF16) qwb_launch(block_gates_kernel<bf16>, grid, 256, 0, stream, u, (const bf16*)wa, ba, (const bf16*)wi, bi, r_out, i_out, T, C, n);
    else if (w_dtype == QWB_DT_F32) qwb_launch(block_gates_kernel<float>, grid, 256, 0, stream, u, (const float*)wa, ba, (const float*)wi, bi, r_out, i_out, T, C, n);
    else return qwb_fail(QWB_ERR_ARG, "block_gates: unknown dtype %d", w_dtype);
    return qwb_check_launch("block_gates");
}

// one token's decay and input: a = exp(-k r), b = sqrt(1 - a^2) i u
__device__ __forceinline__ void rglru_coeffs(float k, float r, float ig, float u, float* a, float* b) {
    const float loga = -k * r;
    *a = expf(loga);
    *b = sqrtf(-expm1f(2.f * loga)) * ig * u;
}

// ---------------------------------------------------------------------------------
// scan in order: grid (ceil(C / 128), B); a thread loads four tokens ahead of their use.
// ---------------------------------------------------------------------------------
template <typename TOut>
__global__ void rglru_scan_kernel(const float* __restrict__ u, const float* __restrict__ r, const float* __restrict__ ig,
                                  const float* __restrict__ lam, const float* __restrict__ y, int ld_y, const float* __restrict__ y_bias,
                                  float* state, const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
                                  TOut* __restrict__ out, int C, float sharpness, int write_state) {
    pdl_wait();
    pdl_launch_dependents();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, b = blockIdx.y;
    if (c >= C) return;
    const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
    const float k = sharpness * softplus_f(lam[c]);
    const float yb = y_bias ? y_bias[c] : 0.f;
    float* st = state + (size_t)slots[b] * C + c;
    float S = *st;
    constexpr int U = 4;
    for (int t = t0; t < t1; t += U) {
        float rr[U], ii[U], uu[U], yy[U];
#pragma unroll
        for (int j = 0; j < U; ++j) {
            const bool in = t + j < t1;
            const size_t at = (size_t)(t + j) * C + c;
            rr[j] = in ? r[at] : 0.f;
            ii[j] = in ? ig[at] : 0.f;
            uu[j] = in ? u[at] : 0.f;
            yy[j] = in ? y[(size_t)(t + j) * ld_y + c] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < U; ++j) {
            if (t + j < t1) {
                float a, bb;
                rglru_coeffs(k, rr[j], ii[j], uu[j], &a, &bb);
                S = a * S + bb;
                out[(size_t)(t + j) * C + c] = from_f32<TOut>(S * gelu_tanh_f(yy[j] + yb));
            }
        }
    }
    if (write_state) *st = S;
}

// ---------------------------------------------------------------------------------
// long prompts in chunks of L tokens.  The chunks of all sequences are numbered in the packed order: chunk_seq[k] is
// chunk k's sequence and chunk_t0[k] its first token (the host lays this out; a sequence's chunks are consecutive).
//   pass 1, grid (ceil(C / 128), chunks): A = product of the chunk's decays, Q = its sum from a zero state
//   pass 2, grid (ceil(C / 128), B):      the state that enters every chunk, in order, and the sequence's new state
//   pass 3, grid (ceil(C / 128), chunks): the chunk again from the state that enters it, with the read-out
// ---------------------------------------------------------------------------------
__global__ void rglru_chunk_sums_kernel(const float* __restrict__ u, const float* __restrict__ r, const float* __restrict__ ig,
                                        const float* __restrict__ lam, const int* __restrict__ chunk_t0, const int* __restrict__ chunk_seq,
                                        const int* __restrict__ cu_seqlens, float* __restrict__ A, float* __restrict__ Q, int C, int L,
                                        float sharpness) {
    pdl_wait();
    pdl_launch_dependents();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, k = blockIdx.y;
    if (c >= C) return;
    const int t0 = chunk_t0[k];
    if (t0 < 0) return;
    const int t1 = min(t0 + L, cu_seqlens[chunk_seq[k] + 1]);
    const float kk = sharpness * softplus_f(lam[c]);
    float a_all = 1.f, S = 0.f;
#pragma unroll 4
    for (int t = t0; t < t1; ++t) {
        const size_t at = (size_t)t * C + c;
        float a, b;
        rglru_coeffs(kk, r[at], ig[at], u[at], &a, &b);
        S = a * S + b;
        a_all *= a;
    }
    A[(size_t)k * C + c] = a_all;
    Q[(size_t)k * C + c] = S;
}

__global__ void rglru_chunk_carry_kernel(const float* __restrict__ A, float* Q, float* state, const int* __restrict__ seq_chunk0,
                                         const int* __restrict__ slots, int C, int write_state) {
    pdl_wait();
    pdl_launch_dependents();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, b = blockIdx.y;
    if (c >= C) return;
    float* st = state + (size_t)slots[b] * C + c;
    float S = *st;
    for (int k = seq_chunk0[b]; k < seq_chunk0[b + 1]; ++k) {
        const size_t at = (size_t)k * C + c;
        const float next = A[at] * S + Q[at];
        Q[at] = S;                      // what enters chunk k
        S = next;
    }
    if (write_state) *st = S;
}

template <typename TOut>
__global__ void rglru_chunk_out_kernel(const float* __restrict__ u, const float* __restrict__ r, const float* __restrict__ ig,
                                       const float* __restrict__ lam, const float* __restrict__ y, int ld_y,
                                       const float* __restrict__ y_bias, const int* __restrict__ chunk_t0,
                                       const int* __restrict__ chunk_seq, const int* __restrict__ cu_seqlens,
                                       const float* __restrict__ S_in, TOut* __restrict__ out, int C, int L, float sharpness) {
    pdl_wait();
    pdl_launch_dependents();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, k = blockIdx.y;
    if (c >= C) return;
    const int t0 = chunk_t0[k];
    if (t0 < 0) return;
    const int t1 = min(t0 + L, cu_seqlens[chunk_seq[k] + 1]);
    const float kk = sharpness * softplus_f(lam[c]);
    const float yb = y_bias ? y_bias[c] : 0.f;
    float S = S_in[(size_t)k * C + c];
#pragma unroll 4
    for (int t = t0; t < t1; ++t) {
        const size_t at = (size_t)t * C + c;
        float a, b;
        rglru_coeffs(kk, r[at], ig[at], u[at], &a, &b);
        S = a * S + b;
        out[at] = from_f32<TOut>(S * gelu_tanh_f(y[(size_t)t * ld_y + c] + yb));
    }
}

// The chunk tables from the step's sequence starts, on the device: one block; thread 0 numbers the sequences' first
// chunks, then every thread fills its sequences' entries; the entries beyond the last chunk get a first token of -1.
__global__ void rglru_chunk_table_kernel(const int* __restrict__ cu_seqlens, int* seq_chunk0, int* chunk_t0, int* chunk_seq, int B,
                                         int L, int max_chunks) {
    pdl_wait();
    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        int k = 0;
        for (int b = 0; b < B; ++b) { seq_chunk0[b] = k; k += (cu_seqlens[b + 1] - cu_seqlens[b] + L - 1) / L; }
        seq_chunk0[B] = k;
    }
    __syncthreads();
    for (int b = threadIdx.x; b < B; b += blockDim.x) {
        const int k0 = seq_chunk0[b], k1 = seq_chunk0[b + 1];
        for (int k = k0; k < k1 && k < max_chunks; ++k) { chunk_t0[k] = cu_seqlens[b] + (k - k0) * L; chunk_seq[k] = b; }
    }
    for (int k = seq_chunk0[B] + threadIdx.x; k < max_chunks; k += blockDim.x) { chunk_t0[k] = -1; chunk_seq[k] = 0; }
}

// u, r, ig [T, C] float; y: columns of a float matrix with rows of ld_y values (the caller offsets the pointer); state
// [slots, C] float; out [T, C] in out_dtype.  With chunk_len > 0 the three-pass form runs: max_chunks >= the number of
// chunks (ceil(T / chunk_len) + B is enough), tables 2 * max_chunks + B + 1 ints and scratch 2 * max_chunks * C floats.
extern "C" int qwb_rglru_scan(const float* u, const float* r, const float* ig, const float* lam, const float* y, int ld_y,
                              const float* y_bias, float* state, const int* cu_seqlens, const int* slots, void* out, int out_dtype,
                              int B, int C, float sharpness, int write_state, int chunk_len, int max_chunks, int* tables,
                              float* scratch, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (C <= 0 || ld_y < C) return qwb_fail(QWB_ERR_ARG, "rglru_scan: %d channels, row stride %d", C, ld_y);
    if (B > 65535 || max_chunks > 65535) return qwb_fail(QWB_ERR_ARG, "rglru_scan: %d sequences or %d chunks are too many", B, max_chunks);
    if (out_dtype != QWB_DT_BF16 && out_dtype != QWB_DT_F32) return qwb_fail(QWB_ERR_ARG, "rglru_scan: unknown dtype %d", out_dtype);
    const int block = 128, gx = (C + block - 1) / block;
    if (chunk_len <= 0) {
        if (out_dtype == QWB_DT_BF16)
            qwb_launch(rglru_scan_kernel<bf16>, dim3(gx, B), block, 0, stream, u, r, ig, lam, y, ld_y, y_bias, state, cu_seqlens, slots, (bf16*)out, C, sharpness, write_state);
        else
            qwb_launch(rglru_scan_kernel<float>, dim3(gx, B), block, 0, stream, u, r, ig, lam, y, ld_y, y_bias, state, cu_seqlens, slots, (float*)out, C, sharpness, write_state);
        return qwb_check_launch("rglru_scan");
    }
    if (max_chunks <= 0 || !tables || !scratch) return qwb_fail(QWB_ERR_ARG, "rglru_scan: the chunked form needs its tables and scratch");
    int* seq_chunk0 = tables;
    int* chunk_t0 = tables + B + 1;
    int* chunk_seq = chunk_t0 + max_chunks;
    float* A = scratch;
    float* Q = scratch + (size_t)max_chunks * C;
    const int n_chunks = max_chunks;
    qwb_launch(rglru_chunk_table_kernel, 1, 256, 0, stream, cu_seqlens, seq_chunk0, chunk_t0, chunk_seq, B, chunk_len, max_chunks);
    if (int rc = qwb_check_launch("rglru_chunk_table")) return rc;
    qwb_launch(rglru_chunk_sums_kernel, dim3(gx, n_chunks), block, 0, stream, u, r, ig, lam, (const int*)chunk_t0, (const int*)chunk_seq, cu_seqlens, A, Q, C, chunk_len, sharpness);
    if (int rc = qwb_check_launch("rglru_chunk_sums")) return rc;
    qwb_launch(rglru_chunk_carry_kernel, dim3(gx, B), block, 0, stream, (const float*)A, Q, state, (const int*)seq_chunk0, slots, C, write_state);
    if (int rc = qwb_check_launch("rglru_chunk_carry")) return rc;
    if (out_dtype == QWB_DT_BF16)
        qwb_launch(rglru_chunk_out_kernel<bf16>, dim3(gx, n_chunks), block, 0, stream, u, r, ig, lam, y, ld_y, y_bias, (const int*)chunk_t0, (const int*)chunk_seq, cu_seqlens, (const float*)Q, (bf16*)out, C, chunk_len, sharpness);
    else
        qwb_launch(rglru_chunk_out_kernel<float>, dim3(gx, n_chunks), block, 0, stream, u, r, ig, lam, y, ld_y, y_bias, (const int*)chunk_t0, (const int*)chunk_seq, cu_seqlens, (const float*)Q, (float*)out, C, chunk_len, sharpness);
    return qwb_check_launch("rglru_chunk_out");
}
