// Attention over a sliding window plus pooled blocks of what lies before it, over the paged cache.
//
// The query at position p sees the keys j with p - window < j <= p, and beside them ONE key and value for every block
// of `pool` consecutive positions that lies wholly before the window: block b = positions b*pool .. b*pool + pool - 1 is
// seen when b*pool + pool - 1 <= p - window, i.e. the first floor((p - window + 1) / pool) blocks.  A block's key and value
// are the means of its keys and values as the cache holds them; they are kept in a second pair of paged pools (one row
// per complete block, written once, when the block's last token arrives: pool_update), so a step reads `window` keys
// and len / pool block rows instead of len keys.  Tokens that have left the window and whose block is not complete in
// that sense are not seen at all.  Tokens and blocks share one softmax.  window = 0: plain causal attention, no blocks.
//
// Keys and values may have different sizes (dim, vdim; multiples of 8 up to 256); query head h reads key/value head
// h / (H / G).  Per-head RMS norm of q and k with a weight shared by the heads, a rotation of the first `rdims` values of
// q and k, and (rotate_v) a rotation of ALL of a value by its own position before it is cached, undone on each head's
// output by the query's position (so the output depends on relative positions of values only).  Pairs of a rotation:
// (i, i + n/2) ("halves") or (2i, 2i + 1) ("interleaved"); cos and sin come as tables [T, n/2] for this step's tokens.
// Scores, maxima, sums and accumulators are 32-bit; q and the cache are float or bfloat16.
//
//   pool_prep      norm, rotations, cache write of a step's tokens; q out
//   pool_update    rows of the pooled pools for the blocks that this step completes
//   pool_prefill   any number of new tokens per sequence
//   pool_decode    one new token per sequence: runs of pages of the block rows and of the window, one block of
//                  threads a run, then a merge that also turns the output back
#include "common.cuh"

#define QWB_POOL_MAX_DIM 256
#define QWB_POOL_PAGE 64
#define QWB_POOL_RUN_PAGES 2          // pages per run of the decode kernel: fixed, so a sequence's sums do not depend on the batch

// value i of a head after its first n values were turned by the angle whose cos and sin are cs[m], sn[m] for pair m
__device__ __forceinline__ float turned(const float* v, int i, int n, const float* cs, const float* sn, int interleaved, float sign) {
    if (i >= n) return v[i];
    const int half = n >> 1;
    int m, first;
    float a, b;
    if (interleaved) { m = i >> 1; first = !(i & 1); a = v[2 * m]; b = v[2 * m + 1]; }
    else { m = i < half ? i : i - half; first = i < half; a = v[m]; b = v[m + half]; }
    const float c = cs[m], s = sign * sn[m];
    return first ? a * c - b * s : b * c + a * s;
}

__device__ __forceinline__ int blocks_seen(int p, int window, int pool) {
    return (window > 0 && pool > 0 && p - window + 1 >= pool) ? (p - window + 1) / pool : 0;
}

// ---------------------------------------------------------------------------------
// prep: grid (T, ceil((H + 2 G) / 4)), 4 warps, a warp per (token, head of q | k | v).
// ---------------------------------------------------------------------------------
template <typename T>
__global__ void pool_prep_kernel(const float* __restrict__ qkv, const float* __restrict__ qw, const float* __restrict__ kw,
                                 const float* __restrict__ cos_qk, const float* __restrict__ sin_qk, const float* __restrict__ cos_v,
                                 const float* __restrict__ sin_v, const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                 const int* __restrict__ page_table, int table_width, T* __restrict__ q_out, T* __restrict__ k_pool,
                                 T* __restrict__ v_pool, int H, int G, int dim, int vdim, int rdims, int interleaved, int rotate_v,
                                 float eps, int store_kv) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float bufs[4][QWB_POOL_MAX_DIM];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int item = blockIdx.y * 4 + warp, t = blockIdx.x;
    if (item >= H + 2 * G) return;
    float* buf = bufs[warp];
    const int ld = (H + G) * dim + G * vdim;
    const bool is_q = item < H, is_k = !is_q && item < H + G;
    const int n = (is_q || is_k) ? dim : vdim;
    const int head = is_q ? item : (is_k ? item - H : item - H - G);
    const float* src = qkv + (size_t)t * ld + (is_q ? head * dim : (is_k ? H * dim + head * dim : (H + G) * dim + head * vdim));
    float ss = 0.f;
    for (int i = lane; i < n; i += 32) { const float v = src[i]; buf[i] = v; ss += v * v; }
    const float* w = is_q ? qw : (is_k ? kw : nullptr);
    if (w) {
        const float scale = rsqrtf(warp_sum(ss) / (float)n + eps);
        for (int i = lane; i < n; i += 32) buf[i] = buf[i] * scale * w[i];
    }
    __syncwarp();
    const bool is_v = !is_q && !is_k;
    const int rd = is_v ? (rotate_v ? vdim : 0) : rdims;
    const float* cs = is_v ? cos_v : cos_qk;
    const float* sn = is_v ? sin_v : sin_qk;
    if (rd > 0) { cs += (size_t)t * (rd >> 1); sn += (size_t)t * (rd >> 1); }
    T* dst;
    if (is_q) dst = q_out + ((size_t)t * H + head) * dim;
    else {
        if (!store_kv) return;
        const int b = tok_seq[t], p = tok_pos[t];
        const size_t row = ((size_t)page_table[(size_t)b * table_width + p / QWB_POOL_PAGE] * G + head) * QWB_POOL_PAGE + p % QWB_POOL_PAGE;
        dst = is_k ? k_pool + row * dim : v_pool + row * vdim;
    }
    for (int i = lane; i < n; i += 32) dst[i] = from_f32<T>(rd > 0 ? turned(buf, i, rd, cs, sn, interleaved, 1.f) : buf[i]);
}

extern "C" int qwb_pool_prep(const float* qkv, const float* qw, const float* kw, const float* cos_qk, const float* sin_qk,
                             const float* cos_v, const float* sin_v, const int* tok_seq, const int* tok_pos, const int* page_table,
                             int table_width, void* q_out, void* k_pool, void* v_pool, int dtype, int T, int H, int G, int dim, int vdim,
                             int rdims, int interleaved, int rotate_v, float eps, int store_kv, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G) return qwb_fail(QWB_ERR_ARG, "pool_prep: %d query heads are not a multiple of %d key/value heads", H, G);
    if (dim <= 0 || vdim <= 0 || dim > QWB_POOL_MAX_DIM || vdim > QWB_POOL_MAX_DIM)
        return qwb_fail(QWB_ERR_ARG, "pool_prep: key size %d or value size %d outside 1..%d", dim, vdim, QWB_POOL_MAX_DIM);
    if (rdims < 0 || rdims > dim || rdims % 2 || (rotate_v && vdim % 2))
        return qwb_fail(QWB_ERR_ARG, "pool_prep: a rotation of %d of %d values (values: %d) needs even sizes", rdims, dim, vdim);
    if ((rdims > 0 && (!cos_qk || !sin_qk)) || (rotate_v && (!cos_v || !sin_v))) return qwb_fail(QWB_ERR_ARG, "pool_prep: a rotation without its table");
    dim3 grid(T, (H + 2 * G + 3) / 4);
    if (dtype == QWB_DT_F32)
        qwb_launch(pool_prep_kernel<float>, grid, 128, 0, stream, qkv, qw, kw, cos_qk, sin_qk, cos_v, sin_v, tok_seq, tok_pos, page_table, table_width,
                   (float*)q_out, (float*)k_pool, (float*)v_pool, H, G, dim, vdim, rdims, interleaved, rotate_v, eps, store_kv);
    else if (dtype == QWB_DT_BF16)
        qwb_launch(pool_prep_kernel<bf16>, grid, 128, 0, stream, qkv, qw, kw, cos_qk, sin_qk, cos_v, sin_v, tok_seq, tok_pos, page_table, table_width,
                   (bf16*)q_out, (bf16*)k_pool, (bf16*)v_pool, H, G, dim, vdim, rdims, interleaved, rotate_v, eps, store_kv);
    else return qwb_fail(QWB_ERR_ARG, "pool_prep: unknown dtype %d", dtype);
    return qwb_check_launch("pool_prep");
}

// ---------------------------------------------------------------------------------
// update: grid (most blocks a sequence completes in this step, G, B).  Block `blk` of a sequence is complete once the
// sequence holds (blk + 1) * pool tokens; this step completes the blocks pos0 / pool .. seq_len / pool - 1.  The sums run
// over the block's tokens in order, in float; the mean is the sum divided by pool.
// ---------------------------------------------------------------------------------
template <typename T>
__global__ void pool_update_kernel(const T* __restrict__ k_pool, const T* __restrict__ v_pool, T* __restrict__ pk_pool, T* __restrict__ pv_pool,
                                   const int* __restrict__ page_table, const int* __restrict__ block_table, int table_width,
                                   const int* __restrict__ pos0, const int* __restrict__ seq_len, int G, int dim, int vdim, int pool) {
    pdl_wait();
    pdl_launch_dependents();
    const int b = blockIdx.z, g = blockIdx.y;
    const int blk = pos0[b] / pool + blockIdx.x;
    if (blk >= seq_len[b] / pool) return;
    const int* pages = page_table + (size_t)b * table_width;
    const size_t to = ((size_t)block_table[(size_t)b * table_width + blk / QWB_POOL_PAGE] * G + g) * QWB_POOL_PAGE + blk % QWB_POOL_PAGE;
    for (int d = threadIdx.x; d < dim + vdim; d += blockDim.x) {
        const bool key = d < dim;
        const int n = key ? dim : vdim, e = key ? d : d - dim;
        const T* src = key ? k_pool : v_pool;
        float s = 0.f;
        for (int j = blk * pool; j < (blk + 1) * pool; ++j)
            s += to_f32(src[(((size_t)pages[j / QWB_POOL_PAGE] * G + g) * QWB_POOL_PAGE + j % QWB_POOL_PAGE) * n + e]);
        (key ? pk_pool : pv_pool)[to * n + e] = from_f32<T>(s / (float)pool);
    }
}

extern "C" int qwb_pool_update(const void* k_pool, const void* v_pool, void* pk_pool, void* pv_pool, const int* page_table,
                               const int* block_table, int table_width, const int* pos0, const int* seq_len, int dtype, int B, int max_blocks,
                               int G, int dim, int vdim, int pool, cudaStream_t stream) {
    if (B <= 0 || max_blocks <= 0) return 0;
    if (pool <= 0 || G <= 0 || G > 65535 || B > 65535) return qwb_fail(QWB_ERR_ARG, "pool_update: blocks of %d tokens, %d heads, %d sequences", pool, G, B);
    dim3 grid(max_blocks, G, B);
    if (dtype == QWB_DT_F32)
        qwb_launch(pool_update_kernel<float>, grid, 128, 0, stream, (const float*)k_pool, (const float*)v_pool, (float*)pk_pool, (float*)pv_pool,
                   page_table, block_table, table_width, pos0, seq_len, G, dim, vdim, pool);
    else if (dtype == QWB_DT_BF16)
        qwb_launch(pool_update_kernel<bf16>, grid, 128, 0, stream, (const bf16*)k_pool, (const bf16*)v_pool, (bf16*)pk_pool, (bf16*)pv_pool,
                   page_table, block_table, table_width, pos0, seq_len, G, dim, vdim, pool);
    else return qwb_fail(QWB_ERR_ARG, "pool_update: unknown dtype %d", dtype);
    return qwb_check_launch("pool_update");
}

// ---------------------------------------------------------------------------------
// prefill: one block per (tile of 16 queries, query head, sequence); 4 warps, each owns 4 queries; keys come in tiles of
// 32 (one key per lane): first the block rows that the tile's last query sees, then the tokens from the first query's
// window start to the last query.
// ---------------------------------------------------------------------------------
template <typename T, int NC>   // NC = ceil(vdim / 32) rounded up to 2, 4 or 8
__global__ void pool_prefill_kernel(const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                                    const T* __restrict__ pk_pool, const T* __restrict__ pv_pool, const int* __restrict__ page_table,
                                    const int* __restrict__ block_table, const int* __restrict__ cu_seqlens, const int* __restrict__ pos0,
                                    const float* __restrict__ cos_v, const float* __restrict__ sin_v, T* __restrict__ out, int H, int G,
                                    int dim, int vdim, int table_width, float scale, int window, int pool, int interleaved) {
    pdl_wait();
    pdl_launch_dependents();
    constexpr int BQ = 16, BK = 32, QPW = 4, PG = QWB_POOL_PAGE;
    extern __shared__ float smem[];
    float* Qs = smem;                         // [BQ][dim], already scaled
    float* Ks = Qs + BQ * dim;                // [BK][dim + 1]
    float* Vs = Ks + BK * (dim + 1);          // [BK][vdim]; at the end [BQ][vdim] outputs

    const int b = blockIdx.z, h = blockIdx.y, q0 = blockIdx.x * BQ;
    const int t0 = cu_seqlens[b], n_new = cu_seqlens[b + 1] - t0;
    if (q0 >= n_new) return;
    const int g = h / (H / G);
    const int p0 = pos0[b];
    const int nq = min(BQ, n_new - q0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    for (int idx = threadIdx.x; idx < BQ * dim; idx += blockDim.x) {
        const int i = idx / dim, d = idx - i * dim;
        Qs[idx] = i < nq ? to_f32(q[((size_t)(t0 + q0 + i) * H + h) * dim + d]) * scale : 0.f;
    }

    float m[QPW], l[QPW], acc[QPW][NC];
    int seen[QPW];
#pragma unroll
    for (int i = 0; i < QPW; ++i) {
        m[i] = -INFINITY; l[i] = 0.f;
        seen[i] = blocks_seen(p0 + q0 + warp * QPW + i, window, pool);
#pragma unroll
        for (int c = 0; c < NC; ++c) acc[i][c] = 0.f;
    }

    const int k_last = p0 + q0 + nq - 1;                                  // last key any query of the tile sees
    const int k_first = window > 0 ? max(0, p0 + q0 - window + 1) : 0;    // first key the first query sees
    const int n_blocks = blocks_seen(k_last, window, pool);               // block rows the last query sees
    const int* pages = page_table + (size_t)b * table_width;
    const int* bpages = block_table ? block_table + (size_t)b * table_width : nullptr;

    for (int phase = 0; phase < 2; ++phase) {
        const int kt0 = phase ? (k_first / BK) * BK : 0, kt_end = phase ? k_last + 1 : n_blocks;
        const T* kp = phase ? k_pool : pk_pool;
        const T* vp = phase ? v_pool : pv_pool;
        const int* pg = phase ? pages : bpages;
        for (int kt = kt0; kt < kt_end; kt += BK) {
            __syncthreads();
            for (int idx = threadIdx.x; idx < BK * dim; idx += blockDim.x) {
                const int j = idx / dim, d = idx - j * dim, key = kt + j;
                Ks[j * (dim + 1) + d] = key < kt_end ? to_f32(kp[(((size_t)pg[key / PG] * G + g) * PG + key % PG) * dim + d]) : 0.f;
            }
            for (int idx = threadIdx.x; idx < BK * vdim; idx += blockDim.x) {
                const int j = idx / vdim, d = idx - j * vdim, key = kt + j;
                Vs[idx] = key < kt_end ? to_f32(vp[(((size_t)pg[key / PG] * G + g) * PG + key % PG) * vdim + d]) : 0.f;
            }
            __syncthreads();

            float s[QPW];
#pragma unroll
            for (int i = 0; i < QPW; ++i) s[i] = 0.f;
            const float* krow = Ks + lane * (dim + 1);
            for (int d = 0; d < dim; ++d) {
                const float kd = krow[d];
#pragma unroll
                for (int i = 0; i < QPW; ++i) s[i] += Qs[(warp * QPW + i) * dim + d] * kd;
            }
            const int key = kt + lane;
            float p[QPW];
#pragma unroll
            for (int i = 0; i < QPW; ++i) {
                const int qi = warp * QPW + i;
                const int qp = p0 + q0 + qi;
                const bool ok = qi < nq && (phase ? (key <= qp && (window <= 0 || key > qp - window)) : key < seen[i]);
                const float si = ok ? s[i] : -INFINITY;
                const float m_new = fmaxf(m[i], warp_max(si));
                if (m_new == -INFINITY) { p[i] = 0.f; continue; }       // nothing visible so far (whole warp agrees)
                const float alpha = expf(m[i] - m_new);                 // m = -inf gives 0
                p[i] = ok ? expf(si - m_new) : 0.f;
                l[i] = l[i] * alpha + warp_sum(p[i]);
                m[i] = m_new;
#pragma unroll
                for (int c = 0; c < NC; ++c) acc[i][c] *= alpha;
            }
            for (int j = 0; j < BK; ++j) {
                float pj[QPW];
#pragma unroll
                for (int i = 0; i < QPW; ++i) pj[i] = __shfl_sync(0xffffffffu, p[i], j);
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    const int d = lane + 32 * c;
                    if (d < vdim) {
                        const float v = Vs[j * vdim + d];
#pragma unroll
                        for (int i = 0; i < QPW; ++i) acc[i][c] += pj[i] * v;
                    }
                }
            }
        }
    }

    __syncthreads();                          // Vs is free: the outputs pass through it so that a value finds its partner
#pragma unroll
    for (int i = 0; i < QPW; ++i) {
        const int qi = warp * QPW + i;
        const float inv = 1.f / l[i];
#pragma unroll
        for (int c = 0; c < NC; ++c) {
            const int d = lane + 32 * c;
            if (d < vdim) Vs[qi * vdim + d] = acc[i][c] * inv;
        }
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < QPW; ++i) {
        const int qi = warp * QPW + i;
        if (qi >= nq) continue;
        const size_t t = t0 + q0 + qi;
        T* o = out + (t * H + h) * vdim;
        const float* row = Vs + qi * vdim;
        for (int d = lane; d < vdim; d += 32)
            o[d] = from_f32<T>(cos_v ? turned(row, d, vdim, cos_v + t * (vdim >> 1), sin_v + t * (vdim >> 1), interleaved, -1.f) : row[d]);
    }
}

static int check_pool_sizes(const char* what, int H, int G, int dim, int vdim, int table_width, int window, int pool) {
    if (H <= 0 || G <= 0 || H % G) return qwb_fail(QWB_ERR_ARG, "%s: %d query heads are not a multiple of %d key/value heads", what, H, G);
    if (dim <= 0 || dim % 8 || dim > QWB_POOL_MAX_DIM || vdim <= 0 || vdim % 8 || vdim > QWB_POOL_MAX_DIM)
        return qwb_fail(QWB_ERR_ARG, "%s: key size %d or value size %d is not a multiple of 8 in [8, %d]", what, dim, vdim, QWB_POOL_MAX_DIM);
    if (table_width <= 0 || window < 0 || pool < 0) return qwb_fail(QWB_ERR_ARG, "%s: bad table width %d, window %d or block size %d", what, table_width, window, pool);
    return 0;
}

template <typename T>
static int launch_pool_prefill(const void* q, const void* k_pool, const void* v_pool, const void* pk_pool, const void* pv_pool,
                               const int* page_table, const int* block_table, const int* cu_seqlens, const int* pos0, const float* cos_v,
                               const float* sin_v, void* out, int B, int max_new, int H, int G, int dim, int vdim, int table_width,
                               float scale, int window, int pool, int interleaved, cudaStream_t stream) {
    const size_t smem = ((size_t)16 * dim + 32 * (dim + 1) + 32 * vdim) * sizeof(float);
    dim3 grid((max_new + 15) / 16, H, B);
    const int nc = (vdim + 31) / 32;
#define QWB_LAUNCH_POOL_PREFILL(NC)                                                                              \
    do {                                                                                                         \
        if (smem > 48 * 1024) {                                                                                  \
            cudaError_t e = cudaFuncSetAttribute(pool_prefill_kernel<T, NC>,                                     \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);        \
            if (e != cudaSuccess) return qwb_fail(QWB_ERR_CUDA, "pool_prefill: %s", cudaGetErrorString(e));      \
        }                                                                                                        \
        qwb_launch(pool_prefill_kernel<T, NC>, grid, 128, smem, stream, (const T*)q, (const T*)k_pool, (const T*)v_pool, \
            (const T*)pk_pool, (const T*)pv_pool, page_table, block_table, cu_seqlens, pos0, cos_v, sin_v, (T*)out, H, G, dim, vdim, \
            table_width, scale, window, pool, interleaved);                                                      \
    } while (0)
    if (nc <= 2) QWB_LAUNCH_POOL_PREFILL(2);
    else if (nc <= 4) QWB_LAUNCH_POOL_PREFILL(4);
    else QWB_LAUNCH_POOL_PREFILL(8);
#undef QWB_LAUNCH_POOL_PREFILL
    return qwb_check_launch("pool_prefill");
}

// q [T, H, dim]; out [T, H * vdim]; cos_v, sin_v [T, vdim / 2] or null (values not rotated).
extern "C" int qwb_pool_prefill(const void* q, const void* k_pool, const void* v_pool, const void* pk_pool, const void* pv_pool,
                                const int* page_table, const int* block_table, const int* cu_seqlens, const int* pos0,
                                const float* cos_v, const float* sin_v, void* out, int dtype, int B, int max_new, int H, int G, int dim,
                                int vdim, int table_width, float scale, int window, int pool, int interleaved, cudaStream_t stream) {
    if (B <= 0 || max_new <= 0) return 0;
    if (int rc = check_pool_sizes("pool_prefill", H, G, dim, vdim, table_width, window, pool)) return rc;
    if (B > 65535 || H > 65535) return qwb_fail(QWB_ERR_ARG, "pool_prefill: batch %d or heads %d above 65535", B, H);
    if (window > 0 && pool > 0 && (!pk_pool || !pv_pool || !block_table)) return qwb_fail(QWB_ERR_ARG, "pool_prefill: blocks without their pools");
    if (dtype == QWB_DT_F32)
        return launch_pool_prefill<float>(q, k_pool, v_pool, pk_pool, pv_pool, page_table, block_table, cu_seqlens, pos0, cos_v, sin_v, out,
                                          B, max_new, H, G, dim, vdim, table_width, scale, window, pool, interleaved, stream);
    if (dtype == QWB_DT_BF16)
        return launch_pool_prefill<bf16>(q, k_pool, v_pool, pk_pool, pv_pool, page_table, block_table, cu_seqlens, pos0, cos_v, sin_v, out,
                                         B, max_new, H, G, dim, vdim, table_width, scale, window, pool, interleaved, stream);
    return qwb_fail(QWB_ERR_ARG, "pool_prefill: unknown dtype %d", dtype);
}

// ---------------------------------------------------------------------------------
// prefill on the tensor cores (bfloat16, mma.sync m16n8k16): block = 64 queries of one (sequence, query head), 4 warps of
// 16 rows; keys in tiles of 64 = one page of the block rows' pools, then of the tokens' pools, so a tile is one contiguous
// piece of the cache.  Q, K and V tiles sit in shared memory with rows padded by 16 bytes (conflict-free ldmatrix); K has
// two buffers, V one: the next tile's keys are copied in (cp.async) under this tile's work, its values under its own
// scores and softmax.  Scores, maxima, sums and
// the accumulator are 32-bit; probabilities are rounded to bfloat16 for the second product.  The normed outputs pass
// through shared memory once, so that each value finds its partner when the head is turned back.
// dim a multiple of 16, vdim of 8.
// ---------------------------------------------------------------------------------
#define PM_BQ 64
#define PM_BK 64
#define PM_PAD 8

__device__ __forceinline__ void pm_ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const bf16* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void pm_ldsm_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const bf16* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void pm_mma(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// 16 bytes from global to shared memory; `bytes` 0 writes zeros (src must still be a valid address)
__device__ __forceinline__ void pm_cp16(bf16* dst, const bf16* src, int bytes) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void pm_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void pm_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint32_t pm_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int NV>       // n-tiles of 8 value columns the accumulator has room for
__global__ void __launch_bounds__(128)
pool_prefill_mma_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pool, const bf16* __restrict__ v_pool,
                        const bf16* __restrict__ pk_pool, const bf16* __restrict__ pv_pool, const int* __restrict__ page_table,
                        const int* __restrict__ block_table, const int* __restrict__ cu_seqlens, const int* __restrict__ pos0,
                        const float* __restrict__ cos_v, const float* __restrict__ sin_v, bf16* __restrict__ out, int H, int G,
                        int dim, int vdim, int table_width, float scale, int window, int pool, int interleaved) {
    pdl_wait();
    pdl_launch_dependents();
    const int ldq = dim + PM_PAD, ldv = vdim + PM_PAD;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);           // [64][ldq]
    bf16* Kbuf = Qs + PM_BQ * ldq;                          // [2][64][ldq]
    bf16* Vbuf = Kbuf + 2 * PM_BK * ldq;                    // [64][ldv]
    float* Obuf = reinterpret_cast<float*>(Kbuf);           // at the end, over the key buffers: [64][vdim] floats

    const int b = blockIdx.z, h = blockIdx.y, q0 = blockIdx.x * PM_BQ;
    const int t0 = cu_seqlens[b], n = cu_seqlens[b + 1] - t0;
    if (q0 >= n) return;
    const int g_kv = h / (H / G);
    const int p0 = pos0[b];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nq = min(PM_BQ, n - q0);

    for (int idx = tid; idx < PM_BQ * (dim / 8); idx += blockDim.x) {
        const int r = idx / (dim / 8), c = (idx - r * (dim / 8)) * 8;
        const bool in = r < nq;
        pm_cp16(Qs + r * ldq + c, q + ((size_t)(t0 + (in ? q0 + r : 0)) * H + h) * dim + c, in ? 16 : 0);
    }

    float o[NV][4];
#pragma unroll
    for (int j = 0; j < NV; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;      // rows gr and gr + 8 of the warp's 16
    const int gr = lane >> 2, tq = lane & 3;
    const int pos_a = p0 + q0 + warp * 16 + gr, pos_b = pos_a + 8;  // positions of the thread's two rows
    const int seen_a = blocks_seen(pos_a, window, pool), seen_b = blocks_seen(pos_b, window, pool);

    const int k_hi = p0 + q0 + nq - 1;                              // last key any query of the tile sees
    const int k_lo = window > 0 ? max(0, p0 + q0 - window + 1) : 0;
    const int n_blocks = blocks_seen(k_hi, window, pool);           // block rows the last query sees
    const int nv_used = vdim / 8;
    const int block_tiles = (n_blocks + PM_BK - 1) / PM_BK;
    const int first_page = k_lo / PM_BK, token_tiles = k_hi / PM_BK - first_page + 1;
    const int n_tiles = block_tiles + token_tiles;
    const int* pages = page_table + (size_t)b * table_width;
    const int* bpages = block_table ? block_table + (size_t)b * table_width : nullptr;

    auto tile_source = [&](int it, const bf16** ks, const bf16** vs, int* rows) {
        const bool blocks = it < block_tiles;
        const int page = blocks ? it : first_page + (it - block_tiles);
        *rows = blocks ? min(PM_BK, n_blocks - page * PM_BK) : min(PM_BK, k_hi + 1 - page * PM_BK);
        const size_t tile = ((size_t)(blocks ? bpages : pages)[page] * G + g_kv) * PM_BK;
        *ks = (blocks ? pk_pool : k_pool) + tile * dim;
        *vs = (blocks ? pv_pool : v_pool) + tile * vdim;
    };
    auto copy_keys = [&](int it, int stage) {                       // one commit group
        const bf16 *ks, *vs;
        int rows;
        tile_source(it, &ks, &vs, &rows);
        bf16* Kd = Kbuf + stage * PM_BK * ldq;
        for (int idx = tid; idx < PM_BK * (dim / 8); idx += blockDim.x) {
            const int r = idx / (dim / 8), c = (idx - r * (dim / 8)) * 8;
            pm_cp16(Kd + r * ldq + c, ks + (size_t)(r < rows ? r : 0) * dim + c, r < rows ? 16 : 0);
        }
        pm_commit();
    };
    auto copy_values = [&](int it) {                                // one commit group
        const bf16 *ks, *vs;
        int rows;
        tile_source(it, &ks, &vs, &rows);
        for (int idx = tid; idx < PM_BK * (vdim / 8); idx += blockDim.x) {
            const int r = idx / (vdim / 8), c = (idx - r * (vdim / 8)) * 8;
            pm_cp16(Vbuf + r * ldv + c, vs + (size_t)(r < rows ? r : 0) * vdim + c, r < rows ? 16 : 0);
        }
        pm_commit();
    };
    // Keys have two buffers, values one: tile i + 1's keys are copied in under tile i's work, tile i + 1's values under its
    // own scores and softmax (three blocks of threads then fit an SM instead of two).  Groups in the order of their
    // commits: [Q, K0], V0, K1, V1, K2, ...
    copy_keys(0, 0);
    copy_values(0);
    const float scale2 = scale * 1.4426950408889634f;               // scores in units of ln 2: exp2f below
    const int warp_lo = p0 + q0 + warp * 16, warp_hi = warp_lo + 15;
    const int warp_seen = blocks_seen(warp_lo, window, pool);       // block rows that every row of the warp sees

    for (int it = 0; it < n_tiles; ++it) {
        const bf16* Ks = Kbuf + (it & 1) * PM_BK * ldq;
        const bf16* Vs = Vbuf;
        const bool more = it + 1 < n_tiles;
        if (more) {                                                 // the next keys into the other buffer (its last readers
            copy_keys(it + 1, (it + 1) & 1);                        // passed the barrier at the end of the round before)
            pm_wait<2>();                                           // this tile's keys (and Q) are there
        } else {
            pm_wait<1>();
        }
        __syncthreads();
        const bool blocks = it < block_tiles;
        const int key0 = (blocks ? it : first_page + (it - block_tiles)) * PM_BK;

        float s[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
        for (int d = 0; d < dim; d += 16) {
            uint32_t a0, a1, a2, a3;
            pm_ldsm_x4(a0, a1, a2, a3, Qs + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldq + d + (lane >> 4) * 8);
#pragma unroll
            for (int j = 0; j < 8; j += 2) {                        // two tiles of 8 keys a load
                uint32_t b0, b1, b2, b3;
                pm_ldsm_x4(b0, b1, b2, b3, Ks + (j * 8 + (lane & 7) + (lane >> 4) * 8) * ldq + d + ((lane >> 3) & 1) * 8);
                pm_mma(s[j], a0, a1, a2, a3, b0, b1);
                pm_mma(s[j + 1], a0, a1, a2, a3, b2, b3);
            }
        }
        // a tile that every row of the warp sees whole needs no mask (most tiles of a long prompt)
        const bool whole = blocks ? key0 + PM_BK <= warp_seen : (key0 + PM_BK - 1 <= warp_lo && (window <= 0 || key0 > warp_hi - window));
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                bool ok = true;
                if (!whole) {
                    const int key = key0 + j * 8 + tq * 2 + (e & 1);
                    const int pos = e < 2 ? pos_a : pos_b;
                    ok = blocks ? key < (e < 2 ? seen_a : seen_b) : (key <= pos && key <= k_hi && (window <= 0 || key > pos - window));
                }
                s[j][e] = ok ? s[j][e] * scale2 : -INFINITY;
            }
            mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
            mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float base0 = mn0 == -INFINITY ? 0.f : mn0, base1 = mn1 == -INFINITY ? 0.f : mn1;
        const float alpha0 = exp2f(m0 - base0), alpha1 = exp2f(m1 - base1);    // m = -inf gives 0
        float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            s[j][0] = exp2f(s[j][0] - base0); s[j][1] = exp2f(s[j][1] - base0);
            s[j][2] = exp2f(s[j][2] - base1); s[j][3] = exp2f(s[j][3] - base1);
            sum0 += s[j][0] + s[j][1];
            sum1 += s[j][2] + s[j][3];
        }
        sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1); sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
        sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1); sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
        l0 = l0 * alpha0 + sum0; l1 = l1 * alpha1 + sum1;
        m0 = mn0; m1 = mn1;
#pragma unroll
        for (int j = 0; j < NV; ++j) { o[j][0] *= alpha0; o[j][1] *= alpha0; o[j][2] *= alpha1; o[j][3] *= alpha1; }

        if (more) pm_wait<1>(); else pm_wait<0>();                  // this tile's values are there
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {                            // O += P V, 16 keys a step
            const uint32_t a0 = pm_pack(s[2 * ks][0], s[2 * ks][1]), a1 = pm_pack(s[2 * ks][2], s[2 * ks][3]);
            const uint32_t a2 = pm_pack(s[2 * ks + 1][0], s[2 * ks + 1][1]), a3 = pm_pack(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
            for (int j = 0; j < NV; j += 2) {
                if (j < nv_used) {                                  // vdim / 8 may be odd: the second tile of a pair reads padding
                    uint32_t b0, b1, b2, b3;                        // or the next row's start, and its result is never stored
                    pm_ldsm_x4_trans(b0, b1, b2, b3, Vs + (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldv + j * 8 + (lane >> 4) * 8);
                    pm_mma(o[j], a0, a1, a2, a3, b0, b1);
                    if (j + 1 < NV) pm_mma(o[j + 1], a0, a1, a2, a3, b2, b3);
                }
            }
        }
        __syncthreads();                                            // the values' buffer may be copied into again
        if (more) copy_values(it + 1);
    }

    // the warp's 16 rows of normed output through shared memory (the buffers are free), then turned back and stored
    float* Os = Obuf + (size_t)warp * 16 * vdim;
    const float inv0 = 1.f / l0, inv1 = 1.f / l1;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        if (j < nv_used) {
            const int col = j * 8 + tq * 2;
            Os[gr * vdim + col] = o[j][0] * inv0; Os[gr * vdim + col + 1] = o[j][1] * inv0;
            Os[(gr + 8) * vdim + col] = o[j][2] * inv1; Os[(gr + 8) * vdim + col + 1] = o[j][3] * inv1;
        }
    }
    __syncwarp();
    const int half = vdim >> 1;
    for (int r = 0; r < 16; ++r) {
        const int row = warp * 16 + r;
        if (row >= nq) break;
        const size_t t = (size_t)t0 + q0 + row;
        const float* src = Os + r * vdim;
        bf16* dst = out + (t * H + h) * vdim;
        for (int c = lane * 2; c < vdim; c += 64) {
            float x0 = src[c], x1 = src[c + 1];
            if (cos_v) {
                x0 = turned(src, c, vdim, cos_v + t * half, sin_v + t * half, interleaved, -1.f);
                x1 = turned(src, c + 1, vdim, cos_v + t * half, sin_v + t * half, interleaved, -1.f);
            }
            *reinterpret_cast<uint32_t*>(dst + c) = pm_pack(x0, x1);
        }
    }
}

// Q and two key buffers [64][dim + 8] and one value buffer [64][vdim + 8] of bfloat16; the outputs' [64][vdim] floats lie
// over the key buffers at the end
static size_t pm_smem_bytes(int dim, int vdim) {
    const size_t keys = (size_t)2 * PM_BK * (dim + PM_PAD) * sizeof(bf16), outs = (size_t)PM_BQ * vdim * sizeof(float);
    return (size_t)PM_BQ * (dim + PM_PAD) * sizeof(bf16) + (keys > outs ? keys : outs) + (size_t)PM_BK * (vdim + PM_PAD) * sizeof(bf16);
}

extern "C" int qwb_pool_prefill_mma_fits(int dtype, int dim, int vdim) {
    const size_t smem = pm_smem_bytes(dim, vdim);
    return dtype == QWB_DT_BF16 && dim > 0 && dim % 16 == 0 && vdim > 0 && vdim % 8 == 0 && dim <= QWB_POOL_MAX_DIM &&
           vdim <= QWB_POOL_MAX_DIM && smem <= 220 * 1024;
}

extern "C" int qwb_pool_prefill_mma(const void* q, const void* k_pool, const void* v_pool, const void* pk_pool, const void* pv_pool,
                                    const int* page_table, const int* block_table, const int* cu_seqlens, const int* pos0,
                                    const float* cos_v, const float* sin_v, void* out, int B, int max_new, int H, int G, int dim,
                                    int vdim, int table_width, float scale, int window, int pool, int interleaved, cudaStream_t stream) {
    if (B <= 0 || max_new <= 0) return 0;
    if (int rc = check_pool_sizes("pool_prefill_mma", H, G, dim, vdim, table_width, window, pool)) return rc;
    if (!qwb_pool_prefill_mma_fits(QWB_DT_BF16, dim, vdim))
        return qwb_fail(QWB_ERR_ARG, "pool_prefill_mma: keys of %d (a multiple of 16) and values of %d (of 8) that fit in shared memory", dim, vdim);
    if (B > 65535 || H > 65535) return qwb_fail(QWB_ERR_ARG, "pool_prefill_mma: batch %d or heads %d above 65535", B, H);
    if (window > 0 && pool > 0 && (!pk_pool || !pv_pool || !block_table)) return qwb_fail(QWB_ERR_ARG, "pool_prefill_mma: blocks without their pools");
    for (const void* p : {q, k_pool, v_pool, (const void*)out})
        if ((uintptr_t)p % 16) return qwb_fail(QWB_ERR_ARG, "pool_prefill_mma: a tensor is not 16-byte aligned");
    const size_t smem = pm_smem_bytes(dim, vdim);
    const dim3 grid((max_new + PM_BQ - 1) / PM_BQ, H, B);
#define QWB_PM(NV)                                                                                                              \
    do {                                                                                                                        \
        if (smem > 48 * 1024) {                                                                                                 \
            cudaError_t e = cudaFuncSetAttribute(pool_prefill_mma_kernel<NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return qwb_fail(QWB_ERR_CUDA, "pool_prefill_mma: %s", cudaGetErrorString(e));                 \
        }                                                                                                                       \
        qwb_launch(pool_prefill_mma_kernel<NV>, grid, 128, smem, stream, (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, \
                   (const bf16*)pk_pool, (const bf16*)pv_pool, page_table, block_table, cu_seqlens, pos0, cos_v, sin_v, (bf16*)out, H, G, \
                   dim, vdim, table_width, scale, window, pool, interleaved);                                                   \
    } while (0)
    if (vdim <= 32) QWB_PM(4); else if (vdim <= 64) QWB_PM(8); else if (vdim <= 128) QWB_PM(16); else QWB_PM(32);
#undef QWB_PM
    return qwb_check_launch("pool_prefill_mma");
}

// ---------------------------------------------------------------------------------
// decode: one new token per sequence (its position is len - 1).  Runs 0 .. block_runs - 1 walk the block rows, two pages
// of 64 rows each; the runs after them walk the window's pages, counted from the page of the window's first key.  Which
// rows a run holds follows from the sequence's own length alone.  Block = (run, key/value head and slice of its query
// heads, sequence), 128 threads: a page's K and V tiles go to shared memory; thread (key, head slice) forms the scores;
// one warp per head updates maximum and sum; thread d accumulates p v for all heads.
// ---------------------------------------------------------------------------------
#define QWB_POOL_GT 8      // query heads per block

__device__ __forceinline__ void pool_cp16(void* dst, const void* src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src));
}

// rows [first, end) of run `run` in its source (source 0: block rows, 1: tokens); empty if first >= end
__device__ __forceinline__ void pool_run_rows(int len, int window, int pool, int block_runs, int run, int* source, int* first, int* end) {
    constexpr int RUN = QWB_POOL_RUN_PAGES * QWB_POOL_PAGE;
    if (run < block_runs) {
        *source = 0;
        *first = run * RUN;
        *end = min(blocks_seen(len - 1, window, pool), (run + 1) * RUN);
    } else {
        const int w = run - block_runs;
        const int k_lo = window > 0 ? max(0, len - window) : 0;
        const int page_lo = k_lo / QWB_POOL_PAGE;
        *source = 1;
        *first = max(k_lo, (page_lo + w * QWB_POOL_RUN_PAGES) * QWB_POOL_PAGE);
        *end = min(len, (page_lo + (w + 1) * QWB_POOL_RUN_PAGES) * QWB_POOL_PAGE);
    }
}

template <typename T>
__global__ void pool_decode_kernel(const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                                   const T* __restrict__ pk_pool, const T* __restrict__ pv_pool, const int* __restrict__ page_table,
                                   const int* __restrict__ block_table, const int* __restrict__ seq_len, float* __restrict__ part_acc,
                                   float* __restrict__ part_m, float* __restrict__ part_l, int H, int G, int dim, int vdim,
                                   int table_width, float scale, int window, int pool, int block_runs, int n_runs) {
    pdl_wait();
    pdl_launch_dependents();
    constexpr int GT = QWB_POOL_GT, VEC = Vec16<T>::N, PG = QWB_POOL_PAGE;
    const int b = blockIdx.z, run = blockIdx.x;
    const int len = seq_len[b];
    int source, row_first, row_end;
    pool_run_rows(len, window, pool, block_runs, run, &source, &row_first, &row_end);
    if (row_first >= row_end) return;

    const int QG = H / G, slices = (QG + GT - 1) / GT;
    const int g = blockIdx.y / slices, g0 = (blockIdx.y % slices) * GT;
    const int gcount = min(GT, QG - g0);
    const int h0 = g * QG + g0;                         // first query head of this block

    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int kld = dim + VEC;                          // a key row and 16 bytes: rows start in different banks
    T* Kt = reinterpret_cast<T*>(smem_raw);             // [PG][dim + VEC]
    T* Vt = Kt + (size_t)PG * kld;                      // [PG][vdim]
    float* qs = reinterpret_cast<float*>(Vt + (size_t)PG * vdim);   // [GT][dim], scaled
    float* sc = qs + GT * dim;                          // [GT][PG]
    float* m_s = sc + GT * PG;                          // [GT]
    float* l_s = m_s + GT;
    float* a_s = l_s + GT;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int idx = tid; idx < GT * dim; idx += blockDim.x) {
        const int gi = idx / dim, d = idx - gi * dim;
        qs[idx] = gi < gcount ? to_f32(q[((size_t)b * H + h0 + gi) * dim + d]) * scale : 0.f;
    }
    if (tid < GT) { m_s[tid] = -INFINITY; l_s[tid] = 0.f; a_s[tid] = 1.f; }

    float acc[GT][2];
#pragma unroll
    for (int gi = 0; gi < GT; ++gi) acc[gi][0] = acc[gi][1] = 0.f;

    const T* kp = source ? k_pool : pk_pool;
    const T* vp = source ? v_pool : pv_pool;
    const int* pages = (source ? page_table : block_table) + (size_t)b * table_width;
    const int key_slices = blockDim.x / PG;                           // threads per key
    const int my_key = tid % PG, my_slice = tid / PG;
    const int nchunk = dim / VEC;

    for (int base = (row_first / PG) * PG; base < row_end; base += PG) {
        const int n_keys = min(PG, row_end - base);                   // rows of this page up to the run's end
        const size_t tile = (size_t)pages[base / PG] * G + g;
        __syncthreads();                                              // the last page's tiles are no longer read
        {   // asynchronous copies: all of a thread's pieces are in flight together (loads through registers in a loop wait
            // for one another: 16 round trips to memory a page)
            const uint4* ksrc = reinterpret_cast<const uint4*>(kp + tile * PG * dim);
            const uint4* vsrc = reinterpret_cast<const uint4*>(vp + tile * PG * vdim);
            uint4* kdst = reinterpret_cast<uint4*>(Kt);
            uint4* vdst = reinterpret_cast<uint4*>(Vt);
            for (int i = tid; i < n_keys * nchunk; i += blockDim.x) pool_cp16(kdst + i + i / nchunk, ksrc + i);    // row r starts at r * (nchunk + 1)
            for (int i = tid; i < n_keys * vdim / VEC; i += blockDim.x) pool_cp16(vdst + i, vsrc + i);
            asm volatile("cp.async.commit_group;" ::: "memory");
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();

        if (my_slice < key_slices && my_key < n_keys) {
            float s[GT];
#pragma unroll
            for (int gi = 0; gi < GT; ++gi) s[gi] = 0.f;
            const Vec16<T>* krow = reinterpret_cast<const Vec16<T>*>(Kt + (size_t)my_key * kld);
            for (int ch = 0; ch < nchunk; ++ch) {                     // every lane the same piece of q: one broadcast read
                float kf[VEC];
                krow[ch].get(kf);
#pragma unroll
                for (int gi = 0; gi < GT; ++gi) {
                    const int gq = my_slice + gi * key_slices;
                    if (gq < gcount) {
                        const float* qg = qs + gq * dim + ch * VEC;
#pragma unroll
                        for (int e = 0; e < VEC; ++e) s[gi] += qg[e] * kf[e];
                    }
                }
            }
            const bool ok = base + my_key >= row_first;
#pragma unroll
            for (int gi = 0; gi < GT; ++gi) {
                const int gq = my_slice + gi * key_slices;
                if (gq < gcount) sc[gq * PG + my_key] = ok ? s[gi] : -INFINITY;
            }
        }
        __syncthreads();

        for (int gq = warp; gq < gcount; gq += (blockDim.x >> 5)) {
            float mx = -INFINITY;
            for (int j = lane; j < n_keys; j += 32) mx = fmaxf(mx, sc[gq * PG + j]);
            mx = warp_max(mx);
            const float m_old = m_s[gq], m_new = fmaxf(m_old, mx);
            float sum = 0.f;
            for (int j = lane; j < n_keys; j += 32) {
                const float sj = sc[gq * PG + j];
                const float pj = (m_new == -INFINITY || sj == -INFINITY) ? 0.f : expf(sj - m_new);
                sc[gq * PG + j] = pj;
                sum += pj;
            }
            sum = warp_sum(sum);
            if (lane == 0) {
                const float alpha = m_new == -INFINITY ? 1.f : expf(m_old - m_new);
                a_s[gq] = alpha;
                l_s[gq] = l_s[gq] * alpha + sum;
                m_s[gq] = m_new;
            }
        }
        __syncthreads();

#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const int d = tid + c * 128;
            if (d < vdim) {
#pragma unroll
                for (int gi = 0; gi < GT; ++gi) if (gi < gcount) acc[gi][c] *= a_s[gi];
                for (int j = 0; j < n_keys; ++j) {
                    const float v = to_f32(Vt[(size_t)j * vdim + d]);
#pragma unroll
                    for (int gi = 0; gi < GT; ++gi) if (gi < gcount) acc[gi][c] += sc[gi * PG + j] * v;
                }
            }
        }
    }
    __syncthreads();

#pragma unroll
    for (int c = 0; c < 2; ++c) {
        const int d = tid + c * 128;
        if (d >= vdim) continue;
#pragma unroll
        for (int gi = 0; gi < GT; ++gi)
            if (gi < gcount) part_acc[(((size_t)b * H + h0 + gi) * n_runs + run) * vdim + d] = acc[gi][c];
    }
    if (tid < gcount) {
        const size_t at = ((size_t)b * H + h0 + tid) * n_runs + run;
        part_m[at] = m_s[tid];
        part_l[at] = l_s[tid];
    }
}

// out = sum_r acc_r e^(m_r - M) / sum_r l_r e^(m_r - M), M = max_r m_r, over the runs that hold rows, in index order; then
// each head's output is turned back by the query's position.  grid (H, B).
template <typename T>
__global__ void pool_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_m, const float* __restrict__ part_l,
                                  const int* __restrict__ seq_len, const float* __restrict__ cos_v, const float* __restrict__ sin_v,
                                  T* __restrict__ out, int H, int vdim, int window, int pool, int block_runs, int n_runs, int interleaved) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float row[QWB_POOL_MAX_DIM];
    const int h = blockIdx.x, b = blockIdx.y;
    const int len = seq_len[b];
    const size_t at = ((size_t)b * H + h) * n_runs;
    float M = -INFINITY;
    for (int r = 0; r < n_runs; ++r) {
        int source, first, end;
        pool_run_rows(len, window, pool, block_runs, r, &source, &first, &end);
        if (first < end) M = fmaxf(M, part_m[at + r]);
    }
    float L = 0.f;
    for (int r = 0; r < n_runs; ++r) {
        int source, first, end;
        pool_run_rows(len, window, pool, block_runs, r, &source, &first, &end);
        if (first < end) L += part_l[at + r] * expf(part_m[at + r] - M);
    }
    for (int d = threadIdx.x; d < vdim; d += blockDim.x) {
        float a = 0.f;
        for (int r = 0; r < n_runs; ++r) {
            int source, first, end;
            pool_run_rows(len, window, pool, block_runs, r, &source, &first, &end);
            if (first < end) a += part_acc[(at + r) * vdim + d] * expf(part_m[at + r] - M);
        }
        row[d] = a / L;
    }
    __syncthreads();
    for (int d = threadIdx.x; d < vdim; d += blockDim.x)
        out[((size_t)b * H + h) * vdim + d] =
            from_f32<T>(cos_v ? turned(row, d, vdim, cos_v + (size_t)b * (vdim >> 1), sin_v + (size_t)b * (vdim >> 1), interleaved, -1.f) : row[d]);
}

// Runs for sequences of up to max_len tokens: runs of block rows, then runs of the window's pages.
extern "C" int qwb_pool_decode_runs(int max_len, int window, int pool, int* block_runs) {
    const int run = QWB_POOL_RUN_PAGES * QWB_POOL_PAGE;
    int rows = (window > 0 && pool > 0 && max_len - window >= pool) ? (max_len - window) / pool : 0;
    *block_runs = (rows + run - 1) / run;
    // a window of `window` keys touches at most ceil(window / 64) + 1 pages, counted from its first key's page
    const int pages = window > 0 ? (window + QWB_POOL_PAGE - 1) / QWB_POOL_PAGE + 1 : (max_len + QWB_POOL_PAGE - 1) / QWB_POOL_PAGE;
    return *block_runs + (pages + QWB_POOL_RUN_PAGES - 1) / QWB_POOL_RUN_PAGES;
}

extern "C" long long qwb_pool_decode_scratch_floats(int B, int H, int vdim, int n_runs) {
    return (long long)B * H * n_runs * (vdim + 2);
}

template <typename T>
static int launch_pool_decode(const void* q, const void* k_pool, const void* v_pool, const void* pk_pool, const void* pv_pool,
                              const int* page_table, const int* block_table, const int* seq_len, const float* cos_v, const float* sin_v,
                              float* scratch, void* out, int B, int H, int G, int dim, int vdim, int table_width, float scale, int window,
                              int pool, int block_runs, int n_runs, int interleaved, cudaStream_t stream) {
    constexpr int GT = QWB_POOL_GT, PG = QWB_POOL_PAGE;
    const size_t smem = (size_t)PG * (dim + vdim) * sizeof(T) + (size_t)PG * 16 + ((size_t)GT * dim + GT * PG + 3 * GT) * sizeof(float);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(pool_decode_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return qwb_fail(QWB_ERR_CUDA, "pool_decode: %s", cudaGetErrorString(e));
    }
    float* part_acc = scratch;
    float* part_m = scratch + (size_t)B * H * n_runs * vdim;
    float* part_l = part_m + (size_t)B * H * n_runs;
    const int QG = H / G, slices = (QG + GT - 1) / GT;
    qwb_launch(pool_decode_kernel<T>, dim3(n_runs, G * slices, B), 128, smem, stream, (const T*)q, (const T*)k_pool, (const T*)v_pool,
               (const T*)pk_pool, (const T*)pv_pool, page_table, block_table, seq_len, part_acc, part_m, part_l, H, G, dim, vdim, table_width,
               scale, window, pool, block_runs, n_runs);
    if (int rc = qwb_check_launch("pool_decode")) return rc;
    qwb_launch(pool_merge_kernel<T>, dim3(H, B), 128, 0, stream, (const float*)part_acc, (const float*)part_m, (const float*)part_l, seq_len,
               cos_v, sin_v, (T*)out, H, vdim, window, pool, block_runs, n_runs, interleaved);
    return qwb_check_launch("pool_merge");
}

// q [B, H, dim]; seq_len [B] counts the new token; out [B, H * vdim]; cos_v, sin_v [B, vdim / 2] or null; scratch holds
// qwb_pool_decode_scratch_floats floats; block_runs and n_runs from qwb_pool_decode_runs for a bound on the lengths.
extern "C" int qwb_pool_decode(const void* q, const void* k_pool, const void* v_pool, const void* pk_pool, const void* pv_pool,
                               const int* page_table, const int* block_table, const int* seq_len, const float* cos_v, const float* sin_v,
                               float* scratch, void* out, int dtype, int B, int H, int G, int dim, int vdim, int table_width, float scale,
                               int window, int pool, int block_runs, int n_runs, int interleaved, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (int rc = check_pool_sizes("pool_decode", H, G, dim, vdim, table_width, window, pool)) return rc;
    if (n_runs <= 0 || block_runs < 0 || block_runs >= n_runs) return qwb_fail(QWB_ERR_ARG, "pool_decode: %d runs, %d of them of block rows", n_runs, block_runs);
    if (block_runs > 0 && (!pk_pool || !pv_pool || !block_table)) return qwb_fail(QWB_ERR_ARG, "pool_decode: blocks without their pools");
    if (B > 65535 || H > 65535) return qwb_fail(QWB_ERR_ARG, "pool_decode: batch %d or heads %d above 65535", B, H);
    if (dtype == QWB_DT_F32)
        return launch_pool_decode<float>(q, k_pool, v_pool, pk_pool, pv_pool, page_table, block_table, seq_len, cos_v, sin_v, scratch, out, B, H,
                                         G, dim, vdim, table_width, scale, window, pool, block_runs, n_runs, interleaved, stream);
    if (dtype == QWB_DT_BF16)
        return launch_pool_decode<bf16>(q, k_pool, v_pool, pk_pool, pv_pool, page_table, block_table, seq_len, cos_v, sin_v, scratch, out, B, H,
                                        G, dim, vdim, table_width, scale, window, pool, block_runs, n_runs, interleaved, stream);
    return qwb_fail(QWB_ERR_ARG, "pool_decode: unknown dtype %d", dtype);
}
