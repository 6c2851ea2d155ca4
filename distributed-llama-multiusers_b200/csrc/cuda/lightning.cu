// Linear attention with a fixed decay per head ("lightning" attention).  Per head, with q_t, k_t in R^dim and v_t in
// R^vdim (already activated) and a constant 0 <= decay_h <= 1:
//     S <- lambda S + k (x) v     (outer product)      S: [dim][vdim], f32, one per sequence slot and head, lambda = decay_h
//     y  = S^T q                  (with the S just updated)
// Everything here is f32: the state, the scores inside a chunk, the powers of the decay.  A batch is any mix of
// sequences with one or more consecutive rows each (DlMambaBatch); a sequence whose first row is position 0 starts from
// zeros whatever its slot held.
//
// Two forms.  Token by token (decoding, short portions): one CTA per (sequence, head, slab of 64 state columns), the
// slab in shared memory, the rows' q and k staged a few tokens at a time.  Chunked (long portions): a sequence's rows are cut into chunks of
// LC = 64 rows, counted from the portion's first row, and unrolled as
//     y_i = sum_{j <= i in chunk} decay^(i-j) (q_i . k_j) v_j  +  decay^(i+1) P^T q_i        i, j: offsets in the chunk
//     P   = the state before the chunk;  state after it = decay^len P + sum_j decay^(len-1-j) k_j v_j^T
// in three launches: every chunk's own sum, the prefix over a sequence's chunks (which also leaves the slot's new
// state), then the outputs.  Only non-negative powers of the decay are ever formed, so a fast decay cannot overflow.
#include "layer_common.cuh"
#include "../../../include/dllama_b200.h"

#define LT_TB 8                 // tokens staged per barrier pair of the token-by-token kernel
#define LC DL_LIGHTNING_CHUNK

__device__ __forceinline__ float decay_pow(float log_decay, int n) { return n == 0 ? 1.f : expf((float)n * log_decay); }

// ------------------------------------------------------------------------------------------------
// token by token
// ------------------------------------------------------------------------------------------------
// grid (sequence, head, column slab): the columns of S are independent of one another, so a CTA keeps LT_COLS of them
// (thread = column) and every slab of a head runs in parallel
#define LT_COLS 64
__global__ void __launch_bounds__(LT_COLS) lightning_scan_kernel(DlMambaBatch b, DlLightningArgs a) {
    extern __shared__ float sm[];
    const int n = blockIdx.x, h = blockIdx.y, c = blockIdx.z * LT_COLS + threadIdx.x;
    const int D = a.dim, V = a.vdim, H = a.n_heads;
    float* S = sm;                              // [D][LT_COLS]
    float* qs = S + (size_t)D * LT_COLS;        // [LT_TB][D]
    float* ks = qs + LT_TB * D;                 // [LT_TB][D]
    float* Sg = a.state + ((size_t)b.seq_slot[n] * H + h) * D * V;
    const bool fresh = b.seq_pos0[n] == 0, live = c < V;
    if (live)
        for (int d = 0; d < D; ++d) S[d * LT_COLS + threadIdx.x] = fresh ? 0.f : Sg[(size_t)d * V + c];
    const float decay = a.decay[h];
    const int r0 = b.seq_start[n], r1 = b.seq_start[n + 1];
    for (int rb = r0; rb < r1; rb += LT_TB) {
        const int nt = min(LT_TB, r1 - rb);
        __syncthreads();
        for (int i = threadIdx.x; i < nt * D; i += LT_COLS) {
            const int t = i / D, d = i - t * D;
            const int row = b.seq_rows[rb + t];
            qs[i] = a.q[(size_t)row * a.ldq + h * D + d];
            ks[i] = a.k[(size_t)row * a.ldk + h * D + d];
        }
        __syncthreads();
        if (!live) continue;
        for (int t = 0; t < nt; ++t) {
            const int row = b.seq_rows[rb + t];
            const float v = a.v[(size_t)row * a.ldv + h * V + c];
            const float* q = qs + t * D;
            const float* k = ks + t * D;
            float y0 = 0.f, y1 = 0.f;
            int d = 0;
            for (; d + 1 < D; d += 2) {
                const float s0 = fmaf(decay, S[d * LT_COLS + threadIdx.x], k[d] * v);
                const float s1 = fmaf(decay, S[(d + 1) * LT_COLS + threadIdx.x], k[d + 1] * v);
                S[d * LT_COLS + threadIdx.x] = s0;
                S[(d + 1) * LT_COLS + threadIdx.x] = s1;
                y0 = fmaf(s0, q[d], y0);
                y1 = fmaf(s1, q[d + 1], y1);
            }
            if (d < D) {
                const float s0 = fmaf(decay, S[d * LT_COLS + threadIdx.x], k[d] * v);
                S[d * LT_COLS + threadIdx.x] = s0;
                y0 = fmaf(s0, q[d], y0);
            }
            a.y[(size_t)row * a.ld_y + h * V + c] = y0 + y1;
        }
    }
    if (live)
        for (int d = 0; d < D; ++d) Sg[(size_t)d * V + c] = S[d * LT_COLS + threadIdx.x];
}

static int lightning_args_ok(const DlLightningArgs& a, const char* who) {
    if (a.n_heads < 1 || a.dim < 1 || a.vdim < 1) { dl_set_error("%s: bad shape (heads %d, dim %d, vdim %d)", who, a.n_heads, a.dim, a.vdim); return -1; }
    return 0;
}

// The same with the state in registers, for dim <= 4 * NR: a CTA owns LR_COLS columns of one head's S; thread (column, dq)
// keeps rows dq, dq + 4, ... of its column (NR registers), the four threads of a column are neighbouring lanes and sum
// their shares of y by two shuffles.  Many small CTAs: a decode step of one sequence still fills heads * vdim / 32 of them.
#define LR_COLS 32
template <int NR>
__global__ void __launch_bounds__(LR_COLS * 4) lightning_scan_reg_kernel(DlMambaBatch b, DlLightningArgs a) {
    extern __shared__ float sm[];
    const int n = blockIdx.x, h = blockIdx.y, dq = threadIdx.x & 3, c = blockIdx.z * LR_COLS + (threadIdx.x >> 2);
    const int D = a.dim, V = a.vdim, H = a.n_heads;
    float* qs = sm;                             // [LT_TB][D]
    float* ks = qs + LT_TB * D;                 // [LT_TB][D]
    float* Sg = a.state + ((size_t)b.seq_slot[n] * H + h) * D * V;
    const bool fresh = b.seq_pos0[n] == 0, live = c < V;
    float s[NR];
#pragma unroll
    for (int i = 0; i < NR; ++i) {
        const int d = i * 4 + dq;
        s[i] = (live && !fresh && d < D) ? Sg[(size_t)d * V + c] : 0.f;
    }
    const float decay = a.decay[h];
    const int r0 = b.seq_start[n], r1 = b.seq_start[n + 1];
    for (int rb = r0; rb < r1; rb += LT_TB) {
        const int nt = min(LT_TB, r1 - rb);
        __syncthreads();
        for (int i = threadIdx.x; i < nt * D; i += LR_COLS * 4) {
            const int t = i / D, d = i - t * D;
            const int row = b.seq_rows[rb + t];
            qs[i] = a.q[(size_t)row * a.ldq + h * D + d];
            ks[i] = a.k[(size_t)row * a.ldk + h * D + d];
        }
        __syncthreads();
        for (int t = 0; t < nt; ++t) {
            const int row = b.seq_rows[rb + t];
            const float v = live ? a.v[(size_t)row * a.ldv + h * V + c] : 0.f;
            const float* q = qs + t * D;
            const float* k = ks + t * D;
            float y0 = 0.f, y1 = 0.f;
#pragma unroll
            for (int i = 0; i < NR; i += 2) {
                const int d = i * 4 + dq;
                if (d < D) { s[i] = fmaf(decay, s[i], k[d] * v); y0 = fmaf(s[i], q[d], y0); }
                if (d + 4 < D) { s[i + 1] = fmaf(decay, s[i + 1], k[d + 4] * v); y1 = fmaf(s[i + 1], q[d + 4], y1); }
            }
            float y = y0 + y1;
            y += __shfl_xor_sync(0xffffffffu, y, 1);
            y += __shfl_xor_sync(0xffffffffu, y, 2);
            if (live && dq == 0) a.y[(size_t)row * a.ld_y + h * V + c] = y;
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < NR; ++i) {
            const int d = i * 4 + dq;
            if (d < D) Sg[(size_t)d * V + c] = s[i];
        }
    }
}

extern "C" int dl_lightning_scan(const DlMambaBatch* batch, int n_seq, const DlLightningArgs* args, void* stream) {
    const DlLightningArgs& a = *args;
    if (lightning_args_ok(a, "dl_lightning_scan")) return -1;
    if (n_seq < 1) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (a.dim <= 256) {                        // the state in registers
        const size_t smem = 2 * (size_t)LT_TB * a.dim * sizeof(float);
        dim3 grid(n_seq, a.n_heads, (a.vdim + LR_COLS - 1) / LR_COLS);
        if (a.dim <= 32) lightning_scan_reg_kernel<8><<<grid, LR_COLS * 4, smem, st>>>(*batch, a);
        else if (a.dim <= 64) lightning_scan_reg_kernel<16><<<grid, LR_COLS * 4, smem, st>>>(*batch, a);
        else if (a.dim <= 128) lightning_scan_reg_kernel<32><<<grid, LR_COLS * 4, smem, st>>>(*batch, a);
        else lightning_scan_reg_kernel<64><<<grid, LR_COLS * 4, smem, st>>>(*batch, a);
        LAYER_CHECK_LAUNCH("dl_lightning_scan");
        return 0;
    }
    const size_t smem = ((size_t)a.dim * LT_COLS + 2 * (size_t)LT_TB * a.dim) * sizeof(float);
    if (smem > 227 * 1024) { dl_set_error("dl_lightning_scan: dim %d does not fit shared memory", a.dim); return -1; }
    cudaError_t e = cudaFuncSetAttribute(lightning_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { dl_set_error("dl_lightning_scan: shared memory attribute: %s", cudaGetErrorString(e)); return -(int)e; }
    lightning_scan_kernel<<<dim3(n_seq, a.n_heads, (a.vdim + LT_COLS - 1) / LT_COLS), LT_COLS, smem, st>>>(*batch, a);
    LAYER_CHECK_LAUNCH("dl_lightning_scan");
    return 0;
}

// ------------------------------------------------------------------------------------------------
// chunked.  Chunk c of sequence n covers rows seq_start[n] + c LC .. of the batch; its scratch slot is
// seq_start[n] / LC + n + c (the sequences before n use at most seq_start[n] / LC + n slots).  256 threads;
// thread t = (tb, cb) = (t / 16, t % 16) owns output columns cb, cb + 16, ... and rows tb-wise (see each kernel).
// ------------------------------------------------------------------------------------------------
#define LC_THREADS 256

__device__ __forceinline__ bool chunk_of(const DlMambaBatch& b, int n, int c, int& row0, int& len, int& slot_idx) {
    const int s0 = b.seq_start[n], total = b.seq_start[n + 1] - s0;
    if (c * LC >= total) return false;
    row0 = s0 + c * LC;
    len = min(LC, total - c * LC);
    slot_idx = s0 / LC + n + c;
    return true;
}

// pass 1: scratch[chunk][h] = sum_j decay^(len-1-j) k_j v_j^T
__global__ void __launch_bounds__(LC_THREADS) lightning_chunk_state_kernel(DlMambaBatch b, DlLightningArgs a, float* __restrict__ scratch) {
    extern __shared__ float sm[];
    const int n = blockIdx.x, c = blockIdx.y, h = blockIdx.z;
    int row0, len, ci;
    if (!chunk_of(b, n, c, row0, len, ci)) return;
    const int D = a.dim, V = a.vdim, H = a.n_heads;
    float* ks = sm;                             // [LC][D], already weighted
    float* vs = ks + (size_t)LC * D;            // [LC][V]
    const float logd = logf(a.decay[h]);
    for (int i = threadIdx.x; i < LC * D; i += LC_THREADS) {
        const int j = i / D, d = i - j * D;
        ks[i] = j < len ? a.k[(size_t)b.seq_rows[row0 + j] * a.ldk + h * D + d] * decay_pow(logd, len - 1 - j) : 0.f;
    }
    for (int i = threadIdx.x; i < LC * V; i += LC_THREADS) {
        const int j = i / V, cc = i - j * V;
        vs[i] = j < len ? a.v[(size_t)b.seq_rows[row0 + j] * a.ldv + h * V + cc] : 0.f;
    }
    __syncthreads();
    float* out = scratch + ((size_t)ci * H + h) * D * V;
    const int tb = threadIdx.x >> 4, cb = threadIdx.x & 15;
    for (int d0 = 0; d0 < D; d0 += 128) {
        for (int c0 = 0; c0 < V; c0 += 128) {
            float acc[8][8];
#pragma unroll
            for (int r = 0; r < 8; ++r)
#pragma unroll
                for (int u = 0; u < 8; ++u) acc[r][u] = 0.f;
            for (int j = 0; j < len; ++j) {
                float kv[8], vv[8];
#pragma unroll
                for (int r = 0; r < 8; ++r) { const int d = d0 + tb + 16 * r; kv[r] = d < D ? ks[j * D + d] : 0.f; }
#pragma unroll
                for (int u = 0; u < 8; ++u) { const int cc = c0 + cb + 16 * u; vv[u] = cc < V ? vs[j * V + cc] : 0.f; }
#pragma unroll
                for (int r = 0; r < 8; ++r)
#pragma unroll
                    for (int u = 0; u < 8; ++u) acc[r][u] = fmaf(kv[r], vv[u], acc[r][u]);
            }
#pragma unroll
            for (int r = 0; r < 8; ++r)
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int d = d0 + tb + 16 * r, cc = c0 + cb + 16 * u;
                    if (d < D && cc < V) out[(size_t)d * V + cc] = acc[r][u];
                }
        }
    }
}

// pass 2: over a sequence's chunks in order, scratch[chunk] <- the state BEFORE the chunk; the slot gets the state after
// the last one.  One thread per state element.
__global__ void __launch_bounds__(256) lightning_chunk_prefix_kernel(DlMambaBatch b, DlLightningArgs a, float* __restrict__ scratch) {
    const int n = blockIdx.x, h = blockIdx.y;
    const int D = a.dim, V = a.vdim, H = a.n_heads;
    const int e = blockIdx.z * blockDim.x + threadIdx.x;
    if (e >= D * V) return;
    const int s0 = b.seq_start[n], total = b.seq_start[n + 1] - s0;
    float* Sg = a.state + ((size_t)b.seq_slot[n] * H + h) * D * V + e;
    const float logd = logf(a.decay[h]);
    float R = b.seq_pos0[n] == 0 ? 0.f : *Sg;
    const int nc = (total + LC - 1) / LC;
    const float full = decay_pow(logd, LC);
    float* p0 = scratch + ((size_t)(s0 / LC + n) * H + h) * D * V + e;
    const size_t step = (size_t)H * D * V;
    for (int c0 = 0; c0 < nc; c0 += 8) {          // eight chunks' sums are loaded together, then chained
        float own[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) own[i] = c0 + i < nc ? p0[(size_t)(c0 + i) * step] : 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int c = c0 + i;
            if (c < nc) {
                p0[(size_t)c * step] = R;
                R = fmaf(c == nc - 1 ? decay_pow(logd, total - c * LC) : full, R, own[i]);
            }
        }
    }
    *Sg = R;
}

// pass 3: the outputs of a chunk
__global__ void __launch_bounds__(LC_THREADS) lightning_chunk_out_kernel(DlMambaBatch b, DlLightningArgs a, const float* __restrict__ scratch) {
    extern __shared__ float sm[];
    const int n = blockIdx.x, c = blockIdx.y, h = blockIdx.z;
    int row0, len, ci;
    if (!chunk_of(b, n, c, row0, len, ci)) return;
    const int D = a.dim, V = a.vdim, H = a.n_heads, DP = D + 1;
    float* qs = sm;                             // [LC][D + 1]
    float* ks = qs + (size_t)LC * DP;           // [LC][D + 1]
    float* vs = ks + (size_t)LC * max(DP, 128); // [LC][V]
    float* A = vs + (size_t)LC * V;             // [LC][LC + 1]
    const float logd = logf(a.decay[h]);
    for (int i = threadIdx.x; i < LC * D; i += LC_THREADS) {
        const int j = i / D, d = i - j * D;
        float qv = 0.f, kv = 0.f;
        if (j < len) {
            const size_t row = (size_t)b.seq_rows[row0 + j];
            qv = a.q[row * a.ldq + h * D + d];
            kv = a.k[row * a.ldk + h * D + d];
        }
        qs[j * DP + d] = qv;
        ks[j * DP + d] = kv;
    }
    for (int i = threadIdx.x; i < LC * V; i += LC_THREADS) {
        const int j = i / V, cc = i - j * V;
        vs[i] = j < len ? a.v[(size_t)b.seq_rows[row0 + j] * a.ldv + h * V + cc] : 0.f;
    }
    __syncthreads();
    const int tb = threadIdx.x >> 4, cb = threadIdx.x & 15;
    {   // A[i][j] = decay^(i-j) q_i . k_j for j <= i, rows i = tb * 4 + r, columns j = cb * 4 + u
        float acc[4][4];
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int u = 0; u < 4; ++u) acc[r][u] = 0.f;
        if (cb <= tb) {
            for (int d = 0; d < D; ++d) {
                float qv[4], kv[4];
#pragma unroll
                for (int r = 0; r < 4; ++r) qv[r] = qs[(tb * 4 + r) * DP + d];
#pragma unroll
                for (int u = 0; u < 4; ++u) kv[u] = ks[(cb * 4 + u) * DP + d];
#pragma unroll
                for (int r = 0; r < 4; ++r)
#pragma unroll
                    for (int u = 0; u < 4; ++u) acc[r][u] = fmaf(qv[r], kv[u], acc[r][u]);
            }
        }
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = tb * 4 + r, j = cb * 4 + u;
                A[i * (LC + 1) + j] = j <= i ? acc[r][u] * decay_pow(logd, i - j) : 0.f;
            }
    }
    __syncthreads();
    const float* P = scratch + ((size_t)ci * H + h) * D * V;
    float* Ps = ks;                             // [LC][128]: LC rows of the carried state, in the keys' place
    float carry[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) carry[r] = decay_pow(logd, tb * 4 + r + 1);
    for (int c0 = 0; c0 < V; c0 += 128) {
        const int cw = min(128, V - c0);
        float acc[4][8], pacc[4][8];
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int u = 0; u < 8; ++u) acc[r][u] = pacc[r][u] = 0.f;
        const int jmax = min(len, tb * 4 + 4);
        for (int j = 0; j < jmax; ++j) {
            float av[4], vv[8];
#pragma unroll
            for (int r = 0; r < 4; ++r) av[r] = A[(tb * 4 + r) * (LC + 1) + j];
#pragma unroll
            for (int u = 0; u < 8; ++u) { const int cc = c0 + cb + 16 * u; vv[u] = cc < V ? vs[j * V + cc] : 0.f; }
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int u = 0; u < 8; ++u) acc[r][u] = fmaf(av[r], vv[u], acc[r][u]);
        }
        for (int d0 = 0; d0 < D; d0 += LC) {        // LC rows of P at a time
            const int dn = min(LC, D - d0);
            __syncthreads();                        // the scores (first pass) or the previous rows are done with
            for (int i = threadIdx.x; i < dn * 128; i += LC_THREADS) {
                const int d = i >> 7, cc = i & 127;
                Ps[i] = cc < cw ? P[(size_t)(d0 + d) * V + c0 + cc] : 0.f;
            }
            __syncthreads();
            if (tb * 4 < len) {
                for (int d = 0; d < dn; ++d) {
                    float qv[4], pv[8];
#pragma unroll
                    for (int r = 0; r < 4; ++r) qv[r] = qs[(tb * 4 + r) * DP + d0 + d];
#pragma unroll
                    for (int u = 0; u < 8; ++u) pv[u] = Ps[d * 128 + cb + 16 * u];
#pragma unroll
                    for (int r = 0; r < 4; ++r)
#pragma unroll
                        for (int u = 0; u < 8; ++u) pacc[r][u] = fmaf(qv[r], pv[u], pacc[r][u]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int i = tb * 4 + r;
            if (i >= len) continue;
            float* y = a.y + (size_t)b.seq_rows[row0 + i] * a.ld_y + h * V;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int cc = c0 + cb + 16 * u;
                if (cc < V) y[cc] = fmaf(carry[r], pacc[r][u], acc[r][u]);
            }
        }
    }
}

static size_t lightning_out_smem(int dim, int vdim) {      // the keys' region later holds LC x 128 values of the carried state
    const size_t keys = (size_t)LC * (dim + 1) > (size_t)LC * 128 ? (size_t)LC * (dim + 1) : (size_t)LC * 128;
    return ((size_t)LC * (dim + 1) + keys + (size_t)LC * vdim + (size_t)LC * (LC + 1)) * sizeof(float);
}

// 0 if the chunked kernels take these sizes
extern "C" int dl_lightning_scan_chunked_supported(int dim, int vdim) {
    return (dim >= 1 && vdim >= 1 && lightning_out_smem(dim, vdim) <= 227 * 1024) ? 0 : -1;
}

// f32 of scratch for a batch of M rows in n_seq sequences
extern "C" long long dl_lightning_chunk_floats(int M, int n_seq, int n_heads, int dim, int vdim) {
    return (long long)(M / LC + n_seq) * n_heads * dim * vdim;
}

// max_chunks: the most chunks any sequence of the batch has (ceil(longest portion / LC))
extern "C" int dl_lightning_scan_chunked(const DlMambaBatch* batch, int n_seq, int max_chunks, const DlLightningArgs* args,
                                         float* scratch, void* stream) {
    const DlLightningArgs& a = *args;
    if (lightning_args_ok(a, "dl_lightning_scan_chunked")) return -1;
    if (dl_lightning_scan_chunked_supported(a.dim, a.vdim) != 0 || scratch == nullptr) { dl_set_error("dl_lightning_scan_chunked: sizes not supported (dim %d, vdim %d)", a.dim, a.vdim); return -1; }
    if (n_seq < 1 || max_chunks < 1) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t smem1 = (size_t)LC * (a.dim + a.vdim) * sizeof(float), smem3 = lightning_out_smem(a.dim, a.vdim);
    cudaError_t e = cudaFuncSetAttribute(lightning_chunk_state_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(lightning_chunk_out_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem3);
    if (e != cudaSuccess) { dl_set_error("dl_lightning_scan_chunked: shared memory attribute: %s", cudaGetErrorString(e)); return -(int)e; }
    dim3 grid(n_seq, max_chunks, a.n_heads);
    lightning_chunk_state_kernel<<<grid, LC_THREADS, smem1, st>>>(*batch, a, scratch);
    lightning_chunk_prefix_kernel<<<dim3(n_seq, a.n_heads, (a.dim * a.vdim + 255) / 256), 256, 0, st>>>(*batch, a, scratch);
    lightning_chunk_out_kernel<<<grid, LC_THREADS, smem3, st>>>(*batch, a, scratch);
    LAYER_CHECK_LAUNCH("dl_lightning_scan_chunked");
    return 0;
}
