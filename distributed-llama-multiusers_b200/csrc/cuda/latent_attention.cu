// Latent attention: keys and values of all heads are up-projections of one small latent vector per token, plus one
// rotated key part that all heads share.  The cache holds, per token, [latent: rank | rotated key: rot] and nothing
// per head.  Attention runs in the latent space ("absorbed" form):
//     score_h(i, j) = scale * ( (U_k,h^T q_h,i) . c_j  +  qrot_h,i . krot_j )         softmax over j <= i
//     out_h(i)      = U_v,h ( sum_j p_h(i, j) c_j )
// Options: a sliding window (only i - j < window is visible; pages behind it are never read), a sink per head (one more
// term exp(sink_h) in the softmax denominator, without a value) and a gate per row and head (the head's output leaves
// multiplied by sigmoid(gate): a scalar commutes with the value up-projection that follows).
// so the per-head work against the cache is a dot product with, and a weighted sum of, the same rows for every head.
// The two per-head projections (U_k^T q before, U_v after) are batched dense products (dense.cu).
//
// Kernels here: the cache writer (RMS norm of the latent + rotary on the shared key part + paged store), rotary on
// a slice of each head of a row-major activation, and the attention itself over the paged latent cache, one CTA per
// query row with every head of the row sharing each page it stages in shared memory.  Softmax, norms and rotary
// angles are f32 (angles in f64); the cache is bf16 or f32.
#include "mma_common.cuh"
#include "../../../include/dllama_b200.h"

// rotate-half layout: dimension i pairs with i + dims/2; (u, v) -> (u cos a - v sin a, v cos a + u sin a), a = pos * f_i
__device__ __forceinline__ void rot_pair(float u, float v, int pos, double f, float& ou, float& ov) {
    double s, c;
    sincos((double)pos * f, &s, &c);
    ou = (float)((double)u * c - (double)v * s);
    ov = (float)((double)v * c + (double)u * s);
}

// ------------------------------------------------------------------------------------------------
// cache writer: row m of kv = [rank latent | rot key part]
// ------------------------------------------------------------------------------------------------
template <typename CT>
__global__ void __launch_bounds__(128) latent_kv_write_kernel(DlLatentKvArgs a) {
    __shared__ float red[32];
    const int m = blockIdx.x;
    const float* in = a.kv + (size_t)m * a.ld;
    const int pos = a.pos[m], slot = a.slot[m];
    const int page = a.block_table[(size_t)slot * a.max_pages + pos / a.page_size];
    const int D = a.rank + a.rot;
    CT* dst = (CT*)a.cache + ((size_t)page * a.page_size + pos % a.page_size) * D;
    float ss = 0.f;
    for (int i = threadIdx.x; i < a.rank; i += blockDim.x) ss = fmaf(in[i], in[i], ss);
    ss = block_sum(ss, red);
    const float inv = 1.f / sqrtf(ss / (float)a.rank + a.eps);
    for (int i = threadIdx.x; i < a.rank; i += blockDim.x) st_f(dst + i, in[i] * inv * a.norm_w[i]);
    const int half = a.rope_dims / 2;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const int iu = a.interleaved ? 2 * i : i, iv = a.interleaved ? 2 * i + 1 : i + half;
        float u, v;
        rot_pair(in[a.rank + iu], in[a.rank + iv], pos, a.freqs[i], u, v);
        st_f(dst + a.rank + iu, u);
        st_f(dst + a.rank + iv, v);
    }
    for (int i = a.rope_dims + threadIdx.x; i < a.rot; i += blockDim.x) st_f(dst + a.rank + i, in[a.rank + i]);
}

extern "C" int dl_latent_kv_write(const DlLatentKvArgs* args, int M, void* stream) {
    const DlLatentKvArgs& a = *args;
    if (a.rope_dims > a.rot || (a.rope_dims & 1)) { dl_set_error("dl_latent_kv_write: bad rotary size"); return -1; }
    cudaStream_t st = (cudaStream_t)stream;
    if (a.ctype == DL_T_BF16) latent_kv_write_kernel<__nv_bfloat16><<<M, 128, 0, st>>>(a);
    else latent_kv_write_kernel<float><<<M, 128, 0, st>>>(a);
    LAYER_CHECK_LAUNCH("dl_latent_kv_write");
    return 0;
}

// ------------------------------------------------------------------------------------------------
// rotary on dims [offset, offset + rope_dims) of each head of x[M][n_heads][head_stride], in place
// ------------------------------------------------------------------------------------------------
__global__ void rope_rows_kernel(float* x, long long ld, int n_heads, int head_stride, int offset, int rope_dims,
                                 const double* __restrict__ freqs, const int* __restrict__ pos, int interleaved, float mag) {
    const int m = blockIdx.x, half = rope_dims / 2;
    const int p = pos[m];
    for (int t = threadIdx.x; t < n_heads * half; t += blockDim.x) {
        const int h = t / half, i = t % half;
        float* q = x + (size_t)m * ld + (size_t)h * head_stride + offset;
        const int iu = interleaved ? 2 * i : i, iv = interleaved ? 2 * i + 1 : i + half;
        float u, v;
        rot_pair(q[iu], q[iv], p, freqs[i], u, v);
        q[iu] = u * mag;
        q[iv] = v * mag;
    }
}

// interleaved: dimension 2i pairs with 2i + 1 (else i with i + dims/2); mag multiplies cos and sin (1: a pure rotation)
extern "C" int dl_rope_rows(float* x, long long ld, int M, int n_heads, int head_stride, int offset, int rope_dims,
                            const double* freqs, const int* pos, int interleaved, float mag, void* stream) {
    if ((rope_dims & 1) || offset + rope_dims > head_stride) { dl_set_error("dl_rope_rows: bad rotary size"); return -1; }
    rope_rows_kernel<<<M, 128, 0, (cudaStream_t)stream>>>(x, ld, n_heads, head_stride, offset, rope_dims, freqs, pos, interleaved, mag);
    LAYER_CHECK_LAUNCH("dl_rope_rows");
    return 0;
}

// ------------------------------------------------------------------------------------------------
// attention over the paged latent cache; one CTA per query row, one page (LA_TILE tokens) per step
// ------------------------------------------------------------------------------------------------
#define LA_TILE 32

template <typename CT>
__global__ void latent_attention_kernel(DlLatentAttnArgs a) {
    extern __shared__ float sm[];
    const int m = blockIdx.x;
    const int H = a.n_heads, R = a.rank, D = a.rank + a.rot, DP = D + 1;
    const int nw = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* q_s = sm;                                  // [H][D]   absorbed query | rotated query part
    float* tile = q_s + (size_t)H * D;                // [LA_TILE][D + 1]
    float* acc = tile + (size_t)LA_TILE * DP;         // [H][R]
    float* p_s = acc + (size_t)H * R;                 // [nw][LA_TILE]
    float* ml = p_s + (size_t)nw * LA_TILE;           // [H][2]   running maximum, running sum
    const int pos = a.pos[m], slot = a.slot[m];
    for (int t = threadIdx.x; t < H * D; t += blockDim.x) {
        const int h = t / D, d = t % D;
        q_s[t] = d < R ? a.q_lat[((size_t)m * H + h) * R + d]
                       : a.q[(size_t)m * a.ldq + (size_t)h * a.q_head_stride + a.q_rot_offset + (d - R)];
    }
    for (int t = threadIdx.x; t < H * R; t += blockDim.x) acc[t] = 0.f;
    for (int t = threadIdx.x; t < H; t += blockDim.x) { ml[2 * t] = -INFINITY; ml[2 * t + 1] = 0.f; }
    const int n_tiles = pos / LA_TILE + 1;
    const int first = a.window > 0 ? max(0, pos - a.window + 1) : 0;      // oldest visible position; pages before it are never read
    for (int t = first / LA_TILE; t < n_tiles; ++t) {
        __syncthreads();                              // q_s / acc ready; previous tile consumed
        const int page = a.block_table[(size_t)slot * a.max_pages + t];
        const CT* src = (const CT*)a.cache + (size_t)page * LA_TILE * D;
        const int valid = min(LA_TILE, pos + 1 - t * LA_TILE), j_lo = max(0, first - t * LA_TILE);      // visible lines [j_lo, valid)
        for (int i = threadIdx.x; i < LA_TILE * D; i += blockDim.x) {
            const int j = i / D, d = i % D;
            tile[j * DP + d] = (j >= j_lo && j < valid) ? ld_f(src + i) : 0.f;
        }
        __syncthreads();
        for (int h = warp; h < H; h += nw) {
            const float* qh = q_s + (size_t)h * D;
            const float* row = tile + lane * DP;
            float s = 0.f;
            for (int d = 0; d < D; ++d) s = fmaf(qh[d], row[d], s);
            const bool vis = lane >= j_lo && lane < valid;
            s = vis ? s * a.scale : -INFINITY;
            const float m_old = ml[2 * h], m_new = fmaxf(m_old, warp_max(s));
            const float p = vis ? expf(s - m_new) : 0.f;
            const float alpha = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
            const float l_new = ml[2 * h + 1] * alpha + warp_sum(p);
            p_s[warp * LA_TILE + lane] = p;
            __syncwarp();
            if (lane == 0) { ml[2 * h] = m_new; ml[2 * h + 1] = l_new; }
            float* ah = acc + (size_t)h * R;
            const float* ps = p_s + warp * LA_TILE;
            for (int d = lane; d < R; d += 32) {
                float v = ah[d] * alpha;
                for (int j = j_lo; j < valid; ++j) v = fmaf(ps[j], tile[j * DP + d], v);
                ah[d] = v;
            }
            __syncwarp();
        }
    }
    __syncthreads();
    for (int t = threadIdx.x; t < H * R; t += blockDim.x) {
        const int h = t / R;
        float l = ml[2 * h + 1];
        if (a.sink) l += expf(a.sink[h] - ml[2 * h]);
        float v = acc[t] / l;
        if (a.gate) v *= sigmoid_f(a.gate[(size_t)m * a.ld_gate + h]);
        a.out[(size_t)m * H * R + t] = v;
    }
}

static size_t latent_attention_smem(int H, int rank, int rot, int nw) {
    const size_t D = (size_t)rank + rot;
    return ((size_t)H * D + (size_t)LA_TILE * (D + 1) + (size_t)H * rank + (size_t)nw * LA_TILE + 2 * (size_t)H) * sizeof(float);
}

extern "C" int dl_latent_attention(const DlLatentAttnArgs* args, int M, void* stream) {
    const DlLatentAttnArgs& a = *args;
    if (a.page_size != LA_TILE) { dl_set_error("dl_latent_attention: page size must be %d", LA_TILE); return -1; }
    const int nw = a.n_heads < 8 ? a.n_heads : 8;
    const size_t smem = latent_attention_smem(a.n_heads, a.rank, a.rot, nw);
    if (smem > 227 * 1024) { dl_set_error("dl_latent_attention: %d heads x rank %d need %zu bytes of shared memory", a.n_heads, a.rank, smem); return -1; }
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    if (a.ctype == DL_T_BF16) {
        e = cudaFuncSetAttribute(latent_attention_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) latent_attention_kernel<__nv_bfloat16><<<M, nw * 32, smem, st>>>(a);
    } else {
        e = cudaFuncSetAttribute(latent_attention_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) latent_attention_kernel<float><<<M, nw * 32, smem, st>>>(a);
    }
    if (e != cudaSuccess) { dl_set_error("dl_latent_attention: shared memory attribute: %s", cudaGetErrorString(e)); return -(int)e; }
    LAYER_CHECK_LAUNCH("dl_latent_attention");
    return 0;
}

// ------------------------------------------------------------------------------------------------
// Tensor-core variant (bf16 cache): a CTA owns a tile of up to 16 * NI (32 or 64) "query rows x heads" of one sequence
// (consecutive positions x all heads: every head reads the same cache lines, so heads stack on the M dimension of
// the MMA) and walks the sequence's pages.  Per page (32 tokens):
//     S[32 x 32]  = Q[32 x D] . C[32 x D]^T        each of the NJ column-warps takes D / NJ of the K dimension;
//                                                  the partial products meet in shared memory
//     softmax     (f32, online; every warp of a row tile redoes the cheap 16 x 32 part)
//     O[32 x R]  += P[32 x 32] . C[32 x R]         each column-warp owns R / NJ output columns in registers
// Warps: NI row tiles of 16 x NJ column-warps.  mma.sync m16n8k16 bf16; B fragments of P.C by ldmatrix.trans.
// Pages arrive by cp.async into two buffers: page k + 1 is in flight while page k is multiplied.
// With `n_splits` > 1 (decode: few tiles, long contexts) CTAs along grid.y take page ranges and leave unnormalised
// partial sums that latent_merge_kernel combines.
// ------------------------------------------------------------------------------------------------
#define LQ_MAX_ROWS 64
#define LQ_NJ 4
#define LQ_SP_LD 34                       // even: partial scores move as float2

// NT: n-tiles (8 columns) of O per column-warp; the kernel covers rank <= NT * 8 * LQ_NJ.  NI: row tiles of 16.
template <int NT, int NI>
__global__ void __launch_bounds__(32 * LQ_NJ * NI) latent_attention_mma_kernel(DlLatentAttnArgs a, DlLatentTiles tl) {
    constexpr int LQ_ROWS = 16 * NI, LQ_THREADS = 32 * LQ_NJ * NI;
    extern __shared__ __align__(16) uint8_t smraw[];
    const int H = a.n_heads, R = a.rank, D = a.rank + a.rot;
    const int Dp = tl.d_pad, LD = Dp + 8;                 // row stride in bf16: 16-byte multiple, conflict-free
    __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smraw);         // [LQ_ROWS][LD]
    __nv_bfloat16* c_buf = q_s + LQ_ROWS * LD;                            // [2][32][LD]
    float* sp = reinterpret_cast<float*>(c_buf + 2 * 32 * LD);            // [NI][LQ_NJ][16][LQ_SP_LD]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wi = warp / LQ_NJ, wj = warp % LQ_NJ, g = lane >> 2, t = lane & 3;
    const int tile = tl.n_tiles - 1 - blockIdx.x, split = blockIdx.y;   // a sequence's later tiles walk more pages: start them first
    const int* trows = tl.tile_rows + (size_t)tile * tl.rq;
    const int row_first = trows[0];
    const int slot = a.slot[row_first], pos0 = a.pos[row_first];
    int n_rows = 0;
    for (int i = 0; i < tl.rq; ++i) n_rows += trows[i] >= 0 ? 1 : 0;
    const int m_live = n_rows * H;                        // stacked rows: mr = rq * H + h
    // ---- stage Q (absorbed part | rotated part | zero padding) as bf16 ----
    for (int i = tid; i < LQ_ROWS * Dp; i += LQ_THREADS) {
        const int mr = i / Dp, d = i % Dp;
        float v = 0.f;
        if (mr < m_live && d < D) {
            const int row = trows[mr / H], h = mr % H;
            v = d < R ? a.q_lat[((size_t)row * H + h) * R + d]
                      : a.q[(size_t)row * a.ldq + (size_t)h * a.q_head_stride + a.q_rot_offset + (d - R)];
        }
        q_s[mr * LD + d] = __float2bfloat16_rn(v);
    }
    float o[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};      // rows g and g + 8 of this warp's row tile
    const int mr0 = wi * 16 + g, mr1 = mr0 + 8;
    const int qpos0 = pos0 + (mr0 < m_live ? mr0 / H : 0), qpos1 = pos0 + (mr1 < m_live ? mr1 / H : 0);
    const bool live0 = mr0 < m_live, live1 = mr1 < m_live;
    const int last_pos = pos0 + n_rows - 1;
    const int pg_first = a.window > 0 ? max(0, pos0 - a.window + 1) / 32 : 0;      // pages before the first row's window are never read
    const int n_pages = last_pos / 32 + 1;
    const int per = (n_pages - pg_first + tl.n_splits - 1) / tl.n_splits;
    const int p_begin = pg_first + split * per, p_end = min(n_pages, p_begin + per);
    const int win = a.window > 0 ? a.window : 0x7fffffff;
    const int ks_per = Dp / LQ_NJ / 16;                  // k steps of this warp's share of D
    const int ocol0 = wj * NT * 8;                       // this warp's output columns
    // page `pg` -> buffer `buf`: lines past the last position and the padding columns are zeroed, the rest is copied
    // asynchronously (16-byte chunks)
    auto stage = [&](int pg, int buf) {
        const int page = a.block_table[(size_t)slot * a.max_pages + pg];
        const __nv_bfloat16* src = (const __nv_bfloat16*)a.cache + (size_t)page * 32 * D;
        __nv_bfloat16* dst = c_buf + buf * 32 * LD;
        const int valid = min(32, last_pos + 1 - pg * 32);
        const int dv = D >> 3, dpv = Dp >> 3;             // 16-byte chunks per line
        for (int i = tid; i < 32 * dpv; i += LQ_THREADS) {
            const int j = i / dpv, c = i % dpv;
            if (j < valid && c < dv) cp_async16(dst + j * LD + c * 8, src + (size_t)j * D + c * 8);
            else *reinterpret_cast<uint4*>(dst + j * LD + c * 8) = make_uint4(0u, 0u, 0u, 0u);
        }
    };
    if (p_begin < p_end) stage(p_begin, 0);
    for (int pg = p_begin; pg < p_end; ++pg) {
        const int cur = (pg - p_begin) & 1;
        const __nv_bfloat16* c_s = c_buf + cur * 32 * LD;
        cp_async_wait_all();
        __syncthreads();                                  // this page has landed (and q_s is staged); everybody is done with the other buffer
        if (pg + 1 < p_end) stage(pg + 1, cur ^ 1);
        // ---- partial scores over this warp's share of D ----
        float s[4][4];
#pragma unroll
        for (int n = 0; n < 4; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
        for (int ks = 0; ks < ks_per; ++ks) {
            const int k0 = (wj * ks_per + ks) * 16;
            const int mat = lane >> 3, rr = lane & 7;     // each lane addresses one row of one 8 x 8 block
            uint32_t af[4];
            ldmatrix_x4(af, q_s + (wi * 16 + (mat & 1) * 8 + rr) * LD + k0 + (mat >> 1) * 8);
#pragma unroll
            for (int n = 0; n < 4; n += 2) {
                uint32_t bf[4];                           // tokens of n-tiles n, n + 1 x the two k halves
                ldmatrix_x4(bf, c_s + ((n + (mat >> 1)) * 8 + rr) * LD + k0 + (mat & 1) * 8);
                mma_bf16(s[n], af, bf[0], bf[1]);
                mma_bf16(s[n + 1], af, bf[2], bf[3]);
            }
        }
        float* my_sp = sp + ((wi * LQ_NJ + wj) * 16) * LQ_SP_LD;
#pragma unroll
        for (int n = 0; n < 4; ++n) {
            *reinterpret_cast<float2*>(my_sp + g * LQ_SP_LD + n * 8 + 2 * t) = make_float2(s[n][0], s[n][1]);
            *reinterpret_cast<float2*>(my_sp + (g + 8) * LQ_SP_LD + n * 8 + 2 * t) = make_float2(s[n][2], s[n][3]);
        }
        __syncthreads();
        // ---- softmax of rows g, g + 8; this lane's tokens: 2t, 2t+1, 2t+8, 2t+9, 2t+16, ... (the A fragment of P.C) ----
        float p0[8], p1[8];
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int e2 = 0; e2 < 4; ++e2) {
            const int col = e2 * 8 + 2 * t;
            float2 v0 = make_float2(0.f, 0.f), v1 = make_float2(0.f, 0.f);
#pragma unroll
            for (int j = 0; j < LQ_NJ; ++j) {
                const float* q = sp + ((wi * LQ_NJ + j) * 16) * LQ_SP_LD;
                const float2 u0 = *reinterpret_cast<const float2*>(q + g * LQ_SP_LD + col);
                const float2 u1 = *reinterpret_cast<const float2*>(q + (g + 8) * LQ_SP_LD + col);
                v0.x += u0.x; v0.y += u0.y; v1.x += u1.x; v1.y += u1.y;
            }
            const int tok = pg * 32 + col;
            p0[2 * e2] = (live0 && tok <= qpos0 && qpos0 - tok < win) ? v0.x * a.scale : -INFINITY;
            p0[2 * e2 + 1] = (live0 && tok + 1 <= qpos0 && qpos0 - tok - 1 < win) ? v0.y * a.scale : -INFINITY;
            p1[2 * e2] = (live1 && tok <= qpos1 && qpos1 - tok < win) ? v1.x * a.scale : -INFINITY;
            p1[2 * e2 + 1] = (live1 && tok + 1 <= qpos1 && qpos1 - tok - 1 < win) ? v1.y * a.scale : -INFINITY;
            mx0 = fmaxf(mx0, fmaxf(p0[2 * e2], p0[2 * e2 + 1]));
            mx1 = fmaxf(mx1, fmaxf(p1[2 * e2], p1[2 * e2 + 1]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
        const float al0 = mn0 == -INFINITY ? 1.f : expf(m_run[0] - mn0), al1 = mn1 == -INFINITY ? 1.f : expf(m_run[1] - mn1);
        float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            p0[e] = mn0 == -INFINITY ? 0.f : expf(p0[e] - mn0);
            p1[e] = mn1 == -INFINITY ? 0.f : expf(p1[e] - mn1);
            sum0 += p0[e];
            sum1 += p1[e];
        }
        m_run[0] = mn0; m_run[1] = mn1;
        l_run[0] = l_run[0] * al0 + sum0;                 // per-lane share of the row sum; the 4 lanes of a row meet at the end
        l_run[1] = l_run[1] * al1 + sum1;
#pragma unroll
        for (int n = 0; n < NT; ++n) { o[n][0] *= al0; o[n][1] *= al0; o[n][2] *= al1; o[n][3] *= al1; }
        // ---- O += P . C over this warp's columns: two k steps of 16 tokens ----
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
            uint32_t af[4];
            af[0] = pack_bf16(p0[4 * ks], p0[4 * ks + 1]);
            af[1] = pack_bf16(p1[4 * ks], p1[4 * ks + 1]);
            af[2] = pack_bf16(p0[4 * ks + 2], p0[4 * ks + 3]);
            af[3] = pack_bf16(p1[4 * ks + 2], p1[4 * ks + 3]);
#pragma unroll
            for (int n = 0; n < NT; n += 2) {
                // four 8 x 8 blocks: tokens ks*16 + {0..7, 8..15} x columns {n*8.., (n+1)*8..}; lane supplies one row address
                const int mat = lane >> 3, rr = lane & 7;
                const __nv_bfloat16* addr = c_s + (ks * 16 + (mat & 1) * 8 + rr) * LD + ocol0 + (n + (mat >> 1)) * 8;
                uint32_t b0, b1, b2, b3;
                const uint32_t sa = (uint32_t)__cvta_generic_to_shared(addr);
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(sa));
                mma_bf16(o[n], af, b0, b1);
                mma_bf16(o[n + 1], af, b2, b3);
            }
        }
    }
    // ---- finish: row sums across the 4 lanes of a row, then store (normalised, or partial for the merge) ----
    l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 1); l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 2);
    l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 1); l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 2);
    if (tl.n_splits == 1) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int mr = half ? mr1 : mr0;
            if (mr >= m_live) continue;
            const int row = trows[mr / H], h = mr % H;
            float l = l_run[half];
            if (a.sink) l += expf(a.sink[h] - m_run[half]);
            float inv = 1.f / l;
            if (a.gate) inv *= sigmoid_f(a.gate[(size_t)row * a.ld_gate + h]);
            float* dst = a.out + ((size_t)row * H + h) * R;
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                const int col = ocol0 + n * 8 + 2 * t;
                if (col < R) dst[col] = o[n][2 * half] * inv;
                if (col + 1 < R) dst[col + 1] = o[n][2 * half + 1] * inv;
            }
        }
    } else {
        // partial[tile][split][mr][rpad + 2]: unnormalised sums, then running maximum and row sum
        const int rpad = NT * 8 * LQ_NJ;
        float* base = tl.partial + (((size_t)tile * tl.n_splits + split) * LQ_MAX_ROWS) * (rpad + 2);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int mr = half ? mr1 : mr0;
            float* dst = base + (size_t)mr * (rpad + 2);
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                const int col = ocol0 + n * 8 + 2 * t;
                dst[col] = o[n][2 * half];
                dst[col + 1] = o[n][2 * half + 1];
            }
            if (wj == 0 && t == 0) { dst[rpad] = m_run[half]; dst[rpad + 1] = l_run[half]; }
        }
    }
}

// out[row][h][:] = sum_s w_s O_s / sum_s w_s l_s,  w_s = exp(m_s - max_s m_s); one CTA per (tile, stacked row)
__global__ void __launch_bounds__(128) latent_merge_kernel(DlLatentAttnArgs a, DlLatentTiles tl, int rpad) {
    const int tile = blockIdx.x, mr = blockIdx.y, H = a.n_heads, R = a.rank;
    const int* trows = tl.tile_rows + (size_t)tile * tl.rq;
    if (mr / H >= tl.rq) return;
    const int row = trows[mr / H], h = mr % H;
    if (row < 0) return;
    const float* base = tl.partial + ((size_t)tile * tl.n_splits * LQ_MAX_ROWS + mr) * (rpad + 2);
    const size_t sstride = (size_t)LQ_MAX_ROWS * (rpad + 2);
    // weights of the splits once, in shared memory; then every output column is a sum of independent loads
    __shared__ float wgt[64], lsum[64];
    const int ns = tl.n_splits;
    if ((int)threadIdx.x < ns) {
        wgt[threadIdx.x] = base[threadIdx.x * sstride + rpad];
        lsum[threadIdx.x] = base[threadIdx.x * sstride + rpad + 1];
    }
    __syncthreads();
    float mx = -INFINITY;
    for (int s = 0; s < ns; ++s) mx = fmaxf(mx, wgt[s]);
    float den = 0.f;
    for (int s = 0; s < ns; ++s) den += (wgt[s] == -INFINITY ? 0.f : expf(wgt[s] - mx)) * lsum[s];
    __syncthreads();
    if ((int)threadIdx.x < ns) wgt[threadIdx.x] = wgt[threadIdx.x] == -INFINITY ? 0.f : expf(wgt[threadIdx.x] - mx);
    __syncthreads();
    if (a.sink) den += expf(a.sink[h] - mx);
    float inv = 1.f / den;
    if (a.gate) inv *= sigmoid_f(a.gate[(size_t)row * a.ld_gate + h]);
    for (int d = threadIdx.x; d < R; d += blockDim.x) {
        float acc = 0.f;
#pragma unroll 8
        for (int s = 0; s < ns; ++s) acc = fmaf(wgt[s], base[s * sstride + d], acc);
        a.out[((size_t)row * H + h) * R + d] = acc * inv;
    }
}

extern "C" int dl_latent_tc_rpad(int rank) {
    const int unit = 8 * LQ_NJ;
    for (int nt = 2; nt <= 16; nt *= 2)
        if (rank <= nt * unit) return nt * unit;
    return -1;
}
extern "C" long long dl_latent_tc_partial_floats(int n_tiles, int n_splits, int rank) {
    const int rpad = dl_latent_tc_rpad(rank);
    return rpad < 0 ? -1 : (long long)n_tiles * n_splits * LQ_MAX_ROWS * (rpad + 2);
}

// 0 if these sizes run on the tensor-core kernel (bf16 cache, rows x heads stacked into <= 64 rows, 16-byte cache lines)
extern "C" int dl_latent_attention_tc_supported(int n_heads, int rank, int rot, int ctype, int rq) {
    if (ctype != DL_T_BF16 || n_heads < 1 || rq < 1 || rq * n_heads > LQ_MAX_ROWS) return -1;
    if ((rank + rot) % 8 != 0 || dl_latent_tc_rpad(rank) < 0) return -1;
    return 0;
}

static size_t latent_mma_smem(int ni, int dp) {
    return (size_t)(16 * ni + 2 * 32) * (dp + 8) * 2 + (size_t)ni * LQ_NJ * 16 * LQ_SP_LD * 4;
}

template <int NT, int NI>
static int launch_latent_mma_ni(const DlLatentAttnArgs& a, const DlLatentTiles& tl, cudaStream_t st) {
    const size_t smem = latent_mma_smem(NI, tl.d_pad);
    if (smem > 227 * 1024) { dl_set_error("dl_latent_attention_tc: rank %d needs %zu bytes of shared memory", a.rank, smem); return -1; }
    cudaError_t e = cudaFuncSetAttribute(latent_attention_mma_kernel<NT, NI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { dl_set_error("dl_latent_attention_tc: shared memory attribute: %s", cudaGetErrorString(e)); return -(int)e; }
    latent_attention_mma_kernel<NT, NI><<<dim3(tl.n_tiles, tl.n_splits), 32 * LQ_NJ * NI, smem, st>>>(a, tl);
    return 0;
}

// tiles of up to 32 stacked rows run with 8 warps, larger ones (up to 64) with 16
template <int NT>
static int launch_latent_mma(const DlLatentAttnArgs& a, const DlLatentTiles& tl, cudaStream_t st) {
    return tl.rq * a.n_heads > 32 ? launch_latent_mma_ni<NT, 4>(a, tl, st) : launch_latent_mma_ni<NT, 2>(a, tl, st);
}

extern "C" int dl_latent_attention_tc(const DlLatentAttnArgs* args, const DlLatentTiles* tiles, void* stream) {
    const DlLatentAttnArgs& a = *args;
    DlLatentTiles tl = *tiles;
    if (a.page_size != 32) { dl_set_error("dl_latent_attention_tc: page size must be 32"); return -1; }
    if (dl_latent_attention_tc_supported(a.n_heads, a.rank, a.rot, a.ctype, tl.rq) != 0) {
        dl_set_error("dl_latent_attention_tc: %d heads x %d rows, rank %d + %d not supported", a.n_heads, tl.rq, a.rank, a.rot);
        return -1;
    }
    if (tl.n_tiles < 1 || tl.n_splits < 1 || tl.n_splits > 64 || (tl.n_splits > 1 && tl.partial == nullptr)) { dl_set_error("dl_latent_attention_tc: bad tiling"); return -1; }
    const int rpad = dl_latent_tc_rpad(a.rank);
    const int unit = 16 * LQ_NJ;
    int dp = (a.rank + a.rot + unit - 1) / unit * unit;
    if (dp < rpad) dp = rpad;                             // P.C reads `rpad` columns of every staged line
    tl.d_pad = dp;
    cudaStream_t st = (cudaStream_t)stream;
    int rc;
    switch (rpad / (8 * LQ_NJ)) {
        case 2: rc = launch_latent_mma<2>(a, tl, st); break;
        case 4: rc = launch_latent_mma<4>(a, tl, st); break;
        case 8: rc = launch_latent_mma<8>(a, tl, st); break;
        default: rc = launch_latent_mma<16>(a, tl, st); break;
    }
    if (rc != 0) return rc;
    LAYER_CHECK_LAUNCH("dl_latent_attention_tc");
    if (tl.n_splits > 1) {
        latent_merge_kernel<<<dim3(tl.n_tiles, tl.rq * a.n_heads), 128, 0, st>>>(a, tl, rpad);
        LAYER_CHECK_LAUNCH("dl_latent_attention_tc merge");
    }
    return 0;
}
