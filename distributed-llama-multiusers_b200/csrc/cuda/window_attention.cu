// Grouped-query attention over a sliding window whose values ARE its keys: one projection k per token and key/value
// head; the key is k with rotary positions on its first `rope_dims` dimensions, the value is k as projected.
//     score_h(i, j) = cap( scale * q_h,i . rot(k_g,j) ),   cap(s) = softcap * tanh(s / softcap)   (softcap 0: none)
//     visible: 0 <= i - j < window                                                               (window 0: all j <= i)
//     out_h(i)      = sum_j softmax_j(score_h(i, .)) k_g,j              g = h / (heads / kv_heads)
// Only the first rope_dims dimensions differ between a key and its value, so the cache holds, per token and key/value
// head, ONE line  [ rot(k)[0 : dim] | k[0 : rope_dims] ]:  the key is the first `dim` entries, the value is the tail
// followed by entries rope_dims .. dim of the key.  (dim + rope_dims) instead of 2 dim numbers per token and head.
// Cache layout: [page][kv_head][page_size][dim + rope_dims], bf16 or f32; pages of a sequence from its block table.
//
// Rotary: interleaved pairs (2i, 2i + 1), angle = pos * freqs[i] formed in f64, cos and sin multiplied by rope_scale
// (frequency interpolation schemes that also scale the rotation's magnitude pass their factor here).
//
// The same kernels serve attention with values of their own (vdim > 0): the line is [ key[0 : dim] | value[0 : vdim] ],
// written by attn_kv_write_kernel, which can divide every query and key head by its root mean square first.  Two more
// options of the score side: a chunked mask (chunk > 0: j is visible to i only if floor(j / chunk) == floor(i / chunk);
// the borders are multiples of `chunk` in sequence positions, wherever a portion starts) and a sink per head: the softmax
// denominator gets one more term exp(sink_h) that pulls weight away from the keys and contributes no value.
//
// Kernels: the cache writer, which also turns the queries in place (one launch, cos and sin formed once per row and
// pair); the per-row attention kernel (exact f32 arithmetic on either cache type; one CTA per
// (row, key/value head), all query heads of the group share each staged page; pages outside the window are never
// touched); the tensor-core kernel for prompt portions (bf16 cache) further down.
#include "mma_common.cuh"
#include "../../../include/dllama_b200.h"

#define WA_PAGE 32

// ------------------------------------------------------------------------------------------------
// cache writer
// ------------------------------------------------------------------------------------------------
// One CTA per row.  cos and sin of the row's angles are formed ONCE (f64) into shared memory; then every (head, pair) is
// turned by its own thread: the query heads in place (when q is given), the key heads on their way into the cache; the
// rest of each key is copied.
#define WK_MAX_PAIRS 256
template <typename CT>
__global__ void __launch_bounds__(256) window_kv_write_kernel(DlWindowKvArgs a) {
    __shared__ float cs[WK_MAX_PAIRS], sn[WK_MAX_PAIRS];
    const int m = blockIdx.x;
    const int pos = a.pos[m], slot = a.slot[m];
    const int page = a.block_table[(size_t)slot * a.max_pages + pos / WA_PAGE];
    const int LD = a.dim + a.rope_dims, half = a.rope_dims / 2;
    const float* kin = a.k + (size_t)m * a.ld;
    CT* line0 = (CT*)a.cache + (((size_t)page * a.kv_heads) * WA_PAGE + pos % WA_PAGE) * LD;      // head g: + g * WA_PAGE * LD
    const size_t head_step = (size_t)WA_PAGE * LD;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        double sd, cd;
        sincos((double)pos * a.freqs[i], &sd, &cd);
        cs[i] = (float)(cd * (double)a.rope_scale);
        sn[i] = (float)(sd * (double)a.rope_scale);
    }
    __syncthreads();
    const int nq = a.q ? a.q_heads : 0;
    for (int t = threadIdx.x; t < (a.kv_heads + nq) * half; t += blockDim.x) {
        const int h = t / half, i = t - h * half;
        const float c = cs[i], s = sn[i];
        if (h < a.kv_heads) {
            const float u = kin[h * a.dim + 2 * i], v = kin[h * a.dim + 2 * i + 1];
            CT* dst = line0 + h * head_step;
            st_f(dst + 2 * i, u * c - v * s);
            st_f(dst + 2 * i + 1, v * c + u * s);
            st_f(dst + a.dim + 2 * i, u);
            st_f(dst + a.dim + 2 * i + 1, v);
        } else {
            float* q = a.q + (size_t)m * a.ldq + (size_t)(h - a.kv_heads) * a.dim;
            const float u = q[2 * i], v = q[2 * i + 1];
            q[2 * i] = u * c - v * s;
            q[2 * i + 1] = v * c + u * s;
        }
    }
    const int rest = a.dim - a.rope_dims;
    for (int t = threadIdx.x; t < a.kv_heads * rest; t += blockDim.x) {
        const int g = t / rest, i = a.rope_dims + t - g * rest;
        st_f(line0 + g * head_step + i, kin[g * a.dim + i]);
    }
}

// Separate values: one CTA per row.  The row's queries and keys (and the head mix) are brought into shared memory by all
// threads at once; then a warp per (query or key) head: optional rotary on the first rope_dims dimensions (pairs
// (i, i + rope_dims / 2) with rope_half, else (2i, 2i + 1); cos and sin of the row's angles are formed once, in f64),
// THEN, with qk_norm, the head is divided by sqrt(mean(head^2) + eps): the queries in place, the keys on their way into
// the cache.  The values are copied behind the keys.  With `talk` the head mix of the scores is folded into the queries:
// q_mixed[h][c * dim + i] = sum over the query heads g of key/value head c of talk[h][g] q_g[i].
// Dynamic shared memory: 2 (kv_heads + q_heads) dim + rope_dims + q_heads^2 floats.
template <typename CT>
__global__ void __launch_bounds__(256) attn_kv_write_kernel(DlWindowKvArgs a) {
    extern __shared__ float wk_sm[];
    const int m = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int pos = a.pos[m], slot = a.slot[m];
    const int page = a.block_table[(size_t)slot * a.max_pages + pos / WA_PAGE];
    const int LD = a.dim + a.vdim, D = a.dim, RD = a.rope_dims, half = RD / 2;
    CT* line0 = (CT*)a.cache + (((size_t)page * a.kv_heads) * WA_PAGE + pos % WA_PAGE) * LD;
    const size_t head_step = (size_t)WA_PAGE * LD;
    const int nq = a.q ? a.q_heads : 0, nk = a.k ? a.kv_heads : 0;      // without k (a layer that reads another layer's cache): the queries only
    float* raw_s = wk_sm;                                     // [kv_heads + nq][D]: the heads as projected
    float* heads_s = raw_s + (size_t)(a.kv_heads + nq) * D;   // the same heads as they leave (rotated, normalised)
    float* cs = heads_s + (size_t)(a.kv_heads + nq) * D;      // [half] cos, then [half] sin
    float* sn = cs + half;
    float* talk_s = sn + half;                                // [nq][nq]
    for (int t = threadIdx.x; t < nk * D; t += blockDim.x) raw_s[t] = a.k[(size_t)m * a.ld + t];
    for (int t = threadIdx.x; t < nq * D; t += blockDim.x) raw_s[(size_t)a.kv_heads * D + t] = a.q[(size_t)m * a.ldq + t];
    if (a.talk != nullptr)
        for (int t = threadIdx.x; t < nq * nq; t += blockDim.x) talk_s[t] = a.talk[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        double sd, cd;
        sincos((double)pos * a.freqs[i], &sd, &cd);
        cs[i] = (float)(cd * (double)a.rope_scale);
        sn[i] = (float)(sd * (double)a.rope_scale);
    }
    // the values go straight from the projection into the cache
    for (int t = threadIdx.x; a.v != nullptr && t < a.kv_heads * a.vdim; t += blockDim.x) {
        const int g = t / a.vdim, i = t - g * a.vdim;
        st_f(line0 + g * head_step + a.dim + i, a.v[(size_t)m * a.ldv + t]);
    }
    __syncthreads();
    for (int h = (a.kv_heads - nk) + warp; h < a.kv_heads + nq; h += nw) {
        const bool is_k = h < a.kv_heads;
        const float* src = raw_s + (size_t)h * D;
        float* hs = heads_s + (size_t)h * D;
        float ss = 0.f;
        for (int i = lane; i < D; i += 32) {
            float r = src[i];
            if (i < RD) {
                int p, iu, iv;
                bool second;
                if (a.rope_half) { p = i < half ? i : i - half; iu = p; iv = p + half; second = i >= half; }
                else { p = i >> 1; iu = 2 * p; iv = iu + 1; second = i & 1; }
                const float u = src[iu], v = src[iv];
                r = second ? v * cs[p] + u * sn[p] : u * cs[p] - v * sn[p];
            }
            hs[i] = r;
            ss = fmaf(r, r, ss);
        }
        const float inv = a.qk_norm ? 1.f / sqrtf(warp_sum(ss) / (float)D + a.eps) : 1.f;
        if (is_k) {
            CT* dst = line0 + h * head_step;
            for (int i = lane; i < D; i += 32) st_f(dst + i, hs[i] * inv);
        } else {
            float* qh = a.q + (size_t)m * a.ldq + (size_t)(h - a.kv_heads) * D;
            for (int i = lane; i < D; i += 32) { const float r = hs[i] * inv; hs[i] = r; qh[i] = r; }
        }
    }
    if (a.talk != nullptr && nq > 0) {
        __syncthreads();
        const int rep = nq / a.kv_heads, QD = a.kv_heads * D;
        const float* qs = heads_s + (size_t)a.kv_heads * D;
        float* out = a.q_mixed + (size_t)m * a.ld_qm;
        for (int t = threadIdx.x; t < QD; t += blockDim.x) {      // a thread owns column t = c * D + i of every head's folded query
            const int c = t / D, i = t - c * D;
            const float* qc = qs + (size_t)c * rep * D + i;
            for (int h = 0; h < nq; ++h) {
                const float* tk = talk_s + h * nq + c * rep;
                float acc = 0.f;
                for (int g = 0; g < rep; ++g) acc = fmaf(tk[g], qc[(size_t)g * D], acc);
                out[(size_t)h * QD + t] = acc;
            }
        }
    }
}

extern "C" int dl_window_kv_write(const DlWindowKvArgs* args, int M, void* stream) {
    const DlWindowKvArgs& a = *args;
    if (a.vdim > 0) {
        if ((a.k == nullptr) != (a.v == nullptr) || (a.k == nullptr && a.q == nullptr)) { dl_set_error("dl_window_kv_write: keys and values come together, or the queries alone"); return -1; }
        if (a.rope_dims < 0 || a.rope_dims > a.dim || (a.rope_dims & 1) || a.vdim < 1 || a.page_size != WA_PAGE) { dl_set_error("dl_window_kv_write: bad sizes (rope_dims %d, dim %d, vdim %d)", a.rope_dims, a.dim, a.vdim); return -1; }
        if (a.talk != nullptr && (a.q == nullptr || a.q_mixed == nullptr || a.q_heads % a.kv_heads)) { dl_set_error("dl_window_kv_write: the head mix needs q, q_mixed and whole groups of heads"); return -1; }
        const int nq_ = a.q ? a.q_heads : 0;
        const size_t smem = ((size_t)2 * (a.kv_heads + nq_) * a.dim + a.rope_dims + (a.talk ? (size_t)nq_ * nq_ : 0)) * sizeof(float);
        if (smem > 227 * 1024) { dl_set_error("dl_window_kv_write: %zu bytes of shared memory", smem); return -1; }
        cudaError_t e;
        if (a.ctype == DL_T_BF16) {
            e = cudaFuncSetAttribute(attn_kv_write_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e == cudaSuccess) attn_kv_write_kernel<__nv_bfloat16><<<M, 256, smem, (cudaStream_t)stream>>>(a);
        } else {
            e = cudaFuncSetAttribute(attn_kv_write_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e == cudaSuccess) attn_kv_write_kernel<float><<<M, 256, smem, (cudaStream_t)stream>>>(a);
        }
        if (e != cudaSuccess) { dl_set_error("dl_window_kv_write: shared memory attribute: %s", cudaGetErrorString(e)); return -(int)e; }
        LAYER_CHECK_LAUNCH("dl_window_kv_write");
        return 0;
    }
    if (a.qk_norm) { dl_set_error("dl_window_kv_write: qk_norm belongs to the separate-value form"); return -1; }
    if (a.rope_dims > a.dim || (a.rope_dims & 1) || a.rope_dims > 2 * WK_MAX_PAIRS || a.page_size != WA_PAGE) { dl_set_error("dl_window_kv_write: bad rotary or page size"); return -1; }
    cudaStream_t st = (cudaStream_t)stream;
    if (a.ctype == DL_T_BF16) window_kv_write_kernel<__nv_bfloat16><<<M, 256, 0, st>>>(a);
    else window_kv_write_kernel<float><<<M, 256, 0, st>>>(a);
    LAYER_CHECK_LAUNCH("dl_window_kv_write");
    return 0;
}

// ------------------------------------------------------------------------------------------------
// per-row attention: one CTA per (row, key/value head)
// ------------------------------------------------------------------------------------------------
template <typename CT>
__global__ void window_attention_kernel(DlWindowAttnArgs a) {
    extern __shared__ float sm[];
    const int m = blockIdx.x, g = blockIdx.y;
    const int rep = a.heads / a.kv_heads, D = a.dim, RD = a.rope_dims, DV = a.vdim > 0 ? a.vdim : D;
    const int KH = a.key_heads > 1 ? a.key_heads : 1, QD = KH * D;      // head-mixed scores: a query meets the keys of all KH key/value heads side by side
    const int LD = D + (a.vdim > 0 ? a.vdim : RD), VT = LD - D, LP = QD + VT + 1;
    const int nw = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* q_s = sm;                                   // [rep][QD]
    float* tile = q_s + (size_t)rep * QD;              // [WA_PAGE][QD keys | VT: the rest of head g's line | 1]
    float* acc = tile + (size_t)WA_PAGE * LP;          // [rep][DV]
    float* p_s = acc + (size_t)rep * DV;               // [nw][WA_PAGE]
    float* ml = p_s + (size_t)nw * WA_PAGE;            // [rep][2]
    const int pos = a.pos[m], slot = a.slot[m];
    int first = a.window > 0 ? max(0, pos - a.window + 1) : 0;            // oldest visible position
    if (a.chunk > 0) first = max(first, pos / a.chunk * a.chunk);
    for (int t = threadIdx.x; t < rep * QD; t += blockDim.x) q_s[t] = a.q[(size_t)m * a.ldq + (size_t)g * rep * QD + t];
    for (int t = threadIdx.x; t < rep * DV; t += blockDim.x) acc[t] = 0.f;
    for (int t = threadIdx.x; t < rep; t += blockDim.x) { ml[2 * t] = -INFINITY; ml[2 * t + 1] = 0.f; }
    for (int pg = first / WA_PAGE; pg <= pos / WA_PAGE; ++pg) {
        __syncthreads();
        const int page = a.block_table[(size_t)slot * a.max_pages + pg];
        const CT* src = (const CT*)a.cache + ((size_t)page * a.kv_heads + g) * WA_PAGE * LD;
        const int j_lo = max(0, first - pg * WA_PAGE), j_hi = min(WA_PAGE, pos + 1 - pg * WA_PAGE);   // visible lines [j_lo, j_hi)
        for (int i = threadIdx.x; i < WA_PAGE * LD; i += blockDim.x) {
            const int j = i / LD, d = i - j * LD;
            if (KH > 1 && d < D) continue;             // the keys come from every key/value head, below
            tile[j * LP + (d < D ? d : QD + d - D)] = (j >= j_lo && j < j_hi) ? ld_f(src + i) : 0.f;
        }
        if (KH > 1) {
            for (int i = threadIdx.x; i < KH * WA_PAGE * D; i += blockDim.x) {
                const int c = i / (WA_PAGE * D), j = (i - c * WA_PAGE * D) / D, d = i - (c * WA_PAGE + j) * D;
                const CT* kc = (const CT*)a.cache + (((size_t)page * a.kv_heads + c) * WA_PAGE + j) * LD;
                tile[j * LP + c * D + d] = (j >= j_lo && j < j_hi) ? ld_f(kc + d) : 0.f;
            }
        }
        __syncthreads();
        for (int h = warp; h < rep; h += nw) {
            const float* qh = q_s + (size_t)h * QD;
            const float* row = tile + lane * LP;
            const bool vis = lane >= j_lo && lane < j_hi;
            float s = 0.f;
            for (int d = 0; d < QD; ++d) s = fmaf(qh[d], row[d], s);
            s *= a.scale;
            if (a.softcap > 0.f) s = a.softcap * tanhf(s / a.softcap);
            if (!vis) s = -INFINITY;
            const float m_old = ml[2 * h], m_new = fmaxf(m_old, warp_max(s));
            const float p = vis ? expf(s - m_new) : 0.f;
            const float alpha = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
            const float l_new = ml[2 * h + 1] * alpha + warp_sum(p);
            p_s[warp * WA_PAGE + lane] = p;
            __syncwarp();
            if (lane == 0) { ml[2 * h] = m_new; ml[2 * h + 1] = l_new; }
            float* ah = acc + (size_t)h * DV;
            const float* ps = p_s + warp * WA_PAGE;
            for (int d = lane; d < DV; d += 32) {
                const int col = (a.vdim > 0 || d < RD) ? QD + d : d;     // own values, or the value's first entries, sit behind the key
                float v = ah[d] * alpha;
                for (int j = j_lo; j < j_hi; ++j) v = fmaf(ps[j], tile[j * LP + col], v);
                ah[d] = v;
            }
            __syncwarp();
        }
    }
    __syncthreads();
    for (int t = threadIdx.x; t < rep * DV; t += blockDim.x) {
        const int h = t / DV;
        float l = ml[2 * h + 1];
        if (a.sink) l += expf(a.sink[g * rep + h] - ml[2 * h]);
        a.out[(size_t)m * a.ldo + (size_t)g * rep * DV + t] = acc[t] / l;
    }
}

static int window_args_ok(const DlWindowAttnArgs& a, const char* who) {
    if (a.heads < 1 || a.kv_heads < 1 || a.heads % a.kv_heads || a.dim < 1 || a.rope_dims > a.dim || a.window < 0 || a.page_size != WA_PAGE ||
        a.vdim < 0 || a.chunk < 0 || (a.vdim > 0 && a.rope_dims != 0) || (a.key_heads > 1 && (a.key_heads != a.kv_heads || a.vdim < 1))) {
        dl_set_error("%s: bad shape (heads %d / %d, dim %d, rotary %d, window %d, page %d)", who, a.heads, a.kv_heads, a.dim, a.rope_dims, a.window, a.page_size);
        return -1;
    }
    return 0;
}

extern "C" int dl_window_attention(const DlWindowAttnArgs* args, int M, void* stream) {
    const DlWindowAttnArgs& a = *args;
    if (window_args_ok(a, "dl_window_attention")) return -1;
    const int rep = a.heads / a.kv_heads, nw = rep < 8 ? rep : 8, LD = a.dim + (a.vdim > 0 ? a.vdim : a.rope_dims), DV = a.vdim > 0 ? a.vdim : a.dim;
    const int QD = (a.key_heads > 1 ? a.key_heads : 1) * a.dim;
    const size_t smem = ((size_t)rep * (QD + DV) + (size_t)WA_PAGE * (QD + LD - a.dim + 1) + (size_t)nw * WA_PAGE + 2 * (size_t)rep) * sizeof(float);
    if (smem > 227 * 1024) { dl_set_error("dl_window_attention: %d heads per group x dim %d need %zu bytes of shared memory", rep, a.dim, smem); return -1; }
    cudaStream_t st = (cudaStream_t)stream;
    dim3 grid(M, a.kv_heads);
    cudaError_t e;
    if (a.ctype == DL_T_BF16) {
        e = cudaFuncSetAttribute(window_attention_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) window_attention_kernel<__nv_bfloat16><<<grid, nw * 32, smem, st>>>(a);
    } else {
        e = cudaFuncSetAttribute(window_attention_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) window_attention_kernel<float><<<grid, nw * 32, smem, st>>>(a);
    }
    if (e != cudaSuccess) { dl_set_error("dl_window_attention: shared memory attribute: %s", cudaGetErrorString(e)); return -(int)e; }
    LAYER_CHECK_LAUNCH("dl_window_attention");
    return 0;
}

// ------------------------------------------------------------------------------------------------
// Tensor-core kernel (bf16 cache): a CTA owns a tile of up to `rq` consecutive positions of one sequence and one
// key/value head g; the heads/kv_heads query heads of the group read the same cache lines, so (position, head) pairs
// stack on the M dimension of the MMA: 4 warps x 16 stacked rows.  The CTA walks the pages that the tile's windows
// touch; per page (32 tokens), per warp:
//     S[16 x 32]  = Q[16 x D] . K[32 x D]^T        Q (bf16, staged once per tile) and K by ldmatrix
//     scale, soft cap, window mask, online softmax in f32 and base 2 (two rows per thread, reduced over the quad)
//     O[16 x D]  += P[16 x 32] . V[32 x D]         P from the score registers, V by ldmatrix.trans from the SAME staged
//                                                  line: value column c sits at D + c (c < rope_dims) or at c
// mma.sync m16n8k16 bf16, f32 accumulators.  Pages arrive by cp.async into two buffers (page k + 1 in flight while
// page k is multiplied).  tile_rows[n_tiles][rq]: row indices of the batch, -1 where a tile has fewer rows.
// ------------------------------------------------------------------------------------------------
#define WM_ROWS 64

// The softmax of the tensor-core kernel works in base 2: a score leaves this function already multiplied by log2(e), so a
// probability is one ex2.  With a soft cap, cap * tanh(x / cap) = cap * (1 - 2 / (e^(2x/cap) + 1)) (absolute error about
// 1e-7 of the cap on the fast exponential and reciprocal; exact limits for large |x|):
//     c1 = scale * 2 / cap * log2(e),  K = cap * log2(e):   score2 = K - 2K / (2^(acc * c1) + 1)
// without one: score2 = acc * (scale * log2(e)).
__device__ __forceinline__ float fast_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float fast_rcp(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
#define WM_LOG2E 1.4426950408889634f
#define WM_LN2 0.6931471805599453f

__host__ __device__ __forceinline__ int wm_line_stride(int LD) {      // bf16 elements; rows 16 B apart modulo 128 B
    int s = (LD + 7) / 8 * 8 + 8;
    if ((s * 2) % 128 == 0) s += 8;
    return s;
}

template <int DK>
__global__ void __launch_bounds__(128, 4) window_attention_mma_kernel(DlWindowAttnArgs a, const int* __restrict__ tile_rows, int rq,
                                                                   int n_splits, float* __restrict__ partial) {
    constexpr int D = 16 * DK, NV = D / 8;
    extern __shared__ __align__(16) uint8_t smraw[];
    __shared__ int s_row[WM_ROWS];
    const int RD = a.rope_dims, LD = D + (a.vdim > 0 ? a.vdim : RD), LDS = wm_line_stride(LD);
    const bool own_v = a.vdim > 0;                                                  // values behind the key (vdim == dim here)
    constexpr int QS = D + 8;                                                       // row stride of the query tile (bf16)
    __nv_bfloat16* kv_s = reinterpret_cast<__nv_bfloat16*>(smraw);                  // [2][WA_PAGE][LDS]
    __nv_bfloat16* q_s = kv_s + (size_t)2 * WA_PAGE * LDS;                          // [WM_ROWS][QS]: the stacked queries
    const int tile = blockIdx.x, g = blockIdx.y, rep = a.heads / a.kv_heads;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
    if (threadIdx.x < rq) s_row[threadIdx.x] = tile_rows[(size_t)tile * rq + threadIdx.x];
    __syncthreads();
    int n_rows = 0;
    while (n_rows < rq && s_row[n_rows] >= 0) ++n_rows;
    if (n_rows == 0) return;
    const int p_first = a.pos[s_row[0]], p_last = p_first + n_rows - 1, slot = a.slot[s_row[0]];
    int lo = a.window > 0 ? max(0, p_first - a.window + 1) : 0;
    if (a.chunk > 0) lo = max(lo, p_first / a.chunk * a.chunk);
    int pg_lo = lo / WA_PAGE, pg_hi = p_last / WA_PAGE;
    if (n_splits > 1) {                  // this CTA's share of the tile's pages (possibly none)
        const int per = (pg_hi - pg_lo + n_splits) / n_splits;
        pg_lo += (int)blockIdx.z * per;
        pg_hi = min(pg_hi, pg_lo + per - 1);
    }
    const bool active = warp * 16 < n_rows * rep;
    const bool capped = a.softcap > 0.f;
    const float c1 = capped ? a.scale * 2.f / a.softcap * WM_LOG2E : a.scale * WM_LOG2E;
    const float capK = a.softcap * WM_LOG2E;

    // this thread's two stacked rows: s = position-in-tile * rep + head-in-group
    const int s0 = warp * 16 + gid, s1 = s0 + 8;
    const int r0 = s0 / rep, r1 = s1 / rep;
    const bool ok0 = r0 < n_rows, ok1 = r1 < n_rows;
    const int pos0 = p_first + r0, pos1 = p_first + r1;
    const int cs0 = a.chunk > 0 ? pos0 / a.chunk * a.chunk : 0, cs1 = a.chunk > 0 ? pos1 / a.chunk * a.chunk : 0;      // first position of the row's chunk
    const int cs_last = a.chunk > 0 ? p_last / a.chunk * a.chunk : 0;
    // the tile's queries, rounded to bf16, into shared memory (A fragments come from there by ldmatrix: registers are
    // what limits the CTAs per SM)
    for (int idx = threadIdx.x; idx < WM_ROWS * (D / 4); idx += 128) {
        const int sr = idx / (D / 4), c4 = idx - sr * (D / 4);
        const int r = sr / rep;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < n_rows) v = *reinterpret_cast<const float4*>(a.q + (size_t)s_row[r] * a.ldq + (size_t)(g * rep + sr % rep) * D + c4 * 4);
        uint2 pk;
        pk.x = pack_bf16(v.x, v.y);
        pk.y = pack_bf16(v.z, v.w);
        *reinterpret_cast<uint2*>(q_s + (size_t)sr * QS + c4 * 4) = pk;
    }
    float o[NV][4];
#pragma unroll
    for (int v = 0; v < NV; ++v) { o[v][0] = o[v][1] = o[v][2] = o[v][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    const int chunks_per_line = LD / 8, n_chunks = WA_PAGE * chunks_per_line;
    auto issue = [&](int pg, int buf) {
        const int page = a.block_table[(size_t)slot * a.max_pages + pg];
        const __nv_bfloat16* src = (const __nv_bfloat16*)a.cache + ((size_t)page * a.kv_heads + g) * WA_PAGE * LD;
        __nv_bfloat16* dst = kv_s + (size_t)buf * WA_PAGE * LDS;
        for (int c = threadIdx.x; c < n_chunks; c += 128) {
            const int j = c / chunks_per_line, part = c - j * chunks_per_line;
            cp_async16(dst + (size_t)j * LDS + part * 8, src + (size_t)j * LD + part * 8);
        }
    };
    if (pg_lo <= pg_hi) issue(pg_lo, 0);
    const int mat = lane >> 3, rr = lane & 7;
    for (int pg = pg_lo; pg <= pg_hi; ++pg) {
        const int buf = (pg - pg_lo) & 1;
        cp_async_wait_all();
        __syncthreads();                      // page pg has landed (and the queries); everyone is done with the other buffer
        if (pg < pg_hi) issue(pg + 1, buf ^ 1);
        if (!active) continue;
        const __nv_bfloat16* kv = kv_s + (size_t)buf * WA_PAGE * LDS;
        float sc[4][4];
#pragma unroll
        for (int n = 0; n < 4; ++n) { sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f; }
#pragma unroll
        for (int kk = 0; kk < DK; ++kk) {
            uint32_t qf[4];
            ldmatrix_x4(qf, q_s + (size_t)(warp * 16 + (mat & 1) * 8 + rr) * QS + kk * 16 + (mat >> 1) * 8);
#pragma unroll
            for (int np = 0; np < 2; ++np) {
                uint32_t b[4];
                ldmatrix_x4(b, kv + (size_t)(np * 16 + (mat >> 1) * 8 + rr) * LDS + kk * 16 + (mat & 1) * 8);
                mma_bf16(sc[2 * np], qf, b[0], b[1]);
                mma_bf16(sc[2 * np + 1], qf, b[2], b[3]);
            }
        }
        // scale and soft cap (base-2 scores), window mask (skipped on pages that every row of the tile sees whole)
        const int pg_first = pg * WA_PAGE;
        const bool whole = pg_first + WA_PAGE - 1 <= p_first && (a.window == 0 || p_last - pg_first < a.window) && pg_first >= cs_last;      // stacked rows without a position are never stored
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int n = 0; n < 4; ++n) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float s2 = sc[n][e] * c1;
                if (capped) s2 = fmaf(-2.f * capK, fast_rcp(fast_ex2(s2) + 1.f), capK);
                if (!whole) {
                    const int j = pg_first + n * 8 + tig * 2 + (e & 1);
                    const int pr = (e < 2) ? pos0 : pos1;
                    const bool vis = ((e < 2) ? ok0 : ok1) && j <= pr && (a.window == 0 || pr - j < a.window) && j >= ((e < 2) ? cs0 : cs1);
                    s2 = vis ? s2 : -INFINITY;
                }
                sc[n][e] = s2;
                if (e < 2) mx0 = fmaxf(mx0, s2); else mx1 = fmaxf(mx1, s2);
            }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float al0 = (m0 == -INFINITY) ? 0.f : fast_ex2(m0 - mn0), al1 = (m1 == -INFINITY) ? 0.f : fast_ex2(m1 - mn1);
        const float ref0 = (mn0 == -INFINITY) ? 0.f : mn0, ref1 = (mn1 == -INFINITY) ? 0.f : mn1;      // a row that sees nothing yet: every p = 0
        m0 = mn0; m1 = mn1;
        float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
        for (int n = 0; n < 4; ++n) {
            sc[n][0] = fast_ex2(sc[n][0] - ref0); sc[n][1] = fast_ex2(sc[n][1] - ref0);
            sc[n][2] = fast_ex2(sc[n][2] - ref1); sc[n][3] = fast_ex2(sc[n][3] - ref1);
            ps0 += sc[n][0] + sc[n][1];
            ps1 += sc[n][2] + sc[n][3];
        }
        l0 = l0 * al0 + ps0;
        l1 = l1 * al1 + ps1;
#pragma unroll
        for (int v = 0; v < NV; ++v) { o[v][0] *= al0; o[v][1] *= al0; o[v][2] *= al1; o[v][3] *= al1; }
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
            uint32_t pa[4];
            pa[0] = pack_bf16(sc[2 * ks][0], sc[2 * ks][1]);
            pa[1] = pack_bf16(sc[2 * ks][2], sc[2 * ks][3]);
            pa[2] = pack_bf16(sc[2 * ks + 1][0], sc[2 * ks + 1][1]);
            pa[3] = pack_bf16(sc[2 * ks + 1][2], sc[2 * ks + 1][3]);
#pragma unroll
            for (int vp = 0; vp < NV / 2; ++vp) {
                const int vt = 2 * vp + (mat >> 1);
                const int col = (own_v || vt * 8 < RD) ? D + vt * 8 : vt * 8;      // own values, or the value's first entries, sit behind the key
                uint32_t b[4];
                ldmatrix_x4_trans(b, kv + (size_t)(ks * 16 + (mat & 1) * 8 + rr) * LDS + col);
                mma_bf16(o[2 * vp], pa, b[0], b[1]);
                mma_bf16(o[2 * vp + 1], pa, b[2], b[3]);
            }
        }
    }
    if (!active) return;
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    if (n_splits > 1) {                  // unnormalised sums, running maximum and sum per stacked row, for the merge kernel
        float* base = partial + (((size_t)tile * a.kv_heads + g) * n_splits + blockIdx.z) * WM_ROWS * (D + 2);
        if (ok0) {
            float* dst = base + (size_t)s0 * (D + 2);
#pragma unroll
            for (int v = 0; v < NV; ++v) *reinterpret_cast<float2*>(dst + v * 8 + tig * 2) = make_float2(o[v][0], o[v][1]);
            if (tig == 0) { dst[D] = m0 * WM_LN2; dst[D + 1] = l0; }
        }
        if (ok1) {
            float* dst = base + (size_t)s1 * (D + 2);
#pragma unroll
            for (int v = 0; v < NV; ++v) *reinterpret_cast<float2*>(dst + v * 8 + tig * 2) = make_float2(o[v][2], o[v][3]);
            if (tig == 0) { dst[D] = m1 * WM_LN2; dst[D + 1] = l1; }
        }
        return;
    }
    if (a.sink) {                        // the sink's share of the denominator, in the base-2 scale of the running maximum
        if (ok0) l0 += fast_ex2(a.sink[g * rep + s0 % rep] * WM_LOG2E - m0);
        if (ok1) l1 += fast_ex2(a.sink[g * rep + s1 % rep] * WM_LOG2E - m1);
    }
    if (ok0) {
        float* dst = a.out + (size_t)s_row[r0] * a.ldo + (size_t)(g * rep + s0 % rep) * D;
        const float inv = 1.f / l0;
#pragma unroll
        for (int v = 0; v < NV; ++v) *reinterpret_cast<float2*>(dst + v * 8 + tig * 2) = make_float2(o[v][0] * inv, o[v][1] * inv);
    }
    if (ok1) {
        float* dst = a.out + (size_t)s_row[r1] * a.ldo + (size_t)(g * rep + s1 % rep) * D;
        const float inv = 1.f / l1;
#pragma unroll
        for (int v = 0; v < NV; ++v) *reinterpret_cast<float2*>(dst + v * 8 + tig * 2) = make_float2(o[v][2] * inv, o[v][3] * inv);
    }
}

// merge of the page shares: one CTA per (tile, key/value head, position of the tile).  The shares' maxima and sums are
// gathered into shared memory, every (head, share) weight e^(m_k - m) / l is formed once, then a thread per (head,
// column) sums the shares.
#define WM_MAX_SPLITS 32
__global__ void __launch_bounds__(128) window_merge_kernel(DlWindowAttnArgs a, const int* __restrict__ tile_rows, int rq, int n_splits,
                                                           const float* __restrict__ partial) {
    __shared__ float w_s[WM_ROWS * WM_MAX_SPLITS], l_s[WM_ROWS * WM_MAX_SPLITS];
    const int tile = blockIdx.x, g = blockIdx.y, r = blockIdx.z, D = a.dim, rep = a.heads / a.kv_heads;
    const int m = tile_rows[(size_t)tile * rq + r];
    if (m < 0) return;
    const float* base = partial + ((size_t)tile * a.kv_heads + g) * n_splits * WM_ROWS * (D + 2);
    for (int idx = threadIdx.x; idx < rep * n_splits; idx += blockDim.x) {
        const int hg = idx / n_splits, k = idx - hg * n_splits;
        const float* p = base + ((size_t)k * WM_ROWS + r * rep + hg) * (D + 2);
        w_s[idx] = p[D];
        l_s[idx] = p[D + 1];
    }
    __syncthreads();
    for (int hg = threadIdx.x; hg < rep; hg += blockDim.x) {
        float mx = -INFINITY, l = 0.f;
        for (int k = 0; k < n_splits; ++k) mx = fmaxf(mx, w_s[hg * n_splits + k]);
        for (int k = 0; k < n_splits; ++k) {
            const float mk = w_s[hg * n_splits + k];
            const float e = mk == -INFINITY ? 0.f : expf(mk - mx);
            l += l_s[hg * n_splits + k] * e;
            w_s[hg * n_splits + k] = e;
        }
        if (a.sink) l += expf(a.sink[g * rep + hg] - mx);
        const float inv = 1.f / l;
        for (int k = 0; k < n_splits; ++k) w_s[hg * n_splits + k] *= inv;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < rep * D; idx += blockDim.x) {
        const int hg = idx / D, c = idx - hg * D;
        const float* p = base + (size_t)(r * rep + hg) * (D + 2) + c;
        float acc = 0.f;                      // a share without pages left zeros and weighs 0: every load can go out at once
#pragma unroll 8
        for (int k = 0; k < n_splits; ++k) acc = fmaf(w_s[hg * n_splits + k], p[(size_t)k * WM_ROWS * (D + 2)], acc);
        a.out[(size_t)m * a.ldo + (size_t)(g * rep + hg) * D + c] = acc;
    }
}

// rows of one sequence per tile: as many positions as fit 64 stacked (position, head) pairs
extern "C" int dl_window_tc_rows(int heads, int kv_heads) {
    if (heads < 1 || kv_heads < 1 || heads % kv_heads) return 0;
    const int rep = heads / kv_heads;
    return rep > WM_ROWS ? 0 : WM_ROWS / rep;
}

// 0 if the tensor-core kernel takes these sizes
extern "C" int dl_window_attention_tc_supported(int heads, int kv_heads, int dim, int rope_dims, int ctype) {
    if (ctype != DL_T_BF16 || dl_window_tc_rows(heads, kv_heads) == 0) return -1;
    if (dim % 16 != 0 || dim > 128 || dim / 16 == 5 || dim / 16 == 7 || rope_dims % 8 != 0 || rope_dims > dim) return -1;
    return 0;
}

// floats of the scratch that n_splits > 1 needs
extern "C" long long dl_window_tc_partial_floats(int n_tiles, int kv_heads, int n_splits, int dim) {
    return (long long)n_tiles * kv_heads * n_splits * WM_ROWS * (dim + 2);
}

// n_splits > 1 (few tiles, e.g. decoding): grid.z CTAs share a tile's pages and leave partial sums in `partial`
// (dl_window_tc_partial_floats() f32) that a merge launch combines.
extern "C" int dl_window_attention_tc(const DlWindowAttnArgs* args, const int* tile_rows, int n_tiles, int rq, int n_splits,
                                      float* partial, void* stream) {
    const DlWindowAttnArgs& a = *args;
    if (window_args_ok(a, "dl_window_attention_tc")) return -1;
    if (a.key_heads > 1) { dl_set_error("dl_window_attention_tc: head-mixed scores run on dl_talk_attention_tc"); return -1; }
    if (a.vdim > 0 && a.vdim != a.dim) { dl_set_error("dl_window_attention_tc: values of their own must be as wide as the keys (dim %d, vdim %d)", a.dim, a.vdim); return -1; }
    if (dl_window_attention_tc_supported(a.heads, a.kv_heads, a.dim, a.rope_dims, a.ctype) != 0 || rq < 1 || rq > dl_window_tc_rows(a.heads, a.kv_heads) ||
        (a.ldq & 3) || (a.ldo & 1) || ((uintptr_t)a.q & 15)) {
        dl_set_error("dl_window_attention_tc: sizes not supported (heads %d / %d, dim %d, rotary %d, rq %d)", a.heads, a.kv_heads, a.dim, a.rope_dims, rq);
        return -1;
    }
    if (n_tiles < 1) return 0;
    if (n_splits < 1 || n_splits > WM_MAX_SPLITS || (n_splits > 1 && partial == nullptr)) { dl_set_error("dl_window_attention_tc: n_splits %d without scratch", n_splits); return -1; }
    const size_t smem = ((size_t)2 * WA_PAGE * wm_line_stride(a.dim + (a.vdim > 0 ? a.vdim : a.rope_dims)) + (size_t)WM_ROWS * (a.dim + 8)) * sizeof(__nv_bfloat16);
    dim3 grid(n_tiles, a.kv_heads, n_splits);
    cudaStream_t st = (cudaStream_t)stream;
    switch (a.dim / 16) {
#define WM_CASE(DK_)                                                                                                      \
    case DK_:                                                                                                             \
        if (smem > 48 * 1024) cudaFuncSetAttribute(window_attention_mma_kernel<DK_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        window_attention_mma_kernel<DK_><<<grid, 128, smem, st>>>(a, tile_rows, rq, n_splits, partial);                  \
        break;
        WM_CASE(1) WM_CASE(2) WM_CASE(3) WM_CASE(4) WM_CASE(6) WM_CASE(8)
#undef WM_CASE
        default: dl_set_error("dl_window_attention_tc: dim %d", a.dim); return -1;
    }
    if (n_splits > 1) window_merge_kernel<<<dim3(n_tiles, a.kv_heads, rq), 128, 0, st>>>(a, tile_rows, rq, n_splits, partial);
    LAYER_CHECK_LAUNCH("dl_window_attention_tc");
    return 0;
}
