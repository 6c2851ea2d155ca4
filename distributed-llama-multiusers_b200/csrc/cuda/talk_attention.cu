// Grouped-query attention on the tensor cores whose values have a width of their own and whose scores may be mixed
// across heads before the softmax ("talking heads"):
//     s_g(i, j)  = scale * q_g,i . k_c(g),j                       c(g) = g / (heads / kv_heads)
//     s'_h(i, j) = sum_g talk[h][g] s_g(i, j)                     then mask, softmax, sink as in window_attention.cu
//     out_h(i)   = sum_j p_h(i, j) v_c(h),j
// The mix is linear in the queries, so the cache writer (attn_kv_write_kernel) folds it into them:
//     s'_h(i, j) = scale * sum_c Q_h,i[c] . k_c,j,     Q_h,i[c] = sum_{g: c(g) = c} talk[h][g] q_g,i
// -- head h carries ONE query of key_heads * dim numbers that meets the keys of ALL key/value heads side by side, and
// the kernel is an ordinary attention tile kernel whose K dimension is key_heads * dim: nothing is exchanged between
// heads here.  key_heads <= 1 is plain grouped-query attention (the query meets its own group's key only).
//
// Cache [page][kv_head][32][dim + vdim] bf16, one line = key | value.  A CTA owns a tile of up to `rq` consecutive
// positions of one sequence and the query heads of ONE key/value head g: (position, head-of-the-group) pairs stack on the
// M dimension, NR warps x 16 stacked rows: NR = 8 (256 threads, 128 stacked rows) for long portions, where a staged page
// serves twice the queries; 4 for medium ones; 1 for decoding (one warp multiplies, all four stage; the small query tile
// lets two CTAs share an SM).  Decoding with 2 to 8 key/value heads runs the ALLG form instead: ONE CTA per tile, warp g
// multiplies the heads of key/value head g, and the page staged for all of them holds every head's keys and values once.  Per page of 32 tokens it stages the keys of every key/value head and the values
// of head g (cp.async, two buffers: page k + 1 is in flight while page k is multiplied), then per warp
//     S[16 x 32]  = Q[16 x KH * DP] . K[32 x KH * DP]^T      Q (bf16, staged once per tile) and K by ldmatrix
//     scale, mask, online softmax in f32 and base 2
//     O[16 x DVP] += P[16 x 32] . V[32 x DVP]                  P from the score registers, V by ldmatrix.trans
// mma.sync m16n8k16 bf16, f32 accumulators.  DP / DVP: dim / vdim rounded up to the template's sizes, the padding kept at
// zero in shared memory.  Few tiles (decoding): n_splits CTAs share a tile's pages and talk_merge_kernel combines them.
#include "mma_common.cuh"
#include "../../../include/dllama_b200.h"

#define TA_PAGE 32
#define TA_MAX_ROWS 128
#define TA_MAX_SPLITS 32
#define TA_LOG2E 1.4426950408889634f
#define TA_LN2 0.6931471805599453f

__device__ __forceinline__ float ta_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__host__ __device__ __forceinline__ int ta_stride(int n) {      // bf16 elements; rows 16 B apart modulo 128 B
    int s = (n + 7) / 8 * 8 + 8;
    if ((s * 2) % 128 == 0) s += 8;
    return s;
}

template <int DK, int NV, int NR, bool ALLG>
__global__ void __launch_bounds__((NR == 8 || ALLG) ? 256 : 128) talk_attention_mma_kernel(DlWindowAttnArgs a, const int* __restrict__ tile_rows, int rq, int n_splits,
                                                                float* __restrict__ partial) {
    constexpr int DP = 16 * DK, DVP = 8 * NV, TA_ROWS = 16 * NR;
    const int THREADS = blockDim.x;
    extern __shared__ __align__(16) uint8_t smraw[];
    __shared__ int s_row[TA_ROWS];
    const int D = a.dim, DV = a.vdim, LD = D + DV;
    const int KH = a.key_heads > 1 ? a.key_heads : 1, QD = KH * D, QDP = KH * DP;
    // staged line: [ keys of KS heads | values of VS heads ]; ALLG: every head's, else all (or this group's) keys and this group's values
    const int KS = ALLG ? a.kv_heads : KH, VS = ALLG ? a.kv_heads : 1, VOFF = KS * DP;
    const int LDS = ta_stride(VOFF + VS * DVP), QS = ta_stride(QDP);
    __nv_bfloat16* kv_s = reinterpret_cast<__nv_bfloat16*>(smraw);                  // [2][TA_PAGE][LDS]
    __nv_bfloat16* q_s = kv_s + (size_t)2 * TA_PAGE * LDS;                          // [TA_ROWS (ALLG: per key/value head)][QS]: the stacked queries
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
    // grid (key/value heads, tiles, page shares).  A sequence's later tiles walk more pages: they start first, so that the
    // short ones fill the SMs at the end
    const int tile = (int)gridDim.y - 1 - (int)blockIdx.y, rep = a.heads / a.kv_heads;
    const int g = ALLG ? min(warp, a.kv_heads - 1) : (int)blockIdx.x;              // ALLG: warp g multiplies key/value head g
    const int wrow = ALLG ? 0 : warp;                                               // this warp's block of 16 stacked rows among its group's
    const int qrow0 = ALLG ? g * 16 : warp * 16;                                    // ... and where that block's queries sit in q_s
    if (threadIdx.x < rq) s_row[threadIdx.x] = tile_rows[(size_t)tile * rq + threadIdx.x];
    // the padding of keys and values stays zero: the copies below never touch it
    if (D != DP || DV != DVP)
        for (int i = threadIdx.x; i < 2 * TA_PAGE * LDS / 8; i += THREADS) reinterpret_cast<uint4*>(kv_s)[i] = make_uint4(0u, 0u, 0u, 0u);
    __syncthreads();
    int n_rows = 0;
    while (n_rows < rq && s_row[n_rows] >= 0) ++n_rows;
    if (n_rows == 0) return;
    const int p_first = a.pos[s_row[0]], p_last = p_first + n_rows - 1, slot = a.slot[s_row[0]];
    int lo = a.window > 0 ? max(0, p_first - a.window + 1) : 0;
    if (a.chunk > 0) lo = max(lo, p_first / a.chunk * a.chunk);
    int pg_lo = lo / TA_PAGE, pg_hi = p_last / TA_PAGE;
    if (n_splits > 1) {                  // this CTA's share of the tile's pages (possibly none)
        const int per = (pg_hi - pg_lo + n_splits) / n_splits;
        pg_lo += (int)blockIdx.z * per;
        pg_hi = min(pg_hi, pg_lo + per - 1);
    }
    const bool active = ALLG ? warp < a.kv_heads : (warp < NR && warp * 16 < n_rows * rep);
    const float c1 = a.scale * TA_LOG2E;

    // this thread's two stacked rows: s = position-in-tile * rep + head-in-group
    const int s0 = wrow * 16 + gid, s1 = s0 + 8;
    const int r0 = s0 / rep, r1 = s1 / rep;
    const bool ok0 = r0 < n_rows, ok1 = r1 < n_rows;
    const int pos0 = p_first + r0, pos1 = p_first + r1;
    const int cs0 = a.chunk > 0 ? pos0 / a.chunk * a.chunk : 0, cs1 = a.chunk > 0 ? pos1 / a.chunk * a.chunk : 0;
    const int cs_last = a.chunk > 0 ? p_last / a.chunk * a.chunk : 0;
    // the tile's queries, rounded to bf16, zero-padded per key head
    for (int idx = threadIdx.x; idx < (ALLG ? a.kv_heads : 1) * TA_ROWS * (QDP / 4); idx += THREADS) {
        const int sr = idx / (QDP / 4), col = (idx - sr * (QDP / 4)) * 4;
        const int gq = ALLG ? sr / TA_ROWS : g, sg = ALLG ? sr % TA_ROWS : sr;      // key/value head and stacked row within it
        const int c = col / DP, d = col - c * DP, r = sg / rep;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < n_rows && d < D) v = *reinterpret_cast<const float4*>(a.q + (size_t)s_row[r] * a.ldq + (size_t)(gq * rep + sg % rep) * QD + c * D + d);
        uint2 pk;
        pk.x = pack_bf16(v.x, v.y);
        pk.y = pack_bf16(v.z, v.w);
        *reinterpret_cast<uint2*>(q_s + (size_t)sr * QS + col) = pk;
    }
    float o[NV][4];
#pragma unroll
    for (int v = 0; v < NV; ++v) { o[v][0] = o[v][1] = o[v][2] = o[v][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    // staging: THREADS / 32 threads share a cache line's chunks of 16 bytes, head after head (no index arithmetic per chunk)
    const int kch = D / 8, vch = DV / 8, TPL = THREADS / TA_PAGE;
    const int sj = threadIdx.x / TPL, sl = threadIdx.x - sj * TPL;                  // this thread's line of a page and its lane among the line's threads
    auto issue = [&](int pg, int buf) {
        const int page = a.block_table[(size_t)slot * a.max_pages + pg];
        const __nv_bfloat16* src0 = (const __nv_bfloat16*)a.cache + ((size_t)page * a.kv_heads * TA_PAGE + sj) * LD;      // head c: + c * TA_PAGE * LD
        __nv_bfloat16* dst = kv_s + (size_t)buf * TA_PAGE * LDS + (size_t)sj * LDS;
        for (int c = 0; c < KS; ++c) {
            const __nv_bfloat16* sk = src0 + (size_t)(KS > 1 ? c : g) * TA_PAGE * LD;
            for (int p = sl; p < kch; p += TPL) cp_async16(dst + c * DP + p * 8, sk + p * 8);
        }
        for (int c = 0; c < VS; ++c) {
            const __nv_bfloat16* sv = src0 + (size_t)(ALLG ? c : g) * TA_PAGE * LD + D;
            for (int p = sl; p < vch; p += TPL) cp_async16(dst + VOFF + c * DVP + p * 8, sv + p * 8);
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
        const __nv_bfloat16* kv = kv_s + (size_t)buf * TA_PAGE * LDS;
        float sc[4][4];
#pragma unroll
        for (int n = 0; n < 4; ++n) { sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f; }
        const int kcol0 = (ALLG && KH == 1) ? g * DP : 0;      // plain grouped-query attention in the ALLG form: the group's own key among all staged
        for (int c = 0; c < KH; ++c) {
#pragma unroll
            for (int kk = 0; kk < DK; ++kk) {
                uint32_t qf[4];
                ldmatrix_x4(qf, q_s + (size_t)(qrow0 + (mat & 1) * 8 + rr) * QS + c * DP + kk * 16 + (mat >> 1) * 8);
#pragma unroll
                for (int np = 0; np < 2; ++np) {
                    uint32_t b[4];
                    ldmatrix_x4(b, kv + (size_t)(np * 16 + (mat >> 1) * 8 + rr) * LDS + kcol0 + c * DP + kk * 16 + (mat & 1) * 8);
                    mma_bf16(sc[2 * np], qf, b[0], b[1]);
                    mma_bf16(sc[2 * np + 1], qf, b[2], b[3]);
                }
            }
        }
        // scale (base-2 scores) and mask (skipped on pages that every row of the tile sees whole)
        const int pg_first = pg * TA_PAGE;
        const bool whole = pg_first + TA_PAGE - 1 <= p_first && (a.window == 0 || p_last - pg_first < a.window) && pg_first >= cs_last;
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int n = 0; n < 4; ++n) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float s2 = sc[n][e] * c1;
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
        const float al0 = (m0 == -INFINITY) ? 0.f : ta_ex2(m0 - mn0), al1 = (m1 == -INFINITY) ? 0.f : ta_ex2(m1 - mn1);
        const float ref0 = (mn0 == -INFINITY) ? 0.f : mn0, ref1 = (mn1 == -INFINITY) ? 0.f : mn1;      // a row that sees nothing yet: every p = 0
        m0 = mn0; m1 = mn1;
        float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
        for (int n = 0; n < 4; ++n) {
            sc[n][0] = ta_ex2(sc[n][0] - ref0); sc[n][1] = ta_ex2(sc[n][1] - ref0);
            sc[n][2] = ta_ex2(sc[n][2] - ref1); sc[n][3] = ta_ex2(sc[n][3] - ref1);
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
                uint32_t b[4];
                ldmatrix_x4_trans(b, kv + (size_t)(ks * 16 + (mat & 1) * 8 + rr) * LDS + VOFF + (ALLG ? g * DVP : 0) + vt * 8);
                mma_bf16(o[2 * vp], pa, b[0], b[1]);
                mma_bf16(o[2 * vp + 1], pa, b[2], b[3]);
            }
        }
    }
    if (!active) return;
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    if (n_splits > 1) {                  // unnormalised sums, running maximum and sum per stacked row, for the merge kernel
        float* base = partial + (((size_t)tile * a.kv_heads + g) * n_splits + blockIdx.z) * TA_ROWS * (DVP + 2);
        if (ok0) {
            float* dst = base + (size_t)s0 * (DVP + 2);
#pragma unroll
            for (int v = 0; v < NV; ++v) *reinterpret_cast<float2*>(dst + v * 8 + tig * 2) = make_float2(o[v][0], o[v][1]);
            if (tig == 0) { dst[DVP] = m0 * TA_LN2; dst[DVP + 1] = l0; }
        }
        if (ok1) {
            float* dst = base + (size_t)s1 * (DVP + 2);
#pragma unroll
            for (int v = 0; v < NV; ++v) *reinterpret_cast<float2*>(dst + v * 8 + tig * 2) = make_float2(o[v][2], o[v][3]);
            if (tig == 0) { dst[DVP] = m1 * TA_LN2; dst[DVP + 1] = l1; }
        }
        return;
    }
    if (a.sink) {                        // the sink's share of the denominator, in the base-2 scale of the running maximum
        if (ok0) l0 += ta_ex2(a.sink[g * rep + s0 % rep] * TA_LOG2E - m0);
        if (ok1) l1 += ta_ex2(a.sink[g * rep + s1 % rep] * TA_LOG2E - m1);
    }
    if (ok0) {
        float* dst = a.out + (size_t)s_row[r0] * a.ldo + (size_t)(g * rep + s0 % rep) * DV;
        const float inv = 1.f / l0;
#pragma unroll
        for (int v = 0; v < NV; ++v)
            if (v * 8 < DV) *reinterpret_cast<float2*>(dst + v * 8 + tig * 2) = make_float2(o[v][0] * inv, o[v][1] * inv);
    }
    if (ok1) {
        float* dst = a.out + (size_t)s_row[r1] * a.ldo + (size_t)(g * rep + s1 % rep) * DV;
        const float inv = 1.f / l1;
#pragma unroll
        for (int v = 0; v < NV; ++v)
            if (v * 8 < DV) *reinterpret_cast<float2*>(dst + v * 8 + tig * 2) = make_float2(o[v][2] * inv, o[v][3] * inv);
    }
}

// merge of the page shares: one CTA per (tile, key/value head, position of the tile).  The shares' maxima and sums are
// gathered into shared memory, every (head, share) weight e^(m_k - m) / l is formed once, then a thread per (head,
// column) sums the shares.
__global__ void __launch_bounds__(128) talk_merge_kernel(DlWindowAttnArgs a, const int* __restrict__ tile_rows, int rq, int n_splits,
                                                         const float* __restrict__ partial, int DVP, int TA_ROWS) {
    __shared__ float w_s[64 * TA_MAX_SPLITS], l_s[64 * TA_MAX_SPLITS];      // heads of one group x shares
    const int tile = blockIdx.x, g = blockIdx.y, r = blockIdx.z, DV = a.vdim, rep = a.heads / a.kv_heads;
    const int m = tile_rows[(size_t)tile * rq + r];
    if (m < 0) return;
    const float* base = partial + ((size_t)tile * a.kv_heads + g) * n_splits * TA_ROWS * (DVP + 2);
    for (int idx = threadIdx.x; idx < rep * n_splits; idx += blockDim.x) {
        const int hg = idx / n_splits, k = idx - hg * n_splits;
        const float* p = base + ((size_t)k * TA_ROWS + r * rep + hg) * (DVP + 2);
        w_s[idx] = p[DVP];
        l_s[idx] = p[DVP + 1];
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
    for (int idx = threadIdx.x; idx < rep * DV; idx += blockDim.x) {
        const int hg = idx / DV, c = idx - hg * DV;
        const float* p = base + (size_t)(r * rep + hg) * (DVP + 2) + c;
        float acc = 0.f;                      // a share without pages left zeros and weighs 0: every load can go out at once
#pragma unroll 8
        for (int k = 0; k < n_splits; ++k) acc = fmaf(w_s[hg * n_splits + k], p[(size_t)k * TA_ROWS * (DVP + 2)], acc);
        a.out[(size_t)m * a.ldo + (size_t)(g * rep + hg) * DV + c] = acc;
    }
}

static int ta_dk(int dim) { return dim <= 32 ? 2 : dim <= 64 ? 4 : 8; }
static int ta_nv(int vdim) { return vdim <= 64 ? 8 : vdim <= 96 ? 12 : 16; }
static size_t ta_smem(int dim, int vdim, int key_heads, int rows) {
    const int KH = key_heads > 1 ? key_heads : 1, QDP = KH * 16 * ta_dk(dim);
    return ((size_t)2 * TA_PAGE * ta_stride(QDP + 8 * ta_nv(vdim)) + (size_t)rows * ta_stride(QDP)) * sizeof(__nv_bfloat16);
}
// the ALLG form: every head's keys and values in a staged line, 16 stacked rows of queries per key/value head
static size_t ta_smem_allg(int dim, int vdim, int key_heads, int kv_heads) {
    const int KH = key_heads > 1 ? key_heads : 1, DP = 16 * ta_dk(dim);
    return ((size_t)2 * TA_PAGE * ta_stride(kv_heads * (DP + 8 * ta_nv(vdim))) + (size_t)kv_heads * 16 * ta_stride(KH * DP)) * sizeof(__nv_bfloat16);
}
#define TA_SMEM_MAX (220 * 1024)
static bool ta_allg(int kv_heads, int dim, int vdim, int key_heads) {
    return kv_heads >= 2 && kv_heads <= 8 && ta_smem_allg(dim, vdim, key_heads, kv_heads) <= TA_SMEM_MAX;
}

// Stacked rows of a tile for portions of `longest` rows of a sequence: 128 where long portions fit the shared memory, 16
// for decoding (at most 16 query heads per key/value head), else 64; 0: the sizes do not fit at all.
extern "C" int dl_talk_tc_tile_rows(int heads, int kv_heads, int dim, int vdim, int key_heads, int longest) {
    if (heads < 1 || kv_heads < 1 || heads % kv_heads) return 0;
    const int rep = heads / kv_heads;
    if (rep <= 16 && longest <= 16 / rep && ta_smem(dim, vdim, key_heads, 16) <= TA_SMEM_MAX) return 16;
    if (rep <= 128 && longest > 64 / rep && ta_smem(dim, vdim, key_heads, 128) <= TA_SMEM_MAX) return 128;
    if (rep <= 64 && ta_smem(dim, vdim, key_heads, 64) <= TA_SMEM_MAX) return 64;
    return 0;
}

// 0 if the kernel takes these sizes: a bf16 cache, dim and vdim multiples of 8 up to 128, at most 64 query heads per
// key/value head, and a tile's queries plus two pages of all key heads within the shared memory of an SM
extern "C" int dl_talk_attention_tc_supported(int heads, int kv_heads, int dim, int vdim, int key_heads, int ctype) {
    if (ctype != DL_T_BF16 || heads < 1 || kv_heads < 1 || heads % kv_heads || heads / kv_heads > 64) return -1;
    if (dim < 8 || dim % 8 || dim > 128 || vdim < 8 || vdim % 8 || vdim > 128) return -1;
    if (key_heads > 1 && key_heads != kv_heads) return -1;
    if (ta_smem(dim, vdim, key_heads, 64) > TA_SMEM_MAX) return -1;
    return 0;
}

// partial sums of the page shares: tiles x key/value heads x shares x stacked rows (rq rows x heads of a group, rounded up
// to the kernel's 16, 64 or 128)
static int ta_rows_of(int rq, int rep) { return rq * rep <= 16 ? 16 : rq * rep <= 64 ? 64 : 128; }
extern "C" long long dl_talk_tc_partial_floats(int n_tiles, int kv_heads, int n_splits, int vdim, int rows) {
    return (long long)n_tiles * kv_heads * n_splits * rows * (8 * ta_nv(vdim) + 2);
}

template <int DK, int NV, int NR, bool ALLG>
static int launch_talk_nr(const DlWindowAttnArgs& a, const int* tile_rows, int n_tiles, int rq, int n_splits, float* partial, cudaStream_t st) {
    const size_t smem = ALLG ? ta_smem_allg(a.dim, a.vdim, a.key_heads, a.kv_heads) : ta_smem(a.dim, a.vdim, a.key_heads, 16 * NR);
    if (smem > TA_SMEM_MAX) { dl_set_error("dl_talk_attention_tc: %zu bytes of shared memory", smem); return -1; }
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(talk_attention_mma_kernel<DK, NV, NR, ALLG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) { dl_set_error("dl_talk_attention_tc: shared memory attribute: %s", cudaGetErrorString(e)); return -(int)e; }
    }
    const dim3 grid(ALLG ? 1 : a.kv_heads, n_tiles, n_splits);
    const int threads = ALLG ? (a.kv_heads > 4 ? 256 : 128) : (NR == 8 ? 256 : 128);
    talk_attention_mma_kernel<DK, NV, NR, ALLG><<<grid, threads, smem, st>>>(a, tile_rows, rq, n_splits, partial);
    return 0;
}

template <int DK, int NV>
static int launch_talk(const DlWindowAttnArgs& a, const int* tile_rows, int n_tiles, int rq, int n_splits, float* partial, cudaStream_t st) {
    const int rows = ta_rows_of(rq, a.heads / a.kv_heads);
    // many small tiles (batched decoding): one CTA per tile stages every head's keys and values once; few (one stream): a CTA
    // per key/value head, so that more SMs share the pages
    if (rows == 16 && n_tiles * a.kv_heads * n_splits >= 512 && ta_allg(a.kv_heads, a.dim, a.vdim, a.key_heads)) return launch_talk_nr<DK, NV, 1, true>(a, tile_rows, n_tiles, rq, n_splits, partial, st);
    if (rows == 16) return launch_talk_nr<DK, NV, 1, false>(a, tile_rows, n_tiles, rq, n_splits, partial, st);
    if (rows == 64) return launch_talk_nr<DK, NV, 4, false>(a, tile_rows, n_tiles, rq, n_splits, partial, st);
    return launch_talk_nr<DK, NV, 8, false>(a, tile_rows, n_tiles, rq, n_splits, partial, st);
}

// tile_rows[n_tiles][rq] (device; -1 where a tile has fewer rows): up to rq consecutive rows of one sequence per tile,
// rq * (heads / kv_heads) <= 128 stacked rows (dl_talk_tc_tile_rows() / (heads / kv_heads) is the rq to use).
// q: [M][heads][max(key_heads, 1) * dim].  n_splits > 1: that many CTAs share each tile's pages and leave partial sums in
// `partial` (dl_talk_tc_partial_floats() f32) that a merge launch combines.
extern "C" int dl_talk_attention_tc(const DlWindowAttnArgs* args, const int* tile_rows, int n_tiles, int rq, int n_splits,
                                    float* partial, void* stream) {
    const DlWindowAttnArgs& a = *args;
    if (a.page_size != TA_PAGE || a.softcap != 0.f || a.rope_dims != 0 || a.window < 0 || a.chunk < 0 ||
        dl_talk_attention_tc_supported(a.heads, a.kv_heads, a.dim, a.vdim, a.key_heads, a.ctype) != 0 || rq < 1 ||
        rq * (a.heads / a.kv_heads) > TA_MAX_ROWS || (a.ldq & 3) || (a.ldo & 1) || ((uintptr_t)a.q & 15) || ((uintptr_t)a.out & 7)) {
        dl_set_error("dl_talk_attention_tc: sizes not supported (heads %d / %d, dim %d, vdim %d, key heads %d, rq %d)", a.heads, a.kv_heads, a.dim, a.vdim, a.key_heads, rq);
        return -1;
    }
    if (n_tiles < 1) return 0;
    if (n_tiles > 65535) { dl_set_error("dl_talk_attention_tc: %d tiles in one launch", n_tiles); return -1; }
    if (n_splits < 1 || n_splits > TA_MAX_SPLITS || (n_splits > 1 && partial == nullptr)) { dl_set_error("dl_talk_attention_tc: n_splits %d without scratch", n_splits); return -1; }
    cudaStream_t st = (cudaStream_t)stream;
    const int dk = ta_dk(a.dim), nv = ta_nv(a.vdim);
    int rc = -1;
#define TA_CASE(DK_, NV_) if (dk == DK_ && nv == NV_) rc = launch_talk<DK_, NV_>(a, tile_rows, n_tiles, rq, n_splits, partial, st);
    TA_CASE(2, 8) TA_CASE(2, 12) TA_CASE(2, 16)
    TA_CASE(4, 8) TA_CASE(4, 12) TA_CASE(4, 16)
    TA_CASE(8, 8) TA_CASE(8, 12) TA_CASE(8, 16)
#undef TA_CASE
    if (rc != 0) return rc;
    if (n_splits > 1)
        talk_merge_kernel<<<dim3(n_tiles, a.kv_heads, rq), 128, 0, st>>>(a, tile_rows, rq, n_splits, partial, 8 * nv, ta_rows_of(rq, a.heads / a.kv_heads));
    LAYER_CHECK_LAUNCH("dl_talk_attention_tc");
    return 0;
}
