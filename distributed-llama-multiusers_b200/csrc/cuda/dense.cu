// Dense (unquantised) weights: embedding gather and  Y[M][N] = epi(X[M][K] . W[N][K]^T)  for bf16 or f32 weights,
// f32 activations, f32 accumulation.  Two kernels: a weight-streaming one for up to 8 rows (decode: every weight
// byte is read once, lanes stride K) and a shared-memory tiled one for more rows.  Both take a batch dimension
// (grid.z) with element strides, which is how per-head products (a head's slice of a weight against a head's slice
// of the activations) run as one launch.  In bf16 mode (`round_x`) the activation operand is rounded to bf16 on
// load, so products are exact in f32 and only the accumulation order differs from a tensor-core product.
//
// Epilogues (what other models of this library fuse into their matmul kernels too): plain store, relu(.)^2,
// aux * sigmoid(.) (an output gate), cap * tanh(. / cap) (logit soft-capping), . * sigmoid(.) (SiLU), aux * (.) (the second
// half of a gated unit), xIELU (a quadratic for z > 0, an exponential for z <= 0, two constants), and a sum into Y behind one
// sigmoid gate per row.
#include "layer_common.cuh"
#include "../../../include/dllama_b200.h"

__device__ __forceinline__ float dense_epi(float acc, int epi, float aux, float param, float param2) {
    switch (epi) {
        case DL_DENSE_RELU2: { const float r = fmaxf(acc, 0.f); return r * r; }
        case DL_DENSE_SIGMOID_MUL: return aux * sigmoid_f(acc);
        case DL_DENSE_SOFTCAP: return param * tanhf(acc / param);
        case DL_DENSE_SILU: return silu_f(acc);
        case DL_DENSE_MUL: return aux * acc;
        case DL_DENSE_XIELU: return acc > 0.f ? fmaf(param * acc, acc, 0.5f * acc) : fmaf(param2, expm1f(acc) - acc, 0.5f * acc);
        default: return acc;
    }
}

// element (m, n) of batch b leaves through the epilogue; the row-gated sum reads what Y holds first
__device__ __forceinline__ void dense_store(const DlDenseArgs& a, int b, int m, int n, float acc) {
    float* y = a.Y + (size_t)b * a.y_bs + (size_t)m * a.ldy + n;
    if (a.epi == DL_DENSE_ROWGATE_ADD) {
        *y = fmaf(sigmoid_f(a.aux[(size_t)b * a.aux_bs + (size_t)m * a.ld_aux]), acc, *y);
        return;
    }
    const float aux = a.aux ? a.aux[(size_t)b * a.aux_bs + (size_t)m * a.ld_aux + n] : 0.f;
    *y = dense_epi(acc, a.epi, aux, a.param, a.param2);
}

// ------------------------------------------------------------------------------------------------
// embedding gather: x[m][c] = scale * table[tokens[m]] for each of `copies` copies of the row (row layout [copies][dim])
// ------------------------------------------------------------------------------------------------
template <typename WT>
__global__ void embed_rows_kernel(const WT* __restrict__ table, const int* __restrict__ tokens, float* __restrict__ x, int dim,
                                  float scale, int copies) {
    const int m = blockIdx.x;
    const WT* src = table + (size_t)tokens[m] * dim;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float v = ld_f(src + i) * scale;
        for (int c = 0; c < copies; ++c) x[((size_t)m * copies + c) * dim + i] = v;
    }
}

extern "C" int dl_embed_rows(const void* table, int wtype, const int* tokens, float* x, int M, int dim, float scale, int copies,
                             void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    if (copies < 1) { dl_set_error("dl_embed_rows: copies < 1"); return -1; }
    if (wtype == DL_T_BF16) embed_rows_kernel<<<M, 128, 0, st>>>((const __nv_bfloat16*)table, tokens, x, dim, scale, copies);
    else embed_rows_kernel<<<M, 128, 0, st>>>((const float*)table, tokens, x, dim, scale, copies);
    LAYER_CHECK_LAUNCH("dl_embed_rows");
    return 0;
}

// ------------------------------------------------------------------------------------------------
// rows <= 8: one warp per output column, lanes stride K, MT accumulators per lane
// ------------------------------------------------------------------------------------------------
#define GV_WARPS 8

template <typename WT, int MT, bool RX>
__global__ void __launch_bounds__(GV_WARPS * 32) dense_gemv_kernel(DlDenseArgs a) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * GV_WARPS + warp;
    const int b = blockIdx.z;
    if (n >= a.N) return;
    const WT* w = (const WT*)a.W + (size_t)b * a.w_bs + (size_t)n * a.ldw;
    const float* x = a.X + (size_t)b * a.x_bs;
    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.f;
    for (int k = lane; k < a.K; k += 32) {
        const float wv = ld_f(w + k);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m < a.M) {
                float xv = x[(size_t)m * a.ldx + k];
                if (RX) xv = round_bf16(xv);
                acc[m] = fmaf(xv, wv, acc[m]);
            }
        }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = warp_sum(acc[m]);
    if (lane == 0) {
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m < a.M) dense_store(a, b, m, n, acc[m]);
        }
    }
}

// vectorised variant: K % 8 == 0, rows 16-byte aligned (checked on the host)
template <typename WT> struct WVec;
template <> struct WVec<float> {
    static __device__ __forceinline__ void load8(const float* p, float* o) {
        const float4 u = *reinterpret_cast<const float4*>(p), v = *reinterpret_cast<const float4*>(p + 4);
        o[0] = u.x; o[1] = u.y; o[2] = u.z; o[3] = u.w; o[4] = v.x; o[5] = v.y; o[6] = v.z; o[7] = v.w;
    }
};
template <> struct WVec<__nv_bfloat16> {
    static __device__ __forceinline__ void load8(const __nv_bfloat16* p, float* o) {
        const uint4 u = *reinterpret_cast<const uint4*>(p);
        const uint32_t r[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            o[2 * i] = __uint_as_float(r[i] << 16);
            o[2 * i + 1] = __uint_as_float(r[i] & 0xffff0000u);
        }
    }
};

template <typename WT, int MT, bool RX>
__global__ void __launch_bounds__(GV_WARPS * 32) dense_gemv_vec_kernel(DlDenseArgs a) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * GV_WARPS + warp;
    const int b = blockIdx.z;
    if (n >= a.N) return;
    const WT* w = (const WT*)a.W + (size_t)b * a.w_bs + (size_t)n * a.ldw;
    const float* x = a.X + (size_t)b * a.x_bs;
    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.f;
    for (int k = lane * 8; k < a.K; k += 256) {
        float wv[8];
        WVec<WT>::load8(w + k, wv);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m < a.M) {
                float xv[8];
                WVec<float>::load8(x + (size_t)m * a.ldx + k, xv);
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[m] = fmaf(RX ? round_bf16(xv[i]) : xv[i], wv[i], acc[m]);
            }
        }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = warp_sum(acc[m]);
    if (lane == 0) {
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m < a.M) dense_store(a, b, m, n, acc[m]);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// more rows: 64 x 64 output tile per CTA, 16-wide K steps through shared memory, 4 x 4 outputs per thread
// ------------------------------------------------------------------------------------------------
#define GT_BM 64
#define GT_BN 64
#define GT_BK 16

template <typename WT, bool RX>
__global__ void __launch_bounds__(256) dense_tile_kernel(DlDenseArgs a) {
    __shared__ float Xs[GT_BK][GT_BM + 1];
    __shared__ float Ws[GT_BK][GT_BN + 1];
    const int b = blockIdx.z;
    const WT* W = (const WT*)a.W + (size_t)b * a.w_bs;
    const float* X = a.X + (size_t)b * a.x_bs;
    const int m0 = blockIdx.y * GT_BM, n0 = blockIdx.x * GT_BN;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < a.K; k0 += GT_BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = threadIdx.x + i * 256;
            const int r = idx >> 4, k = idx & 15;
            float xv = 0.f, wv = 0.f;
            if (k0 + k < a.K) {
                if (m0 + r < a.M) xv = X[(size_t)(m0 + r) * a.ldx + k0 + k];
                if (n0 + r < a.N) wv = ld_f(W + (size_t)(n0 + r) * a.ldw + k0 + k);
            }
            Xs[k][r] = RX ? round_bf16(xv) : xv;
            Ws[k][r] = wv;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < GT_BK; ++k) {
            float xr[4], wr[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { xr[i] = Xs[k][ty * 4 + i]; wr[i] = Ws[k][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(xr[i], wr[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= a.M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= a.N) continue;
            dense_store(a, b, m, n, acc[i][j]);
        }
    }
}

template <typename WT, bool RX>
static void launch_dense(const DlDenseArgs& a, cudaStream_t st) {
    if (a.M <= 8) {
        const bool vec = a.K % 8 == 0 && a.ldw % 8 == 0 && a.w_bs % 8 == 0 && a.ldx % 4 == 0 && a.x_bs % 4 == 0 &&
                         ((uintptr_t)a.W & 15) == 0 && ((uintptr_t)a.X & 15) == 0;
        dim3 grid((a.N + GV_WARPS - 1) / GV_WARPS, 1, a.batch);
        const int mt = a.M <= 1 ? 1 : a.M <= 2 ? 2 : a.M <= 4 ? 4 : 8;
#define GV_CASE(MT_)                                                                                   \
    case MT_:                                                                                          \
        if (vec) dense_gemv_vec_kernel<WT, MT_, RX><<<grid, GV_WARPS * 32, 0, st>>>(a);                \
        else dense_gemv_kernel<WT, MT_, RX><<<grid, GV_WARPS * 32, 0, st>>>(a);                        \
        break;
        switch (mt) { GV_CASE(1) GV_CASE(2) GV_CASE(4) GV_CASE(8) }
#undef GV_CASE
    } else {
        dim3 grid((a.N + GT_BN - 1) / GT_BN, (a.M + GT_BM - 1) / GT_BM, a.batch);
        dense_tile_kernel<WT, RX><<<grid, 256, 0, st>>>(a);
    }
}

extern "C" int dl_dense(const DlDenseArgs* args, void* stream) {
    const DlDenseArgs& a = *args;
    if (a.M < 1 || a.N < 1 || a.K < 1 || a.batch < 1) { dl_set_error("dl_dense: empty problem"); return -1; }
    if ((a.epi == DL_DENSE_SIGMOID_MUL || a.epi == DL_DENSE_MUL || a.epi == DL_DENSE_ROWGATE_ADD) && a.aux == nullptr) { dl_set_error("dl_dense: the gate epilogue needs aux"); return -1; }
    if (a.epi == DL_DENSE_GLU_CLAMP || a.epi == DL_DENSE_GLU_SILU) { dl_set_error("dl_dense: the paired-column epilogue belongs to the tensor-core GEMM"); return -1; }
    cudaStream_t st = (cudaStream_t)stream;
    if (a.wtype == DL_T_BF16) {
        if (a.round_x) launch_dense<__nv_bfloat16, true>(a, st);
        else launch_dense<__nv_bfloat16, false>(a, st);
    } else if (a.wtype == DL_T_F32) {
        if (a.round_x) launch_dense<float, true>(a, st);
        else launch_dense<float, false>(a, st);
    } else {
        dl_set_error("dl_dense: unknown weight type %d", a.wtype);
        return -1;
    }
    LAYER_CHECK_LAUNCH("dl_dense");
    return 0;
}

// ------------------------------------------------------------------------------------------------
// operand images of the tcgen05 GEMM (gemm_wh_tc.cu) for bf16 weights: element (row, k) of a 128 x 128 tile lives at
//   (row >> 3) * 2048 + (k >> 3) * 128 + (row & 7) * 16 + (k & 7) * 2      (8 x 16 B core matrices, K-major)
// weights: tiles [row_tile][k_tile][32 KB]; activations: [k_tile][ncap / 8][2048 B].  One thread per 8 K values.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) wh_from_dense_kernel(const __nv_bfloat16* __restrict__ w, int N, int K, long long ldw,
                                                            uint8_t* __restrict__ wh, int KT) {
    const int tile = blockIdx.x, rt = tile / KT, kt = tile % KT;
    uint8_t* out = wh + (size_t)tile * 32768;
    for (int i = threadIdx.x; i < 128 * 16; i += blockDim.x) {
        const int r = i >> 4, c = i & 15;
        const int row = rt * 128 + r, k0 = kt * 128 + c * 8;
        __align__(16) __nv_bfloat16 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = (row < N && k0 + j < K) ? w[(size_t)row * ldw + k0 + j] : __float2bfloat16_rn(0.f);
        *reinterpret_cast<uint4*>(out + (size_t)(r >> 3) * 2048 + c * 128 + (r & 7) * 16) = *reinterpret_cast<const uint4*>(v);
    }
}

__global__ void __launch_bounds__(256) xh_from_rows_kernel(const float* __restrict__ x, long long ldx, int M, int K, int ncap,
                                                           uint8_t* __restrict__ xh) {
    const int g = blockIdx.x, kt = blockIdx.y;           // row group of 8, k tile
    uint8_t* out = xh + ((size_t)kt * (ncap >> 3) + g) * 2048;
    for (int i = threadIdx.x; i < 8 * 16; i += blockDim.x) {
        const int r = i & 7, c = i >> 3;
        const int m = g * 8 + r, k0 = kt * 128 + c * 8;
        __align__(16) __nv_bfloat16 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = __float2bfloat16_rn((m < M && k0 + j < K) ? x[(size_t)m * ldx + k0 + j] : 0.f);
        *reinterpret_cast<uint4*>(out + c * 128 + r * 16) = *reinterpret_cast<const uint4*>(v);
    }
}

// the same image with a row gather: image row i < n_rows holds source row rows[i] (negative: a row of zeros) -- the rows of
// a routed feed-forward sorted by expert
__global__ void __launch_bounds__(256) xh_gather_rows_kernel(const float* __restrict__ x, long long ldx, int n_rows, int K, int ncap,
                                                             uint8_t* __restrict__ xh, const int* __restrict__ rows) {
    const int g = blockIdx.x, kt = blockIdx.y;
    uint8_t* out = xh + ((size_t)kt * (ncap >> 3) + g) * 2048;
    for (int i = threadIdx.x; i < 8 * 16; i += blockDim.x) {
        const int r = i & 7, c = i >> 3;
        const int k0 = kt * 128 + c * 8;
        const int at = g * 8 + r;
        const int m = at < n_rows ? rows[at] : -1;
        __align__(16) __nv_bfloat16 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = __float2bfloat16_rn((m >= 0 && k0 + j < K) ? x[(size_t)m * ldx + k0 + j] : 0.f);
        *reinterpret_cast<uint4*>(out + c * 128 + r * 16) = *reinterpret_cast<const uint4*>(v);
    }
}

extern "C" int dl_wh_from_dense(const void* w, int N, int K, long long ldw, uint8_t* wh, void* stream) {
    if (N < 1 || K < 1) { dl_set_error("dl_wh_from_dense: empty matrix"); return -1; }
    const int KT = (K + 127) / 128, RT = (N + 127) / 128;
    wh_from_dense_kernel<<<RT * KT, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)w, N, K, ldw, wh, KT);
    LAYER_CHECK_LAUNCH("dl_wh_from_dense");
    return 0;
}

extern "C" int dl_xh_from_rows(const float* x, long long ldx, int M, int K, int ncap, uint8_t* xh, void* stream) {
    if (M < 1 || K < 1 || ncap % 8 != 0 || ncap < M) { dl_set_error("dl_xh_from_rows: bad M=%d / ncap=%d", M, ncap); return -1; }
    dim3 grid((M + 7) / 8, (K + 127) / 128);
    xh_from_rows_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(x, ldx, M, K, ncap, xh);
    LAYER_CHECK_LAUNCH("dl_xh_from_rows");
    return 0;
}

// image row i < n_rows holds source row rows[i] of x (device map; negative: zeros)
extern "C" int dl_xh_gather_rows(const float* x, long long ldx, const int* rows, int n_rows, int K, int ncap, uint8_t* xh, void* stream) {
    if (n_rows < 1 || K < 1 || ncap % 8 != 0 || ncap < n_rows || rows == nullptr) { dl_set_error("dl_xh_gather_rows: bad n_rows=%d / ncap=%d", n_rows, ncap); return -1; }
    dim3 grid((n_rows + 7) / 8, (K + 127) / 128);
    xh_gather_rows_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(x, ldx, n_rows, K, ncap, xh, rows);
    LAYER_CHECK_LAUNCH("dl_xh_gather_rows");
    return 0;
}
