// RMS normalisation in its variants, all in f32:  y = v / sqrt(mean(v^2) + eps) * scale
//   * scale = w  or  (1 + w)  (a weight stored around zero)  or 1 (no weight);
//   * the row may be normalised in `groups` equal parts, each by its own root mean square;
//   * v = x  or  x * silu(gate)  (a gate applied before the norm);
//   * the result is stored, or added to what y holds (a norm on a sublayer's output, summed into the residual stream);
//   * an optional row map gathers source rows (the final norm of the rows whose logits are wanted).
// One CTA per (row, group); groups of up to 4096 values stay in registers between the sum of squares and the scaling.
#include "layer_common.cuh"
#include "../../../include/dllama_b200.h"

#define RN_THREADS 256
#define RN_CACHE 16                // values a thread keeps in registers between the two passes (groups of up to 4096)

__global__ void __launch_bounds__(RN_THREADS) rms_norm_kernel(DlNormArgs a) {
    __shared__ float red[32];
    const int m = blockIdx.x, g = blockIdx.y;
    const int src = a.rows ? a.rows[m] : m;
    const int gd = a.dim / a.groups;
    const float* x = a.x + (size_t)src * a.ldx + (size_t)g * gd;
    const float* gate = a.gate ? a.gate + (size_t)src * a.ld_gate + (size_t)g * gd : nullptr;
    const bool cached = gd <= RN_THREADS * RN_CACHE;
    float v[RN_CACHE];
    float ss = 0.f;
    if (cached) {
#pragma unroll
        for (int k = 0; k < RN_CACHE; ++k) {
            const int i = threadIdx.x + k * RN_THREADS;
            float t = 0.f;
            if (i < gd) {
                t = x[i];
                if (gate) t *= silu_f(gate[i]);
            }
            v[k] = t;
            ss = fmaf(t, t, ss);
        }
    } else {
        for (int i = threadIdx.x; i < gd; i += RN_THREADS) {
            float t = x[i];
            if (gate) t *= silu_f(gate[i]);
            ss = fmaf(t, t, ss);
        }
    }
    ss = block_sum(ss, red);
    const float inv = 1.f / sqrtf(ss / (float)gd + a.eps);
    float* y = a.y + (size_t)m * a.ldy + (size_t)g * gd;
    const float* w = a.w ? a.w + (size_t)g * gd : nullptr;
    if (cached) {
#pragma unroll
        for (int k = 0; k < RN_CACHE; ++k) {
            const int i = threadIdx.x + k * RN_THREADS;
            if (i < gd) {
                float t = v[k] * inv;
                if (w) t *= a.plus_one ? 1.f + w[i] : w[i];
                y[i] = a.accumulate ? y[i] + t : t;
            }
        }
    } else {
        for (int i = threadIdx.x; i < gd; i += RN_THREADS) {
            float t = x[i];
            if (gate) t *= silu_f(gate[i]);
            t *= inv;
            if (w) t *= a.plus_one ? 1.f + w[i] : w[i];
            y[i] = a.accumulate ? y[i] + t : t;
        }
    }
}

extern "C" int dl_rms_norm(const DlNormArgs* args, void* stream) {
    const DlNormArgs& a = *args;
    if (a.M < 1 || a.dim < 1 || a.groups < 1 || a.dim % a.groups != 0) { dl_set_error("dl_rms_norm: bad shape"); return -1; }
    if (a.accumulate && (const float*)a.y == a.x) { dl_set_error("dl_rms_norm: accumulate needs y != x"); return -1; }
    dim3 grid(a.M, a.groups);
    rms_norm_kernel<<<grid, RN_THREADS, 0, (cudaStream_t)stream>>>(a);
    LAYER_CHECK_LAUNCH("dl_rms_norm");
    return 0;
}

// ------------------------------------------------------------------------------------------------
// PolyNorm: y = c0 N(z) + c1 N(z^2) + c2 N(z^3) + c3, N(u) = u / sqrt(mean(u^2) + eps), powers element by element.
// One CTA per row: the sums of z^2, z^4 and z^6 in one pass (the row stays in registers up to 4096 values), then the
// three scalings.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(RN_THREADS) poly_norm_kernel(const float* __restrict__ x, long long ldx, float* __restrict__ y, long long ldy,
                                                               int dim, const float* __restrict__ coef, float eps) {
    __shared__ float red[32];
    const int m = blockIdx.x;
    const float* xr = x + (size_t)m * ldx;
    const bool cached = dim <= RN_THREADS * RN_CACHE;
    float v[RN_CACHE];
    float s2 = 0.f, s4 = 0.f, s6 = 0.f;
    if (cached) {
#pragma unroll
        for (int k = 0; k < RN_CACHE; ++k) {
            const int i = threadIdx.x + k * RN_THREADS;
            const float t = i < dim ? xr[i] : 0.f;
            v[k] = t;
            const float t2 = t * t, t3 = t2 * t;
            s2 = fmaf(t, t, s2); s4 = fmaf(t2, t2, s4); s6 = fmaf(t3, t3, s6);
        }
    } else {
        for (int i = threadIdx.x; i < dim; i += RN_THREADS) {
            const float t = xr[i], t2 = t * t, t3 = t2 * t;
            s2 = fmaf(t, t, s2); s4 = fmaf(t2, t2, s4); s6 = fmaf(t3, t3, s6);
        }
    }
    s2 = block_sum(s2, red);
    s4 = block_sum(s4, red);
    s6 = block_sum(s6, red);
    const float c1 = coef[0] / sqrtf(s2 / (float)dim + eps), c2 = coef[1] / sqrtf(s4 / (float)dim + eps),
                c3 = coef[2] / sqrtf(s6 / (float)dim + eps), c0 = coef[3];
    float* yr = y + (size_t)m * ldy;
    if (cached) {
#pragma unroll
        for (int k = 0; k < RN_CACHE; ++k) {
            const int i = threadIdx.x + k * RN_THREADS;
            if (i < dim) { const float t = v[k]; yr[i] = fmaf(t, fmaf(t, fmaf(t, c3, c2), c1), c0); }
        }
    } else {
        for (int i = threadIdx.x; i < dim; i += RN_THREADS) { const float t = xr[i]; yr[i] = fmaf(t, fmaf(t, fmaf(t, c3, c2), c1), c0); }
    }
}

extern "C" int dl_poly_norm(const float* x, long long ldx, float* y, long long ldy, int M, int dim, const float* coef, float eps,
                            void* stream) {
    if (M < 1 || dim < 1 || coef == nullptr) { dl_set_error("dl_poly_norm: bad shape"); return -1; }
    poly_norm_kernel<<<M, RN_THREADS, 0, (cudaStream_t)stream>>>(x, ldx, y, ldy, dim, coef, eps);
    LAYER_CHECK_LAUNCH("dl_poly_norm");
    return 0;
}
