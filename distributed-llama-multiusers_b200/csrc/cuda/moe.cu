// Routed experts: every token runs `top` of `experts` small feed-forward layers  W_down act(W_up h),  act = relu(.)^2,
// and sums their outputs weighted by the router's scores.  Gated experts (a third matrix W_gate per expert) use
// hidden = a sigma(1.702 a) (1 + b) with a = min(gate . h, limit), b = clamp(up . h, +-limit) instead (sigma: logistic), or
// (gate_act 1) the plain gated unit hidden = silu(gate . h) (up . h).
//
// Routing (dl_moe_select), from the router logits z[M][experts] (a dense product, f32):  s = sigmoid(z), or s =
// softmax(z) over all experts (`score` 1), z with an optional bias per expert added; the chosen weights may be multiplied
// by a constant (`scale`).  Softmax scores divided by the sum of the chosen ones (`renorm`) are the softmax over the
// chosen logits alone.  The experts
// form `groups` equal groups of neighbours; a group's score is the sum of its `group_top` largest scores and only the
// `keep` best groups stay eligible; the `top` eligible experts with the largest scores are chosen, their weights are
// their scores (divided by the sum of the chosen scores if `renorm`).  Ties go to the lower index.  groups = keep = 1
// is plain top-k routing.
//
// Expert products, two forms:
//   * per (row, chosen expert) pair, weight-streaming (dl_moe_rows: f32 weights at any size, bf16 weights for
//     decode-sized batches): up-projection + relu^2 into act[M * top][ff], then one warp per output column does the
//     `top` down-projections of a row and their weighted sum in the order the experts were chosen;
//   * grouped for the tensor cores (dl_moe_plan / dl_moe_combine around the grouped tcgen05 GEMM of gemm_wh_tc.cu):
//     the (row, expert) pairs are sorted by expert into segments padded to 8 rows, the rows are gathered into the
//     GEMM's activation image, one grouped GEMM per projection runs all experts, and the combine kernel sums each
//     row's `top` results with its weights, in the order chosen -- a row's result does not depend on the batch.
// All expert weights of a layer are stacked: w_up [experts][ff][width], w_down [experts][width][ff].
#include "layer_common.cuh"
#include "../../../include/dllama_b200.h"

// ------------------------------------------------------------------------------------------------
// routing: one warp per row; scores in shared memory, selection by lane 0 (experts and top are small)
// ------------------------------------------------------------------------------------------------
#define MS_WARPS 4

// the best (value, index) over the warp: larger value first, lower index on ties; index -1 = nothing
__device__ __forceinline__ void warp_best(float& v, int& i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (oi >= 0 && (i < 0 || ov > v || (ov == v && oi < i))) { v = ov; i = oi; }
    }
}

// One warp per row.  Scores sit in shared memory (taken ones are set to -1: sigmoid scores are >= 0); every pick is a
// strided scan by the lanes and one warp reduction.
__global__ void __launch_bounds__(MS_WARPS * 32) moe_select_kernel(DlMoeSelectArgs a) {
    extern __shared__ float sm[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m = blockIdx.x * MS_WARPS + warp;
    if (m >= a.M) return;
    const int E = a.experts, G = a.groups, per = E / G;
    float* s = sm + (size_t)warp * (2 * E + G);             // [E] scores, [E] working copy, [G] group scores (< 0: dropped)
    float* w = s + E;
    float* gs = w + E;
    const float* zr = a.z + (size_t)m * a.ldz;
    if (a.score == 1) {                                     // softmax over all experts
        float mx = -INFINITY;
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, zr[e] + (a.bias ? a.bias[e] : 0.f));
        mx = warp_max(mx);
        float sum = 0.f;
        for (int e = lane; e < E; e += 32) { const float p = expf(zr[e] + (a.bias ? a.bias[e] : 0.f) - mx); s[e] = p; sum += p; }
        sum = warp_sum(sum);
        for (int e = lane; e < E; e += 32) w[e] = s[e] = s[e] / sum;
    } else {
        for (int e = lane; e < E; e += 32) w[e] = s[e] = sigmoid_f(zr[e] + (a.bias ? a.bias[e] : 0.f));
    }
    __syncwarp();
    if (G > 1) {
        for (int g = 0; g < G; ++g) {                        // the group's score: its group_top largest, picked off the copy
            float sum = 0.f;
            for (int k = 0; k < a.group_top && k < per; ++k) {
                float bv = -1.f;
                int bi = -1;
                for (int i = lane; i < per; i += 32)
                    if (w[g * per + i] >= 0.f && (bi < 0 || w[g * per + i] > bv)) { bv = w[g * per + i]; bi = i; }
                warp_best(bv, bi);
                sum += bv;
                if (lane == 0) w[g * per + bi] = -1.f;
                __syncwarp();
            }
            if (lane == 0) gs[g] = sum;
        }
        __syncwarp();
        for (int k = 0; k < G - a.keep; ++k) {               // drop the worst group; among equals the one with the higher index
            float bv = 0.f;
            int bi = -1;                                     // ordered by (-score down, G - 1 - g up)
            for (int g = lane; g < G; g += 32) {
                if (gs[g] < 0.f) continue;
                const float v = -gs[g];
                const int idx = G - 1 - g;
                if (bi < 0 || v > bv || (v == bv && idx < bi)) { bv = v; bi = idx; }
            }
            warp_best(bv, bi);
            if (lane == 0) gs[G - 1 - bi] = -1.f;
            __syncwarp();
        }
    } else if (lane == 0) gs[0] = 0.f;
    __syncwarp();
    for (int e = lane; e < E; e += 32) w[e] = gs[e / per] >= 0.f ? s[e] : -1.f;      // eligible experts
    __syncwarp();
    float total = 0.f;
    for (int k = 0; k < a.top; ++k) {
        float bv = -1.f;
        int bi = -1;
        for (int e = lane; e < E; e += 32)
            if (w[e] >= 0.f && (bi < 0 || w[e] > bv)) { bv = w[e]; bi = e; }
        warp_best(bv, bi);
        total += bv;
        if (lane == 0) {
            a.sel[(size_t)m * a.top + k] = bi;
            a.wgt[(size_t)m * a.top + k] = bv;
            w[bi] = -1.f;
        }
        __syncwarp();
    }
    __syncwarp();
    for (int k = lane; k < a.top; k += 32) {
        float v = a.wgt[(size_t)m * a.top + k];
        if (a.renorm) v /= total + 1e-20f;
        if (a.scale != 0.f) v *= a.scale;
        a.wgt[(size_t)m * a.top + k] = v;
    }
}

extern "C" int dl_moe_select(const DlMoeSelectArgs* args, void* stream) {
    const DlMoeSelectArgs& a = *args;
    if (a.M < 1 || a.experts < 1 || a.groups < 1 || a.experts % a.groups || a.keep < 1 || a.keep > a.groups || a.top < 1 ||
        a.top > a.keep * (a.experts / a.groups) || a.group_top < 1 || a.score < 0 || a.score > 1) {
        dl_set_error("dl_moe_select: %d experts in %d groups, keep %d, top %d", a.experts, a.groups, a.keep, a.top);
        return -1;
    }
    const size_t smem = (size_t)MS_WARPS * (2 * a.experts + a.groups) * sizeof(float);
    if (smem > 48 * 1024) { dl_set_error("dl_moe_select: too many experts (%d)", a.experts); return -1; }
    moe_select_kernel<<<(a.M + MS_WARPS - 1) / MS_WARPS, MS_WARPS * 32, smem, (cudaStream_t)stream>>>(a);
    LAYER_CHECK_LAUNCH("dl_moe_select");
    return 0;
}

// ------------------------------------------------------------------------------------------------
// per-pair products: a warp per output column, lanes stride K (16-byte loads where the rows allow)
// ------------------------------------------------------------------------------------------------
template <typename WT> struct MoeVec;
template <> struct MoeVec<float> {
    static __device__ __forceinline__ void load8(const float* p, float* o) {
        const float4 u = *reinterpret_cast<const float4*>(p), v = *reinterpret_cast<const float4*>(p + 4);
        o[0] = u.x; o[1] = u.y; o[2] = u.z; o[3] = u.w; o[4] = v.x; o[5] = v.y; o[6] = v.z; o[7] = v.w;
    }
};
template <> struct MoeVec<__nv_bfloat16> {
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

// sum_k w[k] x[k] over the warp (every lane gets it); vec: K % 8 == 0 and both rows 16-byte aligned
template <typename WT, bool RX>
__device__ __forceinline__ float warp_dot(const WT* __restrict__ w, const float* __restrict__ x, int K, bool vec, int lane) {
    float acc = 0.f;
    if (vec) {
        for (int k = lane * 8; k < K; k += 256) {
            float wv[8], xv[8];
            MoeVec<WT>::load8(w + k, wv);
            MoeVec<float>::load8(x + k, xv);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc = fmaf(RX ? round_bf16(xv[i]) : xv[i], wv[i], acc);
        }
    } else {
        for (int k = lane; k < K; k += 32) acc = fmaf(RX ? round_bf16(x[k]) : x[k], ld_f(w + k), acc);
    }
    return warp_sum(acc);
}

#define MR_WARPS 8

template <typename WT, bool RX>
__global__ void __launch_bounds__(MR_WARPS * 32) moe_up_rows_kernel(DlMoeArgs a, bool vec) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pair = blockIdx.x, f = blockIdx.y * MR_WARPS + warp;
    if (f >= a.ff) return;
    const int m = pair / a.top, e = a.sel[pair];
    const WT* w = (const WT*)a.w_up + ((size_t)e * a.ff + f) * a.width;
    const float v = warp_dot<WT, RX>(w, a.x + (size_t)m * a.ldx, a.width, vec, lane);
    if (a.w_gate != nullptr) {                // gated: a sigma(1.702 a) (1 + b) on the clamped products
        const WT* wg = (const WT*)a.w_gate + ((size_t)e * a.ff + f) * a.width;
        float g = warp_dot<WT, RX>(wg, a.x + (size_t)m * a.ldx, a.width, vec, lane), u = v;
        if (a.gate_act == 1) {                // silu(gate) * up
            if (lane == 0) a.act[(size_t)pair * a.ff + f] = silu_f(g) * u;
            return;
        }
        if (a.limit > 0.f) { g = fminf(g, a.limit); u = fminf(fmaxf(u, -a.limit), a.limit); }
        if (lane == 0) a.act[(size_t)pair * a.ff + f] = g / (1.f + expf(-1.702f * g)) * (u + 1.f);
    } else if (lane == 0) {
        const float r = fmaxf(v, 0.f);
        a.act[(size_t)pair * a.ff + f] = r * r;
    }
}

// One warp per (row, output column): the row's experts are taken four at a time, their weight rows loaded side by side
// (independent accumulators), then reduced and summed with the weights in the order the experts were chosen.
template <typename WT, bool RX>
__global__ void __launch_bounds__(MR_WARPS * 32) moe_down_rows_kernel(DlMoeArgs a, bool vec) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m = blockIdx.x, c = blockIdx.y * MR_WARPS + warp;
    if (c >= a.width) return;
    float out = 0.f;
    for (int k0 = 0; k0 < a.top; k0 += 4) {
        const WT* w[4];
        const float* x[4];
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int pair = m * a.top + min(k0 + j, a.top - 1);
            w[j] = (const WT*)a.w_down + ((size_t)a.sel[pair] * a.width + c) * a.ff;
            x[j] = a.act + (size_t)pair * a.ff;
        }
        if (vec) {
#pragma unroll 4
            for (int k = lane * 8; k < a.ff; k += 256) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float wv[8], xv[8];
                    MoeVec<WT>::load8(w[j] + k, wv);
                    MoeVec<float>::load8(x[j] + k, xv);
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[j] = fmaf(RX ? round_bf16(xv[i]) : xv[i], wv[i], acc[j]);
                }
            }
        } else {
            for (int k = lane; k < a.ff; k += 32)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[j] = fmaf(RX ? round_bf16(x[j][k]) : x[j][k], ld_f(w[j] + k), acc[j]);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float d = warp_sum(acc[j]);
            if (k0 + j < a.top) out = fmaf(a.wgt[m * a.top + k0 + j], d, out);
        }
    }
    if (lane == 0) a.y[(size_t)m * a.ldy + c] = out;
}

template <typename WT, bool RX>
static void launch_moe_rows(const DlMoeArgs& a, cudaStream_t st) {
    const bool al = ((uintptr_t)a.w_up & 15) == 0 && ((uintptr_t)a.w_gate & 15) == 0 && ((uintptr_t)a.w_down & 15) == 0 && ((uintptr_t)a.x & 15) == 0 &&
                    ((uintptr_t)a.act & 15) == 0;
    const bool vec_up = al && a.width % 8 == 0 && a.ldx % 4 == 0, vec_down = al && a.ff % 8 == 0;
    moe_up_rows_kernel<WT, RX><<<dim3(a.M * a.top, (a.ff + MR_WARPS - 1) / MR_WARPS), MR_WARPS * 32, 0, st>>>(a, vec_up);
    moe_down_rows_kernel<WT, RX><<<dim3(a.M, (a.width + MR_WARPS - 1) / MR_WARPS), MR_WARPS * 32, 0, st>>>(a, vec_down);
}

extern "C" int dl_moe_rows(const DlMoeArgs* args, void* stream) {
    const DlMoeArgs& a = *args;
    if (a.M < 1 || a.width < 1 || a.ff < 1 || a.top < 1) { dl_set_error("dl_moe_rows: empty problem"); return -1; }
    cudaStream_t st = (cudaStream_t)stream;
    if (a.wtype == DL_T_BF16) {
        if (a.round_x) launch_moe_rows<__nv_bfloat16, true>(a, st);
        else launch_moe_rows<__nv_bfloat16, false>(a, st);
    } else if (a.wtype == DL_T_F32) {
        if (a.round_x) launch_moe_rows<float, true>(a, st);
        else launch_moe_rows<float, false>(a, st);
    } else {
        dl_set_error("dl_moe_rows: unknown weight type %d", a.wtype);
        return -1;
    }
    LAYER_CHECK_LAUNCH("dl_moe_rows");
    return 0;
}

// ------------------------------------------------------------------------------------------------
// grouped form: sort the (row, expert) pairs by expert -- stable, so nothing depends on timing -- into segments whose
// first rows are multiples of 8 (the row granularity of the GEMM's activation image)
//   cnt[e]              pairs of expert e                                  (moe_count_kernel; cnt zeroed before)
//   grp[e] = {first, n} segment of expert e among the sorted rows
//   slot_row[i]         the batch row whose input sorted row i holds, -1 for padding rows (up to `cap`)
//   pair_pos[m*top+k]   the sorted row of pair (m, k)
// ------------------------------------------------------------------------------------------------
__global__ void moe_count_kernel(const int* __restrict__ sel, int n_pairs, int* __restrict__ cnt) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n_pairs) atomicAdd(cnt + sel[i], 1);
}

#define MP_THREADS 1024

__global__ void __launch_bounds__(MP_THREADS) moe_place_kernel(DlMoePlanArgs a) {
    __shared__ int wc[MP_THREADS / 32];
    const int e = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = MP_THREADS / 32;
    const int n_pairs = a.M * a.top;
    int first = 0;
    for (int i = 0; i < e; ++i) first += (a.cnt[i] + 7) & ~7;
    const int mine = a.cnt[e];
    // every warp takes a contiguous run of pairs (a multiple of 32): count, prefix over the warps, place
    const int seg = ((n_pairs + nw - 1) / nw + 31) & ~31;
    const int lo = warp * seg, hi = min(n_pairs, lo + seg);
    int c = 0;
    for (int b = lo; b < hi; b += 32) {
        const bool hit = b + lane < hi && a.sel[b + lane] == e;
        c += __popc(__ballot_sync(0xffffffffu, hit));
    }
    if (lane == 0) wc[warp] = c;
    __syncthreads();
    int at = first;
    for (int w = 0; w < warp; ++w) at += wc[w];
    for (int b = lo; b < hi; b += 32) {
        const bool hit = b + lane < hi && a.sel[b + lane] == e;
        const unsigned bal = __ballot_sync(0xffffffffu, hit);
        if (hit) {
            const int p = at + __popc(bal & ((1u << lane) - 1u));
            a.slot_row[p] = (b + lane) / a.top;
            a.pair_pos[b + lane] = p;
        }
        at += __popc(bal);
    }
    const int end = first + ((mine + 7) & ~7);
    for (int p = first + mine + threadIdx.x; p < (e == a.experts - 1 ? a.cap : end); p += MP_THREADS) a.slot_row[p] = -1;
    if (threadIdx.x == 0) { a.grp[2 * e] = first; a.grp[2 * e + 1] = mine; }
}

extern "C" int dl_moe_plan(const DlMoePlanArgs* args, void* stream) {
    const DlMoePlanArgs& a = *args;
    if (a.M < 1 || a.top < 1 || a.experts < 1 || a.cap < a.M * a.top + 7 * a.experts) { dl_set_error("dl_moe_plan: bad sizes"); return -1; }
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e = cudaMemsetAsync(a.cnt, 0, sizeof(int) * a.experts, st);
    if (e != cudaSuccess) { dl_set_error("dl_moe_plan: %s", cudaGetErrorString(e)); return -(int)e; }
    const int n_pairs = a.M * a.top;
    moe_count_kernel<<<(n_pairs + 255) / 256, 256, 0, st>>>(a.sel, n_pairs, a.cnt);
    moe_place_kernel<<<a.experts, MP_THREADS, 0, st>>>(a);
    LAYER_CHECK_LAUNCH("dl_moe_plan");
    return 0;
}

// y[m] = sum_k wgt[m][k] * yp[pair_pos[m][k]], in the order the experts were chosen
__global__ void __launch_bounds__(256) moe_combine_kernel(const float* __restrict__ yp, long long ldp, const int* __restrict__ pair_pos,
                                                          const float* __restrict__ wgt, int top, int width, float* __restrict__ y, long long ldy) {
    const int m = blockIdx.x;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < top; ++k) acc = fmaf(wgt[m * top + k], yp[(size_t)pair_pos[m * top + k] * ldp + c], acc);
        y[(size_t)m * ldy + c] = acc;
    }
}

extern "C" int dl_moe_combine(const float* yp, long long ldp, const int* pair_pos, const float* wgt, int M, int top, int width,
                              float* y, long long ldy, void* stream) {
    moe_combine_kernel<<<M, 256, 0, (cudaStream_t)stream>>>(yp, ldp, pair_pos, wgt, top, width, y, ldy);
    LAYER_CHECK_LAUNCH("dl_moe_combine");
    return 0;
}
