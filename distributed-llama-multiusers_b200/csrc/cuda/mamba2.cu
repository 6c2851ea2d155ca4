// Mamba-2 mixer (a selective state-space recurrence with a scalar decay per head):
//     xBC_t  = silu(conv_taps(xBC)_t + bias)                 short causal convolution per channel
//     dt_t   = softplus(dt_t + dt_bias_h)
//     S_t    = exp(-exp(A_log_h) dt_t) S_(t-1) + dt_t B_t x_t^T          S: [state][vdim] per head, f32
//     y_t    = S_t^T C_t + D_h x_t
// Per sequence slot the recurrent state S and the last taps-1 convolution inputs live in f32 device pools; a batch
// is any mix of sequences, each with one or more consecutive rows (a prompt portion, or one decoded token), described
// by a row list per sequence.  A sequence whose first row of the batch is position 0 starts from zeros, whatever its
// slot held before.
//
// Kernels: the convolution over batch rows + carried inputs, the update of the carried inputs, and the scan
// (one CTA per sequence and head, the state in shared memory, tokens in order).
#include "layer_common.cuh"
#include "../../../include/dllama_b200.h"

#define MB_MAX_TAPS 16

// input of channel ch at position q of sequence n, where the batch holds positions p0 .. p0+len-1 of the sequence
__device__ __forceinline__ float conv_input(const DlMambaBatch& b, const float* __restrict__ in, long long ld, int in_off,
                                            const float* __restrict__ conv_state, int channels, int taps,
                                            int n, int q, int ch) {
    if (q < 0) return 0.f;
    const int p0 = b.seq_pos0[n];
    if (q >= p0) {
        const int row = b.seq_rows[b.seq_start[n] + (q - p0)];
        return in[(size_t)row * ld + in_off + ch];
    }
    const int k = q - p0 + (taps - 1);                // carried inputs hold positions p0-(taps-1) .. p0-1
    return conv_state[((size_t)b.seq_slot[n] * (taps - 1) + k) * channels + ch];
}

// out[row][ch] = act(bias[ch] + sum_k w[ch][k] * input(pos - (taps-1) + k)) (+ input(pos) if residual).  Where each tap's
// inputs lie (a row of the batch, a carried row of the slot, or nothing before the sequence's start) is the same for all
// channels of a row: found once per CTA, then every channel reads through the taps' pointers.
template <typename WT>
__global__ void __launch_bounds__(256) mamba_conv_kernel(DlMambaBatch b, const float* __restrict__ in, long long ld, int in_off,
                                                         const WT* __restrict__ w, const WT* __restrict__ bias,
                                                         const float* __restrict__ conv_state, float* __restrict__ out, long long ld_out,
                                                         int channels, int taps, int act, int residual) {
    __shared__ const float* src[MB_MAX_TAPS];
    const int m = blockIdx.x;
    if (threadIdx.x < taps) {
        const int n = b.row_seq[m], q = b.pos[m] - (taps - 1) + threadIdx.x, p0 = b.seq_pos0[n];
        const float* p = nullptr;
        if (q >= p0) p = in + (size_t)b.seq_rows[b.seq_start[n] + (q - p0)] * ld + in_off;
        else if (q >= 0) p = conv_state + ((size_t)b.seq_slot[n] * (taps - 1) + (q - p0 + (taps - 1))) * channels;
        src[threadIdx.x] = p;
    }
    __syncthreads();
    for (int ch = blockIdx.y * blockDim.x + threadIdx.x; ch < channels; ch += gridDim.y * blockDim.x) {
        float acc = bias ? ld_f(bias + ch) : 0.f;
        for (int k = 0; k < taps; ++k)
            if (src[k]) acc = fmaf(ld_f(w + (size_t)ch * taps + k), src[k][ch], acc);
        if (act) acc = silu_f(acc);
        if (residual) acc += in[(size_t)m * ld + in_off + ch];
        out[(size_t)m * ld_out + ch] = acc;
    }
}

// carried inputs after the batch: positions last-(taps-2) .. last of each sequence (runs after the convolution)
__global__ void __launch_bounds__(256) mamba_conv_carry_kernel(DlMambaBatch b, const float* __restrict__ in, long long ld, int in_off,
                                                               float* __restrict__ conv_state, int channels, int taps) {
    const int n = blockIdx.x;
    const int last = b.seq_pos0[n] + (b.seq_start[n + 1] - b.seq_start[n]) - 1;
    for (int ch = blockIdx.y * blockDim.x + threadIdx.x; ch < channels; ch += gridDim.y * blockDim.x) {
        float v[MB_MAX_TAPS];
#pragma unroll
        for (int k = 0; k < MB_MAX_TAPS - 1; ++k)
            if (k < taps - 1) v[k] = conv_input(b, in, ld, in_off, conv_state, channels, taps, n, last - (taps - 2) + k, ch);
#pragma unroll
        for (int k = 0; k < MB_MAX_TAPS - 1; ++k)
            if (k < taps - 1) conv_state[((size_t)b.seq_slot[n] * (taps - 1) + k) * channels + ch] = v[k];
    }
}

extern "C" int dl_causal_conv(const DlMambaBatch* batch, int M, int n_seq, const DlConvArgs* args, void* stream) {
    const DlConvArgs& a = *args;
    if (a.taps < 1 || a.taps > MB_MAX_TAPS) { dl_set_error("dl_causal_conv: 1..%d taps", MB_MAX_TAPS); return -1; }
    if (a.out == a.in) { dl_set_error("dl_causal_conv: out must not alias in"); return -1; }
    cudaStream_t st = (cudaStream_t)stream;
    const int gy = (a.channels + 255) / 256;
    if (a.wtype == DL_T_BF16)
        mamba_conv_kernel<<<dim3(M, gy), 256, 0, st>>>(*batch, a.in, a.ld, a.in_off, (const __nv_bfloat16*)a.w, (const __nv_bfloat16*)a.bias, a.conv_state,
                                                       a.out, a.ld_out, a.channels, a.taps, a.act, a.residual);
    else
        mamba_conv_kernel<<<dim3(M, gy), 256, 0, st>>>(*batch, a.in, a.ld, a.in_off, (const float*)a.w, (const float*)a.bias, a.conv_state,
                                                       a.out, a.ld_out, a.channels, a.taps, a.act, a.residual);
    LAYER_CHECK_LAUNCH("dl_causal_conv");
    if (a.taps > 1) {
        mamba_conv_carry_kernel<<<dim3(n_seq, gy), 256, 0, st>>>(*batch, a.in, a.ld, a.in_off, a.conv_state, a.channels, a.taps);
        LAYER_CHECK_LAUNCH("dl_causal_conv carry");
    }
    return 0;
}

extern "C" int dl_mamba_conv(const DlMambaBatch* batch, int M, int n_seq, const float* in, long long ld, int in_off,
                             const void* w, const void* bias, int wtype, float* conv_state, float* out, int channels,
                             int taps, void* stream) {
    DlConvArgs a;
    a.in = in; a.ld = ld; a.in_off = in_off; a.w = w; a.bias = bias; a.wtype = wtype; a.conv_state = conv_state;
    a.out = out; a.ld_out = channels; a.channels = channels; a.taps = taps; a.act = 1; a.residual = 0;
    return dl_causal_conv(batch, M, n_seq, &a, stream);
}

// ------------------------------------------------------------------------------------------------
// the scan: CTA = (sequence, head); thread p owns column p of S (state x vdim) in shared memory
// ------------------------------------------------------------------------------------------------
__global__ void mamba_scan_kernel(DlMambaBatch b, DlMambaScanArgs a) {
    extern __shared__ float sm[];
    const int n = blockIdx.x, h = blockIdx.y;
    const int N = a.state, P = a.vdim, H = a.n_heads;
    const int g = h / (H / a.groups);
    float* S = sm;                       // [N][P]
    float* Bs = S + (size_t)N * P;       // [N]
    float* Cs = Bs + N;                  // [N]
    const int p = threadIdx.x;
    const int slot = b.seq_slot[n];
    float* Sg = a.ssm_state + ((size_t)slot * H + h) * N * P;
    const bool fresh = b.seq_pos0[n] == 0;
    if (p < P)
        for (int i = 0; i < N; ++i) S[i * P + p] = fresh ? 0.f : Sg[i * P + p];
    const float A = -expf(a.A_log[h]), Dh = a.D[h], dtb = a.dt_bias[h];
    const int r0 = b.seq_start[n], r1 = b.seq_start[n + 1];
    const int inner = H * P;
    for (int r = r0; r < r1; ++r) {
        const int row = b.seq_rows[r];
        const float* xbc = a.xbc + (size_t)row * a.ld_xbc;
        __syncthreads();
        for (int i = threadIdx.x; i < N; i += blockDim.x) {
            Bs[i] = xbc[inner + g * N + i];
            Cs[i] = xbc[inner + a.groups * N + g * N + i];
        }
        __syncthreads();
        if (p < P) {
            const float dt = softplus_f(a.dt[(size_t)row * a.ld_dt + h] + dtb);
            const float decay = expf(A * dt);
            const float x = xbc[h * P + p];
            const float dx = dt * x;
            float y = 0.f;
            for (int i = 0; i < N; ++i) {
                const float s = fmaf(decay, S[i * P + p], Bs[i] * dx);
                S[i * P + p] = s;
                y = fmaf(s, Cs[i], y);
            }
            a.y[(size_t)row * a.ld_y + h * P + p] = fmaf(Dh, x, y);
        }
    }
    if (p < P)
        for (int i = 0; i < N; ++i) Sg[i * P + p] = S[i * P + p];
}

// ------------------------------------------------------------------------------------------------
// the same scan with the state in registers, for state sizes 16 / 32 / 64 / 128: thread (p, nq) owns rows
// nq, nq + 4, nq + 8, ... of column p; MS_TB tokens' inputs (B, C, x, step size, decay) are staged per barrier pair,
// so the token loop touches shared memory and registers only.  y is the sum over the 4 lanes of a column.
// ------------------------------------------------------------------------------------------------
#define MS_TB 16
#define MS_NQ 4

template <int NR>
__global__ void mamba_scan_reg_kernel(DlMambaBatch b, DlMambaScanArgs a) {
    extern __shared__ float sm[];
    const int n = blockIdx.x, h = blockIdx.y;
    const int N = NR * MS_NQ, P = a.vdim, H = a.n_heads;
    const int g = h / (H / a.groups);
    float2* bc = reinterpret_cast<float2*>(sm);          // [MS_TB][N]  (B, C)
    float* xs = sm + 2 * MS_TB * N;                       // [MS_TB][P]
    float* ys = xs + MS_TB * P;                           // [MS_TB][P]
    float* dts = ys + MS_TB * P;                          // [MS_TB]
    float* dec = dts + MS_TB;                             // [MS_TB]
    const int tid = threadIdx.x, nq = tid % MS_NQ;
    const bool act = tid / MS_NQ < P;
    const int p = act ? tid / MS_NQ : P - 1;              // idle lanes shadow the last column (they take part in the shuffles)
    float* Sg = a.ssm_state + ((size_t)b.seq_slot[n] * H + h) * N * P;
    const bool fresh = b.seq_pos0[n] == 0;
    float s[NR];
#pragma unroll
    for (int i = 0; i < NR; ++i) s[i] = fresh ? 0.f : Sg[(size_t)(i * MS_NQ + nq) * P + p];
    const float A = -expf(a.A_log[h]), Dh = a.D[h], dtb = a.dt_bias[h];
    const int r0 = b.seq_start[n], r1 = b.seq_start[n + 1];
    const int inner = H * P, GN = a.groups * N;
    for (int r = r0; r < r1; r += MS_TB) {
        const int nt = min(MS_TB, r1 - r);
        __syncthreads();                                  // the previous block's outputs are stored, its inputs consumed
        for (int idx = tid; idx < nt * N; idx += blockDim.x) {
            const int tt = idx / N, i = idx % N;
            const float* xbc = a.xbc + (size_t)b.seq_rows[r + tt] * a.ld_xbc + inner + g * N + i;
            bc[idx] = make_float2(xbc[0], xbc[GN]);
        }
        for (int idx = tid; idx < nt * P; idx += blockDim.x) {
            const int tt = idx / P, pp = idx % P;
            xs[idx] = a.xbc[(size_t)b.seq_rows[r + tt] * a.ld_xbc + h * P + pp];
        }
        if (tid < nt) {
            const float dt = softplus_f(a.dt[(size_t)b.seq_rows[r + tid] * a.ld_dt + h] + dtb);
            dts[tid] = dt;
            dec[tid] = expf(A * dt);
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float x = xs[tt * P + p], dx = dts[tt] * x, d = dec[tt];
            const float2* row = bc + tt * N + nq;
            float y = 0.f;
#pragma unroll
            for (int i = 0; i < NR; ++i) {
                const float2 v = row[i * MS_NQ];
                s[i] = fmaf(d, s[i], v.x * dx);
                y = fmaf(s[i], v.y, y);
            }
            y += __shfl_xor_sync(0xffffffffu, y, 1);
            y += __shfl_xor_sync(0xffffffffu, y, 2);
            if (act && nq == 0) ys[tt * P + p] = fmaf(Dh, x, y);
        }
        __syncthreads();
        for (int idx = tid; idx < nt * P; idx += blockDim.x) {
            const int tt = idx / P, pp = idx % P;
            a.y[(size_t)b.seq_rows[r + tt] * a.ld_y + h * P + pp] = ys[idx];
        }
    }
    if (act) {
#pragma unroll
        for (int i = 0; i < NR; ++i) Sg[(size_t)(i * MS_NQ + nq) * P + p] = s[i];
    }
}

// ------------------------------------------------------------------------------------------------
// Long prompt portions: the recurrence is linear in the state, so a sequence's rows are cut into chunks that run in
// parallel.  Pass 1 (mamba_chunk_local_kernel): every chunk runs the recurrence from zeros (the sequence's first chunk:
// from the slot's state), writes its outputs, its final state, its total decay, and per row the decay accumulated since
// the chunk's start.  Pass 2 (mamba_chunk_fix_kernel): chunk j rebuilds the state it should have started from out of
// the final states and decays of chunks 0 .. j-1, adds that state's contribution  cum_t * (S_init^T C_t)  to its rows'
// outputs, and the sequence's last chunk leaves the final state in the slot.
// ------------------------------------------------------------------------------------------------
template <int NR>
__global__ void mamba_chunk_local_kernel(DlMambaBatch b, DlMambaScanArgs a, DlMambaChunks ck) {
    extern __shared__ float sm[];
    const int c = blockIdx.x, h = blockIdx.y;
    const int n = ck.chunk_seq[c], off = ck.chunk_off[c];
    const int N = NR * MS_NQ, P = a.vdim, H = a.n_heads;
    const int g = h / (H / a.groups);
    float2* bc = reinterpret_cast<float2*>(sm);
    float* xs = sm + 2 * MS_TB * N;
    float* ys = xs + MS_TB * P;
    float* dts = ys + MS_TB * P;
    float* dec = dts + MS_TB;
    float* cums = dec + MS_TB;                            // [MS_TB + 1]: decay since the chunk's start; [MS_TB] carries over
    const int tid = threadIdx.x, nq = tid % MS_NQ;
    const bool act = tid / MS_NQ < P;
    const int p = act ? tid / MS_NQ : P - 1;
    const float* Sg = a.ssm_state + ((size_t)b.seq_slot[n] * H + h) * N * P;
    const bool from_slot = off == 0 && b.seq_pos0[n] != 0;
    float s[NR];
#pragma unroll
    for (int i = 0; i < NR; ++i) s[i] = from_slot ? Sg[(size_t)(i * MS_NQ + nq) * P + p] : 0.f;
    const float A = -expf(a.A_log[h]), Dh = a.D[h], dtb = a.dt_bias[h];
    const int r0 = b.seq_start[n] + off, r1 = min(b.seq_start[n + 1], r0 + ck.chunk);
    const int inner = H * P, GN = a.groups * N;
    if (tid == 0) cums[MS_TB] = 1.f;
    for (int r = r0; r < r1; r += MS_TB) {
        const int nt = min(MS_TB, r1 - r);
        __syncthreads();
        for (int idx = tid; idx < nt * N; idx += blockDim.x) {
            const int tt = idx / N, i = idx % N;
            const float* xbc = a.xbc + (size_t)b.seq_rows[r + tt] * a.ld_xbc + inner + g * N + i;
            bc[idx] = make_float2(xbc[0], xbc[GN]);
        }
        for (int idx = tid; idx < nt * P; idx += blockDim.x) {
            const int tt = idx / P, pp = idx % P;
            xs[idx] = a.xbc[(size_t)b.seq_rows[r + tt] * a.ld_xbc + h * P + pp];
        }
        if (tid < nt) {
            const float dt = softplus_f(a.dt[(size_t)b.seq_rows[r + tid] * a.ld_dt + h] + dtb);
            dts[tid] = dt;
            dec[tid] = expf(A * dt);
        }
        __syncthreads();
        if (tid == 0) {
            float cv = cums[MS_TB];
            for (int tt = 0; tt < nt; ++tt) {
                cv *= dec[tt];
                cums[tt] = cv;
                ck.cum[(size_t)b.seq_rows[r + tt] * H + h] = cv;
            }
            cums[MS_TB] = cv;
        }
        for (int tt = 0; tt < nt; ++tt) {
            const float x = xs[tt * P + p], dx = dts[tt] * x, d = dec[tt];
            const float2* row = bc + tt * N + nq;
            float y = 0.f;
#pragma unroll
            for (int i = 0; i < NR; ++i) {
                const float2 v = row[i * MS_NQ];
                s[i] = fmaf(d, s[i], v.x * dx);
                y = fmaf(s[i], v.y, y);
            }
            y += __shfl_xor_sync(0xffffffffu, y, 1);
            y += __shfl_xor_sync(0xffffffffu, y, 2);
            if (act && nq == 0) ys[tt * P + p] = fmaf(Dh, x, y);
        }
        __syncthreads();
        for (int idx = tid; idx < nt * P; idx += blockDim.x) {
            const int tt = idx / P, pp = idx % P;
            a.y[(size_t)b.seq_rows[r + tt] * a.ld_y + h * P + pp] = ys[idx];
        }
    }
    __syncthreads();
    float* So = ck.state + ((size_t)c * H + h) * N * P;
    if (act) {
#pragma unroll
        for (int i = 0; i < NR; ++i) So[(size_t)(i * MS_NQ + nq) * P + p] = s[i];
    }
    if (tid == 0) ck.decay[(size_t)c * H + h] = cums[MS_TB];
}

template <int NR>
__global__ void mamba_chunk_fix_kernel(DlMambaBatch b, DlMambaScanArgs a, DlMambaChunks ck) {
    extern __shared__ float sm[];
    const int c = blockIdx.x, h = blockIdx.y;
    const int n = ck.chunk_seq[c], off = ck.chunk_off[c];
    const int N = NR * MS_NQ, P = a.vdim, H = a.n_heads;
    const int g = h / (H / a.groups);
    const int j = off / ck.chunk, c0 = c - j;             // a sequence's chunks are adjacent in the list
    const int r0 = b.seq_start[n] + off, r1 = min(b.seq_start[n + 1], r0 + ck.chunk);
    const bool last = r1 == b.seq_start[n + 1];
    if (j == 0 && !last) return;
    float* cs = sm;                                       // [MS_TB][N]  C
    float* ys = cs + MS_TB * N;                           // [MS_TB][P]
    float* cums = ys + MS_TB * P;                         // [MS_TB]
    const int tid = threadIdx.x, nq = tid % MS_NQ;
    const bool act = tid / MS_NQ < P;
    const int p = act ? tid / MS_NQ : P - 1;
    float s[NR];
#pragma unroll
    for (int i = 0; i < NR; ++i) s[i] = 0.f;
    for (int jj = 0; jj < j; ++jj) {
        const float d = ck.decay[(size_t)(c0 + jj) * H + h];
        const float* Sj = ck.state + ((size_t)(c0 + jj) * H + h) * N * P;
#pragma unroll
        for (int i = 0; i < NR; ++i) s[i] = fmaf(d, s[i], Sj[(size_t)(i * MS_NQ + nq) * P + p]);
    }
    if (j > 0) {
        const int inner = H * P, GN = a.groups * N;
        for (int r = r0; r < r1; r += MS_TB) {
            const int nt = min(MS_TB, r1 - r);
            __syncthreads();
            for (int idx = tid; idx < nt * N; idx += blockDim.x) {
                const int tt = idx / N, i = idx % N;
                cs[idx] = a.xbc[(size_t)b.seq_rows[r + tt] * a.ld_xbc + inner + GN + g * N + i];
            }
            if (tid < nt) cums[tid] = ck.cum[(size_t)b.seq_rows[r + tid] * H + h];
            __syncthreads();
            for (int tt = 0; tt < nt; ++tt) {
                const float* row = cs + tt * N + nq;
                float y = 0.f;
#pragma unroll
                for (int i = 0; i < NR; ++i) y = fmaf(s[i], row[i * MS_NQ], y);
                y += __shfl_xor_sync(0xffffffffu, y, 1);
                y += __shfl_xor_sync(0xffffffffu, y, 2);
                if (act && nq == 0) ys[tt * P + p] = cums[tt] * y;
            }
            __syncthreads();
            for (int idx = tid; idx < nt * P; idx += blockDim.x) {
                const int tt = idx / P, pp = idx % P;
                a.y[(size_t)b.seq_rows[r + tt] * a.ld_y + h * P + pp] += ys[idx];
            }
        }
    }
    if (last && act) {
        const float d = ck.decay[(size_t)c * H + h];
        const float* Sc = ck.state + ((size_t)c * H + h) * N * P;
        float* Sg = a.ssm_state + ((size_t)b.seq_slot[n] * H + h) * N * P;
#pragma unroll
        for (int i = 0; i < NR; ++i) Sg[(size_t)(i * MS_NQ + nq) * P + p] = fmaf(d, s[i], Sc[(size_t)(i * MS_NQ + nq) * P + p]);
    }
}

template <int NR>
static void launch_scan_chunked(const DlMambaBatch& b, const DlMambaScanArgs& a, const DlMambaChunks& ck, cudaStream_t st) {
    const int N = NR * MS_NQ;
    const size_t smem = ((size_t)2 * MS_TB * N + 2 * (size_t)MS_TB * a.vdim + 3 * MS_TB + 1) * sizeof(float);
    const int threads = (a.vdim * MS_NQ + 31) / 32 * 32;
    mamba_chunk_local_kernel<NR><<<dim3(ck.n_chunks, a.n_heads), threads, smem, st>>>(b, a, ck);
    mamba_chunk_fix_kernel<NR><<<dim3(ck.n_chunks, a.n_heads), threads, smem, st>>>(b, a, ck);
}

extern "C" int dl_mamba_scan_chunked_supported(int vdim, int state) {
    return (vdim * MS_NQ <= 1024 && vdim <= 128 && (state == 16 || state == 32 || state == 64 || state == 128)) ? 0 : -1;
}

// scratch: ck.state [n_chunks][heads][state][vdim], ck.decay [n_chunks][heads], ck.cum [rows][heads] (all f32)
extern "C" int dl_mamba_scan_chunked(const DlMambaBatch* batch, const DlMambaScanArgs* args, const DlMambaChunks* chunks, void* stream) {
    const DlMambaScanArgs& a = *args;
    if (a.n_heads % a.groups != 0) { dl_set_error("dl_mamba_scan_chunked: heads must be a multiple of groups"); return -1; }
    if (dl_mamba_scan_chunked_supported(a.vdim, a.state) != 0) { dl_set_error("dl_mamba_scan_chunked: vdim %d / state %d not supported", a.vdim, a.state); return -1; }
    if (chunks->n_chunks < 1 || chunks->chunk < MS_TB) { dl_set_error("dl_mamba_scan_chunked: bad chunking"); return -1; }
    cudaStream_t st = (cudaStream_t)stream;
    switch (a.state) {
        case 16: launch_scan_chunked<4>(*batch, a, *chunks, st); break;
        case 32: launch_scan_chunked<8>(*batch, a, *chunks, st); break;
        case 64: launch_scan_chunked<16>(*batch, a, *chunks, st); break;
        default: launch_scan_chunked<32>(*batch, a, *chunks, st); break;
    }
    LAYER_CHECK_LAUNCH("dl_mamba_scan_chunked");
    return 0;
}

template <int NR>
static void launch_scan_reg(const DlMambaBatch& b, const DlMambaScanArgs& a, int n_seq, cudaStream_t st) {
    const int N = NR * MS_NQ;
    const size_t smem = ((size_t)2 * MS_TB * N + 2 * (size_t)MS_TB * a.vdim + 2 * MS_TB) * sizeof(float);
    const int threads = (a.vdim * MS_NQ + 31) / 32 * 32;
    mamba_scan_reg_kernel<NR><<<dim3(n_seq, a.n_heads), threads, smem, st>>>(b, a);
}

extern "C" int dl_mamba_scan(const DlMambaBatch* batch, int n_seq, const DlMambaScanArgs* args, void* stream) {
    const DlMambaScanArgs& a = *args;
    if (a.n_heads % a.groups != 0) { dl_set_error("dl_mamba_scan: heads must be a multiple of groups"); return -1; }
    if (a.vdim > 1024) { dl_set_error("dl_mamba_scan: vdim > 1024"); return -1; }
    if (a.vdim * MS_NQ <= 1024 && a.vdim <= 128 && (a.state == 16 || a.state == 32 || a.state == 64 || a.state == 128)) {
        cudaStream_t st = (cudaStream_t)stream;
        switch (a.state) {
            case 16: launch_scan_reg<4>(*batch, a, n_seq, st); break;
            case 32: launch_scan_reg<8>(*batch, a, n_seq, st); break;
            case 64: launch_scan_reg<16>(*batch, a, n_seq, st); break;
            default: launch_scan_reg<32>(*batch, a, n_seq, st); break;
        }
        LAYER_CHECK_LAUNCH("dl_mamba_scan");
        return 0;
    }
    const size_t smem = ((size_t)a.state * a.vdim + 2 * (size_t)a.state) * sizeof(float);
    if (smem > 227 * 1024) { dl_set_error("dl_mamba_scan: state %d x vdim %d does not fit shared memory", a.state, a.vdim); return -1; }
    cudaError_t e = cudaFuncSetAttribute(mamba_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { dl_set_error("dl_mamba_scan: shared memory attribute: %s", cudaGetErrorString(e)); return -(int)e; }
    const int threads = (a.vdim + 31) / 32 * 32;
    mamba_scan_kernel<<<dim3(n_seq, a.n_heads), threads, smem, (cudaStream_t)stream>>>(*batch, a);
    LAYER_CHECK_LAUNCH("dl_mamba_scan");
    return 0;
}
