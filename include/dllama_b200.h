/* b200-dllama C ABI: every CUDA entry point of libdllama_b200_cuda.so.
 *
 * All pointers are device pointers unless stated otherwise; `stream` is a cudaStream_t.  Functions
 * return 0 on success or a negative/CUDA error code; dl_last_error() gives the message.
 * Citations name the reference component each entry point replaces (paths relative to the
 * reference tree).
 */
#ifndef DLLAMA_B200_H
#define DLLAMA_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DL_MAX_PEERS 8

/* ---- epilogue selector for the Q40 GEMV / GEMM kernels ---------------------------------- */
enum {
    DL_EPI_STORE = 0,     /* f32 store (optionally Q80 round-trip) to 1..8 (peer) buffers + flags  */
    DL_EPI_QKV_ROPE = 1,  /* RoPE on q,k rows; q -> buffer; k,v -> paged KV cache                   */
    DL_EPI_SILU_MUL = 2,  /* rows interleaved (gate,up): act(g)*u -> Q80 activation slabs           */
    DL_EPI_DENSE = 3,     /* f32 store to dst[0] through one of the DL_DENSE_* element-wise ops      */
};
/* element-wise ops on a matmul result (dense-weight models): store, relu(.)^2, aux * sigmoid(.), param * tanh(. / param) */
enum { DL_DENSE_STORE = 0, DL_DENSE_RELU2 = 1, DL_DENSE_SIGMOID_MUL = 2, DL_DENSE_SOFTCAP = 3, DL_DENSE_SILU = 4,
       DL_DENSE_GLU_CLAMP = 5 /* tensor-core epilogue only: output columns (2j, 2j+1) = (gate, up) of value j, see DlMoeArgs */,
       DL_DENSE_MUL = 6          /* aux[m][n] * (.)                                                                  */,
       DL_DENSE_XIELU = 7        /* z > 0: param z^2 + z / 2;  else: param2 (exp(z) - 1 - z) + z / 2                 */,
       DL_DENSE_ROWGATE_ADD = 8  /* y[m][n] + sigmoid(aux[m * ld_aux]) * (.): one gate per row, added to what y holds */,
       DL_DENSE_GLU_SILU = 9     /* tensor-core epilogue only, columns paired like GLU_CLAMP: silu(gate) * up        */ };

typedef struct {
    int kind;
    /* DL_EPI_STORE: dst[p][dst_off + m*ld + row] for p < n_dst  (reference: OP_CAST y->ZQ slice +
     * SYNC_NODE_SLICES, src/llm.cpp:308-314,381-387; logits gather :426-432) */
    float* dst[DL_MAX_PEERS];
    int n_dst;
    int ld;
    long long dst_off;
    int q80_roundtrip;
    const float* residual;            /* NULL, or value += residual[m*residual_ld + row] (TP=1 residual add) */
    int residual_ld;
    uint32_t* flag[DL_MAX_PEERS];     /* flag word to release on each destination (NULL: none) */
    const uint32_t* step_counter;     /* epoch = *step_counter * flag_mul + flag_add           */
    uint32_t flag_mul, flag_add;
    uint32_t* cta_counter;            /* zero-initialised, self-resetting completion counter   */
    /* DL_EPI_QKV_ROPE (reference: OP_ROPE_LLAMA + OP_SHIFT, src/llm.cpp:259-286) */
    float* q_out;                     /* [M][q_dim] */
    int q_dim, kv_dim, head_size;
    const float* rope_freqs;          /* [head_size/2] */
    const int* pos;                   /* [M] */
    const int* slot;                  /* [M] */
    const int* block_table;           /* [n_slots][max_pages] */
    int max_pages, page_size, n_kv_heads;
    void* k_cache;                    /* [n_pages][n_kv_heads][page_size][head_size] */
    void* v_cache;
    int kv_f32;                       /* 1: f32 cache, 0: fp16 cache */
    /* DL_EPI_SILU_MUL (reference: OP_SILU + OP_MUL + OP_CAST d->dq, src/llm.cpp:355-374) */
    uint8_t* xq_out;                  /* XQ slabs of the hidden activation (may be NULL) */
    uint8_t* xh_out;                  /* XH slabs (may be NULL) */
    int out_mcap;                     /* row capacity of the XQ/XH slabs */
    int act_gelu;                     /* 0 = SiLU, 1 = tanh-GELU */
    /* DL_EPI_STORE, tensor-parallel partial sums: 1 = dst[] are arrays of {f32 bits, epoch} 8-byte words (LL
     * protocol: no fence, no flags; step_counter / flag_mul / flag_add give the epoch), 0 = plain f32 */
    int ll;
    /* DL_EPI_DENSE: dst[0][dst_off + m*ld + row] = op(value, dense_aux[m*dense_aux_ld + row], dense_param) */
    int dense_op;
    float dense_param;
    const float* dense_aux;
    long long dense_aux_ld;
    float dense_param2;
} DlEpilogue;

/* Fused activation producer for dl_gemv_q40: the kernel itself computes
 *   x = x_in + sum_src partial[src];  y = rmsnorm(x) * norm_w;  Q80(y)
 * for its own K range straight into shared memory (no global round trip, no separate kernel), after
 * waiting on the peers' release flags.  The CTAs of row tile 0 also write x to x_out.
 * (reference: OP_MERGE_ADD + OP_INV_RMS + OP_RMS_NORM + OP_CAST, src/llm.cpp:204-239,317-342) */
typedef struct {
    const float* x_in;                /* [M][dim] residual stream */
    float* x_out;                     /* [M][dim] or NULL */
    const float* partials;            /* [n_src][..] partial sums, src_stride floats apart; may be NULL */
    int n_src;
    long long src_stride;
    const uint32_t* flags;            /* [n_src] release flags to wait on, or NULL */
    const uint32_t* step_counter;
    uint32_t flag_mul, flag_add;
    const float* norm_w;              /* [dim] */
    float eps;
    int ll;                           /* 1: partials are LL words {f32 bits, epoch}; wait on the words, not on flags */
} DlNormProlog;

const char* dl_last_error(void);
int dl_device_sm_count(void);

/* ---- weight preparation ------------------------------------------------------------------ */
/* bytes of a Q40T image of a [d][n] matrix (d padded to 128) */
long long dl_q40t_bytes(int d, int n);
/* scatter `rows` raw Q40 rows (file layout, n/32 blocks of 18 B each) into a Q40T image at
 * destination rows dst_row0 + i*dst_row_step.  (reference: splitRowMatmulWeight /
 * splitColMatmulWeight + NnCpuDevice weight copy, src/nn/nn-core.cpp:270-303) */
int dl_q40_repack(const uint8_t* raw, int rows, int n, uint8_t* q40t, int d_pad, int dst_row0,
                  int dst_row_step, void* stream);
/* Q40T -> f32 [d][n] (tests, cuBLAS baseline path) */
int dl_q40t_dequant(const uint8_t* q40t, int d, int n, float* out, void* stream);

/* ---- activation producers ---------------------------------------------------------------- */
/* x_out = x_in + sum_src partial[src] ; y = rmsnorm(x_out)*w ; y -> Q80 -> XQ and/or XH slabs.
 * Waits (acquire.sys) on flags[src] >= epoch before reading partials when flags != NULL.
 * (reference: OP_MERGE_ADD + OP_INV_RMS + OP_RMS_NORM + OP_CAST, src/llm.cpp:204-239,317-342) */
int dl_reduce_norm_quant(const float* x_in, float* x_out, const float* partials /*f32, or LL words when ll*/, int n_src, int src_stride,
                         const uint32_t* flags, const uint32_t* step_counter, uint32_t flag_mul,
                         uint32_t flag_add, int ll, const float* norm_w, float eps, int dim, int M, int mcap,
                         uint8_t* xq_out, uint8_t* xh_out, float* y_out, int pdl, void* stream);
/* plain f32 [M][K] -> XQ / XH (no norm); (reference: OP_CAST F32->Q80, nn-cpu-ops.cpp:1221-1235) */
int dl_quant_q80(const float* x, int M, int K, int mcap, uint8_t* xq_out, uint8_t* xh_out, void* stream);
/* embedding gather: x[m][:] = table[token[m]][:]  (reference: OP_EMBEDDING, nn-cpu-ops.cpp:880-892) */
int dl_embedding(const float* table, const int* tokens, float* x, int M, int dim, uint32_t* step_counter,
                 void* stream);

/* per-row sampling on the device (reference: Sampler::sample, src/tokenizer.cpp:382-510): temperature 0 -> first
 * argmax; else softmax(logits / temperature) and top-p nucleus (0 < topp < 1) or multinomial, drawn with coin[m] in
 * [0,1) (the caller's per-request RNG).  All arrays are device pointers with M entries; one CTA per row. */
int dl_sample_rows(const float* logits, int M, int vocab, int ld, const float* temperature, const float* topp,
                   const float* coin, int* tokens_out, void* stream);

/* F32 x F32 -> F32 matmul (f32-weights / f32-buffer path; reference: matmul_F32_F32_F32, nn-cpu-ops.cpp:182-220):
 * y[m][r] (+)= sum_k w[r*ldw + k] * x[m*ldx + k], plain f32 FMAs; n, ldw, ldx multiples of 4, w and x 16-byte aligned */
int dl_gemm_f32(const float* w, int d, int n, long long ldw, const float* x, int M, int ldx, float* y, int ldy,
                int accumulate, void* stream);

/* The other kernels of the f32 path (no Q80 cast anywhere; with dl_gemm_f32, dl_reduce_norm_quant (y_out), dl_attention,
 * dl_embedding and dl_argmax they cover the whole forward pass):
 * RoPE on the q and k rows of qkv[M][q_dim + 2 kv_dim], q -> q_out, k / v -> the paged KV cache
 * (reference: OP_ROPE_LLAMA + OP_SHIFT, nn-cpu-ops.cpp:1090-1120,1253-1275) */
int dl_f32_rope_kv(const float* qkv, int M, int q_dim, int kv_dim, int head_size, int n_kv_heads, const float* freqs,
                   const int* pos, const int* slot, const int* block_table, int max_pages, float* q_out,
                   void* k_cache, void* v_cache, int kv_f32, void* stream);
/* out = act(g) * u, act = SiLU or tanh-GELU (reference: OP_SILU / OP_GELU + OP_MUL, nn-cpu-ops.cpp:1058-1078,1163-1183) */
int dl_f32_silu_mul(const float* g, const float* u, float* out, long long n, int gelu, void* stream);
/* store src[M][w] into every destination buffer (peer memory) at dst_off + m*ld_dst and release one flag per destination
 * with epoch *step_counter*flag_mul+flag_add (reference: SYNC_NODE_SLICES of f32 slices, nn-network.cpp:537-569; the
 * merge-add of nn-cpu-ops.cpp:835-852 is done by the consumer, dl_reduce_norm_quant) */
int dl_f32_push(const float* src, int M, int w, int ld_src, float* const* dst /*host array*/, int n_dst, long long dst_off,
                int ld_dst, uint32_t* const* flags /*host array or NULL*/, const uint32_t* step_counter, uint32_t flag_mul,
                uint32_t flag_add, uint32_t* cta_counter /*zero-initialised, self-resetting*/, void* stream);

/* ---- Q40 x Q80 matmuls ------------------------------------------------------------------- */
/* dp4a GEMV, M <= 8 rows: bulk-copy fed, cluster split-K (reference: matmul_Q80_Q40_F32,
 * src/nn/nn-cpu-ops.cpp:222-440) */
int dl_gemv_q40(const uint8_t* w_q40t, int d, int n, const uint8_t* xq /*XQ slabs with mcap == M; unused when norm != NULL*/,
                int M, int row_split /*1,2,4*/, int k_split /*1..8, cluster size*/, int tiles_per_cta /*>=1, only with k_split==1*/,
                const DlNormProlog* norm /*host, NULL = read xq*/,
                const DlEpilogue* epi /*host*/, int pdl, void* stream);
/* shared-memory bytes the GEMV needs for (n, M, k_split); callers pick k_split so that it fits */
long long dl_gemv_q40_smem_bytes(int n, int M, int k_split);
/* tcgen05 GEMM, M up to 256 per tile: Q40 dequantised to fp16 in the smem pipeline, UMMA with
 * TMEM accumulators (reference: llamafile_sgemm Q40xQ80, src/nn/llamafile/sgemm.cpp:593-783) */
int dl_gemm_q40_tc(const uint8_t* w_q40t, int d, int n, const uint8_t* xh, int ncap, int M, int k_split,
                   const DlEpilogue* epi /*host*/, int pdl, void* stream);
/* prompt-sized batches, two phases: the Q40T image is expanded once into WH (fp16 tiles of 128 x 128 in the UMMA
 * K-major core-matrix image, dl_wh_bytes(d, n) bytes), then a persistent SS-mode tcgen05 GEMM with CTA pairs
 * (cta_group::2, 256 x 256 tiles, double-buffered TMEM accumulators) runs on it; same epilogues as above.
 * force_cg: 0 = CTA pairs when the number of 128-row tiles is even, 1 = single CTAs */
long long dl_wh_bytes(int d, int n);
int dl_q40t_to_wh(const uint8_t* w_q40t, int d, int n, uint8_t* wh, void* stream);
int dl_gemm_wh_tc(const uint8_t* wh, int d, int n, const uint8_t* xh, int ncap, int M, const DlEpilogue* epi /*host*/,
                  int force_cg, int pdl, void* stream);

/* ---- attention ---------------------------------------------------------------------------- */
/* per-row paged GQA attention over positions 0..pos[m] (decode rows and prefill-chunk rows alike);
 * output Q80-quantised into XQ/XH slabs for the wo matmul and/or f32.
 * scratch: >= dl_attention_scratch_bytes(); (reference: OP_MULTIHEAD_ATT, nn-cpu-ops.cpp:749-784,1135-1161) */
long long dl_attention_scratch_bytes(int M, int n_heads, int head_size, int max_splits);
int dl_attention(const float* q, int M, int n_heads, int n_kv_heads, int head_size, const void* k_cache,
                 const void* v_cache, int kv_f32, const int* pos, const int* slot, const int* block_table,
                 int max_pages, int page_size, int n_splits, void* scratch, uint8_t* xq_out, uint8_t* xh_out,
                 int out_mcap, float* y_out, const int* row_skip /*device, NULL or [M]: non-zero rows are left to
                 dl_attention_prefill*/, int pdl, void* stream);

/* causal attention of prompt chunks on the tensor cores (mma.sync fp16, f32 accumulate).  meta (device):
 * meta[0] = n_seg (<= 8), then [begin, end) row ranges; each range is consecutive positions of ONE sequence
 * (slot[begin], first position pos[begin]).  Rows outside the ranges are not touched (dl_attention with row_skip
 * serves them).  fp16 KV cache, head_size 64 or 128.  Same outputs as dl_attention. */
int dl_attention_prefill(const float* q, int M, int n_heads, int n_kv_heads, int head_size, const void* k_cache,
                         const void* v_cache, const int* pos, const int* slot, const int* block_table, int max_pages,
                         int page_size, const int* meta /*device*/, uint8_t* xq_out, uint8_t* xh_out, int out_mcap,
                         float* y_out, int pdl, void* stream);

/* same job on tcgen05 (head_size 128): S = Q K^T and O += P V as UMMA with the score / probability / output tiles in
 * tensor memory, 128 query rows x one head per CTA, 128 tokens per step, lazy softmax rescaling */
int dl_attention_prefill_tc(const float* q, int M, int n_heads, int n_kv_heads, int head_size, const void* k_cache,
                            const void* v_cache, const int* pos, const int* slot, const int* block_table, int max_pages,
                            int page_size, const int* meta /*device*/, uint8_t* xq_out, uint8_t* xh_out, int out_mcap,
                            float* y_out, int n_cache_pages /*pages in k_cache / v_cache: bounds of the TMA tensor maps*/,
                            int pdl, void* stream);

/* ---- sampling helpers --------------------------------------------------------------------- */
/* argmax over logits[m][0..vocab) -> tokens[m]  (reference: Sampler::sample temperature==0,
 * src/tokenizer.cpp:472-502) */
int dl_argmax(const float* logits, int M, int vocab, int ld, int* tokens_out,
              const uint32_t* flags /*NULL: no wait*/, int n_flags, const uint32_t* step_counter,
              uint32_t flag_mul, uint32_t flag_add, int* pos_inc /*NULL or pos[m] += 1*/,
              int* history /*NULL or [cap][M] ring indexed by *step_counter-1*/, int history_cap,
              void* scratch /*zero-initialised, dl_argmax_scratch_bytes(M)*/, int pdl, void* stream);
long long dl_argmax_scratch_bytes(int M);
/* Greedy pick without any device allocation (this entry point has no counterpart in the reference).
 * For callers that are not allowed to call cudaMalloc -- plugins living inside someone else's memory
 * budget, serving loops that ban allocator calls after start-up, hosts that only hand out raw
 * pointers.  Same result as dl_argmax(), but the scratch it needs lives in a fixed 17 KB array inside
 * the library (held by every GPU that loads it, until exit), so the caller passes only logits and the
 * output.  M <= 64 rows, larger M is rejected.  The first call on a device resolves the array's
 * address and should happen before any stream capture; calls on one device share the array, so calls
 * that can overlap on the GPU race -- keep them ordered. */
int dl_argmax_noalloc(const float* logits, int M, int vocab, int ld, int* tokens_out, void* stream);
/* block the stream until flags[i] >= *step_counter*flag_mul+flag_add for i<n (logits gather to the
 * sampling rank; reference: SYNC_NODE_SLICES_EXCEPT_ROOT, src/llm.cpp:432) */
int dl_wait_flags(const uint32_t* flags, int n, const uint32_t* step_counter, uint32_t flag_mul,
                  uint32_t flag_add, void* stream);

/* ---- persistent decode step ----------------------------------------------------------------
 * One cooperative kernel runs a whole forward pass for 1..4 rows (decode): embedding, every layer's
 * norm -> qkv(+RoPE, KV write) -> paged attention -> wo -> norm -> w1|w3 (SiLU*mul) -> w2, final norm,
 * logits, greedy pick.  Phases are separated by device-side grid barriers instead of kernel
 * boundaries and the Q40T weight stream is prefetched across them, so the per-kernel fixed latency
 * of the launch sequence is paid once per token.  Tensor-parallel partial sums travel as Q80 LL
 * words ({4 x int8 | fp16 scale, epoch} in one 8-byte store) written straight into every peer's
 * exchange buffer; the next phase polls the words themselves (no fence, counter or flag).
 * (reference: the whole per-token step list of NnExecutor::forward, src/nn/nn-executor.cpp:134-163,
 * over the graph of src/llm.cpp:126-438; SYNC_NODE_SLICES + OP_MERGE_ADD, src/nn/nn-network.cpp:537-569) */
#define DL_MEGA_MAX_ROWS 4
typedef struct {
    const uint8_t* qkv;               /* Q40T [q_dim + 2 kv_dim][dim]                      */
    const uint8_t* wo;                /* Q40T [dim][q_dim]                                 */
    const uint8_t* w13;               /* Q40T [2 hid][dim], rows interleaved (gate, up)    */
    const uint8_t* w2;                /* Q40T [dim][hid]                                   */
    const float* rms_att;
    const float* rms_ffn;
    void* k_cache;                    /* fp16 [n_pages][n_kv_heads][32][head_size]         */
    void* v_cache;
} DlDecodeLayer;

typedef struct {
    /* model, per-rank slice sizes */
    int n_layers, dim, q_dim, kv_dim, hid, vocab_loc, vocab, head_size, n_heads, n_kv_heads;
    int rank, world;
    float eps;
    int act_gelu;
    int q80_sync;                     /* must be 1: the wo / w2 partial sums travel as Q80 words */
    const DlDecodeLayer* layers;      /* device array [n_layers] */
    const float* rms_final;
    const uint8_t* wcls;              /* Q40T [vocab_loc][dim] */
    const float* embedding;           /* [vocab][dim] f32 */
    const float* rope_freqs;          /* [head_size/2] */
    /* batch */
    int M, row0;                      /* rows; logits / tokens are produced for rows row0..M-1 */
    int* tokens;                      /* [M] */
    int* pos;                         /* [M] */
    const int* slot;                  /* [M] */
    const int* block_table;           /* [n_slots][max_pages] */
    int max_pages;
    /* activations and scratch of this rank (device) */
    float* x[2];                      /* residual stream [4][dim], ping-pong */
    float* q;                         /* [4][q_dim] */
    float* h;                         /* [4][hid] */
    float* att_o;                     /* [4][n_heads][max_splits][head_size] */
    float* att_ml;                    /* [4][n_heads][max_splits][2] */
    int max_splits;                   /* capacity of the split dimension above (<= 32) */
    int att_splits;                   /* split-KV grid: CTAs per (row, kv head) */
    float* cta_best;                  /* [grid][4][2] greedy candidates */
    unsigned* grid_bar;               /* 64 zero-initialised words: [0] arrival counter, [1] exit counter (left at zero by the
                                       * kernel), [16, 32) release flags of the merge-add CTAs (epochs, only grow) */
    uint32_t* step_counter;
    /* tensor-parallel exchange: rank p's buffers as mapped into this process (p < world) */
    uint8_t* ll_att[DL_MAX_PEERS];    /* [world src][4][dim/32][9] 8-byte LL words */
    uint8_t* ll_ffn[DL_MAX_PEERS];
    uint8_t* ll_tok[DL_MAX_PEERS];    /* [world src][4][2] LL words: best logit, its index */
    float* logits[DL_MAX_PEERS];      /* [rows][vocab] on every rank (only logits[rank] when world == 1) */
    uint32_t* flag_logits[DL_MAX_PEERS]; /* word to release on rank p once this rank's logits slice is there */
    /* output */
    int greedy;                       /* 1: pick argmax in the kernel (logits are not written) */
    int* tokens_out;                  /* [M - row0] (greedy) */
    int advance;                      /* 1: tokens[m] = pick, pos[m] += 1 (device-resident loop) */
    int* history;                     /* NULL or [cap][M] ring indexed by step - 1 */
    int history_cap;
    unsigned long long timeout_ns;    /* spin limit before the kernel traps (0 = none) */
    uint32_t* debug;                  /* NULL or a word in mapped pinned host memory: 0x80000000 | wait code << 16 | CTA
                                       * is stored there before a time-out trap (device memory is lost with the context) */
    unsigned long long* trace;        /* NULL or [n_layers * 32 + 32] globaltimer stamps of CTA trace_cta */
    int trace_cta;
    int dbg;                          /* timing probes (results are garbage): 1 = matmul phases skip the arithmetic, 2 = they do not wait for the weights */
    int pf_dist;                      /* pipeline chunks (<= 9 KB) the L2 prefetch of the weight stream runs ahead of the
                                       * shared-memory ring; 0 = no L2 prefetch */
} DlDecodeArgs;

/* 0 if the shapes fit the persistent kernel (shared memory, register-resident row, head size), else -1
 * with the reason in dl_last_error(); callers fall back to the multi-kernel launch sequence. */
int dl_decode_mega_supported(const DlDecodeArgs* args /*host*/, int grid);
int dl_decode_mega(const DlDecodeArgs* args /*host*/, int grid /*CTAs, <= SM count*/, void* stream);
/* work split of one matmul phase for CTA `cta` of `grid`: rows [r0, r1) and the number of pipeline
 * chunks they take (host helper, used by tests) */
int dl_decode_mega_plan(int d, int n, int align, int grid, int cta, int* r0, int* r1, int* n_chunks);

/* ---- peer memory (symmetric buffers over NVLink) ------------------------------------------ */
int dl_ipc_alloc(void** dev_ptr, long long bytes, uint8_t* handle_out /*64 B host*/);
int dl_ipc_open(const uint8_t* handle /*64 B host*/, void** dev_ptr);
int dl_ipc_close(void* dev_ptr);
int dl_ipc_free(void* dev_ptr);
/* all ranks: flag barrier over peer memory (one CTA) */
int dl_peer_barrier(uint32_t* const* flags_on_peers /*host array*/, uint32_t* my_flags, int rank, int world,
                    uint32_t epoch, void* stream);

/* ==== layer-list models: dense bf16 / f32 weights, latent attention, Mamba-2 ===================
 * Built into libdllama_b200_layers.so (dense.cu, norms.cu, latent_attention.cu, mamba2.cu, hyper.cu, window_attention.cu,
 * talk_attention.cu, lightning.cu, moe.cu, plus the shared prep.cu, sampler.cu and gemm_wh_tc.cu).  Activations between kernels are f32; `wtype` / `ctype`: 0 = f32, 1 = bf16. */

/* Y[b][m][n] = epi( sum_k X[b][m][k] * W[b][n][k] ),  b < batch (element strides *_bs).  round_x: the activation
 * operand is rounded to bf16 on load (bf16 mode).  DL_DENSE_SIGMOID_MUL: aux[m][n] * sigmoid(.);
 * DL_DENSE_SOFTCAP: param * tanh(. / param); DL_DENSE_SILU: . * sigmoid(.); DL_DENSE_MUL: aux[m][n] * (.);
 * DL_DENSE_XIELU: param z^2 + z / 2 for z > 0, else param2 (exp(z) - 1 - z) + z / 2;
 * DL_DENSE_ROWGATE_ADD: Y[m][n] + sigmoid(aux[m * ld_aux]) * (.) (Y is read, then written). */
typedef struct {
    const void* W; int wtype; long long ldw, w_bs;
    const float* X; long long ldx, x_bs;
    float* Y; long long ldy, y_bs;
    int M, N, K, batch;
    int round_x;
    int epi;
    const float* aux; long long ld_aux, aux_bs;
    float param;
    float param2;
} DlDenseArgs;
int dl_dense(const DlDenseArgs* args /*host*/, void* stream);
/* x[m][c][dim] = scale * table[tokens[m]] for c < copies */
int dl_embed_rows(const void* table, int wtype, const int* tokens, float* x, int M, int dim, float scale, int copies,
                  void* stream);
/* Tensor-core path of the same product for bf16 weights and many rows: dl_gemm_wh_tc (flags bit 1 = bf16 operands) on
 * the pre-tiled images these two write.  Weights [N][K] row-major bf16 -> tiles of 128 rows x 128 K in the UMMA K-major
 * core-matrix image, [ceil(N/128)][ceil(K/128)][32 KB], zero-padded (dl_wh_bytes(N, round_up(K, 128)) bytes).
 * Activations: columns [0, K) of M f32 rows -> bf16 slabs [ceil(K/128)][ncap/8][2048 B], zero-padded along K. */
int dl_wh_from_dense(const void* w /*bf16*/, int N, int K, long long ldw, uint8_t* wh, void* stream);
int dl_xh_from_rows(const float* x, long long ldx, int M, int K, int ncap, uint8_t* xh, void* stream);

/* y[m] (+)= v / sqrt(mean(v^2) + eps) * scale per group of dim/groups values; v = x[rows ? rows[m] : m] (* silu(gate));
 * scale = w, 1 + w (plus_one) or 1 (w NULL).  In place (y == x) is allowed without `accumulate`. */
typedef struct {
    const float* x; long long ldx;
    const float* gate; long long ld_gate;
    const float* w;
    float* y; long long ldy;
    const int* rows;
    int M, dim, groups;
    float eps;
    int plus_one, accumulate;
} DlNormArgs;
int dl_rms_norm(const DlNormArgs* args /*host*/, void* stream);
/* y[m] = c0 N(z) + c1 N(z^2) + c2 N(z^3) + c3 with z = x[m], powers element-wise, N(u) = u / sqrt(mean(u^2) + eps);
 * coef: 4 f32 on the device.  In place is allowed. */
int dl_poly_norm(const float* x, long long ldx, float* y, long long ldy, int M, int dim, const float* coef, float eps,
                 void* stream);

/* latent-attention cache writer: row m of kv[M][ld] = [rank | rot]; the first `rank` are RMS-normed (* norm_w), the
 * first rope_dims of the last `rot` are rotated by the row's position (freqs: f64 [rope_dims / 2]); the token's
 * cache line is cache[page][pos % page_size][rank + rot], page = block_table[slot][pos / page_size]. */
typedef struct {
    const float* kv; long long ld;
    const float* norm_w; float eps;
    int rank, rot, rope_dims;
    const double* freqs;
    const int* pos; const int* slot; const int* block_table;
    int max_pages, page_size;
    void* cache; int ctype;
    int interleaved;                          /* rotary pairs: 0: dimension i with i + rope_dims / 2, 1: 2i with 2i + 1 */
} DlLatentKvArgs;
int dl_latent_kv_write(const DlLatentKvArgs* args /*host*/, int M, void* stream);
/* rotary on dims [offset, offset + rope_dims) of every head of x, in place.  interleaved: dimension 2i pairs with 2i + 1
 * (else i with i + rope_dims / 2); mag multiplies cos and sin (1: a pure rotation) */
int dl_rope_rows(float* x, long long ld, int M, int n_heads, int head_stride, int offset, int rope_dims,
                 const double* freqs, const int* pos, int interleaved, float mag, void* stream);

/* attention of M rows over the paged latent cache.  q_lat[M][n_heads][rank]: queries already multiplied by the
 * key up-projection; q[M][ldq] holds each head's rotated part at q_head_stride * h + q_rot_offset.
 * out[M][n_heads][rank] = softmax-weighted sum of the latents (the value up-projection follows as a dense product). */
typedef struct {
    const float* q_lat;
    const float* q; long long ldq; int q_head_stride, q_rot_offset;
    float* out;
    int n_heads, rank, rot;
    float scale;
    const int* pos; const int* slot; const int* block_table;
    int max_pages, page_size;
    const void* cache; int ctype;
    int window;                               /* > 0: only the positions j with pos[m] - j < window are visible */
    const float* sink;                        /* [n_heads] or NULL: exp(sink[h]) joins the softmax denominator, without a value */
    const float* gate; long long ld_gate;     /* NULL, or [M][ld_gate]: head h of row m leaves multiplied by sigmoid(gate[m][h]) */
} DlLatentAttnArgs;
int dl_latent_attention(const DlLatentAttnArgs* args /*host*/, int M, void* stream);
/* Tensor-core variant (bf16 cache).  The batch's rows are grouped on the host into tiles of up to `rq` rows of one
 * sequence at consecutive positions: tile_rows[n_tiles][rq] holds row indices, -1 where a tile has fewer rows
 * (rq * n_heads <= 32).  n_splits > 1: CTAs share a tile's pages and `partial` (dl_latent_tc_partial_floats() f32)
 * holds their unnormalised sums for the merge kernel that follows. */
typedef struct {
    const int* tile_rows;
    int n_tiles, rq, n_splits;
    float* partial;
    int d_pad;                                /* set by the library */
} DlLatentTiles;
int dl_latent_attention_tc_supported(int n_heads, int rank, int rot, int ctype, int rq);
long long dl_latent_tc_partial_floats(int n_tiles, int n_splits, int rank);
int dl_latent_attention_tc(const DlLatentAttnArgs* args /*host*/, const DlLatentTiles* tiles /*host*/, void* stream);

/* batch description for recurrent layers (device arrays): sequence n owns rows seq_rows[seq_start[n] .. seq_start[n+1])
 * in position order, starting at position seq_pos0[n], with its state in slot seq_slot[n]; row_seq / pos are per row */
typedef struct {
    const int* pos; const int* row_seq;
    const int* seq_start; const int* seq_rows; const int* seq_slot; const int* seq_pos0;
} DlMambaBatch;
/* out[M][channels] = silu(causal conv over in[row][in_off + ch] + bias); conv_state[slot][taps-1][channels] carries
 * the last taps-1 inputs of each slot and is updated */
int dl_mamba_conv(const DlMambaBatch* batch /*host*/, int M, int n_seq, const float* in, long long ld, int in_off,
                  const void* w, const void* bias, int wtype, float* conv_state, float* out, int channels, int taps,
                  void* stream);
/* The general form: out[m][ch] = act(bias[ch] + conv) (+ in[m][ch] if residual); bias may be NULL; act 0: none, 1: silu.
 * out must not alias in. */
typedef struct {
    const float* in; long long ld; int in_off;
    const void* w; const void* bias; int wtype;     /* w [channels][taps] */
    float* conv_state;                              /* [n_slots][taps - 1][channels] f32 */
    float* out; long long ld_out;
    int channels, taps, act, residual;
} DlConvArgs;
int dl_causal_conv(const DlMambaBatch* batch /*host*/, int M, int n_seq, const DlConvArgs* args /*host*/, void* stream);
typedef struct {
    const float* xbc; long long ld_xbc;      /* [M][x: heads*vdim | B: groups*state | C: groups*state] after conv + silu */
    const float* dt; long long ld_dt;        /* raw dt of head h at dt[m * ld_dt + h] */
    const float* dt_bias; const float* A_log; const float* D;   /* [heads] f32 */
    float* y; long long ld_y;                /* [M][heads*vdim] */
    float* ssm_state;                        /* [n_slots][heads][state][vdim] f32 */
    int n_heads, vdim, state, groups;
} DlMambaScanArgs;
int dl_mamba_scan(const DlMambaBatch* batch /*host*/, int n_seq, const DlMambaScanArgs* args /*host*/, void* stream);
/* The same scan for long prompt portions, chunks of `chunk` rows of a sequence in parallel (two launches).  chunk_seq /
 * chunk_off [n_chunks] (device): the sequence and the offset among its rows of every chunk, a sequence's chunks adjacent
 * and in order.  Scratch (f32): state [n_chunks][heads][state][vdim], decay [n_chunks][heads], cum [rows][heads]. */
typedef struct {
    const int* chunk_seq; const int* chunk_off;
    int n_chunks, chunk;
    float* state; float* decay; float* cum;
} DlMambaChunks;
int dl_mamba_scan_chunked_supported(int vdim, int state);
int dl_mamba_scan_chunked(const DlMambaBatch* batch /*host*/, const DlMambaScanArgs* args /*host*/,
                          const DlMambaChunks* chunks /*host*/, void* stream);

/* ---- linear attention with a fixed decay per head ("lightning", lightning.cu) ----------------------------------------
 * Per head, state S [dim][vdim] f32 per slot:  S <- lambda S + k (x) v (lambda = decay[h]), then y = S^T q.  q, k [M][heads * dim]
 * and v [M][heads * vdim] are f32 rows (already activated); a sequence whose first row is position 0 starts from zeros. */
typedef struct {
    const float* q; const float* k; const float* v; long long ldq, ldk, ldv;
    const float* decay;                      /* [heads] f32 */
    float* y; long long ld_y;                /* [M][heads * vdim] */
    float* state;                            /* [n_slots][heads][dim][vdim] f32 */
    int n_heads, dim, vdim;
} DlLightningArgs;
int dl_lightning_scan(const DlMambaBatch* batch /*host*/, int n_seq, const DlLightningArgs* args /*host*/, void* stream);
/* Long portions: every sequence's rows in chunks of DL_LIGHTNING_CHUNK, counted from its first row of the batch, run in
 * parallel (three launches: the chunks' own k v^T sums, their prefix over a sequence's chunks, then the scores inside a
 * chunk plus the carried state).  max_chunks = ceil(longest portion / DL_LIGHTNING_CHUNK); scratch:
 * dl_lightning_chunk_floats() f32. */
#define DL_LIGHTNING_CHUNK 64
int dl_lightning_scan_chunked_supported(int dim, int vdim);
long long dl_lightning_chunk_floats(int M, int n_seq, int n_heads, int dim, int vdim);
int dl_lightning_scan_chunked(const DlMambaBatch* batch /*host*/, int n_seq, int max_chunks, const DlLightningArgs* args /*host*/,
                              float* scratch, void* stream);

/* ---- hyper-connections: `streams` copies of the residual stream per row, x[m * ldx + s * dim + i] (hyper.cu) --------
 * write (y != NULL):  x_t <- sum_s mix[s * streams + t] x_s + mult * w_out[t] * y[m]     for all t, from the old copies
 * read  (h != NULL):  u = sum_s w_in[s] x_s (w_in NULL: ones);  h[m] = u / sqrt(mean(u^2) + eps) * norm_w (NULL: 1)
 * Both in one launch: the write of one sublayer with the read of the next.  `rows` gathers source rows (read only).
 * streams = 1, mix = w_out = {1}: the plain residual sum x += mult * y. */
#define DL_HC_MAX_STREAMS 16
typedef struct {
    float* x; long long ldx;
    int streams, dim, M;
    const float* y; long long ldy;
    const float* mix; const float* w_out; float mult;
    const float* w_in; const float* norm_w; float eps;
    const int* rows;
    float* h; long long ldh;
    float* u_out;                             /* optional: the mixed vector [M][dim] */
} DlHyperArgs;
int dl_hyper_step(const DlHyperArgs* args /*host*/, void* stream);

/* ---- sliding-window grouped-query attention whose values are its keys (window_attention.cu) -------------------------
 * Cache line per token and key/value head: [ rot(k)[0 : dim] | k[0 : rope_dims] ]; cache [page][kv_head][page_size][dim +
 * rope_dims].  Rotary: interleaved pairs, angle pos * freqs[i] (f64 [rope_dims / 2]), cos and sin times rope_scale. */
typedef struct {
    const float* k; long long ld;             /* [M][kv_heads * dim] projected keys, unrotated */
    float* q; long long ldq; int q_heads;     /* optional: [M][q_heads * dim] queries, rotated in place by the same launch */
    int kv_heads, dim, rope_dims;
    const double* freqs; float rope_scale;
    const int* pos; const int* slot; const int* block_table;
    int max_pages, page_size;
    void* cache; int ctype;
    /* separate values (vdim > 0): the line is [ key[0 : dim] | value[0 : vdim] ].  k and v both NULL: only the queries are
     * prepared (a layer that reads the cache another layer writes) */
    const float* v; long long ldv; int vdim;
    int qk_norm; float eps;                   /* every query and key head h becomes h / sqrt(mean(h^2) + eps) */
    /* separate values with rotary (rope_dims > 0): the first rope_dims dimensions of every query and key head are turned
     * BEFORE the unit norm; rope_half 1: dimension i pairs with i + rope_dims / 2, 0: 2i with 2i + 1 */
    int rope_half;
    /* head-mixed scores ("talking heads" in front of the softmax): talk [q_heads][q_heads] f32.  Since
     * score'_h = sum_g talk[h][g] q_g . k_c(g) = sum_c (sum_{g in group c} talk[h][g] q_g) . k_c, the mix is folded into the
     * queries: q_mixed[m][h][c * dim + i] = sum_{g in group c} talk[h][g] q[m][g][i] (after rotary and norm), a query of
     * kv_heads * dim numbers per head that meets the concatenated keys of all key/value heads (DlWindowAttnArgs.key_heads) */
    const float* talk; float* q_mixed; long long ld_qm;
} DlWindowKvArgs;
int dl_window_kv_write(const DlWindowKvArgs* args /*host*/, int M, void* stream);
/* out[m][h] = sum_j softmax_j(cap(scale q[m][h] . key_j)) value_j over the positions j with 0 <= pos[m] - j < window
 * (window 0: every j <= pos[m]); cap(s) = softcap tanh(s / softcap) (softcap 0: none); q already rotated. */
typedef struct {
    const float* q; long long ldq;            /* [M][heads * dim] */
    float* out; long long ldo;                /* [M][heads * dim] */
    int heads, kv_heads, dim, rope_dims;
    float scale, softcap;
    int window;
    const int* pos; const int* slot; const int* block_table;
    int max_pages, page_size;
    const void* cache; int ctype;
    int vdim;                                 /* > 0: separate values, line [ key | value[0 : vdim] ], out [M][heads * vdim] */
    int chunk;                                /* > 0: j is visible only inside i's chunk, floor(j / chunk) == floor(i / chunk) */
    const float* sink;                        /* [heads] or NULL: exp(sink[h]) joins the softmax denominator, without a value */
    int key_heads;                            /* 0 / 1: a head's key is its key/value head's; kv_heads: q is [M][heads][kv_heads * dim] and
                                                 meets the keys of ALL key/value heads side by side (head-mixed scores, see DlWindowKvArgs.talk);
                                                 the values stay those of the head's own key/value head */
} DlWindowAttnArgs;
int dl_window_attention(const DlWindowAttnArgs* args /*host*/, int M, void* stream);

/* ---- routed experts (moe.cu) ---------------------------------------------------------------------------------------- */
/* s = sigmoid(z); groups of experts/groups neighbours scored by the sum of their group_top largest s, the `keep` best
 * groups stay; sel / wgt [M][top]: the `top` eligible experts with the largest s, in that order, and their s (divided
 * by their sum if renorm). */
typedef struct {
    const float* z; long long ldz;
    int M, experts, top, groups, keep, group_top, renorm;
    int* sel; float* wgt;
    int score;                                /* 0: s = sigmoid(z); 1: s = softmax(z) over all experts */
    float scale;                              /* 0 / 1: none; else the weights are multiplied by it (after renorm, whose
                                                 divisor is the sum of the chosen scores + 1e-20) */
    const float* bias;                        /* [experts] or NULL: added to z before the scores */
} DlMoeSelectArgs;
int dl_moe_select(const DlMoeSelectArgs* args /*host*/, void* stream);
/* y[m] = sum_k wgt[m][k] * W_down[e] relu(W_up[e] x[m])^2, e = sel[m][k]; w_up [experts][ff][width], w_down
 * [experts][width][ff]; act: scratch [M * top][ff].  Weight-streaming form: one product per (row, expert) pair. */
typedef struct {
    const void* w_up; const void* w_down; int wtype;
    int width, ff, top, M, round_x;
    const float* x; long long ldx;
    const int* sel; const float* wgt;
    float* act;
    float* y; long long ldy;
    /* w_gate != NULL: gated experts, [experts][ff][width] like w_up:  a = min(gate . x, limit), b = clamp(up . x, +-limit),
     * hidden = a * sigma(1.702 a) * (1 + b)  (limit <= 0: no clamps) */
    const void* w_gate; float limit;
    int gate_act;                             /* gated experts, 1: hidden = silu(gate . x) * (up . x), no clamps */
} DlMoeArgs;
int dl_moe_rows(const DlMoeArgs* args /*host*/, void* stream);
/* Grouped form for the tensor cores.  dl_moe_plan sorts the M * top (row, expert) pairs by expert (stable) into segments
 * whose first rows are multiples of 8: grp[e] = {first sorted row, rows}, slot_row[i] = batch row of sorted row i (-1:
 * padding, up to cap >= M * top + 7 * experts), pair_pos[m * top + k] = sorted row of the pair; cnt: scratch [experts].
 * dl_xh_gather_rows builds the GEMM's activation image of the sorted rows, dl_gemm_wh_tc_grouped runs one product per
 * segment against that expert's weight image, dl_moe_combine sums a row's `top` results weighted, in the order chosen. */
typedef struct {
    const int* sel; int M, top, experts, cap;
    int* cnt; int* grp; int* slot_row; int* pair_pos;
} DlMoePlanArgs;
int dl_moe_plan(const DlMoePlanArgs* args /*host*/, void* stream);
int dl_moe_combine(const float* yp, long long ldp, const int* pair_pos, const float* wgt, int M, int top, int width,
                   float* y, long long ldy, void* stream);
int dl_xh_gather_rows(const float* x, long long ldx, const int* rows /*device*/, int n_rows, int K, int ncap, uint8_t* xh,
                      void* stream);
int dl_gemm_wh_tc_grouped(const uint8_t* wh, long long wh_group_bytes, int n_groups, const int* grp /*device*/, int d, int n,
                          const uint8_t* xh, int ncap, int max_group_rows, const DlEpilogue* epi /*host*/, int force_cg,
                          void* stream);
/* tensor-core windowed attention (bf16 cache): tiles of up to rq = dl_window_tc_rows() consecutive rows of one sequence,
 * tile_rows[n_tiles][rq] (device; -1 where a tile has fewer rows) */
int dl_window_tc_rows(int heads, int kv_heads);
int dl_window_attention_tc_supported(int heads, int kv_heads, int dim, int rope_dims, int ctype);
/* n_splits > 1: that many CTAs share each tile's pages; partial: dl_window_tc_partial_floats() f32 of scratch */
long long dl_window_tc_partial_floats(int n_tiles, int kv_heads, int n_splits, int dim);
int dl_window_attention_tc(const DlWindowAttnArgs* args /*host*/, const int* tile_rows, int n_tiles, int rq, int n_splits,
                           float* partial, void* stream);
/* The tile kernel for values of a width of their own (vdim > 0, any multiple of 8 up to 128; rope_dims 0, no soft cap) and
 * for head-mixed scores (key_heads = kv_heads: q [M][heads][kv_heads * dim], talk_attention.cu).  Tiles as above. */
int dl_talk_attention_tc_supported(int heads, int kv_heads, int dim, int vdim, int key_heads, int ctype);
/* stacked (row x head-of-a-group) rows per tile for portions of `longest` rows: 16 (decoding), 64 or 128; rq = that / (heads / kv_heads) */
int dl_talk_tc_tile_rows(int heads, int kv_heads, int dim, int vdim, int key_heads, int longest);
long long dl_talk_tc_partial_floats(int n_tiles, int kv_heads, int n_splits, int vdim, int tile_rows);
int dl_talk_attention_tc(const DlWindowAttnArgs* args /*host*/, const int* tile_rows, int n_tiles, int rq, int n_splits,
                         float* partial, void* stream);

#ifdef __cplusplus
}
#endif
#endif
