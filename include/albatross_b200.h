/*
 * albatross_b200 — C ABI of the sm_100a kernels for the RWKV-7 decode hot path.
 *
 * Plain pointers and sizes only; every pointer is a DEVICE pointer unless said otherwise; `stream`
 * is a cudaStream_t passed as void*. Every function returns 0 on success and a negative code
 * otherwise (AB_ERR_*); ab_last_error() gives the message of the calling thread's last failure.
 * Kernels are asynchronous on `stream`; nothing here allocates device memory.
 *
 * Each entry point names the reference interface it replaces (paths inside the reference project).
 */
#ifndef ALBATROSS_B200_H
#define ALBATROSS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AB_OK 0
#define AB_ERR_BAD_ARG (-1)
#define AB_ERR_CUDA (-2)
#define AB_ERR_TOO_LARGE (-3)
#define AB_ERR_DEVICE_WAIT (-4)

/* weight formats */
#define AB_FMT_F16 0   /* fp16 rows                                                        */
#define AB_FMT_I8 1    /* int8 rows + fp32 scale per output row (+ optional per-input scale) */
#define AB_FMT_FP4 2   /* NVFP4: e2m1 pairs, e4m3 scale per 16 inputs, fp32 tensor scale     */

/* A weight matrix in the reference's storage order: [n_out, k] row-major, i.e. nn.Linear's
 * [out, in] storage that reference/rwkv7.py:88-90 views transposed. */
typedef struct ab_mat {
    int32_t fmt, n_out, k, _pad;
    const void* w;          /* int8 [n_out,k] | fp16 [n_out,k] | uint8 [n_out,k/2] (even k in the low nibble) */
    const void* scale;      /* I8: float [n_out] | FP4: uint8 e4m3 [n_out,k/16] | F16: NULL */
    const float* col_scale; /* I8 only, optional float [k]: W ~= q * row_scale * col_scale */
    float tscale;           /* FP4 tensor scale (1.0f otherwise) */
    float _pad2;
} ab_mat;

/* One RWKV-7 block. Vectors are fp16 [n_embd]; names follow the checkpoint keys read at
 * reference/rwkv7.py:142-152. Adapter down-projections are stored TRANSPOSED ([rank, n_embd],
 * fp16, AB_FMT_F16 mats) so that they stream like any other output row; up-projections keep the
 * checkpoint layout [rank, n_embd]. */
typedef struct ab_layer {
    const void *ln1_w, *ln1_b, *ln2_w, *ln2_b;
    const void *x_r, *x_w, *x_k, *x_v, *x_a, *x_g;
    const void *w0, *a0, *v0, *k_k, *k_a, *r_k, *lnx_w, *lnx_b;
    const void* ffn_x_k;
    ab_mat receptance, key, value, output, ffn_key, ffn_value;
    ab_mat w1t, a1t, v1t, g1t;
    const void *w2, *a2, *v2, *g2;
    /* batched path: the four up-projections as [n_embd, rank] fp16 AB_FMT_F16 mats (may be empty at batch 1) */
    ab_mat w2t, a2t, v2t, g2t;
} ab_layer;

typedef struct ab_model_desc {
    int32_t n_layer, n_embd, vocab, _pad;
    const void* emb;              /* fp16 [vocab, n_embd], ln0 already folded in (reference/rwkv7.py:93) */
    const void *lnout_w, *lnout_b;
    ab_mat head;
    const ab_layer* layers;       /* HOST array of n_layer entries; copied by ab_model_create */
} ab_model_desc;

typedef struct ab_model ab_model;

/* ---- diagnostics ------------------------------------------------------------------------- */
const char* ab_last_error(void);
int ab_version(void);
/* Reads and clears the device-side status word. Bits: 1, 2, 4 = a bounded device wait gave up in the matrix-vector,
 * tensor-core or WKV / persistent kernels; 8 = a token id outside [0, vocab) reached a kernel (it was clamped to the
 * table, never followed). Synchronises the device. Host pointer. After a non-zero wait bit, split-K arrival counters
 * may be stale: those of ab_gemm_static's built-in area are cleared here, a caller's own scratch / workspace is not. */
int ab_device_status(uint32_t* status_host);

/* ---- WKV-7 state update -------------------------------------------------------------------
 * Replaces torch.ops.rwkv7_state_fwd_fp16.forward(B,T,C,H,state,r,w,k,v,a,b,y)
 * (reference/cuda/rwkv7_state_fwd_fp16.cpp:8-14; kernel reference/cuda/rwkv7_state_fwd_fp16.cu:7-62).
 * state fp32 [B,H,64,64] updated in place; r,w,k,v,a,b,y fp16 [B,T,C]; w is the pre-transform decay
 * (the kernel applies exp(-exp(w))). Unlike the reference it launches on `stream`, not the legacy stream. */
int ab_wkv7_fwd(int B, int T, int C, int H, float* state, const void* r, const void* w, const void* k,
                const void* v, const void* a, const void* b, void* y, void* stream);

/* ---- batch-1 matrix-vector products -------------------------------------------------------
 * Replace the fp16 `x @ W` call sites at batch 1 (reference/rwkv7.py:230,232,233,250,308,309,156)
 * with de-quantisation fused into the product. x fp16 [k], y fp16 [n_out]. */
int ab_gemv(const ab_mat* m, const void* x, void* y, void* stream);

/* Host-only self-check of how ab_gemv and the persistent kernel split a list of matrices between `n_blocks` blocks
 * (all arrays are HOST arrays of `nseg` entries: weight format, output rows, input length): every group of four
 * rows is owned by exactly one block and a block's share of a matrix is contiguous. Runs without a GPU. */
int ab_gemv_plan_selftest(const int32_t* fmt, const int32_t* n_rows, const int32_t* k, int nseg, int n_blocks,
                          int32_t* max_items, int32_t* max_cost_spread_pct);

/* ---- batched matrix products (tensor cores) -----------------------------------------------
 * Replace the `[B,T,D] @ W` call sites of the batch path (reference/rwkv7.py:283,285,286,300,322,323,220).
 * x fp16 [rows, k] row-major, y fp16 [rows, n_out]; epi is one of AB_EPI_*; resid (fp16 [rows,n_out])
 * is added when epi == AB_EPI_RESID and may alias y. `scratch` holds at least
 * ab_gemm_scratch_bytes(m, rows) bytes (split-K arrival counters and fp32 partial tiles); it must be zero the
 * first time it is used and is left with zeroed counters. Calls that share a scratch area must not overlap. */
#define AB_EPI_NONE 0
#define AB_EPI_TANH 1
#define AB_EPI_SIGMOID 2
#define AB_EPI_RELU2 3
#define AB_EPI_RESID 4
size_t ab_gemm_scratch_bytes(const ab_mat* m, int rows);
int ab_gemm(const ab_mat* m, int rows, const void* x, void* y, int epi, const void* resid, void* scratch,
            void* stream);

/* ab_gemm without a scratch argument (no counterpart in the reference). The split-K counters and partial tiles
 * live in a fixed AB_GEMM_STATIC_SCRATCH_BYTES array inside the library, so the call neither receives nor makes
 * any device allocation. It is for callers that have no device memory to hand over and must not create any at
 * this point: an operator running under a host framework that owns the whole device heap through its own caching
 * allocator (a raw allocation there can fail although the pool has room, and allocating or freeing may synchronise
 * the device in the middle of a decode step), or a code path whose buffers are all planned ahead of time.
 * Same results as ab_gemm. Products that need more scratch than the array holds (ab_gemm_scratch_bytes(m, rows) >
 * AB_GEMM_STATIC_SCRATCH_BYTES: long-k products with few output rows at large batch) fail with AB_ERR_TOO_LARGE
 * and a message; use ab_gemm for those. The first call on each device looks the array up (cudaGetSymbolAddress,
 * a host-side call, not a stream operation) and clears its counters on `stream`: make that first call during
 * set-up, before any stream capture begins. There is ONE array per device: two ab_gemm_static calls that can
 * overlap in time (different streams, or different host threads on different streams) race on it; keep them
 * on one stream or order them with events. The look-up itself is guarded by a lock, so the first calls of two host
 * threads may coincide.
 * Recovery: the kernels leave the arrival counters at zero, except when a bounded device wait gave up (a non-zero
 * ab_device_status) or a launch was aborted half-way. ab_device_status clears the counters of this built-in area
 * whenever it reports a non-zero status; ab_gemm_static_reset(stream) does the same on request. (The scratch a
 * caller passes to ab_gemm, and the workspace of ab_forward, are the caller's to clear in that case.) */
#define AB_GEMM_STATIC_SCRATCH_BYTES (8u * 1024u * 1024u)
int ab_gemm_static(const ab_mat* m, int rows, const void* x, void* y, int epi, const void* resid, void* stream);
int ab_gemm_static_reset(void* stream);
/* Test hook (no counterpart in the reference): reads (write == 0) or overwrites (write != 0) arrival counter `index`
 * of the built-in area of the current device through the HOST pointer `value_host`; synchronises the device. */
int ab_gemm_static_debug_counter(int index, int write, uint32_t* value_host);

/* ---- token sampling on the device -----------------------------------------------------------
 * Replaces sampler_simple_batch (reference/utils.py:43-45: uniform noise in [0, noise) added to the logits, then
 * the first column of a descending argsort) without sorting and without leaving the device: out[r] = argmax over
 * the row of logits[r, :] + U(0, noise), ties to the lowest index. logits fp16 [rows, vocab], out int32 [rows].
 * noise == 0 is plain greedy decoding. The noise is a hash of (seed, row, column), not torch's generator. */
int ab_sample_rows(const void* logits, int rows, int vocab, float noise, uint32_t seed, int32_t* out, void* stream);
/* The same with 64-bit ids (the dtype the reference's sampler returns). `out` may be device memory or pinned host
 * memory that the device can address: the ids then need no copy of their own on the way to the host. */
int ab_sample_rows_i64(const void* logits, int rows, int vocab, float noise, uint32_t seed, int64_t* out, void* stream);

/* ---- de-quantisation dump (parity checks) ---------------------------------------------------
 * Writes the kernels' in-register de-quantised weights as fp32 [n_out,k] (tensor/row/column scales applied). */
int ab_dequant(const ab_mat* m, float* out, void* stream);

/* ---- whole-model forward -------------------------------------------------------------------
 * ab_forward replaces RWKV_x070.forward / forward_batch (reference/rwkv7.py:98-126, :128-221):
 * tokens int32 [B,T] on the device; state = HOST array of 3*n_layer device pointers laid out as
 * reference/rwkv7.py:102-105 / :122-125 ([3i] fp16 [B,D], [3i+1] fp32 [B,H,64,64], [3i+2] fp16 [B,D]),
 * all updated in place; logits fp16 [B,V] (or [B,T,V] when full_output). `workspace` holds at
 * least ab_workspace_bytes(model, B, T) bytes and is scratch. */
int ab_model_create(const ab_model_desc* desc, ab_model** out);
void ab_model_destroy(ab_model* m);
size_t ab_workspace_bytes(const ab_model* m, int B, int T);
int ab_forward(ab_model* m, int B, int T, const int32_t* tokens, void* const* state, void* workspace,
               void* logits, int full_output, void* stream);
/* One stage of a layer pipeline (no counterpart in the reference, which is single-GPU; the per-block math is
 * reference/rwkv7.py:198-216). The model holds a contiguous run of blocks; option "layer_offset" gives the index
 * of its first block in the whole network (block 0 defines v_first, reference/rwkv7.py:239, :292).
 * First stage: tokens != NULL (needs desc.emb), later stages: x_in fp16 [B*T, D]. v_first fp16 [B*T, D] is written
 * by the first stage and read by the others. Last stage: logits fp16 [B,V] (needs desc.head / lnout), other
 * stages: x_out fp16 [B*T, D]. State and workspace as in ab_forward (sized by ab_workspace_bytes). */
int ab_forward_stage(ab_model* m, int B, int T, const int32_t* tokens, const void* x_in, void* v_first,
                     void* const* state, void* workspace, void* x_out, void* logits, void* stream);
/* Batch-1 decode as ONE persistent kernel per token (same results as ab_forward with B = T = 1).
 * ab_decode_program_build writes the token's phase list for a fixed set of buffers (token id, state
 * tensors, workspace, logits) into `program` (device memory, at least ab_decode_program_bytes(m) bytes,
 * 256-byte aligned) and synchronises `stream`; ab_decode_run launches the kernel (cooperative launch,
 * one block per SM). A program stays valid while those buffers stay where they are. Replaces the loop
 * body of RWKV_x070.forward_one (reference/rwkv7.py:128-157). */
size_t ab_decode_program_bytes(const ab_model* m);
/* Profiling aid: byte offset, inside the program buffer, of the per-phase timestamps that the kernel writes
 * when the "timeline" option was set before ab_decode_program_build. */
size_t ab_decode_timeline_offset(const ab_model* m);
int ab_decode_program_build(ab_model* m, const int32_t* token, void* const* state, void* workspace, void* logits,
                            void* program, void* stream);
int ab_decode_run(ab_model* m, void* program, void* stream);
/* Options (set before ab_decode_program_build for those of the persistent kernel):
 *   "pdl" (1)             programmatic dependent launch between the kernels of a step
 *   "debug_sync" (0)      synchronise and check after every launch
 *   "timeline" (0)        persistent kernel records per-phase timestamps (ab_decode_timeline_offset)
 *   "layer_offset" (0)    index of this model's first block in the whole network (pipeline stages)
 *   "stage_gemv" (0)      ab_forward_stage with B = T = 1 runs the batch-1 matrix-vector kernels (the launches of
 *                         ab_forward at B = T = 1) instead of the row-wise program
 *   "merge_ups" (0)       persistent kernel: adapter up-projections inside the per-head phase instead of a phase
 *                         of matrix-vector rows of their own (bit-identical to ab_forward at B = T = 1, 3 % slower;
 *                         switches "smem_prefetch" and "barrier_prefetch" off)
 *   "fuse_heads" (1)      persistent kernel in dataflow mode: no barrier among all blocks; the vectors that cross
 *                         blocks are tagged words their readers wait for, and block 2h runs head h right after its
 *                         share of the r/k/v rows (needs 2 * heads + 4 blocks; else the barrier mode is used)
 *   "pair_split" (16)     dataflow mode: how many of a head's 48 r/k/v row groups block 2h takes (block 2h+1: the rest)
 *   "early_slice" (-1)    first weight slice of every warp requested into shared memory ahead of the phase's input
 *                         vector: 1 = at the start of the phase, 2 = once the inputs have arrived, 0 = off,
 *                         -1 = 1 in dataflow mode, 0 otherwise
 *   "l2_prefetch_kb" (-1), "l2_prefetch2_kb" (-1)
 *                         per block: KB of its share of the next matrix-vector phase asked into L2 when it has
 *                         streamed its last weights of the current one, and KB more when that phase's inputs have
 *                         arrived; -1 = 64 and 128 in dataflow mode, 0 otherwise
 *   "timeline_block" (0)  block whose timestamps "timeline" records; -1: every block, each into its own run of
 *                         6 * (6 * n_layer + 1) entries behind ab_decode_timeline_offset
 *   "smem_prefetch" (0), "barrier_prefetch" (0)
 *                         barrier mode only: earlier ways of requesting the next phase's weights early (measured
 *                         slower than not doing it there: they delay the loads of the phase's input vector)
 *   "stages"              accepted and ignored */
int ab_model_set_option(ab_model* m, const char* name, int value);

#ifdef __cplusplus
}
#endif
#endif /* ALBATROSS_B200_H */
