// Parameter blocks of the batch-1 streaming matrix-vector product (see gemv_body.cuh, gemv.cu).
#pragma once
#include "common.cuh"

namespace ab {

enum Fmt : int { FMT_F16 = 0, FMT_I8 = 1, FMT_FP4 = 2 };
enum Epi : int { EPI_NONE = 0, EPI_TANH = 1, EPI_SIGMOID = 2, EPI_RELU2 = 3, EPI_RESID = 4 };

constexpr int GEMV_MAX_SEG = 7;
constexpr int GEMV_WARPS = 16;                  // every warp streams weights straight into registers
constexpr int GEMV_THREADS = GEMV_WARPS * 32;
constexpr int GEMV_ROWS = 4;                    // output rows a warp works on at a time (they share the input loads)
constexpr int GEMV_SWEEPS = 4;                  // 512-byte warp loads of each row issued back to back
constexpr int GEMV_SLICE_BYTES = GEMV_SWEEPS * 512;   // bytes of each row per slice: 16 loads of 16 bytes per lane
constexpr int GEMV_PART_FLOATS = 4096;          // per-block partial sums: rows of the block x K slices
constexpr int GEMV_MAX_ROWS_PER_BLOCK = 1024;   // one epilogue thread per output row of the block

// One matrix (a contiguous run of output rows) inside a fused launch.
struct GemvSeg {
    const void* w;           // int8 [n,K] | fp16 [n,K] | e2m1 pairs [n,K/2]; rows K-contiguous
    const void* scale;       // int8: float[n] row scales | NVFP4: e4m3 [n,K/16] | fp16: unused
    const __half* x;         // own plain input vector [K], or null: the launch's (normalised, shifted) input
    const __half* mix;       // token-shift lerp vector [K], or null: take the input as is (needs x == null)
    const float* col_scale;  // optional per-input-column scale folded into x (int8 only)
    const __half* resid;     // EPI_RESID: vector added to the result (may alias out)
    __half* out;             // [n]
    float tscale;            // NVFP4 per-tensor scale, 1 otherwise
    int fmt, epi, n_rows;
    int K;                   // input length of this matrix (== GemvParams::K when x is null)
    // Persistent kernel, dataflow mode: a vector that crosses blocks is an array of 32-bit words, fp16 value in the low
    // half and a 16-bit tag of the phase that wrote it in the high half, so that its readers can tell a word that has
    // arrived from one that has not without any barrier. 0 = plain fp16 array; else 1 + index of the writing phase.
    int tag_x, tag_resid, tag_out;
    int pad_;
};

struct __align__(16) GemvParams {
    GemvSeg seg[GEMV_MAX_SEG];
    int nseg, K;            // K: length of the launch's shared input (0 when every segment brings its own)
    const __half* x;        // shared input vector [K] (ignored when emb != null)
    const __half* emb;      // optional embedding table [V,K]: x = emb[token[0]]
    const int* token;
    int tag_in;             // shared input `x` (and `x_copy`): 0 = plain fp16, else 1 + index of the phase that wrote it
    int emb_rows;           // rows of the embedding table: a token id outside [0, emb_rows) is clamped and reported
    const __half* x_prev;   // token-shift state [K] (needed when any seg has mix)
    const __half* ln_w;     // layer-norm weight/bias [K], or null: no normalisation
    const __half* ln_b;
    __half* ln_out;         // optional: block 0 stores the normalised input here
    __half* x_copy;         // optional: block 0 stores the raw input here (embedding row -> residual stream)
    const __half* copy_src; // optional: block 0 copies copy_n halves to copy_dst (token-shift state hand-over)
    __half* copy_dst;
    int copy_n;
    int use_pdl;            // kernel was launched with programmatic stream serialization
};

__host__ __device__ inline int gemv_row_bytes(int fmt, int K) { return fmt == FMT_I8 ? K : (fmt == FMT_F16 ? 2 * K : K / 2); }
__host__ __device__ inline int gemv_slices(int fmt, int K) { return (gemv_row_bytes(fmt, K) + GEMV_SLICE_BYTES - 1) / GEMV_SLICE_BYTES; }
__host__ __device__ inline int gemv_groups_of(int n_rows) { return (n_rows + GEMV_ROWS - 1) / GEMV_ROWS; }
// Relative cost of one row group: blocks get equal cost, not equal bytes, because NVFP4 rows take more
// instructions per byte than int8 rows. fp16 rows cost what int8 rows cost per byte (measured per work item in
// the r/k/v + adapter phase of the persistent kernel: 0.24 us vs 0.23 us per 8 KiB item).
// Rows shorter than a slice (the adapter up-projections, K = rank) cost in proportion to their bytes, with a floor
// for the fixed work per item.
__host__ __device__ inline int gemv_group_cost(int fmt, int K) {
    const int per_slice = fmt == FMT_FP4 ? 32 : 16;
    const int rb = gemv_row_bytes(fmt, K);
    if (rb >= GEMV_SLICE_BYTES) return gemv_slices(fmt, K) * per_slice;
    const int c = (per_slice * rb + GEMV_SLICE_BYTES - 1) / GEMV_SLICE_BYTES;
    return c < per_slice / 4 ? per_slice / 4 : c;
}
// Shared-memory bytes of one segment's prepared input (int8: high + low bytes; otherwise fp16).
__host__ __device__ inline int gemv_xq_bytes(int K) { return 2 * ((K + 511) & ~511); }

int gemv_check(GemvParams& p);   // validates and fills per-segment defaults
int gemv_groups(const GemvParams& p);
int gemv_check_partials(const GemvParams& p, int grid);
int gemv_launch(const GemvParams& p, cudaStream_t stream);

}  // namespace ab
