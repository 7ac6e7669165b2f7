// Parameter blocks of the batch-1 streaming matrix-vector kernel (see gemv.cu).
#pragma once
#include "common.cuh"

namespace ab {

enum Fmt : int { FMT_F16 = 0, FMT_I8 = 1, FMT_FP4 = 2 };
enum Epi : int { EPI_NONE = 0, EPI_TANH = 1, EPI_SIGMOID = 2, EPI_RELU2 = 3, EPI_RESID = 4 };

constexpr int GEMV_MAX_SEG = 7;
constexpr int GEMV_WARPS = 16;                        // consumer warps; one more warp produces
constexpr int GEMV_THREADS = (GEMV_WARPS + 1) * 32;
constexpr int GEMV_TILE_BYTES = 4096;  // weight bytes of one pipeline stage
constexpr int GEMV_SCALE_BYTES = 512;  // NVFP4 block scales of one stage
constexpr int GEMV_STAGE_BYTES = GEMV_TILE_BYTES + GEMV_SCALE_BYTES;
constexpr int GEMV_PIECE_BYTES = 4096; // bytes of one row inside a stage: bulk copies below ~4 KB lose bandwidth

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
};

struct __align__(16) GemvParams {
    GemvSeg seg[GEMV_MAX_SEG];
    int nseg, K;            // K: length of the launch's shared input (0 when every segment brings its own)
    const __half* x;        // shared input vector [K] (ignored when emb != null)
    const __half* emb;      // optional embedding table [V,K]: x = emb[token[0]]
    const int* token;
    const __half* x_prev;   // token-shift state [K] (needed when any seg has mix)
    const __half* ln_w;     // layer-norm weight/bias [K], or null: no normalisation
    const __half* ln_b;
    __half* ln_out;         // optional: block 0 stores the normalised input here
    __half* x_copy;         // optional: block 0 stores the raw input here (embedding row -> residual stream)
    const __half* copy_src; // optional: block 0 copies copy_n halves to copy_dst (token-shift state hand-over)
    __half* copy_dst;
    int copy_n;
    int stages;             // pipeline depth per warp
    int use_pdl;            // kernel was launched with programmatic stream serialization
};

__host__ __device__ inline int gemv_row_bytes(int fmt, int K) { return fmt == FMT_I8 ? K : (fmt == FMT_F16 ? 2 * K : K / 2); }

// A stage holds R rows x `piece` bytes of each row. Rows shorter than GEMV_PIECE_BYTES are taken whole,
// and then the R rows of a group are one contiguous run of memory (a single bulk copy).
struct GemvGeom {
    int R;        // rows per group
    int piece;    // bytes of a row per stage
    int kc;       // K elements per stage
    int nkc;      // stages per group
    int contig;   // rows of a stage are contiguous in memory
};
__host__ __device__ inline GemvGeom gemv_geom(int fmt, int K) {
    GemvGeom g;
    const int rb = gemv_row_bytes(fmt, K);
    g.piece = rb < GEMV_PIECE_BYTES ? rb : GEMV_PIECE_BYTES;
    g.R = GEMV_TILE_BYTES / g.piece;
    if (g.R > 8) g.R = 8;
    g.kc = fmt == FMT_I8 ? g.piece : (fmt == FMT_F16 ? g.piece / 2 : g.piece * 2);
    g.nkc = (K + g.kc - 1) / g.kc;
    g.contig = g.piece == rb;
    return g;
}
__host__ __device__ inline int gemv_rows_per_group(int fmt, int K) { return gemv_geom(fmt, K).R; }
// Relative consumer cost of one row group (stages x per-stage cost of the format): blocks get equal cost,
// not equal bytes, because fp16 and NVFP4 rows take more instructions per byte than int8 rows.
__host__ __device__ inline int gemv_group_cost(int fmt, int K) {
    return gemv_geom(fmt, K).nkc * (fmt == FMT_I8 ? 2 : (fmt == FMT_F16 ? 3 : 5));
}

int gemv_check(GemvParams& p);   // validates and fills per-segment defaults
int gemv_groups(const GemvParams& p);
int gemv_launch(const GemvParams& p, cudaStream_t stream);

}  // namespace ab
