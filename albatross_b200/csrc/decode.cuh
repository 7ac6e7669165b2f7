// Phase list executed by the persistent batch-1 decode kernel (see decode.cu).
#pragma once
#include "gemv.cuh"
#include "head.cuh"

namespace ab {

enum PhaseType : int { PHASE_GEMV = 0, PHASE_HEAD = 1 };

struct __align__(16) DecodePhase {
    int type;
    int next_gemv;   // index of the next matrix-vector phase after this one, or -1
    int no_barrier;  // what follows the phase: 0 = barrier among all blocks; 1 or 2 = a block barrier only (1: the next
                     // phase consumes what this block itself produced; 2: dataflow mode, the phase's outputs are
                     // tagged words and their readers wait on the words themselves)
    int rows_per_block;  // > 0: block b owns rows [b * rows_per_block, +rows_per_block) of every segment
    GemvParams g;
    HeadParams h;
};

struct __align__(16) BlockPlan;

struct DecodeProgram {
    int n_phases, Kn, xq_bytes, first_gemv;
    int n_blocks;
    int l2_prefetch_bytes;   // per block: how much of its share of the next matrix-vector phase is pulled into L2 early
    int smem_prefetch;       // warps start the copy of their first slice of the next phase before the barrier
    int early_slice;         // warps request the first slice of their first item right behind the input loads
    int barrier_prefetch;    // ... or while the block waits at the grid barrier before that phase
    int l2_prefetch2_bytes;  // ... and how much more once the phase's own inputs have arrived (dataflow mode)
    int pad1[2];
    const BlockPlan* plans;  // [n_phases][n_blocks], computed on the host (device copy follows the phases)
    unsigned* barrier;       // points at barrier_word of the device copy
    unsigned long long* timeline;  // optional: block 0 stores %globaltimer at [2i] phase start, [2i+1] phase end
    unsigned barrier_word;
    unsigned epoch;          // dataflow mode: tag base of the next token (tags are epoch + phase index + 1, 16 bits); the
                             // kernel advances it by n_phases when a token is done, so no two writes of a word that
                             // follow one another carry the same tag
    int timeline_block;      // block that records the timeline; < 0: all of them
    unsigned timeline_stride;   // entries per block in that case
    DecodePhase phases[1];   // n_phases entries
};

size_t decode_program_bytes(int n_layer, int n_blocks);
size_t decode_plans_offset(int n_phases);       // byte offset of the plan table inside the program buffer
size_t decode_timeline_offset(int n_phases, int n_blocks);
int decode_launch(const DecodeProgram* prog_dev, unsigned* barrier_dev, int Kn, int xq_bytes, cudaStream_t stream);

}  // namespace ab
