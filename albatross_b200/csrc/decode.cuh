// Phase list executed by the persistent batch-1 decode kernel (see decode.cu).
#pragma once
#include "gemv.cuh"
#include "head.cuh"

namespace ab {

enum PhaseType : int { PHASE_GEMV = 0, PHASE_HEAD = 1 };

struct __align__(16) DecodePhase {
    int type, pad[3];
    GemvParams g;
    HeadParams h;
};

struct DecodeProgram {
    int n_phases, stages, Kn, Kq;
    unsigned* barrier;       // points at barrier_word of the device copy
    unsigned long long* timeline;  // optional: block 0 stores %globaltimer at [2i] phase start, [2i+1] phase end
    unsigned barrier_word, pad[3];
    DecodePhase phases[1];   // n_phases entries
};

size_t decode_program_bytes(int n_layer);
int decode_launch(const DecodeProgram* prog_dev, unsigned* barrier_dev, int stages, int Kn, int Kq, cudaStream_t stream);

}  // namespace ab
