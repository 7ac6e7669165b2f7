// Single translation unit of the library: the kernels share one device-side status word and are
// compiled together for sm_100a (see albatross_b200/build.py for the command line).
#include "decode.cu"
#include "engine.cu"
#include "gemm.cu"
#include "gemv.cu"
#include "head.cu"
#include "rows.cu"
