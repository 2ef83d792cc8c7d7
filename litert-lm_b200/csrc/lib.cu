// Single translation unit of libb200lm.so: the kernels live in headers, so the
// executor and the operator-level ABI are compiled together.
#include "executor.cu"
#include "ops.cu"
#include "ops_static.cu"
