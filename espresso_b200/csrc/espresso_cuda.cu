// Single translation unit of libespresso_cuda.so: the kernels live in headers that define __global__
// functions, so the engine and the C ABI are compiled together.
#include "engine.cu"
#include "capi.cu"
#include "gguf_reader.cu"
#include "static_head.cu"
#include "tc_host.cu"
