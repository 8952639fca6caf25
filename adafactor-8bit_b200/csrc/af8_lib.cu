// libaf8: single translation unit.  The kernels share two constant-memory
// codebooks, so everything is compiled together:
//   nvcc -gencode arch=compute_100a,code=sm_100a -fmad=false ... af8_lib.cu
#include "common.cuh"
#include "fullrank_fast.cuh"
#include "fullrank_generic.cuh"
#include "fullrank_api.cuh"
#include "codec.cuh"
#include "scale.cuh"
#include "factored.cuh"
#include "apollo.cuh"
#include "noalloc.cuh"

extern "C" int af8_version(void) { return AF8_VERSION; }

extern "C" const char *af8_last_error(void) { return af8::error_buffer(); }
