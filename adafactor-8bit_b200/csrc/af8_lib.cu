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
#include "apollo_rules.cuh"
#include "noalloc.cuh"

extern "C" int af8_version(void) { return AF8_VERSION; }

extern "C" const char *af8_last_error(void) { return af8::error_buffer(); }

extern "C" int32_t af8_struct_size(int32_t index)
{
    static const int32_t sizes[] = {
        (int32_t)sizeof(af8_fullrank_tensor), (int32_t)sizeof(af8_dyn_scalars), (int32_t)sizeof(af8_fullrank_cfg),
        (int32_t)sizeof(af8_norm_tensor), (int32_t)sizeof(af8_scale_tensor), (int32_t)sizeof(af8_small_state),
        (int32_t)sizeof(af8_factored_tensor), (int32_t)sizeof(af8_factored_cfg),
        (int32_t)sizeof(af8_apollo_scalars_in), (int32_t)sizeof(af8_apollo_scalars), (int32_t)sizeof(af8_apollo_proj_desc),
        (int32_t)sizeof(af8_apollo_finish_tensor), (int32_t)sizeof(af8_lag_tensor), (int32_t)sizeof(af8_apollo_rule),
        (int32_t)sizeof(af8_apollo_apply_tensor),
    };
    if (index < 0 || index >= (int32_t)(sizeof(sizes) / sizeof(sizes[0]))) return -1;
    return sizes[index];
}
