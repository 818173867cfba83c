// One part of the tiled kernels for one storage type: compiled several times with different
// -DNDC_DW4_PART (0 forward, 1 backward of volumes, 2 backward of images) and -DNDC_DW4_T
// (0 float32, 1 bfloat16).  ndc_abi.cu declares the same instances `extern`.
#include "ndc_b200.h"
#include "ndc_common.cuh"
#include "ndc_dw4_host.cuh"

#if NDC_DW4_T == 0
typedef float ndc_inst_t;
#else
typedef __nv_bfloat16 ndc_inst_t;
#endif

namespace ndc {
namespace dw4 {
#if NDC_DW4_PART == 0
NDC_DW4_FWD_INSTANCES(template, ndc_inst_t)
#elif NDC_DW4_PART == 1
NDC_DW4_BWD3D_INSTANCES(template, ndc_inst_t)
#else
NDC_DW4_BWD2D_INSTANCES(template, ndc_inst_t)
#endif
}  // namespace dw4
}  // namespace ndc
