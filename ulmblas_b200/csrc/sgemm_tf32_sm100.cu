// placeholder until the tcgen05 kernel lands (replaced below in this file's history)
#include "common.h"
namespace ulmb200 {
int sgemm_3xtf32_device(cudaStream_t, int, int, int64_t, int64_t, int64_t, float, const float *, int64_t,
                        const float *, int64_t, float, float *, int64_t)
{
    fprintf(stderr, "ulmblas_b200: 3xTF32 SGEMM is not built into this library\n");
    return ULMB200_BAD_ARGUMENT;
}
}  // namespace ulmb200
