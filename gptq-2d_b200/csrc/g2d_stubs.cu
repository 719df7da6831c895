// Entry points declared in the header whose kernels are not built yet.
#include "g2d_common.cuh"

extern "C" int g2d_ldl_workspace_bytes(int, int64_t, size_t *) { return G2D_ERR_UNSUPPORTED; }
extern "C" int g2d_ldl_of_inverse(int, int64_t, void *, int32_t, void *, int32_t *, void *, size_t, void *) { return G2D_ERR_UNSUPPORTED; }
