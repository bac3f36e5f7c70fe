#include "tc_kernels.cuh"

namespace natten {

int tc_fused_fwd(int, const Geo&, const void*, const void*, const void*, const void*, const void*,
                 void*, void*, cudaStream_t)
{
    return -2;
}

int tc_fused_bwd(int, const Geo&, const void*, const void*, const void*, const void*, const void*,
                 const void*, const void*, const void*, const void*, void*, void*, void*, void*, void*,
                 void*, cudaStream_t)
{
    return -2;
}

size_t tc_bwd_workspace_bytes(int, const Geo&) { return 0; }

} // namespace natten
