// Placeholder until the tcgen05 backward lands: reports "not covered" so that the
// CUDA-core kernels serve every backward call.
#include "common.cuh"
#include "launch.h"

namespace evo {
bool sm100_bwd_supported(int, const Args&) { return false; }
size_t sm100_bwd_workspace_bytes(int, const Args&) { return 0; }
int launch_sm100_bwd(int, const Args&, void*, size_t, cudaStream_t, int*) { return EVOATTN_ERR_UNSUPPORTED; }
}  // namespace evo
