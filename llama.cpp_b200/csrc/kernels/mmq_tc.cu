// Prefill-time quantized GEMM on the 5th-generation tensor cores (placeholder
// until the tcgen05 kernel lands: reports "not supported" so callers take the
// mat-vec path for every N).
#include "common.cuh"
#include "kernels.h"

namespace b200 {
bool mmq_tc_supported(int, int64_t, int64_t, int64_t) { return false; }
size_t mmq_tc_workspace_bytes(int64_t, int64_t) { return 0; }
cudaError_t launch_mmq_tc(int, const void *, int64_t, const float *, int64_t, float *, int64_t, int64_t, int64_t, int64_t,
                          void *, const LaunchCtx &) { return cudaErrorNotSupported; }
}  // namespace b200
