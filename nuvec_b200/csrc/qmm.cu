// Placeholder until the tcgen05 kernel lands: nothing is eligible, callers use the other kernels.
#include "qmm.cuh"
namespace nvc {
bool qmm_eligible(int32_t, int32_t, int32_t, int32_t, int32_t, int64_t, int64_t, int64_t, const void *, int64_t,
                  const uint32_t *) { return false; }
int32_t launch_qmm(nvc_device *, const QmmParams &) { return set_error(NVC_ERR_UNSUPPORTED, "qmm: not built"); }
}  // namespace nvc
