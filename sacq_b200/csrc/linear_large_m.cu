// placeholder until the tcgen05 kernel lands
#include "common.cuh"
namespace sacq {
bool large_m_supported(const sacq_layer*) { return false; }
int launch_large_m(const sacq_layer*, const void*, const float*, int64_t, void*, int64_t, cudaStream_t) {
  return set_error(SACQ_ERR_UNSUPPORTED, "large-M kernel not built");
}
void large_m_release(sacq_layer*) {}
}  // namespace sacq
