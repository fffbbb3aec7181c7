#include "b2_common.cuh"
#include "b2_launch.h"
namespace b2 {
unsigned int read_clear_status_flash() { return 0; }
int launch_flash_fwd(const void*, const void*, const void*, void*, int, int, int, const int64_t*,
                     const int64_t*, const int64_t*, float, cudaStream_t) {
  return fail(B2_NOT_WHITELISTED, "flash_fwd: not built yet");
}
}  // namespace b2
