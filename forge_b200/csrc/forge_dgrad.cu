// dX = dY W.  Placeholder entry until the tcgen05 kernel lands.
#include "forge_host.h"

using namespace forge;

extern "C" int forge_dgrad(const void* dY, const void* W, void* dX, int64_t BT, int64_t V, int64_t H,
                           int64_t ld_dy, int64_t ld_w, int64_t ld_dx, int32_t* status, void* cuda_stream) {
  (void)dY; (void)W; (void)dX; (void)BT; (void)V; (void)H; (void)ld_dy; (void)ld_w; (void)ld_dx;
  (void)status; (void)cuda_stream;
  return fail(FORGE_ERR_UNSUPPORTED, "forge_dgrad is not built yet");
}
