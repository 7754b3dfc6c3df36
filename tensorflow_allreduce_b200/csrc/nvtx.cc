// NVTX ranges of the runtime (see NvtxRange in common.h). BC_NVTX=0 switches them off.
#include <nvtx3/nvToolsExt.h>

#include <cstdlib>
#include <cstring>

#include "common.h"

namespace bc {

namespace {
bool enabled() {
  static const bool on = [] {
    const char* v = getenv("BC_NVTX");
    const bool use = !(v && strcmp(v, "0") == 0);
    if (use) {
      // NVTX binds its entry points on first use; do that here, once, under the static
      // initialiser's lock, instead of from whichever threads call first.
      nvtxRangePushA("bcoll.init");
      nvtxRangePop();
    }
    return use;
  }();
  return on;
}
}  // namespace

NvtxRange::NvtxRange(const char* name) {
  if (enabled()) nvtxRangePushA(name);
}

NvtxRange::~NvtxRange() {
  if (enabled()) nvtxRangePop();
}

}  // namespace bc
