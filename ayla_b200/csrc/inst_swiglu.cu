// Fused SwiGLU variants: gate and up weights share one stream of x.
#include "kernel_registry.h"

namespace ayla_b200 {
void append_variants_swiglu(KernelEntry* out, int* count) {
  out[(*count)++] = make_entry<256, 1, EPI_SWIGLU, false>();
  out[(*count)++] = make_entry<256, 2, EPI_SWIGLU, false>();
}
}  // namespace ayla_b200
