// Row-major-output variants with the activation epilogue, a CTA pair per 256-row tile.
#include "kernel_registry.h"

namespace ayla_b200 {
void append_variants_act_cg2(KernelEntry* out, int* count) {
  out[(*count)++] = make_entry<64, 2, EPI_PLAIN, false, true>();
  out[(*count)++] = make_entry<128, 2, EPI_PLAIN, false, true>();
  out[(*count)++] = make_entry<192, 2, EPI_PLAIN, false, true>();
  out[(*count)++] = make_entry<256, 2, EPI_PLAIN, false, true>();
  out[(*count)++] = make_entry<64, 2, EPI_BIAS, false, true>();
  out[(*count)++] = make_entry<128, 2, EPI_BIAS, false, true>();
  out[(*count)++] = make_entry<192, 2, EPI_BIAS, false, true>();
  out[(*count)++] = make_entry<256, 2, EPI_BIAS, false, true>();
}
}  // namespace ayla_b200
