// Row-major-output variants with the activation epilogue, one CTA per 128-row tile.
#include "kernel_registry.h"

namespace ayla_b200 {
void append_variants_act_cg1(KernelEntry* out, int* count) {
  out[(*count)++] = make_entry<64, 1, EPI_PLAIN, false, true>();
  out[(*count)++] = make_entry<128, 1, EPI_PLAIN, false, true>();
  out[(*count)++] = make_entry<192, 1, EPI_PLAIN, false, true>();
  out[(*count)++] = make_entry<256, 1, EPI_PLAIN, false, true>();
  out[(*count)++] = make_entry<64, 1, EPI_BIAS, false, true>();
  out[(*count)++] = make_entry<128, 1, EPI_BIAS, false, true>();
  out[(*count)++] = make_entry<192, 1, EPI_BIAS, false, true>();
  out[(*count)++] = make_entry<256, 1, EPI_BIAS, false, true>();
}
}  // namespace ayla_b200
