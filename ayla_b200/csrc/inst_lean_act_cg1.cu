// Row-major-output activation variants, one CTA per 128-row tile, compiled without the k-split
// epilogues: the kernels of launches that do not split k.
#include "kernel_registry.h"

namespace ayla_b200 {
void append_variants_lean_act_cg1(KernelEntry* out, int* count) {
  out[(*count)++] = make_entry<64, 1, EPI_PLAIN, false, true, true>();
  out[(*count)++] = make_entry<128, 1, EPI_PLAIN, false, true, true>();
  out[(*count)++] = make_entry<192, 1, EPI_PLAIN, false, true, true>();
  out[(*count)++] = make_entry<256, 1, EPI_PLAIN, false, true, true>();
  out[(*count)++] = make_entry<64, 1, EPI_BIAS, false, true, true>();
  out[(*count)++] = make_entry<128, 1, EPI_BIAS, false, true, true>();
  out[(*count)++] = make_entry<192, 1, EPI_BIAS, false, true, true>();
  out[(*count)++] = make_entry<256, 1, EPI_BIAS, false, true, true>();
}
}  // namespace ayla_b200
