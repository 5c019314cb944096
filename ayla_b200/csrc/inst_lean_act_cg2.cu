// Row-major-output activation variants, a CTA pair per 256-row tile, compiled without the k-split
// epilogues: the kernels of launches that do not split k.
#include "kernel_registry.h"

namespace ayla_b200 {
void append_variants_lean_act_cg2(KernelEntry* out, int* count) {
  out[(*count)++] = make_entry<64, 2, EPI_PLAIN, false, true, true>();
  out[(*count)++] = make_entry<128, 2, EPI_PLAIN, false, true, true>();
  out[(*count)++] = make_entry<192, 2, EPI_PLAIN, false, true, true>();
  out[(*count)++] = make_entry<256, 2, EPI_PLAIN, false, true, true>();
  out[(*count)++] = make_entry<64, 2, EPI_BIAS, false, true, true>();
  out[(*count)++] = make_entry<128, 2, EPI_BIAS, false, true, true>();
  out[(*count)++] = make_entry<192, 2, EPI_BIAS, false, true, true>();
  out[(*count)++] = make_entry<256, 2, EPI_BIAS, false, true, true>();
}
}  // namespace ayla_b200
