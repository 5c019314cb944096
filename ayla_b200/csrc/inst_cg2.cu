// Row-major-output variants, a CTA pair per 256-row tile (tcgen05 cta_group::2).
#include "kernel_registry.h"

namespace ayla_b200 {
void append_variants_cg2(KernelEntry* out, int* count) {
  out[(*count)++] = make_entry<64, 2, EPI_PLAIN, false>();
  out[(*count)++] = make_entry<128, 2, EPI_PLAIN, false>();
  out[(*count)++] = make_entry<192, 2, EPI_PLAIN, false>();
  out[(*count)++] = make_entry<256, 2, EPI_PLAIN, false>();
  out[(*count)++] = make_entry<64, 2, EPI_BIAS, false>();
  out[(*count)++] = make_entry<128, 2, EPI_BIAS, false>();
  out[(*count)++] = make_entry<192, 2, EPI_BIAS, false>();
  out[(*count)++] = make_entry<256, 2, EPI_BIAS, false>();
}
}  // namespace ayla_b200
