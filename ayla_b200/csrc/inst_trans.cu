// Transposed-output variants for the swapped (small-M) form: the 128-row tile is
// filled with rows of bt, the narrow accumulator width covers M.
#include "kernel_registry.h"

namespace ayla_b200 {
void append_variants_trans(KernelEntry* out, int* count) {
  out[(*count)++] = make_entry<16, 1, EPI_PLAIN, true>();
  out[(*count)++] = make_entry<32, 1, EPI_PLAIN, true>();
  out[(*count)++] = make_entry<64, 1, EPI_PLAIN, true>();
  out[(*count)++] = make_entry<128, 1, EPI_PLAIN, true>();
  out[(*count)++] = make_entry<16, 1, EPI_BIAS, true>();
  out[(*count)++] = make_entry<32, 1, EPI_BIAS, true>();
  out[(*count)++] = make_entry<64, 1, EPI_BIAS, true>();
  out[(*count)++] = make_entry<128, 1, EPI_BIAS, true>();
}
}  // namespace ayla_b200
