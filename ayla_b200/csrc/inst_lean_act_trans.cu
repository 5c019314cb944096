// Transposed-output activation variants of the swapped (small-M) form, compiled without the k-split
// epilogues: the kernels of launches that do not split k.
#include "kernel_registry.h"

namespace ayla_b200 {
void append_variants_lean_act_trans(KernelEntry* out, int* count) {
  out[(*count)++] = make_entry<16, 1, EPI_PLAIN, true, true, true>();
  out[(*count)++] = make_entry<32, 1, EPI_PLAIN, true, true, true>();
  out[(*count)++] = make_entry<64, 1, EPI_PLAIN, true, true, true>();
  out[(*count)++] = make_entry<128, 1, EPI_PLAIN, true, true, true>();
  out[(*count)++] = make_entry<16, 1, EPI_BIAS, true, true, true>();
  out[(*count)++] = make_entry<32, 1, EPI_BIAS, true, true, true>();
  out[(*count)++] = make_entry<64, 1, EPI_BIAS, true, true, true>();
  out[(*count)++] = make_entry<128, 1, EPI_BIAS, true, true, true>();
}
}  // namespace ayla_b200
