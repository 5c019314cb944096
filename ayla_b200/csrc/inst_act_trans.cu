// Transposed-output (swapped, small-M) variants with the activation epilogue.
#include "kernel_registry.h"

namespace ayla_b200 {
void append_variants_act_trans(KernelEntry* out, int* count) {
  out[(*count)++] = make_entry<16, 1, EPI_PLAIN, true, true>();
  out[(*count)++] = make_entry<32, 1, EPI_PLAIN, true, true>();
  out[(*count)++] = make_entry<64, 1, EPI_PLAIN, true, true>();
  out[(*count)++] = make_entry<128, 1, EPI_PLAIN, true, true>();
  out[(*count)++] = make_entry<16, 1, EPI_BIAS, true, true>();
  out[(*count)++] = make_entry<32, 1, EPI_BIAS, true, true>();
  out[(*count)++] = make_entry<64, 1, EPI_BIAS, true, true>();
  out[(*count)++] = make_entry<128, 1, EPI_BIAS, true, true>();
}
}  // namespace ayla_b200
