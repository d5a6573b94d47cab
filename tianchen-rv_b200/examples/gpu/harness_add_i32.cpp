// GPU harness for the i32 add slice: the inputs, size and check of the reference's worked
// example (examples/qemu/harness_add.cpp:15-33), against the same entry symbol.
#include "harness_common.h"

extern "C" void tcrv_emitc_explicit_selected_body_add_kernel_explicit_selected_body_rvv_i32_add(
    const int32_t *lhs, const int32_t *rhs, int32_t *out, size_t n);

int main() {
  const size_t n = 1031;
  std::vector<int32_t> lhs(n), rhs(n), out(n, 0);
  for (size_t i = 0; i < n; ++i) {
    lhs[i] = static_cast<int32_t>(i * 3 - 17);
    rhs[i] = static_cast<int32_t>(41 - static_cast<int32_t>(i * 2));
  }
  tcrv_emitc_explicit_selected_body_add_kernel_explicit_selected_body_rvv_i32_add(lhs.data(), rhs.data(), out.data(), n);
  for (size_t i = 0; i < n; ++i) {
    if (out[i] != lhs[i] + rhs[i]) {
      std::printf("mismatch at %zu: got %d expected %d\n", i, out[i], lhs[i] + rhs[i]);
      return 1;
    }
  }
  std::printf("add proof ok: %zu elements checked\n", n);
  return 0;
}
