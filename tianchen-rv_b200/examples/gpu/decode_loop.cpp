// The decode step as a C++ application runs it: the layers of a step called one after the other
// through the host-pointer entry points (activations and results in the caller's host buffers,
// weights registered beforehand), either one blocking call per layer or queued calls and one
// tcrv_cuda_host_sync() per step.  Built as a small shared library so that a benchmark written
// in another language can time the loop without its own per-call overhead in the timed region:
// the callee is the C ABI of include/tcrv_emitc_host.h and nothing else.
#include <chrono>
#include <cstddef>
#include <cstdint>

#include "tcrv_emitc_host.h"

extern "C" {

// One layer: the arguments of tcrv_cuda_host_gemm_q4_0_q8_0 in ABI order.
struct tcrv_decode_call {
  size_t n;
  float *s;
  const uint8_t *vx;
  const uint8_t *vy;
  size_t by, nr, nc, bx, bs;
};

// Runs `steps` decode steps of `ncalls` layers each and writes the elapsed wall time to
// *seconds.  queued != 0: the `_async` twins and one sync per step; else one blocking call per
// layer.  Returns the first non-zero status of an entry, 0 otherwise.
int tcrv_decode_loop_run(const tcrv_decode_call *calls, int ncalls, int steps, int queued, double *seconds) {
  const auto t0 = std::chrono::steady_clock::now();
  for (int step = 0; step < steps; ++step) {
    for (int i = 0; i < ncalls; ++i) {
      const tcrv_decode_call &c = calls[i];
      const int st = queued ? tcrv_cuda_host_gemm_q4_0_q8_0_async(c.n, c.s, c.vx, c.vy, c.by, c.nr, c.nc, c.bx, c.bs)
                            : tcrv_cuda_host_gemm_q4_0_q8_0(c.n, c.s, c.vx, c.vy, c.by, c.nr, c.nc, c.bx, c.bs);
      if (st != 0)
        return st;
    }
    if (queued) {
      const int st = tcrv_cuda_host_sync();
      if (st != 0)
        return st;
    }
  }
  *seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
  return 0;
}

}  // extern "C"
