// Diagnostics of the library's own safety nets, callable through the C ABI.
#include "ttb_common.cuh"
#include "ttb_sm100.cuh"

using namespace ttb;
using namespace ttb::sm100;

namespace {

// One thread waits, with the given cycle limit, on an mbarrier that nothing ever arrives at. The wait must give up by
// itself: it returns false, raises the CTA's abort flag, and the kernel reports TTB_ERR_DEVICE_WAIT through the status
// word, exactly as the tensor-core kernels do when one of their waits runs out. Nothing faults and nothing spins on.
__global__ void wait_times_out_kernel(long long limit_cycles, int* status, int* observed) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    mbar_init_fence();
    const long long t0 = clock64();
    const bool completed = mbar_wait(smem_u32(&bar), 0, &abort_flag, limit_cycles);
    observed[0] = completed ? 1 : 0;
    observed[1] = abort_flag;
    observed[2] = (int)((clock64() - t0) >> 10);  // how long the wait lasted, in units of 1024 cycles
    if (abort_flag) atomicExch(status, (int)TTB_ERR_DEVICE_WAIT);
  }
}

}  // namespace

extern "C" int ttb_selftest_bounded_wait(ttb_ctx* ctx, int64_t limit_cycles, int32_t* observed_device) {
  if (!ctx) return TTB_ERR_INVALID;
  TTB_REQUIRE(ctx, limit_cycles > 0 && limit_cycles <= 100000000ll, "selftest_bounded_wait: the limit must be in (0, 1e8] cycles");
  TTB_REQUIRE(ctx, observed_device != nullptr, "selftest_bounded_wait: null pointer");
  DeviceGuard g(ctx->device);
  wait_times_out_kernel<<<1, 32, 0, ctx->stream>>>((long long)limit_cycles, ctx->d_status, observed_device);
  return launched(ctx, "selftest_bounded_wait");
}
