// Self-test of the failure path that the tensor-core kernels share: every wait of theirs on an
// mbarrier is bounded; a wait that runs out records a code in the context's device status word
// and the kernel returns normally, and the next mb_stream_sync turns the word into
// MACE_RUNTIME_ERROR (the analogue of an error code travelling up through MACE_RETURN_IF_ERROR,
// include/mace/utils/logging.h:86-95).  In the product kernels the budget is about a second and
// nothing ever makes it run out; this kernel calls the SAME wait helper with a short budget on a
// barrier at which nobody ever arrives, so that the whole path -- helper, status word, host
// report, and a context that keeps working afterwards -- can be run.  It touches no TMA, no
// tensor memory and no other kernel's data, and it ends by itself after `budget_cycles`.
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace {

__global__ void __launch_bounds__(32) wait_timeout_selftest_kernel(long long budget_cycles, int *status,
                                                                  long long *waited_cycles) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    sm100::mbar_init(sm100::smem_u32(&bar), 1);
    abort_flag = 0;
    sm100::fence_barrier_init();
  }
  __syncwarp();
  if (threadIdx.x == 0) {
    const long long t0 = clock64();
    const bool ok = sm100::mbar_wait(sm100::smem_u32(&bar), 0, &abort_flag, budget_cycles);
    if (waited_cycles != nullptr) *waited_cycles = clock64() - t0;
    if (!ok) atomicCAS(status, 0, MB_DEV_TIMEOUT_PRODUCER);
  }
}

}  // namespace

extern "C" int mb_wait_timeout_selftest(mb_context *ctx, long long budget_cycles, long long *host_waited_cycles) {
  if (ctx == nullptr) return MB_INVALID_ARGS;
  if (budget_cycles < 1 || budget_cycles > (1ll << 31))
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_wait_timeout_selftest: budget must be 1 .. 2^31 cycles");
  if (ctx->capturing)
    return mb_fail(ctx, MB_RUNTIME_ERROR, "mb_wait_timeout_selftest: not inside a graph capture");
  MB_CUDA(ctx, cudaSetDevice(ctx->device));
  long long *cell = nullptr;
  if (host_waited_cycles != nullptr) MB_RETURN_IF_ERROR(mb_scratch(ctx, 8, reinterpret_cast<void **>(&cell)));
  wait_timeout_selftest_kernel<<<1, 32, 0, ctx->stream>>>(budget_cycles, ctx->dev_status, cell);
  MB_CUDA(ctx, cudaGetLastError());
  ctx->launches++;
  if (host_waited_cycles != nullptr) {
    MB_CUDA(ctx, cudaMemcpyAsync(host_waited_cycles, cell, 8, cudaMemcpyDeviceToHost, ctx->stream));
    MB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));  // the status word stays set for mb_stream_sync
  }
  return MB_SUCCESS;
}
