// Self-test of the bounded device-side wait that every tcgen05 kernel of this library uses
// (ptx::mbar_wait_bounded): a one-CTA kernel waits on an mbarrier that expects one arrival.
// With `arrive` set a second thread makes that arrival and the wait succeeds; without it nobody
// ever arrives, the wait gives up after `limit_ns`, raises the CTA's abort flag and the kernel
// ORs VTLB_ST_GEMM_TIMEOUT into the status word exactly as the GEMM kernels' teardown does --
// so the path from a wait that ran out to VTLB_ETIMEOUT on the host can be exercised without a
// kernel that is actually stuck.  The kernel always returns; the context stays usable.
#include "common.cuh"
#include "ptx.cuh"

namespace {

__global__ void __launch_bounds__(64) wait_probe_kernel(uint64_t limit_ns, int arrive, uint32_t* status) {
  __shared__ __align__(8) uint64_t bar_storage;
  __shared__ uint32_t abort_word;
  const uint32_t bar = ptx::smem_u32(&bar_storage);
  volatile uint32_t* abort_flag = &abort_word;
  if (threadIdx.x == 0) {
    ptx::mbar_init(bar, 1);
    abort_word = 0;
    ptx::fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 32 && arrive) ptx::mbar_arrive(bar);
  if (threadIdx.x == 0) ptx::mbar_wait_bounded(bar, 0, abort_flag, limit_ns);  // raises abort_word on expiry
  __syncthreads();
  if (abort_word && threadIdx.x == 0) atomicOr(status, VTLB_ST_GEMM_TIMEOUT);
}

}  // namespace

VTLB_API int vtlb_wait_probe(vtlb_ctx* ctx, uint64_t limit_ns, int arrive) {
  VTLB_ENTER(ctx);
  if (limit_ns == 0 || limit_ns > 100000000ull)
    return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_wait_probe: the limit must be between 1 ns and 100 ms");
  wait_probe_kernel<<<1, 64, 0, ctx->stream>>>(limit_ns, arrive, ctx->d_status);
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}
