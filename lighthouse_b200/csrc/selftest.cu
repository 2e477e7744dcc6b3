// A wait that is allowed to run out: evidence that the bounded waits of the kernels give up
// the way they are meant to, produced without any fault. One block waits on an mbarrier in
// its own shared memory that nothing arrives on, and on a flag in this GPU's own global memory
// that nothing writes, through the same helpers (ptx.cuh) the GEMM / attention kernels and
// the cross-rank collective use, with a caller-chosen short limit. On expiry the helpers raise
// the block's abort flag and write a code into the context's status word; the kernel then
// returns normally, lh_b200_sync reports LH_ERR_DEVICE once, and the context stays usable.
#include "common.cuh"
#include "ptx.cuh"

namespace lh {
namespace {

__global__ void __launch_bounds__(64) bounded_wait_selftest_kernel(const uint32_t* flag, uint64_t limit_ns, int* dev_status, int* outcome) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  bool ok;
  if (threadIdx.x < 32) ok = mbar_wait_limit(&bar, 0, &abort_flag, dev_status, DEV_TIMEOUT_SELFTEST, limit_ns);
  else ok = flag_wait_limit(flag, 1u, &abort_flag, dev_status, DEV_TIMEOUT_SELFTEST, limit_ns);
  const int gave_up = __syncthreads_count(ok ? 0 : 1);
  if (threadIdx.x == 0) *outcome = gave_up;  // how many of the 64 waits returned "timed out"
}

}  // namespace
}  // namespace lh

using namespace lh;

extern "C" int lh_b200_selftest_bounded_wait(lh_ctx_t* ctx, uint64_t limit_ns, int* timed_out_waits) {
  if (!ctx) return LH_ERR_INVALID;
  if (limit_ns == 0 || limit_ns > 100000000ull)
    return set_error(ctx, LH_ERR_INVALID, "selftest_bounded_wait: limit must be in (0, 100 ms], got %llu ns", (unsigned long long)limit_ns);
  // two words of device memory for the duration of the call: the flag nobody sets, the outcome
  int* words = nullptr;
  LH_CUDA_CHECK(ctx, cudaMalloc(&words, 2 * sizeof(int)));
  cudaError_t e = cudaMemsetAsync(words, 0, 2 * sizeof(int), ctx->stream);
  if (e == cudaSuccess) {
    bounded_wait_selftest_kernel<<<1, 64, 0, ctx->stream>>>(reinterpret_cast<const uint32_t*>(words), limit_ns, ctx->dev_status, words + 1);
    e = cudaGetLastError();
  }
  int outcome = -1;
  if (e == cudaSuccess) e = cudaMemcpyAsync(&outcome, words + 1, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
  cudaFree(words);
  LH_CUDA_CHECK(ctx, e);
  ctx->launches++;
  if (timed_out_waits) *timed_out_waits = outcome;
  return LH_OK;  // the status word now holds DEV_TIMEOUT_SELFTEST: the next lh_b200_sync reports it
}
