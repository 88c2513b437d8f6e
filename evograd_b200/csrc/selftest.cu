// Self-test of the bounded-wait protocol every kernel with an mbarrier uses.
//
// One small block waits, through the same `mbar_wait` helper as the product
// kernels, for a barrier phase that nothing will ever complete. The wait gives
// up after `limit_cycles`, records its identity in the block's abort word and
// in the sticky device status, and the kernel returns normally: the context
// stays usable and the host reads EVG_ETIMEOUT from evg_device_status().
// Nothing faults, traps or spins without a bound.
#include "evg_common.cuh"
#include "sm100_umma.cuh"

namespace evg {
namespace {

__device__ int g_selftest_status = 0;
constexpr int kSelftestWaitId = 901;
constexpr long long kMaxSelftestCycles = 400000000ll;  // about 0.2 s at 2 GHz

__global__ void __launch_bounds__(64) bounded_wait_selftest_kernel(long long limit_cycles,
                                                                   int* observed) {
  using namespace umma;
  __shared__ uint64_t never;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&never, 1);
    fence_mbar_init();
  }
  __syncthreads();
  const WaitCtx ctx{&abort_flag, &g_selftest_status, limit_cycles};
  mbar_wait(&never, 0, ctx, kSelftestWaitId);  // no thread arrives on `never`
  __syncthreads();
  // Later waits of an aborted block fall through at once.
  mbar_wait(&never, 0, ctx, kSelftestWaitId + 1);
  if (threadIdx.x == 0 && observed) *observed = abort_flag;
}

int read_selftest_status(int reset) {
  int code = 0;
  if (cudaMemcpyFromSymbol(&code, g_selftest_status, sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  if (reset && code != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_selftest_status, &zero, sizeof(int));
  }
  return code;
}
const bool g_selftest_registered = (register_device_status(read_selftest_status), true);

}  // namespace
}  // namespace evg

using namespace evg;

extern "C" int evg_selftest_bounded_wait(int64_t limit_cycles, int* observed_abort_word,
                                         void* stream) {
  if (limit_cycles <= 0 || limit_cycles > kMaxSelftestCycles)
    return fail(EVG_EBADSHAPE, "selftest_bounded_wait: limit_cycles must be in (0, %lld]",
                kMaxSelftestCycles);
  bounded_wait_selftest_kernel<<<1, 64, 0, (cudaStream_t)stream>>>((long long)limit_cycles,
                                                                   observed_abort_word);
  return check_launch("selftest_bounded_wait");
}
