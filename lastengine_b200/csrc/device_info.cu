// What the host asks the device once (its SM count), and a self-test of the bounded wait that
// the tcgen05 kernels rest on.
#include "tc_common.cuh"

// SMs of the current device (0 when it cannot be asked).  Grid sizes and split counts that are
// chosen on the host for "a wave of blocks" take it from here.
LEB_API int leb_sm_count() {
  static int count[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (count[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    count[dev] = n;
  }
  return count[dev];
}

// One block waits, with the kernels' own bounded wait, on a barrier that nobody arrives on: the
// wait must run out after `limit` polls, the block must set the status word to `role` as the
// matrix products do and return.  Nothing here faults or spins without end; it shows that a
// wait that gives up leaves the context usable and is seen by the host.
__global__ void bounded_wait_selftest_kernel(int* __restrict__ status, uint32_t limit, int role) {
  __shared__ uint64_t bar;
  __shared__ int abort_word;
  volatile int* abort_flag = (volatile int*)&abort_word;
  if (threadIdx.x == 0) {
    abort_word = 0;
    mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (!mbar_wait_limit(&bar, 0, abort_flag, limit)) atomicExch(status, role);
  }
  __syncthreads();
  // the other threads see the flag as the other roles of a product would
  if (threadIdx.x == 32 && *abort_flag == 0) atomicExch(status, -role);
}

LEB_API int leb_selftest_bounded_wait(int* status, int limit, int role, cudaStream_t st) {
  LEB_REQUIRE(status != nullptr, "leb_selftest_bounded_wait: a status word is required");
  LEB_REQUIRE(limit > 0 && limit <= (1 << 16), "leb_selftest_bounded_wait: limit %d outside 1..65536 polls", limit);
  LEB_REQUIRE(role > 0, "leb_selftest_bounded_wait: the role written to the status word must be positive");
  bounded_wait_selftest_kernel<<<1, 64, 0, st>>>(status, (uint32_t)limit, role);
  LEB_CHECK_LAUNCH("leb_selftest_bounded_wait");
  return 0;
}
