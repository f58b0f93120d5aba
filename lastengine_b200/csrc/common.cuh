// Shared helpers of the sm_100a kernels: element types, warp reductions, error reporting.
//
// Every entry point is `extern "C"`, takes raw device pointers, sizes and a stream, launches
// asynchronously on that stream and returns 0, or returns non-zero after recording a message
// that leb_last_error() hands out.  Nothing here allocates device memory.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define LEB_API extern "C" __attribute__((visibility("default")))

// element type codes shared with the Python side
enum LebDtype { LEB_F32 = 0, LEB_BF16 = 1 };

int leb_fail(const char* fmt, ...);  // records the message, returns 1

// Kernels launched by this library since it was loaded (each check stands for one launch).
extern long long g_leb_launches;

#define LEB_CHECK_LAUNCH(name)                                                        \
  do {                                                                                \
    cudaError_t e_ = cudaGetLastError();                                              \
    if (e_ != cudaSuccess) return leb_fail("%s: %s", name, cudaGetErrorString(e_));   \
    g_leb_launches++;                                                                 \
  } while (0)

// Launch with programmatic dependent launch: the kernel may be scheduled while the one before
// it on the stream is still running, so its start-up (and whatever it does before pdl_wait())
// overlaps the tail of its predecessor.  A decode step is a chain of ~100 short kernels; this
// takes the launch gap out of every link.  Kernels launched this way call pdl_wait() before they
// touch anything the previous kernel wrote, and write nothing before it.
extern int g_leb_pdl;   // 1: use the attribute (default), 0: plain launches
template <typename... KArgs, typename... Args>
static inline cudaError_t leb_launch(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                     cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_leb_pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
// silu(g) * u.  The bfloat16 products' epilogues take 2^x and the reciprocal from the special
// function unit (relative error about 1e-6, far below the rounding of the bfloat16 they store):
// with exact expf and division an epilogue of a few warps is bound by its instructions.
template <typename T>
__device__ __forceinline__ float silu_mul(float g, float u) {
  if (sizeof(T) == 2) return __fdividef(g, 1.0f + __expf(-g)) * u;
  return g / (1.0f + expf(-g)) * u;
}
// Device side.  pdl_trigger(): the next kernel on the stream may be scheduled (once every block
// of this one has said so); it then runs its own start-up and waits in its pdl_wait() until this
// kernel has completed.  Said first thing, even before this kernel's own wait: a product two
// launches down the stream can then fetch its weights while the one before it still runs (its
// wait covers everything before it, since the kernel it waits for has itself waited).
// pdl_wait(): wait until the previous kernel has completed and its writes are visible (a no-op
// for a plain launch).
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() {
  pdl_trigger();
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

#define LEB_REQUIRE(cond, ...)                 \
  do {                                         \
    if (!(cond)) return leb_fail(__VA_ARGS__); \
  } while (0)

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `red` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // `red` may still be read from an earlier call
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nw ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// SMs of the current device, asked once per device (device_info.cu); launch shapes that are
// chosen for "a wave of blocks" use it.
extern "C" int leb_sm_count();
static inline int sm_count() {
  int n = leb_sm_count();
  return n > 0 ? n : 1;
}
