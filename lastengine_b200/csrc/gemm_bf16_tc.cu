// bfloat16 matrix product on the 5th-generation tensor cores (tcgen05) for prompts:
//   C[M,N] (+)= A[M,K] . W[N,K]^T, float accumulation in tensor memory.
//
// The reference multiplies prompt chunks with tiled mma.sync kernels over weights it
// dequantises into shared memory (src/cuda/kernels.cu:965-1235, tiles 64x64 to 128x128).  Here
// a block works through 128 x BN tiles (one block per SM, tiles dealt out round-robin):
//   warps 0, 6  one thread each issues the TMA loads (cp.async.bulk.tensor, 128-byte swizzle) of the
//            A tiles (warp 0) and the W tiles (warp 6) of 64 k-values into a ring of shared-memory
//            stages; issuing a TMA load costs its thread some hundred cycles, so two threads
//            keep the ring fuller than one;
//   warp 1   allocates tensor memory; one thread issues tcgen05.mma (128 x BN x 16 per
//            instruction, operands from shared memory through descriptors, accumulator in tensor
//            memory) and commits each stage back to the producer;
//   warps 2-5  wait for the accumulator, read it with tcgen05.ld (32 rows per warp, 32 columns at
//            a time) and apply the epilogue: store, add into the float residual, or SwiGLU over
//            gate/up rows interleaved in blocks of 16.
// Tensor memory holds two accumulators, so the epilogue of one tile runs while the products of
// the next are issued.
// Rows and columns beyond M, N and K are zero-filled by TMA and masked in the epilogue, so any
// M, N and any K that is a multiple of 8 are taken.
//
// Every wait on an mbarrier is bounded: when a wait gives up, the block records where in
// *status, every role leaves its loop, tensor memory is freed, and the block returns.
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

#define TC_BM 128
#define TC_BK 64
#define TC_THREADS 224
#define TC_SPIN_LIMIT (1u << 22)

// ---- PTX wrappers ---------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false when it gave up (and *abort is set so that the other roles leave too).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < TC_SPIN_LIMIT; i++) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (i > 4096) __nanosleep(64);
  }
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols));
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols));
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile with rows of 128 bytes under the 128-byte
// swizzle: start address / 16; leading offset 1 (unused with a swizzle); stride between groups
// of 8 rows 1024 bytes; descriptor version 1 (bit 46); layout type 2 = 128-byte swizzle.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
  uint64_t d = (uint64_t)((saddr & 0x3FFFF) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

template <typename TC, int BN, int STAGES>
__global__ void __launch_bounds__(TC_THREADS)
gemm_bf16_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    TC* __restrict__ C, int M, int N, int K, int ldc, int epilogue, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment for the swizzled tiles
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  constexpr int A_BYTES = TC_BM * TC_BK * 2, B_BYTES = BN * TC_BK * 2;
  uint8_t* sa = smem;
  uint8_t* sb = smem + STAGES * A_BYTES;
  uint64_t* full = (uint64_t*)(sb + STAGES * B_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;      // [2]
  uint64_t* acc_empty = acc_full + 2;       // [2]
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  float* stage_out = (float*)(tmem_slot + 4);   // 4 warps x 32 rows x 36 floats for the epilogue

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nk = (K + TC_BK - 1) / TC_BK;
  const int m_tiles = (M + TC_BM - 1) / TC_BM, n_tiles = (N + BN - 1) / BN;
  const int num_tiles = m_tiles * n_tiles;   // tile t: rows (t % m_tiles), columns (t / m_tiles):
                                             // blocks running together share weight tiles in L2

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) {
      mbar_init(&full[s], 2);    // the two producers each announce their bytes
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; i++) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 4);   // one arrival per epilogue warp
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * BN);   // two accumulators of BN columns x 128 lanes x 32 bits
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_acc = *tmem_slot;

  if (warp == 0 || warp == 6) {
    if (lane == 0) {
      const bool loads_a = warp == 0;
      uint32_t it = 0;   // k-slices loaded so far, over all tiles of this block
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % m_tiles) * TC_BM, n0 = (tile / m_tiles) * BN;
        for (int kb = 0; kb < nk; kb++, it++) {
          const int s = it % STAGES;
          if (!mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1, abort_flag)) { atomicExch(status, 1); ok = false; break; }
          mbar_expect_tx(&full[s], loads_a ? A_BYTES : B_BYTES);
          // Tiles that share rows of A start their walk over k at different places, so that
          // blocks running in step do not all ask L2 for the same lines at the same moment.
          const int kk = (kb + (tile / m_tiles) * 5) % nk;
          if (loads_a) tma_load_2d(sa + s * A_BYTES, &map_a, &full[s], kk * TC_BK, m0);
          else tma_load_2d(sb + s * B_BYTES, &map_w, &full[s], kk * TC_BK, n0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // instruction descriptor: float accumulator, bfloat16 A and B, both K-major, N, M
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
      bool ok = true;
      uint32_t it = 0, t = 0;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, t++) {
        const uint32_t buf = t & 1;
        // the epilogue must have emptied this accumulator (two tiles ago)
        if (!mbar_wait(&acc_empty[buf], ((t >> 1) & 1) ^ 1, abort_flag)) { atomicExch(status, 4); ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_acc + buf * BN;
        for (int kb = 0; kb < nk; kb++, it++) {
          const int s = it % STAGES;
          if (!mbar_wait(&full[s], (it / STAGES) & 1, abort_flag)) { atomicExch(status, 2); ok = false; break; }
          tc_fence_after();
          const uint64_t da = make_desc(smem_u32(sa + s * A_BYTES));
          const uint64_t db = make_desc(smem_u32(sb + s * B_BYTES));
#pragma unroll
          for (int k = 0; k < TC_BK / 16; k++)   // 16 k-values = 32 bytes along the swizzled row
            umma_bf16(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb | k) != 0);
          umma_commit(&empty[s]);   // the stage is free once these products have read it
        }
        if (ok) umma_commit(&acc_full[buf]);
      }
    }
  } else {
    // epilogue warps: tensor-memory lanes 32*(warp%4) .. +31 are rows of the tile
    const int quad = warp & 3;
    // Each warp stages its 32 rows of a 32-column piece in shared memory (the pipeline's first
    // stage, free once the accumulator is complete) and writes them out row by row, so that a
    // store covers whole 128-byte lines instead of one element in each of 32 rows.
    float* stg = stage_out + quad * (32 * 36);
    uint32_t t = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, t++) {
    const int m0 = (tile % m_tiles) * TC_BM, n0 = (tile / m_tiles) * BN;
    const uint32_t buf = t & 1;
    const int row_base = m0 + quad * 32;
    bool ok = mbar_wait(&acc_full[buf], (t >> 1) & 1, abort_flag);
    if (!ok && lane == 0) atomicExch(status, 3);
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;   // the warp leaves together
    if (!ok) break;
    tc_fence_after();
    {
      const int ncols = epilogue == 2 ? 16 : 32;          // output columns per piece
      const int n_out = epilogue == 2 ? N / 2 : N;
      const int lpr = ncols / 4, rpp = 32 / lpr;          // lanes per row, rows per pass
      const int lr = lane / lpr, lc = (lane % lpr) * 4;
      const bool vec = (ldc % 4 == 0) && (((uintptr_t)C % 16) == 0);
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t v[32];
        tmem_ld32(tmem_acc + ((uint32_t)(quad * 32) << 16) + buf * BN + (uint32_t)c0, v);
        tmem_ld_wait();
        float* mine = stg + lane * 36;
        if (epilogue == 2) {
          // columns c0..c0+15 gate, c0+16..c0+31 up of outputs (n0 + c0)/2 + i
#pragma unroll
          for (int i = 0; i < 16; i += 4) {
            float4 f;
            float* fp = reinterpret_cast<float*>(&f);
#pragma unroll
            for (int e = 0; e < 4; e++) {
              const float g = __uint_as_float(v[i + e]), u = __uint_as_float(v[16 + i + e]);
              fp[e] = g / (1.0f + expf(-g)) * u;
            }
            *reinterpret_cast<float4*>(mine + i) = f;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            *reinterpret_cast<float4*>(mine + i) = make_float4(__uint_as_float(v[i]), __uint_as_float(v[i + 1]),
                                                                __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
        }
        __syncwarp();
        const int col = (epilogue == 2 ? ((n0 + c0) >> 1) : (n0 + c0)) + lc;
        if (epilogue == 1 && sizeof(TC) == 4 && vec && col + 3 < n_out) {
          // adding into the residual: fetch all eight old pieces first, then add and store, so
          // the eight loads are in flight together instead of one round trip per row
          float4 old[8];
#pragma unroll
          for (int it = 0; it < 8; it++) {
            const int row = row_base + lr + 4 * it;
            old[it] = row < M ? __ldcs(reinterpret_cast<const float4*>(C + (size_t)row * ldc + col))
                              : make_float4(0.f, 0.f, 0.f, 0.f);
          }
#pragma unroll
          for (int it = 0; it < 8; it++) {
            const int rr = lr + 4 * it, row = row_base + rr;
            if (row >= M) continue;
            const float4 f = *reinterpret_cast<const float4*>(stg + rr * 36 + lc);
            *reinterpret_cast<float4*>(C + (size_t)row * ldc + col) =
                make_float4(f.x + old[it].x, f.y + old[it].y, f.z + old[it].z, f.w + old[it].w);
          }
          __syncwarp();
          continue;
        }
        for (int rr = lr; rr < 32; rr += rpp) {
          const int row = row_base + rr;
          if (row >= M || col >= n_out) continue;
          float4 f = *reinterpret_cast<const float4*>(stg + rr * 36 + lc);
          TC* o = C + (size_t)row * ldc + col;
          if (vec && col + 3 < n_out) {
            if (sizeof(TC) == 4) {
              float4* o4 = reinterpret_cast<float4*>(o);
              if (epilogue == 1) {
                const float4 old = *o4;
                f.x += old.x; f.y += old.y; f.z += old.z; f.w += old.w;
              }
              *o4 = f;
            } else {
              __nv_bfloat162 lo = __floats2bfloat162_rn(f.x, f.y), hi = __floats2bfloat162_rn(f.z, f.w);
              uint2 pk = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
              *reinterpret_cast<uint2*>(o) = pk;
            }
          } else {
            const float* fp = reinterpret_cast<const float*>(&f);
            for (int e = 0; e < 4 && col + e < n_out; e++) {
              float a = fp[e];
              if (epilogue == 1) a += to_f32(o[e]);
              o[e] = from_f32<TC>(a);
            }
          }
        }
        __syncwarp();
      }
    }
    // this warp has read its part of the accumulator: hand the buffer back to the issuing thread
    tc_fence_before();
    __syncwarp();
    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&acc_empty[buf])) : "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_acc, 2 * BN);
  }
}

// ---- host side -------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  });
  return fn;
}

struct MapKey {
  const void* ptr;
  int rows, cols, ld, box_rows;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = std::hash<const void*>()(k.ptr);
    for (int v : {k.rows, k.cols, k.ld, k.box_rows}) h = h * 1000003u ^ std::hash<int>()(v);
    return h;
  }
};

// A [rows, cols] bfloat16 matrix with row stride ld (elements), read in boxes of box_rows x 64
// under the 128-byte swizzle; out-of-range elements read as zero.
static int tensor_map(CUtensorMap* out, const void* ptr, int rows, int cols, int ld, int box_rows) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  static std::mutex mu;
  MapKey key{ptr, rows, cols, ld, box_rows};
  std::lock_guard<std::mutex> g(mu);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return 0;
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return leb_fail("leb_gemm_bf16_tc: the driver has no cuTensorMapEncodeTiled");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return leb_fail("leb_gemm_bf16_tc: cuTensorMapEncodeTiled failed (%d) for [%d,%d] ld %d", (int)r, rows, cols, ld);
  if (cache.size() > 4096) cache.clear();
  cache[key] = *out;
  return 0;
}

template <typename TC, int BN, int STAGES>
static int launch_tc(void* C, const CUtensorMap& ma, const CUtensorMap& mw, int M, int N, int K, int ldc,
                     int epilogue, int* status, cudaStream_t st) {
  constexpr size_t smem = (size_t)STAGES * (TC_BM * TC_BK * 2 + BN * TC_BK * 2) + (2 * STAGES + 4) * 8 + 16 +
                          4 * 32 * 36 * 4 + 1024;
  auto kern = gemm_bf16_tc_kernel<TC, BN, STAGES>;
  static bool set = false;
  if (!set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return leb_fail("leb_gemm_bf16_tc: shared memory %zu: %s", smem, cudaGetErrorString(e));
    set = true;
  }
  static int n_sm = 0;
  if (!n_sm) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sm <= 0) n_sm = 148;
  }
  const long tiles = (long)ceil_div(N, BN) * ceil_div(M, TC_BM);
  dim3 grid((unsigned)(tiles < n_sm ? tiles : n_sm));
  kern<<<grid, TC_THREADS, smem, st>>>(ma, mw, (TC*)C, M, N, K, ldc, epilogue, status);
  LEB_CHECK_LAUNCH("leb_gemm_bf16_tc");
  return 0;
}

// Returns 1 when the operands can go through TMA (16-byte aligned bases and row strides).
LEB_API int leb_gemm_bf16_tc_supported(const void* A, const void* W, int K, int lda) {
  return K > 0 && K % 8 == 0 && lda % 8 == 0 && ((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0;
}

// epilogue: 0 store, 1 add into float C, 2 SwiGLU over 16/16 interleaved gate/up rows (C has N/2 columns).
// status: device int, set non-zero by a block whose bounded wait gave up.
LEB_API int leb_gemm_bf16_tc(void* C, int c_dtype, const void* A, const void* W, int M, int N, int K, int lda,
                             int ldc, int epilogue, int* status, cudaStream_t st) {
  if (M <= 0 || N <= 0) return 0;
  LEB_REQUIRE(leb_gemm_bf16_tc_supported(A, W, K, lda), "leb_gemm_bf16_tc: operands not aligned for TMA (K %d, lda %d)", K, lda);
  LEB_REQUIRE(epilogue >= 0 && epilogue <= 2, "leb_gemm_bf16_tc: unknown epilogue %d", epilogue);
  LEB_REQUIRE(epilogue != 1 || c_dtype == LEB_F32, "leb_gemm_bf16_tc: adding needs a float C");
  LEB_REQUIRE(epilogue != 2 || N % 32 == 0, "leb_gemm_bf16_tc: the SwiGLU epilogue needs N (%d) to be a multiple of 32", N);
  LEB_REQUIRE(status != nullptr, "leb_gemm_bf16_tc: a status word is required");
  // wide tiles read less per flop; narrow ones spread a small product over more SMs
  // With few rows (a decode step of some dozens of sequences) the product is bound by reading W:
  // narrow tiles then give every SM a stripe of W to stream.
  const long m_tiles = ceil_div(M, TC_BM);
  int BN = 32;
  if (N > 128 && m_tiles * ceil_div(N, 256) >= 64) BN = 256;
  else if (m_tiles * ceil_div(N, 128) >= 96) BN = 128;
  else if (m_tiles * ceil_div(N, 64) >= 96) BN = 64;
  CUtensorMap ma, mw;
  if (tensor_map(&ma, A, M, K, lda, TC_BM)) return 1;
  if (tensor_map(&mw, W, N, K, K, BN)) return 1;
  if (c_dtype == LEB_BF16) {
    if (BN == 256) return launch_tc<bf16, 256, 4>(C, ma, mw, M, N, K, ldc, epilogue, status, st);
    if (BN == 128) return launch_tc<bf16, 128, 6>(C, ma, mw, M, N, K, ldc, epilogue, status, st);
    if (BN == 64) return launch_tc<bf16, 64, 8>(C, ma, mw, M, N, K, ldc, epilogue, status, st);
    return launch_tc<bf16, 32, 8>(C, ma, mw, M, N, K, ldc, epilogue, status, st);
  }
  if (c_dtype == LEB_F32) {
    if (BN == 256) return launch_tc<float, 256, 4>(C, ma, mw, M, N, K, ldc, epilogue, status, st);
    if (BN == 128) return launch_tc<float, 128, 6>(C, ma, mw, M, N, K, ldc, epilogue, status, st);
    if (BN == 64) return launch_tc<float, 64, 8>(C, ma, mw, M, N, K, ldc, epilogue, status, st);
    return launch_tc<float, 32, 8>(C, ma, mw, M, N, K, ldc, epilogue, status, st);
  }
  return leb_fail("leb_gemm_bf16_tc: unknown C dtype %d", c_dtype);
}
