// bfloat16 matrix product for prompts on pairs of SMs (tcgen05 with cta_group::2):
//   C[M,N] (+)= A[M,K] . W[N,K]^T, float accumulation in tensor memory.
//
// The one-SM kernel (gemm_bf16_tc.cu) is bound by what a single SM can pull out of L2: a 128 x 256
// tile needs 48 KB of operands for every 64 values of k.  Here two blocks on neighbouring SMs
// (a cluster of 2) share a 256 x 256 tile: block r loads rows [128 r, 128 r + 128) of the A tile
// and rows [128 r, 128 r + 128) of the W tile, 32 KB per block and k-step, and ONE thread of the
// pair's first block issues tcgen05.mma.cta_group::2, which reads both blocks' shared memory and
// leaves rows [128 r, ..) x 256 columns of the result in block r's tensor memory.  Per flop each
// SM fetches a third less than before.
//
// Roles per block: warp 0 one thread issues the TMA loads (its A half and its W half of every
// stage; the bytes of both blocks are counted on the first block's barrier); warp 1 allocates
// tensor memory (both blocks ask, with cta_group::2; they get the same address) and, in the first
// block only, one thread issues the MMAs and commits them to both blocks' barriers
// (tcgen05.commit with multicast); warps 2-5 read the block's accumulator rows and apply the
// epilogue (store, add into the float residual, SwiGLU over gate/up rows interleaved in blocks
// of 16), then tell the first block that the accumulator is free.  Two accumulators (all 512
// columns), so the epilogue of one tile runs under the products of the next.
//
// Every wait on an mbarrier is bounded; a wait that gives up sets the status word and every role
// leaves its loop.  Both blocks always meet at a cluster barrier before they free tensor memory
// and return, so neither leaves while the other may still read its shared memory.
#include "tc_common.cuh"

#define T2_THREADS 192
#define T2_STAGES 6
#define T2_BN 256

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t smem_addr, uint32_t rank) {   // the same place in another block
  uint32_t a;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(smem_addr), "r"(rank));
  return a;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// TMA load whose bytes are counted on a barrier that may lie in the pair's other block
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void umma2_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrives, once the MMAs issued so far are complete, on the barrier at this address in both blocks
__device__ __forceinline__ void umma2_commit_both(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}

template <typename TC>
__global__ void __launch_bounds__(T2_THREADS)
gemm_bf16_tc2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                     TC* __restrict__ C, int M, int N, int K, int ldc, int epilogue, int* __restrict__ status) {
  constexpr int BN = T2_BN, STAGES = T2_STAGES;
  constexpr int A_BYTES = 128 * TC_BK * 2, B_BYTES = 128 * TC_BK * 2;   // this block's halves
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sa = smem;
  uint8_t* sb = smem + STAGES * A_BYTES;
  uint64_t* full = (uint64_t*)(sb + STAGES * B_BYTES);   // used in the first block
  uint64_t* empty = full + STAGES;                       // one set per block
  uint64_t* acc_full = empty + STAGES;                   // [2], one set per block
  uint64_t* acc_empty = acc_full + 2;                    // [2], used in the first block
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  float* stage_out = (float*)(tmem_slot + 4);            // 4 warps x 32 rows x 36 floats for the epilogue

  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();                  // 0: the block that issues the MMAs
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int nk = (K + TC_BK - 1) / TC_BK;
  const int m_tiles = (M + 255) / 256, n_tiles = (N + BN - 1) / BN;
  const int num_tiles = m_tiles * n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) {
      mbar_init(&full[s], 1);     // the first block's producer announces the bytes of both blocks
      mbar_init(&empty[s], 1);    // the multicast commit
    }
    for (int i = 0; i < 2; i++) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 8);   // four epilogue warps in each of the two blocks
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();     // both blocks' barriers exist before anything is sent to them
  tc_fence_after();
  const uint32_t tmem_acc = *tmem_slot;
  pdl_wait();

  if (warp == 0) {
    if (lane == 0) {
      const uint32_t full0 = map_to_rank(smem_u32(&full[0]), 0);   // the first block's barriers, as seen from here
      uint32_t it = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += n_pairs) {
        const int nt = tile / m_tiles;
        const int m0 = (tile % m_tiles) * 256 + 128 * (int)rank, n0 = nt * BN + 128 * (int)rank;
        for (int kb = 0; kb < nk; kb++, it++) {
          const int s = it % STAGES;
          if (!mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1, abort_flag)) { atomicExch(status, 21); ok = false; break; }
          if (rank == 0) mbar_expect_tx(&full[s], 2 * (A_BYTES + B_BYTES));
          const int kk = (kb + nt * 5) % nk;   // tiles that share rows of A start at different k
          tma_load_2d_pair(sa + s * A_BYTES, &map_a, full0 + s * 8, kk * TC_BK, m0);
          tma_load_2d_pair(sb + s * B_BYTES, &map_w, full0 + s * 8, kk * TC_BK, n0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      // float accumulator, bfloat16 A and B, both K-major, N = 256, M = 256 over the pair
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
      bool ok = true;
      uint32_t it = 0, t = 0;
      for (int tile = pair; tile < num_tiles && ok; tile += n_pairs, t++) {
        const uint32_t buf = t & 1;
        if (!mbar_wait(&acc_empty[buf], ((t >> 1) & 1) ^ 1, abort_flag)) { atomicExch(status, 24); ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_acc + buf * BN;
        for (int kb = 0; kb < nk; kb++, it++) {
          const int s = it % STAGES;
          if (!mbar_wait(&full[s], (it / STAGES) & 1, abort_flag)) { atomicExch(status, 22); ok = false; break; }
          tc_fence_after();
          const uint64_t da = make_desc(smem_u32(sa + s * A_BYTES));
          const uint64_t db = make_desc(smem_u32(sb + s * B_BYTES));
#pragma unroll
          for (int k = 0; k < TC_BK / 16; k++)
            umma2_bf16(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb | k) != 0);
          umma2_commit_both(&empty[s]);
        }
        if (ok) umma2_commit_both(&acc_full[buf]);
      }
    }
  } else {
    const int quad = warp & 3;
    float* stg = stage_out + quad * (32 * 36);
    const uint32_t acc_empty0 = map_to_rank(smem_u32(&acc_empty[0]), 0);
    uint32_t t = 0;
    for (int tile = pair; tile < num_tiles; tile += n_pairs, t++) {
      const int m0 = (tile % m_tiles) * 256 + 128 * (int)rank, n0 = (tile / m_tiles) * BN;
      const uint32_t buf = t & 1;
      const int row_base = m0 + quad * 32;
      // adding epilogue with 16-byte rows: a lane's eight old values (rows lane/8 + 4j, four columns
      // from (lane%8)*4) of a 32-column piece; the first piece's are on their way while the products run
      float4 nxt[8];
      auto load_old = [&](int c0) {
        const int col = n0 + c0 + (lane & 7) * 4;
#pragma unroll
        for (int j = 0; j < 8; j++) {
          const int row = row_base + (lane >> 3) + 4 * j;
          nxt[j] = (row < M && col + 3 < N) ? __ldcs(reinterpret_cast<const float4*>(C + (size_t)row * ldc + col))
                                            : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      };
      if (epilogue == 1 && sizeof(TC) == 4 && (ldc % 4 == 0) && (((uintptr_t)C % 16) == 0)) load_old(0);
      bool ok = mbar_wait(&acc_full[buf], (t >> 1) & 1, abort_flag);
      if (!ok && lane == 0) atomicExch(status, 23);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      tc_fence_after();
      {
        const int ncols = epilogue == 2 ? 16 : 32;
        const int n_out = epilogue == 2 ? N / 2 : N;
        const int lpr = ncols / 4, rpp = 32 / lpr;
        const int lr = lane / lpr, lc = (lane % lpr) * 4;
        const bool vec = (ldc % 4 == 0) && (((uintptr_t)C % 16) == 0);
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t v[32];
          tmem_ld32(tmem_acc + ((uint32_t)(quad * 32) << 16) + buf * BN + (uint32_t)c0, v);
          tmem_ld_wait();
          float* mine = stg + lane * 36;
          if (epilogue == 2) {
#pragma unroll
            for (int i = 0; i < 16; i += 4) {
              float4 f;
              float* fp = reinterpret_cast<float*>(&f);
#pragma unroll
              for (int e = 0; e < 4; e++) {
                const float g = __uint_as_float(v[i + e]), u = __uint_as_float(v[16 + i + e]);
                fp[e] = silu_mul<TC>(g, u);
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
            // the old values of this piece were asked for a piece ago (the first before the products
            // were complete); now ask for the next piece's, so that they travel under this piece's stores
            float4 old[8];
#pragma unroll
            for (int j = 0; j < 8; j++) old[j] = nxt[j];
            if (c0 + 32 < BN) load_old(c0 + 32);
#pragma unroll
            for (int j = 0; j < 8; j++) {
              const int rr = lr + 4 * j, row = row_base + rr;
              if (row >= M) continue;
              const float4 f = *reinterpret_cast<const float4*>(stg + rr * 36 + lc);
              *reinterpret_cast<float4*>(C + (size_t)row * ldc + col) =
                  make_float4(f.x + old[j].x, f.y + old[j].y, f.z + old[j].z, f.w + old[j].w);
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
                *reinterpret_cast<uint2*>(o) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
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
      // this warp has read its rows of the accumulator: tell the block that issues the MMAs
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_empty0 + buf * 8);
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();     // nobody frees tensor memory or leaves while the other block may still use it
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(512u));
  }
}

template <typename TC>
static int launch_tc2(void* C, const CUtensorMap& ma, const CUtensorMap& mw, int M, int N, int K, int ldc, int epilogue,
                      int* status, cudaStream_t st) {
  constexpr size_t smem = (size_t)T2_STAGES * (2 * 128 * TC_BK * 2) + (2 * T2_STAGES + 4) * 8 + 16 + 4 * 32 * 36 * 4 + 1024;
  auto kern = gemm_bf16_tc2_kernel<TC>;
  static bool set = false;
  if (!set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return leb_fail("leb_gemm_bf16_tc2: shared memory %zu: %s", smem, cudaGetErrorString(e));
    set = true;
  }
  static int n_sm = 0;
  if (!n_sm) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sm <= 0) n_sm = 148;
  }
  const long tiles = (long)ceil_div(N, T2_BN) * ceil_div(M, 256);
  const long pairs = tiles < n_sm / 2 ? tiles : n_sm / 2;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(2 * pairs));
  cfg.blockDim = dim3(T2_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_leb_pdl ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, ma, mw, (TC*)C, M, N, K, ldc, epilogue, status);
  if (e != cudaSuccess) return leb_fail("leb_gemm_bf16_tc2: %s", cudaGetErrorString(e));
  LEB_CHECK_LAUNCH("leb_gemm_bf16_tc2");
  return 0;
}

// The product on pairs of SMs; for many rows (the tiles are 256 x 256).  Same operands, epilogues
// and status word as leb_gemm_bf16_tc.
LEB_API int leb_gemm_bf16_tc2(void* C, int c_dtype, const void* A, const void* W, int M, int N, int K, int lda,
                              int ldc, int epilogue, int* status, cudaStream_t st) {
  if (M <= 0 || N <= 0) return 0;
  LEB_REQUIRE(K > 0 && K % 8 == 0 && lda % 8 == 0 && ((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0,
              "leb_gemm_bf16_tc2: operands not aligned for TMA (K %d, lda %d)", K, lda);
  LEB_REQUIRE(epilogue >= 0 && epilogue <= 2, "leb_gemm_bf16_tc2: unknown epilogue %d", epilogue);
  LEB_REQUIRE(epilogue != 1 || c_dtype == LEB_F32, "leb_gemm_bf16_tc2: adding needs a float C");
  LEB_REQUIRE(epilogue != 2 || N % 32 == 0, "leb_gemm_bf16_tc2: the SwiGLU epilogue needs N (%d) to be a multiple of 32", N);
  LEB_REQUIRE(status != nullptr, "leb_gemm_bf16_tc2: a status word is required");
  CUtensorMap ma, mw;
  if (tensor_map(&ma, A, M, K, lda, 128)) return 1;
  if (tensor_map(&mw, W, N, K, K, 128)) return 1;
  if (c_dtype == LEB_BF16) return launch_tc2<bf16>(C, ma, mw, M, N, K, ldc, epilogue, status, st);
  if (c_dtype == LEB_F32) return launch_tc2<float>(C, ma, mw, M, N, K, ldc, epilogue, status, st);
  return leb_fail("leb_gemm_bf16_tc2: unknown C dtype %d", c_dtype);
}
