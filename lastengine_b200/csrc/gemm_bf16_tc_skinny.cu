// bfloat16 matrix product for a few dozen rows (decode steps of 17 to 128 sequences):
//   C[M,N] (+)= A[M,K] . W[N,K]^T on tcgen05, with the roles of the operands swapped.
//
// With so few rows the product is bound by streaming W, and a 128-row tcgen05 tile of A would be
// mostly padding.  So W is the 128-row operand: a block takes 128 rows of W and a slice of K,
// the activations (padded to a multiple of 16 rows) are the narrow operand, and the accumulator
// in tensor memory is the transposed tile C^T[n, m].  Slicing K as well gives every SM a block
// even when N/128 is small; the slices' partial tiles go to a float workspace and a second small
// kernel adds them in slice order (so the result does not depend on timing) and applies the
// epilogue.  With one slice the first kernel writes C itself.
//
// A thread of the epilogue owns one row n of W and holds its values for 32 activation rows; for
// a fixed activation row the lanes of a warp are 32 consecutive n, so every store is a whole
// 128-byte line without staging.
//
// Roles, ring, bounded waits and status word as in gemm_bf16_tc.cu.
#include "tc_common.cuh"

#define SK_THREADS 192
// Stages of the ring.  Up to 64 activation rows a stage has 24 KB and four of them leave room for two
// blocks per SM: the next product's blocks then start, and fetch their first weights, under this one's.
#define SK_STAGES_OF(MP) ((MP) > 64 ? 6 : 4)

template <int MP>  // activation rows padded to 16..128 (the MMA's N)
__global__ void __launch_bounds__(SK_THREADS)
gemm_tc_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                      float* __restrict__ part, void* __restrict__ C, int c_dtype, int M, int N, int K, int ldc,
                      int epilogue, int n_slices, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  constexpr int SK_STAGES = SK_STAGES_OF(MP);
  constexpr int W_BYTES = 128 * TC_BK * 2, X_BYTES = MP * TC_BK * 2;
  uint8_t* sw = smem;
  uint8_t* sx = smem + SK_STAGES * W_BYTES;
  uint64_t* full = (uint64_t*)(sx + SK_STAGES * ((X_BYTES + 1023) / 1024 * 1024));
  uint64_t* empty = full + SK_STAGES;
  uint64_t* acc_full = empty + SK_STAGES;
  uint32_t* tmem_slot = (uint32_t*)(acc_full + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  constexpr int X_STRIDE = (X_BYTES + 1023) / 1024 * 1024;   // stages stay 1024-byte aligned
  constexpr uint32_t TMEM_COLS = MP <= 32 ? 32 : (MP <= 64 ? 64 : 128);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * 128;
  const int slice = blockIdx.y;
  const int nk = (K + TC_BK - 1) / TC_BK;
  const int per = (nk + n_slices - 1) / n_slices;
  const int kb_lo = slice * per, kb_hi = min(nk, kb_lo + per);
  const int my_nk = max(0, kb_hi - kb_lo);

  if (threadIdx.x == 0) {
    for (int s = 0; s < SK_STAGES; s++) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_acc = *tmem_slot;
  pdl_trigger();
  if (warp == 0 && lane == 0) {
    // The weights do not depend on the kernel before this one: the weight tiles of the first
    // stages are asked for before the wait, the activation tiles of those stages after it.
    const int first = min(my_nk, SK_STAGES);
    for (int i = 0; i < first; i++) {
      mbar_expect_tx(&full[i], W_BYTES + X_BYTES);
      tma_load_2d(sw + i * W_BYTES, &map_w, &full[i], (kb_lo + i) * TC_BK, n0);
    }
    pdl_wait();
    for (int i = 0; i < first; i++) tma_load_2d(sx + i * X_STRIDE, &map_x, &full[i], (kb_lo + i) * TC_BK, 0);
    for (int i = first; i < my_nk; i++) {
      const int s = i % SK_STAGES;
      if (!mbar_wait(&empty[s], ((i / SK_STAGES) & 1) ^ 1, abort_flag)) { atomicExch(status, 11); break; }
      mbar_expect_tx(&full[s], W_BYTES + X_BYTES);
      tma_load_2d(sw + s * W_BYTES, &map_w, &full[s], (kb_lo + i) * TC_BK, n0);
      tma_load_2d(sx + s * X_STRIDE, &map_x, &full[s], (kb_lo + i) * TC_BK, 0);
    }
  } else {
    pdl_wait();   // the activations come from the kernel before this one; nothing is written before it
  }

  if (warp == 0) {
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(MP >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      bool ok = true;
      for (int i = 0; i < my_nk; i++) {
        const int s = i % SK_STAGES;
        if (!mbar_wait(&full[s], (i / SK_STAGES) & 1, abort_flag)) { atomicExch(status, 12); ok = false; break; }
        tc_fence_after();
        const uint64_t da = make_desc(smem_u32(sw + s * W_BYTES));
        const uint64_t db = make_desc(smem_u32(sx + s * X_STRIDE));
#pragma unroll
        for (int k = 0; k < TC_BK / 16; k++)
          umma_bf16(tmem_acc, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (i | k) != 0);
        umma_commit(&empty[s]);
      }
      if (ok) umma_commit(acc_full);   // with no k-slices of its own this arrives at once
    }
  } else {
    const int quad = warp & 3;
    const int n = n0 + quad * 32 + lane;
    bool ok = mbar_wait(acc_full, 0, abort_flag);
    if (!ok && lane == 0) atomicExch(status, 13);
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    tc_fence_after();
    if (ok) {
#pragma unroll 1
      for (int c0 = 0; c0 < MP; c0 += 32) {
        uint32_t v[32];
        if (my_nk > 0) {
          if (MP - c0 >= 32) {
            tmem_ld32(tmem_acc + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0, v);
          } else {   // 16 columns left
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                  "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                : "r"(tmem_acc + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0));
#pragma unroll
            for (int i = 16; i < 32; i++) v[i] = 0u;
          }
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; i++) v[i] = 0u;   // a slice beyond K contributes nothing
        }
        if (n < N) {
          if (n_slices > 1) {
            float* p = part + ((size_t)slice * M + c0) * N + n;
#pragma unroll
            for (int i = 0; i < 32; i++)
              if (c0 + i < M) p[(size_t)i * N] = __uint_as_float(v[i]);
          } else if (c_dtype == LEB_F32) {
            float* o = (float*)C + (size_t)c0 * ldc + n;
            if (epilogue == 1) {
              float old[32];
#pragma unroll
              for (int i = 0; i < 32; i++) old[i] = c0 + i < M ? o[(size_t)i * ldc] : 0.f;
#pragma unroll
              for (int i = 0; i < 32; i++)
                if (c0 + i < M) o[(size_t)i * ldc] = old[i] + __uint_as_float(v[i]);
            } else {
#pragma unroll
              for (int i = 0; i < 32; i++)
                if (c0 + i < M) o[(size_t)i * ldc] = __uint_as_float(v[i]);
            }
          } else {
            bf16* o = (bf16*)C + (size_t)c0 * ldc + n;
#pragma unroll
            for (int i = 0; i < 32; i++)
              if (c0 + i < M) o[(size_t)i * ldc] = __float2bfloat16_rn(__uint_as_float(v[i]));
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_acc, TMEM_COLS);
  }
}

// The halves of a norm split between two products (see StreamNorm in gemm_bf16_stream.cu), as the
// second kernel of this product takes them: `ssq_in` scales the rows, `emit_*` leave what the next
// norm needs (adding epilogue only).
struct FinishNorm {
  const float* ssq_in;
  int parts_in, d_in;
  float eps;
  bf16* emit_vals;
  const float* emit_g;
  float* emit_ssq;
};

// Adds the slices in order and applies the epilogue.  part: [slices][M][N] float.
template <typename TC>
__global__ void __launch_bounds__(256)
skinny_finish_kernel(TC* __restrict__ C, const float* __restrict__ part, int M, int N, int ldc, int epilogue,
                     int n_slices, FinishNorm nm) {
  pdl_wait();
  const int m = blockIdx.y;
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  const size_t slab = (size_t)M * N;
  float r = 1.f;
  if (nm.ssq_in) {   // the row's factor: every thread of the block takes part
    __shared__ float warp_part[8];
    float sum = 0.f;
    for (int p = threadIdx.x; p < nm.parts_in; p += blockDim.x) sum += nm.ssq_in[(size_t)m * nm.parts_in + p];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = sum;
    __syncthreads();
    sum = 0.f;
#pragma unroll
    for (int w = 0; w < 8; w++) sum += warp_part[w];
    r = 1.0f / sqrtf(sum / (float)nm.d_in + nm.eps);
  }
  if (epilogue == 2) {
    // column n = 32*(j/16) + (j%16) is the gate of output j, n + 16 its up value
    if (j >= N / 2) return;
    const int n = 32 * (j >> 4) + (j & 15);
    float g = 0.f, u = 0.f;
    for (int s = 0; s < n_slices; s++) {
      g += part[s * slab + (size_t)m * N + n];
      u += part[s * slab + (size_t)m * N + n + 16];
    }
    g *= r;
    u *= r;
    C[(size_t)m * ldc + j] = from_f32<TC>(g / (1.0f + expf(-g)) * u);
    return;
  }
  const bool in = j < N;
  float a = 0.f;
  if (in) {
    for (int s = 0; s < n_slices; s++) a += part[s * slab + (size_t)m * N + j];
    a *= r;
    TC* o = C + (size_t)m * ldc + j;
    if (epilogue == 1) a += to_f32(*o);
    *o = from_f32<TC>(a);
  }
  if (nm.emit_vals) {   // the new residual, for the norm that follows: bf16(x * g) and the sum of x^2 per 16 columns
    float sq = in ? a * a : 0.f;
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    if (in) {
      nm.emit_vals[(size_t)m * N + j] = __float2bfloat16_rn(a * nm.emit_g[j]);
      if ((j & 15) == 0) nm.emit_ssq[(size_t)m * ((N + 15) / 16) + j / 16] = sq;
    }
  }
}

template <int MP>
static int launch_skinny(const CUtensorMap& mw, const CUtensorMap& mx, float* part, void* C, int c_dtype, int M,
                         int N, int K, int ldc, int epilogue, int n_slices, int* status, cudaStream_t st) {
  constexpr int SK_STAGES = SK_STAGES_OF(MP);
  constexpr size_t x_stride = ((size_t)MP * TC_BK * 2 + 1023) / 1024 * 1024;
  constexpr size_t smem = SK_STAGES * (128 * TC_BK * 2 + x_stride) + (2 * SK_STAGES + 1) * 8 + 16 + 1024;
  auto kern = gemm_tc_skinny_kernel<MP>;
  static bool set = false;
  if (!set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return leb_fail("leb_gemm_bf16_skinny: shared memory %zu: %s", smem, cudaGetErrorString(e));
    set = true;
  }
  dim3 grid(ceil_div(N, 128), n_slices);
  cudaError_t e = leb_launch(kern, grid, dim3(SK_THREADS), smem, st, mw, mx, part, C, c_dtype, M, N, K, ldc, epilogue,
                             n_slices, status);
  if (e != cudaSuccess) return leb_fail("leb_gemm_bf16_skinny: %s", cudaGetErrorString(e));
  LEB_CHECK_LAUNCH("leb_gemm_bf16_skinny");
  return 0;
}

// How many K slices the product is cut into (the caller sizes the workspace with it):
// enough blocks for every SM, at least four k-blocks of 64 per slice.
LEB_API int leb_gemm_bf16_skinny_slices(int N, int K) {
  const int tiles = ceil_div(N, 128), nk = ceil_div(K, TC_BK);
  int s = 160 / tiles;
  if (s > nk / 4) s = nk / 4;
  if (s < 1) s = 1;
  if (s > 32) s = 32;
  return s;
}

LEB_API int leb_gemm_bf16_skinny_supported(const void* A, const void* W, int M, int K, int lda) {
  return M >= 1 && M <= 128 && K > 0 && K % 8 == 0 && lda % 8 == 0 && ((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0;
}

// part: float workspace of slices*M*N elements (unused with one slice).
// The split-norm halves are optional (null): they need at least two slices, since the second kernel applies them.
LEB_API int leb_gemm_bf16_skinny(void* C, int c_dtype, const void* A, const void* W, int M, int N, int K, int lda,
                                 int ldc, int epilogue, float* part, int n_slices, const float* ssq_in, int parts_in,
                                 int d_in, float eps, void* emit_vals, const float* emit_g, float* emit_ssq, int* status,
                                 cudaStream_t st) {
  if (M <= 0 || N <= 0) return 0;
  LEB_REQUIRE(leb_gemm_bf16_skinny_supported(A, W, M, K, lda), "leb_gemm_bf16_skinny: takes 1..128 rows and TMA-aligned operands (M %d, K %d, lda %d)", M, K, lda);
  LEB_REQUIRE(epilogue >= 0 && epilogue <= 2, "leb_gemm_bf16_skinny: unknown epilogue %d", epilogue);
  LEB_REQUIRE(epilogue != 1 || c_dtype == LEB_F32, "leb_gemm_bf16_skinny: adding needs a float C");
  LEB_REQUIRE(epilogue != 2 || N % 32 == 0, "leb_gemm_bf16_skinny: the SwiGLU epilogue needs N (%d) to be a multiple of 32", N);
  LEB_REQUIRE(status != nullptr, "leb_gemm_bf16_skinny: a status word is required");
  if (epilogue == 2 && n_slices < 2) n_slices = 2;   // SwiGLU pairs columns: it is applied by the second kernel
  LEB_REQUIRE(!(ssq_in || emit_vals) || n_slices >= 2, "leb_gemm_bf16_skinny: a split norm needs at least two slices");
  LEB_REQUIRE(!emit_vals || (epilogue == 1 && emit_g && emit_ssq), "leb_gemm_bf16_skinny: only an adding product leaves the next norm's input");
  LEB_REQUIRE(!ssq_in || (parts_in > 0 && d_in > 0), "leb_gemm_bf16_skinny: the sums of squares need their count and the row width");
  const FinishNorm nm{ssq_in, parts_in, d_in, eps, (bf16*)emit_vals, emit_g, emit_ssq};
  LEB_REQUIRE(n_slices >= 1 && (n_slices == 1 || part), "leb_gemm_bf16_skinny: slices need a workspace");
  const int MP = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
  CUtensorMap mw, mx;
  if (tensor_map(&mw, W, N, K, K, 128)) return 1;
  if (tensor_map(&mx, A, M, K, lda, MP)) return 1;
  int rc;
  switch (MP) {
    case 16: rc = launch_skinny<16>(mw, mx, part, C, c_dtype, M, N, K, ldc, epilogue, n_slices, status, st); break;
    case 32: rc = launch_skinny<32>(mw, mx, part, C, c_dtype, M, N, K, ldc, epilogue, n_slices, status, st); break;
    case 64: rc = launch_skinny<64>(mw, mx, part, C, c_dtype, M, N, K, ldc, epilogue, n_slices, status, st); break;
    default: rc = launch_skinny<128>(mw, mx, part, C, c_dtype, M, N, K, ldc, epilogue, n_slices, status, st); break;
  }
  if (rc || n_slices == 1) return rc;
  const int cols = epilogue == 2 ? N / 2 : N;
  dim3 grid(ceil_div(cols, 256), M);
  if (c_dtype == LEB_F32)
    leb_launch(skinny_finish_kernel<float>, grid, dim3(256), 0, st, (float*)C, (const float*)part, M, N, ldc, epilogue, n_slices, nm);
  else if (c_dtype == LEB_BF16)
    leb_launch(skinny_finish_kernel<bf16>, grid, dim3(256), 0, st, (bf16*)C, (const float*)part, M, N, ldc, epilogue, n_slices, nm);
  else
    return leb_fail("leb_gemm_bf16_skinny: unknown C dtype %d", c_dtype);
  LEB_CHECK_LAUNCH("leb_gemm_bf16_skinny finish");
  return 0;
}
