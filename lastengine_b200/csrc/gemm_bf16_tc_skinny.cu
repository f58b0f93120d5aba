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

// The halves of a norm split between two products (see StreamNorm in gemm_bf16_stream.cu), as this
// product takes them (its second kernel, or with one slice the first): `ssq_in` scales the rows, `emit_*` leave what the next
// norm needs (adding epilogue only).
struct FinishNorm {
  const float* ssq_in;
  int parts_in, d_in;
  float eps;
  bf16* emit_vals;
  const float* emit_g;
  float* emit_ssq;
};

// With four stages of up to 24 KB two blocks fit an SM, and must: the next product's blocks then start,
// and fetch their first weights, under this one's (hence the register bound).
template <int MP, int SK_STAGES>  // activation rows padded to 16, 32, 64, 96 or 128 (the MMA's N); stages of the ring
__global__ void __launch_bounds__(SK_THREADS, SK_STAGES <= 4 ? 2 : 1)
gemm_tc_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                      float* __restrict__ part, void* __restrict__ C, int c_dtype, int M, int N, int K, int ldc,
                      int epilogue, int n_slices, int* __restrict__ status, FinishNorm nm) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ float row_scale[MP];
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
    if (n_slices == 1) {
      // the rows' factors of a split norm (1 without one): warp w takes rows w, w + 4, ...
      for (int m = warp - 2; m < MP; m += 4) {
        float sum = 0.f;
        if (nm.ssq_in && m < M)
          for (int p = lane; p < nm.parts_in; p += 32) sum += nm.ssq_in[(size_t)m * nm.parts_in + p];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (lane == 0) row_scale[m] = nm.ssq_in ? 1.0f / sqrtf(sum / (float)nm.d_in + nm.eps) : 1.f;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");   // the four epilogue warps
    }
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
        if (n_slices > 1) {
          if (n < N) {
            float* p = part + ((size_t)slice * M + c0) * N + n;
#pragma unroll
            for (int i = 0; i < 32; i++)
              if (c0 + i < M) p[(size_t)i * N] = __uint_as_float(v[i]);
          }
        } else if (epilogue == 2) {
          // lanes 0-15 hold the gate rows of 16 outputs, lanes 16-31 their up rows
          const int j = 16 * (n >> 5) + (lane & 15);
#pragma unroll
          for (int i = 0; i < 32; i++) {
            const float rs = c0 + i < M ? row_scale[c0 + i] : 0.f;
            const float gt = __uint_as_float(v[i]) * rs;
            const float up = __shfl_down_sync(0xffffffffu, gt, 16);
            if (lane < 16 && c0 + i < M && 2 * j < N) {
              const float a = c_dtype == LEB_F32 ? silu_mul<float>(gt, up) : silu_mul<bf16>(gt, up);
              if (c_dtype == LEB_F32) ((float*)C)[(size_t)(c0 + i) * ldc + j] = a;
              else ((bf16*)C)[(size_t)(c0 + i) * ldc + j] = __float2bfloat16_rn(a);
            }
          }
        } else if (c_dtype == LEB_F32) {
          float* o = (float*)C + (size_t)c0 * ldc + n;
          float old[32];
#pragma unroll
          for (int i = 0; i < 32; i++) old[i] = (epilogue == 1 && n < N && c0 + i < M) ? o[(size_t)i * ldc] : 0.f;
#pragma unroll
          for (int i = 0; i < 32; i++) {
            const bool in = n < N && c0 + i < M;
            const float a = old[i] + __uint_as_float(v[i]) * (c0 + i < M ? row_scale[c0 + i] : 0.f);
            if (in) o[(size_t)i * ldc] = a;
            if (nm.emit_vals) {   // the new residual, for the norm that follows (adding epilogue)
              float sq = in ? a * a : 0.f;
#pragma unroll
              for (int sh = 8; sh > 0; sh >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, sh);
              if (in) {
                nm.emit_vals[(size_t)(c0 + i) * N + n] = __float2bfloat16_rn(a * nm.emit_g[n]);
                if ((n & 15) == 0) nm.emit_ssq[(size_t)(c0 + i) * ((N + 15) / 16) + n / 16] = sq;
              }
            }
          }
        } else if (n < N) {
          bf16* o = (bf16*)C + (size_t)c0 * ldc + n;
#pragma unroll
          for (int i = 0; i < 32; i++)
            if (c0 + i < M) o[(size_t)i * ldc] = __float2bfloat16_rn(__uint_as_float(v[i]) * row_scale[c0 + i]);
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

// What the convolution epilogue needs (epilogue 3: the product is the conv mixer's in_proj [3D, K] of a
// decode step, and the second kernel does the one-token gated convolution with the state shift, as
// the weight stream's epilogue does for up to 16 rows; gemm_bf16_stream.cu).
struct FinishConv {
  const float* w;        // [D, Lc] taps, oldest first
  const float* bias;     // [D] or null
  float* state;          // [slots, D, Lc-1]
  const int* row_seq;    // row -> sequence of the step
  const int* seq_slot;   // sequence -> cache slot (-1: padding)
  int Lc;
};
#define SK_CONV_MAX_LC 5

// One element's partial sums added in slice order.  Eight loads are issued before the first is
// used: a thread that fetched one slice at a time spent a round trip to L2 on each.
__device__ __forceinline__ float sum_slices(const float* __restrict__ p, size_t slab, int n_slices) {
  float a = 0.f;
  for (int s0 = 0; s0 < n_slices; s0 += 8) {
    float v[8];
#pragma unroll
    for (int u = 0; u < 8; u++) v[u] = s0 + u < n_slices ? __ldcs(p + (size_t)(s0 + u) * slab) : 0.f;
#pragma unroll
    for (int u = 0; u < 8; u++) a += v[u];
  }
  return a;
}

// Adds the slices in order and applies the epilogue.  part: [slices][M][N] float.
template <typename TC>
__global__ void __launch_bounds__(256)
skinny_finish_kernel(TC* __restrict__ C, const float* __restrict__ part, int M, int N, int ldc, int epilogue,
                     int n_slices, FinishNorm nm, FinishConv cv) {
  pdl_trigger();   // the kernel after this one may start and wait (see common.cuh)
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
  if (epilogue == 3) {
    // channel j: B, C and x are D columns apart.  The projections are rounded to bfloat16 as if they
    // had been stored, taps oldest first, the state shifted by one (shortconv.cu, one-token form).
    const int D = N / 3;
    if (j >= D) return;
    const float* p0 = part + (size_t)m * N + j;
    const float pb = sum_slices(p0, slab, n_slices), pc = sum_slices(p0 + D, slab, n_slices),
                px = sum_slices(p0 + 2 * D, slab, n_slices);
    TC* yo = C + (size_t)m * ldc + j;
    const int slot = cv.seq_slot[cv.row_seq[m]];
    if (slot < 0) {   // padding row
      *yo = from_f32<TC>(0.f);
      return;
    }
    const float bx = to_f32(from_f32<TC>(pb * r)) * to_f32(from_f32<TC>(px * r));
    float* sc = cv.state + ((size_t)slot * D + j) * (cv.Lc - 1);
    float st[SK_CONV_MAX_LC - 1];
#pragma unroll
    for (int k = 0; k < SK_CONV_MAX_LC - 1; k++) st[k] = k < cv.Lc - 1 ? sc[k] : 0.f;
    float acc = cv.bias ? cv.bias[j] : 0.f;
#pragma unroll
    for (int k = 0; k < SK_CONV_MAX_LC - 1; k++)
      if (k < cv.Lc - 1) acc += cv.w[(size_t)j * cv.Lc + k] * st[k];
    acc += cv.w[(size_t)j * cv.Lc + cv.Lc - 1] * bx;
#pragma unroll
    for (int k = 0; k < SK_CONV_MAX_LC - 2; k++)
      if (k < cv.Lc - 2) sc[k] = st[k + 1];
    sc[cv.Lc - 2] = bx;
    *yo = from_f32<TC>(to_f32(from_f32<TC>(pc * r)) * acc);
    return;
  }
  if (epilogue == 2) {
    // column n = 32*(j/16) + (j%16) is the gate of output j, n + 16 its up value
    if (j >= N / 2) return;
    const int n = 32 * (j >> 4) + (j & 15);
    const float g = sum_slices(part + (size_t)m * N + n, slab, n_slices) * r;
    const float u = sum_slices(part + (size_t)m * N + n + 16, slab, n_slices) * r;
    C[(size_t)m * ldc + j] = from_f32<TC>(silu_mul<TC>(g, u));
    return;
  }
  const bool in = j < N;
  float a = 0.f;
  if (in) {
    a = sum_slices(part + (size_t)m * N + j, slab, n_slices) * r;
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

int leb_slices_finish(void* C, int c_dtype, const float* part, int M, int N, int ldc, int epilogue, int n_slices,
                      cudaStream_t st) {
  const int cols = epilogue == 2 ? N / 2 : N;
  dim3 grid(ceil_div(cols, 256), M);
  if (c_dtype == LEB_F32)
    leb_launch(skinny_finish_kernel<float>, grid, dim3(256), 0, st, (float*)C, part, M, N, ldc, epilogue, n_slices, FinishNorm{}, FinishConv{});
  else if (c_dtype == LEB_BF16)
    leb_launch(skinny_finish_kernel<bf16>, grid, dim3(256), 0, st, (bf16*)C, part, M, N, ldc, epilogue, n_slices, FinishNorm{}, FinishConv{});
  else
    return leb_fail("leb_slices_finish: unknown C dtype %d", c_dtype);
  LEB_CHECK_LAUNCH("leb_slices_finish");
  return 0;
}

template <int MP, int SK_STAGES>
static int launch_skinny(const CUtensorMap& mw, const CUtensorMap& mx, float* part, void* C, int c_dtype, int M,
                         int N, int K, int ldc, int epilogue, int n_slices, int* status, FinishNorm nm, cudaStream_t st) {
  constexpr size_t x_stride = ((size_t)MP * TC_BK * 2 + 1023) / 1024 * 1024;
  constexpr size_t smem = SK_STAGES * (128 * TC_BK * 2 + x_stride) + (2 * SK_STAGES + 1) * 8 + 16 + 1024;
  auto kern = gemm_tc_skinny_kernel<MP, SK_STAGES>;
  static bool set = false;
  if (!set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return leb_fail("leb_gemm_bf16_skinny: shared memory %zu: %s", smem, cudaGetErrorString(e));
    set = true;
  }
  dim3 grid(ceil_div(N, 128), n_slices);
  cudaError_t e = leb_launch(kern, grid, dim3(SK_THREADS), smem, st, mw, mx, part, C, c_dtype, M, N, K, ldc, epilogue,
                             n_slices, status, nm);
  if (e != cudaSuccess) return leb_fail("leb_gemm_bf16_skinny: %s", cudaGetErrorString(e));
  LEB_CHECK_LAUNCH("leb_gemm_bf16_skinny");
  return 0;
}

// How many K slices the product is cut into (the caller sizes the workspace with it): about one
// block per SM, at least four k-blocks of 64 per slice, none of them empty.  With one slice the
// first kernel writes the result itself.
LEB_API int leb_gemm_bf16_skinny_slices(int N, int K) {
  const int tiles = ceil_div(N, 128), nk = ceil_div(K, TC_BK);
  const int n_sm = sm_count();
  int s = n_sm / tiles;                       // one block per SM at most
  if (tiles * s < n_sm * 3 / 4) s++;          // unless that leaves a quarter of the SMs without a block
  if (s > nk / 4) s = nk / 4;
  if (s < 1) s = 1;
  if (s > 32) s = 32;
  const int per = ceil_div(nk, s);
  return ceil_div(nk, per);
}

LEB_API int leb_gemm_bf16_skinny_supported(const void* A, const void* W, int M, int K, int lda) {
  return M >= 1 && M <= 128 && K > 0 && K % 8 == 0 && lda % 8 == 0 && ((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0;
}

// part: float workspace of slices*M*N elements (unused with one slice).
// The split-norm halves are optional (null).
static int skinny_product(void* C, int c_dtype, const void* A, const void* W, int M, int N, int K, int lda,
                          int ldc, int epilogue, float* part, int n_slices, FinishNorm nm, FinishConv cv, int* status,
                          cudaStream_t st) {
  const int MP = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : (M <= 96 ? 96 : 128)));
  CUtensorMap mw, mx;
  if (tensor_map(&mw, W, N, K, K, 128)) return 1;
  if (tensor_map(&mx, A, M, K, lda, MP)) return 1;
  int rc;
  // Up to 64 activation rows a stage has 24 KB: four of them leave room for two blocks per SM (the next
  // product's blocks then start, and fetch their first weights, under this one's).  Eight stages and one
  // block per SM were measured too: faster for a product alone (a 23 MB product of 64 rows 11.9 us
  // against 16.4), no faster inside a decode step, where the next product can then not start early.

  const int first_ep = epilogue == 3 ? 0 : epilogue;   // the convolution is the second kernel's
  // From 65 rows on a stage has 28 or 32 KB: three of them, so that two blocks still fit an SM
  // (measured at batch 96 and 128: 1.26 and 1.47 ms a decode step, against 1.35 and 1.56 with four
  // stages and 1.38 and 1.55 with six stages of the 128-row form alone).
  switch (MP) {
    case 16: rc = launch_skinny<16, 4>(mw, mx, part, C, c_dtype, M, N, K, ldc, first_ep, n_slices, status, nm, st); break;
    case 32: rc = launch_skinny<32, 4>(mw, mx, part, C, c_dtype, M, N, K, ldc, first_ep, n_slices, status, nm, st); break;
    case 64: rc = launch_skinny<64, 4>(mw, mx, part, C, c_dtype, M, N, K, ldc, first_ep, n_slices, status, nm, st); break;
    case 96: rc = launch_skinny<96, 3>(mw, mx, part, C, c_dtype, M, N, K, ldc, first_ep, n_slices, status, nm, st); break;
    default: rc = launch_skinny<128, 3>(mw, mx, part, C, c_dtype, M, N, K, ldc, first_ep, n_slices, status, nm, st); break;
  }
  if (rc || n_slices == 1) return rc;
  const int cols = epilogue == 2 ? N / 2 : (epilogue == 3 ? N / 3 : N);
  dim3 grid(ceil_div(cols, 256), M);
  if (c_dtype == LEB_F32)
    leb_launch(skinny_finish_kernel<float>, grid, dim3(256), 0, st, (float*)C, (const float*)part, M, N, ldc, epilogue, n_slices, nm, cv);
  else if (c_dtype == LEB_BF16)
    leb_launch(skinny_finish_kernel<bf16>, grid, dim3(256), 0, st, (bf16*)C, (const float*)part, M, N, ldc, epilogue, n_slices, nm, cv);
  else
    return leb_fail("leb_gemm_bf16_skinny: unknown C dtype %d", c_dtype);
  LEB_CHECK_LAUNCH("leb_gemm_bf16_skinny finish");
  return 0;
}

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
  LEB_REQUIRE(!emit_vals || (epilogue == 1 && emit_g && emit_ssq), "leb_gemm_bf16_skinny: only an adding product leaves the next norm's input");
  LEB_REQUIRE(!ssq_in || (parts_in > 0 && d_in > 0), "leb_gemm_bf16_skinny: the sums of squares need their count and the row width");
  LEB_REQUIRE(n_slices >= 1 && (n_slices == 1 || part), "leb_gemm_bf16_skinny: slices need a workspace");
  const FinishNorm nm{ssq_in, parts_in, d_in, eps, (bf16*)emit_vals, emit_g, emit_ssq};
  return skinny_product(C, c_dtype, A, W, M, N, K, lda, ldc, epilogue, part, n_slices, nm, FinishConv{}, status, st);
}

// The conv mixer's decode step for 17 to 128 sequences: y[M, D] = conv(in_proj . h) with the state
// updated (every row is the one new token of its sequence).  W: in_proj [3D, K]; conv_w [D, Lc];
// state [slots, D, Lc-1] float.  Needs at least two slices (the convolution is the second kernel's).
LEB_API int leb_gemm_bf16_skinny_conv(void* y, const void* A, const void* W, int M, int D, int K, int lda, int ldy,
                                      const float* conv_w, const float* bias, float* state, const int* row_seq,
                                      const int* seq_slot, int Lc, float* part, int n_slices, const float* ssq_in,
                                      int parts_in, int d_in, float eps, int* status, cudaStream_t st) {
  if (M <= 0 || D <= 0) return 0;
  LEB_REQUIRE(leb_gemm_bf16_skinny_supported(A, W, M, K, lda), "leb_gemm_bf16_skinny_conv: takes 1..128 rows and TMA-aligned operands (M %d, K %d, lda %d)", M, K, lda);
  LEB_REQUIRE(Lc >= 2 && Lc <= SK_CONV_MAX_LC, "leb_gemm_bf16_skinny_conv: conv length %d outside 2..%d", Lc, SK_CONV_MAX_LC);
  LEB_REQUIRE(conv_w && state && row_seq && seq_slot && status, "leb_gemm_bf16_skinny_conv: taps, state, the step's tables and a status word are required");
  LEB_REQUIRE(n_slices >= 2 && part, "leb_gemm_bf16_skinny_conv: needs at least two slices and their workspace");
  LEB_REQUIRE(!ssq_in || (parts_in > 0 && d_in > 0), "leb_gemm_bf16_skinny_conv: the sums of squares need their count and the row width");
  const FinishNorm nm{ssq_in, parts_in, d_in, eps, nullptr, nullptr, nullptr};
  const FinishConv cv{conv_w, bias, state, row_seq, seq_slot, Lc};
  return skinny_product(y, LEB_BF16, A, W, M, 3 * D, K, lda, ldy, 3, part, n_slices, nm, cv, status, st);
}
