// bfloat16 matrix product for few rows (decode):  C[M,N] (+)= A[M,K] . W[N,K]^T, float accumulate.
//
// With M <= 64 the product is bound by reading W once, so the kernel is built around the
// weight stream, as the reference's decode matvec is (src/cuda/kernels.cu:371-392: one pass over
// the weight rows, 8 warps per block).  Roles are swapped for the tensor core: 16 weight rows
// are the "M" side of mma.m16n8k16 and 8 activation rows are its "N" side.  A block owns 16
// weight rows and up to 64 activation rows; its 8 warps split K in slices of 32 and their
// partial sums are added in warp order through shared memory, so the result of a row does not
// depend on which other rows are in the launch.
//
// Each lane reads 16 contiguous bytes (8 values of k) of a weight row and of an activation
// row and feeds them to two mma.k16 as k-pairs (0,1)(2,3) and (4,5)(6,7): both operands use the
// same assignment of real k to the instruction's k slots, and a sum over k does not care
// about the order.
//
// With group_offsets the rows of A and C are grouped by expert (group e: rows
// [off[e], off[e+1]), weights W + e*w_group_stride).  epilogue: 0 store, 1 add into float C,
// 2 SwiGLU over interleaved weights (rows 32j..32j+15 gate, 32j+16..32j+31 up of the same 16
// outputs): C[m, 16j+i] = silu(gate_i) * up_i, so C has N/2 columns.
#include "common.cuh"

#define SM_WARPS 8
#define SM_ROWS 16

__device__ __forceinline__ void mma_bf16_16816(float* d, uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// MT tiles of 8 activation rows, NSUB tiles of 16 weight rows, U k-slices of a warp loaded at once
template <typename TC, int MT, int NSUB, int U>
__global__ void __launch_bounds__(32 * SM_WARPS)
gemm_bf16_small_kernel(TC* __restrict__ C, const bf16* __restrict__ A, const bf16* __restrict__ W,
                       int M, int N, int K, int lda, int ldc, int epilogue,
                       const int* __restrict__ group_offsets, size_t w_group_stride) {
  __shared__ float red[SM_WARPS][NSUB][SM_ROWS][8 * MT + 1];
  int row_begin = 0, row_end = M;
  const int n0 = blockIdx.x * (SM_ROWS * NSUB);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (!group_offsets) {
    // The weights do not depend on the kernel before this one: ask for this block's rows to be
    // brought into L2 now, while that kernel finishes, and only then wait for the activations.
    const size_t bytes = (size_t)K * 2;
    for (int rr = 0; rr < SM_ROWS * NSUB; rr++) {
      const int n = n0 + rr;
      if (n >= N) break;
      const char* p = (const char*)(W + (size_t)n * K);
      for (size_t off = (size_t)threadIdx.x * 128; off < bytes; off += (size_t)blockDim.x * 128)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(p + off));
    }
  }
  pdl_trigger();   // the kernel after this one may start and wait (see common.cuh)
  pdl_wait();
  if (group_offsets) {
    row_begin = group_offsets[blockIdx.z];
    row_end = group_offsets[blockIdx.z + 1];
    W += (size_t)blockIdx.z * w_group_stride;
  }
  const int m0 = row_begin + blockIdx.y * (8 * MT);
  if (m0 >= row_end) return;
  const int r = lane >> 2, c = lane & 3;

  float acc[NSUB][MT][4];
#pragma unroll
  for (int s = 0; s < NSUB; s++)
#pragma unroll
    for (int t = 0; t < MT; t++)
#pragma unroll
      for (int e = 0; e < 4; e++) acc[s][t][e] = 0.f;

  const bf16* wrow[NSUB][2];
#pragma unroll
  for (int s = 0; s < NSUB; s++) {
    int na = n0 + s * SM_ROWS + r, nb = na + 8;
    wrow[s][0] = W + (size_t)(na < N ? na : N - 1) * K;
    wrow[s][1] = W + (size_t)(nb < N ? nb : N - 1) * K;
  }
  const bf16* arow[MT];
#pragma unroll
  for (int t = 0; t < MT; t++) {
    int m = m0 + t * 8 + r;
    arow[t] = m < row_end ? A + (size_t)m * lda : nullptr;
  }

  const int n_kb = (K + 31) / 32;
  // The stream is only as fast as the bytes in flight: a warp first issues the loads of U of
  // its k-slices (U * (2 NSUB + MT) 16-byte loads per lane), and only then multiplies.  A deep
  // U costs registers, hence resident blocks: the launcher picks the deepest U whose blocks
  // still all fit on the GPU at once (a second, partial wave would double the time).
  const uint4 zero = make_uint4(0, 0, 0, 0);
  for (int kb0 = warp; kb0 < n_kb; kb0 += SM_WARPS * U) {
    uint4 wa[U][NSUB][2], xb[U][MT];
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int k = (kb0 + u * SM_WARPS) * 32 + c * 8;
      const bool kin = k < K;  // K is a multiple of 8: a 16-byte piece is inside or outside as a whole
#pragma unroll
      for (int s = 0; s < NSUB; s++) {
        wa[u][s][0] = kin ? __ldg((const uint4*)(wrow[s][0] + k)) : zero;
        wa[u][s][1] = kin ? __ldg((const uint4*)(wrow[s][1] + k)) : zero;
      }
#pragma unroll
      for (int t = 0; t < MT; t++) xb[u][t] = (kin && arow[t]) ? *(const uint4*)(arow[t] + k) : zero;
    }
#pragma unroll
    for (int u = 0; u < U; u++)
#pragma unroll
      for (int s = 0; s < NSUB; s++)
#pragma unroll
        for (int t = 0; t < MT; t++) {
          mma_bf16_16816(acc[s][t], wa[u][s][0].x, wa[u][s][1].x, wa[u][s][0].y, wa[u][s][1].y, xb[u][t].x, xb[u][t].y);
          mma_bf16_16816(acc[s][t], wa[u][s][0].z, wa[u][s][1].z, wa[u][s][0].w, wa[u][s][1].w, xb[u][t].z, xb[u][t].w);
        }
  }

  // accumulator fragment: [0] (row r, col 2c) [1] (r, 2c+1) [2] (r+8, 2c) [3] (r+8, 2c+1)
#pragma unroll
  for (int s = 0; s < NSUB; s++)
#pragma unroll
    for (int t = 0; t < MT; t++) {
      red[warp][s][r][t * 8 + 2 * c] = acc[s][t][0];
      red[warp][s][r][t * 8 + 2 * c + 1] = acc[s][t][1];
      red[warp][s][r + 8][t * 8 + 2 * c] = acc[s][t][2];
      red[warp][s][r + 8][t * 8 + 2 * c + 1] = acc[s][t][3];
    }
  __syncthreads();

  if (epilogue == 2) {
    // NSUB == 2: sub-tile 0 holds the gate rows, sub-tile 1 the up rows of outputs 16*blockIdx.x + i
    const int jbase = blockIdx.x * SM_ROWS;
    for (int idx = threadIdx.x; idx < SM_ROWS * 8 * MT; idx += blockDim.x) {
      const int col = idx / SM_ROWS, i = idx % SM_ROWS;  // consecutive threads: consecutive outputs
      const int m = m0 + col;
      if (m >= row_end || 2 * (jbase + i) >= N) continue;
      float g = 0.f, u = 0.f;
#pragma unroll
      for (int w = 0; w < SM_WARPS; w++) {
        g += red[w][0][i][col];
        u += red[w][NSUB - 1][i][col];
      }
      C[(size_t)m * ldc + jbase + i] = from_f32<TC>(silu_mul<TC>(g, u));
    }
    return;
  }
  for (int idx = threadIdx.x; idx < NSUB * SM_ROWS * 8 * MT; idx += blockDim.x) {
    const int col = idx / (NSUB * SM_ROWS), rr = idx % (NSUB * SM_ROWS);
    const int m = m0 + col, n = n0 + rr;
    if (m >= row_end || n >= N) continue;
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < SM_WARPS; w++) v += red[w][rr / SM_ROWS][rr % SM_ROWS][col];
    TC* cp = C + (size_t)m * ldc + n;
    if (epilogue == 1) v += to_f32(*cp);
    *cp = from_f32<TC>(v);
  }
}

template <typename TC, int NSUB>
static int launch_small(void* C, const bf16* A, const bf16* W, int M, int N, int K, int lda, int ldc,
                        int epilogue, const int* group_offsets, int n_groups, size_t w_group_stride,
                        int rows_hint, cudaStream_t st) {
  // rows_hint: the most rows one group can have (M without groups)
  int mt = rows_hint <= 8 ? 1 : (rows_hint <= 16 ? 2 : (rows_hint <= 32 ? 4 : 8));
  if (NSUB == 2 && mt == 8) mt = 4;  // shared memory of the reduction
  dim3 grid(ceil_div(N, SM_ROWS * NSUB), ceil_div(rows_hint, 8 * mt), group_offsets ? n_groups : 1);
  if (grid.y > 65535 || grid.z > 65535) return leb_fail("leb_gemm_bf16_small: grid too large");
  dim3 block(32 * SM_WARPS);
#define LEB_SM(MT_, U_)                                                                          \
  leb_launch(gemm_bf16_small_kernel<TC, MT_, NSUB, U_>, grid, block, 0, st, (TC*)C, A, W, M, N, K, lda, \
             ldc, epilogue, group_offsets, w_group_stride)
  switch (mt) {
    case 1: {
      // blocks resident per SM for each depth (asked once), and the SM count
      static int occ[3] = {0, 0, 0}, n_sm = 0;
      if (!n_sm) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ[0], gemm_bf16_small_kernel<TC, 1, NSUB, 8>, 32 * SM_WARPS, 0);
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ[1], gemm_bf16_small_kernel<TC, 1, NSUB, 4>, 32 * SM_WARPS, 0);
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ[2], gemm_bf16_small_kernel<TC, 1, NSUB, 2>, 32 * SM_WARPS, 0);
        if (n_sm <= 0) n_sm = 148;
      }
      const long blocks = (long)grid.x * grid.y * grid.z;
      if (blocks <= (long)occ[0] * n_sm || blocks > 4L * occ[2] * n_sm) LEB_SM(1, 8);   // one wave, or many
      else if (blocks <= (long)occ[1] * n_sm) LEB_SM(1, 4);
      else LEB_SM(1, 2);
      break;
    }
    case 2: LEB_SM(2, 2); break;
    case 4: LEB_SM(4, (NSUB == 1 ? 2 : 1)); break;
    default:
      if constexpr (NSUB == 1) LEB_SM(8, 1);
      break;
  }
#undef LEB_SM
  LEB_CHECK_LAUNCH("leb_gemm_bf16_small");
  return 0;
}

LEB_API int leb_gemm_bf16_small(void* C, int c_dtype, const void* A, const void* W, int M, int N,
                                int K, int lda, int ldc, int epilogue, const int* group_offsets,
                                int n_groups, size_t w_group_stride, int rows_hint,
                                cudaStream_t st) {
  if (M <= 0 || N <= 0) return 0;
  LEB_REQUIRE(K > 0 && K % 8 == 0, "leb_gemm_bf16_small: K (%d) must be a multiple of 8", K);
  LEB_REQUIRE(lda % 8 == 0, "leb_gemm_bf16_small: row stride of A (%d) must be a multiple of 8", lda);
  LEB_REQUIRE(((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0, "leb_gemm_bf16_small: A and W must be 16-byte aligned");
  LEB_REQUIRE(epilogue >= 0 && epilogue <= 2, "leb_gemm_bf16_small: unknown epilogue %d", epilogue);
  LEB_REQUIRE(epilogue != 1 || c_dtype == LEB_F32, "leb_gemm_bf16_small: adding needs a float C");
  if (rows_hint <= 0 || rows_hint > M) rows_hint = M;
  const bf16* a = (const bf16*)A;
  const bf16* w = (const bf16*)W;
  if (epilogue == 2) {
    LEB_REQUIRE(N % 32 == 0, "leb_gemm_bf16_small: the SwiGLU epilogue needs N (%d) to be a multiple of 32", N);
    if (c_dtype == LEB_BF16)
      return launch_small<bf16, 2>(C, a, w, M, N, K, lda, ldc, 2, group_offsets, n_groups, w_group_stride, rows_hint, st);
    if (c_dtype == LEB_F32)
      return launch_small<float, 2>(C, a, w, M, N, K, lda, ldc, 2, group_offsets, n_groups, w_group_stride, rows_hint, st);
  } else {
    if (c_dtype == LEB_BF16)
      return launch_small<bf16, 1>(C, a, w, M, N, K, lda, ldc, epilogue, group_offsets, n_groups, w_group_stride, rows_hint, st);
    if (c_dtype == LEB_F32)
      return launch_small<float, 1>(C, a, w, M, N, K, lda, ldc, epilogue, group_offsets, n_groups, w_group_stride, rows_hint, st);
  }
  return leb_fail("leb_gemm_bf16_small: unknown C dtype %d", c_dtype);
}
