// True 32-bit matrix product on the CUDA cores:  C[M,N] (+)= A[M,K] . W[N,K]^T.
//
// FFMA only: no tensor cores, no TF32, no reduced-precision mode of any kind.  Every output
// element is one thread's sum over k = 0..K-1 in ascending order, whatever M is, so a row's
// result does not depend on which other rows share the launch: a token gives the same bits
// in a prompt, alone, or in a batch.  (The reference's all-float path is its CPU forward,
// src/dense.rs:94-102, one dot product per output row.)
//
// Weights are [N,K] row-major as in the reference (src/dense.rs:96).  With group_offsets the
// rows of A and C are grouped by expert: group e owns rows [off[e], off[e+1]) and the weight
// matrix W + e * w_group_stride.
#include "common.cuh"

#define F32_BM 64
#define F32_BN 64
#define F32_BK 16

__global__ void __launch_bounds__(256)
gemm_f32_kernel(float* __restrict__ C, const float* __restrict__ A, const float* __restrict__ W,
                int M, int N, int K, int lda, int ldc, int accumulate,
                const int* __restrict__ group_offsets, size_t w_group_stride) {
  __shared__ float As[F32_BK][F32_BM + 4];
  __shared__ float Ws[F32_BK][F32_BN + 4];
  int row_begin = 0, row_end = M;
  if (group_offsets) {
    row_begin = group_offsets[blockIdx.z];
    row_end = group_offsets[blockIdx.z + 1];
    W += (size_t)blockIdx.z * w_group_stride;
  }
  const int m0 = row_begin + blockIdx.y * F32_BM;
  if (m0 >= row_end) return;
  const int n0 = blockIdx.x * F32_BN;
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int lrow = tid >> 2, lk = (tid & 3) * 4;  // loader: row of the tile, first of 4 k

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += F32_BK) {
    {
      const int r = m0 + lrow;
      const float* src = A + (size_t)r * lda + k0 + lk;
#pragma unroll
      for (int e = 0; e < 4; e++) As[lk + e][lrow] = (r < row_end && k0 + lk + e < K) ? src[e] : 0.f;
      const int n = n0 + lrow;
      const float* wsrc = W + (size_t)n * K + k0 + lk;
#pragma unroll
      for (int e = 0; e < 4; e++) Ws[lk + e][lrow] = (n < N && k0 + lk + e < K) ? wsrc[e] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < F32_BK; kk++) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; i++) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; j++) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int r = m0 + ty * 4 + i;
    if (r >= row_end) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float* c = C + (size_t)r * ldc + n;
      *c = accumulate ? *c + acc[i][j] : acc[i][j];
    }
  }
}

LEB_API int leb_gemm_f32(float* C, const float* A, const float* W, int M, int N, int K, int lda,
                         int ldc, int accumulate, const int* group_offsets, int n_groups,
                         size_t w_group_stride, cudaStream_t st) {
  if (M <= 0 || N <= 0) return 0;
  LEB_REQUIRE(K > 0, "leb_gemm_f32: K must be positive");
  dim3 grid(ceil_div(N, F32_BN), ceil_div(M, F32_BM), group_offsets ? n_groups : 1);
  LEB_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "leb_gemm_f32: too many row tiles (%u) or groups (%u)", grid.y, grid.z);
  gemm_f32_kernel<<<grid, 256, 0, st>>>(C, A, W, M, N, K, lda, ldc, accumulate, group_offsets,
                                        w_group_stride);
  LEB_CHECK_LAUNCH("leb_gemm_f32");
  return 0;
}
