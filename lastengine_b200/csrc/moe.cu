// Expert routing on the device: router scores and top-k, the expert-sorted order of the
// (token, choice) pairs, and the weighted sum of the experts' outputs.  Nothing goes through
// the host (the reference groups tokens by expert on the host for its other architecture,
// src/gpu/prefill.rs:153-163).
//
// Router of this architecture: z = Wr . h (float), s = sigmoid(z), selection score c = s + bias
// (the bias chooses, it does not weigh), I = the k largest c with ties to the lower index (the
// reference's router breaks ties the same way, src/cuda/kernels.cu:450), weight_e = s_e, divided
// by the sum of the chosen s when norm_topk is set, times the scaling factor.
#include "common.cuh"

#define MOE_MAX_E 256
#define MOE_MAX_K 16

template <typename T>
__global__ void moe_router_kernel(int* __restrict__ topk_ids, float* __restrict__ topk_w,
                                  const T* __restrict__ h, const float* __restrict__ wr,
                                  const float* __restrict__ bias, int D, int E, int k, int norm_topk,
                                  float scaling) {
  extern __shared__ float sm[];  // h row as float [D], then s[E], c[E]
  float* hs = sm;
  float* s_ = hs + D;
  float* c_ = s_ + E;
  const int m = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int i = threadIdx.x; i < D; i += blockDim.x) hs[i] = to_f32(h[(size_t)m * D + i]);
  __syncthreads();
  for (int e = warp; e < E; e += nw) {
    const float* w = wr + (size_t)e * D;
    float z = 0.f;
    for (int i = lane; i < D; i += 32) z += w[i] * hs[i];
    z = warp_sum(z);
    if (lane == 0) {
      float s = 1.0f / (1.0f + expf(-z));
      s_[e] = s;
      c_[e] = s + (bias ? bias[e] : 0.f);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int ids[MOE_MAX_K];
    float sum = 0.f;
    for (int j = 0; j < k; j++) {
      int best = -1;
      float bv = 0.f;
      for (int e = 0; e < E; e++) {
        bool taken = false;
        for (int t = 0; t < j; t++) taken |= ids[t] == e;
        if (taken) continue;
        if (best < 0 || c_[e] > bv) { best = e; bv = c_[e]; }  // strict: ties keep the lower index
      }
      ids[j] = best;
      sum += s_[best];
    }
    for (int j = 0; j < k; j++) {
      float w = s_[ids[j]];
      if (norm_topk) w = w / sum;
      topk_ids[(size_t)m * k + j] = ids[j];
      topk_w[(size_t)m * k + j] = w * scaling;
    }
  }
}

LEB_API int leb_moe_router(int* topk_ids, float* topk_w, const void* h, int dtype, const float* wr,
                           const float* bias, int M, int D, int E, int k, int norm_topk,
                           float scaling, cudaStream_t st) {
  if (M <= 0) return 0;
  LEB_REQUIRE(E >= 1 && E <= MOE_MAX_E, "leb_moe_router: %d experts outside 1..%d", E, MOE_MAX_E);
  LEB_REQUIRE(k >= 1 && k <= MOE_MAX_K && k <= E, "leb_moe_router: top-%d outside 1..min(%d, experts)", k, MOE_MAX_K);
  size_t smem = ((size_t)D + 2 * E) * sizeof(float);
  LEB_REQUIRE(smem <= 48 * 1024, "leb_moe_router: hidden size %d too large for the router kernel", D);
  if (dtype == LEB_F32)
    moe_router_kernel<float><<<M, 128, smem, st>>>(topk_ids, topk_w, (const float*)h, wr, bias, D, E, k, norm_topk, scaling);
  else if (dtype == LEB_BF16)
    moe_router_kernel<bf16><<<M, 128, smem, st>>>(topk_ids, topk_w, (const bf16*)h, wr, bias, D, E, k, norm_topk, scaling);
  else
    return leb_fail("leb_moe_router: unknown dtype %d", dtype);
  LEB_CHECK_LAUNCH("leb_moe_router");
  return 0;
}

// Expert-sorted order of the P = M*k pairs (pair p = token p/k, choice p%k), stable in p:
//   offsets[e] .. offsets[e+1]  rows of expert e in the sorted order
//   sorted_pair[row] = p,  pair_row[p] = row
// One block; warp w owns experts w, w+32, ... and walks the pairs in order with a ballot, so the
// order is fixed without atomics.
__global__ void moe_align_kernel(int* __restrict__ offsets, int* __restrict__ sorted_pair,
                                 int* __restrict__ pair_row, const int* __restrict__ topk_ids,
                                 int P, int E) {
  __shared__ int counts[MOE_MAX_E + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int e = warp; e < E; e += nw) {
    int cnt = 0;
    for (int p0 = 0; p0 < P; p0 += 32) {
      int p = p0 + lane;
      bool mine = p < P && topk_ids[p] == e;
      cnt += __popc(__ballot_sync(0xffffffffu, mine));
    }
    if (lane == 0) counts[e] = cnt;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; e++) {
      int c = counts[e];
      counts[e] = run;
      offsets[e] = run;
      run += c;
    }
    counts[E] = run;
    offsets[E] = run;
  }
  __syncthreads();
  for (int e = warp; e < E; e += nw) {
    int base = counts[e];
    for (int p0 = 0; p0 < P; p0 += 32) {
      int p = p0 + lane;
      bool mine = p < P && topk_ids[p] == e;
      unsigned mask = __ballot_sync(0xffffffffu, mine);
      if (mine) {
        int row = base + __popc(mask & ((1u << lane) - 1u));
        sorted_pair[row] = p;
        pair_row[p] = row;
      }
      base += __popc(mask);
    }
  }
}

LEB_API int leb_moe_align(int* offsets, int* sorted_pair, int* pair_row, const int* topk_ids, int P,
                          int E, cudaStream_t st) {
  LEB_REQUIRE(E >= 1 && E <= MOE_MAX_E, "leb_moe_align: %d experts outside 1..%d", E, MOE_MAX_E);
  if (P < 0) return leb_fail("leb_moe_align: negative pair count");
  moe_align_kernel<<<1, 1024, 0, st>>>(offsets, sorted_pair, pair_row, topk_ids, P, E);
  LEB_CHECK_LAUNCH("leb_moe_align");
  return 0;
}

// x[m, :] (+)= sum_j w[m, j] * ys[pair_row[m*k + j], :]   in the order j = 0..k-1, float.
__global__ void moe_combine_kernel(float* __restrict__ x, const float* __restrict__ ys,
                                   const int* __restrict__ pair_row, const float* __restrict__ topk_w,
                                   int D, int k, int accumulate) {
  const size_t m = blockIdx.x;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float a = 0.f;
    for (int j = 0; j < k; j++)
      a += topk_w[m * k + j] * ys[(size_t)pair_row[m * k + j] * D + i];
    float* o = x + m * D + i;
    *o = accumulate ? *o + a : a;
  }
}

LEB_API int leb_moe_combine(float* x, const float* ys, const int* pair_row, const float* topk_w,
                            int M, int D, int k, int accumulate, cudaStream_t st) {
  if (M <= 0) return 0;
  moe_combine_kernel<<<M, 256, 0, st>>>(x, ys, pair_row, topk_w, D, k, accumulate);
  LEB_CHECK_LAUNCH("leb_moe_combine");
  return 0;
}
