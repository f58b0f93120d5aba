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

// One row's choice by one warp: the k largest selection scores c, ties to the lower index; the
// weights are the sigmoids sg of the chosen, divided by their sum when norm_topk is set, times scaling.
__device__ __forceinline__ void router_choose(int* __restrict__ ids, float* __restrict__ wts, const float* c,
                                              const float* sg, int E, int k, int norm_topk, float scaling, int lane) {
  unsigned taken = 0;   // bit j: this lane's candidate lane + 32 j is chosen already
  int chosen[MOE_MAX_K];
  float sum = 0.f;
  for (int j = 0; j < k; j++) {
    float bv = -INFINITY;
    int be = 0x7fffffff;
    for (int q = 0; lane + 32 * q < E; q++) {
      const int e = lane + 32 * q;
      if (!((taken >> q) & 1u) && (c[e] > bv || be == 0x7fffffff)) { bv = c[e]; be = e; }   // ascending e: ties keep the lower
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (oe != 0x7fffffff && (be == 0x7fffffff || ov > bv || (ov == bv && oe < be))) { bv = ov; be = oe; }
    }
    if ((be & 31) == lane) taken |= 1u << (be >> 5);
    chosen[j] = be;
    sum += sg[be];
  }
  if (lane == 0) {
    for (int j = 0; j < k; j++) {
      float w = sg[chosen[j]];
      if (norm_topk) w = w / sum;
      ids[j] = chosen[j];
      wts[j] = w * scaling;
    }
  }
}

// A block takes R rows; warp w takes experts w, w + warps, ...: it reads the expert's router row
// once (16-byte loads when D is a multiple of 4) and forms the dot product with each of the R
// rows, so a single row costs one pass of one warp per expert, all experts at once, and many rows
// share the router's weights R at a time.  A lane's partial sum runs over elements lane, lane +
// 32, ... (in pieces of VEC), whatever R and the number of rows are: a row's scores do not
// depend on the rows around it.  The top k are then found by warp 0 with shuffles.
template <typename T, int R, int VEC>
__global__ void __launch_bounds__(1024)
moe_router_kernel(int* __restrict__ topk_ids, float* __restrict__ topk_w, const T* __restrict__ h,
                  const float* __restrict__ wr, const float* __restrict__ bias, int M, int D, int E, int k,
                  int norm_topk, float scaling) {
  extern __shared__ __align__(16) float sm[];  // R rows of h as float [R][D], then s[R][E], c[R][E]
  float* hs = sm;
  float* s_ = hs + (size_t)R * D;
  float* c_ = s_ + R * E;
  pdl_trigger();   // the kernel after this one may start and wait (see common.cuh)
  pdl_wait();
  const int m0 = blockIdx.x * R;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int i = threadIdx.x; i < R * D; i += blockDim.x) {
    const int r = i / D;
    hs[i] = m0 + r < M ? to_f32(h[(size_t)(m0 + r) * D + (i - r * D)]) : 0.f;
  }
  __syncthreads();
  for (int e = warp; e < E; e += nw) {
    const float* w = wr + (size_t)e * D;
    float z[R];
#pragma unroll
    for (int r = 0; r < R; r++) z[r] = 0.f;
    if (VEC == 4) {
      // eight pieces of the router row are asked for before the first is used: a loop that fetched
      // a piece and used it spent a round trip to L2 on each (16 of them for a width of 2,048)
      const float4* w4 = reinterpret_cast<const float4*>(w);
      const int n4 = D / 4;
      for (int i0 = lane; i0 < n4; i0 += 32 * 8) {
        float4 a[8];
#pragma unroll
        for (int u = 0; u < 8; u++) a[u] = i0 + 32 * u < n4 ? w4[i0 + 32 * u] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int u = 0; u < 8; u++) {
          const int i = i0 + 32 * u;
          if (i >= n4) break;
#pragma unroll
          for (int r = 0; r < R; r++) {
            const float4 x = reinterpret_cast<const float4*>(hs + (size_t)r * D)[i];
            z[r] += a[u].x * x.x;
            z[r] += a[u].y * x.y;
            z[r] += a[u].z * x.z;
            z[r] += a[u].w * x.w;
          }
        }
      }
    } else {
      for (int i = lane; i < D; i += 32) {
        const float a = w[i];
#pragma unroll
        for (int r = 0; r < R; r++) z[r] += a * hs[(size_t)r * D + i];
      }
    }
#pragma unroll
    for (int r = 0; r < R; r++) {
      const float zz = warp_sum(z[r]);
      if (lane == 0) {
        const float sg = 1.0f / (1.0f + expf(-zz));
        s_[r * E + e] = sg;
        c_[r * E + e] = sg + (bias ? bias[e] : 0.f);
      }
    }
  }
  __syncthreads();
  // the k largest c of each row, ties to the lower index: warp r' takes rows r', r' + warps, ...
  for (int r = warp; r < R; r += nw) {
    if (m0 + r >= M) continue;
    router_choose(topk_ids + (size_t)(m0 + r) * k, topk_w + (size_t)(m0 + r) * k, c_ + r * E, s_ + r * E, E, k, norm_topk,
                  scaling, lane);
  }
}

// The same router for the many rows of a prompt: a block of 8 warps takes RB rows (kept in shared
// memory as they come), and a warp takes four experts at a time for all RB rows, so that one
// piece of a router row from L2 and one piece of a row of h from shared memory feed 4 x RB
// multiply-adds (the form above issues a load for every four; with thousands of rows it is bound by
// its instructions, 45 us for 2,048 rows of 2,048 and 32 experts).  A lane's partial sums run over
// the same elements in the same order as above and are added up by the same shuffles: the same bits.
template <typename T, int RB>
__global__ void __launch_bounds__(256)
moe_router_rows_kernel(int* __restrict__ topk_ids, float* __restrict__ topk_w, const T* __restrict__ h,
                       const float* __restrict__ wr, const float* __restrict__ bias, int M, int D, int E, int k,
                       int norm_topk, float scaling) {
  extern __shared__ __align__(16) unsigned char rsm[];
  T* hs = reinterpret_cast<T*>(rsm);                                   // [RB][D] as stored
  float* s_ = reinterpret_cast<float*>(rsm + (size_t)RB * D * sizeof(T));
  float* c_ = s_ + RB * E;
  pdl_trigger();   // the kernel after this one may start and wait (see common.cuh)
  pdl_wait();
  const int m0 = blockIdx.x * RB;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  {
    constexpr int PER = 16 / sizeof(T);            // elements of a 16-byte piece
    const int pieces = D / PER;
    for (int i = threadIdx.x; i < RB * pieces; i += blockDim.x) {
      const int r = i / pieces, pc = i - r * pieces;
      reinterpret_cast<uint4*>(hs)[i] = m0 + r < M ? reinterpret_cast<const uint4*>(h + (size_t)(m0 + r) * D)[pc]
                                                   : make_uint4(0, 0, 0, 0);
    }
  }
  __syncthreads();
  const int n4 = D / 4;
  for (int eb = 0; eb < E; eb += 32) {
    const float4* wq[4];
    bool on[4];
#pragma unroll
    for (int q = 0; q < 4; q++) {
      const int e = eb + warp + 8 * q;
      on[q] = e < E;
      wq[q] = reinterpret_cast<const float4*>(wr + (size_t)(on[q] ? e : 0) * D);
    }
    float z[4][RB];
#pragma unroll
    for (int q = 0; q < 4; q++)
#pragma unroll
      for (int r = 0; r < RB; r++) z[q][r] = 0.f;
    float4 nxt[4];
#pragma unroll
    for (int q = 0; q < 4; q++) nxt[q] = lane < n4 ? wq[q][lane] : make_float4(0.f, 0.f, 0.f, 0.f);
    for (int i = lane; i < n4; i += 32) {
      float4 a[4];
#pragma unroll
      for (int q = 0; q < 4; q++) a[q] = nxt[q];
      if (i + 32 < n4) {
#pragma unroll
        for (int q = 0; q < 4; q++) nxt[q] = wq[q][i + 32];      // the next pieces travel under this one's products
      }
#pragma unroll
      for (int r = 0; r < RB; r++) {
        float4 x;
        if (sizeof(T) == 2) {
          const uint2 raw = reinterpret_cast<const uint2*>(hs + (size_t)r * D)[i];
          x = make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                          __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
        } else {
          x = reinterpret_cast<const float4*>(hs + (size_t)r * D)[i];
        }
#pragma unroll
        for (int q = 0; q < 4; q++) {
          z[q][r] += a[q].x * x.x;
          z[q][r] += a[q].y * x.y;
          z[q][r] += a[q].z * x.z;
          z[q][r] += a[q].w * x.w;
        }
      }
    }
#pragma unroll
    for (int q = 0; q < 4; q++) {
      const int e = eb + warp + 8 * q;
#pragma unroll
      for (int r = 0; r < RB; r++) {
        const float zz = warp_sum(z[q][r]);
        if (lane == 0 && on[q]) {
          const float sg = 1.0f / (1.0f + expf(-zz));
          s_[r * E + e] = sg;
          c_[r * E + e] = sg + (bias ? bias[e] : 0.f);
        }
      }
    }
  }
  __syncthreads();
  for (int r = warp; r < RB; r += 8) {
    if (m0 + r >= M) continue;
    router_choose(topk_ids + (size_t)(m0 + r) * k, topk_w + (size_t)(m0 + r) * k, c_ + r * E, s_ + r * E, E, k, norm_topk,
                  scaling, lane);
  }
}

LEB_API int leb_moe_router(int* topk_ids, float* topk_w, const void* h, int dtype, const float* wr,
                           const float* bias, int M, int D, int E, int k, int norm_topk,
                           float scaling, cudaStream_t st) {
  if (M <= 0) return 0;
  LEB_REQUIRE(E >= 1 && E <= MOE_MAX_E, "leb_moe_router: %d experts outside 1..%d", E, MOE_MAX_E);
  LEB_REQUIRE(k >= 1 && k <= MOE_MAX_K && k <= E, "leb_moe_router: top-%d outside 1..min(%d, experts)", k, MOE_MAX_K);
  // many rows (prompts): blocks of 4 rows (8 from 4,096 rows on) with four experts per warp
  // (2,048 rows of 2,048 and 32 experts: 25 us with 4 rows a block, 31 with 8, 41 with 16; 8,192 rows: 73, 67, 81)
  {
    const size_t esz = dtype == LEB_BF16 ? 2 : 4;
    const int rb = M >= 4096 ? 8 : 4;
    const size_t smem_rows = (size_t)rb * D * esz + (size_t)2 * rb * E * sizeof(float);
    if (M > sm_count() && D % 8 == 0 && ((uintptr_t)wr & 15) == 0 && ((uintptr_t)h & 15) == 0 &&
        smem_rows <= 100 * 1024 && (dtype == LEB_BF16 || dtype == LEB_F32)) {
#define LEB_ROUTER_ROWS(T_, RB_)                                                                                    \
  {                                                                                                                \
    static bool set = false;                                                                                       \
    if (!set) {                                                                                                    \
      if (cudaFuncSetAttribute(moe_router_rows_kernel<T_, RB_>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024) != cudaSuccess) \
        return leb_fail("leb_moe_router: %zu bytes of shared memory per block refused", smem_rows);              \
      set = true;                                                                                                  \
    }                                                                                                              \
    leb_launch(moe_router_rows_kernel<T_, RB_>, dim3(ceil_div(M, RB_)), dim3(256), smem_rows, st, topk_ids, topk_w, \
               (const T_*)h, wr, bias, M, D, E, k, norm_topk, scaling);                                            \
  }
      if (dtype == LEB_BF16) { if (rb == 8) LEB_ROUTER_ROWS(bf16, 8) else LEB_ROUTER_ROWS(bf16, 4) }
      else { if (rb == 8) LEB_ROUTER_ROWS(float, 8) else LEB_ROUTER_ROWS(float, 4) }
#undef LEB_ROUTER_ROWS
      LEB_CHECK_LAUNCH("leb_moe_router");
      return 0;
    }
  }
  // rows per block: 1 while every row can have an SM of its own (a block's pace is set by one SM
  // reading the router's weights), 4 for many rows when they fit shared memory
  const bool four = M > sm_count() && ((size_t)4 * D + 8 * E) * sizeof(float) <= 48 * 1024;
  const int R = four ? 4 : 1;
  const size_t smem = ((size_t)R * D + 2 * R * E) * sizeof(float);
  LEB_REQUIRE(smem <= 48 * 1024, "leb_moe_router: hidden size %d too large for the router kernel", D);
  const bool vec = D % 4 == 0 && ((uintptr_t)wr & 15) == 0;
  const dim3 grid(ceil_div(M, R)), block(32 * (E < 32 ? E : 32));
#define LEB_ROUTER(T_, R_, V_) \
  leb_launch(moe_router_kernel<T_, R_, V_>, grid, block, smem, st, topk_ids, topk_w, (const T_*)h, wr, bias, M, D, E, k, norm_topk, scaling)
  if (dtype == LEB_F32) {
    if (four) { if (vec) LEB_ROUTER(float, 4, 4); else LEB_ROUTER(float, 4, 1); }
    else { if (vec) LEB_ROUTER(float, 1, 4); else LEB_ROUTER(float, 1, 1); }
  } else if (dtype == LEB_BF16) {
    if (four) { if (vec) LEB_ROUTER(bf16, 4, 4); else LEB_ROUTER(bf16, 4, 1); }
    else { if (vec) LEB_ROUTER(bf16, 1, 4); else LEB_ROUTER(bf16, 1, 1); }
  } else {
    return leb_fail("leb_moe_router: unknown dtype %d", dtype);
  }
#undef LEB_ROUTER
  LEB_CHECK_LAUNCH("leb_moe_router");
  return 0;
}

// Expert-sorted order of the P = M*k pairs (pair p = token p/k, choice p%k), stable in p:
//   offsets[e] .. offsets[e+1]  rows of expert e in the sorted order
//   sorted_pair[row] = p,  pair_row[p] = row
// One block of 32 warps, a counting sort without atomics: warp w owns the pairs of chunk w (in
// order), counts them per expert with __match_any_sync (lanes with the same expert find each other;
// the first of them adds their number), the counts are turned into the first row of every
// (warp, expert), and a second walk gives every pair its row: first row + pairs of the same
// expert before it.  The order within an expert is the order of the pairs, run after run.
__global__ void __launch_bounds__(1024)
moe_align_kernel(int* __restrict__ offsets, int* __restrict__ sorted_pair, int* __restrict__ pair_row,
                 const int* __restrict__ topk_ids, int P, int E) {
  __shared__ int cnt[32][MOE_MAX_E];
  pdl_trigger();   // the kernel after this one may start and wait (see common.cuh)
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int chunk = ((P + 31) / 32 + 31) / 32 * 32;   // pairs per warp, a multiple of 32
  const int lo = warp * chunk, hi = min(P, lo + chunk);
  for (int e = lane; e < E; e += 32) cnt[warp][e] = 0;
  __syncwarp();
  for (int p0 = lo; p0 < hi; p0 += 32) {
    const int p = p0 + lane;
    const bool valid = p < hi;
    const int id = valid ? topk_ids[p] : -1 - lane;   // lanes past the end match nobody
    const unsigned same = __match_any_sync(0xffffffffu, id);
    if (valid && lane == __ffs(same) - 1) cnt[warp][id] += __popc(same);
    __syncwarp();
  }
  __syncthreads();
  // thread e: the experts' totals, then (thread 0) their first rows, then the first row of each warp's share
  __shared__ int first[MOE_MAX_E + 1];
  if ((int)threadIdx.x < E) {
    int t = 0;
    for (int w = 0; w < 32; w++) t += cnt[w][threadIdx.x];
    first[threadIdx.x] = t;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; e++) {
      const int c = first[e];
      first[e] = run;
      offsets[e] = run;
      run += c;
    }
    first[E] = run;
    offsets[E] = run;
  }
  __syncthreads();
  if ((int)threadIdx.x < E) {
    int run = first[threadIdx.x];
    for (int w = 0; w < 32; w++) {
      const int c = cnt[w][threadIdx.x];
      cnt[w][threadIdx.x] = run;
      run += c;
    }
  }
  __syncthreads();
  for (int p0 = lo; p0 < hi; p0 += 32) {
    const int p = p0 + lane;
    const bool valid = p < hi;
    const int id = valid ? topk_ids[p] : -1 - lane;
    const unsigned same = __match_any_sync(0xffffffffu, id);
    if (valid) {
      const int row = cnt[warp][id] + __popc(same & ((1u << lane) - 1u));
      sorted_pair[row] = p;
      pair_row[p] = row;
    }
    __syncwarp();   // everyone has read its first row before the first of each expert moves it on
    if (valid && lane == __ffs(same) - 1) cnt[warp][id] += __popc(same);
    __syncwarp();
  }
}

LEB_API int leb_moe_align(int* offsets, int* sorted_pair, int* pair_row, const int* topk_ids, int P,
                          int E, cudaStream_t st) {
  LEB_REQUIRE(E >= 1 && E <= MOE_MAX_E, "leb_moe_align: %d experts outside 1..%d", E, MOE_MAX_E);
  if (P < 0) return leb_fail("leb_moe_align: negative pair count");
  leb_launch(moe_align_kernel, dim3(1), dim3(1024), 0, st, offsets, sorted_pair, pair_row, topk_ids, P, E);
  LEB_CHECK_LAUNCH("leb_moe_align");
  return 0;
}

// x[m, :] (+)= sum_j w[m, j] * ys[pair_row[m*k + j], :]   in the order j = 0..k-1, float.
// A thread owns VEC consecutive columns of one token; the token's k rows and weights are read
// first and then all k pieces of ys are asked for before any is used, so the kernel costs two
// trips to memory whatever k is.
template <int VEC, int KMAX>   // columns a thread owns; the most rows per token (k <= KMAX)
__global__ void __launch_bounds__(256)
moe_combine_kernel(float* __restrict__ x, const float* __restrict__ ys, const int* __restrict__ pair_row,
                   const float* __restrict__ topk_w, int D, int k, int accumulate) {
  pdl_trigger();   // the kernel after this one may start and wait (see common.cuh)
  pdl_wait();
  const size_t m = blockIdx.x;
  const int i = (blockIdx.y * blockDim.x + threadIdx.x) * VEC;
  if (i >= D) return;
  int row[KMAX];
  float w[KMAX], old[VEC], v[KMAX][VEC];
#pragma unroll
  for (int j = 0; j < KMAX; j++) {
    row[j] = j < k ? pair_row[m * k + j] : 0;
    w[j] = j < k ? topk_w[m * k + j] : 0.f;
  }
  float* o = x + m * D + i;
  if (VEC == 4) {
    const float4 t = accumulate ? *reinterpret_cast<const float4*>(o) : make_float4(0.f, 0.f, 0.f, 0.f);
    old[0] = t.x; old[1 % VEC] = t.y; old[2 % VEC] = t.z; old[3 % VEC] = t.w;
  } else {
    old[0] = accumulate ? *o : 0.f;
  }
#pragma unroll
  for (int j = 0; j < KMAX; j++) {
    if (j < k) {
      const float* p = ys + (size_t)row[j] * D + i;
      if (VEC == 4) {
        const float4 t = __ldcs(reinterpret_cast<const float4*>(p));     // read once: no need to keep it in L2
        v[j][0] = t.x; v[j][1 % VEC] = t.y; v[j][2 % VEC] = t.z; v[j][3 % VEC] = t.w;
      } else {
        v[j][0] = *p;
      }
    }
  }
  float a[VEC];
#pragma unroll
  for (int e = 0; e < VEC; e++) a[e] = 0.f;
#pragma unroll
  for (int j = 0; j < KMAX; j++)
    if (j < k)
#pragma unroll
      for (int e = 0; e < VEC; e++) a[e] += w[j] * v[j][e];
  if (VEC == 4)
    *reinterpret_cast<float4*>(o) = accumulate ? make_float4(old[0] + a[0], old[1 % VEC] + a[1 % VEC], old[2 % VEC] + a[2 % VEC], old[3 % VEC] + a[3 % VEC])
                                               : make_float4(a[0], a[1 % VEC], a[2 % VEC], a[3 % VEC]);
  else
    *o = accumulate ? old[0] + a[0] : a[0];
}

LEB_API int leb_moe_combine(float* x, const float* ys, const int* pair_row, const float* topk_w,
                            int M, int D, int k, int accumulate, cudaStream_t st) {
  if (M <= 0) return 0;
  LEB_REQUIRE(k >= 1 && k <= MOE_MAX_K, "leb_moe_combine: %d rows per token outside 1..%d", k, MOE_MAX_K);
  if (D % 4 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)ys & 15) == 0) {
    // up to four rows per token (the usual case) with arrays of four: fewer registers, more blocks per SM
    if (k <= 4) leb_launch(moe_combine_kernel<4, 4>, dim3(M, ceil_div(D, 1024)), dim3(256), 0, st, x, ys, pair_row, topk_w, D, k, accumulate);
    else leb_launch(moe_combine_kernel<4, MOE_MAX_K>, dim3(M, ceil_div(D, 1024)), dim3(256), 0, st, x, ys, pair_row, topk_w, D, k, accumulate);
  } else {
    leb_launch(moe_combine_kernel<1, MOE_MAX_K>, dim3(M, ceil_div(D, 256)), dim3(256), 0, st, x, ys, pair_row, topk_w, D, k, accumulate);
  }
  LEB_CHECK_LAUNCH("leb_moe_combine");
  return 0;
}
