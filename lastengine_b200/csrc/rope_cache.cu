// Per-head RMSNorm on q and k, rotary position encoding, and the write of k and v into the
// paged cache, one launch for all rows of a step.
//
// Order as in the reference (src/dense.rs:119-128): norm each head of q and k over head_dim with
// the shared [head_dim] weights and the model's eps, then rotate, then append k and v at the
// token's position.  Rotation (src/dense.rs:103-111): half = rope_dim/2, angle_i = pos * inv_freq[i]
// with inv_freq[i] = theta^(-2i/rope_dim) (divided by a frequency factor where the model has one);
// split-half pairing (i, i+half) or adjacent pairing (2i, 2i+1); a' = a cos - b sin,
// b' = a sin + b cos.  The reference does the three jobs in one decode launch too
// (src/cuda/dense.cu:80-93); here the same launch also serves prompts.
// Norm, angle, sine and cosine are float; sinf/cosf are the full-range versions.
//
// Cache layout of one layer: keys [page][kv_head][page_size][head_dim]; values transposed,
// [page][kv_head][head_dim][page_size], so that the positions of a page are contiguous for each
// dimension (the tensor-core attention kernels contract over positions and read them 8 at a
// time).  The page of position p of sequence b is block_table[b][p / page_size].
#include "common.cuh"

constexpr int ROPE_WARPS = 8;   // warps of a block; each takes one head of the block's row
constexpr int VT_ROWS = 32;     // rows of a value tile
constexpr int VT_DIMS = 64;     // dimensions of a value tile

// A tile of VT_ROWS rows of one kv head's values, turned through shared memory so that a warp
// writes 32 consecutive positions of one dimension (64 bytes in bfloat16) instead of 32
// scattered elements.  Every row's page and offset is looked up on its own, so rows of
// different sequences or pages in one tile are fine.
template <typename T, typename CT>
__device__ __forceinline__ void store_value_tile(
    int t, const T* __restrict__ v_in, int kv_stride, CT* __restrict__ v_pool,
    const int* __restrict__ block_table, int bt_width, const int* __restrict__ row_seq,
    const int* __restrict__ row_pos, const int* __restrict__ seq_slot, int M, int nkv, int hd,
    int page_size) {
  constexpr int LD = VT_DIMS + (sizeof(CT) == 2 ? 2 : 1);     // odd number of 32-bit words
  __shared__ CT tile[VT_ROWS * LD];
  __shared__ long long dst[VT_ROWS];                          // element offset of (row, dim 0), or -1
  const int kvh = t % nkv, m0 = (t / nkv) * VT_ROWS;
  if (threadIdx.x < VT_ROWS) {
    int m = m0 + threadIdx.x;
    long long off = -1;
    if (m < M) {
      int b = row_seq[m], pos = row_pos[m];
      if (seq_slot[b] >= 0) {
        int page = block_table[(size_t)b * bt_width + pos / page_size];
        if (page >= 0) off = ((long long)page * nkv + kvh) * hd * page_size + pos % page_size;
      }
    }
    dst[threadIdx.x] = off;
  }
  for (int d0 = 0; d0 < hd; d0 += VT_DIMS) {
    int nd = min(VT_DIMS, hd - d0);
    __syncthreads();
    for (int i = threadIdx.x; i < VT_ROWS * VT_DIMS; i += blockDim.x) {
      int r = i / VT_DIMS, d = i % VT_DIMS;
      if (d < nd && m0 + r < M)
        tile[r * LD + d] = from_f32<CT>(to_f32(v_in[(size_t)(m0 + r) * kv_stride + (size_t)kvh * hd + d0 + d]));
    }
    __syncthreads();
    for (int i = threadIdx.x; i < VT_ROWS * VT_DIMS; i += blockDim.x) {
      int d = i / VT_ROWS, r = i % VT_ROWS;
      if (d < nd && dst[r] >= 0) v_pool[dst[r] + (size_t)(d0 + d) * page_size] = tile[r * LD + d];
    }
  }
}

// Blocks (x < M, y): row x, heads [8y, 8y + 8) of its q and k heads, one per warp: norm, rotate
// (sine and cosine of the row's position are computed once per block, not per head), write q
// and the cached k.  Blocks (x in [M, M + tiles * nkv), y = 0): a value tile.
template <typename T, typename CT>
__global__ void __launch_bounds__(ROPE_WARPS * 32) qk_rope_store_kernel(
    T* __restrict__ q_out, const T* __restrict__ q_in, int q_stride, const T* __restrict__ k_in,
    const T* __restrict__ v_in, int kv_stride, CT* __restrict__ k_pool, CT* __restrict__ v_pool,
    const int* __restrict__ block_table, int bt_width, const int* __restrict__ row_seq,
    const int* __restrict__ row_pos, const int* __restrict__ seq_slot,
    const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w, float eps,
    const float* __restrict__ inv_freq, int rope_dim, int neox, int M, int nh, int nkv, int hd,
    int page_size) {
  extern __shared__ float sm[];
  pdl_trigger();   // the kernel after this one may start and wait (see common.cuh)
  pdl_wait();
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if ((int)blockIdx.x >= M) {
    if (blockIdx.y == 0)
      store_value_tile<T, CT>(blockIdx.x - M, v_in, kv_stride, v_pool, block_table, bt_width, row_seq, row_pos,
                              seq_slot, M, nkv, hd, page_size);
    return;
  }
  // ---- one row: q and k heads ----
  int m = blockIdx.x;
  int b = row_seq[m];
  int slot = seq_slot[b];
  int pos = row_pos[m];
  int half = rope_dim / 2;
  float* cs = sm;                                   // [half] cosine, [half] sine
  float* v = sm + 2 * half + warp * hd;             // one head vector per warp
  if (inv_freq) {
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
      float th = (float)pos * inv_freq[i];
      cs[i] = cosf(th);
      cs[half + i] = sinf(th);
    }
  }
  __syncthreads();
  int total = nh + (k_in ? nkv : 0);
  long long kdst = -1;
  if (k_in && slot >= 0) {
    int page = block_table[(size_t)b * bt_width + pos / page_size];
    if (page >= 0) kdst = ((long long)page * nkv * page_size + pos % page_size) * hd;
  }
  int head = blockIdx.y * ROPE_WARPS + warp;
  if (head < total) {
    bool is_q = head < nh;
    if (!is_q && kdst < 0) return;  // padding rows and positions outside a window own no cache
    const T* src = is_q ? q_in + (size_t)m * q_stride + (size_t)head * hd
                        : k_in + (size_t)m * kv_stride + (size_t)(head - nh) * hd;
    const float* nw = is_q ? q_norm_w : k_norm_w;
    float ss = 0.f;
    for (int i = lane; i < hd; i += 32) {
      float x = to_f32(src[i]);
      v[i] = x;
      ss += x * x;
    }
    if (nw) {
      ss = warp_sum(ss);
      float r = 1.0f / sqrtf(ss / (float)hd + eps);
      __syncwarp();
      for (int i = lane; i < hd; i += 32) v[i] = v[i] * r * nw[i];
    }
    __syncwarp();
    if (inv_freq) {
      for (int i = lane; i < half; i += 32) {
        float c = cs[i], s = cs[half + i];
        int ia = neox ? i : 2 * i, ib = neox ? i + half : 2 * i + 1;
        float a = v[ia], bb = v[ib];
        v[ia] = a * c - bb * s;
        v[ib] = a * s + bb * c;
      }
    }
    __syncwarp();
    if (is_q) {
      T* o = q_out + ((size_t)m * nh + head) * hd;
      for (int i = lane; i < hd; i += 32) o[i] = from_f32<T>(v[i]);
    } else {
      CT* o = k_pool + kdst + (size_t)(head - nh) * page_size * hd;
      for (int i = lane; i < hd; i += 32) o[i] = from_f32<CT>(v[i]);
    }
  }
}

// The usual case (split-half pairing over the whole head, head size 64 or 128) without shared
// memory: a lane holds elements lane, lane + 32, ... of a head, so both halves of a rotation
// pair are in the same lane.  A warp takes `per_warp` consecutive heads of its row, four at a
// time so that their loads are in flight together; sine and cosine are formed once per warp.
// Same operations in the same order as the kernel above: the results are the same bit for bit.
template <typename T, typename CT, int EPL>
__global__ void __launch_bounds__(ROPE_WARPS * 32) qk_rope_store_lanes_kernel(
    T* __restrict__ q_out, const T* __restrict__ q_in, int q_stride, const T* __restrict__ k_in,
    const T* __restrict__ v_in, int kv_stride, CT* __restrict__ k_pool, CT* __restrict__ v_pool,
    const int* __restrict__ block_table, int bt_width,
    const int* __restrict__ row_seq, const int* __restrict__ row_pos, const int* __restrict__ seq_slot,
    const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w, float eps,
    const float* __restrict__ inv_freq, int M, int nh, int nkv, int page_size, int per_warp) {
  constexpr int HD = EPL * 32, NP = EPL / 2, U = 4;
  pdl_trigger();   // the kernel after this one may start and wait (see common.cuh)
  pdl_wait();
  if ((int)blockIdx.x >= M) {
    if (blockIdx.y == 0)
      store_value_tile<T, CT>(blockIdx.x - M, v_in, kv_stride, v_pool, block_table, bt_width, row_seq, row_pos,
                              seq_slot, M, nkv, HD, page_size);
    return;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int m = blockIdx.x;
  const int total = nh + (k_in ? nkv : 0);
  const int h0 = (blockIdx.y * ROPE_WARPS + warp) * per_warp;
  if (h0 >= total) return;
  const int h1 = min(h0 + per_warp, total);
  const int b = row_seq[m], pos = row_pos[m];
  long long kdst = -1;
  if (h1 > nh && seq_slot[b] >= 0) {
    const int page = block_table[(size_t)b * bt_width + pos / page_size];
    if (page >= 0) kdst = ((long long)page * nkv * page_size + pos % page_size) * HD;
  }
  float c[NP], sn[NP], wq[EPL], wk[EPL];
#pragma unroll
  for (int p = 0; p < NP; p++) {
    const float th = (float)pos * inv_freq[lane + 32 * p];
    c[p] = cosf(th);
    sn[p] = sinf(th);
  }
#pragma unroll
  for (int e = 0; e < EPL; e++) {
    wq[e] = q_norm_w ? q_norm_w[lane + 32 * e] : 1.f;
    wk[e] = k_norm_w ? k_norm_w[lane + 32 * e] : 1.f;
  }
  for (int hb = h0; hb < h1; hb += U) {
    float x[U][EPL];
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int head = hb + u;
      if (head < h1) {
        const T* src = head < nh ? q_in + (size_t)m * q_stride + (size_t)head * HD
                                 : k_in + (size_t)m * kv_stride + (size_t)(head - nh) * HD;
#pragma unroll
        for (int e = 0; e < EPL; e++) x[u][e] = to_f32(src[lane + 32 * e]);
      } else {
#pragma unroll
        for (int e = 0; e < EPL; e++) x[u][e] = 0.f;
      }
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int head = hb + u;
      if (head >= h1) break;
      const bool is_q = head < nh;
      if (!is_q && kdst < 0) continue;
      if (is_q ? q_norm_w != nullptr : k_norm_w != nullptr) {
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; e++) ss += x[u][e] * x[u][e];
        ss = warp_sum(ss);
        const float r = 1.0f / sqrtf(ss / (float)HD + eps);
#pragma unroll
        for (int e = 0; e < EPL; e++) x[u][e] = x[u][e] * r * (is_q ? wq[e] : wk[e]);
      }
#pragma unroll
      for (int p = 0; p < NP; p++) {
        const float a = x[u][p], bb = x[u][p + NP];
        x[u][p] = a * c[p] - bb * sn[p];
        x[u][p + NP] = a * sn[p] + bb * c[p];
      }
      if (is_q) {
        T* o = q_out + ((size_t)m * nh + head) * HD;
#pragma unroll
        for (int e = 0; e < EPL; e++) o[lane + 32 * e] = from_f32<T>(x[u][e]);
      } else {
        CT* o = k_pool + kdst + (size_t)(head - nh) * page_size * HD;
#pragma unroll
        for (int e = 0; e < EPL; e++) o[lane + 32 * e] = from_f32<CT>(x[u][e]);
      }
    }
  }
}

LEB_API int leb_qk_rope_store(void* q_out, const void* q_in, int q_stride, const void* k_in,
                              const void* v_in, int kv_stride, void* k_pool, void* v_pool,
                              int dtype, const int* block_table, int bt_width, const int* row_seq,
                              const int* row_pos, const int* seq_slot, const float* q_norm_w,
                              const float* k_norm_w, float eps, const float* inv_freq, int rope_dim,
                              int neox, int M, int nh, int nkv, int hd, int page_size,
                              cudaStream_t st) {
  if (M <= 0) return 0;
  LEB_REQUIRE(hd >= 2 && hd <= 512, "leb_qk_rope_store: head_dim %d outside 2..512", hd);
  LEB_REQUIRE(rope_dim <= hd && rope_dim % 2 == 0, "leb_qk_rope_store: rope_dim %d does not fit head_dim %d", rope_dim, hd);
  int tiles = k_in ? ceil_div(M, VT_ROWS) * nkv : 0;
  int total = nh + (k_in ? nkv : 0);
  dim3 block(32 * ROPE_WARPS);
  if (dtype == LEB_BF16 && inv_freq && neox && rope_dim == hd && (hd == 64 || hd == 128)) {
    // heads per warp: one while the launch is small, up to all of a row's over 8 warps
    int per_warp = 1;
    const long long n_sm = sm_count();
    while (per_warp * ROPE_WARPS < total && (long long)M * ceil_div(total, per_warp * ROPE_WARPS) > 4 * n_sm) per_warp++;
    dim3 grid(M + tiles, ceil_div(total, per_warp * ROPE_WARPS));
    if (hd == 64)
      leb_launch(qk_rope_store_lanes_kernel<bf16, bf16, 2>, grid, block, 0, st,
          (bf16*)q_out, (const bf16*)q_in, q_stride, (const bf16*)k_in, (const bf16*)v_in, kv_stride,
          (bf16*)k_pool, (bf16*)v_pool, block_table, bt_width, row_seq, row_pos, seq_slot, q_norm_w,
          k_norm_w, eps, inv_freq, M, nh, nkv, page_size, per_warp);
    else
      leb_launch(qk_rope_store_lanes_kernel<bf16, bf16, 4>, grid, block, 0, st,
          (bf16*)q_out, (const bf16*)q_in, q_stride, (const bf16*)k_in, (const bf16*)v_in, kv_stride,
          (bf16*)k_pool, (bf16*)v_pool, block_table, bt_width, row_seq, row_pos, seq_slot, q_norm_w,
          k_norm_w, eps, inv_freq, M, nh, nkv, page_size, per_warp);
    LEB_CHECK_LAUNCH("leb_qk_rope_store");
    return 0;
  }
  dim3 grid(M + tiles, ceil_div(total, ROPE_WARPS));
  size_t smem = (size_t)(rope_dim + ROPE_WARPS * hd) * sizeof(float);
  if (dtype == LEB_F32)
    leb_launch(qk_rope_store_kernel<float, float>, grid, block, smem, st,
        (float*)q_out, (const float*)q_in, q_stride, (const float*)k_in, (const float*)v_in,
        kv_stride, (float*)k_pool, (float*)v_pool, block_table, bt_width, row_seq, row_pos,
        seq_slot, q_norm_w, k_norm_w, eps, inv_freq, rope_dim, neox, M, nh, nkv, hd, page_size);
  else if (dtype == LEB_BF16)
    leb_launch(qk_rope_store_kernel<bf16, bf16>, grid, block, smem, st,
        (bf16*)q_out, (const bf16*)q_in, q_stride, (const bf16*)k_in, (const bf16*)v_in, kv_stride,
        (bf16*)k_pool, (bf16*)v_pool, block_table, bt_width, row_seq, row_pos, seq_slot, q_norm_w,
        k_norm_w, eps, inv_freq, rope_dim, neox, M, nh, nkv, hd, page_size);
  else
    return leb_fail("leb_qk_rope_store: unknown dtype %d", dtype);
  LEB_CHECK_LAUNCH("leb_qk_rope_store");
  return 0;
}
