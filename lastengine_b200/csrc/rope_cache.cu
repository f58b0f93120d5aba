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

template <typename T, typename CT>
__global__ void qk_rope_store_kernel(
    T* __restrict__ q_out, const T* __restrict__ q_in, int q_stride, const T* __restrict__ k_in,
    const T* __restrict__ v_in, int kv_stride, CT* __restrict__ k_pool, CT* __restrict__ v_pool,
    const int* __restrict__ block_table, int bt_width, const int* __restrict__ row_seq,
    const int* __restrict__ row_pos, const int* __restrict__ seq_slot,
    const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w, float eps,
    const float* __restrict__ inv_freq, int rope_dim, int neox, int nh, int nkv, int hd,
    int page_size) {
  extern __shared__ float sm[];  // one head vector per warp
  pdl_wait();
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  int m = blockIdx.x;
  int head = blockIdx.y * nwarps + warp;  // [0,nh): q; [nh,nh+nkv): k; [nh+nkv, nh+2nkv): v
  int total = nh + (k_in ? 2 * nkv : 0);
  if (head >= total) return;
  int b = row_seq[m];
  int slot = seq_slot[b];
  int pos = row_pos[m];
  float* v = sm + warp * hd;

  const T* src;
  const float* nw = nullptr;
  int kind;  // 0 q, 1 k, 2 v
  if (head < nh) {
    kind = 0;
    src = q_in + (size_t)m * q_stride + (size_t)head * hd;
    nw = q_norm_w;
  } else if (head < nh + nkv) {
    kind = 1;
    src = k_in + (size_t)m * kv_stride + (size_t)(head - nh) * hd;
    nw = k_norm_w;
  } else {
    kind = 2;
    src = v_in + (size_t)m * kv_stride + (size_t)(head - nh - nkv) * hd;
  }
  if (kind != 0 && slot < 0) return;  // padding rows own no cache

  float ss = 0.f;
  for (int i = lane; i < hd; i += 32) {
    float x = to_f32(src[i]);
    v[i] = x;
    ss += x * x;
  }
  if (kind != 2) {
    if (nw) {
      ss = warp_sum(ss);
      float r = 1.0f / sqrtf(ss / (float)hd + eps);
      __syncwarp();
      for (int i = lane; i < hd; i += 32) v[i] = v[i] * r * nw[i];
    }
    __syncwarp();
    if (inv_freq) {
      int half = rope_dim / 2;
      for (int i = lane; i < half; i += 32) {
        float th = (float)pos * inv_freq[i];
        float s = sinf(th), c = cosf(th);
        int ia = neox ? i : 2 * i, ib = neox ? i + half : 2 * i + 1;
        float a = v[ia], bb = v[ib];
        v[ia] = a * c - bb * s;
        v[ib] = a * s + bb * c;
      }
    }
  }
  __syncwarp();
  if (kind == 0) {
    T* o = q_out + ((size_t)m * nh + head) * hd;
    for (int i = lane; i < hd; i += 32) o[i] = from_f32<T>(v[i]);
  } else {
    int kvh = kind == 1 ? head - nh : head - nh - nkv;
    int page = block_table[(size_t)b * bt_width + pos / page_size];
    if (page < 0) return;  // a position the cache no longer holds (outside a window)
    if (kind == 1) {
      CT* o = k_pool + (((size_t)page * nkv + kvh) * page_size + pos % page_size) * hd;
      for (int i = lane; i < hd; i += 32) o[i] = from_f32<CT>(v[i]);
    } else {
      CT* o = v_pool + ((size_t)page * nkv + kvh) * hd * page_size + pos % page_size;
      for (int i = lane; i < hd; i += 32) o[(size_t)i * page_size] = from_f32<CT>(v[i]);
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
  const int nwarps = 4;
  int total = nh + (k_in ? 2 * nkv : 0);
  dim3 grid(M, ceil_div(total, nwarps)), block(32 * nwarps);
  size_t smem = (size_t)nwarps * hd * sizeof(float);
  if (dtype == LEB_F32)
    leb_launch(qk_rope_store_kernel<float, float>, grid, block, smem, st,
        (float*)q_out, (const float*)q_in, q_stride, (const float*)k_in, (const float*)v_in,
        kv_stride, (float*)k_pool, (float*)v_pool, block_table, bt_width, row_seq, row_pos,
        seq_slot, q_norm_w, k_norm_w, eps, inv_freq, rope_dim, neox, nh, nkv, hd, page_size);
  else if (dtype == LEB_BF16)
    leb_launch(qk_rope_store_kernel<bf16, bf16>, grid, block, smem, st,
        (bf16*)q_out, (const bf16*)q_in, q_stride, (const bf16*)k_in, (const bf16*)v_in, kv_stride,
        (bf16*)k_pool, (bf16*)v_pool, block_table, bt_width, row_seq, row_pos, seq_slot, q_norm_w,
        k_norm_w, eps, inv_freq, rope_dim, neox, nh, nkv, hd, page_size);
  else
    return leb_fail("leb_qk_rope_store: unknown dtype %d", dtype);
  LEB_CHECK_LAUNCH("leb_qk_rope_store");
  return 0;
}
