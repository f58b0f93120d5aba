// Attention over the paged cache for packed rows of several sequences: the general kernel.
//
// It serves prompts (many rows per sequence), decode (one row per sequence, the key range split
// over several blocks and merged by a second kernel) and both cache element types.  Keys and
// values are read only from the cache, so the rows of a step see exactly what single-token
// steps would see.
//
// Math as the reference (src/dense.rs:129-146): for query head h the kv head is h / (nh/nkv);
// score_t = (q . k_t) / sqrt(head_dim) for t in [t0, pos], t0 = pos+1-window when the layer has a
// window and pos+1 > window, else 0; softmax with the maximum subtracted; o = sum_t p_t v_t.
// An optional per-head gate multiplies the head's output by sigmoid(gate) (src/dense.rs:147-150).
// Scores, maximum, exponentials, sums and the value accumulation are float.  The reference's
// GPU kernels keep the same running (max, sum, acc) per warp and merge them
// (src/cuda/dense.cu:94-123 whole range, :152-183 split range, :238-247 merge); this kernel lets
// the G query heads of a kv head and several rows share one staged tile of 32 keys, the idea of
// src/cuda/dense.cu:184-237 without its fixed G = 8 and head_dim = 128.
//
// Block = 4 warps.  A block owns one sequence, one kv head, a chunk of HC <= 8 of its query
// heads, QT rows (QT*HC <= 32 "query vectors") and one split of the key range.  Per tile of 32
// keys, lane = key for q.k, lane = dimension for p.v.
#include "common.cuh"

#define ATT_WARPS 4
#define ATT_RPW 8  // query vectors per warp at most: 32 / 4
#define ATT_NEG (-1e30f)

template <typename T, typename CT, int HDL>  // head_dim <= 32 * HDL
__global__ void __launch_bounds__(32 * ATT_WARPS)
attention_kernel(T* __restrict__ out, float* __restrict__ part, const T* __restrict__ q,
                 const CT* __restrict__ k_pool, const CT* __restrict__ v_pool,
                 const int* __restrict__ block_table, int bt_width,
                 const int* __restrict__ seq_slot, const int* __restrict__ seq_pos0,
                 const int* __restrict__ seq_qstart, const int* __restrict__ seq_qlen,
                 const T* __restrict__ gate, int gate_stride, int nh, int nkv, int hd,
                 int page_size, int window, float scale, int QT, int HC, int n_splits) {
  extern __shared__ float sm[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int G = nh / nkv;
  const int n_hc = (G + HC - 1) / HC;
  const int kvh = blockIdx.y / n_hc, hc = blockIdx.y % n_hc;
  const int b = blockIdx.z / n_splits, split = blockIdx.z % n_splits;
  const int slot = seq_slot[b];
  const int qlen = seq_qlen[b];
  const int row_lo = blockIdx.x * QT;
  if (row_lo >= qlen) return;
  const int nrows = min(QT, qlen - row_lo);
  const int nheads = min(HC, G - hc * HC);
  const int q0 = seq_qstart[b];
  const int pos0 = seq_pos0[b];
  const int R = QT * HC;
  const int KS = hd + 1;  // stride of a staged key row: lanes read different rows, same column

  float* q_s = sm;                 // [R][hd]
  float* k_s = q_s + R * hd;       // [32][hd + 1]
  float* v_s = k_s + 32 * KS;      // [32][hd]
  float* p_s = v_s + 32 * hd;      // [ATT_WARPS][32]

  if (slot < 0) {  // padding sequence: defined output, no cache access
    for (int r = warp; r < R; r += ATT_WARPS) {
      int i = r / HC, j = r % HC;
      if (i >= nrows || j >= nheads) continue;
      int h = kvh * G + hc * HC + j;
      size_t m = (size_t)q0 + row_lo + i;
      if (n_splits == 1) {
        for (int d = lane; d < hd; d += 32) out[(m * nh + h) * hd + d] = from_f32<T>(0.f);
      } else {
        float* pp = part + ((m * nh + h) * n_splits + split) * (size_t)(hd + 2);
        if (lane == 0) { pp[0] = ATT_NEG; pp[1] = 0.f; }
        for (int d = lane; d < hd; d += 32) pp[2 + d] = 0.f;
      }
    }
    return;
  }

  for (int idx = threadIdx.x; idx < R * hd; idx += blockDim.x) {
    int r = idx / hd, d = idx - r * hd;
    int i = r / HC, j = r % HC;
    float v = 0.f;
    if (i < nrows && j < nheads) {
      int h = kvh * G + hc * HC + j;
      v = to_f32(q[((size_t)(q0 + row_lo + i) * nh + h) * hd + d]);
    }
    q_s[idx] = v;
  }

  // keys this block may need: up to the last row's position, from the first row's window start
  const int kv_len = pos0 + qlen;  // keys the cache holds for this sequence after this step's writes
  const int pos_lo = pos0 + row_lo, pos_hi = pos0 + row_lo + nrows - 1;
  const int key_lo = (window > 0 && pos_lo + 1 > window) ? pos_lo + 1 - window : 0;
  const int tile_first = key_lo / 32, tile_last = pos_hi / 32;
  const int n_tiles = tile_last - tile_first + 1;
  const int per_split = (n_tiles + n_splits - 1) / n_splits;
  const int t_lo = tile_first + split * per_split;
  const int t_hi = min(tile_last + 1, t_lo + per_split);

  float mx[ATT_RPW], l[ATT_RPW], acc[ATT_RPW][HDL];
#pragma unroll
  for (int ri = 0; ri < ATT_RPW; ri++) {
    mx[ri] = ATT_NEG;
    l[ri] = 0.f;
#pragma unroll
    for (int jj = 0; jj < HDL; jj++) acc[ri][jj] = 0.f;
  }

  for (int tile = t_lo; tile < t_hi; tile++) {
    const int key0 = tile * 32;
    const int page = block_table[(size_t)b * bt_width + key0 / page_size];
    const size_t base = (((size_t)(page < 0 ? 0 : page) * nkv + kvh) * page_size + key0 % page_size) * hd;
    const size_t vbase = ((size_t)(page < 0 ? 0 : page) * nkv + kvh) * hd * page_size + key0 % page_size;
    __syncthreads();  // the previous tile has been consumed (and q_s is written, first time round)
    for (int idx = threadIdx.x; idx < 32 * hd; idx += blockDim.x) {
      int kk = idx / hd, d = idx - kk * hd;
      float kv = 0.f, vv = 0.f;
      if (page >= 0 && key0 + kk < kv_len) {  // beyond the sequence the pool holds stale bits
        kv = to_f32(k_pool[base + idx]);
        vv = to_f32(v_pool[vbase + (size_t)d * page_size + kk]);   // values are stored [dim][position]
      }
      k_s[kk * KS + d] = kv;
      v_s[idx] = vv;
    }
    __syncthreads();
#pragma unroll
    for (int ri = 0; ri < ATT_RPW; ri++) {
      const int r = warp + ri * ATT_WARPS;
      if (r >= R) break;
      const int i = r / HC, j = r % HC;
      if (i >= nrows || j >= nheads) continue;
      const int qpos = pos0 + row_lo + i;
      const float* qv = q_s + r * hd;
      const float* kr = k_s + lane * KS;
      float s = 0.f;
      for (int d = 0; d < hd; d++) s += qv[d] * kr[d];
      s *= scale;
      const int kp = key0 + lane;
      const bool valid = kp <= qpos && (window <= 0 || kp + window > qpos);
      s = valid ? s : ATT_NEG;
      const float mn = fmaxf(mx[ri], warp_max(s));
      const float p = valid ? expf(s - mn) : 0.f;
      const float corr = expf(mx[ri] - mn);
      l[ri] = l[ri] * corr + warp_sum(p);
      mx[ri] = mn;
      p_s[warp * 32 + lane] = p;
      __syncwarp();
#pragma unroll
      for (int jj = 0; jj < HDL; jj++) {
        const int d = lane + 32 * jj;
        if (d < hd) {
          float a = 0.f;
#pragma unroll 8
          for (int kk = 0; kk < 32; kk++) a += p_s[warp * 32 + kk] * v_s[kk * hd + d];
          acc[ri][jj] = acc[ri][jj] * corr + a;
        }
      }
      __syncwarp();
    }
  }

#pragma unroll
  for (int ri = 0; ri < ATT_RPW; ri++) {
    const int r = warp + ri * ATT_WARPS;
    if (r >= R) break;
    const int i = r / HC, j = r % HC;
    if (i >= nrows || j >= nheads) continue;
    const int h = kvh * G + hc * HC + j;
    const size_t m = (size_t)q0 + row_lo + i;
    if (n_splits == 1) {
      float g = 1.f;
      if (gate) {
        float z = to_f32(gate[m * gate_stride + h]);
        g = 1.0f / (1.0f + expf(-z));
      }
      const float inv = l[ri] > 0.f ? 1.0f / l[ri] : 0.f;
#pragma unroll
      for (int jj = 0; jj < HDL; jj++) {
        const int d = lane + 32 * jj;
        if (d < hd) out[(m * nh + h) * hd + d] = from_f32<T>(acc[ri][jj] * inv * g);
      }
    } else {
      float* pp = part + ((m * nh + h) * n_splits + split) * (size_t)(hd + 2);
      if (lane == 0) { pp[0] = mx[ri]; pp[1] = l[ri]; }
#pragma unroll
      for (int jj = 0; jj < HDL; jj++) {
        const int d = lane + 32 * jj;
        if (d < hd) pp[2 + d] = acc[ri][jj];
      }
    }
  }
}

// Merge of the splits of one (row, head): out = sum_s acc_s e^(m_s - M) / sum_s l_s e^(m_s - M).
// A thread owns one dimension and takes the splits eight at a time: maximum, sum and value of all
// eight are asked for before any is used, so a merge of up to eight splits costs one trip to memory
// (with more, the running sums are rescaled to the new maximum from group to group).
template <typename T>
__global__ void attention_merge_kernel(T* __restrict__ out, const float* __restrict__ part,
                                       const T* __restrict__ gate, int gate_stride, int nh, int hd,
                                       int n_splits) {
  pdl_trigger();   // the kernel after this one may start and wait (see common.cuh)
  pdl_wait();
  const size_t m = blockIdx.x;
  const int h = blockIdx.y;
  const size_t step = hd + 2;
  const float* pp = part + ((m * nh + h) * n_splits) * step;
  const float z = gate ? to_f32(gate[m * gate_stride + h]) : 0.f;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float M = ATT_NEG, L = 0.f, a = 0.f;
    for (int s0 = 0; s0 < n_splits; s0 += 8) {
      float ms[8], ls[8], as[8];
#pragma unroll
      for (int q = 0; q < 8; q++) {
        const bool in = s0 + q < n_splits;
        const float* r = pp + (size_t)(in ? s0 + q : 0) * step;
        ms[q] = in ? r[0] : ATT_NEG;
        ls[q] = in ? r[1] : 0.f;
        as[q] = in ? r[2 + d] : 0.f;
      }
      float cm = M;
#pragma unroll
      for (int q = 0; q < 8; q++) cm = fmaxf(cm, ms[q]);
      const float sc = expf(M - cm);   // 0 for the first group (nothing summed yet), 1 when the maximum stays
      L *= sc;
      a *= sc;
#pragma unroll
      for (int q = 0; q < 8; q++) {
        const float e = expf(ms[q] - cm);
        L += ls[q] * e;
        a += as[q] * e;
      }
      M = cm;
    }
    const float g = gate ? 1.0f / (1.0f + expf(-z)) : 1.f;
    out[(m * nh + h) * hd + d] = from_f32<T>(a * (L > 0.f ? 1.0f / L : 0.f) * g);
  }
}

template <typename T, typename CT, int HDL>
static int launch_attention(void* out, float* part, const void* q, const void* k_pool,
                            const void* v_pool, const int* block_table, int bt_width,
                            const int* seq_slot, const int* seq_pos0, const int* seq_qstart,
                            const int* seq_qlen, const void* gate, int gate_stride, int B, int nh,
                            int nkv, int hd, int page_size, int window, float scale, int max_qlen,
                            int n_splits, cudaStream_t st) {
  const int G = nh / nkv;
  const int HC = G < 8 ? G : 8;
  int QT = 32 / HC;
  if (QT > max_qlen) QT = max_qlen;
  const int R = QT * HC;
  const int n_hc = ceil_div(G, HC);
  size_t smem = ((size_t)R * hd + 32 * (hd + 1) + 32 * hd + ATT_WARPS * 32) * sizeof(float);
  auto kern = attention_kernel<T, CT, HDL>;
  static size_t smem_set = 0;
  if (smem > 48 * 1024 && smem > smem_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return leb_fail("leb_attention: shared memory %zu: %s", smem, cudaGetErrorString(e));
    smem_set = smem;
  }
  dim3 grid(ceil_div(max_qlen, QT), nkv * n_hc, B * n_splits);
  LEB_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "leb_attention: grid too large (%u, %u)", grid.y, grid.z);
  kern<<<grid, 32 * ATT_WARPS, smem, st>>>(
      (T*)out, part, (const T*)q, (const CT*)k_pool, (const CT*)v_pool, block_table, bt_width,
      seq_slot, seq_pos0, seq_qstart, seq_qlen, (const T*)gate, gate_stride, nh, nkv, hd, page_size,
      window, scale, QT, HC, n_splits);
  LEB_CHECK_LAUNCH("leb_attention");
  return 0;
}

// out, q: [M, nh*hd]; key pool [page][nkv][page_size][hd], value pool [page][nkv][hd][page_size];
// part: float scratch of
// M*nh*n_splits*(hd+2) elements, used when n_splits > 1 (then every sequence has one row).
LEB_API int leb_attention(void* out, float* part, const void* q, const void* k_pool,
                          const void* v_pool, int dtype, const int* block_table, int bt_width,
                          const int* seq_slot, const int* seq_pos0, const int* seq_qstart,
                          const int* seq_qlen, const void* gate, int gate_stride, int M, int B,
                          int nh, int nkv, int hd, int page_size, int window, float scale,
                          int max_qlen, int n_splits, cudaStream_t st) {
  if (M <= 0 || B <= 0) return 0;
  LEB_REQUIRE(nkv > 0 && nh % nkv == 0, "leb_attention: %d heads do not divide into %d kv heads", nh, nkv);
  LEB_REQUIRE(hd >= 1 && hd <= 256, "leb_attention: head_dim %d outside 1..256", hd);
  LEB_REQUIRE(page_size % 32 == 0, "leb_attention: page size %d is not a multiple of 32", page_size);
  LEB_REQUIRE(n_splits >= 1 && (n_splits == 1 || (max_qlen == 1 && part)), "leb_attention: splits need single-row sequences and scratch");
  int rc;
#define LEB_ATT(T, CT)                                                                            \
  (hd <= 32    ? launch_attention<T, CT, 1>(out, part, q, k_pool, v_pool, block_table, bt_width,  \
                                            seq_slot, seq_pos0, seq_qstart, seq_qlen, gate,       \
                                            gate_stride, B, nh, nkv, hd, page_size, window,      \
                                            scale, max_qlen, n_splits, st)                        \
   : hd <= 64  ? launch_attention<T, CT, 2>(out, part, q, k_pool, v_pool, block_table, bt_width,  \
                                            seq_slot, seq_pos0, seq_qstart, seq_qlen, gate,       \
                                            gate_stride, B, nh, nkv, hd, page_size, window,      \
                                            scale, max_qlen, n_splits, st)                        \
   : hd <= 128 ? launch_attention<T, CT, 4>(out, part, q, k_pool, v_pool, block_table, bt_width,  \
                                            seq_slot, seq_pos0, seq_qstart, seq_qlen, gate,       \
                                            gate_stride, B, nh, nkv, hd, page_size, window,      \
                                            scale, max_qlen, n_splits, st)                        \
               : launch_attention<T, CT, 8>(out, part, q, k_pool, v_pool, block_table, bt_width,  \
                                            seq_slot, seq_pos0, seq_qstart, seq_qlen, gate,       \
                                            gate_stride, B, nh, nkv, hd, page_size, window,      \
                                            scale, max_qlen, n_splits, st))
  if (dtype == LEB_F32)
    rc = LEB_ATT(float, float);
  else if (dtype == LEB_BF16)
    rc = LEB_ATT(bf16, bf16);
  else
    return leb_fail("leb_attention: unknown dtype %d", dtype);
#undef LEB_ATT
  if (rc) return rc;
  if (n_splits > 1) {
    dim3 grid(M, nh);
    if (dtype == LEB_F32)
      attention_merge_kernel<float><<<grid, 64, 0, st>>>((float*)out, part, (const float*)gate, gate_stride, nh, hd, n_splits);
    else
      attention_merge_kernel<bf16><<<grid, 64, 0, st>>>((bf16*)out, part, (const bf16*)gate, gate_stride, nh, hd, n_splits);
    LEB_CHECK_LAUNCH("leb_attention merge");
  }
  return 0;
}

// Merge of split partial results on its own (for kernels that write the same partial layout).
LEB_API int leb_attention_merge(void* out, const float* part, int dtype, const void* gate,
                                int gate_stride, int M, int nh, int hd, int n_splits, cudaStream_t st) {
  if (M <= 0) return 0;
  dim3 grid(M, nh);
  if (dtype == LEB_F32)
    attention_merge_kernel<float><<<grid, 64, 0, st>>>((float*)out, part, (const float*)gate, gate_stride, nh, hd, n_splits);
  else if (dtype == LEB_BF16)
    leb_launch(attention_merge_kernel<bf16>, grid, dim3(64), 0, st, (bf16*)out, part, (const bf16*)gate, gate_stride, nh, hd, n_splits);
  else
    return leb_fail("leb_attention_merge: unknown dtype %d", dtype);
  LEB_CHECK_LAUNCH("leb_attention_merge");
  return 0;
}
