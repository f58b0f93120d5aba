// Decode attention on the tensor cores: one new token per sequence against its whole cache.
//
// A decode step reads every cached key and value of the live sequences once, so the kernel is
// built around that stream (the reference's split-range decode kernels have the same aim,
// src/cuda/dense.cu:152-237, with the query heads of a kv head sharing each key tile).  A block
// owns one sequence, one kv head and one split of the key range; its 4 warps take blocks of 32
// positions in turn, each with its own running (max, sum, acc), merged through shared memory at
// the end; splits are merged by attention_merge_kernel (attention.cu).
//
// Both products run as mma.m16n8k16 with the G <= 16 query heads of the kv head as the 16 rows:
//   S[head, pos]  = Q[head, :] . K[pos, :]         A = Q (registers), B = K rows from the cache
//   O[head, dim] += P[head, pos] . V[pos, dim]     A = P (the S accumulators), B = V^T rows
// Every warp keeps a ring of stages in shared memory (keys [32][head_dim] and values
// [head_dim][32] of one block of positions) filled by asynchronous copies, two or more blocks
// ahead of the one it multiplies, so the memory latency is paid once per warp and not once per
// block; fragments are read from a stage in 16-byte pieces laid out as in the cache:
//  * over head_dim, a lane's 8 contiguous values feed two k16 steps as pairs (0,1)(2,3) and
//    (4,5)(6,7); Q uses the same assignment, and a dot product does not care about the order;
//  * the value cache is stored [dim][position] per page, so a lane's 16 bytes are 8 positions of
//    one dimension, which is what the second product contracts over;
//  * score tile t of a block holds, in column n, position 8*(n/2) + 2t + (n%2): lane (r, c) then
//    ends up with the probabilities of positions 8c..8c+7, exactly the 8 positions of its value
//    piece, so S feeds the second product without any exchange between lanes.
// Scores, maxima, exponentials and sums are float; P is rounded to bfloat16 for the second
// product, as keys and values are.
#include "common.cuh"

#define ATD_WARPS 4
#define ATD_NEG (-1e30f)

__device__ __forceinline__ void mma16816(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void atd_cp16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ uint4 atd_lds(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
// stages of a warp's ring (8 KB each at head size 64).  Two are enough to keep a block in flight
// while one is multiplied, and leave room for three blocks per SM: the loop is a chain of
// dependent tensor-core and exponential steps, and more warps hide it better than deeper rings.
// A launch of so few blocks that an SM gets two at most takes three stages instead.
#define ATD_STAGES(HD) ((HD) <= 32 ? 3 : 2)

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// zero the 16-bit halves of a value piece whose positions are outside [lo, hi)
__device__ __forceinline__ uint4 mask_positions(uint4 v, int first, int lo, int hi) {
  uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
  for (int i = 0; i < 4; i++) {
    int p0 = first + 2 * i, p1 = p0 + 1;
    uint32_t m = ((p0 >= lo && p0 < hi) ? 0x0000ffffu : 0u) | ((p1 >= lo && p1 < hi) ? 0xffff0000u : 0u);
    w[i] &= m;
  }
  return v;
}

// The step's per-head norm, rotation and cache write done here instead of in a kernel of their own
// (all null: q is ready and the cache holds the new position already).  q_raw, k_raw and v_raw are
// the projections of the step's rows (one per sequence) as the matrix product left them; every
// block norms and rotates the query heads it needs, and the block whose key range ends with the
// new position norms and rotates the new key, stores it and the new value in the cache, and only
// then streams that range.  Same operations in the same order as qk_rope_store_lanes_kernel
// (rope_cache.cu), so the two ways give the same bits.  Head sizes 64 and 128 with a split-half
// rotation over the whole head.
struct AtdPrep {
  const bf16* q_raw;      // [rows, q_stride]
  const bf16* k_raw;      // [rows, kv_stride] or null (the layer stores no keys)
  const bf16* v_raw;
  int q_stride, kv_stride;
  bf16* k_store;          // the pools, writable
  bf16* v_store;
  const float* q_norm_w;  // [HD] or null
  const float* k_norm_w;
  const float* inv_freq;  // [HD / 2]
  float eps;
};

// One head vector by one warp: norm over the head, split-half rotation, rounded to bfloat16.
template <int HD>
__device__ __forceinline__ void atd_prep_head(const bf16* __restrict__ src, const float* __restrict__ nw, float eps,
                                              const float* cs, const float* sn, bf16* dst, int lane) {
  constexpr int EPL = HD / 32, NP = EPL / 2;
  float x[EPL];
#pragma unroll
  for (int e = 0; e < EPL; e++) x[e] = __bfloat162float(src[lane + 32 * e]);
  if (nw) {
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; e++) ss += x[e] * x[e];
    ss = warp_sum(ss);
    const float r = 1.0f / sqrtf(ss / (float)HD + eps);
#pragma unroll
    for (int e = 0; e < EPL; e++) x[e] = x[e] * r * nw[lane + 32 * e];
  }
#pragma unroll
  for (int p = 0; p < NP; p++) {
    const float a = x[p], bb = x[p + NP];
    x[p] = a * cs[p] - bb * sn[p];
    x[p + NP] = a * sn[p] + bb * cs[p];
  }
#pragma unroll
  for (int e = 0; e < EPL; e++) dst[lane + 32 * e] = __float2bfloat16_rn(x[e]);
}

template <int HD, int S>  // head_dim, a multiple of 32; stages of a warp's ring
__global__ void __launch_bounds__(32 * ATD_WARPS)
attention_decode_kernel(bf16* __restrict__ out, float* __restrict__ part, const bf16* __restrict__ q,
                        const bf16* __restrict__ k_pool, const bf16* __restrict__ v_pool,
                        const int* __restrict__ block_table, int bt_width,
                        const int* __restrict__ seq_slot, const int* __restrict__ seq_pos0,
                        const int* __restrict__ seq_qstart, const bf16* __restrict__ gate,
                        int gate_stride, int nh, int nkv, int page_size, int window, float scale,
                        int n_splits, AtdPrep prep) {
  constexpr int KB = HD / 32;  // 32-wide pieces of head_dim
  constexpr int NT = HD / 8;   // 8-wide output tiles over head_dim
  constexpr int KBYTES = 32 * HD * 2, STAGE = 2 * KBYTES;   // keys, then values
  // head sizes whose key rows are a multiple of 128 bytes: the pieces of odd rows are moved by 4
  // places so that the two rows a quarter-warp reads fall on different banks
  constexpr int SWZ = (HD % 64 == 0) ? 4 : 0;
  extern __shared__ __align__(128) unsigned char atd_smem[];
  // after the loop the rings are done with and the same memory holds the warps' results
  float (*o_s)[16][HD + 4] = reinterpret_cast<float (*)[16][HD + 4]>(atd_smem);
  float (*m_s)[16] = reinterpret_cast<float (*)[16]>(atd_smem + sizeof(float) * ATD_WARPS * 16 * (HD + 4));
  float (*l_s)[16] = m_s + ATD_WARPS;
  static_assert(sizeof(float) * ATD_WARPS * 16 * (HD + 4 + 2) <= (size_t)ATD_WARPS * S * STAGE, "results must fit the rings");

  // What follows up to pdl_wait() reads only what earlier steps left: the step's own tables (sent
  // before its first kernel) and cache positions below the new one (written a step ago or more;
  // a step starts with a copy or a graph launch, which orders it after everything before).  The
  // kernel before this one made the step's q, k and v, and nothing here touches them or writes
  // anything before the wait.
  pdl_trigger();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int r = lane >> 2, c = lane & 3;
  const int kvh = blockIdx.x, b = blockIdx.y, split = blockIdx.z;
  const int G = nh / nkv;
  const int slot = seq_slot[b];
  const size_t m_row = seq_qstart[b];
  const int h0 = kvh * G;
  // q, out and the partial results have one row per sequence of the launch (gridDim.y): a row
  // index beyond that (a seq_qstart taken from a step with several rows per sequence) is skipped
  // instead of being written past the end of those buffers
  if (m_row >= gridDim.y) {
    pdl_wait();
    return;
  }

  if (slot < 0) {  // padding sequence
    pdl_wait();
    for (int idx = threadIdx.x; idx < G * HD; idx += blockDim.x) {
      int hh = idx / HD, d = idx % HD;
      if (n_splits == 1)
        out[(m_row * nh + h0 + hh) * HD + d] = __float2bfloat16_rn(0.f);
      else
        part[((m_row * nh + h0 + hh) * n_splits + split) * (size_t)(HD + 2) + 2 + d] = 0.f;
    }
    if (n_splits > 1 && threadIdx.x < G) {
      float* pp = part + ((m_row * nh + h0 + threadIdx.x) * n_splits + split) * (size_t)(HD + 2);
      pp[0] = ATD_NEG;
      pp[1] = 0.f;
    }
    return;
  }

  const int qpos = seq_pos0[b];
  const int kv_len = qpos + 1;
  const int key_lo = (window > 0 && kv_len > window) ? kv_len - window : 0;
  const int blk_first = key_lo / 32, blk_last = (kv_len - 1) / 32;
  const int n_blk = blk_last - blk_first + 1;
  const int per_split = (n_blk + n_splits - 1) / n_splits;
  const int blk_lo = blk_first + split * per_split;
  const int blk_hi = min(blk_last + 1, blk_lo + per_split);

  const int* table = block_table + (size_t)b * bt_width;
  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(atd_smem) + warp * (S * STAGE);
  int p_blk = blk_lo + warp, p_q = 0;      // the next block to ask for and its stage number
  auto issue = [&]() {
    if (p_blk < blk_hi) {
      const int key0 = p_blk * 32;
      const int page = table[key0 / page_size];
      const int off = key0 % page_size;
      const bf16* kbase = k_pool + (((size_t)page * nkv + kvh) * page_size + off) * HD;   // 32 rows of HD, contiguous
      const bf16* vbase = v_pool + ((size_t)page * nkv + kvh) * HD * page_size + off;     // HD rows, 32 positions of each
      const uint32_t base = ring + (p_q % S) * STAGE;
      constexpr int KP = HD / 8;             // 16-byte pieces of a key row
#pragma unroll
      for (int i = 0; i < KP; i++) {         // 32 rows x KP pieces, 32 pieces a pass
        const int idx = i * 32 + lane, row = idx / KP, pc = idx % KP;
        atd_cp16(base + row * (HD * 2) + ((pc ^ ((row & 1) * SWZ)) << 4), kbase + (size_t)row * HD + pc * 8);
      }
#pragma unroll
      for (int i = 0; i < HD / 8; i++) {     // HD rows x 4 pieces
        const int idx = i * 32 + lane, row = idx >> 2, pc = idx & 3;
        atd_cp16(base + KBYTES + row * 64 + (pc << 4), vbase + (size_t)row * page_size + pc * 8);
      }
      p_blk += ATD_WARPS;
      p_q++;
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  // The block of positions that holds the new one is written in this step (by the kernel before
  // this one, or below): the first stages are asked for now unless one of them is that block.
  const bool has_new = blk_lo <= blk_last && blk_last < blk_hi;
  const bool early = !has_new || blk_last >= blk_lo + ATD_WARPS * (S - 1);
  if (early) {
#pragma unroll
    for (int i = 0; i < S - 1; i++) issue();
  }
  pdl_wait();

  // Q fragments: heads r and r+8 of this kv head (zero beyond G)
  uint4 qa[KB], qb[KB];
  const bf16* qrow = q + (m_row * nh + h0) * HD;
  if constexpr (HD == 64 || HD == 128) {
    if (prep.q_raw) {
      __shared__ __align__(16) bf16 q_s[16 * HD];
      constexpr int NP = HD / 64;
      float cs[NP], sn[NP];
#pragma unroll
      for (int p = 0; p < NP; p++) {
        const float th = (float)qpos * prep.inv_freq[lane + 32 * p];
        cs[p] = cosf(th);
        sn[p] = sinf(th);
      }
      for (int hh = warp; hh < G; hh += ATD_WARPS)
        atd_prep_head<HD>(prep.q_raw + m_row * prep.q_stride + (size_t)(h0 + hh) * HD, prep.q_norm_w, prep.eps, cs, sn,
                          q_s + hh * HD, lane);
      // the new key and value: the block whose range holds the last block of positions stores them
      // (before it asks for that block's copy, so that the copy finds them in the cache)
      if (prep.k_raw && has_new) {
        const int page = table[qpos / page_size], off = qpos % page_size;
        if (page >= 0) {
          if (warp == ATD_WARPS - 1)
            atd_prep_head<HD>(prep.k_raw + m_row * prep.kv_stride + (size_t)kvh * HD, prep.k_norm_w, prep.eps, cs, sn,
                              prep.k_store + (((size_t)page * nkv + kvh) * page_size + off) * HD, lane);
          for (int d = threadIdx.x; d < HD; d += blockDim.x)
            prep.v_store[(((size_t)page * nkv + kvh) * HD + d) * page_size + off] =
                prep.v_raw[m_row * prep.kv_stride + (size_t)kvh * HD + d];
        }
        __threadfence();     // the copies read the cache through L2
      }
      __syncthreads();
      qrow = q_s;
    }
  }
  if (!early) {
#pragma unroll
    for (int i = 0; i < S - 1; i++) issue();
  }
  {
    const uint4 zero = make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int j = 0; j < KB; j++) {
      qa[j] = r < G ? *reinterpret_cast<const uint4*>(qrow + (size_t)r * HD + 32 * j + 8 * c) : zero;
      qb[j] = r + 8 < G ? *reinterpret_cast<const uint4*>(qrow + (size_t)(r + 8) * HD + 32 * j + 8 * c) : zero;
    }
  }

  // scores are kept times log2(e), so that the exponentials are single exp2 steps
  const float scale2 = scale * 1.4426950408889634f;
  const bool upper = G > 8;   // rows 8..15 of the tiles hold heads at all
  float mx[2] = {ATD_NEG, ATD_NEG}, l[2] = {0.f, 0.f};
  float acc[NT][4];
#pragma unroll
  for (int n = 0; n < NT; n++)
#pragma unroll
    for (int e = 0; e < 4; e++) acc[n][e] = 0.f;

  uint4 kf[4][KB], vf[NT];      // the block being multiplied
  int q_stage = 0;
  for (int blk = blk_lo + warp; blk < blk_hi; blk += ATD_WARPS, q_stage++) {
    const int key0 = blk * 32;
    asm volatile("cp.async.wait_group %0;" ::"n"(S - 2) : "memory");
    __syncwarp();     // every lane's pieces of this stage have landed; everyone is done with the stage before
    issue();
    {
      const uint32_t base = ring + (q_stage % S) * STAGE;
      // keys: tile t, column n = r -> position 8*(r/2) + 2t + (r%2)
#pragma unroll
      for (int t = 0; t < 4; t++) {
        const int kp = 8 * (r >> 1) + 2 * t + (r & 1);
#pragma unroll
        for (int j = 0; j < KB; j++)
          kf[t][j] = atd_lds(base + kp * (HD * 2) + (((4 * j + c) ^ ((kp & 1) * SWZ)) << 4));
      }
      // values: output tile n, dimension 8n + r, positions 8c..8c+7 of the block
#pragma unroll
      for (int n = 0; n < NT; n++) vf[n] = atd_lds(base + KBYTES + (8 * n + r) * 64 + (c << 4));
    }
    const bool partial = key0 < key_lo || key0 + 32 > kv_len;
    if (partial) {
#pragma unroll
      for (int n = 0; n < NT; n++) vf[n] = mask_positions(vf[n], key0 + 8 * c, key_lo, kv_len);
    }

    float s[4][4];
#pragma unroll
    for (int t = 0; t < 4; t++) {
#pragma unroll
      for (int e = 0; e < 4; e++) s[t][e] = 0.f;
#pragma unroll
      for (int j = 0; j < KB; j++) {
        mma16816(s[t], qa[j].x, qb[j].x, qa[j].y, qb[j].y, kf[t][j].x, kf[t][j].y);
        mma16816(s[t], qa[j].z, qb[j].z, qa[j].w, qb[j].w, kf[t][j].z, kf[t][j].w);
      }
    }
    // s[t][0], s[t][1]: head r, positions key0 + 8c + 2t, +1;  s[t][2], s[t][3]: head r + 8
    float tmax[2] = {ATD_NEG, ATD_NEG};
#pragma unroll
    for (int t = 0; t < 4; t++)
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const int kp = key0 + 8 * c + 2 * t + (e & 1);
        const bool valid = kp >= key_lo && kp < kv_len;
        s[t][e] = valid ? s[t][e] * scale2 : ATD_NEG;
        tmax[e >> 1] = fmaxf(tmax[e >> 1], s[t][e]);
      }
    float corr[2];
#pragma unroll
    for (int hh = 0; hh < 2; hh++) {
      tmax[hh] = fmaxf(tmax[hh], __shfl_xor_sync(0xffffffffu, tmax[hh], 1));
      tmax[hh] = fmaxf(tmax[hh], __shfl_xor_sync(0xffffffffu, tmax[hh], 2));
      const float mn = fmaxf(mx[hh], tmax[hh]);
      corr[hh] = exp2f(mx[hh] - mn);
      mx[hh] = mn;
    }
    float psum[2] = {0.f, 0.f};
    uint32_t pa[4][2];  // [tile][head r | head r+8] as bfloat16 pairs
#pragma unroll
    for (int t = 0; t < 4; t++) {
      float p[4];
#pragma unroll
      for (int e = 0; e < 4; e++) {
        p[e] = (e < 2 || upper) && s[t][e] > 0.5f * ATD_NEG ? exp2f(s[t][e] - mx[e >> 1]) : 0.f;
        psum[e >> 1] += p[e];
      }
      pa[t][0] = pack_bf16(p[0], p[1]);
      pa[t][1] = pack_bf16(p[2], p[3]);
    }
#pragma unroll
    for (int hh = 0; hh < 2; hh++) {
      psum[hh] += __shfl_xor_sync(0xffffffffu, psum[hh], 1);
      psum[hh] += __shfl_xor_sync(0xffffffffu, psum[hh], 2);
      l[hh] = l[hh] * corr[hh] + psum[hh];
    }
#pragma unroll
    for (int n = 0; n < NT; n++) {
      acc[n][0] *= corr[0];
      acc[n][1] *= corr[0];
      acc[n][2] *= corr[1];
      acc[n][3] *= corr[1];
      mma16816(acc[n], pa[0][0], pa[0][1], pa[1][0], pa[1][1], vf[n].x, vf[n].y);
      mma16816(acc[n], pa[2][0], pa[2][1], pa[3][0], pa[3][1], vf[n].z, vf[n].w);
    }
  }

  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();    // the rings are no longer read or written: their memory takes the results
  // merge the warps: acc[n][0..1] -> head r, dims 8n + 2c, +1; acc[n][2..3] -> head r + 8
#pragma unroll
  for (int n = 0; n < NT; n++) {
    o_s[warp][r][8 * n + 2 * c] = acc[n][0];
    o_s[warp][r][8 * n + 2 * c + 1] = acc[n][1];
    o_s[warp][r + 8][8 * n + 2 * c] = acc[n][2];
    o_s[warp][r + 8][8 * n + 2 * c + 1] = acc[n][3];
  }
  if (c == 0) {
    m_s[warp][r] = mx[0];
    l_s[warp][r] = l[0];
    m_s[warp][r + 8] = mx[1];
    l_s[warp][r + 8] = l[1];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * HD; idx += blockDim.x) {
    const int hh = idx / HD, d = idx % HD;
    float M = ATD_NEG;
#pragma unroll
    for (int w = 0; w < ATD_WARPS; w++) M = fmaxf(M, m_s[w][hh]);
    float L = 0.f, a = 0.f;
#pragma unroll
    for (int w = 0; w < ATD_WARPS; w++) {
      const float f = exp2f(m_s[w][hh] - M);
      L += l_s[w][hh] * f;
      a += o_s[w][hh][d] * f;
    }
    const int h = h0 + hh;
    if (n_splits == 1) {
      float g = 1.f;
      if (gate) g = 1.0f / (1.0f + expf(-__bfloat162float(gate[m_row * gate_stride + h])));
      out[(m_row * nh + h) * HD + d] = __float2bfloat16_rn(L > 0.f ? a / L * g : 0.f);
    } else {
      float* pp = part + ((m_row * nh + h) * n_splits + split) * (size_t)(HD + 2);
      if (d == 0) { pp[0] = M * 0.6931471805599453f; pp[1] = L; }   // the merge works with natural exponents
      pp[2 + d] = a;
    }
  }
}

// Returns 1 when the sizes are ones this kernel takes (the caller then uses the general kernel).
LEB_API int leb_attention_decode_supported(int nh, int nkv, int hd, int page_size) {
  if (nkv <= 0 || nh % nkv != 0 || nh / nkv > 16) return 0;
  if (hd != 32 && hd != 64 && hd != 96 && hd != 128) return 0;
  return page_size % 32 == 0;
}

// The first stage of a decode step's attention: every sequence brings one row.  With
// n_splits > 1 the partial results go to `part` (same layout as the general kernel's) and the
// caller merges them.
static int attention_decode_launch(void* out, float* part, const void* q, const void* k_pool,
                                   const void* v_pool, const int* block_table, int bt_width,
                                   const int* seq_slot, const int* seq_pos0, const int* seq_qstart,
                                   const void* gate, int gate_stride, int B, int nh, int nkv, int hd,
                                   int page_size, int window, float scale, int n_splits, AtdPrep prep,
                                   cudaStream_t st) {
  if (B <= 0) return 0;
  LEB_REQUIRE(leb_attention_decode_supported(nh, nkv, hd, page_size),
              "leb_attention_decode: sizes not taken (heads %d, kv heads %d, head_dim %d, page %d)", nh, nkv, hd, page_size);
  LEB_REQUIRE(n_splits >= 1 && (n_splits == 1 || part), "leb_attention_decode: splits need scratch");
  dim3 grid(nkv, B, n_splits);
  LEB_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "leb_attention_decode: grid too large");
#define LEB_ATD(HD_, S_)                                                                          \
  {                                                                                               \
    constexpr int smem = ATD_WARPS * S_ * 2 * 32 * HD_ * 2;                                        \
    static bool set = false;                                                                      \
    if (!set) {                                                                                   \
      if (cudaFuncSetAttribute(attention_decode_kernel<HD_, S_>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) \
        return leb_fail("leb_attention_decode: %d bytes of shared memory per block refused", smem); \
      set = true;                                                                                 \
    }                                                                                             \
    leb_launch(attention_decode_kernel<HD_, S_>, grid, dim3(32 * ATD_WARPS), smem, st,             \
        (bf16*)out, part, (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, block_table,  \
        bt_width, seq_slot, seq_pos0, seq_qstart, (const bf16*)gate, gate_stride, nh, nkv, page_size, \
        window, scale, n_splits, prep);                                                           \
  }
  const bool few = (long)grid.x * grid.y * grid.z <= 2L * sm_count();   // an SM gets two blocks at most: deeper rings
  switch (hd) {
    case 32: LEB_ATD(32, 3); break;
    case 64: if (few) LEB_ATD(64, 3) else LEB_ATD(64, 2) break;
    case 96: LEB_ATD(96, 2); break;
    default: LEB_ATD(128, 2); break;
  }
#undef LEB_ATD
  LEB_CHECK_LAUNCH("leb_attention_decode");
  return 0;
}

LEB_API int leb_attention_decode(void* out, float* part, const void* q, const void* k_pool,
                                 const void* v_pool, const int* block_table, int bt_width,
                                 const int* seq_slot, const int* seq_pos0, const int* seq_qstart,
                                 const void* gate, int gate_stride, int B, int nh, int nkv, int hd,
                                 int page_size, int window, float scale, int n_splits,
                                 cudaStream_t st) {
  return attention_decode_launch(out, part, q, k_pool, v_pool, block_table, bt_width, seq_slot, seq_pos0, seq_qstart, gate,
                                 gate_stride, B, nh, nkv, hd, page_size, window, scale, n_splits, AtdPrep{}, st);
}

// Returns 1 when the kernel can norm, rotate and store the step's q, k and v itself: head size 64 or
// 128 and a split-half rotation over the whole head.
LEB_API int leb_attention_decode_prep_supported(int nh, int nkv, int hd, int page_size, int rope_dim, int neox) {
  return leb_attention_decode_supported(nh, nkv, hd, page_size) && (hd == 64 || hd == 128) && rope_dim == hd && neox != 0;
}

// The same with the step's q, k and v as the projection left them (rows of q_stride / kv_stride
// values; k_raw and v_raw null for a layer that stores no keys): per-head norm (weights may be
// null), rotation by position * inv_freq and the write of the new key and value into the pools
// happen inside the kernel.
LEB_API int leb_attention_decode_prep(void* out, float* part, const void* q_raw, int q_stride, const void* k_raw,
                                      const void* v_raw, int kv_stride, void* k_pool, void* v_pool,
                                      const int* block_table, int bt_width, const int* seq_slot,
                                      const int* seq_pos0, const int* seq_qstart, const float* q_norm_w,
                                      const float* k_norm_w, float eps, const float* inv_freq, int rope_dim,
                                      int neox, const void* gate, int gate_stride, int B, int nh, int nkv,
                                      int hd, int page_size, int window, float scale, int n_splits,
                                      cudaStream_t st) {
  LEB_REQUIRE(leb_attention_decode_prep_supported(nh, nkv, hd, page_size, rope_dim, neox),
              "leb_attention_decode_prep: sizes not taken (head_dim %d, rope_dim %d, split-half %d)", hd, rope_dim, neox);
  LEB_REQUIRE(q_raw && inv_freq, "leb_attention_decode_prep: q and the frequencies are required");
  LEB_REQUIRE((k_raw == nullptr) == (v_raw == nullptr), "leb_attention_decode_prep: keys and values come together");
  AtdPrep prep{(const bf16*)q_raw, (const bf16*)k_raw, (const bf16*)v_raw, q_stride, kv_stride, (bf16*)k_pool,
               (bf16*)v_pool, q_norm_w, k_norm_w, inv_freq, eps};
  return attention_decode_launch(out, part, nullptr, k_pool, v_pool, block_table, bt_width, seq_slot, seq_pos0, seq_qstart,
                                 gate, gate_stride, B, nh, nkv, hd, page_size, window, scale, n_splits, prep, st);
}

// ---- the same step for callers that cannot allocate (see leb_no_alloc.h) ---------------------------
#include "leb_no_alloc.h"

extern "C" int leb_attention_merge(void* out, const float* part, int dtype, const void* gate, int gate_stride,
                                   int M, int nh, int hd, int n_splits, cudaStream_t st);

// The split partial results of leb_attention_decode_static.  In host code this name is only a
// handle for cudaGetSymbolAddress, not a device address.
static __device__ __align__(256) float g_static_scratch[LEB_NO_ALLOC_SCRATCH_FLOATS];

#define LEB_MAX_DEVICES 64
static float* g_static_scratch_ptr[LEB_MAX_DEVICES];   // device address of the array, per device

LEB_API int leb_attention_decode_static(void* out, const void* q, const void* k_pool, const void* v_pool,
                                        const int* block_table, int bt_width, const int* seq_slot,
                                        const int* seq_pos0, const int* seq_qstart, const void* gate,
                                        int gate_stride, int B, int nh, int nkv, int hd, int page_size,
                                        int window, float scale, int n_splits, cudaStream_t st) {
  if (B <= 0) return 0;
  LEB_REQUIRE(n_splits >= 1, "leb_attention_decode_static: n_splits must be at least 1");
  float* scratch = nullptr;
  if (n_splits > 1) {
    const unsigned long long need = (unsigned long long)B * nh * n_splits * (hd + 2);
    LEB_REQUIRE(need <= LEB_NO_ALLOC_SCRATCH_FLOATS,
                "leb_attention_decode_static: %d rows x %d heads x %d splits x (head_dim %d + 2) = %llu floats of "
                "scratch, the built-in array holds %u; use fewer splits or leb_attention_decode with your own scratch",
                B, nh, n_splits, hd, need, (unsigned)LEB_NO_ALLOC_SCRATCH_FLOATS);
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return leb_fail("leb_attention_decode_static: cudaGetDevice: %s", cudaGetErrorString(e));
    LEB_REQUIRE(dev >= 0 && dev < LEB_MAX_DEVICES, "leb_attention_decode_static: device index %d not taken", dev);
    if (!g_static_scratch_ptr[dev]) {   // first call on this device (outside any stream capture)
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_static_scratch);
      if (e != cudaSuccess || !p)
        return leb_fail("leb_attention_decode_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
      g_static_scratch_ptr[dev] = (float*)p;
    }
    scratch = g_static_scratch_ptr[dev];
  }
  int rc = leb_attention_decode(out, scratch, q, k_pool, v_pool, block_table, bt_width, seq_slot, seq_pos0,
                                seq_qstart, gate, gate_stride, B, nh, nkv, hd, page_size, window, scale, n_splits, st);
  if (rc) return rc;
  if (n_splits > 1)
    return leb_attention_merge(out, scratch, LEB_BF16, gate, gate_stride, B, nh, hd, n_splits, st);
  return 0;
}
