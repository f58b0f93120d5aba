// Prompt attention on the tensor cores: many rows per sequence against the paged cache.
//
// Same two products and the same fragment scheme as the decode kernel (attention_decode.cu):
// S = Q K^T and O += P V as mma.m16n8k16 with fragments read in 16-byte pieces, values stored
// [dim][position], and score tiles whose column order makes S the A operand of the second
// product without any exchange between lanes.  The reference's prompt kernel is the same online
// softmax over 64 x 32 tiles with mma.sync (src/cuda/kernels.cu:1275-1390), for head size 128
// only and one query head per block; here the rows of a block are (position, query head) pairs
// of one kv head, so the G query heads that share a kv head also share every key and value
// the block reads.
//
// A block owns one sequence, one kv head and QT consecutive positions: QT*G rows, 16*MT per
// warp.  Every warp walks the key blocks of 32 positions its rows can see, causally and inside
// the window, with a running (max, sum, acc) per row; the fragments of the next block are
// loaded while the current one is multiplied, exponentials are 2^x on scores pre-multiplied by
// log2(e), and blocks wholly below the diagonal skip the mask.  Keys and values come from the cache
// only, which already holds this step's rows.
#include "common.cuh"

#define ATP_WARPS 4
#define ATP_NEG (-1e30f)

__device__ __forceinline__ void mma16816p(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint4 mask_tail(uint4 v, int first, int hi) {
  uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
  for (int i = 0; i < 4; i++) {
    int p0 = first + 2 * i;
    w[i] &= (p0 < hi ? 0x0000ffffu : 0u) | (p0 + 1 < hi ? 0xffff0000u : 0u);
  }
  return v;
}

template <int HD, int MT>  // head_dim (multiple of 32); 16-row tiles per warp
__global__ void __launch_bounds__(32 * ATP_WARPS)
attention_prefill_kernel(bf16* __restrict__ out, const bf16* __restrict__ q,
                         const bf16* __restrict__ k_pool, const bf16* __restrict__ v_pool,
                         const int* __restrict__ block_table, int bt_width,
                         const int* __restrict__ seq_slot, const int* __restrict__ seq_pos0,
                         const int* __restrict__ seq_qstart, const int* __restrict__ seq_qlen,
                         const bf16* __restrict__ gate, int gate_stride, int nh, int nkv, int page_size,
                         int window, float scale, int QT) {
  constexpr int KB = HD / 32, NT = HD / 8;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int r = lane >> 2, c = lane & 3;
  const int kvh = blockIdx.y, b = blockIdx.z;
  const int G = nh / nkv;
  const int qlen = seq_qlen[b];
  // heavy tiles (late positions) first
  const int tile = (int)gridDim.x - 1 - (int)blockIdx.x;
  const int p_lo = tile * QT;
  if (p_lo >= qlen) return;
  const int npos = min(QT, qlen - p_lo);
  const int nrows = npos * G;
  const int slot = seq_slot[b];
  const size_t q0 = seq_qstart[b];
  const int pos0 = seq_pos0[b];
  const int h0 = kvh * G;
  const int row0 = warp * MT * 16;   // first row of this warp
  if (row0 >= nrows) return;

  // rows of this lane: tile mt, halves 0 (row r) and 1 (row r + 8)
  int rpos[MT][2], rhead[MT][2];
  bool rok[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; mt++)
#pragma unroll
    for (int hh = 0; hh < 2; hh++) {
      const int row = row0 + mt * 16 + r + 8 * hh;
      rok[mt][hh] = row < nrows;
      rpos[mt][hh] = p_lo + row / G;       // position within this step's rows of the sequence
      rhead[mt][hh] = row % G;
    }

  if (slot < 0) {   // padding sequence: zeros
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
      for (int hh = 0; hh < 2; hh++)
        if (rok[mt][hh]) {
          bf16* o = out + ((q0 + rpos[mt][hh]) * nh + h0 + rhead[mt][hh]) * HD;
          for (int d = 2 * c; d < HD; d += 8) { o[d] = __float2bfloat16_rn(0.f); o[d + 1] = __float2bfloat16_rn(0.f); }
        }
    return;
  }

  uint4 qa[MT][KB], qb[MT][KB];
  {
    const uint4 zero = make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int mt = 0; mt < MT; mt++) {
      const bf16* ra = q + ((q0 + rpos[mt][0]) * nh + h0 + rhead[mt][0]) * HD;
      const bf16* rb = q + ((q0 + rpos[mt][1]) * nh + h0 + rhead[mt][1]) * HD;
#pragma unroll
      for (int j = 0; j < KB; j++) {
        qa[mt][j] = rok[mt][0] ? *reinterpret_cast<const uint4*>(ra + 32 * j + 8 * c) : zero;
        qb[mt][j] = rok[mt][1] ? *reinterpret_cast<const uint4*>(rb + 32 * j + 8 * c) : zero;
      }
    }
  }

  const int kv_len = pos0 + qlen;
  // this warp's rows see keys [key_lo, key_hi]
  const int first_pos = pos0 + p_lo + row0 / G;
  const int last_row = min(nrows, row0 + MT * 16) - 1;
  const int key_hi = pos0 + p_lo + last_row / G;
  const int key_lo = (window > 0 && first_pos + 1 > window) ? first_pos + 1 - window : 0;

  float mx[MT][2], l[MT][2], acc[MT][NT][4];
#pragma unroll
  for (int mt = 0; mt < MT; mt++) {
    mx[mt][0] = mx[mt][1] = ATP_NEG;
    l[mt][0] = l[mt][1] = 0.f;
#pragma unroll
    for (int n = 0; n < NT; n++)
#pragma unroll
      for (int e = 0; e < 4; e++) acc[mt][n][e] = 0.f;
  }

  const int* table = block_table + (size_t)b * bt_width;
  // Scores are kept in base 2: s2 = (q.k) * scale * log2(e), p = 2^(s2 - max2) = e^(s - max).
  const float scale2 = scale * 1.4426950408889634f;
  // the lowest query position among this lane's rows: blocks wholly at or below it need no mask
  int qmin = 0x7fffffff;
#pragma unroll
  for (int mt = 0; mt < MT; mt++)
#pragma unroll
    for (int hh = 0; hh < 2; hh++) qmin = min(qmin, pos0 + rpos[mt][hh]);
  qmin = min(qmin, __shfl_xor_sync(0xffffffffu, qmin, 4));
  qmin = min(qmin, __shfl_xor_sync(0xffffffffu, qmin, 8));
  qmin = min(qmin, __shfl_xor_sync(0xffffffffu, qmin, 16));

  const int blk_first = key_lo / 32, blk_last = key_hi / 32;
  uint4 kf[4][KB], vf[NT];      // the block being multiplied
  uint4 kn[4][KB], vn[NT];      // the next block, in flight meanwhile
  auto load_block = [&](int blk, uint4 (&kd)[4][KB], uint4 (&vd)[NT]) {
    const int key0 = blk * 32;
    const int page = table[key0 / page_size];
    const int off = key0 % page_size;
    const bf16* kbase = k_pool + (((size_t)page * nkv + kvh) * page_size + off) * HD;
    const bf16* vbase = v_pool + ((size_t)page * nkv + kvh) * HD * page_size + off;
#pragma unroll
    for (int t = 0; t < 4; t++) {
      const int kp = 8 * (r >> 1) + 2 * t + (r & 1);
#pragma unroll
      for (int j = 0; j < KB; j++)
        kd[t][j] = *reinterpret_cast<const uint4*>(kbase + (size_t)kp * HD + 32 * j + 8 * c);
    }
#pragma unroll
    for (int n = 0; n < NT; n++)
      vd[n] = *reinterpret_cast<const uint4*>(vbase + (size_t)(8 * n + r) * page_size + 8 * c);
  };
  constexpr bool PREFETCH = HD <= 64;   // larger heads have no registers to spare for a second block
  // one block of 32 positions against this warp's rows
  auto compute = [&](uint4 (&kf)[4][KB], uint4 (&vf)[NT], int blk) {
    const int key0 = blk * 32;
    if (key0 + 32 > kv_len) {
#pragma unroll
      for (int n = 0; n < NT; n++) vf[n] = mask_tail(vf[n], key0 + 8 * c, kv_len);
    }
    const bool need_mask = window > 0 || key0 + 31 > qmin;

#pragma unroll
    for (int mt = 0; mt < MT; mt++) {
      float s[4][4];
#pragma unroll
      for (int t = 0; t < 4; t++) {
#pragma unroll
        for (int e = 0; e < 4; e++) s[t][e] = 0.f;
#pragma unroll
        for (int j = 0; j < KB; j++) {
          mma16816p(s[t], qa[mt][j].x, qb[mt][j].x, qa[mt][j].y, qb[mt][j].y, kf[t][j].x, kf[t][j].y);
          mma16816p(s[t], qa[mt][j].z, qb[mt][j].z, qa[mt][j].w, qb[mt][j].w, kf[t][j].z, kf[t][j].w);
        }
      }
      float tmax[2] = {ATP_NEG, ATP_NEG};
      if (need_mask) {
#pragma unroll
        for (int t = 0; t < 4; t++)
#pragma unroll
          for (int e = 0; e < 4; e++) {
            const int hh = e >> 1;
            const int kp = key0 + 8 * c + 2 * t + (e & 1);
            const int qp = pos0 + rpos[mt][hh];
            const bool valid = kp <= qp && (window <= 0 || kp + window > qp);
            s[t][e] = valid ? s[t][e] * scale2 : ATP_NEG;
            tmax[hh] = fmaxf(tmax[hh], s[t][e]);
          }
      } else {
#pragma unroll
        for (int t = 0; t < 4; t++)
#pragma unroll
          for (int e = 0; e < 4; e++) {
            s[t][e] *= scale2;
            tmax[e >> 1] = fmaxf(tmax[e >> 1], s[t][e]);
          }
      }
      float corr[2];
#pragma unroll
      for (int hh = 0; hh < 2; hh++) {
        tmax[hh] = fmaxf(tmax[hh], __shfl_xor_sync(0xffffffffu, tmax[hh], 1));
        tmax[hh] = fmaxf(tmax[hh], __shfl_xor_sync(0xffffffffu, tmax[hh], 2));
        const float mn = fmaxf(mx[mt][hh], tmax[hh]);
        corr[hh] = exp2f(mx[mt][hh] - mn);
        mx[mt][hh] = mn;
      }
      float psum[2] = {0.f, 0.f};
      uint32_t pa[4][2];
#pragma unroll
      for (int t = 0; t < 4; t++) {
        float p[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
          // a masked score is -1e30: 2^(-1e30 - max) is 0 unless the whole row is still masked
          p[e] = (need_mask && s[t][e] <= 0.5f * ATP_NEG) ? 0.f : exp2f(s[t][e] - mx[mt][e >> 1]);
          psum[e >> 1] += p[e];
        }
        pa[t][0] = pack2(p[0], p[1]);
        pa[t][1] = pack2(p[2], p[3]);
      }
#pragma unroll
      for (int hh = 0; hh < 2; hh++) {
        psum[hh] += __shfl_xor_sync(0xffffffffu, psum[hh], 1);
        psum[hh] += __shfl_xor_sync(0xffffffffu, psum[hh], 2);
        l[mt][hh] = l[mt][hh] * corr[hh] + psum[hh];
      }
      // after the first blocks a row's maximum seldom moves: skip the rescaling then
      const bool moved = __any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f);
#pragma unroll
      for (int n = 0; n < NT; n++) {
        if (moved) {
          acc[mt][n][0] *= corr[0];
          acc[mt][n][1] *= corr[0];
          acc[mt][n][2] *= corr[1];
          acc[mt][n][3] *= corr[1];
        }
        mma16816p(acc[mt][n], pa[0][0], pa[0][1], pa[1][0], pa[1][1], vf[n].x, vf[n].y);
        mma16816p(acc[mt][n], pa[2][0], pa[2][1], pa[3][0], pa[3][1], vf[n].z, vf[n].w);
      }
    }
  };
  if (PREFETCH) {
    // two sets of fragments take turns: one is multiplied while the other is in flight
    load_block(blk_first, kf, vf);
    for (int blk = blk_first; blk <= blk_last; blk += 2) {
      if (blk + 1 <= blk_last) load_block(blk + 1, kn, vn);
      compute(kf, vf, blk);
      if (blk + 1 <= blk_last) {
        if (blk + 2 <= blk_last) load_block(blk + 2, kf, vf);
        compute(kn, vn, blk + 1);
      }
    }
  } else {
    for (int blk = blk_first; blk <= blk_last; blk++) {
      load_block(blk, kf, vf);
      compute(kf, vf, blk);
    }
  }

#pragma unroll
  for (int mt = 0; mt < MT; mt++)
#pragma unroll
    for (int hh = 0; hh < 2; hh++) {
      if (!rok[mt][hh]) continue;
      const size_t m = q0 + rpos[mt][hh];
      const int h = h0 + rhead[mt][hh];
      float g = 1.f;
      if (gate) g = 1.0f / (1.0f + expf(-__bfloat162float(gate[m * gate_stride + h])));
      const float inv = l[mt][hh] > 0.f ? g / l[mt][hh] : 0.f;
      bf16* o = out + (m * nh + h) * HD;
#pragma unroll
      for (int n = 0; n < NT; n++) {
        const uint32_t v = pack2(acc[mt][n][2 * hh] * inv, acc[mt][n][2 * hh + 1] * inv);
        *reinterpret_cast<uint32_t*>(o + 8 * n + 2 * c) = v;
      }
    }
}

LEB_API int leb_attention_prefill_supported(int nh, int nkv, int hd, int page_size) {
  if (nkv <= 0 || nh % nkv != 0 || nh / nkv > 64) return 0;
  if (hd != 32 && hd != 64 && hd != 96 && hd != 128) return 0;
  return page_size % 32 == 0;
}

LEB_API int leb_attention_prefill(void* out, const void* q, const void* k_pool, const void* v_pool,
                                  const int* block_table, int bt_width, const int* seq_slot,
                                  const int* seq_pos0, const int* seq_qstart, const int* seq_qlen,
                                  const void* gate, int gate_stride, int B, int nh, int nkv, int hd,
                                  int page_size, int window, float scale, int max_qlen, cudaStream_t st) {
  if (B <= 0 || max_qlen <= 0) return 0;
  LEB_REQUIRE(leb_attention_prefill_supported(nh, nkv, hd, page_size),
              "leb_attention_prefill: sizes not taken (heads %d, kv heads %d, head_dim %d, page %d)", nh, nkv, hd, page_size);
  const int G = nh / nkv;
  const int MT = hd <= 32 ? 2 : 1;
  const int rows_per_block = ATP_WARPS * MT * 16;
  int QT = rows_per_block / G;
  if (QT < 1) QT = 1;
  dim3 grid(ceil_div(max_qlen, QT), nkv, B);
  LEB_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "leb_attention_prefill: grid too large");
#define LEB_ATP(HD_, MT_)                                                                            \
  attention_prefill_kernel<HD_, MT_><<<grid, 32 * ATP_WARPS, 0, st>>>(                               \
      (bf16*)out, (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, block_table, bt_width,   \
      seq_slot, seq_pos0, seq_qstart, seq_qlen, (const bf16*)gate, gate_stride, nh, nkv, page_size,  \
      window, scale, QT)
  switch (hd) {
    case 32: LEB_ATP(32, 2); break;
    case 64: LEB_ATP(64, 1); break;
    case 96: LEB_ATP(96, 1); break;
    default: LEB_ATP(128, 1); break;
  }
#undef LEB_ATP
  LEB_CHECK_LAUNCH("leb_attention_prefill");
  return 0;
}
