// Prompt attention on the fifth-generation tensor cores (tcgen05), head size 64, pages of 64.
//
// The reference's prompt attention (src/cuda/dense.cu:239-283) walks the keys of each query in a
// loop per (token, head); here a block owns a tile of 128 rows = the G query heads of one kv head
// times 128/G consecutive positions of one sequence, so that the keys and values of the kv head
// are read once for all its query heads, and walks the cache page by page (64 positions):
//
//   S[128, 64]  = Q[128, 64] . K_page[64, 64]^T        tcgen05.mma, both operands in shared memory
//   P           = exp2(S * scale * log2 e - m)          128 threads, one row each, S read from
//                                                       tensor memory, P written back there (bf16)
//   O[128, 64] += P[128, 64] . V_page[64, 64]           tcgen05.mma, P from tensor memory, V from
//                                                       shared memory
//
// Q, the key page [position][dim] and the value page [dim][position] (the cache stores values
// transposed) are all K-major tiles with rows of 128 bytes, which TMA brings in under the
// 128-byte swizzle straight from the paged cache: no gather, no transposition.
//
// Roles: warps 0-3 softmax (thread r owns row r of S, P and O), warp 4 TMA producer, warp 5 issues
// the MMAs.  S and P are double-buffered in tensor memory, so the product of the next page's
// scores runs while this page's exponentials are taken; two blocks per SM overlap the rest.
// The running maximum is only moved when it grew by more than 8 (a factor 256): exponentials stay
// bounded, the row sum uses the same reference, and the quotient at the end is exact; moving it
// means rescaling O in tensor memory, which then happens a few times per row instead of once
// per page.
//
// Positions outside [window start, query position] get probability zero by selection, never by
// arithmetic on what the cache holds there; the value page that holds the end of the
// sequence has its columns beyond the end set to zero in shared memory before it is used, so
// that whatever lies there (stale numbers, or NaN in tests) cannot reach O through 0 * x.
// Every wait on an mbarrier is bounded; a wait that gives up sets the status word, all roles leave
// their loops, tensor memory is freed and the block returns.
#include "tc_common.cuh"

#define ATC_THREADS 192
#define ATC_STAGES 4
#define ATC_NEG (-1e30f)

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
        "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
        "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
        "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// D[tmem] (+)= A[tmem] . B[smem]
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ float ex2(float x) {   // 2^x, one special-function step; 2^(very negative) = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

template <int GS>   // query heads per kv head (1, 2, 4, 8): a tile is GS heads x 128/GS positions
__global__ void __launch_bounds__(ATC_THREADS, 2)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, bf16* __restrict__ out,
                            const int* __restrict__ block_table, int bt_width, const int* __restrict__ seq_slot,
                            const int* __restrict__ seq_pos0, const int* __restrict__ seq_qstart,
                            const int* __restrict__ seq_qlen, const bf16* __restrict__ gate, int gate_stride,
                            int nh, int nkv, int window, float scale, int* __restrict__ status) {
  constexpr int HD = 64, PAGE = 64, TP = 128 / GS, NS = ATC_STAGES;
  constexpr int Q_BYTES = 128 * HD * 2, KV_BYTES = PAGE * HD * 2;
  extern __shared__ uint8_t atc_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)atc_raw + 1023) & ~(uintptr_t)1023);   // swizzled tiles want 1024
  uint8_t* sq = smem;
  uint8_t* sk = sq + Q_BYTES;
  uint8_t* sv = sk + NS * KV_BYTES;
  __shared__ uint64_t q_full, k_full[NS], v_full[NS], kv_empty[NS], s_full[2], p_full[2], pv_done[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_s;
  volatile int* abort_flag = &abort_s;

  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // blocks start in the order x, y, z: kv heads vary fastest, and the tiles with the longest key
  // range come first, for all heads, so that the short ones fill the gaps at the end
  const int tile = gridDim.y - 1 - blockIdx.y;
  const int kvh = blockIdx.x, b = blockIdx.z;
  const int qlen = seq_qlen[b], row0 = tile * TP;   // step data: copied in long before the kernel before this one
  if (row0 >= qlen) {
    pdl_wait();   // a kernel counts as complete when its blocks are: none may finish before its predecessor has
    return;
  }
  const int rows = min(TP, qlen - row0);
  const int pos0 = seq_pos0[b];
  const size_t m_base = (size_t)seq_qstart[b] + row0;
  const int h0 = kvh * GS;
  if (seq_slot[b] < 0) {   // a padding sequence: its rows are zero
    pdl_wait();
    for (int idx = threadIdx.x; idx < rows * GS * (HD / 8); idx += blockDim.x) {
      const int i = idx / (GS * (HD / 8)), rest = idx % (GS * (HD / 8));
      reinterpret_cast<uint4*>(out + ((m_base + i) * nh + h0) * HD)[rest] = make_uint4(0, 0, 0, 0);
    }
    return;
  }
  const int q_lo = pos0 + row0;                  // position of the tile's first query
  const int key_hi = q_lo + rows;                // keys [.., key_hi) exist for this tile
  const int key_lo_tile = window > 0 ? max(0, q_lo - window + 1) : 0;
  const int jb0 = key_lo_tile / PAGE, nblk = (key_hi - 1) / PAGE - jb0 + 1;
  const int* table = block_table + (size_t)b * bt_width;

  if (threadIdx.x == 0) {
    abort_s = 0;
    mbar_init(&q_full, 1);
    for (int s = 0; s < NS; s++) {
      mbar_init(&k_full[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int i = 0; i < 2; i++) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 4);
      mbar_init(&pv_done[i], 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 4) {
    tmem_alloc(&tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();      // barriers and tensor memory are set up; now q and the cache must be complete
  const uint32_t tmem = tmem_slot;
  const uint32_t t_o = tmem, t_s0 = tmem + 64, t_p0 = tmem + 192;   // O | S0 S1 | P0 P1 (columns)
  // instruction descriptor: float accumulate, bfloat16 operands, both K-major, N = 64, M = 128
  constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((64u >> 3) << 17) | ((128u >> 4) << 24);
  bool ok = true;

  if (warp == 4) {
    // ---- TMA producer ----
    if (lane == 0) {
      mbar_expect_tx(&q_full, Q_BYTES);
      for (int g = 0; g < GS; g++)
        tma_load_2d(sq + g * (TP * HD * 2), &map_q, &q_full, (h0 + g) * HD, (int)m_base);
      int next_page = table[jb0];
      for (int i = 0; i < nblk && ok; i++) {
        const int s = i % NS;
        int page = next_page;
        if (i + 1 < nblk) next_page = table[jb0 + i + 1];   // asked for before the wait below
        if (!mbar_wait(&kv_empty[s], ((i / NS) & 1) ^ 1, abort_flag)) { atomicExch(status, 11); ok = false; break; }
        if (page < 0) page = 0;   // a page the window has left behind: every key of it is masked
        const int y = (page * nkv + kvh) * PAGE;
        mbar_expect_tx(&k_full[s], KV_BYTES);
        tma_load_2d(sk + s * KV_BYTES, &map_k, &k_full[s], 0, y);
        mbar_expect_tx(&v_full[s], KV_BYTES);
        tma_load_2d(sv + s * KV_BYTES, &map_v, &v_full[s], 0, y);
      }
    }
  } else if (warp == 5) {
    // ---- MMA issuer ----
    if (lane == 0) {
      auto scores = [&](int i) -> bool {
        const int s = i % NS;
        if (!mbar_wait(&k_full[s], (i / NS) & 1, abort_flag)) { atomicExch(status, 12); return false; }
        tc_fence_after();
        const uint32_t qa = smem_u32(sq), ka = smem_u32(sk + s * KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < HD / 16; kk++)
          umma_bf16(t_s0 + 64 * (i & 1), make_desc(qa + kk * 32), make_desc(ka + kk * 32), IDESC, kk > 0);
        umma_commit(&s_full[i & 1]);
        return true;
      };
      if (!mbar_wait(&q_full, 0, abort_flag)) { atomicExch(status, 13); ok = false; }
      if (ok) ok = scores(0);
      for (int i = 0; i < nblk && ok; i++) {
        if (i + 1 < nblk && !scores(i + 1)) { ok = false; break; }
        const int s = i % NS;
        if (!mbar_wait(&p_full[i & 1], (i >> 1) & 1, abort_flag)) { atomicExch(status, 14); ok = false; break; }
        if (!mbar_wait(&v_full[s], (i / NS) & 1, abort_flag)) { atomicExch(status, 15); ok = false; break; }
        tc_fence_after();
        const uint32_t va = smem_u32(sv + s * KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < PAGE / 16; kk++)
          umma_bf16_ts(t_o, t_p0 + 32 * (i & 1) + kk * 8, make_desc(va + kk * 32), IDESC, (i > 0 || kk > 0));
        umma_commit(&kv_empty[s]);
        umma_commit(&pv_done[i & 1]);
      }
    }
  } else {
    // ---- softmax: thread r owns row r = (head r / TP, position r % TP) ----
    const int r = threadIdx.x, g = r / TP, pi = r % TP;
    const bool row_valid = pi < rows;
    const int qpos = q_lo + pi;
    const int key_lo_row = window > 0 ? max(0, qpos - window + 1) : 0;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    const float scale2 = scale * 1.4426950408889634f;
    float m_used = ATC_NEG, l = 0.f;
    for (int i = 0; i < nblk && ok; i++) {
      const int key0 = (jb0 + i) * PAGE, bsel = i & 1, s = i % NS;
      if (!mbar_wait(&s_full[bsel], (i >> 1) & 1, abort_flag)) { atomicExch(status, 16); ok = false; break; }
      tc_fence_after();
      uint32_t v[64];
      tmem_ld32(t_s0 + 64 * bsel + lane_base, v);
      tmem_ld32(t_s0 + 64 * bsel + lane_base + 32, v + 32);
      tmem_ld_wait();
      // columns [c_lo, c_hi] of this page are keys this row may see
      const int c_lo = max(0, key_lo_row - key0), c_hi = row_valid ? min(PAGE - 1, qpos - key0) : -1;
      // The scores stay as the product left them; the scale goes into the exponent's multiply-add.
      float rm[4] = {ATC_NEG, ATC_NEG, ATC_NEG, ATC_NEG};   // four chains instead of one of 64 steps
      if (c_lo == 0 && c_hi == PAGE - 1) {
#pragma unroll
        for (int c = 0; c < PAGE; c++) rm[c & 3] = fmaxf(rm[c & 3], __uint_as_float(v[c]));
      } else {
#pragma unroll
        for (int c = 0; c < PAGE; c++) {
          const float sc = (c >= c_lo && c <= c_hi) ? __uint_as_float(v[c]) : ATC_NEG;
          v[c] = __float_as_uint(sc);
          rm[c & 3] = fmaxf(rm[c & 3], sc);
        }
      }
      const float rmax = fmaxf(fmaxf(rm[0], rm[1]), fmaxf(rm[2], rm[3]));
      // maxima are kept times scale * log2(e); a row with no key in this page keeps what it had
      const float m_new = rmax > 0.5f * ATC_NEG ? fmaxf(m_used, rmax * scale2) : m_used;
      bool move = false;
      if (l == 0.f) m_used = m_new;                 // nothing accumulated for this row yet: O's row is zero
      else if (m_new > m_used + 8.f) move = true;   // the reference maximum has to follow
      if (__any_sync(0xffffffffu, move)) {
        // O holds pages < i; the product of page i waits for this warp's P, so O is still once page i-1 is in
        if (!mbar_wait(&pv_done[(i - 1) & 1], ((i - 1) >> 1) & 1, abort_flag)) { atomicExch(status, 17); ok = false; break; }
        tc_fence_after();
        const float f = move ? ex2(m_used - m_new) : 1.f;
#pragma unroll
        for (int hcol = 0; hcol < HD; hcol += 32) {
          uint32_t o[32];
          tmem_ld32(t_o + lane_base + hcol, o);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 32; c++) o[c] = __float_as_uint(__uint_as_float(o[c]) * f);
          tmem_st32(t_o + lane_base + hcol, o);
        }
        tmem_st_wait();
        l *= f;
        if (move) m_used = m_new;
      }
      const float m_ref = m_used > 0.5f * ATC_NEG ? m_used : 0.f;
      uint32_t pk[32];
      float ps[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < PAGE; c += 2) {
        // a masked score is -1e30: 2^(that * scale - m_ref) is exactly zero
        const float p0 = ex2(fmaf(__uint_as_float(v[c]), scale2, -m_ref)), p1 = ex2(fmaf(__uint_as_float(v[c + 1]), scale2, -m_ref));
        ps[(c >> 1) & 3] += p0 + p1;
        __nv_bfloat162 pp = __floats2bfloat162_rn(p0, p1);
        pk[c >> 1] = *reinterpret_cast<uint32_t*>(&pp);
      }
      l += (ps[0] + ps[1]) + (ps[2] + ps[3]);
      // P[bsel] was last read by the product of page i-2
      if (i >= 2 && !mbar_wait(&pv_done[bsel], ((i - 2) >> 1) & 1, abort_flag)) { atomicExch(status, 18); ok = false; break; }
      tc_fence_after();
      tmem_st32(t_p0 + 32 * bsel + lane_base, pk);
      tmem_st_wait();
      if (key0 + PAGE > key_hi) {
        // the page with the end of the sequence: its value columns beyond the end become zero
        if (!mbar_wait(&v_full[s], (i / NS) & 1, abort_flag)) { atomicExch(status, 19); ok = false; break; }
        const int n_valid = key_hi - key0;
        if (r < HD) {
          uint8_t* vrow = sv + s * KV_BYTES + r * 128;   // dimension r: 64 positions, 16-byte pieces swizzled by r & 7
          for (int cc = n_valid / 8; cc < 8; cc++) {
            bf16* piece = reinterpret_cast<bf16*>(vrow + ((cc ^ (r & 7)) << 4));
            for (int e = max(0, n_valid - cc * 8); e < 8; e++) piece[e] = __float2bfloat16_rn(0.f);
          }
        }
        fence_proxy_async_smem();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[bsel]);   // one arrival per softmax warp
    }
    if (ok) {
      if (!mbar_wait(&pv_done[(nblk - 1) & 1], ((nblk - 1) >> 1) & 1, abort_flag)) { atomicExch(status, 20); ok = false; }
    }
    if (ok) {
      tc_fence_after();
      float inv = l > 0.f ? 1.0f / l : 0.f;
      if (gate && row_valid) inv *= 1.0f / (1.0f + expf(-__bfloat162float(gate[(m_base + pi) * gate_stride + h0 + g])));
      uint4* orow = reinterpret_cast<uint4*>(out + ((m_base + pi) * nh + h0 + g) * HD);
#pragma unroll
      for (int hcol = 0; hcol < HD; hcol += 32) {
        uint32_t o[32];
        tmem_ld32(t_o + lane_base + hcol, o);
        tmem_ld_wait();
        if (row_valid) {
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            uint4 w;
            uint32_t* wp = reinterpret_cast<uint32_t*>(&w);
#pragma unroll
            for (int e = 0; e < 4; e++) {
              __nv_bfloat162 pp = __floats2bfloat162_rn(__uint_as_float(o[c + 2 * e]) * inv, __uint_as_float(o[c + 2 * e + 1]) * inv);
              wp[e] = *reinterpret_cast<uint32_t*>(&pp);
            }
            orow[(hcol + c) / 8] = w;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem, 256);
}

LEB_API int leb_attention_prefill_tc_supported(int nh, int nkv, int hd, int page_size) {
  if (hd != 64 || page_size != 64 || nkv <= 0 || nh % nkv != 0) return 0;
  const int G = nh / nkv;
  return G == 1 || G == 2 || G == 4 || G == 8;
}

// Prompt attention of the step's rows over the paged cache (which already holds their keys and
// values).  q: [M, nh*64] with row stride q_stride; k_pool [n_pages][nkv][64][64], v_pool
// [n_pages][nkv][64 dims][64 positions]; out [M, nh*64].  status: device int, set non-zero by a
// block whose bounded wait gave up.
LEB_API int leb_attention_prefill_tc(void* out, const void* q, int q_stride, int M, const void* k_pool,
                                     const void* v_pool, int n_pages, const int* block_table, int bt_width,
                                     const int* seq_slot, const int* seq_pos0, const int* seq_qstart,
                                     const int* seq_qlen, const void* gate, int gate_stride, int B, int nh, int nkv,
                                     int hd, int page_size, int window, float scale, int max_qlen, int* status,
                                     cudaStream_t st) {
  if (B <= 0 || max_qlen <= 0 || M <= 0) return 0;
  LEB_REQUIRE(leb_attention_prefill_tc_supported(nh, nkv, hd, page_size),
              "leb_attention_prefill_tc: sizes not taken (heads %d, kv heads %d, head_dim %d, page %d)", nh, nkv, hd, page_size);
  LEB_REQUIRE(status != nullptr, "leb_attention_prefill_tc: a status word is required");
  LEB_REQUIRE(((uintptr_t)q & 15) == 0 && q_stride % 8 == 0 && ((uintptr_t)out & 15) == 0,
              "leb_attention_prefill_tc: q and out must be 16-byte aligned, q's row stride a multiple of 8");
  const int G = nh / nkv, TP = 128 / G;
  CUtensorMap mq, mk, mv;
  if (tensor_map(&mq, q, M, nh * hd, q_stride, TP)) return 1;
  if (tensor_map(&mk, k_pool, n_pages * nkv * page_size, hd, hd, page_size)) return 1;
  if (tensor_map(&mv, v_pool, n_pages * nkv * hd, page_size, page_size, hd)) return 1;
  dim3 grid(nkv, ceil_div(max_qlen, TP), B);
  LEB_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "leb_attention_prefill_tc: grid too large");
  const size_t smem = 1024 + 128 * 64 * 2 + 2 * ATC_STAGES * 64 * 64 * 2;
#define LEB_ATC(GS_)                                                                                              \
  {                                                                                                               \
    static bool set = false;                                                                                      \
    if (!set) {                                                                                                   \
      if (cudaFuncSetAttribute(attention_prefill_tc_kernel<GS_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) \
        return leb_fail("leb_attention_prefill_tc: %zu bytes of shared memory per block refused", smem);        \
      set = true;                                                                                                 \
    }                                                                                                             \
    leb_launch(attention_prefill_tc_kernel<GS_>, grid, dim3(ATC_THREADS), smem, st,                               \
        mq, mk, mv, (bf16*)out, block_table, bt_width, seq_slot, seq_pos0, seq_qstart, seq_qlen, (const bf16*)gate, \
        gate_stride, nh, nkv, window, scale, status);                                                             \
  }
  switch (G) {
    case 1: LEB_ATC(1); break;
    case 2: LEB_ATC(2); break;
    case 4: LEB_ATC(4); break;
    default: LEB_ATC(8); break;
  }
#undef LEB_ATC
  LEB_CHECK_LAUNCH("leb_attention_prefill_tc");
  return 0;
}
