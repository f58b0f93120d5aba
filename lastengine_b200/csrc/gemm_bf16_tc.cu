// bfloat16 matrix product on the 5th-generation tensor cores (tcgen05) for prompts:
//   C[M,N] (+)= A[M,K] . W[N,K]^T, float accumulation in tensor memory.
//
// The reference multiplies prompt chunks with tiled mma.sync kernels over weights it
// dequantises into shared memory (src/cuda/kernels.cu:965-1235, tiles 64x64 to 128x128).  Here
// a block works through 128 x BN tiles (one block per SM, tiles dealt out round-robin):
//   warps 0, 6  one thread each issues the TMA loads (cp.async.bulk.tensor, 128-byte swizzle) of the
//            A tiles (warp 0) and the W tiles (warp 6) of 64 k-values into a ring of shared-memory
//            stages; issuing a TMA load costs its thread some hundred cycles, so two threads
//            keep the ring fuller than one;
//   warp 1   allocates tensor memory; one thread issues tcgen05.mma (128 x BN x 16 per
//            instruction, operands from shared memory through descriptors, accumulator in tensor
//            memory) and commits each stage back to the producer;
//   warps 2-5  wait for the accumulator, read it with tcgen05.ld (32 rows per warp, 32 columns at
//            a time) and apply the epilogue: store, add into the float residual, or SwiGLU over
//            gate/up rows interleaved in blocks of 16.
// Tensor memory holds two accumulators, so the epilogue of one tile runs while the products of
// the next are issued.
// Rows and columns beyond M, N and K are zero-filled by TMA and masked in the epilogue, so any
// M, N and any K that is a multiple of 8 are taken.
//
// Every wait on an mbarrier is bounded: when a wait gives up, the block records where in
// *status, every role leaves its loop, tensor memory is freed, and the block returns.
#include "tc_common.cuh"

#define TC_MAX_GROUPS 256

// GROUPED: rows [off[e], off[e+1]) of A and C go with expert e's weights, rows [e*N, (e+1)*N) of the
// stacked W.  The offsets are made on the device by the step itself, so the tiles (expert, 128
// rows of it, BN weight rows) are counted in the kernel: a running count of tiles per expert in
// shared memory, and every role walks the tiles b, b + grid, ... of that list.  A tile's last
// rows may belong to the next expert: they are computed and not stored.
// Not GROUPED, n_groups > 1: K is cut into that many slices as well (products of a few hundred rows
// have fewer 128 x BN tiles than there are SMs); tile t is then slice t % slices of tile t / slices,
// TC is float, C the workspace [slices][M][N] and the epilogue a plain store: a second kernel
// (slices_finish) adds the slices up in order and applies the real epilogue.
template <typename TC, int BN, int STAGES, bool GROUPED>
__global__ void __launch_bounds__(TC_THREADS)
gemm_bf16_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    TC* __restrict__ C_all, int M, int N, int K, int ldc, int epilogue, int* __restrict__ status,
                    const int* __restrict__ group_offsets, int n_groups) {
  __shared__ int g_cum[GROUPED ? TC_MAX_GROUPS + 1 : 1], g_off[GROUPED ? TC_MAX_GROUPS + 1 : 1];
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment for the swizzled tiles
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  constexpr int A_BYTES = TC_BM * TC_BK * 2, B_BYTES = BN * TC_BK * 2;
  uint8_t* sa = smem;
  uint8_t* sb = smem + STAGES * A_BYTES;
  uint64_t* full = (uint64_t*)(sb + STAGES * B_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;      // [2]
  uint64_t* acc_empty = acc_full + 2;       // [2]
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  float* stage_out = (float*)(tmem_slot + 4);   // 4 warps x 32 rows x 36 floats for the epilogue

  pdl_trigger();   // the next kernel may set itself up meanwhile
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nk = (K + TC_BK - 1) / TC_BK;
  const int m_tiles = (M + TC_BM - 1) / TC_BM, n_tiles = (N + BN - 1) / BN;
  const int n_slices = GROUPED ? 1 : max(1, n_groups);
  const int k_per = (nk + n_slices - 1) / n_slices;     // k-blocks of a slice (the last may have fewer)
  int num_tiles = m_tiles * n_tiles * n_slices;  // tile t: rows (t % m_tiles), columns (t / m_tiles):
                                                 // blocks running together share weight tiles in L2

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) {
      mbar_init(&full[s], 2);    // the two producers each announce their bytes
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; i++) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 4);   // one arrival per epilogue warp
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * BN);   // two accumulators of BN columns x 128 lanes x 32 bits
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_acc = *tmem_slot;
  pdl_wait();      // barriers and tensor memory are set up; now the kernel before must be done
  if (GROUPED) {
    for (int e = threadIdx.x; e <= n_groups; e += blockDim.x) g_off[e] = group_offsets[e];
    __syncthreads();
    if (threadIdx.x == 0) {
      int c = 0;
      for (int e = 0; e < n_groups; e++) {
        g_cum[e] = c;
        c += ((g_off[e + 1] - g_off[e] + TC_BM - 1) / TC_BM) * n_tiles;
      }
      g_cum[n_groups] = c;
    }
    __syncthreads();
    num_tiles = g_cum[n_groups];
  }
  // where a tile lies: first row of A and C, the row its rows end at, first column of C, first
  // row of W, and the index of its column tile
  auto place = [&](int tile, int& m0, int& m_end, int& n0, int& w0, int& nt, int& kb_lo, int& kb_n) {
    kb_lo = 0;
    kb_n = nk;
    if (!GROUPED && n_slices > 1) {
      const int slice = tile % n_slices;
      tile /= n_slices;
      kb_lo = slice * k_per;
      kb_n = max(0, min(nk, kb_lo + k_per) - kb_lo);
    }
    if (GROUPED) {
      int lo = 0, hi = n_groups;   // the expert with g_cum[lo] <= tile < g_cum[lo + 1]
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (g_cum[mid] <= tile) lo = mid; else hi = mid;
      }
      const int local = tile - g_cum[lo];
      const int mt = (g_off[lo + 1] - g_off[lo] + TC_BM - 1) / TC_BM;
      nt = local / mt;
      m0 = g_off[lo] + (local % mt) * TC_BM;
      m_end = g_off[lo + 1];
      n0 = nt * BN;
      w0 = lo * N + n0;
    } else {
      nt = tile / m_tiles;
      m0 = (tile % m_tiles) * TC_BM;
      m_end = M;
      n0 = nt * BN;
      w0 = n0;
    }
  };

  if (warp == 0 || warp == 6) {
    if (lane == 0) {
      const bool loads_a = warp == 0;
      uint32_t it = 0;   // k-slices loaded so far, over all tiles of this block
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int m0, m_end, n0, w0, nt, kb_lo, kb_n;
        place(tile, m0, m_end, n0, w0, nt, kb_lo, kb_n);
        for (int kb = 0; kb < kb_n; kb++, it++) {
          const int s = it % STAGES;
          if (!mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1, abort_flag)) { atomicExch(status, 1); ok = false; break; }
          mbar_expect_tx(&full[s], loads_a ? A_BYTES : B_BYTES);
          // Tiles that share rows of A start their walk over k at different places, so that
          // blocks running in step do not all ask L2 for the same lines at the same moment.
          const int kk = kb_lo + (kb + nt * 5) % kb_n;
          if (loads_a) tma_load_2d(sa + s * A_BYTES, &map_a, &full[s], kk * TC_BK, m0);
          else tma_load_2d(sb + s * B_BYTES, &map_w, &full[s], kk * TC_BK, w0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // instruction descriptor: float accumulator, bfloat16 A and B, both K-major, N, M
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
      bool ok = true;
      uint32_t it = 0, t = 0;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, t++) {
        const uint32_t buf = t & 1;
        // the epilogue must have emptied this accumulator (two tiles ago)
        if (!mbar_wait(&acc_empty[buf], ((t >> 1) & 1) ^ 1, abort_flag)) { atomicExch(status, 4); ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_acc + buf * BN;
        const int kb_n = n_slices > 1 ? max(0, min(nk, (tile % n_slices + 1) * k_per) - (tile % n_slices) * k_per) : nk;
        for (int kb = 0; kb < kb_n; kb++, it++) {
          const int s = it % STAGES;
          if (!mbar_wait(&full[s], (it / STAGES) & 1, abort_flag)) { atomicExch(status, 2); ok = false; break; }
          tc_fence_after();
          const uint64_t da = make_desc(smem_u32(sa + s * A_BYTES));
          const uint64_t db = make_desc(smem_u32(sb + s * B_BYTES));
#pragma unroll
          for (int k = 0; k < TC_BK / 16; k++)   // 16 k-values = 32 bytes along the swizzled row
            umma_bf16(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb | k) != 0);
          umma_commit(&empty[s]);   // the stage is free once these products have read it
        }
        if (ok) umma_commit(&acc_full[buf]);
      }
    }
  } else {
    // epilogue warps: tensor-memory lanes 32*(warp%4) .. +31 are rows of the tile
    const int quad = warp & 3;
    // Each warp stages its 32 rows of a 32-column piece in shared memory (the pipeline's first
    // stage, free once the accumulator is complete) and writes them out row by row, so that a
    // store covers whole 128-byte lines instead of one element in each of 32 rows.
    float* stg = stage_out + quad * (32 * 36);
    uint32_t t = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, t++) {
    int m0, m_end, n0, w0, nt, kb_lo, kb_n;
    place(tile, m0, m_end, n0, w0, nt, kb_lo, kb_n);
    TC* const C = C_all + (n_slices > 1 ? (size_t)(tile % n_slices) * M * ldc : 0);   // a slice's part of the workspace
    const uint32_t buf = t & 1;
    const int row_base = m0 + quad * 32;
    // adding epilogue with 16-byte rows: a lane's eight old values (rows lane/8 + 4j, four columns
    // from (lane%8)*4) of a 32-column piece; the first piece's are on their way while the products run
    float4 nxt[8];
    auto load_old = [&](int c0) {
      const int col = n0 + c0 + (lane & 7) * 4;
#pragma unroll
      for (int j = 0; j < 8; j++) {
        const int row = row_base + (lane >> 3) + 4 * j;
        nxt[j] = (row < m_end && col + 3 < N) ? __ldcs(reinterpret_cast<const float4*>(C + (size_t)row * ldc + col))
                                              : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    };
    if (epilogue == 1 && sizeof(TC) == 4 && (ldc % 4 == 0) && (((uintptr_t)C % 16) == 0)) load_old(0);
    bool ok = mbar_wait(&acc_full[buf], (t >> 1) & 1, abort_flag);
    if (!ok && lane == 0) atomicExch(status, 3);
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;   // the warp leaves together
    if (!ok) break;
    tc_fence_after();
    {
      const int ncols = epilogue == 2 ? 16 : 32;          // output columns per piece
      const int n_out = epilogue == 2 ? N / 2 : N;
      const int lpr = ncols / 4, rpp = 32 / lpr;          // lanes per row, rows per pass
      const int lr = lane / lpr, lc = (lane % lpr) * 4;
      const bool vec = (ldc % 4 == 0) && (((uintptr_t)C % 16) == 0);
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t v[32];
        tmem_ld32(tmem_acc + ((uint32_t)(quad * 32) << 16) + buf * BN + (uint32_t)c0, v);
        tmem_ld_wait();
        float* mine = stg + lane * 36;
        if (epilogue == 2) {
          // columns c0..c0+15 gate, c0+16..c0+31 up of outputs (n0 + c0)/2 + i
#pragma unroll
          for (int i = 0; i < 16; i += 4) {
            float4 f;
            float* fp = reinterpret_cast<float*>(&f);
#pragma unroll
            for (int e = 0; e < 4; e++) {
              const float g = __uint_as_float(v[i + e]), u = __uint_as_float(v[16 + i + e]);
              fp[e] = silu_mul<TC>(g, u);
            }
            *reinterpret_cast<float4*>(mine + i) = f;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            *reinterpret_cast<float4*>(mine + i) = make_float4(__uint_as_float(v[i]), __uint_as_float(v[i + 1]),
                                                                __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
        }
        __syncwarp();
        const int col = (epilogue == 2 ? ((n0 + c0) >> 1) : (n0 + c0)) + lc;
        if (epilogue == 1 && sizeof(TC) == 4 && vec && col + 3 < n_out) {
          // adding into the residual: the old values of this piece were asked for a piece ago (the
          // first before the products were complete); now ask for the next piece's, so that they
          // travel under this piece's stores
          float4 old[8];
#pragma unroll
          for (int it = 0; it < 8; it++) old[it] = nxt[it];
          if (c0 + 32 < BN) load_old(c0 + 32);
#pragma unroll
          for (int it = 0; it < 8; it++) {
            const int rr = lr + 4 * it, row = row_base + rr;
            if (row >= m_end) continue;
            const float4 f = *reinterpret_cast<const float4*>(stg + rr * 36 + lc);
            *reinterpret_cast<float4*>(C + (size_t)row * ldc + col) =
                make_float4(f.x + old[it].x, f.y + old[it].y, f.z + old[it].z, f.w + old[it].w);
          }
          __syncwarp();
          continue;
        }
        for (int rr = lr; rr < 32; rr += rpp) {
          const int row = row_base + rr;
          if (row >= m_end || col >= n_out) continue;
          float4 f = *reinterpret_cast<const float4*>(stg + rr * 36 + lc);
          TC* o = C + (size_t)row * ldc + col;
          if (vec && col + 3 < n_out) {
            if (sizeof(TC) == 4) {
              float4* o4 = reinterpret_cast<float4*>(o);
              if (epilogue == 1) {
                const float4 old = *o4;
                f.x += old.x; f.y += old.y; f.z += old.z; f.w += old.w;
              }
              *o4 = f;
            } else {
              __nv_bfloat162 lo = __floats2bfloat162_rn(f.x, f.y), hi = __floats2bfloat162_rn(f.z, f.w);
              uint2 pk = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
              *reinterpret_cast<uint2*>(o) = pk;
            }
          } else {
            const float* fp = reinterpret_cast<const float*>(&f);
            for (int e = 0; e < 4 && col + e < n_out; e++) {
              float a = fp[e];
              if (epilogue == 1) a += to_f32(o[e]);
              o[e] = from_f32<TC>(a);
            }
          }
        }
        __syncwarp();
      }
    }
    // this warp has read its part of the accumulator: hand the buffer back to the issuing thread
    tc_fence_before();
    __syncwarp();
    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&acc_empty[buf])) : "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_acc, 2 * BN);
  }
}

template <typename TC, int BN, int STAGES, bool GROUPED = false>
static int launch_tc(void* C, const CUtensorMap& ma, const CUtensorMap& mw, int M, int N, int K, int ldc,
                     int epilogue, int* status, cudaStream_t st, const int* group_offsets = nullptr, int n_groups = 0) {
  constexpr size_t smem = (size_t)STAGES * (TC_BM * TC_BK * 2 + BN * TC_BK * 2) + (2 * STAGES + 4) * 8 + 16 +
                          4 * 32 * 36 * 4 + 1024;
  auto kern = gemm_bf16_tc_kernel<TC, BN, STAGES, GROUPED>;
  static bool set = false;
  if (!set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return leb_fail("leb_gemm_bf16_tc: shared memory %zu: %s", smem, cudaGetErrorString(e));
    set = true;
  }
  static int n_sm = 0;
  if (!n_sm) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sm <= 0) n_sm = 148;
  }
  // grouped: the most tiles the offsets can give (every expert may end with a partly filled tile)
  const long tiles = (long)ceil_div(N, BN) * (ceil_div(M, TC_BM) + (GROUPED ? n_groups : 0)) * (!GROUPED && n_groups > 1 ? n_groups : 1);
  dim3 grid((unsigned)(tiles < n_sm ? tiles : n_sm));
  leb_launch(kern, grid, dim3(TC_THREADS), smem, st, ma, mw, (TC*)C, M, N, K, ldc, epilogue, status, group_offsets,
             n_groups);
  LEB_CHECK_LAUNCH("leb_gemm_bf16_tc");
  return 0;
}

// Returns 1 when the operands can go through TMA (16-byte aligned bases and row strides).
LEB_API int leb_gemm_bf16_tc_supported(const void* A, const void* W, int K, int lda) {
  return K > 0 && K % 8 == 0 && lda % 8 == 0 && ((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0;
}

// epilogue: 0 store, 1 add into float C, 2 SwiGLU over 16/16 interleaved gate/up rows (C has N/2 columns).
// status: device int, set non-zero by a block whose bounded wait gave up.
LEB_API int leb_gemm_bf16_tc(void* C, int c_dtype, const void* A, const void* W, int M, int N, int K, int lda,
                             int ldc, int epilogue, int* status, cudaStream_t st) {
  if (M <= 0 || N <= 0) return 0;
  LEB_REQUIRE(leb_gemm_bf16_tc_supported(A, W, K, lda), "leb_gemm_bf16_tc: operands not aligned for TMA (K %d, lda %d)", K, lda);
  LEB_REQUIRE(epilogue >= 0 && epilogue <= 2, "leb_gemm_bf16_tc: unknown epilogue %d", epilogue);
  LEB_REQUIRE(epilogue != 1 || c_dtype == LEB_F32, "leb_gemm_bf16_tc: adding needs a float C");
  LEB_REQUIRE(epilogue != 2 || N % 32 == 0, "leb_gemm_bf16_tc: the SwiGLU epilogue needs N (%d) to be a multiple of 32", N);
  LEB_REQUIRE(status != nullptr, "leb_gemm_bf16_tc: a status word is required");
  // wide tiles read less per flop; narrow ones spread a small product over more SMs
  // With few rows (a decode step of some dozens of sequences) the product is bound by reading W:
  // narrow tiles then give every SM a stripe of W to stream.
  const long m_tiles = ceil_div(M, TC_BM);
  int BN = 32;
  if (N > 128 && m_tiles * ceil_div(N, 256) >= 64) BN = 256;
  else if (m_tiles * ceil_div(N, 128) >= 96) BN = 128;
  else if (m_tiles * ceil_div(N, 64) >= 96) BN = 64;
  CUtensorMap ma, mw;
  if (tensor_map(&ma, A, M, K, lda, TC_BM)) return 1;
  if (tensor_map(&mw, W, N, K, K, BN)) return 1;
  if (c_dtype == LEB_BF16) {
    if (BN == 256) return launch_tc<bf16, 256, 4>(C, ma, mw, M, N, K, ldc, epilogue, status, st);
    if (BN == 128) return launch_tc<bf16, 128, 6>(C, ma, mw, M, N, K, ldc, epilogue, status, st);
    if (BN == 64) return launch_tc<bf16, 64, 8>(C, ma, mw, M, N, K, ldc, epilogue, status, st);
    return launch_tc<bf16, 32, 8>(C, ma, mw, M, N, K, ldc, epilogue, status, st);
  }
  if (c_dtype == LEB_F32) {
    if (BN == 256) return launch_tc<float, 256, 4>(C, ma, mw, M, N, K, ldc, epilogue, status, st);
    if (BN == 128) return launch_tc<float, 128, 6>(C, ma, mw, M, N, K, ldc, epilogue, status, st);
    if (BN == 64) return launch_tc<float, 64, 8>(C, ma, mw, M, N, K, ldc, epilogue, status, st);
    return launch_tc<float, 32, 8>(C, ma, mw, M, N, K, ldc, epilogue, status, st);
  }
  return leb_fail("leb_gemm_bf16_tc: unknown C dtype %d", c_dtype);
}

// Into how many slices of K a product of M rows is cut (1: not at all): with 256-wide tiles fewer
// than half as many tiles as SMs, K of 4096 or more and at least 16 k-blocks of 64 per slice (the
// slices' trip through the workspace and the second kernel cost some 6 us: measured at K = 2048,
// 4 slices of 8 k-blocks made a 512-row product slower, 14 -> 20 us, where K = 5632 gained, 30 -> 27 us,
// and at 192 rows 29 -> 19 us).  The caller sizes the workspace (slices * M * N floats) with it.
LEB_API int leb_gemm_bf16_tc_slices(int M, int N, int K) {
  const int nk = ceil_div(K, TC_BK), n_sm = sm_count();
  const long tiles = (long)ceil_div(M, TC_BM) * ceil_div(N, 256);
  if (N < 256 || nk < 64 || tiles * 2 > n_sm) return 1;
  int s = (int)(n_sm / tiles);
  if (s > nk / 16) s = nk / 16;
  if (s > 8) s = 8;
  if (s < 2) return 1;
  const int per = ceil_div(nk, s);
  return ceil_div(nk, per);
}

// The product with K cut into n_slices (from leb_gemm_bf16_tc_slices): the slices' partial tiles go to
// `part` [n_slices][M][N] float, and the second kernel of the sliced decode product adds them up in
// slice order and applies the epilogue.
LEB_API int leb_gemm_bf16_tc_sliced(void* C, int c_dtype, const void* A, const void* W, int M, int N, int K, int lda,
                                    int ldc, int epilogue, float* part, int n_slices, int* status, cudaStream_t st) {
  if (M <= 0 || N <= 0) return 0;
  LEB_REQUIRE(leb_gemm_bf16_tc_supported(A, W, K, lda), "leb_gemm_bf16_tc_sliced: operands not aligned for TMA (K %d, lda %d)", K, lda);
  LEB_REQUIRE(epilogue >= 0 && epilogue <= 2, "leb_gemm_bf16_tc_sliced: unknown epilogue %d", epilogue);
  LEB_REQUIRE(epilogue != 1 || c_dtype == LEB_F32, "leb_gemm_bf16_tc_sliced: adding needs a float C");
  LEB_REQUIRE(epilogue != 2 || N % 32 == 0, "leb_gemm_bf16_tc_sliced: the SwiGLU epilogue needs N (%d) to be a multiple of 32", N);
  LEB_REQUIRE(status != nullptr && part != nullptr, "leb_gemm_bf16_tc_sliced: a status word and the slices' workspace are required");
  const int nk = ceil_div(K, TC_BK);
  LEB_REQUIRE(n_slices >= 2 && n_slices <= nk && ceil_div(nk, ceil_div(nk, n_slices)) == n_slices,
              "leb_gemm_bf16_tc_sliced: %d slices leave one of them without a k-block (K %d)", n_slices, K);
  LEB_REQUIRE(N % 4 == 0, "leb_gemm_bf16_tc_sliced: N (%d) must be a multiple of 4", N);
  CUtensorMap ma, mw;
  if (tensor_map(&ma, A, M, K, lda, TC_BM)) return 1;
  if (tensor_map(&mw, W, N, K, K, 256)) return 1;
  if (launch_tc<float, 256, 4>(part, ma, mw, M, N, K, N, 0, status, st, nullptr, n_slices)) return 1;
  return leb_slices_finish(C, c_dtype, part, M, N, ldc, epilogue, n_slices, st);
}

// Grouped form for experts with many rows each (prompts): A [P, K] and C sorted by expert, rows
// [group_offsets[e], group_offsets[e+1]) with the weights W[e] ([n_groups, N, K] stacked);
// group_offsets [n_groups + 1] lives on the device.
LEB_API int leb_gemm_bf16_tc_grouped(void* C, int c_dtype, const void* A, const void* W, int P, int N, int K, int lda,
                                     int ldc, int epilogue, const int* group_offsets, int n_groups, int* status,
                                     cudaStream_t st) {
  if (P <= 0 || N <= 0 || n_groups <= 0) return 0;
  LEB_REQUIRE(n_groups <= TC_MAX_GROUPS, "leb_gemm_bf16_tc_grouped: %d groups; at most %d", n_groups, TC_MAX_GROUPS);
  LEB_REQUIRE(leb_gemm_bf16_tc_supported(A, W, K, lda), "leb_gemm_bf16_tc_grouped: operands not aligned for TMA (K %d, lda %d)", K, lda);
  LEB_REQUIRE(epilogue >= 0 && epilogue <= 2, "leb_gemm_bf16_tc_grouped: unknown epilogue %d", epilogue);
  LEB_REQUIRE(epilogue != 1 || c_dtype == LEB_F32, "leb_gemm_bf16_tc_grouped: adding needs a float C");
  LEB_REQUIRE(epilogue != 2 || N % 32 == 0, "leb_gemm_bf16_tc_grouped: the SwiGLU epilogue needs N (%d) to be a multiple of 32", N);
  LEB_REQUIRE(status != nullptr && group_offsets != nullptr, "leb_gemm_bf16_tc_grouped: a status word and the offsets are required");
  LEB_REQUIRE((long)n_groups * N < (1L << 31), "leb_gemm_bf16_tc_grouped: %d x %d weight rows do not fit a tensor map coordinate", n_groups, N);
  CUtensorMap ma, mw;
  if (tensor_map(&ma, A, P, K, lda, TC_BM)) return 1;
  if (N > 128) {
    if (tensor_map(&mw, W, n_groups * N, K, K, 256)) return 1;
    if (c_dtype == LEB_BF16) return launch_tc<bf16, 256, 4, true>(C, ma, mw, P, N, K, ldc, epilogue, status, st, group_offsets, n_groups);
    if (c_dtype == LEB_F32) return launch_tc<float, 256, 4, true>(C, ma, mw, P, N, K, ldc, epilogue, status, st, group_offsets, n_groups);
  } else {
    if (tensor_map(&mw, W, n_groups * N, K, K, 64)) return 1;
    if (c_dtype == LEB_BF16) return launch_tc<bf16, 64, 8, true>(C, ma, mw, P, N, K, ldc, epilogue, status, st, group_offsets, n_groups);
    if (c_dtype == LEB_F32) return launch_tc<float, 64, 8, true>(C, ma, mw, P, N, K, ldc, epilogue, status, st, group_offsets, n_groups);
  }
  return leb_fail("leb_gemm_bf16_tc_grouped: unknown C dtype %d", c_dtype);
}
