// bfloat16 matrix product for up to 16 rows (the decode step):  C[M,N] (+)= A[M,K] . W[N,K]^T,
// float accumulate, built as a pipelined stream of the weights through shared memory.
//
// Such a product is bound by reading W once (the reference's decode matvec is one pass over the
// weight rows too, src/cuda/kernels.cu:371-392), and a stream is only as fast as the bytes it
// keeps in flight.  Registers hold too few: a warp that loads a batch of weights, waits and
// multiplies pays the memory latency once per batch.  Here every warp owns a ring of S stages in
// shared memory and keeps S-1 asynchronous copies (cp.async, 16 bytes per lane, straight from
// L2 to shared memory) in flight at all times; the weight copies of the first stages are issued
// before the kernel waits for its predecessor, since weights do not depend on it.  A stage
// holds the activations of its 64 values of k as well, so nothing in the loop waits on a load.
//
// A block owns tiles of 16*NSUB weight rows; its NW warps split K in chunks of 64 (warp w takes
// chunks w, w+NW, ...) and their partial sums are added in warp order through shared memory, so
// a row's result does not depend on the other rows of the launch.  Blocks are persistent:
// block b takes tiles b, b+grid, ... and its rings run on across tiles, so there is no bubble
// between them.  The tensor-core roles are swapped as in the register kernel: 16 weight rows
// are the "M" side of mma.m16n8k16, 8 activation rows its "N" side, and a lane's 16 bytes
// (8 values of k) feed two mma as k-pairs (0,1)(2,3) and (4,5)(6,7) on both operands.
//
// A stage holds rows of 128 bytes; the 16-byte piece c of row r lies at c ^ 4*(r & 1), so the
// quarter-warps of a 16-byte shared load (rows 2i and 2i+1, four pieces each) hit all 32 banks.
//
// epilogue: 0 store, 1 add into float C, 2 SwiGLU over interleaved weights (rows 32j..32j+15
// gate, 32j+16..32j+31 up of the same 16 outputs; C has N/2 columns), 3 the gated short
// convolution of a decode step: W is the conv mixer's in_proj [3D, K], a tile takes the rows of
// B, C and x of 16 channels (three sub-tiles D rows apart), and the epilogue does what the
// one-token convolution kernel does (shortconv.cu: bx = B*x, taps over the state, y = C*sum,
// state shifted), so the projection never goes to memory and one launch is saved.
#include "stream_common.cuh"

template <typename TC, int MT, int NSUB, int S, int ST_WARPS>
__global__ void __launch_bounds__(32 * ST_WARPS)
gemm_bf16_stream_kernel(TC* __restrict__ C, const bf16* __restrict__ A, const bf16* __restrict__ W,
                        int M, int N, int K, int lda, int ldc, int epilogue, int n_tiles, StreamConv cv, StreamNorm nm) {
  constexpr int ROWS = ST_ROWS * NSUB, XOFF = ROWS * 128, STAGE = (ROWS + 8 * MT) * 128;
  constexpr bool CONV = NSUB == 3;   // the only user of three sub-tiles
  const int D3 = N / 3;
  extern __shared__ __align__(128) unsigned char st_smem[];
  pdl_trigger();
  float (*red)[NSUB][ST_ROWS][8 * MT + 1] =
      reinterpret_cast<float (*)[NSUB][ST_ROWS][8 * MT + 1]>(st_smem + (size_t)ST_WARPS * S * STAGE);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(st_smem) + warp * (S * STAGE);
  const int n_chunks = (K + ST_CHUNK - 1) / ST_CHUNK;
  const int my_chunks = warp < n_chunks ? (n_chunks - warp + ST_WARPS - 1) / ST_WARPS : 0;
  const int my_tiles = (int)blockIdx.x < n_tiles ? (n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const int total = my_tiles * my_chunks;   // this warp's stages, tile after tile

  // producer state: the next stage to ask for
  int p_q = 0, p_tile = blockIdx.x, p_ci = 0;
  auto issue_x = [&](int q, int ci) {   // the activations of stage q (chunk ci of this warp)
    const int k0 = (warp + ST_WARPS * ci) * ST_CHUNK;
    const uint32_t base = ring + (q % S) * STAGE + XOFF;
#pragma unroll
    for (int i = 0; i < 2 * MT; i++) {
      const int row = i * 4 + (lane >> 3), ch = lane & 7;
      const int k = k0 + ch * 8;
      const bool in = row < M && k < K;
      st_cp16(base + row * 128 + ((ch ^ ((row & 1) << 2)) << 4), A + (in ? (size_t)row * lda + k : 0), in ? 16 : 0);
    }
  };
  auto issue = [&](bool with_x) {
    if (p_q < total) {
      const int k0 = (warp + ST_WARPS * p_ci) * ST_CHUNK, n0 = p_tile * ROWS;
      const uint32_t base = ring + (p_q % S) * STAGE;
      if (with_x) issue_x(p_q, p_ci);
#pragma unroll
      for (int i = 0; i < ROWS / 4; i++) {
        const int row = i * 4 + (lane >> 3), ch = lane & 7;
        // convolution: sub-tile i/4 is B, C or x (D rows apart) of the tile's 16 channels
        const int n = CONV ? (i / 4) * D3 + min(p_tile * ST_ROWS + (row & 15), D3 - 1) : min(n0 + row, N - 1);
        const int k = k0 + ch * 8;
        const bool in = k < K;   // K is a multiple of 8: a piece is inside or outside as a whole
        st_cp16(base + row * 128 + ((ch ^ ((row & 1) << 2)) << 4), W + (size_t)n * K + (in ? k : 0), in ? 16 : 0);
      }
      p_q++;
      if (++p_ci == my_chunks) {
        p_ci = 0;
        p_tile += gridDim.x;
      }
    }
    st_commit();   // an empty group where there is nothing left: the count of groups stays in step
  };
#pragma unroll
  for (int i = 0; i < S - 1; i++) issue(false);
  pdl_wait();
  // the activations of those first stages, in one more group (stage i is chunk i % my_chunks)
#pragma unroll
  for (int i = 0; i < S - 1; i++)
    if (i < total) issue_x(i, i % my_chunks);
  st_commit();
  // split norm: warp w adds up the partial sums of squares of rows w, w + warps, ...; the loads go
  // out now and are used after the first tile's product
  constexpr int NR = (8 * MT + ST_WARPS - 1) / ST_WARPS;   // rows a warp looks after
  constexpr int NP = 8;                                    // partial sums a lane holds per row (more: a loop)
  __shared__ float row_scale[8 * MT];
  float ssq_part[NR][NP];
  if (nm.ssq_in) {
#pragma unroll
    for (int a = 0; a < NR; a++) {
      const int row = warp + a * ST_WARPS;
#pragma unroll
      for (int b = 0; b < NP; b++) {
        const int part = lane + 32 * b;
        ssq_part[a][b] = (row < M && part < nm.parts_in) ? nm.ssq_in[(size_t)row * nm.parts_in + part] : 0.f;
      }
    }
  }
  int q = 0;
  for (int ti = 0; ti < my_tiles; ti++) {
    const int tile = blockIdx.x + ti * gridDim.x;
    // convolution: thread t owns (row, channel) pairs t, t + threads, ...; their taps and state are
    // asked for now and used after the product
    constexpr int CV_PAIRS = CONV ? (ST_ROWS * 8 * MT + 32 * ST_WARPS - 1) / (32 * ST_WARPS) : 1;
    float cv_w[CV_PAIRS][ST_CONV_MAX_LC], cv_s[CV_PAIRS][ST_CONV_MAX_LC - 1], cv_b[CV_PAIRS];
    int cv_slot[CV_PAIRS];
    if constexpr (CONV) {
#pragma unroll
      for (int u = 0; u < CV_PAIRS; u++) {
        const int idx = threadIdx.x + u * 32 * ST_WARPS;
        const int col = idx / ST_ROWS, chn = tile * ST_ROWS + idx % ST_ROWS;
        const bool in = idx < ST_ROWS * 8 * MT && col < M && chn < D3;
        cv_slot[u] = in ? cv.seq_slot[cv.row_seq[col]] : -1;
        cv_b[u] = (in && cv.bias) ? cv.bias[chn] : 0.f;
#pragma unroll
        for (int k = 0; k < ST_CONV_MAX_LC; k++) cv_w[u][k] = (in && k < cv.Lc) ? cv.w[(size_t)chn * cv.Lc + k] : 0.f;
#pragma unroll
        for (int k = 0; k < ST_CONV_MAX_LC - 1; k++)
          cv_s[u][k] = (cv_slot[u] >= 0 && k < cv.Lc - 1) ? cv.state[((size_t)cv_slot[u] * D3 + chn) * (cv.Lc - 1) + k] : 0.f;
      }
    }
    // an adding product: the old values of C (and the next norm's weight) are asked for now and
    // used after the product, so the tail of the kernel does not wait for them
    constexpr int EPT = (ROWS * 8 * MT + 32 * ST_WARPS - 1) / (32 * ST_WARPS);   // outputs a thread writes per tile
    float c_old[EPT], g_next[EPT];
    if (!CONV && epilogue == 1) {
#pragma unroll
      for (int u = 0; u < EPT; u++) {
        const int idx = threadIdx.x + u * 32 * ST_WARPS;
        const int col = idx / ROWS, n = tile * ROWS + idx % ROWS;
        const bool in = idx < ROWS * 8 * MT && col < M && n < N;
        c_old[u] = in ? to_f32(C[(size_t)col * ldc + n]) : 0.f;
        g_next[u] = (in && nm.emit_vals) ? nm.emit_g[n] : 0.f;
      }
    }
    float acc[NSUB][MT][4];
#pragma unroll
    for (int s = 0; s < NSUB; s++)
#pragma unroll
      for (int t = 0; t < MT; t++)
#pragma unroll
        for (int e = 0; e < 4; e++) acc[s][t][e] = 0.f;
    for (int ci = 0; ci < my_chunks; ci++, q++) {
      // the first stages' activations came in one group after all their weights: wait for all
      if (q == 0) st_wait<0>(); else st_wait<S - 2>();
      __syncwarp();      // every lane's copies of stage q have landed; everyone is done with stage q-1
      issue(true);       // refills the slot of stage q-1
      const uint32_t base = ring + (q % S) * STAGE;
#pragma unroll
      for (int j = 0; j < 2; j++) {
        const uint32_t off = g * 128 + (((4 * j + t4) ^ ((g & 1) << 2)) << 4);
        uint4 xc[MT];
#pragma unroll
        for (int t = 0; t < MT; t++) xc[t] = st_lds(base + XOFF + t * 8 * 128 + off);
#pragma unroll
        for (int s = 0; s < NSUB; s++) {
          const uint4 w0 = st_lds(base + s * ST_ROWS * 128 + off), w1 = st_lds(base + s * ST_ROWS * 128 + off + 8 * 128);
#pragma unroll
          for (int t = 0; t < MT; t++) {
            st_mma(acc[s][t], w0.x, w1.x, w0.y, w1.y, xc[t].x, xc[t].y);
            st_mma(acc[s][t], w0.z, w1.z, w0.w, w1.w, xc[t].z, xc[t].w);
          }
        }
      }
    }
    // accumulator fragment: [0] (row g, col 2 t4) [1] (g, 2 t4 + 1) [2] (g + 8, 2 t4) [3] (g + 8, 2 t4 + 1)
#pragma unroll
    for (int s = 0; s < NSUB; s++)
#pragma unroll
      for (int t = 0; t < MT; t++) {
        red[warp][s][g][t * 8 + 2 * t4] = acc[s][t][0];
        red[warp][s][g][t * 8 + 2 * t4 + 1] = acc[s][t][1];
        red[warp][s][g + 8][t * 8 + 2 * t4] = acc[s][t][2];
        red[warp][s][g + 8][t * 8 + 2 * t4 + 1] = acc[s][t][3];
      }
    if (ti == 0) {
#pragma unroll
      for (int a = 0; a < NR; a++) {
        const int row = warp + a * ST_WARPS;
        float sum = 0.f;
        if (nm.ssq_in) {
#pragma unroll
          for (int b = 0; b < NP; b++) sum += ssq_part[a][b];
          for (int part = lane + 32 * NP; part < nm.parts_in; part += 32)   // wider rows than 32 * NP tiles
            if (row < M) sum += nm.ssq_in[(size_t)row * nm.parts_in + part];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        }
        if (lane == 0 && row < 8 * MT) row_scale[row] = nm.ssq_in ? 1.0f / sqrtf(sum / (float)nm.d_in + nm.eps) : 1.f;
      }
    }
    __syncthreads();
    if constexpr (CONV) {
      // as shortconv_single_kernel: the projections rounded to bfloat16 as if they had been stored,
      // taps oldest first, the state shifted by one
#pragma unroll
      for (int u = 0; u < CV_PAIRS; u++) {
        const int idx = threadIdx.x + u * 32 * ST_WARPS;
        const int col = idx / ST_ROWS, i = idx % ST_ROWS, chn = tile * ST_ROWS + i;
        if (idx >= ST_ROWS * 8 * MT || col >= M || chn >= D3) continue;
        float pb = 0.f, pc = 0.f, px = 0.f;
#pragma unroll
        for (int w = 0; w < ST_WARPS; w++) {
          pb += red[w][0][i][col];
          pc += red[w][1][i][col];
          px += red[w][2][i][col];
        }
        pb *= row_scale[col];
        pc *= row_scale[col];
        px *= row_scale[col];
        TC* yo = C + (size_t)col * ldc + chn;
        if (cv_slot[u] < 0) {   // padding row
          *yo = from_f32<TC>(0.f);
          continue;
        }
        const float bx = to_f32(from_f32<TC>(pb)) * to_f32(from_f32<TC>(px));
        float acc = cv_b[u];
#pragma unroll
        for (int k = 0; k < ST_CONV_MAX_LC - 1; k++)
          if (k < cv.Lc - 1) acc += cv_w[u][k] * cv_s[u][k];
        float wl = 0.f;
#pragma unroll
        for (int k = 0; k < ST_CONV_MAX_LC; k++)
          if (k == cv.Lc - 1) wl = cv_w[u][k];
        acc += wl * bx;
        float* sc = cv.state + ((size_t)cv_slot[u] * D3 + chn) * (cv.Lc - 1);
#pragma unroll
        for (int k = 0; k < ST_CONV_MAX_LC - 2; k++)
          if (k < cv.Lc - 2) sc[k] = cv_s[u][k + 1];
        sc[cv.Lc - 2] = bx;
        *yo = from_f32<TC>(to_f32(from_f32<TC>(pc)) * acc);
      }
    } else if (epilogue == 2) {
      // NSUB == 2: sub-tile 0 holds the gate rows, sub-tile 1 the up rows of outputs 16 * tile + i
      const int jbase = tile * ST_ROWS;
      for (int idx = threadIdx.x; idx < ST_ROWS * 8 * MT; idx += blockDim.x) {
        const int col = idx / ST_ROWS, i = idx % ST_ROWS;   // consecutive threads: consecutive outputs
        if (col >= M || 2 * (jbase + i) >= N) continue;
        float gt = 0.f, up = 0.f;
#pragma unroll
        for (int w = 0; w < ST_WARPS; w++) {
          gt += red[w][0][i][col];
          up += red[w][NSUB - 1][i][col];
        }
        gt *= row_scale[col];
        up *= row_scale[col];
        C[(size_t)col * ldc + jbase + i] = from_f32<TC>(silu_mul<TC>(gt, up));
      }
    } else {
      const int n0 = tile * ROWS;
      // ROWS * 8 * MT is a multiple of the block's threads or smaller than them, and ROWS a multiple
      // of 16: the 16 lanes of a half-warp hold 16 consecutive columns of one row, all or none
#pragma unroll
      for (int u = 0; u < EPT; u++) {
        const int idx = threadIdx.x + u * 32 * ST_WARPS;
        if (idx >= ROWS * 8 * MT) break;   // whole warps leave together (ROWS * 8 * MT is a multiple of 32)
        const int col = idx / ROWS, rr = idx % ROWS;
        const int n = n0 + rr;
        const bool in = col < M && n < N;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < ST_WARPS; w++) v += red[w][rr / ST_ROWS][rr % ST_ROWS][col];
        v *= row_scale[col];
        if (in) {
          if (epilogue == 1) v += c_old[u];
          C[(size_t)col * ldc + n] = from_f32<TC>(v);
        }
        if (nm.emit_vals) {   // epilogue 1: the new residual, for the norm that follows
          float sq = in ? v * v : 0.f;
#pragma unroll
          for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
          if (in) nm.emit_vals[(size_t)col * N + n] = __float2bfloat16_rn(v * g_next[u]);
          if ((rr & 15) == 0 && in) nm.emit_ssq[(size_t)col * ((N + 15) / 16) + n / 16] = sq;
        }
      }
    }
    __syncthreads();   // the sums are read before the next tile's are written
  }
  st_wait<0>();
}

// The same stream for products grouped by expert: rows [off[e], off[e+1]) of A and C belong to
// expert e, whose weights are W + e * w_group_stride.  The offsets are made on the device by the
// step itself, so the tiles (expert, block of 8*MT rows, 16*NSUB weight rows) are counted here: the
// block builds the running count of tiles per expert in shared memory and takes the tiles
// b, b + grid, ... of that list; experts without rows have no tiles and cost nothing.  Nothing
// is fetched before the wait (the offsets come from the kernel before this one).
#define ST_MAX_GROUPS 256

template <typename TC, int MT, int NSUB, int S, int ST_WARPS>
__global__ void __launch_bounds__(32 * ST_WARPS, 2)
gemm_bf16_stream_grouped_kernel(TC* __restrict__ C, const bf16* __restrict__ A, const bf16* __restrict__ W, int N,
                                int K, int lda, int ldc, int epilogue, const int* __restrict__ group_offsets,
                                int n_groups, size_t w_group_stride) {
  constexpr int ROWS = ST_ROWS * NSUB, XOFF = ROWS * 128, STAGE = (ROWS + 8 * MT) * 128;
  extern __shared__ __align__(128) unsigned char st_smem[];
  __shared__ int cum[ST_MAX_GROUPS + 1], offs[ST_MAX_GROUPS + 1];
  pdl_wait();
  float (*red)[NSUB][ST_ROWS][8 * MT + 1] =
      reinterpret_cast<float (*)[NSUB][ST_ROWS][8 * MT + 1]>(st_smem + (size_t)ST_WARPS * S * STAGE);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(st_smem) + warp * (S * STAGE);
  const int n_tiles_n = (N + ROWS - 1) / ROWS;
  for (int e = threadIdx.x; e <= n_groups; e += blockDim.x) offs[e] = group_offsets[e];
  __syncthreads();
  if (threadIdx.x == 0) {
    int c = 0;
    for (int e = 0; e < n_groups; e++) {
      cum[e] = c;
      c += ((offs[e + 1] - offs[e] + 8 * MT - 1) / (8 * MT)) * n_tiles_n;
    }
    cum[n_groups] = c;
  }
  __syncthreads();
  const int n_tiles = cum[n_groups];
  const int n_chunks = (K + ST_CHUNK - 1) / ST_CHUNK;
  const int my_chunks = warp < n_chunks ? (n_chunks - warp + ST_WARPS - 1) / ST_WARPS : 0;
  const int my_tiles = (int)blockIdx.x < n_tiles ? (n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const int total = my_tiles * my_chunks;

  struct Tile {
    const bf16* w;   // the expert's weights
    int n0, row0, rows;
  };
  auto tile_of = [&](int t) {
    int lo = 0, hi = n_groups;   // the expert e with cum[e] <= t < cum[e + 1] (experts without tiles are passed over)
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (cum[mid] <= t) lo = mid; else hi = mid;
    }
    const int local = t - cum[lo];
    Tile r;
    r.w = W + (size_t)lo * w_group_stride;
    r.n0 = (local % n_tiles_n) * ROWS;
    r.row0 = offs[lo] + (local / n_tiles_n) * (8 * MT);
    r.rows = min(8 * MT, offs[lo + 1] - r.row0);
    return r;
  };

  int p_q = 0, p_tile = blockIdx.x, p_ci = 0;
  Tile pt = my_tiles > 0 ? tile_of(p_tile) : Tile{W, 0, 0, 0};
  auto issue = [&]() {
    if (p_q < total) {
      const int k0 = (warp + ST_WARPS * p_ci) * ST_CHUNK;
      const uint32_t base = ring + (p_q % S) * STAGE;
#pragma unroll
      for (int i = 0; i < 2 * MT; i++) {
        const int row = i * 4 + (lane >> 3), ch = lane & 7;
        const int k = k0 + ch * 8;
        const bool in = row < pt.rows && k < K;
        st_cp16(base + XOFF + row * 128 + ((ch ^ ((row & 1) << 2)) << 4), A + (in ? (size_t)(pt.row0 + row) * lda + k : 0), in ? 16 : 0);
      }
#pragma unroll
      for (int i = 0; i < ROWS / 4; i++) {
        const int row = i * 4 + (lane >> 3), ch = lane & 7;
        const int n = min(pt.n0 + row, N - 1), k = k0 + ch * 8;
        const bool in = k < K;
        st_cp16(base + row * 128 + ((ch ^ ((row & 1) << 2)) << 4), pt.w + (size_t)n * K + (in ? k : 0), in ? 16 : 0);
      }
      p_q++;
      if (++p_ci == my_chunks) {
        p_ci = 0;
        p_tile += gridDim.x;
        if (p_tile < n_tiles) pt = tile_of(p_tile);
      }
    }
    st_commit();
  };
#pragma unroll
  for (int i = 0; i < S - 1; i++) issue();
  int q = 0;
  for (int ti = 0; ti < my_tiles; ti++) {
    const Tile ct = tile_of(blockIdx.x + ti * gridDim.x);
    float acc[NSUB][MT][4];
#pragma unroll
    for (int s = 0; s < NSUB; s++)
#pragma unroll
      for (int t = 0; t < MT; t++)
#pragma unroll
        for (int e = 0; e < 4; e++) acc[s][t][e] = 0.f;
    for (int ci = 0; ci < my_chunks; ci++, q++) {
      st_wait<S - 2>();
      __syncwarp();
      issue();
      const uint32_t base = ring + (q % S) * STAGE;
#pragma unroll
      for (int j = 0; j < 2; j++) {
        const uint32_t off = g * 128 + (((4 * j + t4) ^ ((g & 1) << 2)) << 4);
        uint4 xc[MT];
#pragma unroll
        for (int t = 0; t < MT; t++) xc[t] = st_lds(base + XOFF + t * 8 * 128 + off);
#pragma unroll
        for (int s = 0; s < NSUB; s++) {
          const uint4 w0 = st_lds(base + s * ST_ROWS * 128 + off), w1 = st_lds(base + s * ST_ROWS * 128 + off + 8 * 128);
#pragma unroll
          for (int t = 0; t < MT; t++) {
            st_mma(acc[s][t], w0.x, w1.x, w0.y, w1.y, xc[t].x, xc[t].y);
            st_mma(acc[s][t], w0.z, w1.z, w0.w, w1.w, xc[t].z, xc[t].w);
          }
        }
      }
    }
#pragma unroll
    for (int s = 0; s < NSUB; s++)
#pragma unroll
      for (int t = 0; t < MT; t++) {
        red[warp][s][g][t * 8 + 2 * t4] = acc[s][t][0];
        red[warp][s][g][t * 8 + 2 * t4 + 1] = acc[s][t][1];
        red[warp][s][g + 8][t * 8 + 2 * t4] = acc[s][t][2];
        red[warp][s][g + 8][t * 8 + 2 * t4 + 1] = acc[s][t][3];
      }
    __syncthreads();
    if (epilogue == 2) {
      const int jbase = ct.n0 / 2;   // gate rows 32j..32j+15 and up rows 32j+16..32j+31 give outputs 16j..16j+15
      for (int idx = threadIdx.x; idx < ST_ROWS * 8 * MT; idx += blockDim.x) {
        const int col = idx / ST_ROWS, i = idx % ST_ROWS;
        if (col >= ct.rows || 2 * (jbase + i) >= N) continue;
        float gt = 0.f, up = 0.f;
#pragma unroll
        for (int w = 0; w < ST_WARPS; w++) {
          gt += red[w][0][i][col];
          up += red[w][NSUB - 1][i][col];
        }
        C[(size_t)(ct.row0 + col) * ldc + jbase + i] = from_f32<TC>(silu_mul<TC>(gt, up));
      }
    } else {
      for (int idx = threadIdx.x; idx < ROWS * 8 * MT; idx += blockDim.x) {
        const int col = idx / ROWS, rr = idx % ROWS;
        const int n = ct.n0 + rr;
        if (col >= ct.rows || n >= N) continue;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < ST_WARPS; w++) v += red[w][rr / ST_ROWS][rr % ST_ROWS][col];
        TC* cp = C + (size_t)(ct.row0 + col) * ldc + n;
        if (epilogue == 1) v += to_f32(*cp);
        *cp = from_f32<TC>(v);
      }
    }
    __syncthreads();
  }
  st_wait<0>();
}

template <typename TC, int MT, int NSUB, int S, int ST_WARPS>
static int launch_stream_grouped(void* C, const bf16* A, const bf16* W, int P, int N, int K, int lda, int ldc,
                                 int epilogue, const int* group_offsets, int n_groups, size_t w_group_stride,
                                 cudaStream_t st) {
  constexpr int ROWS = ST_ROWS * NSUB;
  constexpr size_t smem = (size_t)ST_WARPS * S * (ROWS + 8 * MT) * 128 + sizeof(float) * ST_WARPS * NSUB * ST_ROWS * (8 * MT + 1);
  static int slots = 0;
  if (!slots) {
    int dev = 0, n_sm = 0, per_sm = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
    if (cudaFuncSetAttribute(gemm_bf16_stream_grouped_kernel<TC, MT, NSUB, S, ST_WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return leb_fail("leb_gemm_bf16_stream_grouped: %zu bytes of shared memory per block refused", smem);
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemm_bf16_stream_grouped_kernel<TC, MT, NSUB, S, ST_WARPS>, 32 * ST_WARPS, smem);
    slots = max(1, per_sm) * max(1, n_sm);
  }
  // the most tiles the offsets can give: every expert may end with a partly filled block of rows
  const long most = ((long)ceil_div(P, 8 * MT) + n_groups) * ceil_div(N, ROWS);
  const int grid = (int)(most < slots ? most : slots);
  leb_launch(gemm_bf16_stream_grouped_kernel<TC, MT, NSUB, S, ST_WARPS>, dim3(grid), dim3(32 * ST_WARPS), smem, st,
             (TC*)C, A, W, N, K, lda, ldc, epilogue, group_offsets, n_groups, w_group_stride);
  LEB_CHECK_LAUNCH("leb_gemm_bf16_stream_grouped");
  return 0;
}

template <typename TC, int MT, int NSUB, int S, int ST_WARPS>
static int launch_stream(void* C, const bf16* A, const bf16* W, int M, int N, int K, int lda, int ldc,
                         int epilogue, cudaStream_t st, StreamNorm nm, StreamConv cv = StreamConv{}) {
  constexpr int ROWS = ST_ROWS * NSUB;
  constexpr size_t smem = (size_t)ST_WARPS * S * (ROWS + 8 * MT) * 128 + sizeof(float) * ST_WARPS * NSUB * ST_ROWS * (8 * MT + 1);
  static int slots = 0;   // blocks the GPU holds at once
  if (!slots) {
    int dev = 0, n_sm = 0, per_sm = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
    if (cudaFuncSetAttribute(gemm_bf16_stream_kernel<TC, MT, NSUB, S, ST_WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return leb_fail("leb_gemm_bf16_stream: %zu bytes of shared memory per block refused", smem);
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemm_bf16_stream_kernel<TC, MT, NSUB, S, ST_WARPS>, 32 * ST_WARPS, smem);
    slots = max(1, per_sm) * max(1, n_sm);
  }
  const int n_tiles = NSUB == 3 ? ceil_div(N / 3, ST_ROWS) : ceil_div(N, ROWS);
  // the same number of tiles for every block (as far as it goes), all blocks on the GPU at once
  const int per_block = ceil_div(n_tiles, slots);
  const int grid = ceil_div(n_tiles, per_block);
  leb_launch(gemm_bf16_stream_kernel<TC, MT, NSUB, S, ST_WARPS>, dim3(grid), dim3(32 * ST_WARPS), smem, st, (TC*)C, A, W, M, N,
             K, lda, ldc, epilogue, n_tiles, cv, nm);
  LEB_CHECK_LAUNCH("leb_gemm_bf16_stream");
  return 0;
}

template <typename TC>
static int stream_dispatch(void* C, const bf16* a, const bf16* w, int M, int N, int K, int lda, int ldc, int epilogue,
                           cudaStream_t st, StreamNorm nm) {
  if (epilogue == 2) {
    if (M <= 8) return launch_stream<TC, 1, 2, 4, 4>(C, a, w, M, N, K, lda, ldc, epilogue, st, nm);
    return launch_stream<TC, 2, 2, 4, 4>(C, a, w, M, N, K, lda, ldc, epilogue, st, nm);
  }
  // few tiles (at most one per SM) and a long K: deeper rings instead of a second block per SM
  if (M <= 8 && ceil_div(N, ST_ROWS) <= sm_count() && K >= 4096) return launch_stream<TC, 1, 1, 8, 8>(C, a, w, M, N, K, lda, ldc, epilogue, st, nm);
  if (M <= 8) return launch_stream<TC, 1, 1, 4, 8>(C, a, w, M, N, K, lda, ldc, epilogue, st, nm);
  return launch_stream<TC, 2, 1, 3, 8>(C, a, w, M, N, K, lda, ldc, epilogue, st, nm);
}

// Split norm (see StreamNorm), both optional: `ssq_in` [M, parts_in] with `d_in` and `eps` scales the
// product's rows by rsqrt(sum / d_in + eps); `emit_vals` [M, N], `emit_g` [N], `emit_ssq`
// [M, ceil(N/16)] make an adding product leave what the next norm needs.
LEB_API int leb_gemm_bf16_stream(void* C, int c_dtype, const void* A, const void* W, int M, int N, int K, int lda,
                                 int ldc, int epilogue, const float* ssq_in, int parts_in, int d_in, float eps,
                                 void* emit_vals, const float* emit_g, float* emit_ssq, cudaStream_t st) {
  if (M <= 0 || N <= 0) return 0;
  LEB_REQUIRE(M <= 16, "leb_gemm_bf16_stream: %d rows; this kernel takes at most 16", M);
  LEB_REQUIRE(K > 0 && K % 8 == 0, "leb_gemm_bf16_stream: K (%d) must be a multiple of 8", K);
  LEB_REQUIRE(lda % 8 == 0, "leb_gemm_bf16_stream: row stride of A (%d) must be a multiple of 8", lda);
  LEB_REQUIRE(((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0, "leb_gemm_bf16_stream: A and W must be 16-byte aligned");
  LEB_REQUIRE(epilogue >= 0 && epilogue <= 2, "leb_gemm_bf16_stream: unknown epilogue %d", epilogue);
  LEB_REQUIRE(epilogue != 1 || c_dtype == LEB_F32, "leb_gemm_bf16_stream: adding needs a float C");
  LEB_REQUIRE(epilogue != 2 || N % 32 == 0, "leb_gemm_bf16_stream: the SwiGLU epilogue needs N (%d) to be a multiple of 32", N);
  LEB_REQUIRE(!emit_vals || (epilogue == 1 && emit_g && emit_ssq), "leb_gemm_bf16_stream: only an adding product leaves the next norm's input, and it needs the weight and the sums' place");
  LEB_REQUIRE(!ssq_in || (parts_in > 0 && d_in > 0), "leb_gemm_bf16_stream: the sums of squares need their count and the row width");
  StreamNorm nm{ssq_in, parts_in, d_in, eps, (bf16*)emit_vals, emit_g, emit_ssq};
  if (c_dtype == LEB_BF16) return stream_dispatch<bf16>(C, (const bf16*)A, (const bf16*)W, M, N, K, lda, ldc, epilogue, st, nm);
  if (c_dtype == LEB_F32) return stream_dispatch<float>(C, (const bf16*)A, (const bf16*)W, M, N, K, lda, ldc, epilogue, st, nm);
  return leb_fail("leb_gemm_bf16_stream: unknown C dtype %d", c_dtype);
}

// The conv mixer's decode step in one launch: y[M, D] = conv(in_proj . h) with the state updated
// (every row is the one new token of its sequence).  W: in_proj [3D, K]; conv_w [D, Lc]; state
// [slots, D, Lc-1] float; row_seq / seq_slot as in leb_shortconv.
LEB_API int leb_gemm_bf16_stream_conv(void* y, const void* A, const void* W, int M, int D, int K, int lda, int ldy,
                                      const float* conv_w, const float* bias, float* state, const int* row_seq,
                                      const int* seq_slot, int Lc, const float* ssq_in, int parts_in, int d_in,
                                      float eps, cudaStream_t st) {
  if (M <= 0 || D <= 0) return 0;
  LEB_REQUIRE(M <= 16, "leb_gemm_bf16_stream_conv: %d rows; this kernel takes at most 16", M);
  LEB_REQUIRE(K > 0 && K % 8 == 0 && lda % 8 == 0, "leb_gemm_bf16_stream_conv: K (%d) and the row stride of A (%d) must be multiples of 8", K, lda);
  LEB_REQUIRE(((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0, "leb_gemm_bf16_stream_conv: A and W must be 16-byte aligned");
  LEB_REQUIRE(Lc >= 2 && Lc <= ST_CONV_MAX_LC, "leb_gemm_bf16_stream_conv: conv length %d outside 2..%d", Lc, ST_CONV_MAX_LC);
  LEB_REQUIRE(conv_w && state && row_seq && seq_slot, "leb_gemm_bf16_stream_conv: taps, state and the step's tables are required");
  LEB_REQUIRE(!ssq_in || (parts_in > 0 && d_in > 0), "leb_gemm_bf16_stream_conv: the sums of squares need their count and the row width");
  StreamConv cv{conv_w, bias, state, row_seq, seq_slot, Lc};
  StreamNorm nm{ssq_in, parts_in, d_in, eps, nullptr, nullptr, nullptr};
  if (M <= 8) return launch_stream<bf16, 1, 3, 4, 4>(y, (const bf16*)A, (const bf16*)W, M, 3 * D, K, lda, ldy, 3, st, nm, cv);
  return launch_stream<bf16, 2, 3, 4, 4>(y, (const bf16*)A, (const bf16*)W, M, 3 * D, K, lda, ldy, 3, st, nm, cv);
}

template <typename TC>
static int stream_grouped_dispatch(void* C, const bf16* a, const bf16* w, int P, int N, int K, int lda, int ldc,
                                   int epilogue, const int* off, int n_groups, size_t stride, cudaStream_t st) {
  const bool few = P <= 8 * n_groups;   // on average at most 8 rows per expert: blocks of 8 rows, else of 16
  if (epilogue == 2) {
    if (few) return launch_stream_grouped<TC, 1, 2, 4, 4>(C, a, w, P, N, K, lda, ldc, epilogue, off, n_groups, stride, st);
    return launch_stream_grouped<TC, 2, 2, 4, 4>(C, a, w, P, N, K, lda, ldc, epilogue, off, n_groups, stride, st);
  }
  if (few) return launch_stream_grouped<TC, 1, 1, 4, 8>(C, a, w, P, N, K, lda, ldc, epilogue, off, n_groups, stride, st);
  return launch_stream_grouped<TC, 2, 1, 3, 8>(C, a, w, P, N, K, lda, ldc, epilogue, off, n_groups, stride, st);
}

// Grouped form: rows [group_offsets[e], group_offsets[e+1]) of A [P, K] and C go with the weights
// W + e * w_group_stride ([N, K] each).  group_offsets [n_groups + 1] lives on the device.
LEB_API int leb_gemm_bf16_stream_grouped(void* C, int c_dtype, const void* A, const void* W, int P, int N, int K,
                                         int lda, int ldc, int epilogue, const int* group_offsets, int n_groups,
                                         size_t w_group_stride, cudaStream_t st) {
  if (P <= 0 || N <= 0 || n_groups <= 0) return 0;
  LEB_REQUIRE(n_groups <= ST_MAX_GROUPS, "leb_gemm_bf16_stream_grouped: %d groups; at most %d", n_groups, ST_MAX_GROUPS);
  LEB_REQUIRE(K > 0 && K % 8 == 0 && lda % 8 == 0, "leb_gemm_bf16_stream_grouped: K (%d) and the row stride of A (%d) must be multiples of 8", K, lda);
  LEB_REQUIRE(((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0 && (w_group_stride * 2) % 16 == 0,
              "leb_gemm_bf16_stream_grouped: A, W and the distance between experts must be 16-byte aligned");
  LEB_REQUIRE(epilogue >= 0 && epilogue <= 2, "leb_gemm_bf16_stream_grouped: unknown epilogue %d", epilogue);
  LEB_REQUIRE(epilogue != 1 || c_dtype == LEB_F32, "leb_gemm_bf16_stream_grouped: adding needs a float C");
  LEB_REQUIRE(epilogue != 2 || N % 32 == 0, "leb_gemm_bf16_stream_grouped: the SwiGLU epilogue needs N (%d) to be a multiple of 32", N);
  if (c_dtype == LEB_BF16)
    return stream_grouped_dispatch<bf16>(C, (const bf16*)A, (const bf16*)W, P, N, K, lda, ldc, epilogue, group_offsets, n_groups, w_group_stride, st);
  if (c_dtype == LEB_F32)
    return stream_grouped_dispatch<float>(C, (const bf16*)A, (const bf16*)W, P, N, K, lda, ldc, epilogue, group_offsets, n_groups, w_group_stride, st);
  return leb_fail("leb_gemm_bf16_stream_grouped: unknown C dtype %d", c_dtype);
}
