// Gated short convolution over packed rows of several sequences, with the state carried in
// the cache between steps.
//
// For a token with projections (B, C, xg) = in_proj(h) split in this order
// (src/dense.rs:156-161, src/cuda/dense.cu:126,131):
//     bx_t = B_t * xg_t
//     c_t  = sum_{j=0}^{Lc-1} w[ch, j] * bx_{t-(Lc-1)+j}      (w[ch, Lc-1] takes the current token,
//                                                              src/dense.rs:163-164)
//     y_t  = C_t * c_t  (+ bias[ch] inside c_t when the layer has one)
// Values of bx before the first row of this step come from the state: the last Lc-1 values of
// bx per channel, oldest first (src/dense.rs:165-166); a fresh sequence starts from zeros.
// The reference runs the tokens of a chunk one after another per channel
// (src/cuda/dense.cu:135-148); here every (row, channel) is independent because a tap reaches
// back only Lc-1 rows, so the rows of a prompt are computed in parallel and a second kernel
// writes the new state once all rows have read the old one.
#include "common.cuh"

template <typename T>
__global__ void shortconv_rows_kernel(T* __restrict__ y, const T* __restrict__ bcx,
                                      const float* __restrict__ w, const float* __restrict__ bias,
                                      const float* __restrict__ state,
                                      const int* __restrict__ row_seq,
                                      const int* __restrict__ seq_slot,
                                      const int* __restrict__ seq_qstart, int D, int Lc) {
  pdl_trigger();   // the kernel after this one may start and wait (see common.cuh)
  pdl_wait();
  int m = blockIdx.x;
  int ch = blockIdx.y * blockDim.x + threadIdx.x;
  if (ch >= D) return;
  int b = row_seq[m];
  int slot = seq_slot[b];
  T* yo = y + (size_t)m * D;
  if (slot < 0) {  // padding row
    yo[ch] = from_f32<T>(0.f);
    return;
  }
  int i = m - seq_qstart[b];  // index of this row within its sequence's rows of this step
  const float* wc = w + (size_t)ch * Lc;
  const float* sc = state + ((size_t)slot * D + ch) * (Lc - 1);
  float acc = bias ? bias[ch] : 0.f;
  for (int j = 0; j < Lc; j++) {
    int src = i - (Lc - 1) + j;  // row of this step, negative: before it
    float bx;
    if (src >= 0) {
      const T* r = bcx + (size_t)(m - i + src) * 3 * D;
      bx = to_f32(r[ch]) * to_f32(r[2 * D + ch]);
    } else {
      bx = sc[(Lc - 1) + src];
    }
    acc += wc[j] * bx;
  }
  const T* r = bcx + (size_t)m * 3 * D;
  yo[ch] = from_f32<T>(to_f32(r[D + ch]) * acc);
}

// The same for bfloat16 rows with 16-byte loads: a thread owns 8 channels of one row.
__global__ void shortconv_rows_bf16x8_kernel(bf16* __restrict__ y, const bf16* __restrict__ bcx,
                                             const float* __restrict__ w, const float* __restrict__ bias,
                                             const float* __restrict__ state, const int* __restrict__ row_seq,
                                             const int* __restrict__ seq_slot, const int* __restrict__ seq_qstart,
                                             int D, int Lc) {
  pdl_trigger();   // the kernel after this one may start and wait (see common.cuh)
  pdl_wait();
  const int m = blockIdx.x;
  const int ch0 = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (ch0 >= D) return;
  const int b = row_seq[m];
  const int slot = seq_slot[b];
  uint4* yo = reinterpret_cast<uint4*>(y + (size_t)m * D + ch0);
  if (slot < 0) {
    *yo = make_uint4(0, 0, 0, 0);
    return;
  }
  const int i = m - seq_qstart[b];
  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; e++) acc[e] = bias ? bias[ch0 + e] : 0.f;
  for (int j = 0; j < Lc; j++) {
    const int src = i - (Lc - 1) + j;
    float bx[8];
    if (src >= 0) {
      const bf16* r = bcx + (size_t)(m - i + src) * 3 * D;
      const uint4 Bv = *reinterpret_cast<const uint4*>(r + ch0);
      const uint4 Xv = *reinterpret_cast<const uint4*>(r + 2 * D + ch0);
      const __nv_bfloat162* Bp = reinterpret_cast<const __nv_bfloat162*>(&Bv);
      const __nv_bfloat162* Xp = reinterpret_cast<const __nv_bfloat162*>(&Xv);
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const float2 bf = __bfloat1622float2(Bp[e]), xf = __bfloat1622float2(Xp[e]);
        bx[2 * e] = bf.x * xf.x;
        bx[2 * e + 1] = bf.y * xf.y;
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; e++) bx[e] = state[((size_t)slot * D + ch0 + e) * (Lc - 1) + (Lc - 1) + src];
    }
#pragma unroll
    for (int e = 0; e < 8; e++) acc[e] += w[(size_t)(ch0 + e) * Lc + j] * bx[e];
  }
  const uint4 Cv = *reinterpret_cast<const uint4*>(bcx + (size_t)m * 3 * D + D + ch0);
  const __nv_bfloat162* Cp = reinterpret_cast<const __nv_bfloat162*>(&Cv);
  uint4 o;
  uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
  for (int e = 0; e < 4; e++) {
    const float2 cf = __bfloat1622float2(Cp[e]);
    __nv_bfloat162 v = __floats2bfloat162_rn(cf.x * acc[2 * e], cf.y * acc[2 * e + 1]);
    op[e] = *reinterpret_cast<uint32_t*>(&v);
  }
  *yo = o;
}

// The same again for the usual short lengths: a thread owns 8 channels over CONV_CHUNK consecutive
// rows and keeps the last LC-1 products B*x in registers, so each row's B, C and x are loaded
// once instead of LC times.  Taps, bias and order of the sum are those of the kernels above, so
// the results are the same bit for bit.
constexpr int CONV_CHUNK = 8;

__device__ __forceinline__ void conv_mul8(float* o, const uint4& a, const uint4& b) {
  const __nv_bfloat162* ap = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
  for (int e = 0; e < 4; e++) {
    const float2 af = __bfloat1622float2(ap[e]), bf = __bfloat1622float2(bp[e]);
    o[2 * e] = af.x * bf.x;
    o[2 * e + 1] = af.y * bf.y;
  }
}

template <int LC>
__global__ void __launch_bounds__(128) shortconv_rows_bf16x8_chunk_kernel(
    bf16* __restrict__ y, const bf16* __restrict__ bcx, const float* __restrict__ w,
    const float* __restrict__ bias, const float* __restrict__ state, const int* __restrict__ row_seq,
    const int* __restrict__ seq_slot, const int* __restrict__ seq_qstart, int M, int D) {
  pdl_trigger();   // the kernel after this one may start and wait (see common.cuh)
  pdl_wait();
  const int m0 = blockIdx.x * CONV_CHUNK;
  const int ch0 = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (ch0 >= D) return;
  float wt[LC][8], bs[8], hist[LC - 1][8];
#pragma unroll
  for (int e = 0; e < 8; e++) {
    bs[e] = bias ? bias[ch0 + e] : 0.f;
#pragma unroll
    for (int j = 0; j < LC; j++) wt[j][e] = w[(size_t)(ch0 + e) * LC + j];
  }
#pragma unroll
  for (int k = 0; k < LC - 1; k++) {  // products of the rows just before the chunk
    const int row = m0 - (LC - 1) + k;
    if (row >= 0) {
      const bf16* r = bcx + (size_t)row * 3 * D;
      conv_mul8(hist[k], *reinterpret_cast<const uint4*>(r + ch0), *reinterpret_cast<const uint4*>(r + 2 * D + ch0));
    } else {
#pragma unroll
      for (int e = 0; e < 8; e++) hist[k][e] = 0.f;
    }
  }
#pragma unroll
  for (int rr = 0; rr < CONV_CHUNK; rr++) {
    const int m = m0 + rr;
    if (m >= M) break;
    const bf16* r = bcx + (size_t)m * 3 * D;
    const uint4 Bv = *reinterpret_cast<const uint4*>(r + ch0);
    const uint4 Cv = *reinterpret_cast<const uint4*>(r + D + ch0);
    const uint4 Xv = *reinterpret_cast<const uint4*>(r + 2 * D + ch0);
    const int b = row_seq[m];
    const int slot = seq_slot[b];
    const int i = m - seq_qstart[b];
    float cur[8], acc[8];
    conv_mul8(cur, Bv, Xv);
#pragma unroll
    for (int e = 0; e < 8; e++) acc[e] = bs[e];
#pragma unroll
    for (int j = 0; j < LC - 1; j++) {
      const int src = i - (LC - 1) + j;  // row of this sequence in this step; negative: before it
      if (src >= 0) {
#pragma unroll
        for (int e = 0; e < 8; e++) acc[e] += wt[j][e] * hist[j][e];
      } else if (slot >= 0) {
#pragma unroll
        for (int e = 0; e < 8; e++)
          acc[e] += wt[j][e] * state[((size_t)slot * D + ch0 + e) * (LC - 1) + (LC - 1) + src];
      }
    }
    const __nv_bfloat162* Cp = reinterpret_cast<const __nv_bfloat162*>(&Cv);
    uint4 o;
    uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int e = 0; e < 4; e++) {
      const float2 cf = __bfloat1622float2(Cp[e]);
      __nv_bfloat162 v = __floats2bfloat162_rn(cf.x * (acc[2 * e] + wt[LC - 1][2 * e] * cur[2 * e]),
                                               cf.y * (acc[2 * e + 1] + wt[LC - 1][2 * e + 1] * cur[2 * e + 1]));
      op[e] = *reinterpret_cast<uint32_t*>(&v);
    }
    if (slot < 0) o = make_uint4(0, 0, 0, 0);  // padding row
    *reinterpret_cast<uint4*>(y + (size_t)m * D + ch0) = o;
#pragma unroll
    for (int k = 0; k + 1 < LC - 1; k++)
#pragma unroll
      for (int e = 0; e < 8; e++) hist[k][e] = hist[k + 1][e];
#pragma unroll
    for (int e = 0; e < 8; e++) hist[LC - 2][e] = cur[e];
  }
}

// New state of each sequence: the last Lc-1 values of (old state ++ bx of this step's rows).
template <typename T>
__global__ void shortconv_state_kernel(const T* __restrict__ bcx, float* __restrict__ state,
                                       const int* __restrict__ seq_slot,
                                       const int* __restrict__ seq_qstart,
                                       const int* __restrict__ seq_qlen, int D, int Lc) {
  pdl_trigger();   // the kernel after this one may start and wait (see common.cuh)
  pdl_wait();
  int b = blockIdx.x;
  int ch = blockIdx.y * blockDim.x + threadIdx.x;
  if (ch >= D) return;
  int slot = seq_slot[b];
  if (slot < 0) return;
  int T_ = seq_qlen[b];
  if (T_ <= 0) return;
  int q0 = seq_qstart[b];
  float* sc = state + ((size_t)slot * D + ch) * (Lc - 1);
  float nv[16];
  for (int k = 0; k < Lc - 1; k++) {
    int src = T_ - (Lc - 1) + k;
    if (src >= 0) {
      const T* r = bcx + (size_t)(q0 + src) * 3 * D;
      nv[k] = to_f32(r[ch]) * to_f32(r[2 * D + ch]);
    } else {
      nv[k] = sc[(Lc - 1) + src];
    }
  }
  for (int k = 0; k < Lc - 1; k++) sc[k] = nv[k];
}

// Decode: every sequence brings exactly one row, so one thread per (sequence, channel) reads the
// state, gives the output and shifts the state, as the reference's one-token kernel does
// (src/cuda/dense.cu:124-132); one launch instead of two.
template <typename T>
__global__ void shortconv_single_kernel(T* __restrict__ y, const T* __restrict__ bcx,
                                        const float* __restrict__ w, const float* __restrict__ bias,
                                        float* __restrict__ state, const int* __restrict__ seq_slot,
                                        const int* __restrict__ seq_qstart, int D, int Lc) {
  pdl_trigger();   // the kernel after this one may start and wait (see common.cuh)
  pdl_wait();
  const int b = blockIdx.x;
  const int ch = blockIdx.y * blockDim.x + threadIdx.x;
  if (ch >= D) return;
  const int slot = seq_slot[b];
  const size_t m = seq_qstart[b];
  if (slot < 0) {
    y[m * D + ch] = from_f32<T>(0.f);
    return;
  }
  const T* r = bcx + m * 3 * D;
  const float bx = to_f32(r[ch]) * to_f32(r[2 * D + ch]);
  const float* wc = w + (size_t)ch * Lc;
  float* sc = state + ((size_t)slot * D + ch) * (Lc - 1);
  float acc = bias ? bias[ch] : 0.f;
  float s[16];
  for (int k = 0; k < Lc - 1; k++) {
    s[k] = sc[k];
    acc += wc[k] * s[k];       // same order of taps as the row kernel: oldest first
  }
  acc += wc[Lc - 1] * bx;
  for (int k = 0; k < Lc - 2; k++) sc[k] = s[k + 1];
  sc[Lc - 2] = bx;
  y[m * D + ch] = from_f32<T>(to_f32(r[D + ch]) * acc);
}

LEB_API int leb_shortconv(void* y, const void* bcx, int dtype, const float* w, const float* bias,
                          float* state, const int* row_seq, const int* seq_slot,
                          const int* seq_qstart, const int* seq_qlen, int M, int B, int D, int Lc,
                          cudaStream_t st) {
  if (M <= 0 || B <= 0) return 0;
  LEB_REQUIRE(Lc >= 2 && Lc <= 17, "leb_shortconv: conv length %d outside 2..17", Lc);
  dim3 block(128);
  if (seq_qlen == nullptr) {   // the caller vouches that every sequence has one row
    dim3 g(B, ceil_div(D, 128));
    if (dtype == LEB_F32)
      leb_launch(shortconv_single_kernel<float>, g, block, 0, st, (float*)y, (const float*)bcx, w, bias, state, seq_slot, seq_qstart, D, Lc);
    else if (dtype == LEB_BF16)
      leb_launch(shortconv_single_kernel<bf16>, g, block, 0, st, (bf16*)y, (const bf16*)bcx, w, bias, state, seq_slot, seq_qstart, D, Lc);
    else
      return leb_fail("leb_shortconv: unknown dtype %d", dtype);
    LEB_CHECK_LAUNCH("leb_shortconv");
    return 0;
  }
  dim3 g1(M, ceil_div(D, 128)), g2(B, ceil_div(D, 128));
  if (dtype == LEB_F32) {
    leb_launch(shortconv_rows_kernel<float>, g1, block, 0, st, (float*)y, (const float*)bcx, w, bias, (const float*)state,
               row_seq, seq_slot, seq_qstart, D, Lc);
    leb_launch(shortconv_state_kernel<float>, g2, block, 0, st, (const float*)bcx, state, seq_slot, seq_qstart, seq_qlen, D, Lc);
  } else if (dtype == LEB_BF16) {
    const bool vec = D % 8 == 0 && ((uintptr_t)y % 16) == 0 && ((uintptr_t)bcx % 16) == 0;
    const dim3 gc(ceil_div(M, CONV_CHUNK), ceil_div(D / 8, 128));
    if (vec && Lc == 3 && M >= 256)
      leb_launch(shortconv_rows_bf16x8_chunk_kernel<3>, gc, block, 0, st,
          (bf16*)y, (const bf16*)bcx, w, bias, (const float*)state, row_seq, seq_slot, seq_qstart, M, D);
    else if (vec && Lc == 4 && M >= 256)
      leb_launch(shortconv_rows_bf16x8_chunk_kernel<4>, gc, block, 0, st,
          (bf16*)y, (const bf16*)bcx, w, bias, (const float*)state, row_seq, seq_slot, seq_qstart, M, D);
    else if (vec)
      leb_launch(shortconv_rows_bf16x8_kernel, dim3(M, ceil_div(D / 8, 128)), block, 0, st,
          (bf16*)y, (const bf16*)bcx, w, bias, (const float*)state, row_seq, seq_slot, seq_qstart, D, Lc);
    else
      leb_launch(shortconv_rows_kernel<bf16>, g1, block, 0, st, (bf16*)y, (const bf16*)bcx, w, bias, (const float*)state,
                 row_seq, seq_slot, seq_qstart, D, Lc);
    leb_launch(shortconv_state_kernel<bf16>, g2, block, 0, st, (const bf16*)bcx, state, seq_slot, seq_qstart, seq_qlen, D, Lc);
  } else {
    return leb_fail("leb_shortconv: unknown dtype %d", dtype);
  }
  LEB_CHECK_LAUNCH("leb_shortconv");
  g_leb_launches++;  // two kernels
  return 0;
}
