// Memory-bound row kernels: embedding gather, RMSNorm (plain, gathered, and added to the
// residual), SwiGLU, residual add, row gather.  The residual stream is always float; the
// template parameter is the type of the activations that feed the matrix products.
#include <stdarg.h>

#include "common.cuh"

static thread_local char g_err[512];

int leb_fail(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return 1;
}
LEB_API const char* leb_last_error() { return g_err; }

long long g_leb_launches = 0;
int g_leb_pdl = 1;
LEB_API void leb_set_pdl(int on) { g_leb_pdl = on ? 1 : 0; }
LEB_API long long leb_launch_count() { return g_leb_launches; }

// ---------------------------------------------------------------------------------------------
// x[m, :] = table[tokens[m], :]            (reference: src/dense.rs:172-177 takes the row as is)
template <typename T>
__global__ void embed_kernel(float* __restrict__ x, const T* __restrict__ table,
                             const int* __restrict__ tokens, int D, int V) {
  pdl_trigger();   // the kernel after this one may start and wait (see common.cuh)
  pdl_wait();
  int m = blockIdx.x;
  int tok = tokens[m];
  tok = tok < 0 ? 0 : (tok >= V ? V - 1 : tok);  // ids are validated on the host; never read outside
  const T* row = table + (size_t)tok * D;
  float* o = x + (size_t)m * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x) o[i] = to_f32(row[i]);
}

LEB_API int leb_embed(float* x, const void* table, int table_dtype, const int* tokens, int M, int D,
                      int V, cudaStream_t st) {
  if (M <= 0) return 0;
  int threads = D >= 1024 ? 256 : 128;
  if (table_dtype == LEB_F32)
    leb_launch(embed_kernel<float>, dim3(M), dim3(threads), 0, st, x, (const float*)table, tokens, D, V);
  else if (table_dtype == LEB_BF16)
    leb_launch(embed_kernel<bf16>, dim3(M), dim3(threads), 0, st, x, (const bf16*)table, tokens, D, V);
  else
    return leb_fail("leb_embed: unknown table dtype %d", table_dtype);
  LEB_CHECK_LAUNCH("leb_embed");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// RMSNorm:  r = rsqrt(mean(x^2) + eps);  y = x * r * w      (src/dense.rs:27-30: eps inside the
// root, added to the mean; the weight multiplies directly).  Sum, root and product are float.
//   rows != null : input row m is x[rows[m]]  (the rows whose logits are wanted)
//   ADD          : out (float) += y           (a norm after the mixer or feed-forward, src/dense.rs:185,192)
template <typename TO, bool ADD>
__global__ void rmsnorm_kernel(TO* __restrict__ out, const float* __restrict__ x,
                               const float* __restrict__ w, const int* __restrict__ rows, int D,
                               float eps) {
  __shared__ float red[33];
  pdl_trigger();   // the kernel after this one may start and wait (see common.cuh)
  pdl_wait();
  int m = blockIdx.x;
  const float* xi = x + (size_t)(rows ? rows[m] : m) * D;
  float s = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float v = xi[i];
    s += v * v;
  }
  s = block_sum(s, red);
  float r = 1.0f / sqrtf(s / (float)D + eps);
  TO* o = out + (size_t)m * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float y = xi[i] * r * w[i];
    if (ADD)
      o[i] = from_f32<TO>(to_f32(o[i]) + y);
    else
      o[i] = from_f32<TO>(y);
  }
}

// The same norm for bfloat16 output with 16-byte loads: a thread keeps its CH float4 pieces of
// the row in registers between the sum and the product, so the row is read once.
template <int CH>
__global__ void __launch_bounds__(256)
rmsnorm_bf16_vec_kernel(bf16* __restrict__ out, const float* __restrict__ x, const float* __restrict__ w,
                        const int* __restrict__ rows, int D, float eps) {
  __shared__ float red[33];
  pdl_trigger();   // the kernel after this one may start and wait (see common.cuh)
  pdl_wait();
  const int m = blockIdx.x;
  const float4* xi = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[m] : m) * D);
  const float4* w4 = reinterpret_cast<const float4*>(w);
  const int n4 = D >> 2;
  float4 v[CH];
  float s = 0.f;
#pragma unroll
  for (int c = 0; c < CH; c++) {
    const int i = threadIdx.x + c * 256;
    if (i < n4) {
      v[c] = xi[i];
      s += v[c].x * v[c].x + v[c].y * v[c].y + v[c].z * v[c].z + v[c].w * v[c].w;
    }
  }
  s = block_sum(s, red);
  const float r = 1.0f / sqrtf(s / (float)D + eps);
  uint2* o = reinterpret_cast<uint2*>(out + (size_t)m * D);
#pragma unroll
  for (int c = 0; c < CH; c++) {
    const int i = threadIdx.x + c * 256;
    if (i < n4) {
      const float4 ww = w4[i];
      __nv_bfloat162 lo = __floats2bfloat162_rn(v[c].x * r * ww.x, v[c].y * r * ww.y);
      __nv_bfloat162 hi = __floats2bfloat162_rn(v[c].z * r * ww.z, v[c].w * r * ww.w);
      o[i] = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    }
  }
}

LEB_API int leb_rmsnorm(void* out, int out_dtype, const float* x, const float* w, const int* rows,
                        int M, int D, float eps, int add, cudaStream_t st) {
  if (M <= 0) return 0;
  if (!add && out_dtype == LEB_BF16 && D % 4 == 0 && D <= 8192 && ((uintptr_t)x % 16) == 0 &&
      ((uintptr_t)w % 16) == 0 && ((uintptr_t)out % 8) == 0) {
    const int ch = ceil_div(D / 4, 256);
    bf16* o = (bf16*)out;
    if (ch <= 1) leb_launch(rmsnorm_bf16_vec_kernel<1>, dim3(M), dim3(256), 0, st, o, x, w, rows, D, eps);
    else if (ch <= 2) leb_launch(rmsnorm_bf16_vec_kernel<2>, dim3(M), dim3(256), 0, st, o, x, w, rows, D, eps);
    else if (ch <= 4) leb_launch(rmsnorm_bf16_vec_kernel<4>, dim3(M), dim3(256), 0, st, o, x, w, rows, D, eps);
    else leb_launch(rmsnorm_bf16_vec_kernel<8>, dim3(M), dim3(256), 0, st, o, x, w, rows, D, eps);
    LEB_CHECK_LAUNCH("leb_rmsnorm");
    return 0;
  }
  int threads = D >= 2048 ? 512 : (D >= 512 ? 256 : 128);
  if (add) {
    LEB_REQUIRE(out_dtype == LEB_F32, "leb_rmsnorm: the added form writes the float residual");
    leb_launch(rmsnorm_kernel<float, true>, dim3(M), dim3(threads), 0, st, (float*)out, x, w, rows, D, eps);
  } else if (out_dtype == LEB_F32) {
    leb_launch(rmsnorm_kernel<float, false>, dim3(M), dim3(threads), 0, st, (float*)out, x, w, rows, D, eps);
  } else if (out_dtype == LEB_BF16) {
    leb_launch(rmsnorm_kernel<bf16, false>, dim3(M), dim3(threads), 0, st, (bf16*)out, x, w, rows, D, eps);
  } else {
    return leb_fail("leb_rmsnorm: unknown output dtype %d", out_dtype);
  }
  LEB_CHECK_LAUNCH("leb_rmsnorm");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// a[m, j] = silu(gu[m, j]) * gu[m, F + j],  silu(x) = x / (1 + exp(-x))   (src/dense.rs:31,190)
template <typename TI, typename TO>
__global__ void swiglu_kernel(TO* __restrict__ a, const TI* __restrict__ gu, int F, size_t total) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  size_t m = i / F;
  int j = (int)(i - m * F);
  float g = to_f32(gu[m * 2 * F + j]);
  float u = to_f32(gu[m * 2 * F + F + j]);
  a[i] = from_f32<TO>(silu_mul<TO>(g, u));
}

LEB_API int leb_swiglu(void* a, int out_dtype, const void* gu, int in_dtype, int M, int F,
                       cudaStream_t st) {
  size_t total = (size_t)M * F;
  if (total == 0) return 0;
  unsigned blocks = (unsigned)((total + 255) / 256);
  if (in_dtype == LEB_F32 && out_dtype == LEB_F32)
    swiglu_kernel<float, float><<<blocks, 256, 0, st>>>((float*)a, (const float*)gu, F, total);
  else if (in_dtype == LEB_F32 && out_dtype == LEB_BF16)
    swiglu_kernel<float, bf16><<<blocks, 256, 0, st>>>((bf16*)a, (const float*)gu, F, total);
  else if (in_dtype == LEB_BF16 && out_dtype == LEB_BF16)
    swiglu_kernel<bf16, bf16><<<blocks, 256, 0, st>>>((bf16*)a, (const bf16*)gu, F, total);
  else
    return leb_fail("leb_swiglu: unsupported dtypes in=%d out=%d", in_dtype, out_dtype);
  LEB_CHECK_LAUNCH("leb_swiglu");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// out[p, :] = in[rows[p] / div, :]   (expert-sorted copies of token rows; div = experts per token)
template <typename T>
__global__ void gather_rows_kernel(T* __restrict__ out, const T* __restrict__ in,
                                   const int* __restrict__ rows, int div, int D) {
  pdl_trigger();   // the kernel after this one may start and wait (see common.cuh)
  pdl_wait();
  int p = blockIdx.x;
  int src = rows[p] / div;
  const T* a = in + (size_t)src * D;
  T* o = out + (size_t)p * D;
  if ((((uintptr_t)a | (uintptr_t)o) & 15) == 0 && (D * sizeof(T)) % 16 == 0) {
    const int n = D * (int)sizeof(T) / 16;
    for (int i = threadIdx.x; i < n; i += blockDim.x) reinterpret_cast<uint4*>(o)[i] = reinterpret_cast<const uint4*>(a)[i];
  } else {
    for (int i = threadIdx.x; i < D; i += blockDim.x) o[i] = a[i];
  }
}

LEB_API int leb_gather_rows(void* out, const void* in, int dtype, const int* rows, int div, int P,
                            int D, cudaStream_t st) {
  if (P <= 0) return 0;
  LEB_REQUIRE(div >= 1, "leb_gather_rows: div must be positive");
  if (dtype == LEB_F32)
    leb_launch(gather_rows_kernel<float>, dim3(P), dim3(128), 0, st, (float*)out, (const float*)in, rows, div, D);
  else if (dtype == LEB_BF16)
    leb_launch(gather_rows_kernel<bf16>, dim3(P), dim3(128), 0, st, (bf16*)out, (const bf16*)in, rows, div, D);
  else
    return leb_fail("leb_gather_rows: unknown dtype %d", dtype);
  LEB_CHECK_LAUNCH("leb_gather_rows");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// x += y   (float residual; src/dense.rs:186,193)
__global__ void add_kernel(float* __restrict__ x, const float* __restrict__ y, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] += y[i];
}
LEB_API int leb_add(float* x, const float* y, size_t n, cudaStream_t st) {
  if (n == 0) return 0;
  add_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(x, y, n);
  LEB_CHECK_LAUNCH("leb_add");
  return 0;
}
