// What the weight-streaming products share: the structs of their epilogues and the PTX wrappers of
// the stream (asynchronous copies into shared memory, 16-byte shared loads, mma.m16n8k16).
#pragma once
#include "common.cuh"

// What the convolution epilogue needs beside the product (all null / 0 for the other epilogues).
struct StreamConv {
  const float* w;        // [D, Lc] taps, oldest first
  const float* bias;     // [D] or null
  float* state;          // [slots, D, Lc-1]
  const int* row_seq;    // row -> sequence of the step
  const int* seq_slot;   // sequence -> cache slot (-1: padding)
  int Lc;
};
#define ST_CONV_MAX_LC 5

// An RMSNorm split between the product before it and the product after it (decode steps, where a
// norm kernel of its own costs more in launch latency than in work).  The product that adds into
// the residual x also leaves bf16(x * g) (g: the norm's weight) and, per row and tile of 16
// columns, the sum of x^2; the product that follows reads the former as its activations, adds the
// latter up and multiplies its float sums by rsqrt(sum / D + eps).  Sum of squares, root and the
// scaling are float; the scale is applied after the product instead of before the rounding to
// bfloat16, which leaves the same relative rounding error.
struct StreamNorm {
  const float* ssq_in;   // [rows, parts_in] partial sums of squares of this product's input rows, or null
  int parts_in;
  int d_in;              // width of the input rows (what the mean is taken over)
  float eps;
  bf16* emit_vals;       // [rows, N] bf16(x_new * emit_g), or null (epilogue 1 only)
  const float* emit_g;   // [N]
  float* emit_ssq;       // [rows, ceil(N / 16)]
};

#define ST_ROWS 16
#define ST_CHUNK 64

__device__ __forceinline__ void st_mma(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void st_cp16(uint32_t dst, const void* src, int bytes) {
  // copies `bytes` (16 or 0) and fills the rest of the 16 with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void st_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void st_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint4 st_lds(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

