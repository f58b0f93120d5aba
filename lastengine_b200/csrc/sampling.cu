// Next-token choice on the device, one block per sequence.
//
// The reference samples on the host (src/local.rs:59-80) in this order, kept here:
//   penalties over the last 256 tokens, applied once per occurrence (repeat: l>0 ? l/rp : l*rp;
//   presence: l -= pp) -> temperature <= 0: argmax -> the top_k largest logits (0 means 64, at
//   most 256), sorted descending -> divide by temperature -> softmax with the maximum
//   subtracted -> top-p: keep the shortest prefix whose cumulative probability reaches top_p
//   (when 0 < top_p < 1) -> min-p: cut where p < p[0]*min_p, keeping at least one ->
//   r = u * sum(kept); walk the kept list subtracting p until r <= 0.
// The uniform number u comes from the caller (the reference's xorshift64 runs on the host).
// Differences: equal logits are ordered by lower token id first (the reference's selection is
// unstable, and its argmax returns the last of equal maxima).
#include "common.cuh"

#define SMP_THREADS 1024
#define SMP_MAX_K 256

__device__ __forceinline__ unsigned long long order_key(float v, int idx) {
  unsigned u = __float_as_uint(v);
  u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);  // larger float -> larger unsigned
  return ((unsigned long long)u << 32) | (unsigned)(0xffffffffu - (unsigned)idx);  // lower id wins
}

// one thread per sequence: occurrences compound in order, as in the reference's loop
__global__ void penalties_rows_kernel(float* __restrict__ logits, const int* __restrict__ hist,
                                      const int* __restrict__ hist_len, int hist_stride, int V,
                                      int n, float repeat_penalty, float presence_penalty) {
  int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= n) return;
  float* l = logits + (size_t)b * V;
  const int* h = hist + (size_t)b * hist_stride;
  int len = hist_len[b];
  for (int i = 0; i < len; i++) {
    int t = h[i];
    if (t < 0 || t >= V) continue;
    float v = l[t];
    if (repeat_penalty > 1.0f) v = v > 0.f ? v / repeat_penalty : v * repeat_penalty;
    l[t] = v - presence_penalty;
  }
}

LEB_API int leb_penalties(float* logits, const int* hist, const int* hist_len, int hist_stride,
                          int n, int V, float repeat_penalty, float presence_penalty,
                          cudaStream_t st) {
  if (n <= 0) return 0;
  penalties_rows_kernel<<<ceil_div(n, 64), 64, 0, st>>>(logits, hist, hist_len, hist_stride, V, n,
                                                        repeat_penalty, presence_penalty);
  LEB_CHECK_LAUNCH("leb_penalties");
  return 0;
}

// The same penalties for steps that run without the host (captured decode steps): the recent tokens
// of every sequence live in a ring per cache slot on the device, hist[slot][window], with
// hist_len[slot] the number of tokens the sequence has seen so far.  The order in which a ring's
// entries are applied does not matter: different tokens touch different logits, and the
// occurrences of one token apply the same function again and again.
__global__ void penalties_slots_kernel(float* __restrict__ logits, const int* __restrict__ hist,
                                       const int* __restrict__ hist_len, const int* __restrict__ seq_slot,
                                       int window, int V, int n, float repeat_penalty, float presence_penalty) {
  pdl_trigger();   // the kernel after this one may start and wait (see common.cuh)
  pdl_wait();
  int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= n) return;
  const int slot = seq_slot[b];
  if (slot < 0) return;
  float* l = logits + (size_t)b * V;
  const int* h = hist + (size_t)slot * window;
  const int len = min(hist_len[slot], window);
  for (int i = 0; i < len; i++) {
    int t = h[i];
    if (t < 0 || t >= V) continue;
    float v = l[t];
    if (repeat_penalty > 1.0f) v = v > 0.f ? v / repeat_penalty : v * repeat_penalty;
    l[t] = v - presence_penalty;
  }
}

// The chosen token of every live sequence goes into its ring (over the oldest entry once it is full).
__global__ void history_append_kernel(int* __restrict__ hist, int* __restrict__ hist_len,
                                      const int* __restrict__ seq_slot, const int* __restrict__ chosen,
                                      int window, int n) {
  pdl_trigger();   // the kernel after this one may start and wait (see common.cuh)
  pdl_wait();
  int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= n) return;
  const int slot = seq_slot[b];
  if (slot < 0) return;
  const int len = hist_len[slot];
  hist[(size_t)slot * window + len % window] = chosen[b];
  hist_len[slot] = len + 1;
}

LEB_API int leb_penalties_slots(float* logits, const int* hist, const int* hist_len, const int* seq_slot, int window,
                                int n, int V, float repeat_penalty, float presence_penalty, cudaStream_t st) {
  if (n <= 0) return 0;
  LEB_REQUIRE(window > 0, "leb_penalties_slots: the window must be positive");
  leb_launch(penalties_slots_kernel, dim3(ceil_div(n, 64)), dim3(64), 0, st, logits, hist, hist_len, seq_slot, window, V, n,
             repeat_penalty, presence_penalty);
  LEB_CHECK_LAUNCH("leb_penalties_slots");
  return 0;
}

LEB_API int leb_history_append(int* hist, int* hist_len, const int* seq_slot, const int* chosen, int window, int n,
                               cudaStream_t st) {
  if (n <= 0) return 0;
  LEB_REQUIRE(window > 0, "leb_history_append: the window must be positive");
  leb_launch(history_append_kernel, dim3(ceil_div(n, 64)), dim3(64), 0, st, hist, hist_len, seq_slot, chosen, window, n);
  LEB_CHECK_LAUNCH("leb_history_append");
  return 0;
}

__global__ void argmax_kernel(int* __restrict__ out, const float* __restrict__ logits, int V) {
  __shared__ unsigned long long best[32];
  const float* l = logits + (size_t)blockIdx.x * V;
  unsigned long long k = 0;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    unsigned long long c = order_key(l[i], i);
    k = c > k ? c : k;
  }
  for (int o = 16; o > 0; o >>= 1) {
    unsigned long long c = __shfl_xor_sync(0xffffffffu, k, o);
    k = c > k ? c : k;
  }
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) best[warp] = k;
  __syncthreads();
  if (warp == 0) {
    k = lane < (int)(blockDim.x >> 5) ? best[lane] : 0ull;
    for (int o = 16; o > 0; o >>= 1) {
      unsigned long long c = __shfl_xor_sync(0xffffffffu, k, o);
      k = c > k ? c : k;
    }
    if (lane == 0) out[blockIdx.x] = (int)(0xffffffffu - (unsigned)(k & 0xffffffffull));
  }
}

// Large vocabularies: several blocks per row fold their best (value, id) key into one word per
// row with atomicMax (a maximum does not depend on the order), and a second small kernel turns
// the keys into ids and clears the words for the next call.  The words live in the library
// (zero when it is loaded, zero again after every call).
#define ARGMAX_ROWS 4096
static __device__ unsigned long long g_argmax_best[ARGMAX_ROWS];

__global__ void argmax_part_kernel(const float* __restrict__ logits, int V, int per_block) {
  __shared__ unsigned long long best[8];
  pdl_trigger();   // the kernel after this one may start and wait (see common.cuh)
  pdl_wait();
  const float* l = logits + (size_t)blockIdx.x * V;
  const int lo = blockIdx.y * per_block, hi = min(V, lo + per_block);
  unsigned long long k = 0;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    unsigned long long c = order_key(l[i], i);
    k = c > k ? c : k;
  }
  for (int o = 16; o > 0; o >>= 1) {
    unsigned long long c = __shfl_xor_sync(0xffffffffu, k, o);
    k = c > k ? c : k;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) best[warp] = k;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); w++) k = best[w] > k ? best[w] : k;
    atomicMax(&g_argmax_best[blockIdx.x], k);
  }
}

__global__ void argmax_final_kernel(int* __restrict__ out, int n) {
  pdl_trigger();   // the kernel after this one may start and wait (see common.cuh)
  pdl_wait();
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  out[i] = (int)(0xffffffffu - (unsigned)(g_argmax_best[i] & 0xffffffffull));
  g_argmax_best[i] = 0ull;
}

LEB_API int leb_argmax(int* out, const float* logits, int n, int V, cudaStream_t st) {
  if (n <= 0) return 0;
  LEB_REQUIRE(V >= 1, "leb_argmax: empty vocabulary");
  if (V >= 8192 && n <= ARGMAX_ROWS) {
    const int per_block = 2048;
    dim3 grid(n, ceil_div(V, per_block));
    if (grid.y <= 65535) {
      leb_launch(argmax_part_kernel, grid, dim3(256), 0, st, logits, V, per_block);
      LEB_CHECK_LAUNCH("leb_argmax");
      leb_launch(argmax_final_kernel, dim3(ceil_div(n, 128)), dim3(128), 0, st, out, n);
      LEB_CHECK_LAUNCH("leb_argmax");
      return 0;
    }
  }
  argmax_kernel<<<n, 512, 0, st>>>(out, logits, V);
  LEB_CHECK_LAUNCH("leb_argmax");
  return 0;
}

// descending bitonic sort of n (a power of two) 64-bit keys in shared memory, by the whole block
__device__ __forceinline__ void sort_keys_desc(unsigned long long* a, int n) {
  for (int size = 2; size <= n; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = threadIdx.x; t < n; t += blockDim.x) {
        const int j = t ^ stride;
        if (j > t) {
          const bool desc = (t & size) == 0;
          const unsigned long long x = a[t], y = a[j];
          if (desc ? x < y : x > y) { a[t] = y; a[j] = x; }
        }
      }
      __syncthreads();
    }
  }
}

// The k largest (value, id) keys of the row, sorted, then the reference's serial tail on one thread
// (at most 256 elements).  Fast way: every thread takes the largest key of its share of the row;
// the k-th largest of those 1024 maxima is a bound that at least k keys reach, and in a row that
// is not laid out against it few more than k do: the keys that reach it are gathered in shared
// memory and sorted.  If more than 1024 keys reach the bound, the k-th largest key is found by
// radix selection over the whole row instead (eight passes), as slow as it is sure.
__global__ void __launch_bounds__(SMP_THREADS)
sample_kernel(int* __restrict__ out, const float* __restrict__ logits, const float* __restrict__ u01,
              int V, int k, float temperature, float top_p, float min_p) {
  __shared__ unsigned hist[256];
  __shared__ unsigned long long prefix_s;
  __shared__ int want_s;
  __shared__ unsigned long long list[SMP_THREADS];
  __shared__ unsigned long long cand[SMP_MAX_K];
  __shared__ float prob[SMP_MAX_K];
  __shared__ int n_cand, n_list;
  __shared__ unsigned long long bound_s;
  pdl_trigger();   // the kernel after this one may start and wait (see common.cuh)
  pdl_wait();
  const float* l = logits + (size_t)blockIdx.x * V;
  const int tid = threadIdx.x;

  // a thread's share of the row: pieces of four values, 1024 pieces apart (single values if the row
  // cannot be read in 16-byte pieces); several loads are in flight at a time
  const bool vec = (V & 3) == 0 && ((uintptr_t)l & 15) == 0;
  unsigned long long mine = 0ull;
  if (vec) {
    const float4* l4 = reinterpret_cast<const float4*>(l);
#pragma unroll 8
    for (int i = tid; i < V / 4; i += SMP_THREADS) {
      const float4 v = l4[i];
      const unsigned long long k0 = order_key(v.x, 4 * i), k1 = order_key(v.y, 4 * i + 1), k2 = order_key(v.z, 4 * i + 2),
                               k3 = order_key(v.w, 4 * i + 3);
      const unsigned long long a = k0 > k1 ? k0 : k1, b = k2 > k3 ? k2 : k3, c = a > b ? a : b;
      mine = c > mine ? c : mine;
    }
  } else {
#pragma unroll 8
    for (int i = tid; i < V; i += SMP_THREADS) {
      const unsigned long long key = order_key(l[i], i);
      mine = key > mine ? key : mine;
    }
  }
  // the largest key of each four neighbouring threads: 256 maxima, of which the k-th largest is
  // found by counting, for each, how many are larger (no sorting, one barrier)
#pragma unroll
  for (int o = 1; o <= 2; o <<= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, mine, o);
    mine = other > mine ? other : mine;
  }
  if ((tid & 3) == 0) list[tid >> 2] = mine;
  if (tid == 0) { n_list = 0; bound_s = 0ull; }
  __syncthreads();
  if (tid < 256) {
    const unsigned long long key = list[tid];
    int larger = 0;
#pragma unroll 8
    for (int j = 0; j < 256; j++) larger += list[j] > key ? 1 : 0;
    if (larger == k - 1) bound_s = key;   // empty shares have key 0: with fewer than k others the bound stays 0
  }
  __syncthreads();
  const unsigned long long bound = bound_s;   // at least k keys of the row are >= bound
  __syncthreads();
  auto reach = [&](unsigned long long key) {
    if (key >= bound) {
      const int p = atomicAdd(&n_list, 1);
      if (p < SMP_THREADS) list[p] = key;
    }
  };
  if (vec) {
    const float4* l4 = reinterpret_cast<const float4*>(l);
#pragma unroll 8
    for (int i = tid; i < V / 4; i += SMP_THREADS) {
      const float4 v = l4[i];
      reach(order_key(v.x, 4 * i));
      reach(order_key(v.y, 4 * i + 1));
      reach(order_key(v.z, 4 * i + 2));
      reach(order_key(v.w, 4 * i + 3));
    }
  } else {
#pragma unroll 8
    for (int i = tid; i < V; i += SMP_THREADS) reach(order_key(l[i], i));
  }
  __syncthreads();
  const int reached = n_list;
  if (reached <= 256) {
    // few keys reached the bound (the usual case): each finds its place by counting the larger ones
    if (tid < reached) {
      const unsigned long long key = list[tid];
      int larger = 0;
      for (int j = 0; j < reached; j++) larger += list[j] > key ? 1 : 0;
      if (larger < k) cand[larger] = key;
    }
    __syncthreads();
  } else if (reached <= SMP_THREADS) {
    int n = 2;
    while (n < reached) n <<= 1;
    for (int i = reached + tid; i < n; i += blockDim.x) list[i] = 0ull;
    __syncthreads();
    sort_keys_desc(list, n);
    for (int i = tid; i < SMP_MAX_K; i += blockDim.x) cand[i] = i < k ? list[i] : 0ull;
    __syncthreads();
  } else {
  // k-th largest key: fix its bytes from the top
  if (tid == 0) { prefix_s = 0ull; want_s = k; n_cand = 0; }
  __syncthreads();
  for (int byte = 7; byte >= 0; byte--) {
    if (tid < 256) hist[tid] = 0u;
    __syncthreads();
    const unsigned long long prefix = prefix_s;
    const unsigned long long himask = byte == 7 ? 0ull : (~0ull << (8 * (byte + 1)));
    for (int i = tid; i < V; i += blockDim.x) {
      unsigned long long key = order_key(l[i], i);
      if ((key & himask) == prefix) atomicAdd(&hist[(unsigned)(key >> (8 * byte)) & 255u], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      int want = want_s;  // rank (from the top) of the wanted key among those matching the prefix
      int b = 255;
      for (; b > 0; b--) {
        if ((int)hist[b] >= want) break;
        want -= (int)hist[b];
      }
      prefix_s = prefix | ((unsigned long long)b << (8 * byte));
      want_s = want;
    }
    __syncthreads();
  }
  const unsigned long long kth = prefix_s;  // keys are distinct: exactly k keys are >= kth
  for (int i = tid; i < V; i += blockDim.x) {
    unsigned long long key = order_key(l[i], i);
    if (key >= kth) {
      int p = atomicAdd(&n_cand, 1);
      if (p < SMP_MAX_K) cand[p] = key;
    }
  }
  __syncthreads();
  for (int i = tid; i < SMP_MAX_K; i += blockDim.x)
    if (i >= k) cand[i] = 0ull;
  __syncthreads();
  sort_keys_desc(cand, SMP_MAX_K);
  }
  if (tid == 0) {
    auto logit_of = [&](int i) { return l[(int)(0xffffffffu - (unsigned)(cand[i] & 0xffffffffull))]; };
    const float mx = logit_of(0) / temperature;
    float z = 0.f;
    for (int i = 0; i < k; i++) {
      float p = expf(logit_of(i) / temperature - mx);
      prob[i] = p;
      z += p;
    }
    for (int i = 0; i < k; i++) prob[i] /= z;
    int keep = k;
    float cum = 0.f;
    for (int i = 0; i < k; i++) {
      cum += prob[i];
      if (top_p > 0.f && top_p < 1.f && cum >= top_p) { keep = i + 1; break; }
    }
    if (min_p > 0.f) {
      float thr = prob[0] * min_p;
      int first_below = k;
      for (int i = 0; i < k; i++)
        if (prob[i] < thr) { first_below = i; break; }
      keep = keep < first_below ? keep : first_below;
      keep = keep < 1 ? 1 : keep;
    }
    float zk = 0.f;
    for (int i = 0; i < keep; i++) zk += prob[i];
    float r = u01[blockIdx.x] * zk;
    int pick = keep - 1;
    for (int i = 0; i < keep; i++) {
      r -= prob[i];
      if (r <= 0.f) { pick = i; break; }
    }
    out[blockIdx.x] = (int)(0xffffffffu - (unsigned)(cand[pick] & 0xffffffffull));
  }
}

LEB_API int leb_sample(int* out, const float* logits, const float* u01, int n, int V, int top_k,
                       float temperature, float top_p, float min_p, cudaStream_t st) {
  if (n <= 0) return 0;
  LEB_REQUIRE(temperature > 0.f, "leb_sample: temperature must be positive (use leb_argmax for greedy)");
  int k = top_k == 0 ? 64 : (top_k < SMP_MAX_K ? top_k : SMP_MAX_K);  // src/local.rs:65
  if (k > V) k = V;
  LEB_REQUIRE(k >= 1, "leb_sample: empty vocabulary");
  leb_launch(sample_kernel, dim3(n), dim3(SMP_THREADS), 0, st, out, logits, u01, V, k, temperature, top_p, min_p);
  LEB_CHECK_LAUNCH("leb_sample");
  return 0;
}

// After a decode step whose tokens were chosen on the device: the chosen tokens become the
// next step's input and every live sequence moves one position on, so the same launch
// sequence (a captured graph) can run again without the host.
__global__ void advance_kernel(int* __restrict__ tokens, int* __restrict__ row_pos,
                               int* __restrict__ seq_pos0, const int* __restrict__ seq_slot,
                               const int* __restrict__ chosen, int B) {
  pdl_trigger();   // the kernel after this one may start and wait (see common.cuh)
  pdl_wait();
  int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B || seq_slot[b] < 0) return;
  tokens[b] = chosen[b];
  row_pos[b] += 1;
  seq_pos0[b] += 1;
}

// Before a decode step that was launched ahead of the host reading the previous step's choice:
// sequence b takes as its token what the previous step chose for its place feed[b] there
// (feed[b] < 0: the token the host staged stays).
__global__ void feed_tokens_kernel(int* __restrict__ tokens, const int* __restrict__ chosen,
                                   const int* __restrict__ feed, int B) {
  pdl_trigger();   // the kernel after this one may start and wait (see common.cuh)
  pdl_wait();
  int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  int f = feed[b];
  if (f >= 0) tokens[b] = chosen[f];
}

LEB_API int leb_feed_tokens(int* tokens, const int* chosen, const int* feed, int B, cudaStream_t st) {
  if (B <= 0) return 0;
  leb_launch(feed_tokens_kernel, dim3(ceil_div(B, 128)), dim3(128), 0, st, tokens, chosen, feed, B);
  LEB_CHECK_LAUNCH("leb_feed_tokens");
  return 0;
}

LEB_API int leb_advance(int* tokens, int* row_pos, int* seq_pos0, const int* seq_slot,
                        const int* chosen, int B, cudaStream_t st) {
  if (B <= 0) return 0;
  leb_launch(advance_kernel, dim3(ceil_div(B, 128)), dim3(128), 0, st, tokens, row_pos, seq_pos0, seq_slot, chosen, B);
  LEB_CHECK_LAUNCH("leb_advance");
  return 0;
}
