// Choosing the next token from float32 logits: argmax, or a draw from the
// distribution that temperature, top-k and top-p leave, and the repetition
// penalty that comes before them.  One block per row of logits; every sum is
// taken in a fixed order so that a seed gives the same token on every run.
//
// Rules follow engine/sampling.py of the reference:
//   greedy  argmax (:72-73)
//   scaled = logits / temperature (:75-77)
//   top-k   keep scaled >= the k-th largest, ties kept, k clamped to [1, V] (:138-153)
//   top-p   in descending order drop a token when the probability before it is
//           already >= p; the first always stays (:156-177).  Tokens of equal
//           value are kept or dropped together here.
//   draw    softmax over what is left, then one sample (:86-87).  The sample is
//           the inverse CDF in vocabulary order at a uniform number that is a
//           hash of (seed, key): it depends on the request and its position
//           only, not on what else is in the batch.
#include "common.cuh"

#define SM_THREADS 1024

struct SampleRow {
  float temperature;   // <= 0: greedy
  float top_p;         // >= 1: off
  int top_k;           // <= 0: off
  unsigned int seed_lo, seed_hi, key_lo, key_hi;
};

__device__ __forceinline__ unsigned int order_key(float x) {
  unsigned int u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);   // larger float <=> larger key
}

__device__ __forceinline__ unsigned long long splitmix64(unsigned long long x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

__device__ __forceinline__ int block_sum_int(int v, int* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n_warps = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    int t = lane < n_warps ? scratch[lane] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// ------------------------------------------------------------------- argmax
__global__ void __launch_bounds__(SM_THREADS) argmax_kernel(const float* __restrict__ logits, int* __restrict__ out,
                                                            int vocab, size_t row_stride) {
  __shared__ float sv[32];
  __shared__ int si[32];
  pdl_trigger();
  pdl_wait();
  const float* x = logits + (size_t)blockIdx.x * row_stride;
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = x[i];
    if (v > best || (v == best && i < best_i) || best_i == 0x7fffffff) { best = v; best_i = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sv[warp] = best; si[warp] = best_i; }
  __syncthreads();
  if (warp == 0) {
    const int n_warps = blockDim.x >> 5;
    best = lane < n_warps ? sv[lane] : -INFINITY;
    best_i = lane < n_warps ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (lane == 0) out[blockIdx.x] = best_i == 0x7fffffff ? 0 : best_i;
  }
}

extern "C" int ie_argmax(const float* logits, int* out, int n_rows, int vocab, long long row_stride,
                         cudaStream_t stream) {
  if (n_rows <= 0) return IE_OK;
  if (vocab <= 0) return IE_BAD_SIZE;
  return launch_k(argmax_kernel, n_rows, SM_THREADS, 0, stream, logits, out, vocab, (size_t)row_stride);
}

// --------------------------------------------------------- repetition penalty
// logits[row, t] is divided by `penalty` if positive, multiplied if negative, once
// for every distinct token t among the row's context tokens (engine/sampling.py:126-134;
// the caller passes the last 256 tokens, :90).  Negative ids are padding.
__global__ void repetition_penalty_kernel(float* __restrict__ logits, const int* __restrict__ context,
                                          const float* __restrict__ penalty, int vocab, size_t row_stride,
                                          int ctx_len) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  const float pen = penalty[row];
  if (pen == 1.0f) return;
  const int* c = context + (size_t)row * ctx_len;
  float* x = logits + (size_t)row * row_stride;
  for (int i = threadIdx.x; i < ctx_len; i += blockDim.x) {
    const int t = c[i];
    if (t < 0 || t >= vocab) continue;
    bool first = true;
    for (int j = 0; j < i; ++j)
      if (c[j] == t) { first = false; break; }
    if (!first) continue;
    const float v = x[t];
    x[t] = v < 0.f ? v * pen : v / pen;
  }
}

extern "C" int ie_repetition_penalty(float* logits, const int* context, const float* penalty, int n_rows,
                                     int vocab, long long row_stride, int ctx_len, cudaStream_t stream) {
  if (n_rows <= 0 || ctx_len <= 0) return IE_OK;
  return launch_k(repetition_penalty_kernel, n_rows, 256, 0, stream, logits, context, penalty, vocab,
                  (size_t)row_stride, ctx_len);
}

// --------------------------------------------------------------------- sample
// One row by one block of SM_THREADS threads: x its logits, r its record, *out its token.  The caller gives the
// block's scratch (red, redi: 33 words each; chunk_sum: SM_THREADS floats).
__device__ __forceinline__ void sample_row(const float* __restrict__ x, const SampleRow r, int* __restrict__ out, int vocab,
                                           float* red, int* redi, float* chunk_sum) {
  const int tid = threadIdx.x;

  // the maximum (and its first index, which is the greedy answer)
  float best = -INFINITY;
  for (int i = tid; i < vocab; i += SM_THREADS) best = fmaxf(best, x[i]);
  best = block_max(best, red);
  if (r.temperature <= 0.f) {
    int first = 0x7fffffff;
    for (int i = tid; i < vocab; i += SM_THREADS)
      if (x[i] == best) { first = i; break; }
    // minimum over the block
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) first = min(first, __shfl_xor_sync(0xffffffffu, first, o));
    __syncthreads();
    if ((tid & 31) == 0) redi[tid >> 5] = first;
    __syncthreads();
    if (tid < 32) {
      int t = redi[tid];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) t = min(t, __shfl_xor_sync(0xffffffffu, t, o));
      if (tid == 0) *out = t == 0x7fffffff ? 0 : t;
    }
    return;
  }
  const float m = best / r.temperature;

  // top-k: the key of the k-th largest scaled logit, bit by bit from the top
  unsigned int key_floor = 0u;   // keep keys >= key_floor
  if (r.top_k > 0 && r.top_k < vocab) {
    unsigned int prefix = 0u;
    for (int bit = 31; bit >= 0; --bit) {
      const unsigned int cand = prefix | (1u << bit);
      int cnt = 0;
      for (int i = tid; i < vocab; i += SM_THREADS) cnt += order_key(x[i] / r.temperature) >= cand;
      cnt = block_sum_int(cnt, redi);
      if (cnt >= r.top_k) prefix = cand;   // at least k keys are >= cand: the k-th largest is too
    }
    key_floor = prefix;
  }

  // top-p over what top-k left: the largest key K with mass(keys > K) < p keeps
  // every token whose own predecessors weigh less than p
  if (r.top_p < 1.0f) {
    float z = 0.f;
    for (int i = tid; i < vocab; i += SM_THREADS) {
      const float s = x[i] / r.temperature;
      if (order_key(s) >= key_floor) z += expf(s - m);
    }
    z = block_sum(z, red);
    const float budget = r.top_p * z;
    // smallest key K such that mass(keys > K) < budget; built bit by bit:
    // K has a bit cleared when clearing it still leaves mass(keys > K) < budget
    unsigned int K = 0xffffffffu;
    for (int bit = 31; bit >= 0; --bit) {
      const unsigned int cand = K & ~(1u << bit);
      float above = 0.f;
      for (int i = tid; i < vocab; i += SM_THREADS) {
        const float s = x[i] / r.temperature;
        const unsigned int k = order_key(s);
        if (k > cand && k >= key_floor) above += expf(s - m);
      }
      above = block_sum(above, red);
      if (above < budget) K = cand;
    }
    key_floor = max(key_floor, K);
  }

  // inverse CDF in vocabulary order over the kept tokens
  const int per = (vocab + SM_THREADS - 1) / SM_THREADS;
  const int lo = tid * per, hi = min(vocab, lo + per);
  float mine = 0.f;
  for (int i = lo; i < hi; ++i) {
    const float s = x[i] / r.temperature;
    if (order_key(s) >= key_floor) mine += expf(s - m);
  }
  chunk_sum[tid] = mine;
  __syncthreads();
  if (tid == 0) {
    float total = 0.f;
    for (int t = 0; t < SM_THREADS; ++t) total += chunk_sum[t];
    const unsigned long long seed = ((unsigned long long)r.seed_hi << 32) | r.seed_lo;
    const unsigned long long key = ((unsigned long long)r.key_hi << 32) | r.key_lo;
    const unsigned long long h = splitmix64(splitmix64(seed) ^ key);
    const float u = (float)(h >> 40) * (1.0f / 16777216.0f);   // 24 bits, in [0, 1)
    const float target = u * total;
    float run = 0.f;
    int t = 0;
    for (; t < SM_THREADS - 1; ++t) {
      if (run + chunk_sum[t] > target) break;
      run += chunk_sum[t];
    }
    // walk the chunk; the last kept token catches rounding at the very end
    int pick = -1, last_kept = -1;
    for (int tt = t; tt < SM_THREADS && pick < 0; ++tt) {
      const int l2 = tt * per, h2 = min(vocab, l2 + per);
      for (int i = l2; i < h2; ++i) {
        const float s = x[i] / r.temperature;
        if (order_key(s) < key_floor) continue;
        last_kept = i;
        run += expf(s - m);
        if (run > target) { pick = i; break; }
      }
    }
    if (pick < 0) {
      if (last_kept < 0)
        for (int i = vocab - 1; i >= 0; --i)
          if (order_key(x[i] / r.temperature) >= key_floor) { last_kept = i; break; }
      pick = last_kept < 0 ? 0 : last_kept;
    }
    *out = pick;
  }
}

__global__ void __launch_bounds__(SM_THREADS) sample_kernel(const float* __restrict__ logits,
                                                            const SampleRow* __restrict__ rows,
                                                            int* __restrict__ out, int vocab, size_t row_stride) {
  __shared__ float red[33];
  __shared__ int redi[33];
  __shared__ float chunk_sum[SM_THREADS];
  pdl_trigger();
  pdl_wait();
  sample_row(logits + (size_t)blockIdx.x * row_stride, rows[blockIdx.x], out + blockIdx.x, vocab, red, redi, chunk_sum);
}

// Greedy rows of a large vocabulary, spread over up to SG_CHUNKS blocks per row (fewer when there are many rows: the
// launch is kept near four blocks an SM; 64 rows over 64 blocks each were 4,096 blocks of two elements a thread): one
// block alone reads a row of half a megabyte at the speed of one SM.  Each block finds the maximum of its slice and its first index,
// takes a ticket of the row, and the block with the last ticket picks the best slice (ties: lowest index,
// as argmax does).  A row that is not greedy is sampled by its first block in the same launch (the other blocks of
// that row leave at once): one launch answers every row, whatever the mix.
#ifndef SG_CHUNKS
#define SG_CHUNKS 64
#endif
#define SG_MAX_ROWS 4096
__device__ float g_sg_val[SG_MAX_ROWS * SG_CHUNKS];
__device__ int g_sg_idx[SG_MAX_ROWS * SG_CHUNKS];
__device__ unsigned int g_sg_ticket[SG_MAX_ROWS];   // zero between launches

__global__ void __launch_bounds__(SM_THREADS) greedy_split_kernel(const float* __restrict__ logits,
                                                                  const SampleRow* __restrict__ rows, int* __restrict__ out,
                                                                  int vocab, size_t row_stride, int n_chunks) {
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ unsigned int last;
  __shared__ float red[33];
  __shared__ int redi[33];
  __shared__ float chunk_sum[SM_THREADS];
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.y, chunk = blockIdx.x;
  if (rows[row].temperature > 0.f) {                  // not a greedy row: its first block samples it
    if (chunk == 0) sample_row(logits + (size_t)row * row_stride, rows[row], out + row, vocab, red, redi, chunk_sum);
    return;
  }
  const int per = (vocab + n_chunks - 1) / n_chunks;
  const int lo = chunk * per, hi = min(vocab, lo + per);
  const float* x = logits + (size_t)row * row_stride;
  // four candidates a thread, each walking its own indices upwards (the first maximum of each stays), so that the
  // loads of a round are in flight together; then the lowest index among equal maxima wins, as everywhere below
  float cb[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
  int ci[4] = {0x7fffffff, 0x7fffffff, 0x7fffffff, 0x7fffffff};
  for (int i0 = lo + threadIdx.x; i0 < hi; i0 += 4 * SM_THREADS) {
    float v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] = (i0 + k * SM_THREADS < hi) ? x[i0 + k * SM_THREADS] : -INFINITY;
#pragma unroll
    for (int k = 0; k < 4; ++k)
      if (i0 + k * SM_THREADS < hi && (v[k] > cb[k] || ci[k] == 0x7fffffff)) { cb[k] = v[k]; ci[k] = i0 + k * SM_THREADS; }
  }
  float best = cb[0];
  int best_i = ci[0];
#pragma unroll
  for (int k = 1; k < 4; ++k)
    if (ci[k] != 0x7fffffff && (best_i == 0x7fffffff || cb[k] > best || (cb[k] == best && ci[k] < best_i))) { best = cb[k]; best_i = ci[k]; }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sv[warp] = best; si[warp] = best_i; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < SM_THREADS / 32; ++w)
      if (sv[w] > best || (sv[w] == best && si[w] < best_i)) { best = sv[w]; best_i = si[w]; }
    g_sg_val[row * SG_CHUNKS + chunk] = best;
    g_sg_idx[row * SG_CHUNKS + chunk] = best_i;
    __threadfence();
    last = atomicAdd(&g_sg_ticket[row], 1u);
    if (last == (unsigned int)n_chunks - 1) {
      __threadfence();
      float b = -INFINITY;
      int bi = 0x7fffffff;
      for (int c = 0; c < n_chunks; ++c) {
        const float v = __ldcg(&g_sg_val[row * SG_CHUNKS + c]);
        const int i = __ldcg(&g_sg_idx[row * SG_CHUNKS + c]);
        if (i != 0x7fffffff && (v > b || bi == 0x7fffffff || (v == b && i < bi))) { b = v; bi = i; }
      }
      out[row] = bi == 0x7fffffff ? 0 : bi;
      g_sg_ticket[row] = 0;
    }
  }
}

extern "C" int ie_sample(const float* logits, const void* rows, int* out, int n_rows, int vocab,
                         long long row_stride, cudaStream_t stream) {
  if (n_rows <= 0) return IE_OK;
  if (vocab <= 0) return IE_BAD_SIZE;
  if (vocab >= 32768 && n_rows <= SG_MAX_ROWS) {
    // one launch: greedy rows over several blocks each, every other row by its first block
    int n_chunks = (4 * 148 + n_rows - 1) / n_rows;
    n_chunks = n_chunks < 1 ? 1 : (n_chunks > SG_CHUNKS ? SG_CHUNKS : n_chunks);
    return launch_k(greedy_split_kernel, dim3(n_chunks, n_rows), SM_THREADS, 0, stream, logits, (const SampleRow*)rows, out,
                    vocab, (size_t)row_stride, n_chunks);
  }
  return launch_k(sample_kernel, n_rows, SM_THREADS, 0, stream, logits, (const SampleRow*)rows, out, vocab,
                  (size_t)row_stride);
}
