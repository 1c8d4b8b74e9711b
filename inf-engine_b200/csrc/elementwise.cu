// Embedding gather, RMSNorm fused with the residual sum, rotary position
// encoding fused with the write of keys and values into cache pages, and
// SiLU(gate) * up.  Statistics, angles and sums are float32 whatever the
// activation type is.
#include "common.cuh"

// ------------------------------------------------------------------ embedding
// residual[n, :] = table[ids[n], :]  (the reference gathers rows without
// scaling, engine/llama_model.py:128).  The residual stream is float32.
template <typename TW>
__global__ void embed_gather_kernel(const int* __restrict__ ids, const TW* __restrict__ table,
                                    float* __restrict__ residual, int d, int vocab) {
  pdl_trigger();
  pdl_wait();
  const int n = blockIdx.x;
  int id = ids[n];
  const bool ok = id >= 0 && id < vocab;
#ifdef IE_CHECKS
  if (threadIdx.x == 0) (void)IE_TOKEN(id);
#endif
  const TW* row = table + (size_t)(ok ? id : 0) * d;
  float* out = residual + (size_t)n * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) out[i] = ok ? to_f32(row[i]) : 0.f;
}

extern "C" int ie_embed_gather(const int* ids, const void* table, int table_dtype, float* residual,
                               int n_tokens, int d, int vocab, cudaStream_t stream) {
  if (n_tokens <= 0) return IE_OK;
  const int threads = d >= 1024 ? 256 : 128;
  if (table_dtype == IE_F32)
    return launch_k(embed_gather_kernel<float>, n_tokens, threads, 0, stream, ids, (const float*)table, residual, d, vocab);
  if (table_dtype == IE_BF16)
    return launch_k(embed_gather_kernel<bf16>, n_tokens, threads, 0, stream, ids, (const bf16*)table, residual, d, vocab);
  return IE_BAD_DTYPE;
}

// ids[i] = prev[src[i]] where src[i] >= 0: a token that the step before sampled and that the host has
// not read yet is taken on the device (steps are enqueued one ahead of the host's read of their results)
__global__ void patch_tokens_kernel(int* __restrict__ ids, const int* __restrict__ src, const int* __restrict__ prev, int n) {
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n && src[i] >= 0) ids[i] = prev[src[i]];
}
extern "C" int ie_patch_tokens(int* ids, const int* src, const int* prev, int n, cudaStream_t stream) {
  if (n <= 0) return IE_OK;
  return launch_k(patch_tokens_kernel, (n + 127) / 128, 128, 0, stream, ids, src, prev, n);
}

// A time stamp in stream order, for timelines of a step (diagnostics only): slot[0] = the GPU's nanosecond
// clock at the moment everything launched before it has finished.
__global__ void stamp_kernel(unsigned long long* slot) {
  pdl_trigger();
  pdl_wait();
  if (threadIdx.x == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    *slot = t;
  }
}
extern "C" int ie_stamp(unsigned long long* slot, cudaStream_t stream) {
  return launch_k(stamp_kernel, 1, 32, 0, stream, slot);
}

// -------------------------------------------------------------------- RMSNorm
// x = residual[row] (+ delta[row]);  residual[row] = x (unless rows are gathered);
// out[m] = x / sqrt(mean(x^2) + eps) * gain          (engine/layers.py:24-25)
// One block per output row; x is staged in shared memory between the two passes.
template <typename TA, typename TW>
__global__ void rmsnorm_kernel(float* __restrict__ residual, const TA* __restrict__ delta,
                               const TW* __restrict__ gain, TA* __restrict__ out,
                               const int* __restrict__ row_index, int d, float eps) {
  extern __shared__ float xs[];
  __shared__ float red[33];
  pdl_trigger();
  pdl_wait();
  const int m = blockIdx.x;
  const int row = row_index ? row_index[m] : m;
  float* res = residual + (size_t)row * d;
  const TA* del = delta ? delta + (size_t)row * d : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float x = res[i];
    if (del) x += to_f32(del[i]);
    xs[i] = x;
    ss += x * x;
    if (del && !row_index) res[i] = x;
  }
  const float total = block_sum(ss, red);
  const float rms = sqrtf(total / (float)d + eps);
  TA* o = out + (size_t)m * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = from_f32<TA>((xs[i] / rms) * to_f32(gain[i]));
}

// The same for bfloat16 activations when d is a multiple of 8 and at most 8192: a thread keeps its
// elements in registers (up to four groups of eight) and moves 16 or 32 bytes per access.
template <typename TW>
__global__ void __launch_bounds__(256) rmsnorm_bf16_vec_kernel(float* __restrict__ residual, const bf16* __restrict__ delta,
                                                               const TW* __restrict__ gain, bf16* __restrict__ out,
                                                               const int* __restrict__ row_index, int d, float eps) {
  __shared__ float red[33];
  pdl_trigger();
  pdl_wait();
  const int m = blockIdx.x;
  const int row = row_index ? row_index[m] : m;
  float* res = residual + (size_t)row * d;
  const bf16* del = delta ? delta + (size_t)row * d : nullptr;
  float x[4][8];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int i = (c * 256 + threadIdx.x) * 8;
    if (i < d) {
      const float4 a = *reinterpret_cast<const float4*>(res + i), b = *reinterpret_cast<const float4*>(res + i + 4);
      x[c][0] = a.x; x[c][1] = a.y; x[c][2] = a.z; x[c][3] = a.w; x[c][4] = b.x; x[c][5] = b.y; x[c][6] = b.z; x[c][7] = b.w;
      if (del) {
        const uint4 dv = *reinterpret_cast<const uint4*>(del + i);
        const __nv_bfloat162* dp = reinterpret_cast<const __nv_bfloat162*>(&dv);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(dp[j]);
          x[c][2 * j] += f.x;
          x[c][2 * j + 1] += f.y;
        }
        if (!row_index) {
          *reinterpret_cast<float4*>(res + i) = make_float4(x[c][0], x[c][1], x[c][2], x[c][3]);
          *reinterpret_cast<float4*>(res + i + 4) = make_float4(x[c][4], x[c][5], x[c][6], x[c][7]);
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += x[c][j] * x[c][j];
    }
  }
  const float total = block_sum(ss, red);
  const float rms = sqrtf(total / (float)d + eps);
  bf16* o = out + (size_t)m * d;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int i = (c * 256 + threadIdx.x) * 8;
    if (i < d) {
      uint4 ov;
      __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        op[j] = __floats2bfloat162_rn((x[c][2 * j] / rms) * to_f32(gain[i + 2 * j]),
                                      (x[c][2 * j + 1] / rms) * to_f32(gain[i + 2 * j + 1]));
      *reinterpret_cast<uint4*>(o + i) = ov;
    }
  }
}

template <typename TA, typename TW>
static int launch_rmsnorm(float* residual, const void* delta, const void* gain, void* out, const int* row_index,
                          int n_rows, int d, float eps, cudaStream_t stream) {
  if (sizeof(TA) == 2 && d % 8 == 0 && d <= 8192 && (((uintptr_t)residual | (uintptr_t)delta | (uintptr_t)out) & 15) == 0)
    return launch_k(rmsnorm_bf16_vec_kernel<TW>, n_rows, 256, 0, stream, residual, (const bf16*)delta, (const TW*)gain,
                    (bf16*)out, row_index, d, eps);
  const size_t smem = (size_t)d * sizeof(float);
  if (smem > 200 * 1024) return IE_BAD_SIZE;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(rmsnorm_kernel<TA, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int threads = d >= 2048 ? 512 : (d >= 512 ? 256 : 128);
  return launch_k(rmsnorm_kernel<TA, TW>, n_rows, threads, smem, stream, residual, (const TA*)delta, (const TW*)gain,
                  (TA*)out, row_index, d, eps);
}

extern "C" int ie_rmsnorm(float* residual, const void* delta, const void* gain, int gain_dtype, void* out,
                          int act_dtype, const int* row_index, int n_rows, int d, float eps, cudaStream_t stream) {
  if (n_rows <= 0) return IE_OK;
  if (act_dtype == IE_F32 && gain_dtype == IE_F32)
    return launch_rmsnorm<float, float>(residual, delta, gain, out, row_index, n_rows, d, eps, stream);
  if (act_dtype == IE_F32 && gain_dtype == IE_BF16)
    return launch_rmsnorm<float, bf16>(residual, delta, gain, out, row_index, n_rows, d, eps, stream);
  if (act_dtype == IE_BF16 && gain_dtype == IE_F32)
    return launch_rmsnorm<bf16, float>(residual, delta, gain, out, row_index, n_rows, d, eps, stream);
  if (act_dtype == IE_BF16 && gain_dtype == IE_BF16)
    return launch_rmsnorm<bf16, bf16>(residual, delta, gain, out, row_index, n_rows, d, eps, stream);
  return IE_BAD_DTYPE;
}

// residual[n, :] += delta[n, :]   (for a block arrangement that has no norm to fuse the sum into)
template <typename TA>
__global__ void residual_add_kernel(float* __restrict__ residual, const TA* __restrict__ delta, size_t n) {
  pdl_trigger();
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) residual[i] += to_f32(delta[i]);
}
extern "C" int ie_residual_add(float* residual, const void* delta, int act_dtype, int n_rows, int d,
                               cudaStream_t stream) {
  const size_t n = (size_t)n_rows * d;
  if (n == 0) return IE_OK;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  if (act_dtype == IE_F32) return launch_k(residual_add_kernel<float>, blocks, 256, 0, stream, residual, (const float*)delta, n);
  if (act_dtype == IE_BF16) return launch_k(residual_add_kernel<bf16>, blocks, 256, 0, stream, residual, (const bf16*)delta, n);
  return IE_BAD_DTYPE;
}

// ------------------------------------------------- rotary encoding + cache write
// For token n at position p:  q and k heads are rotated pairwise over (i, i+hd/2)
//   x'[i]      = x[i]*cos[p,i] - x[i+hd/2]*sin[p,i]
//   x'[i+hd/2] = x[i+hd/2]*cos[p,i] + x[i]*sin[p,i]          (engine/layers.py:82-115)
// q is rotated in place; the rotated k and the raw v go to the page slot
// slot_mapping[n] = page*page_size + offset of pools laid out
// [page, kv_head, page_size, head_dim]  (engine/paged_cache.py:119-123, 207-220).
// cos/sin are float32 [max_positions, hd/2]; a null table means no rotation.
// A negative slot (a padding token) writes nothing to the cache.
template <typename TA>
__global__ void rope_kv_write_kernel(TA* __restrict__ q, const TA* __restrict__ k, const TA* __restrict__ v,
                                     int q_stride, int kv_stride, const float* __restrict__ cos_t,
                                     const float* __restrict__ sin_t, const int* __restrict__ positions,
                                     const int* __restrict__ slot_mapping, TA* __restrict__ kpool,
                                     TA* __restrict__ vpool, int n_heads, int n_kv_heads, int hd, int page_size,
                                     int write_kv) {
  pdl_trigger();
  pdl_wait();
  const int n = blockIdx.x;
  const int half = hd >> 1;
  const int pos = positions[n];
  const float* c = cos_t ? cos_t + (size_t)pos * half : nullptr;
  const float* s = sin_t ? sin_t + (size_t)pos * half : nullptr;
  TA* qrow = q + (size_t)n * q_stride;
  const int q_pairs = (write_kv & 2) ? 0 : n_heads * half;      // bit 1: q is rotated elsewhere
  for (int idx = threadIdx.x; idx < q_pairs; idx += blockDim.x) {
    const int h = idx / half, i = idx - h * half;
    TA* x = qrow + h * hd;
    const float a = to_f32(x[i]), b = to_f32(x[i + half]);
    const float cc = c ? c[i] : 1.f, ss = s ? s[i] : 0.f;
    x[i] = from_f32<TA>(a * cc - b * ss);
    x[i + half] = from_f32<TA>(b * cc + a * ss);
  }
  if (!(write_kv & 1)) return;
  const int slot = IE_SLOT(slot_mapping[n]);
  if (slot < 0) return;
  const int page = slot / page_size, off = slot - page * page_size;
  const TA* krow = k + (size_t)n * kv_stride;
  const TA* vrow = v + (size_t)n * kv_stride;
  for (int idx = threadIdx.x; idx < n_kv_heads * half; idx += blockDim.x) {
    const int h = idx / half, i = idx - h * half;
    const size_t base = (((size_t)page * n_kv_heads + h) * page_size + off) * hd;
    const float a = to_f32(krow[h * hd + i]), b = to_f32(krow[h * hd + i + half]);
    const float cc = c ? c[i] : 1.f, ss = s ? s[i] : 0.f;
    kpool[base + i] = from_f32<TA>(a * cc - b * ss);
    kpool[base + i + half] = from_f32<TA>(b * cc + a * ss);
    vpool[base + i] = vrow[h * hd + i];
    vpool[base + i + half] = vrow[h * hd + i + half];
  }
}

// bfloat16, head_dim a multiple of 16: a thread rotates eight pairs (i..i+7 with i+hd/2..) at once.
__global__ void rope_kv_write_bf16_vec_kernel(bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v,
                                              int q_stride, int kv_stride, const float* __restrict__ cos_t,
                                              const float* __restrict__ sin_t, const int* __restrict__ positions,
                                              const int* __restrict__ slot_mapping, bf16* __restrict__ kpool,
                                              bf16* __restrict__ vpool, int n_heads, int n_kv_heads, int hd,
                                              int page_size, int write_kv) {
  pdl_trigger();
  pdl_wait();
  const int n = blockIdx.x;
  const int half = hd >> 1;
  const int groups = half >> 3;                 // groups of eight pairs per head
  const int pos = positions[n];
  const int slot = (write_kv & 1) ? IE_SLOT(slot_mapping[n]) : -1;
  const int page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot - page * page_size : 0;
  const int total = (n_heads + n_kv_heads) * groups;
  const int first = (write_kv & 2) ? n_heads * groups : 0;     // bit 1: q is rotated elsewhere
  for (int idx = first + threadIdx.x; idx < total; idx += blockDim.x) {
    const int h = idx / groups, i = (idx - h * groups) * 8;
    float cc[8], ss[8];
    if (cos_t) {
      const float4 c0 = *reinterpret_cast<const float4*>(cos_t + (size_t)pos * half + i);
      const float4 c1 = *reinterpret_cast<const float4*>(cos_t + (size_t)pos * half + i + 4);
      const float4 s0 = *reinterpret_cast<const float4*>(sin_t + (size_t)pos * half + i);
      const float4 s1 = *reinterpret_cast<const float4*>(sin_t + (size_t)pos * half + i + 4);
      cc[0] = c0.x; cc[1] = c0.y; cc[2] = c0.z; cc[3] = c0.w; cc[4] = c1.x; cc[5] = c1.y; cc[6] = c1.z; cc[7] = c1.w;
      ss[0] = s0.x; ss[1] = s0.y; ss[2] = s0.z; ss[3] = s0.w; ss[4] = s1.x; ss[5] = s1.y; ss[6] = s1.z; ss[7] = s1.w;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) { cc[j] = 1.f; ss[j] = 0.f; }
    }
    const bool is_q = h < n_heads;
    const int hk = h - n_heads;
    const bf16* src = is_q ? q + (size_t)n * q_stride + h * hd : k + (size_t)n * kv_stride + hk * hd;
    const uint4 lo = *reinterpret_cast<const uint4*>(src + i), hi = *reinterpret_cast<const uint4*>(src + i + half);
    const __nv_bfloat162* lp = reinterpret_cast<const __nv_bfloat162*>(&lo);
    const __nv_bfloat162* hp = reinterpret_cast<const __nv_bfloat162*>(&hi);
    uint4 olo, ohi;
    __nv_bfloat162* olp = reinterpret_cast<__nv_bfloat162*>(&olo);
    __nv_bfloat162* ohp = reinterpret_cast<__nv_bfloat162*>(&ohi);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 a = __bfloat1622float2(lp[j]), b = __bfloat1622float2(hp[j]);
      olp[j] = __floats2bfloat162_rn(a.x * cc[2 * j] - b.x * ss[2 * j], a.y * cc[2 * j + 1] - b.y * ss[2 * j + 1]);
      ohp[j] = __floats2bfloat162_rn(b.x * cc[2 * j] + a.x * ss[2 * j], b.y * cc[2 * j + 1] + a.y * ss[2 * j + 1]);
    }
    if (is_q) {
      bf16* dst = q + (size_t)n * q_stride + h * hd;
      *reinterpret_cast<uint4*>(dst + i) = olo;
      *reinterpret_cast<uint4*>(dst + i + half) = ohi;
    } else if (slot >= 0) {
      const size_t base = (((size_t)page * n_kv_heads + hk) * page_size + off) * hd;
      *reinterpret_cast<uint4*>(kpool + base + i) = olo;
      *reinterpret_cast<uint4*>(kpool + base + i + half) = ohi;
      const bf16* vsrc = v + (size_t)n * kv_stride + hk * hd;
      *reinterpret_cast<uint4*>(vpool + base + i) = *reinterpret_cast<const uint4*>(vsrc + i);
      *reinterpret_cast<uint4*>(vpool + base + i + half) = *reinterpret_cast<const uint4*>(vsrc + i + half);
    }
  }
}

// write_kv: bit 0: store the rotated key and the value at slot_mapping; bit 1: leave q alone (it is rotated
// where it is read)
extern "C" int ie_rope_kv_write(void* q, const void* k, const void* v, int q_stride, int kv_stride,
                                const float* cos_t, const float* sin_t, const int* positions,
                                const int* slot_mapping, void* kpool, void* vpool, int n_tokens, int n_heads,
                                int n_kv_heads, int hd, int page_size, int write_kv, int act_dtype,
                                cudaStream_t stream) {
  if (n_tokens <= 0) return IE_OK;
  if (hd % 2) return IE_BAD_SIZE;
  const int work = n_heads * hd / 2;
  const int threads = work >= 512 ? 256 : 128;
  if (act_dtype == IE_F32)
    return launch_k(rope_kv_write_kernel<float>, n_tokens, threads, 0, stream, (float*)q, (const float*)k,
                    (const float*)v, q_stride, kv_stride, cos_t, sin_t, positions, slot_mapping, (float*)kpool,
                    (float*)vpool, n_heads, n_kv_heads, hd, page_size, write_kv);
  if (act_dtype == IE_BF16 && hd % 16 == 0 && q_stride % 8 == 0 && kv_stride % 8 == 0 &&
      (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)kpool | (uintptr_t)vpool | (uintptr_t)cos_t |
        (uintptr_t)sin_t) & 15) == 0) {
    const int work8 = (n_heads + n_kv_heads) * (hd / 16);
    return launch_k(rope_kv_write_bf16_vec_kernel, n_tokens, work8 >= 128 ? 128 : 64, 0, stream, (bf16*)q,
                    (const bf16*)k, (const bf16*)v, q_stride, kv_stride, cos_t, sin_t, positions, slot_mapping,
                    (bf16*)kpool, (bf16*)vpool, n_heads, n_kv_heads, hd, page_size, write_kv);
  }
  if (act_dtype == IE_BF16)
    return launch_k(rope_kv_write_kernel<bf16>, n_tokens, threads, 0, stream, (bf16*)q, (const bf16*)k,
                    (const bf16*)v, q_stride, kv_stride, cos_t, sin_t, positions, slot_mapping, (bf16*)kpool,
                    (bf16*)vpool, n_heads, n_kv_heads, hd, page_size, write_kv);
  return IE_BAD_DTYPE;
}

// ---------------------------------------------------------------- SiLU(gate)*up
// in is [n, 2*inter]: gate in columns [0, inter) and up in [inter, 2*inter), or, when
// `interleaved`, gate_j in column 2j and up_j in column 2j+1;
// out[n, j] = gate*sigmoid(gate) * up          (engine/llama_mlp.py:32, engine/layers.py:28-30)
template <typename TA>
__global__ void silu_mul_kernel(const TA* __restrict__ in, TA* __restrict__ out, int inter, int in_stride,
                                size_t total, int interleaved) {
  pdl_trigger();
  pdl_wait();
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const size_t n = idx / inter;
  const int j = (int)(idx - n * inter);
  const float g = to_f32(in[n * in_stride + (interleaved ? 2 * j : j)]);
  const float u = to_f32(in[n * in_stride + (interleaved ? 2 * j + 1 : inter + j)]);
  const float sg = 1.f / (1.f + expf(-g));
  out[idx] = from_f32<TA>((g * sg) * u);
}

// bfloat16, eight outputs per thread (inter a multiple of 8, 16-byte aligned rows)
__global__ void silu_mul_bf16_vec_kernel(const bf16* __restrict__ in, bf16* __restrict__ out, int inter, int in_stride,
                                         size_t total8, int interleaved) {
  pdl_trigger();
  pdl_wait();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total8) return;
  const int per_row = inter >> 3;
  const size_t n = idx / per_row;
  const int j = (int)(idx - n * per_row) * 8;
  float g[8], u[8];
  const bf16* row = in + n * in_stride;
  if (interleaved) {
    const uint4 a = *reinterpret_cast<const uint4*>(row + 2 * j), b = *reinterpret_cast<const uint4*>(row + 2 * j + 8);
    const __nv_bfloat162* ap = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float2 x = __bfloat1622float2(ap[t]), y = __bfloat1622float2(bp[t]);
      g[t] = x.x; u[t] = x.y; g[4 + t] = y.x; u[4 + t] = y.y;
    }
  } else {
    const uint4 a = *reinterpret_cast<const uint4*>(row + j), b = *reinterpret_cast<const uint4*>(row + inter + j);
    const __nv_bfloat162* ap = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float2 x = __bfloat1622float2(ap[t]), y = __bfloat1622float2(bp[t]);
      g[2 * t] = x.x; g[2 * t + 1] = x.y; u[2 * t] = y.x; u[2 * t + 1] = y.y;
    }
  }
  uint4 o;
  __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const float a0 = g[2 * t], a1 = g[2 * t + 1];
    op[t] = __floats2bfloat162_rn((a0 * (1.f / (1.f + expf(-a0)))) * u[2 * t], (a1 * (1.f / (1.f + expf(-a1)))) * u[2 * t + 1]);
  }
  *reinterpret_cast<uint4*>(out + n * inter + j) = o;
}

extern "C" int ie_silu_mul(const void* in, void* out, int n_rows, int inter, int in_stride, int interleaved,
                           int act_dtype, cudaStream_t stream) {
  const size_t total = (size_t)n_rows * inter;
  if (total == 0) return IE_OK;
  if (act_dtype == IE_BF16 && inter % 8 == 0 && in_stride % 8 == 0 && (((uintptr_t)in | (uintptr_t)out) & 15) == 0) {
    const size_t total8 = total / 8;
    return launch_k(silu_mul_bf16_vec_kernel, (unsigned)((total8 + 255) / 256), 256, 0, stream, (const bf16*)in, (bf16*)out,
                    inter, in_stride, total8, interleaved);
  }
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (act_dtype == IE_F32)
    return launch_k(silu_mul_kernel<float>, blocks, 256, 0, stream, (const float*)in, (float*)out, inter, in_stride, total, interleaved);
  if (act_dtype == IE_BF16)
    return launch_k(silu_mul_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)in, (bf16*)out, inter, in_stride, total, interleaved);
  return IE_BAD_DTYPE;
}

IE_CHECK_API(elementwise)
