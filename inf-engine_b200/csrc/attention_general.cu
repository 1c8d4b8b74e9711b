// Paged causal attention for any mix of prompt portions and decode tokens, any
// head size that is a multiple of 16 up to 256, any number of heads and groups,
// an optional window.  float32 arithmetic on CUDA cores with float32 or
// bfloat16 storage: this is the kernel of the true 32-bit path and the fallback
// of the bfloat16 path for sizes that the tensor-core kernels do not take.
//
// Formula (engine/llama_attention.py:106-137): for query token t of a request at
// absolute position p = ctx_before + t and query head h served by kv head
// c = h / group,  out = softmax(q k^T * scale + mask) v  over the keys j <= p
// (and j > p - window when a window is set).  Keys and values are read from the
// request's pages through its block table; the step's own tokens were written
// there before this kernel runs, so every cut of the work sees the same keys.
// An optional additive term enters the score before the softmax: a float32 table
// bias[head][distance], distance = p - j clamped to the table's last column
// (position encodings that bias scores by how far back a key lies).
//
// Work split: a block takes one (request, kv head) and a tile of 32
// (token, head-in-group) pairs, so the `group` query heads that share a kv head
// also share every key tile that is loaded.  Keys are walked in tiles of 32 at
// absolute multiples of 32, in ascending order, with an online softmax; the
// sequence of tiles that a (token, head) sees is the same however the tokens
// were cut into steps.
#include "common.cuh"

#define AG_ROWS 32
#define AG_KEYS 32
#define AG_THREADS 256
#define AG_MAX_ACC 32  // head_dim / 8 accumulators per thread, head_dim <= 256

struct AttnGeneralParams {
  const void* q;
  void* out;
  const void* kpool;
  const void* vpool;
  const int* block_table;
  const int* q_start;
  const int* ctx_before;
  const int* work_req;
  const int* work_pair0;
  int q_stride, out_stride, table_stride;
  int n_work, n_heads, n_kv_heads, hd, page_size, window;
  float scale;
  const float* score_bias;  // [n_heads][bias_dists] or null
  int bias_dists;
};

template <typename T>
__global__ void __launch_bounds__(AG_THREADS) attention_general_kernel(AttnGeneralParams p) {
  extern __shared__ float smem[];
  pdl_trigger();
  pdl_wait();
  const int hd = p.hd;
  const int ldq = hd + 1;
  float* Qs = smem;                      // [ROWS][hd+1]
  float* Ks = Qs + AG_ROWS * ldq;        // [KEYS][hd+1]
  float* Vs = Ks + AG_KEYS * ldq;        // [KEYS][hd]
  float* Ps = Vs + AG_KEYS * hd;         // [ROWS][KEYS+1]

  const int w = blockIdx.x;
  const int c = blockIdx.y;              // kv head
  const int r_id = p.work_req[w];
  const int pair0 = p.work_pair0[w];
  const int group = p.n_heads / p.n_kv_heads;
  const int q0 = p.q_start[r_id];
  const int q_len = p.q_start[r_id + 1] - q0;
  const int ctx = p.ctx_before[r_id];
  const int n_pairs = q_len * group;
  const int* table = p.block_table + (size_t)r_id * p.table_stride;
  const T* q = (const T*)p.q;
  const T* kpool = (const T*)p.kpool;
  const T* vpool = (const T*)p.vpool;

  const int tid = threadIdx.x;
  const int row = tid >> 3;              // 0..31
  const int sub = tid & 7;               // 0..7

  // stage the tile's queries
  for (int idx = tid; idx < AG_ROWS * hd; idx += AG_THREADS) {
    const int r = idx / hd, d = idx - r * hd;
    const int pr = pair0 + r;
    float val = 0.f;
    if (pr < n_pairs) {
      const int t = pr / group, j = pr - t * group;
      val = to_f32(q[(size_t)(q0 + t) * p.q_stride + (c * group + j) * hd + d]);
    }
    Qs[r * ldq + d] = val;
  }

  const int my_pair = pair0 + row;
  const bool row_valid = my_pair < n_pairs;
  const int my_t = row_valid ? my_pair / group : 0;
  const int my_limit = ctx + my_t;                                    // last visible key
  const int my_first = p.window > 0 ? max(0, my_limit - p.window + 1) : 0;
  const float* my_bias = (p.score_bias != nullptr && row_valid)
                             ? p.score_bias + (size_t)(c * group + (my_pair - my_t * group)) * p.bias_dists
                             : nullptr;

  const int last_pair = min(pair0 + AG_ROWS, n_pairs) - 1;
  const int key_end = ctx + last_pair / group + 1;                     // keys [.., key_end) matter to the tile
  int key_begin = 0;
  if (p.window > 0) {
    const int first_t = pair0 / group;
    key_begin = max(0, ctx + first_t - p.window + 1);
    key_begin = (key_begin / AG_KEYS) * AG_KEYS;
  }

  float acc[AG_MAX_ACC];
#pragma unroll
  for (int i = 0; i < AG_MAX_ACC; ++i) acc[i] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;
  const int n_acc = hd >> 3;

  for (int kt = key_begin; kt < key_end; kt += AG_KEYS) {
    __syncthreads();  // previous tile fully consumed (and Qs staged, first time)
    for (int idx = tid; idx < AG_KEYS * hd; idx += AG_THREADS) {
      const int kk = idx / hd, d = idx - kk * hd;
      const int kp = kt + kk;
      float kv = 0.f, vv = 0.f;
      if (kp < key_end) {
        const int page = IE_PAGE(table[kp / p.page_size]);
        if (page >= 0) {
          const size_t a = (((size_t)page * p.n_kv_heads + c) * p.page_size + (kp % p.page_size)) * hd + d;
          kv = to_f32(kpool[a]);
          vv = to_f32(vpool[a]);
        }
      }
      Ks[kk * ldq + d] = kv;
      Vs[kk * hd + d] = vv;
    }
    __syncthreads();

    // scores of this thread: keys sub, sub+8, sub+16, sub+24 of its row
    float s[4];
    float tile_max = -INFINITY;
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const int kk = sub + 8 * jj;
      const int kp = kt + kk;
      float dot = 0.f;
      const float* qr = Qs + row * ldq;
      const float* kr = Ks + kk * ldq;
      for (int d = 0; d < hd; ++d) dot += qr[d] * kr[d];
      const bool visible = row_valid && kp <= my_limit && kp >= my_first;
      float sc = dot * p.scale;
      if (visible && my_bias != nullptr) sc += my_bias[min(my_limit - kp, p.bias_dists - 1)];
      s[jj] = visible ? sc : -INFINITY;
      tile_max = fmaxf(tile_max, s[jj]);
    }
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, o));
    const float m_new = fmaxf(m_run, tile_max);
    float alpha = 1.f, psum = 0.f;
    if (m_new == -INFINITY) {
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) Ps[row * (AG_KEYS + 1) + sub + 8 * jj] = 0.f;
    } else {
      alpha = expf(m_run - m_new);  // exp(-inf) = 0 on the first tile with a visible key
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const float e = expf(s[jj] - m_new);
        Ps[row * (AG_KEYS + 1) + sub + 8 * jj] = e;
        psum += e;
      }
    }
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
    l_run = l_run * alpha + psum;
    m_run = m_new;
    __syncthreads();

    // out accumulators: dims sub, sub+8, ... of this row
    const float* pr_ = Ps + row * (AG_KEYS + 1);
#pragma unroll
    for (int i = 0; i < AG_MAX_ACC; ++i) {
      if (i < n_acc) {
        float a = acc[i] * alpha;
        const float* vcol = Vs + sub + 8 * i;
#pragma unroll 8
        for (int kk = 0; kk < AG_KEYS; ++kk) a += pr_[kk] * vcol[kk * hd];
        acc[i] = a;
      }
    }
  }

  if (row_valid) {
    const int j = my_pair - my_t * group;
    T* o = (T*)p.out + (size_t)(q0 + my_t) * p.out_stride + (c * group + j) * hd;
    const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
#pragma unroll
    for (int i = 0; i < AG_MAX_ACC; ++i)
      if (i < n_acc) o[sub + 8 * i] = from_f32<T>(acc[i] * inv);
  }
}

extern "C" int ie_attention_general(const void* q, void* out, const void* kpool, const void* vpool,
                                    const int* block_table, const int* q_start, const int* ctx_before,
                                    const int* work_req, const int* work_pair0, int q_stride, int out_stride,
                                    int table_stride, int n_work, int n_heads, int n_kv_heads, int hd,
                                    int page_size, int window, float scale, int act_dtype, const float* score_bias,
                                    int bias_dists, cudaStream_t stream) {
  if (n_work <= 0) return IE_OK;
  if (hd % 16 || hd > 8 * AG_MAX_ACC || hd <= 0) return IE_BAD_SIZE;
  if (n_kv_heads <= 0 || n_heads % n_kv_heads) return IE_BAD_SIZE;
  if (score_bias != nullptr && bias_dists <= 0) return IE_BAD_SIZE;
  AttnGeneralParams p;
  p.q = q; p.out = out; p.kpool = kpool; p.vpool = vpool; p.block_table = block_table;
  p.q_start = q_start; p.ctx_before = ctx_before; p.work_req = work_req; p.work_pair0 = work_pair0;
  p.q_stride = q_stride; p.out_stride = out_stride; p.table_stride = table_stride;
  p.n_work = n_work; p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.hd = hd; p.page_size = page_size;
  p.window = window; p.scale = scale; p.score_bias = score_bias; p.bias_dists = bias_dists;
  const size_t smem = sizeof(float) * ((size_t)AG_ROWS * (hd + 1) + (size_t)AG_KEYS * (hd + 1) +
                                       (size_t)AG_KEYS * hd + (size_t)AG_ROWS * (AG_KEYS + 1));
  dim3 grid(n_work, n_kv_heads);
  cudaError_t e;
  if (act_dtype == IE_F32) {
    e = cudaFuncSetAttribute(attention_general_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    return launch_k(attention_general_kernel<float>, grid, AG_THREADS, smem, stream, p);
  } else if (act_dtype == IE_BF16) {
    e = cudaFuncSetAttribute(attention_general_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    return launch_k(attention_general_kernel<bf16>, grid, AG_THREADS, smem, stream, p);
  }
  return IE_BAD_DTYPE;
}

IE_CHECK_API(attention_general)
