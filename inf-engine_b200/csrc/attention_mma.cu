// Paged attention on tensor cores for bfloat16, one head size per build
// (-DIE_HD=64 or 128): a prefill kernel for prompt portions and mixed batches,
// and a split-key decode kernel with its merge for steps of single tokens.
//
// Both walk a request's keys through its block table in tiles, keep scores,
// running maximum, running sum and the output accumulators in float32
// (online softmax), and pack the `group` query heads that share a kv head into
// the rows of one tile, so every key and value that is loaded serves all of
// them (engine/llama_attention.py:27-44 expands K and V in memory instead).
// Products run as mma.sync m16n8k16 on bfloat16 fragments read from shared
// memory with ldmatrix; tiles arrive with cp.async, double-buffered.
//
// Rows of a tile are (token, head-in-group) pairs p = token*group + j of one
// (request, kv head); a row sees keys first(p) <= key <= ctx_before + token,
// with first = limit - window + 1 when a window is set.
#include "common.cuh"

#ifndef IE_HD
#define IE_HD 64
#endif

namespace {

constexpr int HD = IE_HD;
constexpr int CHUNKS = HD / 8;   // 16-byte chunks in a row of HD bfloat16
constexpr int KSTEPS = HD / 16;  // k-steps of q k^T
constexpr int NT_O = HD / 8;     // 8-wide output tiles
constexpr float LOG2E = 1.4426950408889634f;

struct MmaAttnParams {
  const bf16* q;
  bf16* out;
  const bf16* kpool;
  const bf16* vpool;
  const int* block_table;
  const int* q_start;
  const int* ctx_before;
  const int* work_req;
  const int* work_pair0;
  float* part_o;   // decode: [n_tokens*n_heads, n_blocks, HD]
  float* part_ml;  // decode: [n_tokens*n_heads, n_blocks, 2]
  int* tickets;    // decode: [n_requests * n_kv_heads], zero between launches
  int n_blocks;    // decode: blocks per (request, kv head) = partial results per row
  int cluster_merge;  // decode: the blocks of a (request, kv head) are one thread-block cluster and add up through
                      // distributed shared memory instead of through global memory and a ticket
  int q_stride, out_stride, table_stride;
  int n_heads, n_kv_heads, page_size, window;
  int page_shift;  // log2(page_size) when it is a power of two, else -1
  int n_splits, split_keys;
  float scale_log2;
  // decode with the position encoding and the cache write folded in (every request brings one token):
  // fuse bit 0: q arrives unrotated and is rotated as it is loaded; bit 1: the token's key and value arrive
  // in k_new / v_new ([n_tokens, kv_stride] rows), the key is rotated, both join the keys of the step and
  // are written to their slot of the pool
  int fuse;
  const bf16* k_new;
  const bf16* v_new;
  int kv_stride;
  const float* cos_t;   // [positions, HD/2] float32, or null for no rotation
  const float* sin_t;
  const int* positions;
  const int* slot_mapping;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;  // 0 bytes read: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
// The same with an L2 policy.  A decode step reads every key and value once, and together they are far larger
// than L2: marked "evict first" they do not push out what the step reads again and again (activations, norm
// gains, the kernels' own code).
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ void cp_async16_hint(uint32_t dst, const void* src, bool valid, uint64_t pol) {
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2, %3;\n" ::"r"(dst), "l"(src), "r"(sz), "l"(pol) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3,
                                                  uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// byte offset of 16-byte chunk `chunk` of row `row` in a tile of rows of HD bfloat16;
// the XOR keeps the eight rows that one ldmatrix touches on different banks
__device__ __forceinline__ uint32_t swz(int row, int chunk) {
  return (uint32_t)(row * (HD * 2) + ((chunk ^ (row & 7)) << 4));
}

// Copy keys [k0, k0+KT) of kv head c (K and V) into shared memory, zero where a key
// is outside [0, k_end) or its page is not held.
// Page and offset of key kp: shifts when the page size is a power of two (the usual case), a
// division otherwise; the address arithmetic of a tile must stay far cheaper than its memory latency.
__device__ __forceinline__ void page_of(const MmaAttnParams& p, int kp, int& page_index, int& offset) {
  if (p.page_shift >= 0) {
    page_index = kp >> p.page_shift;
    offset = kp & (p.page_size - 1);
  } else {
    page_index = kp / p.page_size;
    offset = kp - page_index * p.page_size;
  }
}

template <int KT, int NTHREADS, bool STREAM = false>   // STREAM: keys read once (decode), marked "evict first" in L2
__device__ __forceinline__ void load_kv_tile(const MmaAttnParams& p, const int* table, int c, int k0, int k_end,
                                             uint32_t ks_addr, uint32_t vs_addr, int tid) {
  constexpr int ITERS = (KT * CHUNKS + NTHREADS - 1) / NTHREADS;
  constexpr int ROWS_PER_ITER = NTHREADS / CHUNKS;
  static_assert(NTHREADS % CHUNKS == 0, "a thread keeps its chunk column over the iterations");
  // a thread copies chunk `chunk` of rows row0, row0 + ROWS_PER_ITER, ...; first every page lookup
  // (independent loads that overlap), then the copies: a copy is a volatile statement, and a lookup
  // placed after it would have to wait for it
  const int row0 = tid / CHUNKS, chunk = tid - row0 * CHUNKS;
  int src_row[ITERS];   // row of the pool ((page * kv_heads + c) * page_size + offset), or -1
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int row = row0 + it * ROWS_PER_ITER;
    const int kp = k0 + row;
    src_row[it] = -1;
    if (row < KT && kp < k_end && kp >= 0) {
      int pi, po;
      page_of(p, kp, pi, po);
      const int page = IE_PAGE(__ldg(table + pi));
      if (page >= 0) src_row[it] = (page * p.n_kv_heads + c) * p.page_size + po;
    }
  }
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int row = row0 + it * ROWS_PER_ITER;
    if (row < KT) {
      const bool valid = src_row[it] >= 0;
      const size_t off = valid ? (size_t)src_row[it] * HD + chunk * 8 : 0;
      const uint32_t so = swz(row, chunk);
      if (STREAM) {
        const uint64_t pol = l2_evict_first_policy();
        cp_async16_hint(ks_addr + so, p.kpool + off, valid, pol);
        cp_async16_hint(vs_addr + so, p.vpool + off, valid, pol);
      } else {
        cp_async16(ks_addr + so, p.kpool + off, valid);
        cp_async16(vs_addr + so, p.vpool + off, valid);
      }
    }
  }
}

// One warp, 16 rows, one tile of KT keys that lies in shared memory: scores, online
// softmax update, output accumulation.  lim0/lim1 and first0/first1 bound the visible
// keys of the lane's two rows (row = lane/4 and lane/4 + 8).
// HALF: rows 8..15 of the tile do not exist (a decode step of a group of at most 8 heads): their share
// of the softmax arithmetic is left out; the MMAs compute them anyway.
template <int KT, bool HALF = false>
__device__ __forceinline__ void warp_tile(const uint32_t (&qf)[KSTEPS][4], float (&o)[NT_O][4], float (&m)[2],
                                          float (&l)[2], uint32_t ks_addr, uint32_t vs_addr, int k0, int lim0,
                                          int lim1, int first0, int first1, bool need_mask, float scale_log2,
                                          int lane) {
  constexpr int NT_S = KT / 8;
  float s[NT_S][4];
#pragma unroll
  for (int i = 0; i < NT_S; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
  for (int n2 = 0; n2 < KT / 16; ++n2) {
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      uint32_t b0, b1, b2, b3;
      const int key = n2 * 16 + (lane & 7) + ((lane >> 4) << 3);
      const int chunk = ks * 2 + ((lane >> 3) & 1);
      ldmatrix_x4(b0, b1, b2, b3, ks_addr + swz(key, chunk));
      mma_bf16(s[2 * n2], qf[ks], b0, b1);
      mma_bf16(s[2 * n2 + 1], qf[ks], b2, b3);
    }
  }
  const int col = (lane & 3) * 2;
  float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
  for (int i = 0; i < NT_S; ++i) {
    if (need_mask) {
      const int kp = k0 + i * 8 + col;
      if (kp > lim0 || kp < first0) s[i][0] = -INFINITY;
      if (kp + 1 > lim0 || kp + 1 < first0) s[i][1] = -INFINITY;
      if (!HALF) {
        if (kp > lim1 || kp < first1) s[i][2] = -INFINITY;
        if (kp + 1 > lim1 || kp + 1 < first1) s[i][3] = -INFINITY;
      }
    }
    mx0 = fmaxf(mx0, fmaxf(s[i][0], s[i][1]));
    if (!HALF) mx1 = fmaxf(mx1, fmaxf(s[i][2], s[i][3]));
  }
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
  if (!HALF) {
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
  }
  // maxima are kept in the exponent's units (score * scale * log2 e); the scale is positive, so it commutes
  // with the maximum, and it enters each probability as one fused multiply-add: 2^(s*scale - m)
  const float mn0 = fmaxf(m[0], mx0 * scale_log2), mn1 = fmaxf(m[1], mx1 * scale_log2);
  const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;
  const float c0 = fast_exp2(m[0] - ms0), c1 = fast_exp2(m[1] - ms1);  // exp2(-inf) = 0
  m[0] = mn0;
  m[1] = mn1;
  float sum0 = 0.f, sum1 = 0.f;
  uint32_t pf[NT_S][2];
#pragma unroll
  for (int i = 0; i < NT_S; ++i) {
    const float p0 = fast_exp2(fmaf(s[i][0], scale_log2, -ms0)), p1 = fast_exp2(fmaf(s[i][1], scale_log2, -ms0));
    sum0 += p0 + p1;
    pf[i][0] = pack_bf16(p0, p1);
    if (!HALF) {
      const float p2 = fast_exp2(fmaf(s[i][2], scale_log2, -ms1)), p3 = fast_exp2(fmaf(s[i][3], scale_log2, -ms1));
      sum1 += p2 + p3;
      pf[i][1] = pack_bf16(p2, p3);
    } else {
      pf[i][1] = 0u;
    }
  }
  l[0] = l[0] * c0 + sum0;
  l[1] = l[1] * c1 + sum1;
  if (__any_sync(0xffffffffu, c0 != 1.f || c1 != 1.f)) {   // once a row's maximum has settled there is nothing to rescale
#pragma unroll
    for (int i = 0; i < NT_O; ++i) {
      o[i][0] *= c0;
      o[i][1] *= c0;
      if (!HALF) {
        o[i][2] *= c1;
        o[i][3] *= c1;
      }
    }
  }
#pragma unroll
  for (int kk = 0; kk < KT / 16; ++kk) {
    const uint32_t a[4] = {pf[2 * kk][0], pf[2 * kk][1], pf[2 * kk + 1][0], pf[2 * kk + 1][1]};
#pragma unroll
    for (int d2 = 0; d2 < HD / 16; ++d2) {
      uint32_t v0, v1, v2, v3;
      const int key = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
      const int chunk = d2 * 2 + (lane >> 4);
      ldmatrix_x4_trans(v0, v1, v2, v3, vs_addr + swz(key, chunk));
      mma_bf16(o[2 * d2], a, v0, v1);
      mma_bf16(o[2 * d2 + 1], a, v2, v3);
    }
  }
}

// q fragments of the lane's two rows straight from global memory (zeros for rows past the end)
__device__ __forceinline__ void load_q_frags(uint32_t (&qf)[KSTEPS][4], const bf16* row0, const bf16* row1,
                                             int lane) {
  const int col = (lane & 3) * 2;
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) {
    qf[ks][0] = row0 ? *reinterpret_cast<const uint32_t*>(row0 + ks * 16 + col) : 0u;
    qf[ks][1] = row1 ? *reinterpret_cast<const uint32_t*>(row1 + ks * 16 + col) : 0u;
    qf[ks][2] = row0 ? *reinterpret_cast<const uint32_t*>(row0 + ks * 16 + 8 + col) : 0u;
    qf[ks][3] = row1 ? *reinterpret_cast<const uint32_t*>(row1 + ks * 16 + 8 + col) : 0u;
  }
}

// ------------------------------------------------------------------- prefill
constexpr int PF_KT = 64;
constexpr int PF_STAGE_BYTES = 2 * PF_KT * HD * 2;  // K and V of one stage

// PF_WARPS warps of 16 rows each: 4 (tiles of 64 rows) or 8 (tiles of 128 rows, for long portions: a key tile
// that is loaded then serves twice as many rows)
template <int PF_WARPS>
__global__ void __launch_bounds__(PF_WARPS * 32) attention_prefill_kernel(MmaAttnParams p) {
  constexpr int PF_THREADS = PF_WARPS * 32;
  constexpr int PF_ROWS = PF_WARPS * 16;
  extern __shared__ __align__(128) unsigned char smem[];
  pdl_trigger();
  pdl_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int c = blockIdx.y;
  const int r_id = p.work_req[blockIdx.x];
  const int pair0 = p.work_pair0[blockIdx.x];
  const int group = p.n_heads / p.n_kv_heads;
  const int q0 = p.q_start[r_id];
  const int q_len = p.q_start[r_id + 1] - q0;
  const int ctx = p.ctx_before[r_id];
  const int n_pairs = q_len * group;
  const int* table = p.block_table + (size_t)r_id * p.table_stride;

  // the lane's two rows
  const int pr0 = pair0 + warp * 16 + (lane >> 2), pr1 = pr0 + 8;
  const bool v0 = pr0 < n_pairs, v1 = pr1 < n_pairs;
  const int t0 = v0 ? pr0 / group : 0, t1 = v1 ? pr1 / group : 0;
  const int lim0 = v0 ? ctx + t0 : -1, lim1 = v1 ? ctx + t1 : -1;
  const int first0 = p.window > 0 ? max(0, lim0 - p.window + 1) : 0;
  const int first1 = p.window > 0 ? max(0, lim1 - p.window + 1) : 0;
  const bf16* qr0 = v0 ? p.q + (size_t)(q0 + t0) * p.q_stride + (c * group + (pr0 - t0 * group)) * HD : nullptr;
  const bf16* qr1 = v1 ? p.q + (size_t)(q0 + t1) * p.q_stride + (c * group + (pr1 - t1 * group)) * HD : nullptr;
  uint32_t qf[KSTEPS][4];
  load_q_frags(qf, qr0, qr1, lane);

  // keys that matter to the block and to this warp
  const int last_pair = min(pair0 + PF_ROWS, n_pairs) - 1;
  const int k_end = ctx + last_pair / group + 1;
  int k_begin = 0;
  if (p.window > 0) k_begin = (max(0, ctx + pair0 / group - p.window + 1) / PF_KT) * PF_KT;
  const int w_first_pair = pair0 + warp * 16;
  const int w_last_pair = min(w_first_pair + 16, n_pairs) - 1;
  const bool warp_has_rows = w_first_pair < n_pairs;
  const int w_max_lim = warp_has_rows ? ctx + w_last_pair / group : -1;
  const int w_min_lim = warp_has_rows ? ctx + w_first_pair / group : -1;
  const int w_min_first = p.window > 0 ? max(0, w_min_lim - p.window + 1) : 0;
  const int w_max_first = p.window > 0 ? max(0, w_max_lim - p.window + 1) : 0;

  float o[NT_O][4];
#pragma unroll
  for (int i = 0; i < NT_O; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  const uint32_t base = smem_u32(smem);
  const int n_tiles = (k_end - k_begin + PF_KT - 1) / PF_KT;
  load_kv_tile<PF_KT, PF_THREADS>(p, table, c, k_begin, k_end, base, base + PF_KT * HD * 2, tid);
  cp_async_commit();
  for (int i = 0; i < n_tiles; ++i) {
    const int k0 = k_begin + i * PF_KT;
    if (i + 1 < n_tiles) {
      const uint32_t nb = base + ((i + 1) & 1) * PF_STAGE_BYTES;
      load_kv_tile<PF_KT, PF_THREADS>(p, table, c, k0 + PF_KT, k_end, nb, nb + PF_KT * HD * 2, tid);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    // skip tiles that no row of this warp can see
    if (warp_has_rows && k0 <= w_max_lim && k0 + PF_KT > w_min_first) {
      const uint32_t sb = base + (i & 1) * PF_STAGE_BYTES;
      const bool need_mask = (k0 + PF_KT - 1 > w_min_lim) || (k0 < w_max_first);
      warp_tile<PF_KT>(qf, o, m, l, sb, sb + PF_KT * HD * 2, k0, lim0, lim1, first0, first1, need_mask,
                       p.scale_log2, lane);
    }
    __syncthreads();
  }

  // row sums across the quad, normalise, store
  l[0] += __shfl_xor_sync(0xffffffffu, l[0], 1);
  l[0] += __shfl_xor_sync(0xffffffffu, l[0], 2);
  l[1] += __shfl_xor_sync(0xffffffffu, l[1], 1);
  l[1] += __shfl_xor_sync(0xffffffffu, l[1], 2);
  const int col = (lane & 3) * 2;
  if (v0) {
    const float inv = l[0] > 0.f ? 1.f / l[0] : 0.f;
    bf16* dst = p.out + (size_t)(q0 + t0) * p.out_stride + (c * group + (pr0 - t0 * group)) * HD;
#pragma unroll
    for (int i = 0; i < NT_O; ++i)
      *reinterpret_cast<uint32_t*>(dst + i * 8 + col) = pack_bf16(o[i][0] * inv, o[i][1] * inv);
  }
  if (v1) {
    const float inv = l[1] > 0.f ? 1.f / l[1] : 0.f;
    bf16* dst = p.out + (size_t)(q0 + t1) * p.out_stride + (c * group + (pr1 - t1 * group)) * HD;
#pragma unroll
    for (int i = 0; i < NT_O; ++i)
      *reinterpret_cast<uint32_t*>(dst + i * 8 + col) = pack_bf16(o[i][2] * inv, o[i][3] * inv);
  }
}

// ---- rotation folded into the decode kernel (half-split pairs: dim i with dim i + HD/2;
// engine/layers.py:82-115 of the reference: x*cos + rotate_half(x)*sin)
__device__ __forceinline__ void rotate_pair(uint32_t& lo, uint32_t& hi, float c0, float c1, float s0, float s1) {
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&lo));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&hi));
  lo = pack_bf16(a.x * c0 - b.x * s0, a.y * c1 - b.y * s1);
  hi = pack_bf16(b.x * c0 + a.x * s0, b.y * c1 + a.y * s1);
}

// q fragments of one token (both rows of a lane belong to it) rotated in registers: the partner of the
// dims of k-step ks sits at the same place of k-step ks + KSTEPS/2.  cs / sn hold the lane's cosines and
// sines: [ks][0] for dims ks*16 + col, col+1, [ks][1] for dims ks*16 + 8 + col, col+1.
__device__ __forceinline__ float2 ld_nc_f2(const float* p) {   // volatile: stays where it is written (before a wait)
  float2 v;
  asm volatile("ld.global.nc.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "l"(p));
  return v;
}
// cos_row / sin_row: the position's HD/2 cosines and sines in shared memory
__device__ __forceinline__ void rotate_q_frags(uint32_t (&qf)[KSTEPS][4], const float* cos_row, const float* sin_row,
                                               int lane) {
  const int col = (lane & 3) * 2;
#pragma unroll
  for (int ks = 0; ks < KSTEPS / 2; ++ks) {
#pragma unroll
    for (int h8 = 0; h8 < 2; ++h8) {
      const float2 cc = *reinterpret_cast<const float2*>(cos_row + ks * 16 + h8 * 8 + col);
      const float2 ss = *reinterpret_cast<const float2*>(sin_row + ks * 16 + h8 * 8 + col);
      rotate_pair(qf[ks][h8 * 2], qf[ks + KSTEPS / 2][h8 * 2], cc.x, cc.y, ss.x, ss.y);
      rotate_pair(qf[ks][h8 * 2 + 1], qf[ks + KSTEPS / 2][h8 * 2 + 1], cc.x, cc.y, ss.x, ss.y);
    }
  }
}

// The step's own key (rotated) and value of kv head c go into row `row` of the tile in shared memory and, if
// the token has a slot, into the pool.  Lanes [0, HD/16) take the key, eight pairs each; the next HD/8 lanes
// copy the value.  The projections are fetched right after the kernel ahead has finished (NewKv); rotation and
// stores happen when the tile has arrived.
struct NewKv {
  uint4 a, b;   // key lanes: dims lane*8.. and their partners; value lanes: a only
};
__device__ __forceinline__ void load_new_kv(NewKv& n, const MmaAttnParams& p, int token, int c, int lane) {
  constexpr int KL = HD / 16;
  if (lane < KL) {
    const bf16* src = p.k_new + (size_t)token * p.kv_stride + c * HD + lane * 8;
    n.a = *reinterpret_cast<const uint4*>(src);
    n.b = *reinterpret_cast<const uint4*>(src + HD / 2);
  } else if (lane < KL + CHUNKS) {
    n.a = *reinterpret_cast<const uint4*>(p.v_new + (size_t)token * p.kv_stride + c * HD + (lane - KL) * 8);
  }
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, const uint4& v) {
  asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void insert_new_kv(const MmaAttnParams& p, NewKv n, const float* cos_row, const float* sin_row,
                                              bool rotate, int slot, int c, int row, uint32_t ks_addr, uint32_t vs_addr,
                                              int lane) {
  constexpr int KL = HD / 16;
  size_t dst = 0;
  if (slot >= 0) {
    int page, off;
    page_of(p, slot, page, off);
    dst = ((size_t)(page * p.n_kv_heads + c) * p.page_size + off) * HD;
  }
  if (lane < KL) {
    if (rotate) {
      const float4 c0 = *reinterpret_cast<const float4*>(cos_row + lane * 8), c1 = *reinterpret_cast<const float4*>(cos_row + lane * 8 + 4);
      const float4 s0 = *reinterpret_cast<const float4*>(sin_row + lane * 8), s1 = *reinterpret_cast<const float4*>(sin_row + lane * 8 + 4);
      rotate_pair(n.a.x, n.b.x, c0.x, c0.y, s0.x, s0.y);
      rotate_pair(n.a.y, n.b.y, c0.z, c0.w, s0.z, s0.w);
      rotate_pair(n.a.z, n.b.z, c1.x, c1.y, s1.x, s1.y);
      rotate_pair(n.a.w, n.b.w, c1.z, c1.w, s1.z, s1.w);
    }
    st_shared_v4(ks_addr + swz(row, lane), n.a);
    st_shared_v4(ks_addr + swz(row, lane + KL), n.b);
    if (slot >= 0) {
      bf16* kp = const_cast<bf16*>(p.kpool) + dst + lane * 8;
      *reinterpret_cast<uint4*>(kp) = n.a;
      *reinterpret_cast<uint4*>(kp + HD / 2) = n.b;
    }
  } else if (lane < KL + CHUNKS) {
    const int ch = lane - KL;
    st_shared_v4(vs_addr + swz(row, ch), n.a);
    if (slot >= 0) *reinterpret_cast<uint4*>(const_cast<bf16*>(p.vpool) + dst + ch * 8) = n.a;
  }
}

// Diagnostics, compiled in with -DIE_ATTN_TRACE only: thread 0 of block (0, 0, 0) of every decode launch notes the
// GPU's nanosecond clock at eight points of its life; ie_attention_trace_read() hands the notes to the host.
#ifdef IE_ATTN_TRACE
constexpr int TRACE_LAUNCHES = 4096, TRACE_POINTS = 8;
__device__ unsigned long long g_trace[TRACE_LAUNCHES * TRACE_POINTS];
__device__ unsigned int g_trace_n = 0;
__device__ __forceinline__ unsigned long long trace_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define TRACE_BEGIN() unsigned int trace_id = TRACE_LAUNCHES; \
  if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 0) { trace_id = atomicAdd(&g_trace_n, 1u); \
    if (trace_id < TRACE_LAUNCHES) for (int i_ = 0; i_ < TRACE_POINTS; ++i_) g_trace[trace_id * TRACE_POINTS + i_] = 0; }
#define TRACE(point) { if (trace_id < TRACE_LAUNCHES) g_trace[trace_id * TRACE_POINTS + (point)] = trace_now(); }
#else
#define TRACE_BEGIN()
#define TRACE(point)
#endif

// -------------------------------------------------------------------- decode
// A request brings at most 16 rows (q_len * group <= 16).  Block (x, kv head, request) has DC_WARPS warps,
// each with one split of the keys: consecutive splits, so that a block covers DC_WARPS * split_keys keys.
// A warp keeps up to DC_STAGES key tiles in flight (a decode step is a matter of latency: few bytes per
// warp, all of them wanted as early as possible).  The warps of a block add their partial results up
// through shared memory, in ascending order of the splits.  A (request, kv head) that one block covers
// is finished there.  Otherwise, with up to 8 blocks per (request, kv head) in a launch that the SMs hold at once,
// these blocks are launched as one thread-block cluster: each leaves its result in its own shared memory, and after a cluster barrier the first
// of them adds the blocks up in ascending order, reading the others' shared memory.  With more blocks each
// writes one partial result to global memory and takes a ticket, and the block that takes the last ticket adds
// the blocks up, again in ascending order: the result does not depend on which block that is, nor on the path.
// Six warps a block at both head sizes, 96 KB of tiles per block (two blocks share an SM): tiles of 32 keys at head
// size 64, of 16 keys at 128.  (Three warps with tiles of 32 keys at head size 128 read 64 requests of 8,192 keys at
// 4.4 TB/s, six warps with tiles of 16 at 6.4 TB/s: a tile's MMAs and softmax are one dependent chain per warp, and
// three warps a block left the SM waiting on it.)
#ifndef IE_DC_WARPS
#define IE_DC_WARPS 6
#endif
constexpr int DC_WARPS = IE_DC_WARPS;
constexpr int DC_THREADS = DC_WARPS * 32;
#ifndef IE_DC_KT
#define IE_DC_KT (HD <= 64 ? 32 : 16)
#endif
#ifndef IE_DC_STAGES
#define IE_DC_STAGES 2
#endif
constexpr int DC_KT = IE_DC_KT;
constexpr int DC_STAGES = IE_DC_STAGES;
constexpr int DC_STAGE_BYTES = 2 * DC_KT * HD * 2;
constexpr int DC_WARP_BYTES = DC_STAGES * DC_STAGE_BYTES;
constexpr int DC_RESULT_BYTES = (16 * HD + 32) * 4;   // a block's result for the cluster: [16][HD] sums, [16][2] (max, sum)
constexpr int DC_SMEM_BYTES = DC_WARPS * DC_WARP_BYTES + DC_RESULT_BYTES;

__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_map(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  return remote;
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ float2 ld_cluster_f32x2(uint32_t addr) {
  float2 v;
  asm volatile("ld.shared::cluster.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr) : "memory");
  return v;
}

__device__ __forceinline__ void cp_async_wait_pending(int pending) {
  switch (pending) {
    case 0: cp_async_wait<0>(); break;
    case 1: cp_async_wait<1>(); break;
    case 2: cp_async_wait<2>(); break;
    default: cp_async_wait<3>(); break;
  }
}

// head size 64: at most 112 registers at 192 threads, so that the block fits beside the product kernels ahead of
// and behind it in the stream
__global__ void __launch_bounds__(DC_THREADS, HD <= 64 ? 3 : 2) attention_decode_kernel(MmaAttnParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  pdl_trigger();
  TRACE_BEGIN();
  TRACE(0);                                                  // entry
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int split = blockIdx.x * DC_WARPS + warp;
  const int c = blockIdx.y, r_id = blockIdx.z;
  const int group = p.n_heads / p.n_kv_heads;
  const int q0 = p.q_start[r_id];
  const int q_len = p.q_start[r_id + 1] - q0;
  const int ctx = p.ctx_before[r_id];
  const int n_pairs = q_len * group;
  const int* table = p.block_table + (size_t)r_id * p.table_stride;

  const int pr0 = lane >> 2, pr1 = pr0 + 8;
  const bool v0 = pr0 < n_pairs, v1 = pr1 < n_pairs;
  const int t0 = v0 ? pr0 / group : 0, t1 = v1 ? pr1 / group : 0;
  const int lim0 = v0 ? ctx + t0 : -1, lim1 = v1 ? ctx + t1 : -1;
  const int first0 = p.window > 0 ? max(0, lim0 - p.window + 1) : 0;
  const int first1 = p.window > 0 ? max(0, lim1 - p.window + 1) : 0;
  const int max_lim = ctx + q_len - 1;
  const int min_first = p.window > 0 ? max(0, ctx - p.window + 1) : 0;
  const int lo_all = (min_first / DC_KT) * DC_KT;

  // splits that hold at least one key some row can see
  const int s_first = lo_all / p.split_keys, s_last = max_lim / p.split_keys;
  const int k_lo = max(split * p.split_keys, lo_all);
  const int k_hi = min((split + 1) * p.split_keys, max_lim + 1);
  const bool has_work = split >= s_first && split <= s_last && split < p.n_splits && n_pairs > 0;
  // blocks that hold at least one such split
  const int b_first = s_first / DC_WARPS, b_last = s_last / DC_WARPS;
  const int n_active_blocks = b_last - b_first + 1;
  // A block without keys leaves at once and frees its slot.  It need not wait for the kernel ahead:
  // block 0 of every (request, kv head) always has keys and waits, so this kernel still ends after it.
  // (a request with more than 16 rows is not this kernel's: in a mixed step the prefill kernel takes it)
  if (n_pairs <= 0 || n_pairs > 16) return;                   // all blocks of this (request, kv head) alike
  // whether the blocks add up inside their cluster: the same answer in every block of the cluster, and every one
  // of them, with keys or without, then meets both cluster barriers below
  const bool merge_in_cluster = p.cluster_merge != 0 && n_active_blocks > 1;
  if ((int)blockIdx.x < b_first || (int)blockIdx.x > b_last) {
    if (merge_in_cluster) {
      cluster_barrier();
      cluster_barrier();
    }
    return;
  }

  float o[NT_O][4];
#pragma unroll
  for (int i = 0; i < NT_O; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  // Lengths, block tables and the keys of earlier steps are not written by this step's kernels:
  // tiles of old keys only are fetched before the kernel ahead has finished.
  const uint32_t base = smem_u32(smem) + warp * DC_WARP_BYTES;
  const int n_tiles = has_work ? (k_hi - k_lo + DC_KT - 1) / DC_KT : 0;
  const int n_first = min(n_tiles, DC_STAGES);
  int issued = 0;
  for (; issued < n_first && k_lo + (issued + 1) * DC_KT <= ctx; ++issued) {
    const uint32_t sb = base + issued * DC_STAGE_BYTES;
    load_kv_tile<DC_KT, 32, true>(p, table, c, k_lo + issued * DC_KT, k_hi, sb, sb + DC_KT * HD * 2, lane);
    cp_async_commit();
  }
  // what the rotation needs does not depend on the kernel ahead either (positions, tables, slots): the
  // position's cosines and sines go to shared memory before the wait
  __shared__ __align__(16) float s_cos[HD / 2], s_sin[HD / 2];
  const bool rotate = (p.fuse & 1) && p.cos_t != nullptr;
  const bool owner = has_work && (p.fuse & 2) && ctx >= k_lo && ctx < k_hi;   // this warp's keys include the step's own
  int new_slot = -1;
  if (rotate && warp == 0 && lane < HD / 4) {
    const int pos = p.positions[q0];
    *reinterpret_cast<float2*>(s_cos + lane * 2) = ld_nc_f2(p.cos_t + (size_t)pos * (HD / 2) + lane * 2);
    *reinterpret_cast<float2*>(s_sin + lane * 2) = ld_nc_f2(p.sin_t + (size_t)pos * (HD / 2) + lane * 2);
  }
  if (owner && p.slot_mapping) new_slot = IE_SLOT(p.slot_mapping[q0]);
  TRACE(1);                                                  // early tiles requested
  pdl_wait();
  __syncthreads();                                           // the tables' row is in shared memory
  TRACE(2);                                                  // the kernel ahead has finished
  NewKv new_kv;
  if (owner) load_new_kv(new_kv, p, q0, c, lane);
  if (has_work) {
    for (; issued < n_first; ++issued) {
      const uint32_t sb = base + issued * DC_STAGE_BYTES;
      load_kv_tile<DC_KT, 32, true>(p, table, c, k_lo + issued * DC_KT, k_hi, sb, sb + DC_KT * HD * 2, lane);
      cp_async_commit();
    }
    const bf16* qr0 = v0 ? p.q + (size_t)(q0 + t0) * p.q_stride + (c * group + (pr0 - t0 * group)) * HD : nullptr;
    const bf16* qr1 = v1 ? p.q + (size_t)(q0 + t1) * p.q_stride + (c * group + (pr1 - t1 * group)) * HD : nullptr;
    uint32_t qf[KSTEPS][4];
    load_q_frags(qf, qr0, qr1, lane);
    if (rotate) rotate_q_frags(qf, s_cos, s_sin, lane);
    TRACE(3);                                                  // q loaded and rotated (issued)
    for (int i = 0; i < n_tiles; ++i) {
      const int k0 = k_lo + i * DC_KT;
      cp_async_wait_pending(issued - (i + 1));
      __syncwarp();
      if (i == 0) TRACE(4);                                    // first tile has arrived
      const uint32_t sb = base + (i % DC_STAGES) * DC_STAGE_BYTES;
      if (owner && ctx >= k0 && ctx < k0 + DC_KT) {
        // the tile that holds the step's own position: what the cache had there is replaced
        insert_new_kv(p, new_kv, s_cos, s_sin, rotate, new_slot, c, ctx - k0, sb, sb + DC_KT * HD * 2, lane);
        __syncwarp();
      }
      const bool need_mask = (k0 + DC_KT - 1 > ctx) || (p.window > 0);
      if (n_pairs <= 8)
        warp_tile<DC_KT, true>(qf, o, m, l, sb, sb + DC_KT * HD * 2, k0, lim0, lim1, first0, first1, need_mask,
                               p.scale_log2, lane);
      else
        warp_tile<DC_KT, false>(qf, o, m, l, sb, sb + DC_KT * HD * 2, k0, lim0, lim1, first0, first1, need_mask,
                                p.scale_log2, lane);
      __syncwarp();
      if (issued < n_tiles) {
        load_kv_tile<DC_KT, 32, true>(p, table, c, k_lo + issued * DC_KT, k_hi, sb, sb + DC_KT * HD * 2, lane);
        cp_async_commit();
        ++issued;
      }
    }
    l[0] += __shfl_xor_sync(0xffffffffu, l[0], 1);
    l[0] += __shfl_xor_sync(0xffffffffu, l[0], 2);
    l[1] += __shfl_xor_sync(0xffffffffu, l[1], 1);
    l[1] += __shfl_xor_sync(0xffffffffu, l[1], 2);
  }

  // ---- the warps of the block: partial results into shared memory (each warp into its own tile space,
  // which it has finished reading), then every thread adds one (row, dim) up over the warps
  float* w_o = reinterpret_cast<float*>(smem + warp * DC_WARP_BYTES);     // [16][HD]
  float* w_ml = w_o + 16 * HD;                                            // [16][2]
  static_assert(DC_WARP_BYTES >= (16 * HD + 32) * 4, "a warp's tile space holds its partial result");
  {
    const int col = (lane & 3) * 2;
#pragma unroll
    for (int i = 0; i < NT_O; ++i) {
      *reinterpret_cast<float2*>(w_o + pr0 * HD + i * 8 + col) = make_float2(o[i][0], o[i][1]);
      *reinterpret_cast<float2*>(w_o + pr1 * HD + i * 8 + col) = make_float2(o[i][2], o[i][3]);
    }
    if ((lane & 3) == 0) {
      *reinterpret_cast<float2*>(w_ml + pr0 * 2) = make_float2(m[0], l[0]);   // a warp without keys: (-inf, 0)
      *reinterpret_cast<float2*>(w_ml + pr1 * 2) = make_float2(m[1], l[1]);
    }
  }
  TRACE(5);                                                  // warp 0's tiles done, partial in shared memory
  __syncthreads();
  TRACE(6);                                                  // all warps of the block done
  const int n_out = n_pairs * HD;
  const int blk = (int)blockIdx.x - b_first;
  for (int idx = threadIdx.x; idx < n_out; idx += DC_THREADS) {
    const int pr = idx / HD, d = idx - pr * HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < DC_WARPS; ++w) M = fmaxf(M, *(reinterpret_cast<const float*>(smem + w * DC_WARP_BYTES) + 16 * HD + pr * 2));
    float acc = 0.f, den = 0.f;
#pragma unroll
    for (int w = 0; w < DC_WARPS; ++w) {
      const float* wo = reinterpret_cast<const float*>(smem + w * DC_WARP_BYTES);
      const float mw = wo[16 * HD + pr * 2], lw = wo[16 * HD + pr * 2 + 1];
      const float f = (mw > -INFINITY) ? fast_exp2(mw - M) : 0.f;
      acc += f * wo[pr * HD + d];
      den += f * lw;
    }
    const int t = pr / group;
    const size_t row = (size_t)(q0 + t) * p.n_heads + c * group + (pr - t * group);
    if (n_active_blocks == 1) {
      const float inv = den > 0.f ? 1.f / den : 0.f;
      p.out[(size_t)(q0 + t) * p.out_stride + (c * group + (pr - t * group)) * HD + d] = __float2bfloat16(acc * inv);
    } else if (merge_in_cluster) {
      float* res = reinterpret_cast<float*>(smem + DC_WARPS * DC_WARP_BYTES);
      res[pr * HD + d] = acc;
      if (d == 0) *reinterpret_cast<float2*>(res + 16 * HD + pr * 2) = make_float2(M, den);
    } else {
      p.part_o[(row * p.n_blocks + blk) * HD + d] = acc;
      if (d == 0) *reinterpret_cast<float2*>(p.part_ml + (row * p.n_blocks + blk) * 2) = make_float2(M, den);
    }
  }
  TRACE(7);                                                  // block's result written (output or partial)
  if (n_active_blocks == 1) return;

  if (merge_in_cluster) {
    // ---- the cluster of this (request, kv head): its first block with keys adds the blocks up, in ascending
    // order and with the arithmetic of the ticket path below, from the others' shared memory
    cluster_barrier();
    if ((int)blockIdx.x == b_first) {
      const uint32_t res = smem_u32(smem + DC_WARPS * DC_WARP_BYTES);
      for (int idx = threadIdx.x; idx < n_out; idx += DC_THREADS) {
        const int pr = idx / HD, d = idx - pr * HD;
        const int t = pr / group;
        float2 mlv[8];
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const uint32_t peer = cluster_map(res, (uint32_t)(b_first + min(u, n_active_blocks - 1)));   // rank == blockIdx.x
          mlv[u] = ld_cluster_f32x2(peer + (16 * HD + pr * 2) * 4);
          v[u] = ld_cluster_f32(peer + (pr * HD + d) * 4);
        }
        float M = -INFINITY, acc = 0.f, den = 0.f;
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (u < n_active_blocks) M = fmaxf(M, mlv[u].x);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const bool real = u < n_active_blocks && mlv[u].x > -INFINITY;
          const float f = real ? fast_exp2(mlv[u].x - M) : 0.f;
          acc += f * v[u];
          den += f * mlv[u].y;
        }
        const float inv = den > 0.f ? 1.f / den : 0.f;
        p.out[(size_t)(q0 + t) * p.out_stride + (c * group + (pr - t * group)) * HD + d] = __float2bfloat16(acc * inv);
      }
    }
    cluster_barrier();                                         // nobody leaves while the first block still reads
    return;
  }

  // ---- ticket of this (request, kv head): the last block to arrive adds the blocks up
  __shared__ int s_ticket;
  __threadfence();
  __syncthreads();
  int* ticket = p.tickets + r_id * p.n_kv_heads + c;
  if (threadIdx.x == 0) s_ticket = atomicAdd(ticket, 1);
  __syncthreads();
  if (s_ticket != n_active_blocks - 1) return;
  __threadfence();
  if (threadIdx.x == 0) *ticket = 0;   // ready for the next launch

  // out[row] = sum_b o_b 2^(m_b - M) / sum_b l_b 2^(m_b - M), blocks in ascending order; the partials
  // come from L2 (other SMs wrote them), eight blocks' loads in flight together
  for (int idx = threadIdx.x; idx < n_out; idx += DC_THREADS) {
    const int pr = idx / HD, d = idx - pr * HD;
    const int t = pr / group;
    const size_t row = (size_t)(q0 + t) * p.n_heads + c * group + (pr - t * group);
    const float2* ml = reinterpret_cast<const float2*>(p.part_ml + row * p.n_blocks * 2);
    const float* po = p.part_o + row * p.n_blocks * HD + d;
    float M = -INFINITY;
    float acc = 0.f, den = 0.f;
    if (n_active_blocks <= 8) {
      // the usual case: everything in one round of loads, the maximum taken from what they bring
      float2 mlv[8];
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int j = min(u, n_active_blocks - 1);
        mlv[u] = __ldcg(ml + j);
        v[u] = __ldcg(po + (size_t)j * HD);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (u < n_active_blocks) M = fmaxf(M, mlv[u].x);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const bool real = u < n_active_blocks && mlv[u].x > -INFINITY;
        const float f = real ? fast_exp2(mlv[u].x - M) : 0.f;
        acc += f * v[u];
        den += f * mlv[u].y;
      }
    } else {
      for (int j = 0; j < n_active_blocks; ++j) M = fmaxf(M, __ldcg(ml + j).x);
    }
    for (int j0 = 0; j0 < n_active_blocks && n_active_blocks > 8; j0 += 8) {
      float2 mlv[8];
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int j = min(j0 + u, n_active_blocks - 1);   // the tail repeats the last block and gets weight 0
        mlv[u] = __ldcg(ml + j);
        v[u] = __ldcg(po + (size_t)j * HD);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const bool real = j0 + u < n_active_blocks && mlv[u].x > -INFINITY;
        const float f = real ? fast_exp2(mlv[u].x - M) : 0.f;
        acc += f * v[u];
        den += f * mlv[u].y;
      }
    }
    const float inv = den > 0.f ? 1.f / den : 0.f;
    p.out[(size_t)(q0 + t) * p.out_stride + (c * group + (pr - t * group)) * HD + d] = __float2bfloat16(acc * inv);
  }
}

static void fill(MmaAttnParams& p, const void* q, void* out, const void* kpool, const void* vpool,
                 const int* block_table, const int* q_start, const int* ctx_before, int q_stride, int out_stride,
                 int table_stride, int n_heads, int n_kv_heads, int page_size, int window, float scale) {
  p.q = (const bf16*)q; p.out = (bf16*)out; p.kpool = (const bf16*)kpool; p.vpool = (const bf16*)vpool;
  p.block_table = block_table; p.q_start = q_start; p.ctx_before = ctx_before;
  p.work_req = nullptr; p.work_pair0 = nullptr; p.part_o = nullptr; p.part_ml = nullptr; p.tickets = nullptr;
  p.cluster_merge = 0;
  p.q_stride = q_stride; p.out_stride = out_stride; p.table_stride = table_stride;
  p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.page_size = page_size; p.window = window;
  p.n_splits = 0; p.split_keys = 0; p.n_blocks = 0; p.scale_log2 = scale * LOG2E;
  p.fuse = 0; p.k_new = nullptr; p.v_new = nullptr; p.kv_stride = 0; p.cos_t = nullptr; p.sin_t = nullptr;
  p.positions = nullptr; p.slot_mapping = nullptr;
  p.page_shift = -1;
  if ((page_size & (page_size - 1)) == 0)
    for (int b = 0; b < 31; ++b)
      if ((1 << b) == page_size) p.page_shift = b;
}

static int check_common(const void* q, const void* out, const void* kpool, const void* vpool, int q_stride,
                        int out_stride, int n_heads, int n_kv_heads, int hd, int page_size) {
  // pool rows (page * kv_heads + head) * page_size + offset are 32-bit in the kernels: pools of up to 2^31 rows
  if (hd != HD) return IE_BAD_SIZE;
  if (n_kv_heads <= 0 || n_heads % n_kv_heads || page_size <= 0) return IE_BAD_SIZE;
  if (((uintptr_t)q | (uintptr_t)out) & 3) return IE_BAD_ALIGN;
  if (((uintptr_t)kpool | (uintptr_t)vpool) & 15) return IE_BAD_ALIGN;
  if ((q_stride | out_stride) & 1) return IE_BAD_ALIGN;
  return IE_OK;
}

}  // namespace

extern "C" int ie_attention_mma_head_dim() { return HD; }

// rows: rows of a work item's tile, 64 or 128 (the work list must have been cut accordingly)
extern "C" int ie_attention_prefill(const void* q, void* out, const void* kpool, const void* vpool,
                                    const int* block_table, const int* q_start, const int* ctx_before,
                                    const int* work_req, const int* work_pair0, int q_stride, int out_stride,
                                    int table_stride, int n_work, int n_heads, int n_kv_heads, int hd, int page_size,
                                    int window, float scale, int rows, cudaStream_t stream) {
  if (rows != 64 && rows != 128) return IE_BAD_SIZE;
  if (n_work <= 0) return IE_OK;
  int rc = check_common(q, out, kpool, vpool, q_stride, out_stride, n_heads, n_kv_heads, hd, page_size);
  if (rc) return rc;
  MmaAttnParams p;
  fill(p, q, out, kpool, vpool, block_table, q_start, ctx_before, q_stride, out_stride, table_stride, n_heads,
       n_kv_heads, page_size, window, scale);
  p.work_req = work_req;
  p.work_pair0 = work_pair0;
  const int smem = 2 * PF_STAGE_BYTES;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attention_prefill_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  if (rows == 128) return launch_k(attention_prefill_kernel<8>, dim3(n_work, n_kv_heads), 256, smem, stream, p);
  return launch_k(attention_prefill_kernel<4>, dim3(n_work, n_kv_heads), 128, smem, stream, p);
}

// Scratch needed by the decode kernel, in 4-byte words: IE_DECODE_TICKET_WORDS tickets (one per
// request and kv head) at the start, then partial outputs, then maxima and sums.  The tickets
// must be zero before the first launch on a piece of scratch; every launch leaves them zero
// again, whatever the batch, because they always sit in the same place.  The rest may hold anything.
#define IE_DECODE_TICKET_WORDS 16384
#define IE_DECODE_MAX_BLOCKS 64
extern "C" long long ie_attention_decode_scratch_floats(int n_tokens, int n_heads, int n_splits) {
  return IE_DECODE_TICKET_WORDS + (long long)n_tokens * n_heads * n_splits * (HD + 2);
}
// Warps (= splits) of a decode block; a launch takes at most IE_DECODE_MAX_BLOCKS blocks per (request, kv head).
extern "C" int ie_attention_decode_warps() { return DC_WARPS; }
extern "C" int ie_attention_decode_max_blocks() { return IE_DECODE_MAX_BLOCKS; }
// Words at the start of that scratch that must be zero before its first use.
extern "C" long long ie_attention_decode_ticket_words() { return IE_DECODE_TICKET_WORDS; }

static int decode_launch(MmaAttnParams& p, float* scratch, int n_requests, int n_tokens, int n_heads, int n_kv_heads,
                         int n_splits, int split_keys, cudaStream_t stream) {
  if (n_splits <= 0 || split_keys <= 0 || split_keys % DC_KT) return IE_BAD_SIZE;
  if ((uintptr_t)scratch & 15) return IE_BAD_ALIGN;
  p.n_splits = n_splits;
  p.split_keys = split_keys;
  if ((long long)n_requests * n_kv_heads > IE_DECODE_TICKET_WORDS) return IE_BAD_SIZE;
  p.n_blocks = (n_splits + DC_WARPS - 1) / DC_WARPS;
  if (p.n_blocks > IE_DECODE_MAX_BLOCKS) return IE_BAD_SIZE;
  p.tickets = reinterpret_cast<int*>(scratch);
  p.part_o = scratch + IE_DECODE_TICKET_WORDS;
  p.part_ml = p.part_o + (size_t)n_tokens * n_heads * p.n_blocks * HD;
  const int smem = DC_SMEM_BYTES;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  // 2 to 8 blocks per (request, kv head): one cluster along x (-DIE_DC_NO_CLUSTER=1 builds the ticket path only),
  // but only while the whole launch has a place on the SMs at once.  A cluster starts when all its blocks find room
  // in one processing cluster at the same moment, and its blocks without keys stay until the others are done; in a
  // launch of several rounds both keep places empty that single blocks would take one by one (32 requests of 128 to
  // 4,096 keys at head size 128, three blocks each: a run of 162 steps took 1.34 s with clusters, 1.21 s without).
#if defined(IE_DC_NO_CLUSTER) && IE_DC_NO_CLUSTER
  constexpr bool no_cluster = true;
#else
  constexpr bool no_cluster = false;
#endif
  static int block_places = -1;
  if (block_places < 0) {
    block_places = 0;
    int dev = 0, sms = 0, per_sm = 0;
    if (cudaGetDevice(&dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess &&
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attention_decode_kernel, DC_THREADS, smem) == cudaSuccess)
      block_places = sms * per_sm;
  }
  const long long launch_blocks = (long long)p.n_blocks * n_kv_heads * n_requests;
  p.cluster_merge = (!no_cluster && p.n_blocks >= 2 && p.n_blocks <= 8 && launch_blocks <= block_places) ? 1 : 0;
  dim3 grid(p.n_blocks, n_kv_heads, n_requests);
  return launch_k_cluster(attention_decode_kernel, p.cluster_merge ? p.n_blocks : 1, grid, DC_THREADS, smem, stream, p);
}

extern "C" int ie_attention_decode(const void* q, void* out, const void* kpool, const void* vpool,
                                   const int* block_table, const int* q_start, const int* ctx_before, float* scratch,
                                   int q_stride, int out_stride, int table_stride, int n_requests, int n_tokens,
                                   int n_heads, int n_kv_heads, int hd, int page_size, int window, float scale,
                                   int n_splits, int split_keys, cudaStream_t stream) {
  if (n_requests <= 0) return IE_OK;
  int rc = check_common(q, out, kpool, vpool, q_stride, out_stride, n_heads, n_kv_heads, hd, page_size);
  if (rc) return rc;
  // a request takes part with at most 16 (token, head-in-group) rows; larger ones are left to the prefill kernel,
  // and with more than 16 query heads a kv head no request could take part at all
  if ((n_heads / n_kv_heads) > 16) return IE_BAD_SIZE;
  MmaAttnParams p;
  fill(p, q, out, kpool, vpool, block_table, q_start, ctx_before, q_stride, out_stride, table_stride, n_heads,
       n_kv_heads, page_size, window, scale);
  return decode_launch(p, scratch, n_requests, n_tokens, n_heads, n_kv_heads, n_splits, split_keys, stream);
}

// The same for steps in which every request brings exactly one token (n_tokens == n_requests), with the
// position encoding and the cache write folded in: q, k_new and v_new are the projections as they come
// (k_new / v_new rows kv_stride apart); q and the key are rotated by the cos / sin tables ([positions, hd/2]
// float32; null: no rotation) at positions[token]; with write_kv the key and value join the step's keys
// and go to slot_mapping[token] of the pool (a negative slot: not stored), without it the cache must
// already hold them (a layer that reads another layer's cache).
extern "C" int ie_attention_decode_fused(const void* q, const void* k_new, const void* v_new, void* out, void* kpool,
                                         void* vpool, const int* block_table, const int* q_start,
                                         const int* ctx_before, float* scratch, const float* cos_t,
                                         const float* sin_t, const int* positions, const int* slot_mapping,
                                         int q_stride, int kv_stride, int out_stride, int table_stride,
                                         int n_requests, int n_heads, int n_kv_heads, int hd, int page_size,
                                         int window, float scale, int write_kv, int n_splits, int split_keys,
                                         cudaStream_t stream) {
  if (n_requests <= 0) return IE_OK;
  int rc = check_common(q, out, kpool, vpool, q_stride, out_stride, n_heads, n_kv_heads, hd, page_size);
  if (rc) return rc;
  if (!positions || (cos_t == nullptr) != (sin_t == nullptr)) return IE_BAD_SIZE;
  if (((uintptr_t)cos_t | (uintptr_t)sin_t) & 15) return IE_BAD_ALIGN;
  if (write_kv) {
    if (!k_new || !v_new) return IE_BAD_SIZE;
    if ((((uintptr_t)k_new | (uintptr_t)v_new) & 15) || (kv_stride & 7)) return IE_BAD_ALIGN;
  }
  if ((n_heads / n_kv_heads) > 16) return IE_BAD_SIZE;
  MmaAttnParams p;
  fill(p, q, out, kpool, vpool, block_table, q_start, ctx_before, q_stride, out_stride, table_stride, n_heads,
       n_kv_heads, page_size, window, scale);
  p.fuse = 1 | (write_kv ? 2 : 0);
  p.k_new = (const bf16*)k_new; p.v_new = (const bf16*)v_new; p.kv_stride = kv_stride;
  p.cos_t = cos_t; p.sin_t = sin_t; p.positions = positions; p.slot_mapping = slot_mapping;
  return decode_launch(p, scratch, n_requests, n_requests, n_heads, n_kv_heads, n_splits, split_keys, stream);
}

#ifdef IE_ATTN_TRACE
extern "C" int ie_attention_trace_read(unsigned long long* out, int max_launches) {
  unsigned int n = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&n, g_trace_n, sizeof(n)) != cudaSuccess) return -1;
  if ((int)n > max_launches) n = max_launches;
  if (n > TRACE_LAUNCHES) n = TRACE_LAUNCHES;
  if (n && cudaMemcpyFromSymbol(out, g_trace, (size_t)n * TRACE_POINTS * sizeof(unsigned long long)) != cudaSuccess) return -1;
  cudaMemcpyToSymbol(g_trace_n, &zero, sizeof(zero));
  return (int)n;
}
#endif

// ------------------------------------------------- decode without any allocation
// See attention_noalloc.h.  The scratch of the split pass is this static array;
// host code may not use its name as a pointer (on the host it is only a handle
// for the runtime), so the device address is looked up once per device.
#include "attention_noalloc.h"

static __device__ __align__(256) float g_noalloc_scratch[IE_NOALLOC_SCRATCH_FLOATS];

namespace {
constexpr int NOALLOC_MAX_DEVICES = 64;
float* g_noalloc_ptr[NOALLOC_MAX_DEVICES] = {nullptr};
}  // namespace

extern "C" long long ie_attention_decode_noalloc_capacity(void) { return (long long)IE_NOALLOC_SCRATCH_FLOATS; }

extern "C" int ie_attention_decode_noalloc(const void* q, void* out, const void* kpool, const void* vpool,
                                           const int* block_table, const int* q_start, const int* ctx_before,
                                           int q_stride, int out_stride, int table_stride, int n_requests,
                                           int n_tokens, int n_heads, int n_kv_heads, int hd, int page_size,
                                           int window, float scale, int n_splits, int split_keys,
                                           cudaStream_t stream) {
  if (n_requests <= 0) return IE_OK;
  if (n_tokens <= 0 || n_heads <= 0 || n_splits <= 0) return IE_BAD_SIZE;
  const long long need = ie_attention_decode_scratch_floats(n_tokens, n_heads, n_splits);
  if (need > (long long)IE_NOALLOC_SCRATCH_FLOATS) return IE_NOALLOC_TOO_LARGE;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return IE_BAD_SIZE;
  if (g_noalloc_ptr[dev] == nullptr) {
    // first call on this device, with it current: the array's address in device memory
    float* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    if (ptr == nullptr) return IE_BAD_ALIGN;
    g_noalloc_ptr[dev] = ptr;
  }
  return ie_attention_decode(q, out, kpool, vpool, block_table, q_start, ctx_before, g_noalloc_ptr[dev], q_stride,
                             out_stride, table_stride, n_requests, n_tokens, n_heads, n_kv_heads, hd, page_size,
                             window, scale, n_splits, split_keys, stream);
}

IE_CHECK_API(attention_mma)
