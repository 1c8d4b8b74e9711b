// Weight-streaming matrix product for few rows (decode steps): C[M,N] = A[M,K] W[N,K]^T
// with bfloat16 weights, M <= 64, on tensor cores (mma.sync m16n8k16, float32
// accumulators), with the work that surrounds a projection fused in:
//
//   prologue  PLAIN  A is bfloat16 [M, K]
//             NORM   A is the float32 residual stream (rows optionally gathered);
//                    the kernel multiplies by the RMSNorm gain on the way in,
//                    sums the squares in float32 beside the product, and scales
//                    the result by 1/sqrt(mean(x^2)+eps) on the way out, which is
//                    (x/rms*g) W^T of engine/layers.py:24-25 and :48-50 reordered
//   epilogue  STORE_BF16 / STORE_F32
//             RESIDUAL   residual[M,N] += product in float32 (engine/llama_block.py:54,62)
//             SILU_MUL   weight rows alternate gate_j, up_j; out[M, N/2] =
//                        silu(gate_j) * up_j in float32 (engine/llama_mlp.py:30-32)
//
// At these sizes the product is bound by reading W once from HBM.  Every lane
// loads 16 bytes of a weight row straight from global memory into the B
// fragment of two MMAs (the k order inside a 32-wide chunk is permuted the same
// way for A and W, which a dot product allows), so weights never pass through
// shared memory; eight warps of a block split K and are summed in a fixed order.
#include "common.cuh"

namespace {

enum { PRO_PLAIN = 0, PRO_NORM = 1 };
enum { EPI_BF16 = 0, EPI_F32 = 1, EPI_RESIDUAL = 2, EPI_SILU_MUL = 3 };

constexpr int GS_WARPS = 8;
constexpr int GS_THREADS = GS_WARPS * 32;

struct StreamParams {
  const void* A;          // bf16 [M, lda] or float32 residual [*, lda]
  const bf16* W;          // [N, ldw]
  void* C;                // bf16 / float32 [M, ldc]; residual for EPI_RESIDUAL
  const void* gain;       // NORM: [K], bf16 or float32
  const int* row_index;   // NORM: optional gather of residual rows
  int M, N, K, lda, ldw, ldc;
  int gain_is_f32;
  float eps;
};

// Weights are read once a step and are far larger than L2: "evict first" keeps the stream from pushing out
// what the step reads again and again (activations, norm gains, the kernels' own code).
__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p), "l"(pol));
  return v;
}
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// eight consecutive activations of one row as four packed bfloat16 pairs
template <int PRO>
__device__ __forceinline__ uint4 load_a8(const StreamParams& p, int m, int k, bool valid, float& ssq) {
  uint4 out = make_uint4(0u, 0u, 0u, 0u);
  if (PRO == PRO_PLAIN) {
    // an invalid lane reads element 0 of the buffer (always there) and discards it: no branch around the load
    const uint4 v = *reinterpret_cast<const uint4*>((const bf16*)p.A + (valid ? (size_t)m * p.lda + k : 0));
    return valid ? v : out;
  } else {
    if (!valid) return out;
    const int row = p.row_index ? p.row_index[m] : m;
    const float* x = (const float*)p.A + (size_t)row * p.lda + k;
    const float4 x0 = *reinterpret_cast<const float4*>(x), x1 = *reinterpret_cast<const float4*>(x + 4);
    float g[8];
    if (p.gain_is_f32) {
      const float4 g0 = *reinterpret_cast<const float4*>((const float*)p.gain + k);
      const float4 g1 = *reinterpret_cast<const float4*>((const float*)p.gain + k + 4);
      g[0] = g0.x; g[1] = g0.y; g[2] = g0.z; g[3] = g0.w; g[4] = g1.x; g[5] = g1.y; g[6] = g1.z; g[7] = g1.w;
    } else {
      const uint4 gv = *reinterpret_cast<const uint4*>((const bf16*)p.gain + k);
      const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&gv);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(gp[i]);
        g[2 * i] = f.x;
        g[2 * i + 1] = f.y;
      }
    }
    ssq += x0.x * x0.x + x0.y * x0.y + x0.z * x0.z + x0.w * x0.w + x1.x * x1.x + x1.y * x1.y + x1.z * x1.z + x1.w * x1.w;
    out.x = pack2(x0.x * g[0], x0.y * g[1]);
    out.y = pack2(x0.z * g[2], x0.w * g[3]);
    out.z = pack2(x1.x * g[4], x1.y * g[5]);
    out.w = pack2(x1.z * g[6], x1.w * g[7]);
    return out;
  }
}

template <int MB, int NT, int PRO, int EPI>
__global__ void __launch_bounds__(GS_THREADS) gemm_stream_kernel(StreamParams p) {
  __shared__ float red[GS_WARPS][MB * NT * 4][32];
  __shared__ float red_ssq[GS_WARPS][MB * 2][8];
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int n_base = blockIdx.x * (8 * NT);
  const int n_chunks = (p.K + 31) >> 5;
  const int c_lo = (int)((long long)n_chunks * warp / GS_WARPS), c_hi = (int)((long long)n_chunks * (warp + 1) / GS_WARPS);

  float acc[MB][NT][4];
  float ssq[MB][2];
#pragma unroll
  for (int mb = 0; mb < MB; ++mb) {
    ssq[mb][0] = ssq[mb][1] = 0.f;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[mb][nt][0] = acc[mb][nt][1] = acc[mb][nt][2] = acc[mb][nt][3] = 0.f;
  }
  const bf16* wrow[NT];
  bool wvalid[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int n = n_base + nt * 8 + g;
    wvalid[nt] = n < p.N;
    wrow[nt] = p.W + (size_t)(wvalid[nt] ? n : 0) * p.ldw;
  }

  // Weights do not depend on the kernel ahead: the first PREF chunks of every lane are on
  // their way before this kernel waits for its activations.  The buffer then rolls: each
  // chunk that is consumed is replaced by the chunk PREF further on, which keeps PREF
  // 16-byte loads per weight row in flight per lane.
  constexpr int PREF = NT == 4 ? 4 : 8;
  uint4 wbuf[PREF][NT];
#pragma unroll
  for (int j = 0; j < PREF; ++j) {
    const int c = c_lo + j;
    const int k = (c << 5) + t * 8;
    const bool ok = c < c_hi && k < p.K;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
      wbuf[j][nt] = (ok && wvalid[nt]) ? ldg_stream(wrow[nt] + k) : make_uint4(0u, 0u, 0u, 0u);
  }
  pdl_wait();

  // Activations of XG chunks are loaded together, without a branch between them, so that
  // their latencies overlap instead of adding up; then the MMAs of those chunks run and
  // the weight buffer is refilled for the chunks PREF further on.
  constexpr int XG = MB == 1 ? PREF : (MB == 2 ? 4 : 2);
  for (int base = c_lo; base < c_hi; base += PREF) {
#pragma unroll
    for (int j0 = 0; j0 < PREF; j0 += XG) {
      uint4 xa[XG][MB][2];
#pragma unroll
      for (int jj = 0; jj < XG; ++jj) {
        const int c = base + j0 + jj;
        const int k = (c << 5) + t * 8;
        const bool kvalid = c < c_hi && k < p.K;
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
          const int m0 = mb * 16 + g, m1 = m0 + 8;
          xa[jj][mb][0] = load_a8<PRO>(p, m0, k, kvalid && m0 < p.M, ssq[mb][0]);
          xa[jj][mb][1] = load_a8<PRO>(p, m1, k, kvalid && m1 < p.M, ssq[mb][1]);
        }
      }
#pragma unroll
      for (int jj = 0; jj < XG; ++jj) {
        const int j = j0 + jj;
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
          const uint4 x0 = xa[jj][mb][0], x1 = xa[jj][mb][1];
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            mma16816(acc[mb][nt], x0.x, x1.x, x0.y, x1.y, wbuf[j][nt].x, wbuf[j][nt].y);
            mma16816(acc[mb][nt], x0.z, x1.z, x0.w, x1.w, wbuf[j][nt].z, wbuf[j][nt].w);
          }
        }
        const int c2 = base + j + PREF;
        const int k2 = (c2 << 5) + t * 8;
        const bool ok = c2 < c_hi && k2 < p.K;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
          wbuf[j][nt] = (ok && wvalid[nt]) ? ldg_stream(wrow[nt] + k2) : make_uint4(0u, 0u, 0u, 0u);
      }
    }
  }

  // the warps' partial sums, added in warp order
#pragma unroll
  for (int mb = 0; mb < MB; ++mb)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) red[warp][(mb * NT + nt) * 4 + e][lane] = acc[mb][nt][e];
  if (PRO == PRO_NORM) {
#pragma unroll
    for (int mb = 0; mb < MB; ++mb)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float s = ssq[mb][h];
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        if (t == 0) red_ssq[warp][mb * 2 + h][g] = s;
      }
  }
  __syncthreads();

  // one (mb, nt, half, lane) per thread-iteration: two neighbouring outputs of one row
  for (int j = threadIdx.x; j < MB * NT * 2 * 32; j += GS_THREADS) {
    const int ln = j & 31, h = (j >> 5) & 1, tile = j >> 6;   // tile = mb*NT + nt
    const int mb = tile / NT, nt = tile - mb * NT;
    const int gg = ln >> 2, tt = ln & 3;
    const int m = mb * 16 + gg + h * 8;
    const int n = n_base + nt * 8 + tt * 2;
    if (m >= p.M || n >= p.N) continue;
    float v0 = 0.f, v1 = 0.f;
#pragma unroll
    for (int w8 = 0; w8 < GS_WARPS; ++w8) {
      v0 += red[w8][tile * 4 + h * 2][ln];
      v1 += red[w8][tile * 4 + h * 2 + 1][ln];
    }
    if (PRO == PRO_NORM) {
      float s = 0.f;
#pragma unroll
      for (int w8 = 0; w8 < GS_WARPS; ++w8) s += red_ssq[w8][mb * 2 + h][gg];
      const float inv = 1.f / sqrtf(s / (float)p.K + p.eps);
      v0 *= inv;
      v1 *= inv;
    }
    const bool has1 = n + 1 < p.N;
    if (EPI == EPI_BF16) {
      bf16* c = (bf16*)p.C + (size_t)m * p.ldc + n;
      if (has1 && ((((uintptr_t)c) & 3) == 0)) *reinterpret_cast<uint32_t*>(c) = pack2(v0, v1);
      else { c[0] = __float2bfloat16_rn(v0); if (has1) c[1] = __float2bfloat16_rn(v1); }
    } else if (EPI == EPI_F32) {
      float* c = (float*)p.C + (size_t)m * p.ldc + n;
      c[0] = v0;
      if (has1) c[1] = v1;
    } else if (EPI == EPI_RESIDUAL) {
      float* c = (float*)p.C + (size_t)m * p.ldc + n;
      c[0] += v0;
      if (has1) c[1] += v1;
    } else {  // EPI_SILU_MUL: v0 = gate_j, v1 = up_j, j = n / 2
      const float sg = 1.f / (1.f + expf(-v0));
      ((bf16*)p.C)[(size_t)m * p.ldc + (n >> 1)] = __float2bfloat16_rn((v0 * sg) * v1);
    }
  }
}

template <int MB, int NT, int PRO, int EPI>
int launch(const StreamParams& p, cudaStream_t stream) {
  const int grid = (p.N + 8 * NT - 1) / (8 * NT);
  return launch_k(gemm_stream_kernel<MB, NT, PRO, EPI>, grid, GS_THREADS, 0, stream, p);
}

template <int PRO, int EPI>
int dispatch(const StreamParams& p, int nt, cudaStream_t stream) {
  const int mb = (p.M + 15) / 16;
  if (mb == 1) {
    if (nt == 1) return launch<1, 1, PRO, EPI>(p, stream);
    if (nt == 2) return launch<1, 2, PRO, EPI>(p, stream);
    return launch<1, 4, PRO, EPI>(p, stream);
  }
  if (mb == 2) {
    if (nt == 1) return launch<2, 1, PRO, EPI>(p, stream);
    if (nt == 2) return launch<2, 2, PRO, EPI>(p, stream);
    return launch<2, 4, PRO, EPI>(p, stream);
  }
  if (mb <= 4) {
    if (nt == 1) return launch<4, 1, PRO, EPI>(p, stream);
    return launch<4, 2, PRO, EPI>(p, stream);
  }
  return IE_BAD_SIZE;
}

}  // namespace

// pro: 0 plain bf16 A, 1 float32 residual with fused RMSNorm (gain, eps, optional row_index)
// epi: 0 bf16 out, 1 float32 out, 2 residual +=, 3 silu(gate)*up over interleaved weight rows
// nt:  8*nt weight rows per block (1, 2 or 4)
extern "C" int ie_gemm_stream(const void* A, const void* W, void* C, const void* gain, int gain_dtype,
                              const int* row_index, int M, int N, int K, int lda, int ldw, int ldc, float eps,
                              int pro, int epi, int nt, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return IE_OK;
  if (M > 64 || K <= 0 || (K & 7) || (lda & 7) || (ldw & 7)) return IE_BAD_SIZE;
  if (((uintptr_t)A | (uintptr_t)W) & 15) return IE_BAD_ALIGN;
  if (nt != 1 && nt != 2 && nt != 4) return IE_BAD_SIZE;
  if (epi == EPI_SILU_MUL && (N & 1)) return IE_BAD_SIZE;
  StreamParams p;
  p.A = A; p.W = (const bf16*)W; p.C = C; p.gain = gain; p.row_index = row_index;
  p.M = M; p.N = N; p.K = K; p.lda = lda; p.ldw = ldw; p.ldc = ldc;
  p.gain_is_f32 = gain_dtype == IE_F32; p.eps = eps;
  if (pro == PRO_NORM) {
    if (!gain || ((uintptr_t)gain & 15)) return IE_BAD_ALIGN;
    if (epi == EPI_BF16) return dispatch<PRO_NORM, EPI_BF16>(p, nt, stream);
    if (epi == EPI_F32) return dispatch<PRO_NORM, EPI_F32>(p, nt, stream);
    if (epi == EPI_SILU_MUL) return dispatch<PRO_NORM, EPI_SILU_MUL>(p, nt, stream);
    return IE_BAD_DTYPE;
  }
  if (pro == PRO_PLAIN) {
    if (epi == EPI_BF16) return dispatch<PRO_PLAIN, EPI_BF16>(p, nt, stream);
    if (epi == EPI_F32) return dispatch<PRO_PLAIN, EPI_F32>(p, nt, stream);
    if (epi == EPI_RESIDUAL) return dispatch<PRO_PLAIN, EPI_RESIDUAL>(p, nt, stream);
    if (epi == EPI_SILU_MUL) return dispatch<PRO_PLAIN, EPI_SILU_MUL>(p, nt, stream);
    return IE_BAD_DTYPE;
  }
  return IE_BAD_DTYPE;
}
