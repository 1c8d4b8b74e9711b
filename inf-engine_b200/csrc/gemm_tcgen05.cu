// C[M,N] = A[M,K] W[N,K]^T for many rows (prompt portions) on the fifth-generation tensor cores of
// sm_100a: bfloat16 operands staged in shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle),
// tcgen05.mma issued by one thread with the float32 accumulator in tensor memory, read back with
// tcgen05.ld for a fused epilogue:
//   STORE_BF16   C bf16
//   SILU_MUL     weight rows alternate gate_j, up_j; C[M, N/2] = silu(gate_j) * up_j   (engine/llama_mlp.py:30-32)
//   RESIDUAL     C float32 [M, N] += product                                            (engine/llama_block.py:54,62)
// The plain product is what the reference leaves to a library; the fused epilogues save the round trip of
// the [M, 2*intermediate] gate/up matrix and of the projections' outputs through HBM.
//
// One block per SM walks over 128 x BN tiles.  Warp 0 is the TMA producer, warp 1 allocates tensor memory and
// issues the MMAs, warps 2-5 are the epilogue (warp w reads the 32 TMEM lanes of quarter w % 4).  A ring
// of shared-memory stages is handed over with mbarriers: the producer waits for "empty", arms "full" with
// the byte count and issues two tensor copies; the MMA thread waits for "full", issues four MMAs of K = 16
// and lets tcgen05.commit arrive on "empty" when they have read the stage.  Every wait is bounded: on a
// timeout the block records an error word, stops, frees its tensor memory and leaves.
#include "common.cuh"
#include <cuda.h>

namespace {

enum { TC_EPI_BF16 = 0, TC_EPI_SILU_MUL = 3, TC_EPI_RESIDUAL = 2 };

constexpr int BM = 128;
constexpr int BK = 64;               // one 128-byte swizzle atom of bfloat16
constexpr int UMMA_K = 16;
constexpr int TC_THREADS = 192;
constexpr unsigned TC_SPIN_LIMIT = 1u << 20;

__device__ int g_tc_error = 0;

// silu(g) = g / (1 + e^-g) in float32 with ex2.approx and the approximate division: a relative error near 1e-6,
// where the bfloat16 result keeps 4e-3; the precise forms cost the gate/up product 6 % of its time
__device__ __forceinline__ float tc_silu(float g) { return __fdividef(g, 1.f + __expf(-g)); }

struct TcParams {
  void* C;
  int M, N, K, ldc;
  int epi;
  int n_stages;
  int staged;   // the output's base and row pitch are multiples of 16 bytes: full tiles leave through shared memory
};

__device__ __forceinline__ uint32_t saddr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void tc_mbar_init(uint32_t bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void tc_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool tc_mbar_wait(uint32_t bar, uint32_t parity) {
  for (unsigned i = 0; i < TC_SPIN_LIMIT; ++i) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
  }
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar) : "memory");
}
// shared-memory matrix descriptor: K-major tile of rows of 128 bytes, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_byte_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_byte_addr & 0x3FFFF) >> 4);        // start address
  d |= (uint64_t)0 << 16;                                   // leading byte offset: unused for swizzled K-major
  d |= (uint64_t)(1024 >> 4) << 32;                         // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                                   // descriptor version of sm_100
  d |= (uint64_t)2 << 61;                                   // SWIZZLE_128B
  return d;
}
// instruction descriptor: D float32, A and B bfloat16, both K-major, M x N
__device__ __forceinline__ uint32_t umma_idesc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
               ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}

// one row's 32 accumulator columns n .. n+31 through the epilogue p.epi
__device__ __forceinline__ void tc_epilogue_store(const TcParams& p, int m, int n, const uint32_t (&r)[32]) {
  if (m < p.M && n < p.N) {
    if (p.epi == TC_EPI_BF16) {
      bf16* dst = (bf16*)p.C + (size_t)m * p.ldc + n;
      if (n + 32 <= p.N && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 v;
          __nv_bfloat162* vp = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
          for (int q = 0; q < 4; ++q)
            vp[q] = __floats2bfloat162_rn(__uint_as_float(r[j * 8 + 2 * q]), __uint_as_float(r[j * 8 + 2 * q + 1]));
          *reinterpret_cast<uint4*>(dst + j * 8) = v;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (n + j < p.N) dst[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
      }
    } else if (p.epi == TC_EPI_SILU_MUL) {
      bf16* dst = (bf16*)p.C + (size_t)m * p.ldc + (n >> 1);
      if (n + 32 <= p.N && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          uint4 v;
          __nv_bfloat162* vp = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float g0 = __uint_as_float(r[j * 16 + 4 * q]), u0 = __uint_as_float(r[j * 16 + 4 * q + 1]);
            const float g1 = __uint_as_float(r[j * 16 + 4 * q + 2]), u1 = __uint_as_float(r[j * 16 + 4 * q + 3]);
            vp[q] = __floats2bfloat162_rn(tc_silu(g0) * u0, tc_silu(g1) * u1);
          }
          *reinterpret_cast<uint4*>(dst + j * 8) = v;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          if (n + j + 1 < p.N) {
            const float g = __uint_as_float(r[j]), u = __uint_as_float(r[j + 1]);
            dst[j >> 1] = __float2bfloat16_rn(tc_silu(g) * u);
          }
        }
      }
    } else {
      float* dst = (float*)p.C + (size_t)m * p.ldc + n;
      if (n + 32 <= p.N && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float4 v = *reinterpret_cast<float4*>(dst + j * 4);
          v.x += __uint_as_float(r[j * 4]);
          v.y += __uint_as_float(r[j * 4 + 1]);
          v.z += __uint_as_float(r[j * 4 + 2]);
          v.w += __uint_as_float(r[j * 4 + 3]);
          *reinterpret_cast<float4*>(dst + j * 4) = v;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (n + j < p.N) dst[j] += __uint_as_float(r[j]);
      }
    }
  }
}

// ---- full tiles leave through shared memory: a thread holds one ROW of the accumulator, so stores straight from
// registers put 16 bytes into each of 32 different rows per instruction (half-filled sectors, 15 % of the gate/up
// product's time).  Instead each epilogue warp collects 128 bytes of output per row in a tile of its own (32 rows,
// 16-byte units swizzled by row so that neither side has bank conflicts) and writes it out as whole 128-byte lines.
constexpr int TC_STAGE_BYTES = 32 * 128;      // per epilogue warp

// bytes of output that 32 accumulator columns make
__device__ __forceinline__ int tc_out_bytes32(int epi) { return epi == TC_EPI_BF16 ? 64 : (epi == TC_EPI_SILU_MUL ? 32 : 128); }

// this lane's 32 accumulator columns -> its row of the warp's tile, from byte offset off
__device__ __forceinline__ void tc_stage_row(unsigned char* stage, int lane, int off, int epi, const uint32_t (&r)[32]) {
  unsigned char* row = stage + lane * 128;
  const int u0 = off >> 4, sw = lane & 7;
  if (epi == TC_EPI_BF16) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint4 v;
      __nv_bfloat162* vp = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
      for (int q = 0; q < 4; ++q)
        vp[q] = __floats2bfloat162_rn(__uint_as_float(r[j * 8 + 2 * q]), __uint_as_float(r[j * 8 + 2 * q + 1]));
      *reinterpret_cast<uint4*>(row + (((u0 + j) ^ sw) << 4)) = v;
    }
  } else if (epi == TC_EPI_SILU_MUL) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      uint4 v;
      __nv_bfloat162* vp = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float g0 = __uint_as_float(r[j * 16 + 4 * q]), u0f = __uint_as_float(r[j * 16 + 4 * q + 1]);
        const float g1 = __uint_as_float(r[j * 16 + 4 * q + 2]), u1f = __uint_as_float(r[j * 16 + 4 * q + 3]);
        vp[q] = __floats2bfloat162_rn(tc_silu(g0) * u0f, tc_silu(g1) * u1f);
      }
      *reinterpret_cast<uint4*>(row + (((u0 + j) ^ sw) << 4)) = v;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j)
      *reinterpret_cast<uint4*>(row + (((u0 + j) ^ sw) << 4)) = make_uint4(r[j * 4], r[j * 4 + 1], r[j * 4 + 2], r[j * 4 + 3]);
  }
}

// the warp's tile (rows row0 .. row0 + 31, 128 bytes from byte col_byte0 of each output row) to memory, four rows
// per instruction; the residual epilogue adds into what is there
__device__ __forceinline__ void tc_flush(const TcParams& p, const unsigned char* stage, int lane, int row0, size_t col_byte0) {
  const size_t pitch = (size_t)p.ldc * (p.epi == TC_EPI_RESIDUAL ? 4 : 2);
  const int u = lane & 7;
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int r = it * 4 + (lane >> 3), row = row0 + r;
    const uint4 v = *reinterpret_cast<const uint4*>(stage + r * 128 + ((u ^ (r & 7)) << 4));
    if (row < p.M) {
      unsigned char* dst = (unsigned char*)p.C + (size_t)row * pitch + col_byte0 + (u << 4);
      if (p.epi == TC_EPI_RESIDUAL) {
        float4 g = *reinterpret_cast<float4*>(dst);
        g.x += __uint_as_float(v.x);
        g.y += __uint_as_float(v.y);
        g.z += __uint_as_float(v.z);
        g.w += __uint_as_float(v.w);
        *reinterpret_cast<float4*>(dst) = g;
      } else {
        *reinterpret_cast<uint4*>(dst) = v;
      }
    }
  }
}

template <int BN>
__global__ void __launch_bounds__(TC_THREADS, 1) gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                     const __grid_constant__ CUtensorMap map_w,
                                                                     TcParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // full[8], empty[8]: the shared-memory ring; acc_full[2], acc_empty[2]: the two accumulators in tensor memory
  __shared__ __align__(8) unsigned long long bars[2 * 8 + 4];
  __shared__ uint32_t tmem_base_slot;
  __shared__ volatile int failed;
  constexpr uint32_t A_BYTES = BM * BK * 2, W_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + W_BYTES;

  pdl_trigger();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t ring = (saddr(smem_raw) + 1023u) & ~1023u;   // swizzle atoms are 1024 bytes
  const uint32_t full0 = saddr(&bars[0]), empty0 = saddr(&bars[8]);
  const uint32_t acc_full0 = saddr(&bars[16]), acc_empty0 = saddr(&bars[18]);
  const int k_blocks = p.K / BK;
  const int m_tiles = (p.M + BM - 1) / BM, n_tiles = (p.N + BN - 1) / BN;
  const int total_tiles = m_tiles * n_tiles;   // tile t: rows (t % m_tiles), columns (t / m_tiles): blocks that run
                                               // side by side share a weight tile, which then comes from HBM once

  if (tid == 0) {
    failed = 0;
    for (int s = 0; s < p.n_stages; ++s) {
      tc_mbar_init(full0 + 8 * s, 1);
      tc_mbar_init(empty0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      tc_mbar_init(acc_full0 + 8 * b, 1);
      tc_mbar_init(acc_empty0 + 8 * b, 4);     // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    // tensor memory for two accumulators of BN columns x 128 lanes: the epilogue of one tile runs while
    // the MMAs of the next fill the other
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(saddr(&tmem_base_slot)), "n"(2 * BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_slot;

  pdl_wait();   // the activations come from the kernel ahead

  if (warp == 0) {
    if (lane == 0) {
      int s = 0;
      uint32_t phase = 0;
      for (int t = blockIdx.x; t < total_tiles && !failed; t += gridDim.x) {
        const int m0 = (t % m_tiles) * BM, n0 = (t / m_tiles) * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (failed || !tc_mbar_wait(empty0 + 8 * s, phase ^ 1)) { atomicExch(&g_tc_error, 1); failed = 1; break; }
          const uint32_t bar = full0 + 8 * s;
          tc_mbar_expect_tx(bar, STAGE_BYTES);
          const uint32_t a_dst = ring + s * STAGE_BYTES, w_dst = a_dst + A_BYTES;
          tma_load_2d(a_dst, &map_a, kb * BK, m0, bar);
          tma_load_2d(w_dst, &map_w, kb * BK, n0, bar);
          if (++s == p.n_stages) { s = 0; phase ^= 1; }
        }
      }
      if (failed) for (int i = 0; i < 2048; ++i) __nanosleep(64);   // copies already issued still land in this block's memory
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(BM, BN);
      int s = 0;
      uint32_t phase = 0;
      int it = 0;
      for (int t = blockIdx.x; t < total_tiles && !failed; t += gridDim.x, ++it) {
        const int buf = it & 1;
        const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
        // the epilogue has drained this accumulator (immediately true the first time round)
        if (!tc_mbar_wait(acc_empty0 + 8 * buf, acc_phase ^ 1)) { atomicExch(&g_tc_error, 4); failed = 1; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (failed || !tc_mbar_wait(full0 + 8 * s, phase)) { atomicExch(&g_tc_error, 2); failed = 1; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_src = ring + s * STAGE_BYTES, w_src = a_src + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t ad = umma_desc(a_src + k * UMMA_K * 2), wd = umma_desc(w_src + k * UMMA_K * 2);
            umma_f16(d_tmem, ad, wd, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(empty0 + 8 * s);          // arrives when these MMAs have read the stage
          if (++s == p.n_stages) { s = 0; phase ^= 1; }
        }
        if (failed) break;
        umma_commit(acc_full0 + 8 * buf);       // arrives when the whole accumulator is final
      }
    }
  } else {
    // ----------------------------------------------------------- epilogue
    const int quarter = warp & 3;              // TMEM lanes 32*quarter .. +31 belong to this warp
    unsigned char* stage = smem_raw + (ring - saddr(smem_raw)) + (size_t)p.n_stages * STAGE_BYTES + (warp - 2) * TC_STAGE_BYTES;
    const int out32 = tc_out_bytes32(p.epi);
    int it = 0;
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++it) {
      const int buf = it & 1;
      const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
      const int m0 = (t % m_tiles) * BM, n0 = (t / m_tiles) * BN;
      const int m = m0 + quarter * 32 + lane;
      bool ok = !failed && tc_mbar_wait(acc_full0 + 8 * buf, acc_phase);
      if (!ok && lane == 0) { atomicExch(&g_tc_error, 3); failed = 1; }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0 && !failed;
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const bool staged = p.staged && n0 + BN <= p.N;     // full width: whole lines through shared memory
      int off = 0;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + c0), r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (c0 + 32 >= BN) {
          // everything of this accumulator is in registers: the MMA thread may reuse it
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty0 + 8 * buf) : "memory");
        }
        if (staged) {
          tc_stage_row(stage, lane, off, p.epi, r);
          off += out32;
          if (off == 128) {
            __syncwarp();
            tc_flush(p, stage, lane, m - lane, (size_t)(n0 + c0 + 32) * (out32 >> 5) - 128);
            __syncwarp();
            off = 0;
          }
        } else {
          tc_epilogue_store(p, m, n0 + c0, r);
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(2 * BN) : "memory");
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)ptr;
  }
  return fn;
}

// a [rows, cols] bfloat16 matrix with row pitch ld (elements): boxes of box_rows x 64 columns, 128-byte swizzle
static int make_map(CUtensorMap* map, const void* base, int rows, int cols, int ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return IE_BAD_SIZE;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? IE_OK : IE_BAD_ALIGN;
}

template <int BN>
static int launch_tc(const CUtensorMap& ma, const CUtensorMap& mw, TcParams p, int n_sms, cudaStream_t stream) {
  const uint32_t stage = (BM + BN) * BK * 2;
  int n_stages = (200 * 1024 - 1024) / stage;
  if (n_stages > 8) n_stages = 8;
  p.n_stages = n_stages;
  const size_t smem = (size_t)n_stages * stage + 1024 + 4 * TC_STAGE_BYTES;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    attr = true;
  }
  const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
  const int grid = tiles < n_sms ? tiles : n_sms;
  return launch_k(gemm_tcgen05_kernel<BN>, grid, TC_THREADS, smem, stream, ma, mw, p);
}

}  // namespace

extern "C" int ie_gemm_tcgen05_error() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_tc_error, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_tc_error, &zero, sizeof(int));
  return v;
}

// 1 if the kernel takes the product: bfloat16, K a multiple of 64, row pitches multiples of 8 elements
extern "C" int ie_gemm_tcgen05_supports(int M, int N, int K, int lda, int ldw) {
  return (M > 0 && N > 0 && K > 0 && K % BK == 0 && lda % 8 == 0 && ldw % 8 == 0) ? 1 : 0;
}

// epi: 0 bf16 out [M,N]; 2 float32 C[M,N] += product; 3 silu(gate)*up over interleaved weight rows, bf16 out [M, N/2]
// bn:  tile width, 128 or 256
extern "C" int ie_gemm_tcgen05(const void* A, const void* W, void* C, int M, int N, int K, int lda, int ldw, int ldc,
                               int epi, int bn, int n_sms, cudaStream_t stream) {
  if (n_sms <= 0) return IE_BAD_SIZE;
  if (M <= 0 || N <= 0) return IE_OK;
  if (!ie_gemm_tcgen05_supports(M, N, K, lda, ldw)) return IE_BAD_SIZE;
  if (((uintptr_t)A | (uintptr_t)W) & 15) return IE_BAD_ALIGN;
  if (epi != TC_EPI_BF16 && epi != TC_EPI_SILU_MUL && epi != TC_EPI_RESIDUAL) return IE_BAD_DTYPE;
  if (epi == TC_EPI_SILU_MUL && (N & 1)) return IE_BAD_SIZE;
  if (bn != 128 && bn != 256) return IE_BAD_SIZE;
  CUtensorMap ma, mw;
  int rc = make_map(&ma, A, M, K, lda, BM);
  if (rc) return rc;
  rc = make_map(&mw, W, N, K, ldw, bn);
  if (rc) return rc;
  TcParams p;
  p.C = C; p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.epi = epi; p.n_stages = 0;
  p.staged = (((uintptr_t)C & 15) == 0 && ((size_t)ldc * (epi == TC_EPI_RESIDUAL ? 4 : 2)) % 16 == 0) ? 1 : 0;
  return bn == 256 ? launch_tc<256>(ma, mw, p, n_sms, stream) : launch_tc<128>(ma, mw, p, n_sms, stream);
}
