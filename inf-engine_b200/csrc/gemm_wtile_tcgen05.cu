// C[M,N] = X[M,K] W[N,K]^T for decode steps of 17 to 128 requests on the fifth-generation tensor cores of
// sm_100a, reading W once at HBM speed.
//
// With that few rows the product is a read of W, as with 16 rows and fewer (gemm_stream_tma.cu), but the
// arithmetic no longer fits the legacy MMA path beside the stream.  So the product is turned round: 128 weight
// rows are the M of a tcgen05.mma (the lanes of the accumulator in tensor memory), the step's tokens are its N
// (32, 64 or 128 columns).  Each block streams whole weight tiles and multiplies them by the activations, which
// are small and come from L2.
//
// W is stored tile by tile for this kernel (ie_wtile_pack, once at load): tile (n, k) holds rows 128 n .. 128 n +
// 127 and columns 64 k .. 64 k + 63 as the 16 KB image that the MMA reads from shared memory (rows of 128 bytes,
// the 16-byte units of a row XOR-swizzled by row % 8), so a stage of the ring is ONE bulk copy of 16 KB
// (cp.async.bulk, L2 evict-first).  A tiled tensor copy of a row-major W moves rows of 128 bytes, and an SM could
// not issue those fast enough to keep HBM busy at these row counts.  The activations' tile of a stage (tokens x 64
// columns, 4 to 16 KB) is a tensor copy (cp.async.bulk.tensor.2d, 128-byte swizzle, rows past M filled with zeros).
//
// Few weight rows (the projections back into the hidden width have 16 tiles of 128) do not fill 148 SMs, so K is
// split over the blocks of a thread-block cluster (1, 2, 4 or 8): each block multiplies its share of K for the same
// weight rows, writes its partial sums to its own shared memory, and block r of the cluster adds up, in block
// order, the sums of a share of the tokens, reading the others' shared memory (ld.shared::cluster).  Hand-over
// between the blocks is by mbarriers with cluster-scope release/acquire; a cluster barrier at the very end keeps
// every block's shared memory alive until nobody reads it any more.
//
//   warp 0      producer: weight tile (bulk copy) + activation tile (tensor copy) per stage; the weight copies of
//               the first stages are issued BEFORE the wait for the kernel ahead (programmatic dependent launch)
//   warp 1      allocates tensor memory (two accumulators), issues four MMAs of K = 16 per stage
//   warps 2-5   epilogue: thread = weight row; tcgen05.ld of 32 token columns at a time; split-K exchange;
//               bf16 / float32 store, or silu(gate) * up over interleaved weight rows (engine/llama_mlp.py:30-32)
//
// Every wait on an mbarrier is bounded; on a timeout the block records an error word, stops issuing work, still
// meets the cluster's last barrier, frees its tensor memory and leaves.
#include "common.cuh"
#include <cuda.h>

namespace {

enum { WT_EPI_BF16 = 0, WT_EPI_F32 = 1, WT_EPI_SILU_MUL = 3 };

constexpr int WT_BM = 128;                     // weight rows of a tile = lanes of the accumulator
constexpr int WT_BK = 64;                      // one 128-byte swizzle atom of bfloat16
constexpr int WT_UMMA_K = 16;
constexpr int WT_THREADS = 192;
constexpr uint32_t WT_TILE_BYTES = WT_BM * WT_BK * 2;   // 16 KB
constexpr int WT_MAX_STAGES = 10;
constexpr unsigned WT_SPIN_LIMIT = 1u << 20;

__device__ int g_wt_error = 0;

struct WtParams {
  const unsigned char* Wt;   // [n_tiles][k_blocks][WT_TILE_BYTES]
  void* C;                   // [M, ldc] bf16 or float32; SILU_MUL: [M, ldc] bf16 with N/2 columns
  int M, N, K, ldc;
  int epi;
  int n_tiles, k_blocks;     // ceil(N/128), K/64
  int splits;                // blocks of a cluster that share a tile's K
  int n_stages;
};

__device__ __forceinline__ uint32_t wt_saddr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void wt_mbar_init(uint32_t bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void wt_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void wt_mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// arrive on a barrier of another block of the cluster (address from mapa), releasing this thread's earlier writes
__device__ __forceinline__ void wt_mbar_arrive_remote(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ bool wt_mbar_wait(uint32_t bar, uint32_t parity) {
  for (unsigned i = 0; i < WT_SPIN_LIMIT; ++i) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
  }
  return false;
}
// the same with cluster-scope acquire: what the arriving blocks wrote before their release is visible afterwards
__device__ __forceinline__ bool wt_mbar_wait_cluster(uint32_t bar, uint32_t parity) {
  for (unsigned i = 0; i < WT_SPIN_LIMIT; ++i) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
  }
  return false;
}
__device__ __forceinline__ uint32_t wt_map_to_rank(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  return remote;
}
__device__ __forceinline__ float wt_ld_cluster(uint32_t cluster_addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr) : "memory");
  return v;
}
__device__ __forceinline__ void wt_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint64_t wt_evict_first_policy() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ void wt_bulk_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar, uint64_t pol) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(pol) : "memory");
}
__device__ __forceinline__ void wt_tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar) : "memory");
}
// shared-memory matrix descriptor: K-major tile of rows of 128 bytes, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t wt_desc(uint32_t smem_byte_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_byte_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// instruction descriptor: D float32, A and B bfloat16, both K-major, M x N
__device__ __forceinline__ uint32_t wt_idesc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void wt_umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
               ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void wt_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void wt_tmem_ld32(uint32_t taddr, float (&r)[32]) {
  uint32_t u[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]), "=r"(u[8]),
        "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15]), "=r"(u[16]),
        "=r"(u[17]), "=r"(u[18]), "=r"(u[19]), "=r"(u[20]), "=r"(u[21]), "=r"(u[22]), "=r"(u[23]), "=r"(u[24]),
        "=r"(u[25]), "=r"(u[26]), "=r"(u[27]), "=r"(u[28]), "=r"(u[29]), "=r"(u[30]), "=r"(u[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) r[i] = __uint_as_float(u[i]);
}
__device__ __forceinline__ float wt_silu(float g) { return __fdividef(g, 1.f + __expf(-g)); }

// one value of the product, for weight row n (this thread's) and token t, through the epilogue.  Every lane of the
// warp calls this together (the SiLU form exchanges gate and up between neighbouring lanes).
__device__ __forceinline__ void wt_store(const WtParams& p, int n, int t, float v, int lane) {
  if (p.epi == WT_EPI_SILU_MUL) {
    const float up = __shfl_xor_sync(0xffffffffu, v, 1);      // rows alternate gate_j, up_j
    if (!(lane & 1) && n + 1 < p.N && t < p.M)
      ((bf16*)p.C)[(size_t)t * p.ldc + (n >> 1)] = __float2bfloat16_rn(wt_silu(v) * up);
  } else if (n < p.N && t < p.M) {
    if (p.epi == WT_EPI_BF16) ((bf16*)p.C)[(size_t)t * p.ldc + n] = __float2bfloat16_rn(v);
    else ((float*)p.C)[(size_t)t * p.ldc + n] = v;
  }
}

template <int NTOK>
__global__ void __launch_bounds__(WT_THREADS, 1) gemm_wtile_kernel(const __grid_constant__ CUtensorMap map_x, WtParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // full[], empty[]: the ring; acc_full[2], acc_empty[2]: the accumulators; part_full, part_empty: split-K exchange
  __shared__ __align__(8) unsigned long long bars[2 * WT_MAX_STAGES + 6];
  __shared__ uint32_t tmem_base_slot;
  __shared__ volatile int failed;
  constexpr uint32_t X_BYTES = NTOK * 128, STAGE_BYTES = WT_TILE_BYTES + X_BYTES;

  pdl_trigger();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t ring = (wt_saddr(smem_raw) + 1023u) & ~1023u;
  unsigned char* const ring_gen = smem_raw + (ring - wt_saddr(smem_raw));
  const uint32_t full0 = wt_saddr(&bars[0]), empty0 = wt_saddr(&bars[WT_MAX_STAGES]);
  const uint32_t acc_full0 = wt_saddr(&bars[2 * WT_MAX_STAGES]), acc_empty0 = wt_saddr(&bars[2 * WT_MAX_STAGES + 2]);
  const uint32_t part_full = wt_saddr(&bars[2 * WT_MAX_STAGES + 4]), part_empty = wt_saddr(&bars[2 * WT_MAX_STAGES + 5]);
  const int S = p.splits;
  const int rank = (int)blockIdx.x % S, cluster_id = (int)blockIdx.x / S, n_clusters = (int)gridDim.x / S;
  const int kbs = p.k_blocks / S;                 // k blocks of this block's share
  const int kb0 = rank * kbs;
  const int my_tiles = cluster_id < p.n_tiles ? (p.n_tiles - cluster_id + n_clusters - 1) / n_clusters : 0;
  // the partial sums of a tile, [token][weight row] float32, behind the ring
  float* const partial = reinterpret_cast<float*>(ring_gen + (size_t)p.n_stages * STAGE_BYTES);

  if (tid == 0) {
    failed = 0;
    for (int s = 0; s < p.n_stages; ++s) {
      wt_mbar_init(full0 + 8 * s, 1);
      wt_mbar_init(empty0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      wt_mbar_init(acc_full0 + 8 * b, 1);
      wt_mbar_init(acc_empty0 + 8 * b, 4);        // one arrival per epilogue warp
    }
    wt_mbar_init(part_full, 4 * S);               // every epilogue warp of every block of the cluster
    wt_mbar_init(part_empty, 4 * S);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(wt_saddr(&tmem_base_slot)), "n"(2 * NTOK) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  if (S > 1) wt_cluster_sync();                   // the other blocks' barriers exist before anyone arrives on them
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0) {
    // ------------------------------------------------------------- producer
    if (lane == 0) {
      const uint64_t pol = wt_evict_first_policy();
      const long long total = (long long)my_tiles * kbs;          // stages this block fills in its life
      const long long primed = total < p.n_stages ? total : p.n_stages;
      auto w_src = [&](long long i) {
        const int tile = cluster_id + (int)(i / kbs) * n_clusters, kb = kb0 + (int)(i % kbs);
        return p.Wt + ((size_t)tile * p.k_blocks + kb) * WT_TILE_BYTES;
      };
      // the weights do not depend on the kernel ahead: the first stages' weight tiles are on their way before the wait
      for (long long i = 0; i < primed; ++i) {
        const uint32_t bar = full0 + 8 * (int)i;
        wt_mbar_expect_tx(bar, STAGE_BYTES);
        wt_bulk_copy(ring + (uint32_t)i * STAGE_BYTES, w_src(i), WT_TILE_BYTES, bar, pol);
      }
      pdl_wait();                                                  // the activations come from the kernel ahead
      for (long long i = 0; i < primed; ++i)
        wt_tma_load_2d(ring + (uint32_t)i * STAGE_BYTES + WT_TILE_BYTES, &map_x, (kb0 + (int)(i % kbs)) * WT_BK, 0, full0 + 8 * (int)i);
      int s = primed == p.n_stages ? 0 : (int)primed;
      uint32_t phase = primed == p.n_stages ? 1u : 0u;
      for (long long i = primed; i < total; ++i) {
        if (failed || !wt_mbar_wait(empty0 + 8 * s, phase ^ 1)) { atomicExch(&g_wt_error, 1); failed = 1; break; }
        const uint32_t bar = full0 + 8 * s, dst = ring + (uint32_t)s * STAGE_BYTES;
        wt_mbar_expect_tx(bar, STAGE_BYTES);
        wt_bulk_copy(dst, w_src(i), WT_TILE_BYTES, bar, pol);
        wt_tma_load_2d(dst + WT_TILE_BYTES, &map_x, (kb0 + (int)(i % kbs)) * WT_BK, 0, bar);
        if (++s == p.n_stages) { s = 0; phase ^= 1; }
      }
      if (failed) for (int i = 0; i < 2048; ++i) __nanosleep(64);   // copies already issued still land in this block's memory
    } else {
      pdl_wait();
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issue
    if (lane == 0) {
      const uint32_t idesc = wt_idesc(WT_BM, NTOK);
      int s = 0;
      uint32_t phase = 0;
      for (int it = 0; it < my_tiles && !failed; ++it) {
        const int buf = it & 1;
        if (!wt_mbar_wait(acc_empty0 + 8 * buf, ((uint32_t)(it >> 1) & 1u) ^ 1)) { atomicExch(&g_wt_error, 4); failed = 1; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * NTOK);
        for (int kb = 0; kb < kbs; ++kb) {
          if (failed || !wt_mbar_wait(full0 + 8 * s, phase)) { atomicExch(&g_wt_error, 2); failed = 1; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t w_sm = ring + (uint32_t)s * STAGE_BYTES, x_sm = w_sm + WT_TILE_BYTES;
#pragma unroll
          for (int k = 0; k < WT_BK / WT_UMMA_K; ++k)
            wt_umma(d_tmem, wt_desc(w_sm + k * WT_UMMA_K * 2), wt_desc(x_sm + k * WT_UMMA_K * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          wt_commit(empty0 + 8 * s);
          if (++s == p.n_stages) { s = 0; phase ^= 1; }
        }
        if (failed) break;
        wt_commit(acc_full0 + 8 * buf);
      }
    }
    __syncwarp();
    pdl_wait();
  } else {
    // ------------------------------------------------------------- epilogue
    pdl_wait();
    const int quarter = warp & 3;                  // this warp reads TMEM lanes 32 quarter .. + 31
    const int row = quarter * 32 + lane;           // weight row inside the tile
    bool ok = true;
    for (int it = 0; it < my_tiles; ++it) {
      const int buf = it & 1;
      const int tile = cluster_id + it * n_clusters;
      const int n = tile * WT_BM + row;
      ok = ok && !failed && wt_mbar_wait(acc_full0 + 8 * buf, (uint32_t)(it >> 1) & 1u);
      if (!ok && lane == 0) { atomicExch(&g_wt_error, 3); failed = 1; }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0 && !failed;
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t t_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * NTOK);
      if (S == 1) {
#pragma unroll 1
        for (int c0 = 0; c0 < NTOK; c0 += 32) {
          float v[32];
          wt_tmem_ld32(t_addr + c0, v);
          if (c0 + 32 >= NTOK) {                   // everything of this accumulator is in registers
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) wt_mbar_arrive(acc_empty0 + 8 * buf);
          }
          if (c0 < p.M) {
#pragma unroll
            for (int j = 0; j < 32; ++j) wt_store(p, n, c0 + j, v[j], lane);
          }
        }
      } else {
        // this block's partial sums -> its shared memory (the readers of the tile before must be done with it)
        if (it > 0) {
          bool ok2 = wt_mbar_wait_cluster(part_empty, (uint32_t)(it - 1) & 1u);
          if (!ok2 && lane == 0) { atomicExch(&g_wt_error, 6); failed = 1; }
          ok = __shfl_sync(0xffffffffu, ok2 ? 1 : 0, 0) != 0 && !failed;
          if (!ok) break;
        }
#pragma unroll 1
        for (int c0 = 0; c0 < NTOK; c0 += 32) {
          float v[32];
          wt_tmem_ld32(t_addr + c0, v);
          if (c0 + 32 >= NTOK) {
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) wt_mbar_arrive(acc_empty0 + 8 * buf);
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) partial[(c0 + j) * WT_BM + row] = v[j];
        }
        __syncwarp();
        if (lane < S) wt_mbar_arrive_remote(wt_map_to_rank(part_full, (uint32_t)lane));   // release: the stores above
        bool ok2 = wt_mbar_wait_cluster(part_full, (uint32_t)it & 1u);
        if (!ok2 && lane == 0) { atomicExch(&g_wt_error, 5); failed = 1; }
        ok = __shfl_sync(0xffffffffu, ok2 ? 1 : 0, 0) != 0 && !failed;
        if (!ok) break;
        // block `rank` finishes tokens [rank * NTOK / S, (rank + 1) * NTOK / S): the shares are added in block order
        constexpr int MAX_PER = NTOK;              // NTOK / S tokens, at most NTOK / 2
        const int per = NTOK / S, t0 = rank * per;
        const uint32_t mine = wt_saddr(partial) + (uint32_t)row * 4;
        for (int tb = 0; tb < per; tb += 8) {
          float acc[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] = 0.f;
          for (int s2 = 0; s2 < S; ++s2) {
            const uint32_t base = wt_map_to_rank(mine, (uint32_t)s2);
            float x[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) x[j] = (tb + j < per) ? wt_ld_cluster(base + (uint32_t)(t0 + tb + j) * (WT_BM * 4)) : 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += x[j];
          }
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (tb + j < per) wt_store(p, n, t0 + tb + j, acc[j], lane);
        }
        (void)MAX_PER;
        __syncwarp();
        if (lane < S) wt_mbar_arrive_remote(wt_map_to_rank(part_empty, (uint32_t)lane));   // done reading everybody's sums
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (S > 1) wt_cluster_sync();                   // nobody leaves while another block may still read its shared memory
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(2 * NTOK) : "memory");
  }
}

// ------------------------------------------------------------------ packing W into tiles (once, at load)
// tile (nt, kb): 128 rows x 64 columns as the shared-memory image of the MMA's K-major operand with the 128-byte
// swizzle: row r at byte r * 128, its 16-byte unit c at position c ^ (r % 8).  Rows past N are zeros.
__global__ void wtile_pack_kernel(const bf16* __restrict__ W, uint4* __restrict__ out, int N, int K, int ldw, int k_blocks) {
  pdl_trigger();
  pdl_wait();
  const size_t unit = (size_t)blockIdx.x * blockDim.x + threadIdx.x;       // one 16-byte unit of the output
  const size_t n_units = (size_t)((N + WT_BM - 1) / WT_BM) * k_blocks * (WT_TILE_BYTES / 16);
  if (unit >= n_units) return;
  const int in_tile = (int)(unit % (WT_TILE_BYTES / 16));
  const size_t tile_id = unit / (WT_TILE_BYTES / 16);
  const int kb = (int)(tile_id % k_blocks), nt = (int)(tile_id / k_blocks);
  const int r = in_tile >> 3, pos = in_tile & 7, c = pos ^ (r & 7);
  const int n = nt * WT_BM + r, k = kb * WT_BK + c * 8;
  uint4 v = make_uint4(0u, 0u, 0u, 0u);
  if (n < N) v = *reinterpret_cast<const uint4*>(W + (size_t)n * ldw + k);
  out[unit] = v;
}

typedef CUresult (*WtEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

WtEncodeTiledFn wt_encode_fn() {
  static WtEncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (WtEncodeTiledFn)ptr;
  }
  return fn;
}

size_t wt_smem_bytes(int ntok, int n_stages, int splits) {
  return 1024 + (size_t)n_stages * (WT_TILE_BYTES + (size_t)ntok * 128) + (splits > 1 ? (size_t)ntok * WT_BM * 4 : 0);
}

template <int NTOK>
int wt_launch(const CUtensorMap& mx, WtParams p, int n_sms, cudaStream_t stream) {
  const size_t budget = 200 * 1024;
  int n_stages = (int)((budget - 1024 - (p.splits > 1 ? (size_t)NTOK * WT_BM * 4 : 0)) / (WT_TILE_BYTES + (size_t)NTOK * 128));
  if (n_stages > WT_MAX_STAGES) n_stages = WT_MAX_STAGES;
  if (n_stages < 2) return IE_BAD_SIZE;
  p.n_stages = n_stages;
  const size_t smem = wt_smem_bytes(NTOK, n_stages, p.splits);
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(gemm_wtile_kernel<NTOK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(budget + 1024));
    if (e != cudaSuccess) return (int)e;
    attr = true;
  }
  // clusters that the device runs at once (a cluster needs its blocks in one processing cluster at the same moment)
  static int max_clusters[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};
  int n_clusters;
  if (p.splits == 1) {
    n_clusters = n_sms;
  } else {
    if (max_clusters[p.splits] == 0) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3((unsigned)(p.splits * (n_sms / p.splits)));
      cfg.blockDim = dim3(WT_THREADS);
      cfg.dynamicSmemBytes = smem;
      cudaLaunchAttribute a[1];
      a[0].id = cudaLaunchAttributeClusterDimension;
      a[0].val.clusterDim.x = (unsigned)p.splits;
      a[0].val.clusterDim.y = 1;
      a[0].val.clusterDim.z = 1;
      cfg.attrs = a;
      cfg.numAttrs = 1;
      int n = 0;
      cudaError_t e = cudaOccupancyMaxActiveClusters(&n, gemm_wtile_kernel<NTOK>, &cfg);
      if (e != cudaSuccess) return (int)e;
      if (n <= 0) return IE_BAD_SIZE;
      max_clusters[p.splits] = n;
    }
    n_clusters = max_clusters[p.splits];
  }
  if (n_clusters > p.n_tiles) n_clusters = p.n_tiles;
  return launch_k_cluster(gemm_wtile_kernel<NTOK>, p.splits, dim3((unsigned)(n_clusters * p.splits)), dim3(WT_THREADS), smem,
                          stream, mx, p);
}

}  // namespace

extern "C" int ie_gemm_wtile_error() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_wt_error, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_wt_error, &zero, sizeof(int));
  return v;
}

// bytes of the tiled copy of a [N, K] bfloat16 matrix
extern "C" long long ie_wtile_bytes(int N, int K) {
  if (N <= 0 || K <= 0 || K % WT_BK) return -1;
  return (long long)((N + WT_BM - 1) / WT_BM) * (K / WT_BK) * WT_TILE_BYTES;
}

// W [N, K] bfloat16, rows ldw elements apart -> its tiled copy
extern "C" int ie_wtile_pack(const void* W, void* out, int N, int K, int ldw, cudaStream_t stream) {
  if (ie_wtile_bytes(N, K) < 0 || (ldw & 7)) return IE_BAD_SIZE;
  if (((uintptr_t)W | (uintptr_t)out) & 15) return IE_BAD_ALIGN;
  const size_t n_units = (size_t)ie_wtile_bytes(N, K) / 16;
  const int threads = 256;
  return launch_k(wtile_pack_kernel, dim3((unsigned)((n_units + threads - 1) / threads)), dim3(threads), 0, stream,
                  (const bf16*)W, (uint4*)out, N, K, ldw, K / WT_BK);
}

// 1 if the kernel takes the product: 1..128 rows of bfloat16 activations, K a multiple of 64
extern "C" int ie_gemm_wtile_supports(int M, int N, int K, int lda) {
  return (M > 0 && M <= 128 && N > 0 && K > 0 && K % WT_BK == 0 && lda % 8 == 0) ? 1 : 0;
}

// How many blocks share a tile's K: the largest of 1, 2, 4, 8 that still leaves every SM at most one block, divides
// the k blocks and the token columns; many tiles need no split.
extern "C" int ie_gemm_wtile_splits(int M, int N, int K, int n_sms) {
  const int n_tiles = (N + WT_BM - 1) / WT_BM, k_blocks = K / WT_BK;
  const int ntok = M <= 32 ? 32 : (M <= 64 ? 64 : 128);
  int s = 1;
  while (s < 8 && n_tiles * (s * 2) <= n_sms && k_blocks % (s * 2) == 0 && k_blocks / (s * 2) >= 2 && ntok % (s * 2) == 0) s *= 2;
  return s;
}

// X [M, K] bfloat16 (rows lda apart), Wt the tiled copy of W [N, K]; epi 0: C bf16 [M, N]; 1: C float32 [M, N];
// 3: silu(gate) * up over interleaved weight rows, C bf16 [M, N/2].  splits: 0 chooses (ie_gemm_wtile_splits).
extern "C" int ie_gemm_wtile(const void* X, const void* Wt, void* C, int M, int N, int K, int lda, int ldc, int epi,
                             int splits, int n_sms, cudaStream_t stream) {
  if (n_sms <= 0) return IE_BAD_SIZE;
  if (!ie_gemm_wtile_supports(M, N, K, lda)) return IE_BAD_SIZE;
  if (((uintptr_t)X | (uintptr_t)Wt) & 15) return IE_BAD_ALIGN;
  if (epi != WT_EPI_BF16 && epi != WT_EPI_F32 && epi != WT_EPI_SILU_MUL) return IE_BAD_DTYPE;
  if (epi == WT_EPI_SILU_MUL && (N & 1)) return IE_BAD_SIZE;
  const int ntok = M <= 32 ? 32 : (M <= 64 ? 64 : 128);
  if (splits <= 0) splits = ie_gemm_wtile_splits(M, N, K, n_sms);
  const int k_blocks = K / WT_BK;
  if ((splits != 1 && splits != 2 && splits != 4 && splits != 8) || k_blocks % splits || ntok % splits) return IE_BAD_SIZE;
  WtEncodeTiledFn fn = wt_encode_fn();
  if (!fn) return IE_BAD_SIZE;
  CUtensorMap mx;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
  const cuuint64_t strides[1] = {(cuuint64_t)lda * 2};
  const cuuint32_t box[2] = {(cuuint32_t)WT_BK, (cuuint32_t)ntok};
  const cuuint32_t elem[2] = {1, 1};
  if (fn(&mx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(X), dims, strides, box, elem,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return IE_BAD_ALIGN;
  WtParams p;
  p.Wt = (const unsigned char*)Wt; p.C = C; p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.epi = epi;
  p.n_tiles = (N + WT_BM - 1) / WT_BM; p.k_blocks = k_blocks; p.splits = splits; p.n_stages = 0;
  if (ntok == 32) return wt_launch<32>(mx, p, n_sms, stream);
  if (ntok == 64) return wt_launch<64>(mx, p, n_sms, stream);
  return wt_launch<128>(mx, p, n_sms, stream);
}
