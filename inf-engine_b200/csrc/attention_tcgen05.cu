// Causal paged attention for prompt portions on the fifth-generation tensor cores (sm_100a), head sizes 64
// and 128 (key tiles of 64 keys), bfloat16: S = Q K^T and O += P V are tcgen05.mma instructions with their accumulators in tensor memory;
// keys and values arrive page by page through TMA (cp.async.bulk.tensor over the cache pool); the online
// softmax runs one thread per row straight out of tensor memory (tcgen05.ld), with no shuffles.
//
// Same mathematics and same work split as attention_mma.cu (engine/llama_attention.py:106-137 of the
// reference): a block takes one (request, kv head) and a tile of 128 (token, head-in-group) rows, so that the
// query heads of a group share every key tile; keys are walked in tiles of 128 in ascending order.
//
//   warp 0      TMA producer: for each key tile looks the pages up in the block table and issues one tensor
//               copy per page for K and for V into a two-stage ring (a page that is not held or lies past the
//               end is replaced by page 0: its keys are masked, and the value rows from the block's last key on
//               are cleared in shared memory before the MMA reads them, so that nothing stored there, not
//               even a NaN, reaches the output)
//   warp 1      allocates tensor memory and issues  S = Q K^T.  S has two buffers in tensor memory: the scores of
//               tile j+2 go out as soon as the softmax has read those of tile j, so a softmax thread finds its
//               next scores ready when it has written P
//   warps 2-5   thread r owns row r: reads S from tensor memory, masks, keeps the running maximum and sum in
//               float32, rescales O in tensor memory when the maximum moved, writes P as bfloat16 into shared
//               memory in the 128-byte swizzle that the MMA expects (two P buffers where shared memory has room
//               for them: the exponentials of tile j+1 are then written while the MMAs of tile j still read)
//   warp 6      issues  O += P V  (V is the MN-major operand: its rows are keys, as the cache stores them).  A
//               thread of its own, because issuing a tile's MMAs and waiting for their barriers takes one thread
//               about as long as the softmax of a tile takes: with one issuing thread for both products the
//               softmax waited for it half of the time
//
// Every wait on an mbarrier is bounded; on a timeout the block records an error word, stops, frees its tensor
// memory and leaves.
#include "common.cuh"
#include <cuda.h>
#include <type_traits>

namespace {

constexpr int ROWS = 128;            // rows of a block's tile
// One softmax thread a row.  (Two threads a row, each with half of the keys of a tile and an exchange of maxima
// through shared memory, were measured: 48.7 us against 44.9 us at 2,048 tokens, head size 64.)
constexpr int FA_PV_WARP = 6;
constexpr int FA_THREADS = 64 + 128 + 32;
constexpr unsigned FA_SPIN_LIMIT = 1u << 20;
constexpr float LOG2E = 1.4426950408889634f;
constexpr uint32_t ATOM_BYTES = 128 * 64 * 2;   // 16 KB: 128 rows of one 128-byte swizzle atom (64 bfloat16)

// Shared-memory geometry for head size HD, key tiles of KT keys and a ring of STAGES key/value stages.  Operands are kept as "halves" of 64
// elements along their contiguous dimension (one swizzle atom wide): Q is HD/64 halves of [128 rows][64 dims],
// a K or V stage HD/64 halves of [KT keys][64 dims], P is KT/64 (at least one) halves of [128 rows][64 keys].
// PBUF: P buffers in shared memory (1 or 2), or 0: P stays in tensor memory, in the columns of the S buffer it was made
// from, and is the MMA's A operand from there (needs SBUF == 2); SBUF: S buffers in tensor memory (1 or 2).
template <int HD, int KT, int STAGES, int PBUF, int SBUF>
struct Geo {
  static constexpr int HALVES = HD / 64;
  static constexpr uint32_t Q_BYTES = HALVES * ATOM_BYTES;
  static constexpr uint32_t KV_HALF = KT * 128;
  static constexpr uint32_t KV_STAGE = HALVES * KV_HALF;
  static constexpr uint32_t P_BYTES = (KT / 64 > 0 ? KT / 64 : 1) * ATOM_BYTES;
  static constexpr uint32_t K_OFF = Q_BYTES, V_OFF = K_OFF + STAGES * KV_STAGE, P_OFF = V_OFF + STAGES * KV_STAGE;
  static constexpr uint32_t TILES_BYTES = P_OFF + PBUF * P_BYTES;
  // tensor memory: the S buffers in columns [0, SBUF KT), O in [SBUF KT, SBUF KT + HD), rounded up to a power of two
  static constexpr int O_COL = SBUF * KT;
  static constexpr int TMEM_COLS = O_COL + HD <= 128 ? 128 : (O_COL + HD <= 256 ? 256 : 512);
  // blocks that fit an SM (shared memory, tensor memory); the register budget follows from it
  static constexpr int BLOCKS_PER_SM = (TILES_BYTES + 1152) * 3 <= 232448 && TMEM_COLS * 3 <= 512 ? 3
                                       : ((TILES_BYTES + 1152) * 2 <= 232448 && TMEM_COLS * 2 <= 512 ? 2 : 1);
  static_assert(HD % 64 == 0 && HD <= 128 && KT % 64 == 0 && KT <= 128 && STAGES >= 2 && STAGES <= 4 && PBUF >= 0 && PBUF <= 2 && SBUF >= 1 && SBUF <= 2 && (PBUF > 0 || SBUF == 2), "geometry");
};

__device__ int g_fa_error = 0;

struct FaParams {
  const bf16* q;
  bf16* out;
  const int* block_table;
  const int* q_start;
  const int* ctx_before;
  const int* work_req;
  const int* work_pair0;
  int q_stride, out_stride, table_stride;
  int n_heads, n_kv_heads, page_size, page_shift, n_work;
  float scale_log2;
  // q arrives unrotated when these are given: cos / sin tables [positions, HD/2] float32 and each token's position
  // (rotation in pairs (i, i + HD/2), engine/layers.py:82-115 of the reference)
  const float* cos_t;
  const float* sin_t;
  const int* positions;
};

__device__ __forceinline__ uint32_t saddr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void fa_mbar_init(uint32_t bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void fa_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void fa_mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool fa_mbar_wait(uint32_t bar, uint32_t parity) {
  for (unsigned i = 0; i < FA_SPIN_LIMIT; ++i) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
  }
  return false;
}
__device__ __forceinline__ void fa_tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar) : "memory");
}
// K-major operand: rows of 128 bytes, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// MN-major operand (its rows are K, 128 bytes = 64 elements of MN each): K advances by rows, groups of 8 rows
// 1024 bytes apart (stride offset); groups of 64 MN elements `lbo_bytes` apart (leading offset)
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr, uint32_t lbo_bytes) {
  return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
__device__ __forceinline__ uint32_t idesc_f32_bf16(int m, int n, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void fa_umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
               ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// the same with A in tensor memory (rows are lanes, 16 bfloat16 of K are 8 columns of two each)
__device__ __forceinline__ void fa_umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
               ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void fa_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// the load alone: the registers are good after fa_tmem_wait_ld()
__device__ __forceinline__ void fa_tmem_ld32_issue(uint32_t taddr, float* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=f"(r[0]), "=f"(r[1]), "=f"(r[2]), "=f"(r[3]), "=f"(r[4]), "=f"(r[5]), "=f"(r[6]), "=f"(r[7]), "=f"(r[8]),
        "=f"(r[9]), "=f"(r[10]), "=f"(r[11]), "=f"(r[12]), "=f"(r[13]), "=f"(r[14]), "=f"(r[15]), "=f"(r[16]),
        "=f"(r[17]), "=f"(r[18]), "=f"(r[19]), "=f"(r[20]), "=f"(r[21]), "=f"(r[22]), "=f"(r[23]), "=f"(r[24]),
        "=f"(r[25]), "=f"(r[26]), "=f"(r[27]), "=f"(r[28]), "=f"(r[29]), "=f"(r[30]), "=f"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void fa_tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fa_tmem_ld32(uint32_t taddr, float (&r)[32]) {
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
__device__ __forceinline__ void fa_tmem_st32(uint32_t taddr, const float (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(__float_as_uint(r[0])), "r"(__float_as_uint(r[1])), "r"(__float_as_uint(r[2])),
        "r"(__float_as_uint(r[3])), "r"(__float_as_uint(r[4])), "r"(__float_as_uint(r[5])), "r"(__float_as_uint(r[6])),
        "r"(__float_as_uint(r[7])), "r"(__float_as_uint(r[8])), "r"(__float_as_uint(r[9])), "r"(__float_as_uint(r[10])),
        "r"(__float_as_uint(r[11])), "r"(__float_as_uint(r[12])), "r"(__float_as_uint(r[13])), "r"(__float_as_uint(r[14])),
        "r"(__float_as_uint(r[15])), "r"(__float_as_uint(r[16])), "r"(__float_as_uint(r[17])), "r"(__float_as_uint(r[18])),
        "r"(__float_as_uint(r[19])), "r"(__float_as_uint(r[20])), "r"(__float_as_uint(r[21])), "r"(__float_as_uint(r[22])),
        "r"(__float_as_uint(r[23])), "r"(__float_as_uint(r[24])), "r"(__float_as_uint(r[25])), "r"(__float_as_uint(r[26])),
        "r"(__float_as_uint(r[27])), "r"(__float_as_uint(r[28])), "r"(__float_as_uint(r[29])), "r"(__float_as_uint(r[30])),
        "r"(__float_as_uint(r[31]))
      : "memory");
}
__device__ __forceinline__ void fa_tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ float fa_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
// Packed float32 arithmetic of sm_100 (two lanes per instruction) and the three-input maximum: the softmax threads
// are bound by how many instructions they issue per score, not by any one pipe.
__device__ __forceinline__ uint64_t fa_pair(float lo, float hi) {
  uint64_t v;
  asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "f"(lo), "f"(hi));
  return v;
}
__device__ __forceinline__ void fa_unpair(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t fa_fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t fa_add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float fa_max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ uint32_t fa_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// byte offset of 16-byte chunk `chunk` (0..7) of row `row` in a tile of 128-byte rows under the 128-byte swizzle
__device__ __forceinline__ uint32_t sw128(int row, int chunk) { return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4)); }

template <int HD, int KT, int STAGES, int PBUF, int SBUF>
__global__ void __launch_bounds__(FA_THREADS, Geo<HD, KT, STAGES, PBUF, SBUF>::BLOCKS_PER_SM) attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_k,
                                                                          const __grid_constant__ CUtensorMap map_v,
                                                                          FaParams p) {
  // The tiles (Q, STAGES stages of K, as many of V, PBUF of P), then the barriers (kv_full[4], kv_empty[4], s_full[2],
  // p_ready[2], pv_done[2], q_ready), the tensor-memory slot and the failure flag.  No static shared memory and no
  // padding: two blocks have to fit one SM.
  using G = Geo<HD, KT, STAGES, PBUF, SBUF>;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem_raw + G::TILES_BYTES);
  uint32_t* tmem_slot_p = reinterpret_cast<uint32_t*>(smem_raw + G::TILES_BYTES + 120);
  volatile int* failed_p = reinterpret_cast<volatile int*>(smem_raw + G::TILES_BYTES + 124);
#define tmem_slot (*tmem_slot_p)
#define failed (*failed_p)

  pdl_trigger();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t base = saddr(smem_raw);
  if (base & 1023u) {              // the swizzled tiles need 1024-byte alignment: refuse rather than compute nonsense
    if (tid == 0) atomicExch(&g_fa_error, 8);
    return;
  }
  const uint32_t q_sm = base, k_sm = base + G::K_OFF, v_sm = base + G::V_OFF, p_sm = base + G::P_OFF;
  unsigned char* gen_base = smem_raw;
  const uint32_t kv_full0 = saddr(&bars[0]), kv_empty0 = saddr(&bars[4]);
  // p_ready0 + 8 (j & 1): P of tile j is written and S of tile j has been read; pv_done0 + 8 (j & 1): the MMAs
  // that read P of tile j are done.  Two of each, so that a waiter always waits for the newest phase of its barrier
  // or the one before (a tile's barrier is not used again before tile j + 2, which needs what the waiter gives).
  const uint32_t s_full0 = saddr(&bars[8]), p_ready0 = saddr(&bars[10]), pv_done0 = saddr(&bars[12]), q_ready = saddr(&bars[14]);

  // heads are the fast index and the work list is walked from its end: in a long prompt the tiles with the
  // most keys start first, and the short ones fill the tail of the launch
  const int c = blockIdx.x % p.n_kv_heads;
  const int w_id = p.n_work - 1 - blockIdx.x / p.n_kv_heads;
  const int r_id = p.work_req[w_id];
  const int pair0 = p.work_pair0[w_id];
  const int group = p.n_heads / p.n_kv_heads;
  const int q0 = p.q_start[r_id];
  const int q_len = p.q_start[r_id + 1] - q0;
  const int ctx = p.ctx_before[r_id];
  const int n_pairs = q_len * group;
  const int* table = p.block_table + (size_t)r_id * p.table_stride;
  const int last_pair = min(pair0 + ROWS, n_pairs) - 1;
  const int k_end = ctx + last_pair / group + 1;           // keys [0, k_end) matter to the block
  const int n_tiles = (k_end + KT - 1) / KT;

  if (tid == 0) {
    failed = 0;
    for (int s = 0; s < STAGES; ++s) {
      fa_mbar_init(kv_full0 + 8 * s, 1);
      fa_mbar_init(kv_empty0 + 8 * s, 1);
    }
    fa_mbar_init(s_full0, 1);
    fa_mbar_init(s_full0 + 8, 1);
    fa_mbar_init(p_ready0, 4);
    fa_mbar_init(p_ready0 + 8, 4);
    fa_mbar_init(pv_done0, 1);
    fa_mbar_init(pv_done0 + 8, 1);
    fa_mbar_init(q_ready, 4);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(saddr(tmem_slot_p)), "n"(G::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = tmem_slot;
  const uint32_t tmem_s = tmem, tmem_o = tmem + G::O_COL;

  pdl_wait();

  if (warp == 0) {
    // ------------------------------------------------------------- producer
    // lane i takes page i of a tile: the lookups of a tile run side by side (one after the other they cost
    // a trip to L2 each), and every lane issues its own two copies
    const int ps = p.page_size;
    const int pages_per_tile = KT / ps;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int s = j % STAGES;
      const uint32_t phase = (uint32_t)(j / STAGES) & 1u;
      int row = c * ps;                                     // page 0 stands in for what is not held
      if (lane < pages_per_tile) {
        const int kp = j * KT + lane * ps;
        if (kp < k_end) {
          const int page = IE_PAGE(__ldg(table + (kp >> p.page_shift)));
          if (page > 0) row = (page * p.n_kv_heads + c) * ps;
        }
      }
      const uint32_t bar = kv_full0 + 8 * s;
      if (lane == 0) {
        ok = !failed && fa_mbar_wait(kv_empty0 + 8 * s, phase ^ 1);
        if (ok) fa_mbar_expect_tx(bar, 2 * G::KV_STAGE);
        else { atomicExch(&g_fa_error, 1); failed = 1; }
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      if (lane < pages_per_tile) {
#pragma unroll
        for (int h = 0; h < G::HALVES; ++h) {
          fa_tma_load_2d(k_sm + s * G::KV_STAGE + h * G::KV_HALF + lane * ps * 128, &map_k, h * 64, row, bar);
          fa_tma_load_2d(v_sm + s * G::KV_STAGE + h * G::KV_HALF + lane * ps * 128, &map_v, h * 64, row, bar);
        }
      }
    }
    if (!ok) for (int i = 0; i < 2048; ++i) __nanosleep(64);
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issue: S_t = Q K_t^T into buffer t & 1
    if (lane == 0) {
      const uint32_t idesc_s = idesc_f32_bf16(ROWS, KT, 0);
      // descriptors differ only in their address field (bits 0-13, in units of 16 bytes): one base each, offsets added
      const uint64_t q_desc = desc_k_major(q_sm), k_desc = desc_k_major(k_sm);
      // the queries are written to shared memory by the softmax warps
      bool ok = !failed && fa_mbar_wait(q_ready, 0);
      if (!ok) { atomicExch(&g_fa_error, 5); failed = 1; }
      for (int t = 0; t < n_tiles && ok; ++t) {
        if (failed || !fa_mbar_wait(kv_full0 + 8 * (t % STAGES), (uint32_t)(t / STAGES) & 1u)) { atomicExch(&g_fa_error, 2); failed = 1; break; }
        // the buffer was read last for tile t - SBUF: by the softmax, and with P kept in it by the MMAs of that tile
        if (PBUF > 0) {
          if (t >= SBUF && !fa_mbar_wait(p_ready0 + 8 * ((t - SBUF) & 1), (uint32_t)((t - SBUF) >> 1) & 1u)) { atomicExch(&g_fa_error, 3); failed = 1; break; }
        } else {
          if (t >= 2 && !fa_mbar_wait(pv_done0 + 8 * (t & 1), (uint32_t)((t - 2) >> 1) & 1u)) { atomicExch(&g_fa_error, 3); failed = 1; break; }
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t kd = k_desc + (uint64_t)(((uint32_t)(t % STAGES) * G::KV_STAGE) >> 4);
        const uint32_t d = tmem_s + (uint32_t)((t % SBUF) * KT);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks)
          fa_umma(d, q_desc + (uint64_t)(((ks >> 2) * ATOM_BYTES + (ks & 3) * 32) >> 4),
                  kd + (uint64_t)(((ks >> 2) * G::KV_HALF + (ks & 3) * 32) >> 4), idesc_s, ks > 0 ? 1u : 0u);
        fa_commit(s_full0 + 8 * (t & 1));
      }
    }
  } else if (warp == FA_PV_WARP) {
    // ------------------------------------------------------------- MMA issue: O += P_j V_j
    if (lane == 0) {
      const uint32_t idesc_o = idesc_f32_bf16(ROWS, HD, 1);
      const uint64_t p_desc = desc_k_major(p_sm), v_desc = desc_mn_major(v_sm, G::KV_HALF);
      for (int j = 0; j < n_tiles; ++j) {
        if (failed || !fa_mbar_wait(p_ready0 + 8 * (j & 1), (uint32_t)(j >> 1) & 1u)) { atomicExch(&g_fa_error, 3); failed = 1; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int s = j % STAGES;
        const uint64_t vd = v_desc + (uint64_t)(((uint32_t)s * G::KV_STAGE) >> 4);
        if (PBUF > 0) {
          const uint64_t pd = p_desc + (uint64_t)(((uint32_t)(j % (PBUF > 0 ? PBUF : 1)) * G::P_BYTES) >> 4);
#pragma unroll
          for (int kk = 0; kk < KT / 16; ++kk)
            fa_umma(tmem_o, pd + (uint64_t)(((kk >> 2) * ATOM_BYTES + (kk & 3) * 32) >> 4), vd + (uint64_t)((kk * 2048) >> 4),
                    idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
        } else {
          // P of tile j sits in the first KT/2 columns of S buffer j & 1 (two bfloat16 a column)
          const uint32_t pa = tmem_s + (uint32_t)((j & 1) * KT);
#pragma unroll
          for (int kk = 0; kk < KT / 16; ++kk)
            fa_umma_ts(tmem_o, pa + (uint32_t)(kk * 8), vd + (uint64_t)((kk * 2048) >> 4), idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
        }
        // K of the stage was read by S_j, which was complete before the softmax of tile j read it; V by these
        fa_commit(kv_empty0 + 8 * s);
        fa_commit(pv_done0 + 8 * (j & 1));
      }
    }
  } else {
    // ------------------------------------------------------------- softmax
    // Thread r owns row r of the tile; a warp reads the 32 lanes of tensor memory of quarter warp % 4.
    static_assert(KT % 32 == 0 && HD % 32 == 0, "whole loads of 32 columns");
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;                    // row of the tile = TMEM lane
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const int pr = pair0 + r;
    const bool valid = pr < n_pairs;
    const int t = valid ? pr / group : 0;
    const int head = c * group + (valid ? pr - t * group : 0);
    const int limit = valid ? ctx + t : 0x3fffffff;       // last visible key (rows past the end are not stored)

    // queries -> shared memory in the MMA's swizzle, rotated on the way if they arrive unrotated
    {
      const bf16* src = p.q + (size_t)(q0 + t) * p.q_stride + head * HD;
      if (p.cos_t != nullptr) {
        const int pos = valid ? p.positions[q0 + t] : 0;
        const float* cr = p.cos_t + (size_t)pos * (HD / 2);
        const float* sr = p.sin_t + (size_t)pos * (HD / 2);
#pragma unroll
        for (int ch = 0; ch < HD / 16; ++ch) {             // chunk ch holds dims 8 ch .., its partners are chunk ch + HD/16
          uint4 lo = make_uint4(0u, 0u, 0u, 0u), hi = lo;
          if (valid) {
            lo = *reinterpret_cast<const uint4*>(src + ch * 8);
            hi = *reinterpret_cast<const uint4*>(src + HD / 2 + ch * 8);
            const float4 c0 = *reinterpret_cast<const float4*>(cr + ch * 8), c1 = *reinterpret_cast<const float4*>(cr + ch * 8 + 4);
            const float4 s0 = *reinterpret_cast<const float4*>(sr + ch * 8), s1 = *reinterpret_cast<const float4*>(sr + ch * 8 + 4);
            const float cc[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
            const float ss[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
            uint32_t* lw = reinterpret_cast<uint32_t*>(&lo);
            uint32_t* hw = reinterpret_cast<uint32_t*>(&hi);
#pragma unroll
            for (int w = 0; w < 4; ++w) {
              const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&lw[w]));
              const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&hw[w]));
              lw[w] = fa_pack(a.x * cc[2 * w] - b.x * ss[2 * w], a.y * cc[2 * w + 1] - b.y * ss[2 * w + 1]);
              hw[w] = fa_pack(b.x * cc[2 * w] + a.x * ss[2 * w], b.y * cc[2 * w + 1] + a.y * ss[2 * w + 1]);
            }
          }
          const int ch_hi = ch + HD / 16;
          *reinterpret_cast<uint4*>(gen_base + (ch >> 3) * ATOM_BYTES + sw128(r, ch & 7)) = lo;
          *reinterpret_cast<uint4*>(gen_base + (ch_hi >> 3) * ATOM_BYTES + sw128(r, ch_hi & 7)) = hi;
        }
      } else {
#pragma unroll
        for (int ch = 0; ch < HD / 8; ++ch) {
          uint4 v = make_uint4(0u, 0u, 0u, 0u);
          if (valid) v = *reinterpret_cast<const uint4*>(src + ch * 8);
          *reinterpret_cast<uint4*>(gen_base + (ch >> 3) * ATOM_BYTES + sw128(r, ch & 7)) = v;
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> visible to the tensor core
      __syncwarp();
      if (lane == 0) fa_mbar_arrive(q_ready);
    }

    // a bounded wait of the whole warp; false (and the error word set) when it ran out
    // a bounded wait of the whole warp; false (and the error word set) when it ran out.  Every lane polls the same
    // barrier; the failure flag is looked at only when a wait runs out (the other roles' waits are bounded too).
    auto wait_all = [&](uint32_t bar, uint32_t parity, int code) -> bool {
      const bool got = fa_mbar_wait(bar, parity);
      if (!__all_sync(0xffffffffu, got)) {
        if (lane == 0) { atomicExch(&g_fa_error, code); failed = 1; }
        return false;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      return true;
    };

    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      ok = wait_all(s_full0 + 8 * (j & 1), (uint32_t)(j >> 1) & 1u, 4);
      if (!ok) break;
      const int k0 = j * KT;
      // a tile whose last key every row of the warp may see needs no mask
      const bool interior = __all_sync(0xffffffffu, k0 + KT - 1 <= limit);
      // the scores of the row are read twice from tensor memory (once for the maximum, once for the exponentials),
      // each time with all loads on their way before the one wait
      float mx = -INFINITY;
      {
        float sc[KT];
#pragma unroll
        for (int q4 = 0; q4 < KT / 32; ++q4) fa_tmem_ld32_issue(tmem_s + lane_addr + (j % SBUF) * KT + q4 * 32, sc + q4 * 32);
        fa_tmem_wait_ld();
        if (interior) {
          float mb = -INFINITY;                              // two chains of three-input maxima
#pragma unroll
          for (int i = 0; i < KT; i += 4) {
            mx = fa_max3(mx, sc[i], sc[i + 1]);
            mb = fa_max3(mb, sc[i + 2], sc[i + 3]);
          }
          mx = fmaxf(mx, mb);
        } else {
#pragma unroll
          for (int i = 0; i < KT; ++i)
            if (k0 + i <= limit) mx = fmaxf(mx, sc[i]);
        }
      }
      // The maximum in use follows the true one only when that has grown by more than 2^8 (or is the
      // first): until then the exponentials are at most 256, which neither bfloat16 nor the float32 sums
      // mind, and O in tensor memory needs no rescaling.  The result is the same: numerator and
      // denominator carry the same factor.
      const float m_cand = fmaxf(m, mx * p.scale_log2);
      const bool moves = __any_sync(0xffffffffu, m_cand - m > 8.f || (m == -INFINITY && m_cand > -INFINITY));
      float corr = 1.f;
      if (moves) {
        corr = fa_exp2(m - (m_cand == -INFINITY ? 0.f : m_cand));    // 2^(-inf) = 0 the first time
        m = m_cand;
      }
      const float ms = m == -INFINITY ? 0.f : m;
      // this tile's P buffer belongs to the MMAs of tile j - PBUF until they are done
      if (PBUF > 0 && j >= PBUF) {
        ok = wait_all(pv_done0 + 8 * ((j - PBUF) & 1), (uint32_t)((j - PBUF) >> 1) & 1u, 6);
        if (!ok) break;
      }
      if (j > 0 && moves) {
        // O belongs to the MMAs of the tile before until they are done
        if (PBUF != 1) {
          ok = wait_all(pv_done0 + 8 * ((j - 1) & 1), (uint32_t)((j - 1) >> 1) & 1u, 6);
          if (!ok) break;
        }
#pragma unroll
        for (int h = 0; h < HD / 32; ++h) {
          float o[32];
          fa_tmem_ld32(tmem_o + lane_addr + h * 32, o);
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] *= corr;
          fa_tmem_st32(tmem_o + lane_addr + h * 32, o);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      }
      unsigned char* const p_tile = gen_base + G::P_OFF + (uint32_t)(j % (PBUF > 0 ? PBUF : 1)) * G::P_BYTES;
      const uint32_t p_tmem = tmem_s + lane_addr + (uint32_t)((j & 1) * KT);   // PBUF == 0: where this row's P goes
      const uint64_t scale2 = fa_pair(p.scale_log2, p.scale_log2), neg_m2 = fa_pair(-ms, -ms);
      uint64_t sum2a = fa_pair(0.f, 0.f), sum2b = sum2a;
      // exponentials, their sums and P; a tile that needs no mask takes the loop without the comparisons
      auto exp_pass = [&](auto masked) {
        constexpr bool MASKED = decltype(masked)::value;
        uint32_t pk[16];
        float sc[KT];
#pragma unroll
        for (int q4 = 0; q4 < KT / 32; ++q4) fa_tmem_ld32_issue(tmem_s + lane_addr + (j % SBUF) * KT + q4 * 32, sc + q4 * 32);
        fa_tmem_wait_ld();
#pragma unroll
        for (int ch = 0; ch < KT / 8; ++ch) {
          float e[8];
#pragma unroll
          for (int i = 0; i < 8; i += 2) {
            float x0, x1;
            fa_unpair(fa_fma2(fa_pair(sc[ch * 8 + i], sc[ch * 8 + i + 1]), scale2, neg_m2), x0, x1);
            x0 = fa_exp2(x0);
            x1 = fa_exp2(x1);
            e[i] = (!MASKED || k0 + ch * 8 + i <= limit) ? x0 : 0.f;
            e[i + 1] = (!MASKED || k0 + ch * 8 + i + 1 <= limit) ? x1 : 0.f;
            if (i & 2) sum2b = fa_add2(sum2b, fa_pair(e[i], e[i + 1]));
            else sum2a = fa_add2(sum2a, fa_pair(e[i], e[i + 1]));
          }
          const int col = ch * 8;                            // key index inside the tile
          const uint4 v = make_uint4(fa_pack(e[0], e[1]), fa_pack(e[2], e[3]), fa_pack(e[4], e[5]), fa_pack(e[6], e[7]));
          if (PBUF > 0) {
            *reinterpret_cast<uint4*>(p_tile + (col >> 6) * ATOM_BYTES + sw128(r, (col & 63) >> 3)) = v;
          } else {
            // 32 keys (16 columns) at a time into the S buffer's own columns: every score of the tile is in registers
            pk[(ch & 3) * 4] = v.x; pk[(ch & 3) * 4 + 1] = v.y; pk[(ch & 3) * 4 + 2] = v.z; pk[(ch & 3) * 4 + 3] = v.w;
            if ((ch & 3) == 3) fa_tmem_st16(p_tmem + (uint32_t)((ch >> 2) * 16), pk);
          }
        }
      };
      if (interior) exp_pass(std::false_type{});
      else exp_pass(std::true_type{});
      float sum;
      {
        float a0, a1, b0, b1;
        fa_unpair(sum2a, a0, a1);
        fa_unpair(sum2b, b0, b1);
        sum = (a0 + a1) + (b0 + b1);
      }
      l = l * corr + sum;
      if (j == n_tiles - 1 && k_end < (j + 1) * KT) {
        // The last tile came in as whole pages: its rows from key k_end on are the unused tail of the request's last
        // page or a stand-in page, and hold whatever was stored there before (another request's values, NaN).
        // Their P is zero, but 0 x NaN is NaN: the value rows are cleared before the MMA reads them.  The copies
        // have landed (the scores of this tile, which this thread has read, were issued after them).
        const int first_dead = k_end - j * KT;
        unsigned char* vst = gen_base + G::V_OFF + (uint32_t)(j % STAGES) * G::KV_STAGE;
        for (int idx = r; idx < KT * G::HALVES; idx += ROWS) {
          const int row = idx % KT, half = idx / KT;
          if (row >= first_dead) {
            uint4* dst = reinterpret_cast<uint4*>(vst + half * G::KV_HALF + row * 128);
#pragma unroll
            for (int i = 0; i < 8; ++i) dst[i] = make_uint4(0u, 0u, 0u, 0u);
          }
        }
      }
      if (PBUF > 0) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      } else {
        // P went to tensor memory; shared memory was written only if value rows were cleared (the last tile)
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        if (j == n_tiles - 1) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) fa_mbar_arrive(p_ready0 + 8 * (j & 1));
    }
    if (ok) ok = wait_all(pv_done0 + 8 * ((n_tiles - 1) & 1), (uint32_t)((n_tiles - 1) >> 1) & 1u, 7);
    if (ok) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      bf16* dst = p.out + (size_t)(q0 + t) * p.out_stride + head * HD;
#pragma unroll
      for (int h = 0; h < HD / 32; ++h) {
        float o[32];
        fa_tmem_ld32(tmem_o + lane_addr + h * 32, o);
        if (valid) {
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            const uint4 v = make_uint4(fa_pack(o[ch * 8] * inv, o[ch * 8 + 1] * inv), fa_pack(o[ch * 8 + 2] * inv, o[ch * 8 + 3] * inv),
                                       fa_pack(o[ch * 8 + 4] * inv, o[ch * 8 + 5] * inv), fa_pack(o[ch * 8 + 6] * inv, o[ch * 8 + 7] * inv));
            *reinterpret_cast<uint4*>(dst + h * 32 + ch * 8) = v;
          }
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "n"(G::TMEM_COLS) : "memory");
  }
#undef tmem_slot
#undef failed
}

typedef CUresult (*FaEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static FaEncodeFn fa_encode_fn() {
  static FaEncodeFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (FaEncodeFn)ptr;
  }
  return fn;
}

// the pool as a matrix [pool_rows, hd] of bfloat16 (a row is one key of one head); boxes of one page by 64 dims
static int fa_make_map(CUtensorMap* map, const void* base, long long pool_rows, int page_size, int hd) {
  FaEncodeFn fn = fa_encode_fn();
  if (!fn) return IE_BAD_SIZE;
  const cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)pool_rows};
  const cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
  const cuuint32_t box[2] = {64u, (cuuint32_t)page_size};
  const cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? IE_OK : IE_BAD_ALIGN;
}

}  // namespace

extern "C" int ie_attention_tcgen05_error() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_fa_error, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_fa_error, &zero, sizeof(int));
  return v;
}

// keys of a tile for a head size (0: not taken)
static int fa_key_tile(int hd) { return (hd == 64 || hd == 128) ? 64 : 0; }   // pages must divide this many keys

// 1 if the kernel takes the geometry: head size 64 or 128, pages of at least 8 keys, a power of two, that divide a
// key tile (64 keys); no window
extern "C" int ie_attention_tcgen05_supports(int hd, int page_size, int window) {
  const int kt = fa_key_tile(hd);
  if (!kt || window > 0) return 0;
  if (page_size < 8 || page_size > kt || (page_size & (page_size - 1)) || kt % page_size) return 0;
  return 1;
}

template <int HD, int KT, int STAGES, int PBUF, int SBUF>
static int fa_launch(const CUtensorMap& mk, const CUtensorMap& mv, const FaParams& p, int n_work, int n_kv_heads,
                     cudaStream_t stream) {
  const size_t smem = Geo<HD, KT, STAGES, PBUF, SBUF>::TILES_BYTES + 128;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(attention_tcgen05_kernel<HD, KT, STAGES, PBUF, SBUF>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    attr = true;
  }
  return launch_k(attention_tcgen05_kernel<HD, KT, STAGES, PBUF, SBUF>, dim3((unsigned)((long long)n_work * n_kv_heads)), FA_THREADS, smem,
                  stream, mk, mv, p);
}

// The work list cuts each request's (token, head-in-group) rows into tiles of 128; n_pool_pages is the
// number of pages of kpool / vpool; with cos_t / sin_t / positions q arrives unrotated and is rotated as it is read ([pages, kv_heads, page_size, hd]).
extern "C" int ie_attention_tcgen05(const void* q, void* out, const void* kpool, const void* vpool,
                                    const int* block_table, const int* q_start, const int* ctx_before,
                                    const int* work_req, const int* work_pair0, int q_stride, int out_stride,
                                    int table_stride, int n_work, int n_heads, int n_kv_heads, int hd, int page_size,
                                    int n_pool_pages, float scale, const float* cos_t, const float* sin_t,
                                    const int* positions, cudaStream_t stream) {
  if (n_work <= 0) return IE_OK;
  if ((cos_t == nullptr) != (sin_t == nullptr) || (cos_t && !positions)) return IE_BAD_SIZE;
  if (cos_t && (((uintptr_t)cos_t | (uintptr_t)sin_t) & 15)) return IE_BAD_ALIGN;
  if (!ie_attention_tcgen05_supports(hd, page_size, 0)) return IE_BAD_SIZE;
  if (n_kv_heads <= 0 || n_heads % n_kv_heads || n_pool_pages <= 0) return IE_BAD_SIZE;
  if (((uintptr_t)q | (uintptr_t)out | (uintptr_t)kpool | (uintptr_t)vpool) & 15) return IE_BAD_ALIGN;
  if ((q_stride | out_stride) & 7) return IE_BAD_ALIGN;
  CUtensorMap mk, mv;
  const long long rows = (long long)n_pool_pages * n_kv_heads * page_size;
  int rc = fa_make_map(&mk, kpool, rows, page_size, hd);
  if (rc) return rc;
  rc = fa_make_map(&mv, vpool, rows, page_size, hd);
  if (rc) return rc;
  FaParams p;
  p.q = (const bf16*)q; p.out = (bf16*)out; p.block_table = block_table; p.q_start = q_start; p.ctx_before = ctx_before;
  p.work_req = work_req; p.work_pair0 = work_pair0; p.q_stride = q_stride; p.out_stride = out_stride;
  p.table_stride = table_stride; p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.page_size = page_size;
  p.n_work = n_work;
  p.page_shift = 0;
  while ((1 << p.page_shift) < page_size) ++p.page_shift;
  p.scale_log2 = scale * LOG2E;
  p.cos_t = cos_t; p.sin_t = sin_t; p.positions = positions;
  // head size 64: two P buffers beside a ring of four stages (two blocks an SM); at 128 the ring takes that room.
  // (-DIE_FA_KT64=128 -DIE_FA_STAGES64=2 -DIE_FA_PBUF64=1 -DIE_FA_SBUF64=1, key tiles of 128 with one S buffer, was
  // measured: 8,192 tokens 467 us against 450 us)
#ifndef IE_FA_KT64
#define IE_FA_KT64 64
#define IE_FA_STAGES64 4
#define IE_FA_PBUF64 2
#define IE_FA_SBUF64 2
#endif
  if (hd == 64) return fa_launch<64, IE_FA_KT64, IE_FA_STAGES64, IE_FA_PBUF64, IE_FA_SBUF64>(mk, mv, p, n_work, n_kv_heads, stream);
  // head size 128: P stays in tensor memory, in the columns of the S buffer it was made from (shared memory has no
  // room for a second P buffer beside the ring there, and the exponentials of tile j + 1 then need not wait for the
  // MMAs of tile j either: 8,192 tokens 495 -> 447 us).  At head size 64 the same form (-DIE_FA_PBUF64=0) is no
  // faster than two P buffers in shared memory (442 us both; 2,048 tokens 40.9 against 39.7 us).
#ifndef IE_FA_PBUF128
#define IE_FA_PBUF128 0
#endif
  return fa_launch<128, 64, 2, IE_FA_PBUF128, 2>(mk, mv, p, n_work, n_kv_heads, stream);
}

IE_CHECK_API(attention_tcgen05)
