// Persistent weight-streaming product for decode steps on sm_100a:
// C[M,N] = A[M,K] W[N,K]^T, M <= 16, bfloat16 weights read once from HBM by the
// bulk-copy engine (cp.async.bulk, completion on mbarriers) into a ring of shared
// memory stages, one block per SM that walks units of 8 weight rows.
//
// Why this shape: at M <= 16 the product is a read of W.  A block that owns little
// data spends its life on latency (first bytes from HBM, activations from L2,
// reduction, store); here a producer thread keeps the ring full across unit
// boundaries, so HBM requests never stop while consumer warps multiply, reduce and
// store.  Launched with programmatic dependent launch, the producer starts filling
// the ring with this kernel's weights while the kernel ahead is still running; only
// the consumers wait for its output.
//
//   producer  warp 8: for every (unit, k-stage) wait for the stage to be
//             free, arm its mbarrier with the byte count, issue one bulk copy per
//             weight row (rows are contiguous in global memory)
//   consumers warps 0-7: stage the activations once per block in shared memory
//             (bfloat16; with the RMSNorm prologue x*gain and 1/rms are computed here
//             in float32, engine/layers.py:24-25), then per stage each warp takes a
//             eighth of k, builds MMA fragments with 16-byte shared loads and runs
//             mma.sync m16n8k16; at the end of a unit each warp leaves its partial sums in
//             shared memory and goes on with the next unit
//   epilogue  warp 9: adds the eight partial sums of a unit in warp order and applies the
//             epilogue of gemm_stream.cu, one unit behind the consumers (two buffers of sums,
//             handed over through named barriers)
//
// Every wait on an mbarrier is bounded; on a timeout the block records an error
// word that ie_gemm_stream_tma_error() reads, stops issuing copies and leaves.
#include "common.cuh"

namespace {

// Prologues: PLAIN bfloat16 activations; NORM float32 residual rows, RMSNorm inside the kernel; PRENORMED bfloat16
// rows that the product ahead has already multiplied by this norm's gain, with that product's per-block sums of
// squares (the 1/rms is formed from them here and applied to the sums as in NORM).
// Epilogues: ...; RESIDUAL_NORMOUT is RESIDUAL that also prepares the next product's PRENORMED input: for the norm that
// comes next it writes bfloat16(new residual * gain) and its block's sums of squares of the new residual rows.
enum { PRO_PLAIN = 0, PRO_NORM = 1, PRO_PRENORMED = 2 };
enum { EPI_BF16 = 0, EPI_F32 = 1, EPI_RESIDUAL = 2, EPI_SILU_MUL = 3, EPI_RESIDUAL_NORMOUT = 4 };
constexpr int SSQ_SLOT = 16;         // floats per block in the sums-of-squares array (one per activation row)

constexpr int CONSUMER_WARPS = 8;
constexpr int CONSUMER_THREADS = CONSUMER_WARPS * 32;
constexpr int THREADS = CONSUMER_THREADS + 64;          // + the producer warp + the epilogue warp
constexpr int HANDOVER_THREADS = CONSUMER_THREADS + 32; // the consumers and the epilogue warp
constexpr int ROW_PAD = 64;          // bytes added to a row's pitch: keeps 16-byte fragment loads off shared banks
constexpr int MAX_STAGES = 12;
// polls of a wait that normally lasts microseconds.  Two switches exist for the test of the give-up path alone:
// -DIE_STREAM_SPIN_LIMIT=n shortens the waits, -DIE_STREAM_ARM_EXTRA=b arms every stage's barrier for b bytes more
// than are copied, so that no stage ever completes and every role runs into its limit.
#ifndef IE_STREAM_SPIN_LIMIT
#define IE_STREAM_SPIN_LIMIT (1u << 20)
#endif
#ifndef IE_STREAM_ARM_EXTRA
#define IE_STREAM_ARM_EXTRA 0
#endif
constexpr unsigned SPIN_LIMIT = IE_STREAM_SPIN_LIMIT;


__device__ int g_stream_error = 0;

// Diagnostics, compiled in with -DIE_STREAM_TRACE only: thread 0 of block 0 of every launch notes the GPU's
// nanosecond clock at eight points of its life; ie_gemm_stream_trace_read() hands the notes to the host.
#ifdef IE_STREAM_TRACE
constexpr int TRACE_LAUNCHES = 4096, TRACE_POINTS = 8;
__device__ unsigned long long g_trace[TRACE_LAUNCHES * TRACE_POINTS];
__device__ unsigned int g_trace_n = 0;
__device__ __forceinline__ unsigned long long trace_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define TRACE_BEGIN() unsigned int trace_id = TRACE_LAUNCHES; \
  if (blockIdx.x == 0 && threadIdx.x == 0) { trace_id = atomicAdd(&g_trace_n, 1u); \
    if (trace_id < TRACE_LAUNCHES) for (int i_ = 0; i_ < TRACE_POINTS; ++i_) g_trace[trace_id * TRACE_POINTS + i_] = 0; }
#define TRACE(point) { if (trace_id < TRACE_LAUNCHES) g_trace[trace_id * TRACE_POINTS + (point)] = trace_now(); }
#else
#define TRACE_BEGIN()
#define TRACE(point)
#endif

struct TmaParams {
  const void* A;          // PLAIN: bf16 [M, lda];  NORM: float32 residual rows [*, lda]
  const bf16* W;          // [N, ldw]
  void* C;
  const void* gain;
  const int* row_index;
  int M, N, K, lda, ldw, ldc;
  int gain_is_f32;
  float eps;
  int ks;                 // k elements per stage (multiple of 128)
  int n_stages;
  int x_rows;             // 8 or 16 activation rows (one MMA tile of tokens)
  int x_in_smem;          // activations staged in shared memory once per block (else read from L2 per chunk)
  // RESIDUAL_NORMOUT writes, PRENORMED reads:
  bf16* xg_out;           // [M, ld_xg] bfloat16(new residual * gain_next)
  const void* gain_next;  // gain of the norm that comes next
  int gain_next_is_f32;
  int ld_xg;
  float* ssq_out;         // [SSQ_SLOT rows][ssq_blocks] this block's sums of squares of the new residual rows
  const float* ssq_in;    // [SSQ_SLOT rows][ssq_blocks] the sums of the product ahead (PRENORMED)
  int ssq_blocks;
};

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// false when the phase did not complete within SPIN_LIMIT polls
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (unsigned i = 0; i < SPIN_LIMIT; ++i) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
  }
  return false;
}
// Weights are read once a step and are far larger than L2: they are marked "evict first", so that the stream
// does not push out what the step reads again and again (activations, norm gains, the kernels' own code).
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ void bulk_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar, uint64_t pol) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(pol) : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
// barrier 1: consumers and epilogue warp, once, when the activations are staged.  Barriers 2, 3 ("sums of unit are
// in red[0], red[1]") and 4, 5 ("red[0], red[1] have been read"): the consumers arrive on the first pair without
// waiting and the epilogue warp waits there; the other way round on the second pair.  So the consumers go on with the
// next unit's MMAs while the epilogue warp adds up and stores the one before.
__device__ __forceinline__ void handover_sync() { asm volatile("bar.sync 1, %0;" ::"n"(HANDOVER_THREADS) : "memory"); }
__device__ __forceinline__ void named_sync(int id) { asm volatile("bar.sync %0, %1;" ::"r"(id), "n"(HANDOVER_THREADS) : "memory"); }
__device__ __forceinline__ void named_arrive(int id) { asm volatile("bar.arrive %0, %1;" ::"r"(id), "n"(HANDOVER_THREADS) : "memory"); }
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// What a block's roles share: the ring of stages (slots `slot_bytes` apart, so that products with different stage
// shapes can follow one another through the same ring), its barriers, and scratch for the consumers.
struct BlockCtx {
  unsigned char* smem;      // dynamic shared memory: the ring, then the staged activations
  uint32_t ring;            // its shared-memory address
  uint32_t slot_bytes;      // distance between stages
  uint32_t x_off;           // offset of the staged activations
  uint32_t full0, empty0;   // addresses of the barrier arrays
  int n_stages;
  float* red;               // [2 or 4][CONSUMER_WARPS][4 * NT][32]
  float* inv_rms;           // [16]
  volatile int* failed;
};
struct RingPos {
  int s;
  uint32_t phase;
};

// ------------------------------------------------------------- producer (one warp)
// lane 0 waits for the stage and arms its barrier; then lane r issues the copy of weight row r, so that the copies of
// a stage are issued side by side rather than one after the other.  nt: units of 8 * nt rows.
__device__ __forceinline__ bool produce(const TmaParams& p, int nt, const BlockCtx& b, RingPos& pos, int lane) {
  const int unit_rows = 8 * nt;
  const int n_units = (p.N + unit_rows - 1) / unit_rows;
  const int k_stages = p.K / p.ks;
  const uint32_t w_pitch = (uint32_t)p.ks * 2 + ROW_PAD;
  bool ok = true;
  const uint32_t row_bytes = (uint32_t)p.ks * 2;
  const uint64_t pol = l2_evict_first_policy();
  for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
    const int n0 = u * unit_rows;
    const int rows = min(unit_rows, p.N - n0);
    const bf16* src = p.W + (size_t)(n0 + (lane < rows ? lane : 0)) * p.ldw;
    for (int ksi = 0; ksi < k_stages; ++ksi) {
      const uint32_t bar = b.full0 + 8 * pos.s;
      if (lane == 0) {
        ok = mbar_wait(b.empty0 + 8 * pos.s, pos.phase ^ 1);
        if (ok) mbar_expect_tx(bar, row_bytes * rows + IE_STREAM_ARM_EXTRA);
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      if (lane < rows) bulk_copy(b.ring + pos.s * b.slot_bytes + lane * w_pitch, src + (size_t)ksi * p.ks, row_bytes, bar, pol);
      if (++pos.s == b.n_stages) { pos.s = 0; pos.phase ^= 1; }
    }
  }
  return ok;
}

// ------------------------------------------------------------- consumers (eight warps)
// NT: 8*NT weight rows per unit (NT n-tiles of the MMA per warp)
// XS: activations staged in shared memory (true) or read from L2 per stage (false; plain prologue only)
// first: this product is the kernel's first: its consumers wait for the kernel ahead (after asking for the gain)
template <int NT, int PRO, int EPI, bool XS>
__device__ __forceinline__ void consume(const TmaParams& p, const BlockCtx& b, RingPos& pos, bool first, unsigned int trace_id) {
  constexpr int UNIT_ROWS = 8 * NT;
  constexpr int ASETS = 2;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_units = (p.N + UNIT_ROWS - 1) / UNIT_ROWS;
  const int k_stages = p.K / p.ks;
  const uint32_t w_pitch = (uint32_t)p.ks * 2 + ROW_PAD;
  const uint32_t stage_bytes = b.slot_bytes;
  const uint32_t x_pitch = (uint32_t)p.K * 2 + ROW_PAD;
  const uint32_t ring = b.ring;
  const uint32_t xs = ring + b.x_off;
  const uint32_t full0 = b.full0, empty0 = b.empty0;
  unsigned char* const smem = b.smem;
  volatile int& failed = *b.failed;
  float* const inv_rms = b.inv_rms;
  float (*red)[CONSUMER_WARPS][4 * NT][32] = reinterpret_cast<float (*)[CONSUMER_WARPS][4 * NT][32]>(b.red);
  int& s = pos.s;
  uint32_t& phase = pos.phase;
  (void)trace_id;
  TRACE(1);                                                  // barriers set up
  // The norm's gain does not depend on the kernel ahead, and it is cold (read once a step, long evicted): it
  // comes from HBM, behind the weights that every producer is streaming.  Ask for it before waiting.
  // (a lane takes four consecutive columns per round of 128, so that a warp's load is one contiguous 512 bytes)
  uint2 gpre[PRO == PRO_NORM ? 16 : 1];    // bfloat16 gain of the first 2,048 columns (a float32 gain is read later)
  if (PRO == PRO_NORM && XS && !p.gain_is_f32) {
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (lane * 4 + i * 128 < p.K)   // a volatile statement: the compiler must not sink it below the wait
        asm volatile("ld.global.nc.v2.u32 {%0,%1}, [%2];" : "=r"(gpre[i].x), "=r"(gpre[i].y)
                     : "l"((const bf16*)p.gain + lane * 4 + i * 128));
  }
  if (first) pdl_wait();
  TRACE(2);                                                  // the kernel ahead has finished
  const int g = lane >> 2, t = lane & 3;
  // activations -> shared memory, once per block (plain activations of a long K stay in L2 instead:
  // they would crowd the ring out of shared memory)
  if (XS) {
    unsigned char* xsm = smem + b.x_off;
    for (int m = warp; m < p.x_rows; m += CONSUMER_WARPS) {
      bf16* dst = reinterpret_cast<bf16*>(xsm + (size_t)m * x_pitch);
      if (m >= p.M) {
        for (int k = lane * 8; k < p.K; k += 256) *reinterpret_cast<uint4*>(dst + k) = make_uint4(0u, 0u, 0u, 0u);
        continue;
      }
      // PRENORMED: the per-block sums of squares of the product ahead are asked for first and added up (in a
      // fixed order) after the row has been copied, so that both come back in one trip to L2
      float part[8];
      if (PRO == PRO_PRENORMED) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          part[j] = (j * 32 + lane < p.ssq_blocks) ? __ldcg(p.ssq_in + (size_t)m * p.ssq_blocks + (j * 32 + lane)) : 0.f;
      }
      if (PRO == PRO_PLAIN || PRO == PRO_PRENORMED) {
        const bf16* src = (const bf16*)p.A + (size_t)m * p.lda;
        // read-only loads, eight rounds in flight: staging a row is a matter of trips to L2
        for (int kb = lane * 8; kb < p.K; kb += 2048) {
          uint4 v[8];
#pragma unroll
          for (int i = 0; i < 8; ++i)
            if (kb + i * 256 < p.K) v[i] = __ldcg(reinterpret_cast<const uint4*>(src + kb + i * 256));
#pragma unroll
          for (int i = 0; i < 8; ++i)
            if (kb + i * 256 < p.K) *reinterpret_cast<uint4*>(dst + kb + i * 256) = v[i];
        }
        if (PRO == PRO_PRENORMED) {
          float ssq = 0.f;
#pragma unroll
          for (int j = 0; j < 8; ++j) ssq += part[j];
          ssq = warp_sum(ssq);
          if (lane == 0) inv_rms[m] = 1.f / sqrtf(ssq / (float)p.K + p.eps);
        }
      } else {
        const int row = p.row_index ? p.row_index[m] : m;
        const float* src = (const float*)p.A + (size_t)row * p.lda;
        float ssq = 0.f;
        // Four rounds (1,024 columns) at a time: first every load of the batch (read-only loads, which the
        // compiler may move ahead of the stores to shared memory), then the arithmetic: a batch costs one
        // trip to L2, not one per round.
        for (int kb = lane * 4; kb < p.K; kb += 1024) {
          float4 xa[8];
#pragma unroll
          for (int i = 0; i < 8; ++i)
            if (kb + i * 128 < p.K) xa[i] = __ldcg(reinterpret_cast<const float4*>(src + kb + i * 128));
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int k = kb + i * 128;
            if (k < p.K) {
              float gv[4];
              if (p.gain_is_f32) {
                const float4 g0 = __ldg(reinterpret_cast<const float4*>((const float*)p.gain + k));
                gv[0] = g0.x; gv[1] = g0.y; gv[2] = g0.z; gv[3] = g0.w;
              } else {
                uint2 gr = (kb < 1024) ? gpre[i] : gpre[i + 8];     // fetched before the wait
                if (kb >= 2048) gr = __ldg(reinterpret_cast<const uint2*>((const bf16*)p.gain + k));
                const float2 f0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gr.x));
                const float2 f1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gr.y));
                gv[0] = f0.x; gv[1] = f0.y; gv[2] = f1.x; gv[3] = f1.y;
              }
              const float4 x0 = xa[i];
              ssq += x0.x * x0.x + x0.y * x0.y + x0.z * x0.z + x0.w * x0.w;
              uint2 o;
              o.x = pack2(x0.x * gv[0], x0.y * gv[1]);
              o.y = pack2(x0.z * gv[2], x0.w * gv[3]);
              *reinterpret_cast<uint2*>(dst + k) = o;
            }
          }
        }
        ssq = warp_sum(ssq);
        if (lane == 0) inv_rms[m] = 1.f / sqrtf(ssq / (float)p.K + p.eps);
      }
    }
  }
  TRACE(7);                                                  // warp 0 has staged its rows
  handover_sync();
  TRACE(3);                                                  // activations staged

  const int kw = warp * (p.ks / CONSUMER_WARPS);        // this warp's k offset inside a stage
  const int chunks = p.ks / (CONSUMER_WARPS * 32);      // 32-wide chunks per warp per stage
  const bool two = p.x_rows > 8;
  int parity = 0, n_done = 0;
  bool dead = false;   // after a timed-out wait a warp stops waiting and computing but still meets every barrier
  for (int u = blockIdx.x; u < n_units; u += gridDim.x) {
    // two accumulators per n-tile: the two MMAs of a chunk do not wait for each other
    // two accumulators per n-tile: the two MMAs of a chunk do not wait for each other (4 and 8 per n-tile were
    // measured too: a step of 16 layers at batch 8 took 0.968 and 0.985 ms against 0.941, for the registers they cost)
    float acc[NT][ASETS][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int a = 0; a < ASETS; ++a)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[nt][a][e] = 0.f;
    for (int ksi = 0; ksi < k_stages; ++ksi) {
      // activations that stay in L2 (plain bfloat16, long K) are requested before the wait for the stage:
      // they do not depend on it, and their latency then hides behind it
      uint4 xg0[XS ? 1 : 8], xg1[XS ? 1 : 8];
      if (!XS) {
        const bf16* xa = (const bf16*)p.A + (size_t)(g < p.M ? g : 0) * p.lda + (ksi * p.ks + kw + t * 8);
        const bf16* xb = (const bf16*)p.A + (size_t)(g + 8 < p.M ? g + 8 : 0) * p.lda + (ksi * p.ks + kw + t * 8);
        const bool va = g < p.M, vb = g + 8 < p.M;
#pragma unroll
        for (int u = 0; u < (XS ? 1 : 8); ++u) {
          const int c = min(u, chunks - 1);
          xg0[u] = __ldcg(reinterpret_cast<const uint4*>(xa + c * 32));
          xg1[u] = two ? __ldcg(reinterpret_cast<const uint4*>(xb + c * 32)) : make_uint4(0u, 0u, 0u, 0u);
          if (!va) xg0[u] = make_uint4(0u, 0u, 0u, 0u);
          if (!vb) xg1[u] = make_uint4(0u, 0u, 0u, 0u);
        }
      }
      if (!dead && (failed || !mbar_wait(full0 + 8 * s, phase))) {
        dead = true;
        if (lane == 0) { atomicExch(&g_stream_error, 2); failed = 1; }
      }
      if (dead) continue;
      if (u == (int)blockIdx.x && ksi == 0) TRACE(4);        // first stage has arrived
      const uint32_t wbase = ring + s * stage_bytes + g * w_pitch + (kw + t * 8) * 2;
      if (XS) {
        const uint32_t xbase = xs + g * x_pitch + (ksi * p.ks + kw + t * 8) * 2;
        for (int c0 = 0; c0 < chunks; c0 += ASETS / 2) {
#pragma unroll
          for (int cc = 0; cc < ASETS / 2; ++cc) {
            const int c = c0 + cc;
            if (c < chunks) {
              const uint4 x0 = lds128(xbase + c * 64);
              uint4 x1 = make_uint4(0u, 0u, 0u, 0u);
              if (two) x1 = lds128(xbase + 8 * x_pitch + c * 64);
#pragma unroll
              for (int nt = 0; nt < NT; ++nt) {
                const uint4 w = lds128(wbase + nt * 8 * w_pitch + c * 64);
                mma16816(acc[nt][2 * cc], x0.x, x1.x, x0.y, x1.y, w.x, w.y);
                mma16816(acc[nt][2 * cc + 1], x0.z, x1.z, x0.w, x1.w, w.z, w.w);
              }
            }
          }
        }
      } else {
#pragma unroll
        for (int u = 0; u < (XS ? 1 : 8); ++u) {
          if (u < chunks) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              const uint4 w = lds128(wbase + nt * 8 * w_pitch + u * 64);
              mma16816(acc[nt][(2 * u) % ASETS], xg0[u].x, xg1[u].x, xg0[u].y, xg1[u].y, w.x, w.y);
              mma16816(acc[nt][(2 * u + 1) % ASETS], xg0[u].z, xg1[u].z, xg0[u].w, xg1[u].w, w.z, w.w);
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty0 + 8 * s);
      if (++s == b.n_stages) { s = 0; phase ^= 1; }
    }
    // this warp's partial sums -> red[parity]; the buffer was last used two units ago, and the epilogue warp has
    // said when it had read it
    if (n_done >= 2) named_sync(4 + parity);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float sum = acc[nt][0][e];
#pragma unroll
        for (int a = 1; a < ASETS; ++a) sum += acc[nt][a][e];
        red[parity][warp][nt * 4 + e][lane] = sum;
      }
    named_arrive(2 + parity);
    if (u == (int)blockIdx.x) TRACE(5);                      // first unit multiplied
    parity ^= 1;
    ++n_done;
  }
  TRACE(6);                                                  // last unit multiplied
}

// ------------------------------------------------------------- epilogue (one warp)
// Lane ln holds, per n-tile nt and half h, the two neighbouring outputs (m = ln / 4 + 8 h, n = unit + 8 nt + 2 (ln % 4)):
// the layout of the MMA's accumulator, so the sums are read from red[] as the consumers wrote them.
template <int NT, int PRO, int EPI>
__device__ __forceinline__ void finish_units(const TmaParams& p, const BlockCtx& b, bool first) {
  constexpr int UNIT_ROWS = 8 * NT;
  const int lane = threadIdx.x & 31;
  const int n_units = (p.N + UNIT_ROWS - 1) / UNIT_ROWS;
  volatile int& failed = *b.failed;
  const float* const inv_rms = b.inv_rms;
  float (*red)[CONSUMER_WARPS][4 * NT][32] = reinterpret_cast<float (*)[CONSUMER_WARPS][4 * NT][32]>(b.red);
  if (first) pdl_wait();                                     // nothing is written before the kernel ahead has finished
  handover_sync();                                           // inv_rms is there
  const int gg = lane >> 2, tt = lane & 3;
  float ssq_lo = 0.f, ssq_hi = 0.f;    // RESIDUAL_NORMOUT: squares of the new residual values of rows gg and gg + 8
  int parity = 0;
  for (int u = blockIdx.x; u < n_units; u += gridDim.x) {
    named_sync(2 + parity);                                  // every consumer warp has left its sums
    if (!failed) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int m = gg + h * 8;
          const int n = u * UNIT_ROWS + nt * 8 + tt * 2;
          float v0 = 0.f, v1 = 0.f;
#pragma unroll
          for (int w4 = 0; w4 < CONSUMER_WARPS; ++w4) {
            v0 += red[parity][w4][nt * 4 + h * 2][lane];
            v1 += red[parity][w4][nt * 4 + h * 2 + 1][lane];
          }
          if (m < p.M && n < p.N) {
            if (PRO != PRO_PLAIN) {
              v0 *= inv_rms[m];
              v1 *= inv_rms[m];
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
            } else if (EPI == EPI_RESIDUAL_NORMOUT) {
              float* c = (float*)p.C + (size_t)m * p.ldc + n;
              const float r0 = c[0] + v0, r1 = has1 ? c[1] + v1 : 0.f;
              c[0] = r0;
              if (has1) c[1] = r1;
              if (h == 0) ssq_lo += r0 * r0 + r1 * r1;
              else ssq_hi += r0 * r0 + r1 * r1;
              const float g0 = p.gain_next_is_f32 ? ((const float*)p.gain_next)[n] : __bfloat162float(((const bf16*)p.gain_next)[n]);
              const float g1 = !has1 ? 0.f : (p.gain_next_is_f32 ? ((const float*)p.gain_next)[n + 1] : __bfloat162float(((const bf16*)p.gain_next)[n + 1]));
              bf16* xg = p.xg_out + (size_t)m * p.ld_xg + n;
              if (has1 && ((((uintptr_t)xg) & 3) == 0)) *reinterpret_cast<uint32_t*>(xg) = pack2(r0 * g0, r1 * g1);
              else { xg[0] = __float2bfloat16_rn(r0 * g0); if (has1) xg[1] = __float2bfloat16_rn(r1 * g1); }
            } else {
              const float sg = 1.f / (1.f + expf(-v0));
              ((bf16*)p.C)[(size_t)m * p.ldc + (n >> 1)] = __float2bfloat16_rn((v0 * sg) * v1);
            }
          }
        }
      }
    }
    // the consumers write this buffer again for the unit after the next: tell them that it has been read
    if (u + 2 * (int)gridDim.x < n_units) named_arrive(4 + parity);
    parity ^= 1;
  }
  if (EPI == EPI_RESIDUAL_NORMOUT) {
    // the block's sums of squares, row by row, in a fixed order: this lane's units and n-tiles in turn, then the four
    // lanes of a row's quad
    ssq_lo += __shfl_xor_sync(0xffffffffu, ssq_lo, 1);
    ssq_lo += __shfl_xor_sync(0xffffffffu, ssq_lo, 2);
    ssq_hi += __shfl_xor_sync(0xffffffffu, ssq_hi, 1);
    ssq_hi += __shfl_xor_sync(0xffffffffu, ssq_hi, 2);
    if (tt == 0) {
      // laid out [16 rows][ssq_blocks]: the reader's warp takes one row of it, contiguous
      p.ssq_out[(size_t)gg * p.ssq_blocks + blockIdx.x] = ssq_lo;
      p.ssq_out[(size_t)(gg + 8) * p.ssq_blocks + blockIdx.x] = ssq_hi;
      // the reader adds ssq_blocks entries up: those of blocks that this launch does not have are zero
      if (blockIdx.x == 0)
        for (int j = gridDim.x; j < p.ssq_blocks; ++j) {
          p.ssq_out[(size_t)gg * p.ssq_blocks + j] = 0.f;
          p.ssq_out[(size_t)(gg + 8) * p.ssq_blocks + j] = 0.f;
        }
    }
  }
}

// One product per launch.
template <int NT, int PRO, int EPI, bool XS>
// Units of 8 rows (short products: qkv, output) keep within 112 registers, so that the kernel behind them in
// the stream (decode attention, say) finds room on the SM and starts its own fetches early.
__global__ void __launch_bounds__(THREADS, NT == 1 ? 2 : 1) gemm_stream_tma_kernel(TmaParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) unsigned long long bars[2 * MAX_STAGES];   // full[], empty[]
  __shared__ float red[2][CONSUMER_WARPS][4 * NT][32];
  __shared__ float inv_rms[16];
  __shared__ volatile int failed;

  pdl_trigger();
  TRACE_BEGIN();
  TRACE(0);                                                  // entry
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  BlockCtx b;
  b.smem = smem;
  b.ring = smem_addr(smem);
  b.slot_bytes = (uint32_t)(8 * NT) * ((uint32_t)p.ks * 2 + ROW_PAD);
  b.x_off = p.n_stages * b.slot_bytes;
  b.full0 = smem_addr(&bars[0]);
  b.empty0 = smem_addr(&bars[MAX_STAGES]);
  b.n_stages = p.n_stages;
  b.red = &red[0][0][0][0];
  b.inv_rms = inv_rms;
  b.failed = &failed;
  if (tid == 0) {
    failed = 0;
    for (int s = 0; s < p.n_stages; ++s) {
      mbar_init(b.full0 + 8 * s, 1);
      mbar_init(b.empty0 + 8 * s, CONSUMER_WARPS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  RingPos pos = {0, 0};
  if (warp == CONSUMER_WARPS) {
    const bool ok = produce(p, NT, b, pos, lane);
    if (!ok && lane == 0) {
      atomicExch(&g_stream_error, 1);
      failed = 1;
      // copies already issued land in this block's shared memory: stay a bounded while before leaving
      for (int i = 0; i < 4096; ++i) __nanosleep(64);
    }
    pdl_wait();
    return;
  }
  if (warp == CONSUMER_WARPS + 1) {
    finish_units<NT, PRO, EPI>(p, b, true);
    return;
  }
#ifdef IE_STREAM_TRACE
  consume<NT, PRO, EPI, XS>(p, b, pos, true, trace_id);
#else
  consume<NT, PRO, EPI, XS>(p, b, pos, true, 0u);
#endif
}

template <int NT, int PRO, int EPI, bool XS>
int launch_xs(const TmaParams& p, int n_sms, size_t smem, cudaStream_t stream) {
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(gemm_stream_tma_kernel<NT, PRO, EPI, XS>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, 204 * 1024);
    if (e != cudaSuccess) return (int)e;
    attr = true;
  }
  const int n_units = (p.N + 8 * NT - 1) / (8 * NT);
  const int grid = n_units < n_sms ? n_units : n_sms;
  return launch_k(gemm_stream_tma_kernel<NT, PRO, EPI, XS>, grid, THREADS, smem, stream, p);
}

template <int NT, int PRO, int EPI>
int launch_one(const TmaParams& p, int n_sms, size_t smem, cudaStream_t stream) {
  if (p.x_in_smem) return launch_xs<NT, PRO, EPI, true>(p, n_sms, smem, stream);
  if (PRO == PRO_PLAIN) return launch_xs<NT, PRO_PLAIN, EPI, false>(p, n_sms, smem, stream);
  return IE_BAD_SIZE;
}

template <int PRO, int EPI>
int launch_tma(const TmaParams& p, int nt, int n_sms, size_t smem, cudaStream_t stream) {
  if (nt == 2) return launch_one<2, PRO, EPI>(p, n_sms, smem, stream);
  return launch_one<1, PRO, EPI>(p, n_sms, smem, stream);
}

}  // namespace

// 1 if the kernel takes this product (M <= 16, K a multiple of 256, activations fit in shared memory)
// Activations are kept in shared memory when they take at most this much; beyond it the plain prologue
// reads them from L2 and the RMSNorm prologue is not offered.
constexpr size_t X_SMEM_LIMIT = 100 * 1024;

extern "C" int ie_gemm_stream_tma_supports(int M, int N, int K, int pro) {
  if (M <= 0 || M > 16 || N <= 0 || K <= 0 || (K % 256)) return 0;
  const size_t x_bytes = (size_t)(M > 8 ? 16 : 8) * ((size_t)K * 2 + ROW_PAD);
  if (pro == PRO_NORM || pro == PRO_PRENORMED) return x_bytes <= X_SMEM_LIMIT ? 1 : 0;
  return 1;
}

// Reads and clears the error word that a timed-out mbarrier wait leaves (0: none).
extern "C" int ie_gemm_stream_tma_error() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_stream_error, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_stream_error, &zero, sizeof(int));
  return v;
}

#ifdef IE_STREAM_TRACE
// copies the notes of the launches so far to `out` ([launches][8] nanosecond clocks) and starts over; returns the number of launches
extern "C" int ie_gemm_stream_trace_read(unsigned long long* out, int max_launches) {
  unsigned int n = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&n, g_trace_n, sizeof(n)) != cudaSuccess) return -1;
  if ((int)n > max_launches) n = max_launches;
  if (n > TRACE_LAUNCHES) n = TRACE_LAUNCHES;
  if (n && cudaMemcpyFromSymbol(out, g_trace, (size_t)n * TRACE_POINTS * sizeof(unsigned long long)) != cudaSuccess) return -1;
  cudaMemcpyToSymbol(g_trace_n, &zero, sizeof(zero));
  return (int)n;
}
#endif

// pro 2 (PRENORMED): A is the bfloat16 [M, lda] that the product ahead wrote (its xg), ssq its sums of squares
//   ([ssq_blocks, 16] float32), eps the norm's; gain unused.
// epi 4 (RESIDUAL_NORMOUT): C float32 += product, and for the norm that comes next: xg [M, ld_xg] = bfloat16(C * gain_next)
//   and ssq [ssq_blocks, 16] = per-block sums of squares of the new rows of C (ssq_blocks >= the SMs used; N == the
//   width of C: the whole row passes through this launch).
extern "C" int ie_gemm_stream_tma(const void* A, const void* W, void* C, const void* gain, int gain_dtype,
                                  const int* row_index, int M, int N, int K, int lda, int ldw, int ldc, float eps,
                                  int pro, int epi, int n_sms, void* xg, int ld_xg, const void* gain_next,
                                  int gain_next_dtype, float* ssq, int ssq_blocks, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return IE_OK;
  if (!ie_gemm_stream_tma_supports(M, N, K, pro) || (lda & 7) || (ldw & 7)) return IE_BAD_SIZE;
  if (((uintptr_t)A | (uintptr_t)W) & 15) return IE_BAD_ALIGN;
  if (epi == EPI_SILU_MUL && (N & 1)) return IE_BAD_SIZE;
  if (n_sms <= 0) return IE_BAD_SIZE;
  TmaParams p;
  p.A = A; p.W = (const bf16*)W; p.C = C; p.gain = gain; p.row_index = row_index;
  p.M = M; p.N = N; p.K = K; p.lda = lda; p.ldw = ldw; p.ldc = ldc;
  p.gain_is_f32 = gain_dtype == IE_F32; p.eps = eps;
  p.xg_out = (bf16*)xg; p.ld_xg = ld_xg; p.gain_next = gain_next; p.gain_next_is_f32 = gain_next_dtype == IE_F32;
  p.ssq_out = ssq; p.ssq_in = ssq; p.ssq_blocks = ssq_blocks;
  if (epi == EPI_RESIDUAL_NORMOUT &&
      (!xg || !gain_next || !ssq || ssq_blocks < n_sms || (ld_xg & 1) || (((uintptr_t)xg | (uintptr_t)ssq) & 3)))
    return IE_BAD_SIZE;
  if (pro == PRO_PRENORMED && (!ssq || ssq_blocks <= 0 || ssq_blocks > 256)) return IE_BAD_SIZE;
  // units of 16 rows when that still gives every SM several units; a stage is 8 KB..16 KB per 8 rows
  p.x_rows = M > 8 ? 16 : 8;
  size_t x_bytes = (size_t)p.x_rows * ((size_t)K * 2 + ROW_PAD);
  p.x_in_smem = x_bytes <= X_SMEM_LIMIT ? 1 : 0;
  if (!p.x_in_smem) x_bytes = 0;
  // Activations that stay in L2 are read again for every unit (all SMs, the same bytes): with a long K that is as
  // much traffic as the weights.  Units of 16 rows halve it; the longest block's share of the weights stays what
  // it was while there are at least about as many such units as SMs.
  int nt = (N >= 16 * 4 * n_sms) ? 2 : 1;
  if (!p.x_in_smem && (N + 15) / 16 >= (n_sms * 3) / 4) nt = 2;
  const int unit_rows = 8 * nt;
  const int ks_try[4] = {2048, 1024, 512, 256};
  // A product that keeps an SM busy for long wants a deep ring (HBM answers after about 2 us, so about
  // 100 KB per SM must be on its way).  A short one gains more from sharing the SM with the kernel behind
  // it in the chain, which then prefetches its weights early: that needs dynamic + static shared memory
  // of each to stay under 113 KB.
  bool deep = (size_t)N * K * 2 / (size_t)n_sms > 192 * 1024;
#if defined(IE_STREAM_RING_DEEP)      // -DIE_STREAM_RING_DEEP=0|1 fixes the choice (for measurements)
  deep = IE_STREAM_RING_DEEP != 0;
#endif
  size_t budget = (size_t)((deep ? 212 : 113) - (nt == 2 ? 17 : 9)) * 1024;
  int n_stages = 0;
  size_t stage_bytes = 0;
  for (int pass = 0; pass < 2 && n_stages < 3; ++pass) {
    for (int i = 0; i < 4 && n_stages < 3; ++i) {
      const int ks = ks_try[i];
      if (K % ks || ks % (CONSUMER_WARPS * 32)) continue;
      stage_bytes = (size_t)unit_rows * ((size_t)ks * 2 + ROW_PAD);
      if (x_bytes + 3 * stage_bytes > budget) continue;
      p.ks = ks;
      n_stages = (int)((budget - x_bytes) / stage_bytes);
    }
    budget = (size_t)(212 - (nt == 2 ? 17 : 9)) * 1024;
  }
  if (n_stages < 3) return IE_BAD_SIZE;
  if (n_stages > MAX_STAGES) n_stages = MAX_STAGES;
  p.n_stages = n_stages;
  const size_t smem = x_bytes + (size_t)n_stages * stage_bytes;
  if (pro == PRO_NORM) {
    if (!gain || ((uintptr_t)gain & 15)) return IE_BAD_ALIGN;
    if (epi == EPI_BF16) return launch_tma<PRO_NORM, EPI_BF16>(p, nt, n_sms, smem, stream);
    if (epi == EPI_F32) return launch_tma<PRO_NORM, EPI_F32>(p, nt, n_sms, smem, stream);
    if (epi == EPI_SILU_MUL) return launch_tma<PRO_NORM, EPI_SILU_MUL>(p, nt, n_sms, smem, stream);
    return IE_BAD_DTYPE;
  }
  if (pro == PRO_PRENORMED) {
    if (epi == EPI_BF16) return launch_tma<PRO_PRENORMED, EPI_BF16>(p, nt, n_sms, smem, stream);
    if (epi == EPI_F32) return launch_tma<PRO_PRENORMED, EPI_F32>(p, nt, n_sms, smem, stream);
    if (epi == EPI_SILU_MUL) return launch_tma<PRO_PRENORMED, EPI_SILU_MUL>(p, nt, n_sms, smem, stream);
    return IE_BAD_DTYPE;
  }
  if (pro == PRO_PLAIN) {
    if (epi == EPI_RESIDUAL_NORMOUT) return launch_tma<PRO_PLAIN, EPI_RESIDUAL_NORMOUT>(p, nt, n_sms, smem, stream);
    if (epi == EPI_BF16) return launch_tma<PRO_PLAIN, EPI_BF16>(p, nt, n_sms, smem, stream);
    if (epi == EPI_F32) return launch_tma<PRO_PLAIN, EPI_F32>(p, nt, n_sms, smem, stream);
    if (epi == EPI_RESIDUAL) return launch_tma<PRO_PLAIN, EPI_RESIDUAL>(p, nt, n_sms, smem, stream);
    if (epi == EPI_SILU_MUL) return launch_tma<PRO_PLAIN, EPI_SILU_MUL>(p, nt, n_sms, smem, stream);
    return IE_BAD_DTYPE;
  }
  return IE_BAD_DTYPE;
}
