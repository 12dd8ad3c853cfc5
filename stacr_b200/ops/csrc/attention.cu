// Softmax attention forward on the fifth-generation tensor cores (tcgen05 + TMEM), flash style: the S x S score matrix
// never exists in memory.
//
// One CTA owns 128 query rows of one (batch, head) and walks the key/value tiles (64 keys each) that those rows may
// attend to.  Two CTAs share an SM (half of the shared memory and half of the tensor memory each), so one CTA's softmax
// runs under the other's tensor-core work and prologues hide behind main loops.  Warp roles (224 threads):
//   warp 0, lane 0   TMA producer: Q once, K tiles into a two-stage ring.
//   warp 6, lane 0   TMA producer: V tiles into a two-stage ring.
//   warp 1, lane 0   MMA issuer: S_j = Q K_j^T into one of two score accumulators in tensor memory, O += P_j V_j into
//                    the output accumulator.  S_{j+1} is issued before P_j V_j, so the tensor core computes the next
//                    scores while the softmax warps work on the current ones.
//   warps 2..5       softmax: thread t owns query row t of the tile (its TMEM lane): reads the 64 scores of its row into
//                    registers, masks (causal / key padding / sequence end), keeps a running maximum and sum in the base-2
//                    domain, writes P_j as bf16 back into tensor memory (over the scores it came from), from where the
//                    second product takes it as its A operand: P never touches shared memory, whose bandwidth is
//                    what bounds this kernel (the tensor core reads every smem operand at 128 B/clk).  It
//                    rescales the output accumulator in tensor memory only when the running maximum has grown by more
//                    than 2^8 since the last rescale (a stale maximum is exact as long as nothing overflows).
// The epilogue divides by the row sums, writes O as bf16 [tokens, heads * head_dim] and the row log-sum-exp for backward.
//
// Q, K and V are addressed through tensor maps over their source matrices (row = token), so a fused, per-head
// interleaved QKV projection output (GPT-NeoX) or a [Q | K | V] one (GPT-2, BERT) is read in place: no split, no
// transpose, no contiguous copies.  Every wait is bounded (status word + abort flag, as in the GEMM kernels).
// Replaces the library attention the reference reaches through its model code (eager scores + softmax in
// stacr/protocols/tp_gpt2.py:256-283 there, SDPA elsewhere).
#include "common.cuh"

namespace sb {

int make_tensor_map_bf16(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t box_outer);

namespace fa {

constexpr int BQ = 128, BKV = 64, THREADS = 224, UMMA_K = 16;
constexpr int TMEM_COLS = 256;
constexpr int COL_S0 = 0, COL_S1 = 64, COL_O = 128;
constexpr float RESCALE_THRESHOLD = 8.f;   // in log2 units
constexpr int ST_SMEM_MISALIGNED = 90;

struct FwdParams {
  int B, H, S;
  int q_col0, k_col0, v_col0, head_stride;   // first column of head h in the source matrices: col0 + h * head_stride
  int ld_o;                                  // leading dimension of the output [B * S, H * D]
  __nv_bfloat16* out;
  float* lse;                                // [B, H, S] natural-log row sums (for backward)
  const unsigned char* key_mask;             // optional [B, S]: 0 = this key is padding
  float scale_log2;                          // softmax scale * log2(e)
  int causal;
  int* status;
};

__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float y;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
  return y;
}
__device__ __forceinline__ void tmem_st_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
        "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
        "r"(r[30]), "r"(r[31])
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc]: the A operand (M = 128 rows on the 128 lanes, K along the columns, two bf16 per
// 32-bit column) is read from tensor memory.
__device__ __forceinline__ void umma_bf16_ta(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      :
      : "r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory plan (all tile buffers 1024-byte aligned; no slack, so that two CTAs fit on an SM):
//   Q        [D / 64 chunks][128 rows][128 B]
//   K[2]     [D / 64 chunks][64 rows][128 B], two stages
//   V[2]     [D / 64 column atoms][64 rows][128 B], two stages
template <int D>
struct Plan {
  static constexpr int Q_BYTES = BQ * D * 2;
  static constexpr int K_BYTES = BKV * D * 2;
  static constexpr int V_BYTES = BKV * D * 2;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + Q_BYTES;
  static constexpr int OFF_V = OFF_K + 2 * K_BYTES;
  static constexpr int OFF_BAR = OFF_V + 2 * V_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256;
};

// Barriers.  The MMA thread is a serial chain of waits, issues and commits, and each of those costs it a few hundred
// cycles, so every event it needs is folded into as few barriers as possible:
//   QK_GO[s]   K tile (and, for tile 0, Q) landed in stage s  AND  the softmax warps have taken the previous scores out of
//              accumulator s (1 producer arrival with the byte count + 4 warp arrivals; the first use is pre-arrived)
//   PV_GO[s]   V tile landed in stage s  AND  P_j is in tensor memory (1 + 4 arrivals)
//   S_FULL[s]  S_j is complete (commit): read by the softmax warps and by the K producer (stage s may be refilled)
//   PV_DONE[s] P_j V_j is complete (commit): read by the V producer, by a softmax thread that has to rescale the output
//              accumulator, and by the epilogue.  One barrier per stage, like the others: a waiter that names a phase by its
//              parity must never fall two phases behind, and a barrier of stage s cannot complete its next phase before the
//              waiter has refilled (or released) stage s.
enum Bar { QK_GO = 0, PV_GO = 2, S_FULL = 4, PV_DONE = 6, NBARS = 8 };   // every kind has two barriers, indexed by tile parity

// Non-blocking probe first: a barrier that has already completed is the common case on the MMA thread's critical path.
__device__ __forceinline__ bool wait_on(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  if (done) return true;
  return mbar_wait(bar, parity, abort_flag, status, code);
}

template <int D>
__global__ void __launch_bounds__(THREADS, 2)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_v, const FwdParams p) {
  using PL = Plan<D>;
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023u) {   // the swizzled layouts need 1024-byte aligned tiles; nothing has been started yet
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, ST_SMEM_MISALIGNED);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + PL::OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NBARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = (p.S + BQ - 1) / BQ;
  // heavy query tiles (late rows of a causal mask) first
  const int bh = blockIdx.x % (p.B * p.H);
  const int qt = nq - 1 - blockIdx.x / (p.B * p.H);
  const int b = bh / p.H, h = bh - b * p.H;
  const int q0 = qt * BQ;
  const int nkv_all = (p.S + BKV - 1) / BKV;
  const int nkv = p.causal ? min(nkv_all, (q0 + BQ) / BKV) : nkv_all;
  const int row_base = b * p.S;                      // first token row of this batch entry in the source matrices
  const int qcol = p.q_col0 + h * p.head_stride, kcol = p.k_col0 + h * p.head_stride, vcol = p.v_col0 + h * p.head_stride;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars[QK_GO + s], 5);
      mbar_init(&bars[PV_GO + s], 5);
      mbar_init(&bars[S_FULL + s], 1);
    }
    mbar_init(&bars[PV_DONE], 1);
    mbar_init(&bars[PV_DONE + 1], 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmap_q);
      tma_prefetch_desc(&tmap_k);
      for (int j = 0; j < nkv; ++j) {
        const int s = j & 1;
        const int kv0 = j * BKV;
        // stage s is free once S_{j-2}, which read it, is complete
        if (j >= 2 && !wait_on(&bars[S_FULL + s], ((j - 2) >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_SMEM_EMPTY)) break;
        mbar_expect_tx(&bars[QK_GO + s], PL::K_BYTES + (j == 0 ? PL::Q_BYTES : 0));
        if (j == 0) {
#pragma unroll
          for (int c = 0; c < D / 64; ++c) tma_load_2d(smem + PL::OFF_Q + c * (BQ * 128), &tmap_q, &bars[QK_GO], qcol + c * 64, row_base + q0);
        }
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          tma_load_2d(smem + PL::OFF_K + s * PL::K_BYTES + c * (BKV * 128), &tmap_k, &bars[QK_GO + s], kcol + c * 64, row_base + kv0);
      }
    }
  } else if (warp == 6) {
    // ------------------------------------------------------------------ TMA producer for V (its ring drains later than
    // K's: a producer of its own keeps a late V slot from holding back the next K tile)
    if (lane == 0) {
      tma_prefetch_desc(&tmap_v);
      for (int j = 0; j < nkv; ++j) {
        const int s = j & 1;
        const int kv0 = j * BKV;
        // stage s is free once P_{j-2} V_{j-2}, which read it, is complete
        if (j >= 2 && !wait_on(&bars[PV_DONE + s], ((j - 2) >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_SMEM_EMPTY)) break;
        mbar_expect_tx(&bars[PV_GO + s], PL::V_BYTES);
#pragma unroll
        for (int a = 0; a < D / 64; ++a)
          tma_load_2d(smem + PL::OFF_V + s * PL::V_BYTES + a * 8192, &tmap_v, &bars[PV_GO + s], vcol + a * 64, row_base + kv0);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BQ, BKV, false, false);   // S = Q K^T: both operands K-major
      constexpr uint32_t idesc_o = make_idesc_bf16(BQ, D, false, true);      // O = P V: V is MN-major (head_dim contiguous)
      const uint32_t q_addr = smem_u32(smem + PL::OFF_Q);
      auto issue_scores = [&](int j) {   // S_j into accumulator j & 1
        const int s = j & 1;
        const uint32_t k_addr = smem_u32(smem + PL::OFF_K + s * PL::K_BYTES);
        const uint32_t d_tmem = tmem_base + (s ? COL_S1 : COL_S0);
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
#pragma unroll
          for (int k = 0; k < 64 / UMMA_K; ++k)
            umma_bf16(d_tmem, make_smem_desc_sw128(q_addr + c * (BQ * 128) + k * 32, 16, 1024),
                      make_smem_desc_sw128(k_addr + c * (BKV * 128) + k * 32, 16, 1024), idesc_s, (c > 0 || k > 0) ? 1u : 0u);
        umma_commit(&bars[S_FULL + s]);
      };
      bool ok = true;
      if (nkv > 0) {
        ok = wait_on(&bars[QK_GO], 0, abort_flag, p.status, ST_TIMEOUT_SMEM_FULL);
        if (ok) {
          tc_fence_after();
          issue_scores(0);
        }
      }
      for (int j = 0; j < nkv && ok; ++j) {
        const int s = j & 1;
        if (j + 1 < nkv) {
          const int s1 = (j + 1) & 1;
          if (!wait_on(&bars[QK_GO + s1], ((j + 1) >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_SMEM_FULL)) { ok = false; break; }
          tc_fence_after();
          issue_scores(j + 1);
        }
        if (!wait_on(&bars[PV_GO + s], (j >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
        tc_fence_after();
        const uint32_t v_addr = smem_u32(smem + PL::OFF_V + s * PL::V_BYTES);
        // P_j sits in the first 32 columns of the score accumulator it was computed from (two bf16 per column)
        const uint32_t p_tmem = tmem_base + (s ? COL_S1 : COL_S0);
#pragma unroll
        for (int k = 0; k < BKV / UMMA_K; ++k)
          umma_bf16_ta(tmem_base + COL_O, p_tmem + k * (UMMA_K / 2), make_smem_desc_sw128(v_addr + k * 2048, 8192, 1024), idesc_o,
                       (j > 0 || k > 0) ? 1u : 0u);
        umma_commit(&bars[PV_DONE + s]);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax warps: thread = query row
    const int quad = warp & 3;                       // warp w may touch the TMEM lanes of quarter w % 4
    const int r = quad * 32 + lane;                  // row of the tile = TMEM lane
    const int qrow = q0 + r;                         // position in the sequence
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    float m_used = -INFINITY;                        // maximum the stored exponentials are relative to (log2 domain, scaled)
    float m_true = -INFINITY;                        // running maximum
    float l = 0.f;                                   // running sum of 2^(s - m_used)
    bool ok = true;
    if (lane == 0) {   // both score accumulators start out free
      mbar_arrive(&bars[QK_GO]);
      mbar_arrive(&bars[QK_GO + 1]);
    }
    for (int j = 0; j < nkv && ok; ++j) {
      const int s = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      const int kv0 = j * BKV;
      if (!wait_on(&bars[S_FULL + s], ph, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      uint32_t raw[2][32];
      tmem_ld_x32(t_lane + (s ? COL_S1 : COL_S0), raw[0]);
      tmem_ld_x32(t_lane + (s ? COL_S1 : COL_S0) + 32, raw[1]);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[QK_GO + s]);   // the accumulator may be overwritten by S_{j+2}
      // masks: sequence end, causal diagonal, key padding (scores stay unscaled here; the scale is positive)
      const bool edge = (kv0 + BKV > p.S) || (p.causal && kv0 + BKV - 1 > q0) || (p.key_mask != nullptr);
      if (edge) {
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int key = kv0 + c * 32 + i;
            bool keep = key < p.S && (!p.causal || key <= qrow);
            if (keep && p.key_mask) keep = p.key_mask[static_cast<size_t>(b) * p.S + key] != 0;
            if (!keep) raw[c][i] = 0xff800000u;   // -inf
          }
      }
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          const int a = (i >> 3) & 3;
          mx[a] = max3(mx[a], __uint_as_float(raw[c][i]), __uint_as_float(raw[c][i + 1]));
          mx[a] = max3(mx[a], __uint_as_float(raw[c][i + 2]), __uint_as_float(raw[c][i + 3]));
          mx[a] = max3(mx[a], __uint_as_float(raw[c][i + 4]), __uint_as_float(raw[c][i + 5]));
          mx[a] = max3(mx[a], __uint_as_float(raw[c][i + 6]), __uint_as_float(raw[c][i + 7]));
        }
      m_true = fmaxf(m_true, fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale_log2);
      // the output accumulator holds sums relative to m_used; rescale it (and l) only when the maximum has moved far
      float alpha = 1.f;
      bool rescale = false;
      if (m_true > m_used + RESCALE_THRESHOLD || m_used == -INFINITY) {
        if (m_used != -INFINITY) {
          alpha = ex2(m_used - m_true);
          rescale = true;
        }
        m_used = m_true;
      }
      const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used;   // a row with nothing to attend to so far
      float sum[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t packed[32];
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float e0 = ex2(fmaf(__uint_as_float(raw[c][i]), p.scale_log2, neg_m));
          const float e1 = ex2(fmaf(__uint_as_float(raw[c][i + 1]), p.scale_log2, neg_m));
          sum[(i >> 1) & 3] += e0 + e1;
          packed[c * 16 + i / 2] = pack_bf16x2(e0, e1);
        }
      l = l * alpha + ((sum[0] + sum[1]) + (sum[2] + sum[3]));
      if (__any_sync(0xffffffffu, rescale)) {
        // P_{j-1} V_{j-1} must have finished before the output accumulator is touched.  (The barrier of that stage cannot
        // complete another phase before this thread has stored P_{j+1}, so skipping this wait on other tiles is safe.)
        if (j > 0 && !wait_on(&bars[PV_DONE + ((j - 1) & 1)], ((j - 1) >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < D / 16; ++c) {
          uint32_t o[16];
          tmem_ld_x16(t_lane + COL_O + c * 16, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st_x16(t_lane + COL_O + c * 16, o);
        }
      }
      // P_j as the A operand of the second product, in tensor memory: it overwrites the scores it came from (this
      // thread's lane only, already in registers).  The previous user of these columns, P_{j-2} V_{j-2}, ran before S_j
      // was written, because the tensor core executes in issue order.
      tmem_st_x32(t_lane + (s ? COL_S1 : COL_S0), packed);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[PV_GO + s]);
    }
    // ---- epilogue
    if (ok && nkv > 0) ok = wait_on(&bars[PV_DONE + ((nkv - 1) & 1)], ((nkv - 1) >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL);
    if (ok) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const bool live = qrow < p.S;
      __nv_bfloat16* orow = p.out + (static_cast<size_t>(row_base) + qrow) * p.ld_o + h * D;
#pragma unroll 1
      for (int c = 0; c < D / 16; ++c) {
        uint32_t o[16];
        if (nkv > 0) {
          tmem_ld_x16(t_lane + COL_O + c * 16, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) o[i] = 0u;
        }
        if (live) {
          uint4 lo = make_uint4(pack_bf16x2(__uint_as_float(o[0]) * inv, __uint_as_float(o[1]) * inv), pack_bf16x2(__uint_as_float(o[2]) * inv, __uint_as_float(o[3]) * inv),
                                pack_bf16x2(__uint_as_float(o[4]) * inv, __uint_as_float(o[5]) * inv), pack_bf16x2(__uint_as_float(o[6]) * inv, __uint_as_float(o[7]) * inv));
          uint4 hi = make_uint4(pack_bf16x2(__uint_as_float(o[8]) * inv, __uint_as_float(o[9]) * inv), pack_bf16x2(__uint_as_float(o[10]) * inv, __uint_as_float(o[11]) * inv),
                                pack_bf16x2(__uint_as_float(o[12]) * inv, __uint_as_float(o[13]) * inv), pack_bf16x2(__uint_as_float(o[14]) * inv, __uint_as_float(o[15]) * inv));
          *reinterpret_cast<uint4*>(orow + c * 16) = lo;
          *reinterpret_cast<uint4*>(orow + c * 16 + 8) = hi;
        }
      }
      if (live && p.lse) {
        const float lse2 = (l > 0.f) ? m_used + log2f(l) : -INFINITY;
        p.lse[(static_cast<size_t>(b) * p.H + h) * p.S + qrow] = lse2 * 0.6931471805599453f;
      }
      tc_fence_before();
    }
  }

  // common exit: after an abandoned wait give copies in flight time to land, then free the tensor memory
  __syncwarp();
  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int D>
static int launch_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FwdParams& p, cudaStream_t st) {
  constexpr int MAX_DEVICES = 64;
  static bool cfg[MAX_DEVICES] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return -8;
  auto kern = flash_fwd_kernel<D>;
  if (!cfg[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Plan<D>::SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    cfg[dev] = true;
  }
  const int nq = (p.S + BQ - 1) / BQ;
  kern<<<nq * p.B * p.H, THREADS, Plan<D>::SMEM_BYTES, st>>>(tq, tk, tv, p);
  return static_cast<int>(cudaGetLastError());
}


// =====================================================================================================================
// Backward.  One CTA owns 128 keys of one (batch, head): K and V tiles stay in shared memory, dK and dV accumulate in tensor
// memory, and the CTA walks the 64-row query tiles that attend to its keys.  Everything is computed transposed (key = TMEM
// lane), so that P^T and dS^T are produced by the thread that owns a key row and every product has its M dimension on keys
// or on head_dim:
//     S^T  = K Q^T          (A = K,  K-major;  B = Q_i,  K-major)        [128 keys x 64 queries]
//     dP^T = V dO^T         (A = V,  K-major;  B = dO_i, K-major)
//     P^T  = exp2(S^T * scale - lse),   dS^T = P^T * (dP^T - delta)      (softmax warps; bf16, into shared memory)
//     dV  += P^T  dO_i      (A = P^T,  K-major; B = dO_i, MN-major: the same shared-memory tile, described the other way)
//     dK  += dS^T Q_i       (A = dS^T, K-major; B = Q_i,  MN-major)
//     dQ_i^T = K^T dS^T     (A = K, MN-major;   B = dS^T, MN-major)      [head_dim x 64 queries]
// dQ is summed over the key tiles of a row with fp32 reductions into a scratch matrix (coalesced: a warp adds 32 consecutive
// head_dim entries of one query), which a small kernel scales and converts afterwards.  head_dim 128 only.
// Warps: 0 producer (TMA, and lse / delta of the query tile into shared memory), 1 MMA, 2..9 softmax (two threads per key,
// 32 queries each), 10..17 dQ epilogue (two threads per head_dim index).
// =====================================================================================================================
constexpr int BWD_BK = 128, BWD_BQ = 64, BWD_THREADS = 576, BWD_D = 128;
constexpr int BWD_TMEM_COLS = 512;
constexpr int BCOL_S = 0, BCOL_DP = 64, BCOL_DV = 128, BCOL_DK = 256, BCOL_DQ = 384;

struct BwdParams {
  int B, H, S;
  int q_col0, k_col0, v_col0, head_stride;   // columns of head h in the q / k / v source matrices
  const float* lse;                          // [B, H, S] natural log-sum-exp from the forward
  const float* delta;                        // [B, H, S] rowsum(dO * O)
  float* dq32;                               // [B * S, H * D] fp32 scratch, zero on entry: receives sum_k dS K (unscaled)
  __nv_bfloat16* dk;                         // gradient matrices with the layout of the sources (row = token)
  __nv_bfloat16* dv;
  int ld_dk, ld_dv, dk_col0, dv_col0, dhead_stride;
  float scale, scale_log2;
  int causal;
  const unsigned char* key_mask;
  int* status;
};

struct BwdPlan {
  static constexpr int K_BYTES = BWD_BK * BWD_D * 2;        // 32 KB: [2 chunks][128 rows][128 B]
  static constexpr int QT_BYTES = BWD_BQ * BWD_D * 2;       // 16 KB: [2 chunks][64 rows][128 B]
  static constexpr int PT_BYTES = BWD_BK * BWD_BQ * 2;      // 16 KB: [128 rows][128 B]
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = OFF_K + K_BYTES;
  static constexpr int OFF_Q = OFF_V + K_BYTES;             // two stages
  static constexpr int OFF_DO = OFF_Q + 2 * QT_BYTES;       // two stages
  static constexpr int OFF_P = OFF_DO + 2 * QT_BYTES;
  static constexpr int OFF_DS = OFF_P + PT_BYTES;
  static constexpr int OFF_LSE = OFF_DS + PT_BYTES;         // [2 stages][64] lse (log2 domain), then [2][64] delta
  static constexpr int OFF_BAR = OFF_LSE + 2 * 2 * 64 * 4;
  static constexpr int SMEM_BYTES = OFF_BAR + 256;
};

// Barriers of the backward kernel:
//   KV_FULL      K and V tiles landed (once)
//   QDO_FULL[s]  Q_i and dO_i landed in stage s and their lse / delta are in shared memory (byte count + 1 warp arrival)
//   S_FULL       S^T and dP^T of this iteration are complete (commit)
//   S_FREE       the softmax warps have taken both out of tensor memory (8 warp arrivals)
//   PDS_READY    P^T and dS^T are in shared memory (8 warp arrivals)
//   ITER_DONE[s] dV, dK and dQ^T products of this iteration are complete (commit): stage s, the P / dS buffers are free again
//                and dQ^T can be read.  Per stage, so that the producer, which waits for the iteration before last, can
//                never fall two phases behind the barrier it names by parity
//   DQ_FREE      the epilogue warps have taken dQ^T out of tensor memory (8 warp arrivals)
enum BBar { KV_FULL = 0, QDO_FULL = 1, S_FULL_B = 3, S_FREE = 4, PDS_READY = 5, ITER_DONE = 6, DQ_FREE = 8, BNBARS = 9 };

__global__ void __launch_bounds__(BWD_THREADS, 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do, const BwdParams p) {
  using PL = BwdPlan;
  constexpr int D = BWD_D;
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023u) {
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, ST_SMEM_MISALIGNED);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + PL::OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + BNBARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* s_lse = reinterpret_cast<float*>(smem + PL::OFF_LSE);     // [2][64]
  float* s_delta = s_lse + 2 * 64;                                 // [2][64]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.x % (p.B * p.H);
  const int kt = blockIdx.x / (p.B * p.H);           // early key tiles (most query tiles under a causal mask) first
  const int b = bh / p.H, h = bh - b * p.H;
  const int kv0 = kt * BWD_BK;
  const int row_base = b * p.S;
  const int nq_all = (p.S + BWD_BQ - 1) / BWD_BQ;
  const int i_first = p.causal ? kv0 / BWD_BQ : 0;   // query tiles that can see a key of this tile
  const int niter = nq_all - i_first;
  const int qcol = p.q_col0 + h * p.head_stride, kcol = p.k_col0 + h * p.head_stride, vcol = p.v_col0 + h * p.head_stride;
  const int docol = h * D;

  if (threadIdx.x == 0) {
    mbar_init(&bars[KV_FULL], 1);
    mbar_init(&bars[QDO_FULL], 2);
    mbar_init(&bars[QDO_FULL + 1], 2);
    mbar_init(&bars[S_FULL_B], 1);
    mbar_init(&bars[S_FREE], 8);
    mbar_init(&bars[PDS_READY], 8);
    mbar_init(&bars[ITER_DONE], 1);
    mbar_init(&bars[ITER_DONE + 1], 1);
    mbar_init(&bars[DQ_FREE], 8);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, BWD_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer (whole warp: lane 0 issues the copies)
    if (lane == 0) {
      tma_prefetch_desc(&tmap_q);
      tma_prefetch_desc(&tmap_k);
      tma_prefetch_desc(&tmap_v);
      tma_prefetch_desc(&tmap_do);
      mbar_expect_tx(&bars[KV_FULL], 2 * PL::K_BYTES);
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        tma_load_2d(smem + PL::OFF_K + c * (BWD_BK * 128), &tmap_k, &bars[KV_FULL], kcol + c * 64, row_base + kv0);
        tma_load_2d(smem + PL::OFF_V + c * (BWD_BK * 128), &tmap_v, &bars[KV_FULL], vcol + c * 64, row_base + kv0);
      }
    }
    bool ok = true;
    for (int it = 0; it < niter; ++it) {
      const int s = it & 1;
      const int q0 = (i_first + it) * BWD_BQ;
      if (lane == 0) {
        // stage s was last used by iteration it - 2
        if (it >= 2) ok = wait_on(&bars[ITER_DONE + s], ((it - 2) >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_SMEM_EMPTY);
        if (ok) {
          mbar_expect_tx(&bars[QDO_FULL + s], 2 * PL::QT_BYTES);
#pragma unroll
          for (int c = 0; c < D / 64; ++c) {
            tma_load_2d(smem + PL::OFF_Q + s * PL::QT_BYTES + c * (BWD_BQ * 128), &tmap_q, &bars[QDO_FULL + s], qcol + c * 64, row_base + q0);
            tma_load_2d(smem + PL::OFF_DO + s * PL::QT_BYTES + c * (BWD_BQ * 128), &tmap_do, &bars[QDO_FULL + s], docol + c * 64, row_base + q0);
          }
        }
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      // lse (to the base-2 domain) and delta of the 64 queries
#pragma unroll
      for (int j = lane; j < BWD_BQ; j += 32) {
        const int q = q0 + j;
        const size_t at = (static_cast<size_t>(b) * p.H + h) * p.S + q;
        // a query with nothing to attend to has lse = -inf: +inf here makes its probabilities exp2(-inf) = 0
        const float l = q < p.S ? p.lse[at] : 0.f;
        s_lse[s * 64 + j] = l > -INFINITY ? l * 1.4426950408889634f : INFINITY;
        s_delta[s * 64 + j] = q < p.S ? p.delta[at] : 0.f;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[QDO_FULL + s]);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BWD_BK, BWD_BQ, false, false);   // S^T, dP^T
      constexpr uint32_t idesc_kv = make_idesc_bf16(BWD_BK, D, false, true);        // dV, dK: B (dO_i / Q_i) MN-major
      constexpr uint32_t idesc_dq = make_idesc_bf16(D, BWD_BQ, true, true);         // dQ^T: A = K MN-major, B = dS^T MN-major
      const uint32_t k_addr = smem_u32(smem + PL::OFF_K), v_addr = smem_u32(smem + PL::OFF_V);
      const uint32_t p_addr = smem_u32(smem + PL::OFF_P), ds_addr = smem_u32(smem + PL::OFF_DS);
      // S^T and dP^T of iteration it + 1 are issued before the three products of iteration it, so that they run on the tensor
      // core while the softmax warps work on iteration it (whose scores they have already taken into registers).
      auto issue_scores = [&](int it) {
        const int s = it & 1;
        const uint32_t q_addr = smem_u32(smem + PL::OFF_Q + s * PL::QT_BYTES), do_addr = smem_u32(smem + PL::OFF_DO + s * PL::QT_BYTES);
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
#pragma unroll
          for (int k = 0; k < 64 / UMMA_K; ++k) {
            umma_bf16(tmem_base + BCOL_S, make_smem_desc_sw128(k_addr + c * (BWD_BK * 128) + k * 32, 16, 1024),
                      make_smem_desc_sw128(q_addr + c * (BWD_BQ * 128) + k * 32, 16, 1024), idesc_s, (c > 0 || k > 0) ? 1u : 0u);
            umma_bf16(tmem_base + BCOL_DP, make_smem_desc_sw128(v_addr + c * (BWD_BK * 128) + k * 32, 16, 1024),
                      make_smem_desc_sw128(do_addr + c * (BWD_BQ * 128) + k * 32, 16, 1024), idesc_s, (c > 0 || k > 0) ? 1u : 0u);
          }
        umma_commit(&bars[S_FULL_B]);
      };
      bool ok = wait_on(&bars[KV_FULL], 0, abort_flag, p.status, ST_TIMEOUT_SMEM_FULL);
      if (ok && niter > 0) {
        ok = wait_on(&bars[QDO_FULL], 0, abort_flag, p.status, ST_TIMEOUT_SMEM_FULL);
        if (ok) {
          tc_fence_after();
          issue_scores(0);
        }
      }
      for (int it = 0; it < niter && ok; ++it) {
        const int s = it & 1;
        const uint32_t q_addr = smem_u32(smem + PL::OFF_Q + s * PL::QT_BYTES), do_addr = smem_u32(smem + PL::OFF_DO + s * PL::QT_BYTES);
        if (it + 1 < niter) {
          if (!wait_on(&bars[QDO_FULL + ((it + 1) & 1)], ((it + 1) >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_SMEM_FULL)) { ok = false; break; }
          if (!wait_on(&bars[S_FREE], it & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
          tc_fence_after();
          issue_scores(it + 1);
        }
        if (!wait_on(&bars[PDS_READY], it & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
        if (it > 0 && !wait_on(&bars[DQ_FREE], (it - 1) & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < BWD_BQ / UMMA_K; ++k) {   // reduction over the 64 queries of the tile
          umma_bf16(tmem_base + BCOL_DV, make_smem_desc_sw128(p_addr + k * 32, 16, 1024), make_smem_desc_sw128(do_addr + k * 2048, BWD_BQ * 128, 1024),
                    idesc_kv, (it > 0 || k > 0) ? 1u : 0u);
          umma_bf16(tmem_base + BCOL_DK, make_smem_desc_sw128(ds_addr + k * 32, 16, 1024), make_smem_desc_sw128(q_addr + k * 2048, BWD_BQ * 128, 1024),
                    idesc_kv, (it > 0 || k > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < BWD_BK / UMMA_K; ++k)     // reduction over the 128 keys of the tile
          umma_bf16(tmem_base + BCOL_DQ, make_smem_desc_sw128(k_addr + k * 2048, BWD_BK * 128, 1024), make_smem_desc_sw128(ds_addr + k * 2048, 8192, 1024),
                    idesc_dq, k > 0 ? 1u : 0u);
        umma_commit(&bars[ITER_DONE + s]);
      }
    }
  } else if (warp < 10) {
    // ------------------------------------------------------------------ softmax-backward warps: two threads per key row
    // (warp w may touch the TMEM lanes of quarter w % 4; warps 2..5 take queries 0..31 of the tile, warps 6..9 queries 32..63)
    const int quad = warp & 3;
    const int hsel = (warp - 2) >> 2;
    const int r = quad * 32 + lane;
    const int key = kv0 + r;
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    const bool key_ok = key < p.S && (p.key_mask == nullptr || p.key_mask[static_cast<size_t>(b) * p.S + key] != 0);
    uint8_t* p_row = smem + PL::OFF_P + r * 128;
    uint8_t* ds_row = smem + PL::OFF_DS + r * 128;
    bool ok = true;
    for (int it = 0; it < niter && ok; ++it) {
      const int s = it & 1;
      const int q0 = (i_first + it) * BWD_BQ + hsel * 32;   // first query of this thread's half
      if (!wait_on(&bars[QDO_FULL + s], (it >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_SMEM_FULL)) { ok = false; break; }   // lse / delta visible
      if (!wait_on(&bars[S_FULL_B], it & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      // everything into registers first: the accumulators are then free for the next query tile's scores
      uint32_t sv[32], dpv[32];
      tmem_ld_x32(t_lane + BCOL_S + hsel * 32, sv);
      tmem_ld_x32(t_lane + BCOL_DP + hsel * 32, dpv);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[S_FREE]);
      // a tile is an edge tile if any of its entries is masked: sequence end, the causal diagonal, or a padding key
      const bool edge = !key_ok || q0 + 32 > p.S || (p.causal && kv0 + BWD_BK - 1 > q0) || kv0 + BWD_BK > p.S;
      const float4* l4 = reinterpret_cast<const float4*>(s_lse + s * 64 + hsel * 32);
      const float4* d4 = reinterpret_cast<const float4*>(s_delta + s * 64 + hsel * 32);
      uint32_t pp[16], dd[16];
#pragma unroll
      for (int g4 = 0; g4 < 8; ++g4) {
        const float4 lv = l4[g4], dl = d4[g4];
        const float lse4[4] = {lv.x, lv.y, lv.z, lv.w}, del4[4] = {dl.x, dl.y, dl.z, dl.w};
        float pv[4], ds4[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int col = g4 * 4 + u;
          float pr = ex2(fmaf(__uint_as_float(sv[col]), p.scale_log2, -lse4[u]));
          if (edge) {
            const int q = q0 + col;
            if (!(key_ok && q < p.S && (!p.causal || key <= q))) pr = 0.f;
          }
          pv[u] = pr;
          ds4[u] = pr * (__uint_as_float(dpv[col]) - del4[u]);
        }
        pp[g4 * 2] = pack_bf16x2(pv[0], pv[1]);
        pp[g4 * 2 + 1] = pack_bf16x2(pv[2], pv[3]);
        dd[g4 * 2] = pack_bf16x2(ds4[0], ds4[1]);
        dd[g4 * 2 + 1] = pack_bf16x2(ds4[2], ds4[3]);
      }
      // the P / dS buffers were read by the products of iteration it - 1
      if (it > 0 && !wait_on(&bars[ITER_DONE + ((it - 1) & 1)], ((it - 1) >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_SMEM_EMPTY)) { ok = false; break; }
      // K-major, 128-byte-swizzled rows: 16-byte slot k holds queries 8k .. 8k + 7; this thread owns slots 4 * hsel .. + 3
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        const int slot = hsel * 4 + q4;
        *reinterpret_cast<uint4*>(p_row + ((slot ^ (r & 7)) << 4)) = make_uint4(pp[q4 * 4], pp[q4 * 4 + 1], pp[q4 * 4 + 2], pp[q4 * 4 + 3]);
        *reinterpret_cast<uint4*>(ds_row + ((slot ^ (r & 7)) << 4)) = make_uint4(dd[q4 * 4], dd[q4 * 4 + 1], dd[q4 * 4 + 2], dd[q4 * 4 + 3]);
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[PDS_READY]);
    }
    // ---- dK and dV of this key row
    if (ok && niter > 0) ok = wait_on(&bars[ITER_DONE + ((niter - 1) & 1)], ((niter - 1) >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL);
    if (ok) {   // (the tensor-memory loads are warp-collective: every lane runs them, only the stores depend on the key)
      tc_fence_after();
      __nv_bfloat16* dv_row = p.dv + (static_cast<size_t>(row_base) + key) * p.ld_dv + p.dv_col0 + h * p.dhead_stride;
      __nv_bfloat16* dk_row = p.dk + (static_cast<size_t>(row_base) + key) * p.ld_dk + p.dk_col0 + h * p.dhead_stride;
#pragma unroll 1
      for (int c = hsel * (D / 32); c < (hsel + 1) * (D / 32); ++c) {   // this thread's half of the head_dim columns
        uint32_t a[16], k16[16];
        if (niter > 0) {
          tmem_ld_x16(t_lane + BCOL_DV + c * 16, a);
          tmem_ld_x16(t_lane + BCOL_DK + c * 16, k16);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) a[i] = k16[i] = 0u;
        }
        uint32_t o[8], ok8[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          o[i] = pack_bf16x2(__uint_as_float(a[2 * i]), __uint_as_float(a[2 * i + 1]));
          ok8[i] = pack_bf16x2(__uint_as_float(k16[2 * i]) * p.scale, __uint_as_float(k16[2 * i + 1]) * p.scale);
        }
        if (key < p.S) {
          *reinterpret_cast<uint4*>(dv_row + c * 16) = make_uint4(o[0], o[1], o[2], o[3]);
          *reinterpret_cast<uint4*>(dv_row + c * 16 + 8) = make_uint4(o[4], o[5], o[6], o[7]);
          *reinterpret_cast<uint4*>(dk_row + c * 16) = make_uint4(ok8[0], ok8[1], ok8[2], ok8[3]);
          *reinterpret_cast<uint4*>(dk_row + c * 16 + 8) = make_uint4(ok8[4], ok8[5], ok8[6], ok8[7]);
        }
      }
      tc_fence_before();
    }
  } else {
    // ------------------------------------------------------------------ dQ epilogue warps: two threads per head_dim index
    const int quad = warp & 3;
    const int hsel = (warp - 10) >> 2;
    const int dlane = quad * 32 + lane;
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    const size_t row_floats = static_cast<size_t>(p.H) * D;
    bool ok = true;
    for (int it = 0; it < niter && ok; ++it) {
      const int q0 = (i_first + it) * BWD_BQ + hsel * 32;
      if (!wait_on(&bars[ITER_DONE + (it & 1)], (it >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      uint32_t v[32];
      tmem_ld_x32(t_lane + BCOL_DQ + hsel * 32, v);
      tmem_ld_wait();
      tc_fence_before();   // everything is in registers: the next dQ^T may overwrite the accumulator
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[DQ_FREE]);
      float* dst = p.dq32 + (static_cast<size_t>(row_base) + q0) * row_floats + h * D + dlane;
      const int valid = min(32, p.S - q0);
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < valid) atomicAdd(dst + j * row_floats, __uint_as_float(v[j]));
    }
  }

  __syncwarp();
  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, BWD_TMEM_COLS);
  }
}

// delta[b, h, s] = sum_d dO[b, s, h, d] * O[b, s, h, d]: one warp per (token, head).
__global__ void __launch_bounds__(256) attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout, int B, int S, int H,
                                                         int D, float* __restrict__ delta) {
  const int lane = threadIdx.x & 31;
  const long long item = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= static_cast<long long>(B) * S * H) return;
  const long long token = item / H;
  const int h = static_cast<int>(item - token * H);
  const __nv_bfloat16* a = o + token * (static_cast<long long>(H) * D) + static_cast<long long>(h) * D;
  const __nv_bfloat16* g = dout + token * (static_cast<long long>(H) * D) + static_cast<long long>(h) * D;
  float acc = 0.f;
  for (int d = lane * 2; d < D; d += 64) {
    const __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(a + d), y = *reinterpret_cast<const __nv_bfloat162*>(g + d);
    acc = fmaf(__bfloat162float(x.x), __bfloat162float(y.x), acc);
    acc = fmaf(__bfloat162float(x.y), __bfloat162float(y.y), acc);
  }
#pragma unroll
  for (int off = 16; off; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) {
    const long long bidx = token / S, sidx = token - bidx * S;
    delta[(bidx * H + h) * S + sidx] = acc;
  }
}

// dq (bf16, the layout of the q source) = scale * dq32 ([tokens, H * D] fp32).
__global__ void __launch_bounds__(256) attn_dq_convert_kernel(const float* __restrict__ dq32, long long tokens, int H, int D, float scale,
                                                              __nv_bfloat16* __restrict__ dq, int ld_dq, int dq_col0, int dhead_stride) {
  const long long vecs = tokens * H * (D / 8);
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < vecs; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int dv = static_cast<int>(i % (D / 8));
    const long long th = i / (D / 8);
    const int h = static_cast<int>(th % H);
    const long long token = th / H;
    const float4 lo = *reinterpret_cast<const float4*>(dq32 + (token * H + h) * D + dv * 8);
    const float4 hi = *reinterpret_cast<const float4*>(dq32 + (token * H + h) * D + dv * 8 + 4);
    *reinterpret_cast<uint4*>(dq + token * ld_dq + dq_col0 + static_cast<long long>(h) * dhead_stride + dv * 8) =
        make_uint4(pack_bf16x2(lo.x * scale, lo.y * scale), pack_bf16x2(lo.z * scale, lo.w * scale), pack_bf16x2(hi.x * scale, hi.y * scale),
                   pack_bf16x2(hi.z * scale, hi.w * scale));
  }
}

}  // namespace fa
}  // namespace sb

// Softmax attention forward.  q, k, v: bf16 matrices with one row per token ([B * S, ld] each; they may be views of the same
// fused projection output), head h of q at columns [q_col0 + h * head_stride, + D).  out: bf16 [B * S, ld_o] with head h at
// columns [h * D, + D).  lse (optional): fp32 [B, H, S].  key_mask (optional): uint8 [B, S], 0 = padding key.
// D is 64 or 128; column offsets multiples of 8; base pointers 16-byte aligned; leading dimensions multiples of 8.
extern "C" int sb_flash_fwd(const void* q, const void* k, const void* v, int ld_q, int ld_k, int ld_v, int q_col0, int k_col0, int v_col0,
                            int head_stride, void* out, int ld_o, float* lse, const unsigned char* key_mask, int B, int H, int S, int D,
                            float scale, int causal, int* status, void* stream) {
  using namespace sb;
  if (B <= 0 || H <= 0 || S <= 0) return 0;
  if (D != 64 && D != 128) return -2;
  if ((reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(k) & 15) || (reinterpret_cast<uintptr_t>(v) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 15))
    return -3;
  if ((ld_q & 7) || (ld_k & 7) || (ld_v & 7) || (ld_o & 7) || (q_col0 & 7) || (k_col0 & 7) || (v_col0 & 7) || (head_stride & 7)) return -3;
  const uint64_t rows = static_cast<uint64_t>(B) * S;
  // the columns the kernel may touch, counted from each operand's own base pointer
  const uint64_t span_q = static_cast<uint64_t>(q_col0) + static_cast<uint64_t>(H - 1) * head_stride + D;
  const uint64_t span_k = static_cast<uint64_t>(k_col0) + static_cast<uint64_t>(H - 1) * head_stride + D;
  const uint64_t span_v = static_cast<uint64_t>(v_col0) + static_cast<uint64_t>(H - 1) * head_stride + D;
  if (span_q > static_cast<uint64_t>(ld_q) || span_k > static_cast<uint64_t>(ld_k) || span_v > static_cast<uint64_t>(ld_v)) return -2;
  CUtensorMap tq, tk, tv;
  int rc = make_tensor_map_bf16(&tq, q, span_q, rows, ld_q, fa::BQ);
  if (rc) return rc;
  rc = make_tensor_map_bf16(&tk, k, span_k, rows, ld_k, fa::BKV);
  if (rc) return rc;
  rc = make_tensor_map_bf16(&tv, v, span_v, rows, ld_v, 64);
  if (rc) return rc;
  fa::FwdParams p{B, H, S, q_col0, k_col0, v_col0, head_stride, ld_o, static_cast<__nv_bfloat16*>(out), lse, key_mask,
                  scale * 1.4426950408889634f, causal, status};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return D == 64 ? fa::launch_fwd<64>(tq, tk, tv, p, st) : fa::launch_fwd<128>(tq, tk, tv, p, st);
}

// Softmax attention backward (head_dim 128).  q, k, v as in sb_flash_fwd; out, dout: bf16 [B * S, H * D] (head h at columns
// [h * D, + D)); lse: fp32 [B, H, S] from the forward.  dq, dk, dv: bf16 matrices with one row per token, head h of each at
// columns [d*_col0 + h * dhead_stride, + D) (they may be three views of one fused gradient matrix).  Scratch: delta fp32
// [B, H, S] and dq32 fp32 [B * S, H * D], which this call clears.
extern "C" int sb_flash_bwd(const void* q, const void* k, const void* v, int ld_q, int ld_k, int ld_v, int q_col0, int k_col0, int v_col0,
                            int head_stride, const void* out, const void* dout, const float* lse, const unsigned char* key_mask, void* dq, void* dk,
                            void* dv, int ld_dq, int ld_dk, int ld_dv, int dq_col0, int dk_col0, int dv_col0, int dhead_stride, float* delta,
                            float* dq32, int B, int H, int S, int D, float scale, int causal, int sms, int* status, void* stream) {
  using namespace sb;
  if (B <= 0 || H <= 0 || S <= 0) return 0;
  if (D != fa::BWD_D) return -2;
  const uintptr_t ptrs[] = {reinterpret_cast<uintptr_t>(q),  reinterpret_cast<uintptr_t>(k),  reinterpret_cast<uintptr_t>(v), reinterpret_cast<uintptr_t>(out),
                            reinterpret_cast<uintptr_t>(dout), reinterpret_cast<uintptr_t>(dq), reinterpret_cast<uintptr_t>(dk), reinterpret_cast<uintptr_t>(dv),
                            reinterpret_cast<uintptr_t>(dq32)};
  for (uintptr_t a : ptrs)
    if (a & 15) return -3;
  const int mults[] = {ld_q, ld_k, ld_v, q_col0, k_col0, v_col0, head_stride, ld_dq, ld_dk, ld_dv, dq_col0, dk_col0, dv_col0, dhead_stride};
  for (int m : mults)
    if (m & 7) return -3;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const uint64_t rows = static_cast<uint64_t>(B) * S;
  const uint64_t span_q = static_cast<uint64_t>(q_col0) + static_cast<uint64_t>(H - 1) * head_stride + D;
  const uint64_t span_k = static_cast<uint64_t>(k_col0) + static_cast<uint64_t>(H - 1) * head_stride + D;
  const uint64_t span_v = static_cast<uint64_t>(v_col0) + static_cast<uint64_t>(H - 1) * head_stride + D;
  if (span_q > static_cast<uint64_t>(ld_q) || span_k > static_cast<uint64_t>(ld_k) || span_v > static_cast<uint64_t>(ld_v)) return -2;
  CUtensorMap tq, tk, tv, tdo;
  int rc = make_tensor_map_bf16(&tq, q, span_q, rows, ld_q, fa::BWD_BQ);
  if (rc) return rc;
  rc = make_tensor_map_bf16(&tk, k, span_k, rows, ld_k, fa::BWD_BK);
  if (rc) return rc;
  rc = make_tensor_map_bf16(&tv, v, span_v, rows, ld_v, fa::BWD_BK);
  if (rc) return rc;
  rc = make_tensor_map_bf16(&tdo, dout, static_cast<uint64_t>(H) * D, rows, static_cast<uint64_t>(H) * D, fa::BWD_BQ);
  if (rc) return rc;
  const long long items = static_cast<long long>(rows) * H;
  fa::attn_delta_kernel<<<static_cast<unsigned>((items + 7) / 8), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(dout),
                                                                                 B, S, H, D, delta);
  cudaError_t e = cudaMemsetAsync(dq32, 0, static_cast<size_t>(rows) * H * D * sizeof(float), st);
  if (e != cudaSuccess) return static_cast<int>(e);
  static PerDeviceOnce once;
  bool* configured = once.slot();
  if (configured == nullptr) return -8;
  if (!*configured) {
    e = cudaFuncSetAttribute(fa::flash_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, fa::BwdPlan::SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    *configured = true;
  }
  fa::BwdParams p{B, H, S, q_col0, k_col0, v_col0, head_stride, lse, delta, dq32, static_cast<__nv_bfloat16*>(dk), static_cast<__nv_bfloat16*>(dv),
                  ld_dk, ld_dv, dk_col0, dv_col0, dhead_stride, scale, scale * 1.4426950408889634f, causal, key_mask, status};
  const int nkt = (S + fa::BWD_BK - 1) / fa::BWD_BK;
  fa::flash_bwd_kernel<<<nkt * B * H, fa::BWD_THREADS, fa::BwdPlan::SMEM_BYTES, st>>>(tq, tk, tv, tdo, p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  const long long vecs = static_cast<long long>(rows) * H * (D / 8);
  long long blocks = (vecs + 255) / 256;
  if (blocks > static_cast<long long>(sms) * 16) blocks = static_cast<long long>(sms) * 16;
  fa::attn_dq_convert_kernel<<<static_cast<unsigned>(blocks), 256, 0, st>>>(dq32, static_cast<long long>(rows), H, D, scale, static_cast<__nv_bfloat16*>(dq),
                                                                            ld_dq, dq_col0, dhead_stride);
  return static_cast<int>(cudaGetLastError());
}
