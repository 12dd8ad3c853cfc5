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
//   PV_DONE    P_j V_j is complete (commit, one phase per tile): read by the V producer, by a softmax thread that has to
//              rescale the output accumulator, and by the epilogue
enum Bar { QK_GO = 0, PV_GO = 2, S_FULL = 4, PV_DONE = 6, NBARS = 8 };

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
        // stage s is free once P_{j-2} V_{j-2} is complete (one phase of PV_DONE per tile, waited for in order)
        if (j >= 2 && !wait_on(&bars[PV_DONE], (j - 2) & 1, abort_flag, p.status, ST_TIMEOUT_SMEM_EMPTY)) break;
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
        umma_commit(&bars[PV_DONE]);
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
        // P_{j-1} V_{j-1} must have finished before the output accumulator is touched.  (Phase j - 1 of the barrier is
        // the only one that can still be open here, so skipping this wait on other tiles leaves the parity unambiguous.)
        if (j > 0 && !wait_on(&bars[PV_DONE], (j - 1) & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
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
    if (ok && nkv > 0) ok = wait_on(&bars[PV_DONE], (nkv - 1) & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL);
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
