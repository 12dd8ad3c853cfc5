// bf16 GEMM on CTA pairs: tcgen05.mma.cta_group::2 with a 256 x 256 tile per pair.
//
//   D[M,N] = alpha * A[M,K] * B[N,K]^T (+ bias[N]),  operands K-major or MN-major as in gemm_tc.cu.
//
// Two CTAs of a 2-CTA cluster (an SM pair) work on one tile.  Each stages its own 128 rows of A and its own 128 of the
// tile's 256 B rows, so a k-block costs a CTA 32 KB of shared-memory traffic instead of the 48 KB of the one-CTA
// 128 x 256 tile: the tensor pipe of the one-CTA kernel was busy 75 % of the time waiting on exactly that.
// The even CTA of the pair (the leader) issues every MMA; the instruction reads A and B from the same shared-memory
// offsets of both CTAs and writes 128 accumulator lanes into the tensor memory of each.
//
// Synchronisation (all barriers are mbarriers in shared memory, every wait is bounded):
//   full[s]   in the leader: the leader's producer arrives with expect_tx for the bytes of BOTH CTAs; the TMA loads of
//             both CTAs complete on it (the peer's loads name the leader's barrier: cta_group::2 form of the copy).
//   empty[s]  in each CTA: released by the leader's tcgen05.commit, multicast to both CTAs.
//   tfull[a]  in each CTA: accumulator a is ready (same multicast commit); each CTA's epilogue warps wait on their own.
//   tempty[a] in the leader: 8 arrivals, one per epilogue warp of either CTA (the peer's arrive remotely).
// No TMA multicast is used.  Every role of every CTA reaches the common exit, which ends with a cluster barrier, so
// neither CTA's shared memory disappears while the other may still address it.
#include "common.cuh"

namespace sb {

int make_tensor_map_bf16(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t box_outer);

namespace g2 {

constexpr int TM = 256, TN = 256;   // tile of a CTA pair
constexpr int HM = 128, HN = 128;   // what one CTA stages of it
constexpr int BK = 64, UMMA_K = 16;
constexpr int THREADS = 192;
constexpr int A_BYTES = HM * BK * 2, B_BYTES = HN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int STAGES = 6;
constexpr int EPI_BYTES = 4 * 32 * 128;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + 1024 + 256;
constexpr int TMEM_COLS = 512;      // two 256-column accumulators
constexpr uint32_t PEER_MASK = 0xFEFFFFFFu;  // clears the bit that tells the two CTAs' shared::cluster windows apart

struct Params {
  int M, N, K, ldo, out_mode;  // out_mode 0 = bf16, 1 = fp32
  float alpha;
  void* out;
  const float* bias;
  int* status;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar) & PEER_MASK), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      :
      : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at this shared-memory offset in BOTH CTAs once the MMAs issued so far have completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(smem_u32(bar)),
               "h"(static_cast<uint16_t>(3))
               : "memory");
}
// Arrive on the leader's copy of a barrier from either CTA.
__device__ __forceinline__ void mbar_arrive_leader(uint64_t* bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(smem_u32(bar) & PEER_MASK) : "memory");
}

__device__ __forceinline__ void decode(int tile, int num_m, int num_n, int& m_blk, int& n_blk) {
  constexpr int G = 4;
  const int group = G * num_n;
  const int g = tile / group;
  const int first_m = g * G;
  const int gm = (num_m - first_m) < G ? (num_m - first_m) : G;
  const int r = tile - g * group;
  m_blk = first_m + r % gm;
  n_blk = r / gm;
}

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(THREADS, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_stage = smem + STAGES * STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_stage + EPI_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tmem_full = bars + 2 * STAGES;
  uint64_t* tmem_empty = bars + 2 * STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t crank = cluster_ctarank();
  const bool leader = crank == 0;
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int num_m = (p.M + TM - 1) / TM, num_n = (p.N + TN - 1) / TN;
  const int num_kb = (p.K + BK - 1) / BK;
  const int total_tiles = num_m * num_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 8);  // four epilogue warps in each CTA of the pair
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anything remote can touch them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (one per CTA)
    if (lane == 0) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_b);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int tile = pair; tile < total_tiles && ok; tile += npairs) {
        int m_blk, n_blk;
        decode(tile, num_m, num_n, m_blk, n_blk);
        const int m0 = m_blk * TM + static_cast<int>(crank) * HM;
        const int n0 = n_blk * TN + static_cast<int>(crank) * HN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag, p.status, ST_TIMEOUT_SMEM_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb_ = sa + A_BYTES;
          if (leader) mbar_expect_tx(&full_bar[s], 2 * STAGE_BYTES);  // the bytes of both CTAs land on this barrier
          if (A_MN) {
#pragma unroll
            for (int h = 0; h < HM / 64; ++h) tma_load_2d_pair(sa + h * 8192, &tmap_a, &full_bar[s], m0 + h * 64, kb * BK);
          } else {
            tma_load_2d_pair(sa, &tmap_a, &full_bar[s], kb * BK, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int h = 0; h < HN / 64; ++h) tma_load_2d_pair(sb_ + h * 8192, &tmap_b, &full_bar[s], n0 + h * 64, kb * BK);
          } else {
            tma_load_2d_pair(sb_, &tmap_b, &full_bar[s], kb * BK, n0);
          }
          if (++s == STAGES) {
            s = 0;
            ph ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (leader && lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(TM, TN, A_MN, B_MN);
      int s = 0;
      uint32_t ph = 0;
      int local = 0;
      bool ok = true;
      for (int tile = pair; tile < total_tiles && ok; tile += npairs, ++local) {
        const int acc = local & 1;
        const uint32_t acc_ph = (local >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_ph ^ 1u, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * TN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[s], ph, abort_flag, p.status, ST_TIMEOUT_SMEM_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sb_ = sa + A_BYTES;
#pragma unroll
          for (int j = 0; j < BK / UMMA_K; ++j) {
            const uint64_t adesc = A_MN ? make_smem_desc_sw128(sa + j * 2048, 8192, 1024) : make_smem_desc_sw128(sa + j * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc_sw128(sb_ + j * 2048, 8192, 1024) : make_smem_desc_sw128(sb_ + j * 32, 16, 1024);
            umma_bf16_pair(d_tmem, adesc, bdesc, idesc, (kb > 0 || j > 0) ? 1u : 0u);
          }
          umma_commit_pair(&empty_bar[s]);  // frees this stage in both CTAs once the MMAs have read it
          if (++s == STAGES) {
            s = 0;
            ph ^= 1u;
          }
        }
        if (ok) umma_commit_pair(&tmem_full[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps (2..5) of both CTAs
    const int quad = warp & 3;
    int local = 0;
    bool ok = true;
    uint4* my_stage = reinterpret_cast<uint4*>(epi_stage) + quad * (32 * 8);
    const bool staged = p.out_mode == 0 && (p.ldo % 8 == 0) && (p.N % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0);
    for (int tile = pair; tile < total_tiles && ok; tile += npairs, ++local) {
      int m_blk, n_blk;
      decode(tile, num_m, num_n, m_blk, n_blk);
      const int acc = local & 1;
      const uint32_t acc_ph = (local >> 1) & 1;
      if (!mbar_wait(&tmem_full[acc], acc_ph, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int row_base = m_blk * TM + static_cast<int>(crank) * HM + quad * 32;
      const int row = row_base + lane;
      const bool row_ok = row < p.M;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * TN;
      // Two chunks of 16 accumulator columns are in flight: the TMEM load of chunk c + 1 is issued before chunk c is
      // processed, and the chunk's 16 bias values are fetched (four 16-byte loads, or guarded scalars at the edge) before
      // the wait, so that neither latency sits on the critical path of this warp (with K = 2048 the epilogue of a tile
      // takes as long as its main loop: bias cost 20 % of the kernel before).
      auto load_bias = [&](int c, float (&bv)[16]) {
        const int col0 = n_blk * TN + c * 16;
        if (p.bias == nullptr) {
#pragma unroll
          for (int i = 0; i < 16; ++i) bv[i] = 0.f;
        } else if (col0 + 16 <= p.N && ((reinterpret_cast<uintptr_t>(p.bias) & 15) == 0)) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            const float4 t = __ldg(reinterpret_cast<const float4*>(p.bias + col0) + q4);
            bv[4 * q4] = t.x; bv[4 * q4 + 1] = t.y; bv[4 * q4 + 2] = t.z; bv[4 * q4 + 3] = t.w;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) bv[i] = (col0 + i < p.N) ? __ldg(p.bias + col0 + i) : 0.f;
        }
      };
      auto process = [&](int c, const uint32_t (&v)[16], const float (&bv)[16]) {
        const int col0 = n_blk * TN + c * 16;
        float f[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          f[i] = fmaf(__uint_as_float(v[i]), p.alpha, bv[i]);
        }
        if (staged) {
          const int cu = (c * 2) % 8;
          my_stage[lane * 8 + (cu ^ (lane & 7))] = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
          my_stage[lane * 8 + ((cu + 1) ^ (lane & 7))] = make_uint4(pack_bf16x2(f[8], f[9]), pack_bf16x2(f[10], f[11]), pack_bf16x2(f[12], f[13]), pack_bf16x2(f[14], f[15]));
          if ((c & 3) != 3) return;  // 64 columns make a group
          __syncwarp();
          const int gcol0 = n_blk * TN + (c - 3) * 16;
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int idx = it * 32 + lane;
            const int r = idx >> 3, u = idx & 7;
            const int grow = row_base + r, gcol = gcol0 + u * 8;
            if (grow < p.M && gcol < p.N)
              *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(grow) * p.ldo + gcol) = my_stage[r * 8 + (u ^ (r & 7))];
          }
          __syncwarp();
          return;
        }
        if (!row_ok || col0 >= p.N) return;
        const bool full = (col0 + 16 <= p.N);
        if (p.out_mode == 0) {
          __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(row) * p.ldo + col0;
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (col0 + i < p.N) o[i] = __float2bfloat16_rn(f[i]);
        } else {
          float* o = reinterpret_cast<float*>(p.out) + static_cast<size_t>(row) * p.ldo + col0;
          if (full && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
#pragma unroll
            for (int i = 0; i < 4; ++i) reinterpret_cast<float4*>(o)[i] = make_float4(f[4 * i], f[4 * i + 1], f[4 * i + 2], f[4 * i + 3]);
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (col0 + i < p.N) o[i] = f[i];
          }
        }
      };
      uint32_t va[16], vb[16];
      float ba[16], bb[16];
      tmem_ld_x16(t_row, va);
      load_bias(0, ba);
#pragma unroll 1
      for (int c = 0; c < TN / 16; c += 2) {
        tmem_ld_wait();                                   // chunk c is in va
        tmem_ld_x16(t_row + (c + 1) * 16, vb);
        load_bias(c + 1, bb);
        process(c, va, ba);
        tmem_ld_wait();                                   // chunk c + 1 is in vb
        if (c + 2 < TN / 16) {
          tmem_ld_x16(t_row + (c + 2) * 16, va);
          load_bias(c + 2, ba);
        }
        process(c + 1, vb, bb);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_leader(&tmem_empty[acc]);
    }
  }

  // Common exit.  After an abandoned wait, give copies that may still be in flight time to land.
  __syncwarp();
  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer has issued its last access to this CTA's shared memory and barriers
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

template <bool A_MN, bool B_MN>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const Params& p, int sms, cudaStream_t stream) {
  static PerDeviceOnce once;
  bool* configured = once.slot();
  if (configured == nullptr) return -8;
  auto kern = gemm2_bf16_kernel<A_MN, B_MN>;
  if (!*configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    *configured = true;
  }
  const int tiles = ((p.M + TM - 1) / TM) * ((p.N + TN - 1) / TN);
  int pairs = sms / 2;
  if (pairs > tiles) pairs = tiles;
  if (pairs < 1) pairs = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(THREADS, 1, 1);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return static_cast<int>(cudaLaunchKernelEx(&cfg, kern, ta, tb, p));
}

}  // namespace g2
}  // namespace sb

// Same contract as sb_gemm_bf16 restricted to out_mode 0 (bf16) / 1 (fp32), no split-K, 256 x 256 pair tiles.
extern "C" int sb_gemm_bf16_2cta(const void* A, const void* B, void* out, const float* bias, int M, int N, int K, int lda, int ldb, int ldo,
                                 int a_mn, int b_mn, int out_mode, float alpha, int sms, int* status, void* stream) {
  using namespace sb;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda & 7) || (ldb & 7)) return -3;
  if (out_mode < 0 || out_mode > 1) return -7;
  CUtensorMap ta, tb;
  int rc = a_mn ? make_tensor_map_bf16(&ta, A, M, K, lda, 64) : make_tensor_map_bf16(&ta, A, K, M, lda, g2::HM);
  if (rc) return rc;
  rc = b_mn ? make_tensor_map_bf16(&tb, B, N, K, ldb, 64) : make_tensor_map_bf16(&tb, B, K, N, ldb, g2::HN);
  if (rc) return rc;
  g2::Params p{M, N, K, ldo, out_mode, alpha, out, bias, status};
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (!a_mn && !b_mn) return g2::launch<false, false>(ta, tb, p, sms, st);
  if (!a_mn && b_mn) return g2::launch<false, true>(ta, tb, p, sms, st);
  if (a_mn && !b_mn) return g2::launch<true, false>(ta, tb, p, sms, st);
  return g2::launch<true, true>(ta, tb, p, sms, st);
}
