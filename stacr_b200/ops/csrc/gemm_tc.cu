// Persistent, warp-specialised bf16 GEMM for sm_100a: TMA -> shared memory (128B swizzle) ->
// tcgen05.mma with fp32 accumulators in TMEM -> tcgen05.ld epilogue.
//
//   D[M,N] = alpha * A[M,K] * B[N,K]^T (+ bias[N])
//
// Either operand may be "K-major" (the reduction index is contiguous in memory, e.g. the
// activations X[rows, in] and the weight W[out, in] of a forward linear) or "MN-major"
// (the output index is contiguous, e.g. W[out, in] as the B operand of dX = dY * W, or
// dY[rows, out] as the A operand of dY^T * C).  That covers every contraction of the
// compressed linear layer (forward, input gradient, projection, skinny A^T*B for the basis
// update and the low-rank weight-gradient chain) without materialising a transpose.
//
// CTA layout (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner,
// warps 2..5 = epilogue (each reads the 32 TMEM lanes its warp id modulo 4 may access).
// The accumulator is double-buffered in TMEM so the epilogue of tile i overlaps the main
// loop of tile i+1.  Split-K tiles reduce with fp32 atomics.
//
// Replaces the library GEMMs the reference issues from its autograd function
// (stacr/layers.py:128-137 and :168-173 of the reference project).
#include <cstdio>

#include "common.cuh"

namespace sb {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int GEMM_THREADS = 192;

struct GemmParams {
  int M, N, K;
  int splits;      // split-K factor (>=1); every split owns >=1 k-block
  int kb_per;      // k-blocks per split
  int ldo;         // leading dimension of the output (elements)
  int out_mode;    // 0 = bf16 store, 1 = fp32 store, 2 = fp32 atomic add, 3 = bf16 store into this rank's slot of every rank's staging buffer
  float alpha;
  void* out;
  const float* bias;  // optional, length N (added by split 0 only)
  int* status;
  // out_mode 3: the staging buffer is symmetric memory holding `world` slots of M x ldo bf16; this rank's partial tile
  // is stored into slot `slot_off` (bytes) of all `world` copies, through one multicast address or the peer pointers.
  int world;
  unsigned long long slot_off;
  unsigned long long mc_out;         // multicast address of the buffer, 0 = use peer_out
  unsigned long long peer_out[8];    // every rank's copy as mapped on this GPU
};

__device__ __forceinline__ void multimem_st_v4(void* addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(__uint_as_float(a)), "f"(__uint_as_float(b)),
               "f"(__uint_as_float(c)), "f"(__uint_as_float(d))
               : "memory");
}

template <int BN>
struct GemmCfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int MAX_SMEM = 200 * 1024;
  static constexpr int STAGES_RAW = MAX_SMEM / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int TMEM_COLS = (2 * BN <= 32) ? 32 : (2 * BN <= 64) ? 64 : (2 * BN <= 128) ? 128 : (2 * BN <= 256) ? 256 : 512;
  static constexpr int EPI_BYTES = 4 * 32 * 128;  // per epilogue warp: 32 rows x 64 bf16 columns
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
};

__device__ __forceinline__ void decode_tile(int tile, int num_m, int num_n, int& m_blk, int& n_blk,
                                            int& sp) {
  const int per_split = num_m * num_n;
  sp = tile / per_split;
  int t = tile - sp * per_split;
  constexpr int G = 8;  // m-blocks per raster group: neighbouring CTAs share A/B panels in L2
  const int group = G * num_n;
  const int g = t / group;
  const int first_m = g * G;
  const int gm = (num_m - first_m) < G ? (num_m - first_m) : G;
  const int r = t - g * group;
  m_blk = first_m + r % gm;
  n_blk = r / gm;
}

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const GemmParams p) {
  using Cfg = GemmCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_stage = smem + STAGES * Cfg::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_stage + Cfg::EPI_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tmem_full = bars + 2 * STAGES;
  uint64_t* tmem_empty = bars + 2 * STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = (p.M + BM - 1) / BM;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_kb = (p.K + BK - 1) / BK;
  const int total_tiles = num_m * num_n * p.splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 4);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_b);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        int m_blk, n_blk, sp;
        decode_tile(tile, num_m, num_n, m_blk, n_blk, sp);
        const int kb0 = sp * p.kb_per;
        const int kb1 = min(num_kb, kb0 + p.kb_per);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag, p.status, ST_TIMEOUT_SMEM_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + s * Cfg::STAGE_BYTES;
          uint8_t* sb_ = sa + Cfg::A_BYTES;
          mbar_expect_tx(&full_bar[s], Cfg::STAGE_BYTES);
          if (A_MN) {
#pragma unroll
            for (int h = 0; h < BM / 64; ++h)
              tma_load_2d(sa + h * 8192, &tmap_a, &full_bar[s], m_blk * BM + h * 64, kb * BK);
          } else {
            tma_load_2d(sa, &tmap_a, &full_bar[s], kb * BK, m_blk * BM);
          }
          if (B_MN) {
#pragma unroll
            for (int h = 0; h < BN / 64; ++h)
              tma_load_2d(sb_ + h * 8192, &tmap_b, &full_bar[s], n_blk * BN + h * 64, kb * BK);
          } else {
            tma_load_2d(sb_, &tmap_b, &full_bar[s], kb * BK, n_blk * BN);
          }
          if (++s == STAGES) {
            s = 0;
            ph ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      int s = 0;
      uint32_t ph = 0;
      int local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
        int m_blk, n_blk, sp;
        decode_tile(tile, num_m, num_n, m_blk, n_blk, sp);
        const int kb0 = sp * p.kb_per;
        const int kb1 = min(num_kb, kb0 + p.kb_per);
        const int acc = local & 1;
        const uint32_t acc_ph = (local >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_ph ^ 1u, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[s], ph, abort_flag, p.status, ST_TIMEOUT_SMEM_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * Cfg::STAGE_BYTES);
          const uint32_t sb_ = sa + Cfg::A_BYTES;
#pragma unroll
          for (int j = 0; j < BK / UMMA_K; ++j) {
            const uint64_t adesc = A_MN ? make_smem_desc_sw128(sa + j * 2048, 8192, 1024)
                                        : make_smem_desc_sw128(sa + j * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc_sw128(sb_ + j * 2048, 8192, 1024)
                                        : make_smem_desc_sw128(sb_ + j * 32, 16, 1024);
            umma_bf16(d_tmem, adesc, bdesc, idesc, (kb > kb0 || j > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[s]);  // frees the smem stage once these MMAs have read it
          if (++s == STAGES) {
            s = 0;
            ph ^= 1u;
          }
        }
        if (ok) umma_commit(&tmem_full[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps (2..5)
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    int local = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
      int m_blk, n_blk, sp;
      decode_tile(tile, num_m, num_n, m_blk, n_blk, sp);
      const int acc = local & 1;
      const uint32_t acc_ph = (local >> 1) & 1;
      if (!mbar_wait(&tmem_full[acc], acc_ph, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int row = m_blk * BM + quad * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN;
      const bool add_bias = (p.bias != nullptr) && (sp == 0);
      // bf16 outputs whose rows are 16-byte aligned go through shared memory: every lane owns one ROW of the
      // accumulator, so direct stores would be 32-byte pieces 2*ldo bytes apart; staged, a warp writes whole
      // 128-byte row segments (8 lanes x 16 bytes), which is what peer writes over NVLink need.
      constexpr int GW = BN < 64 ? BN : 64;          // columns per staged group
      constexpr int UNITS = GW / 8;                  // 16-byte units per staged row
      const bool staged = (p.out_mode == 0 || p.out_mode == 3) && (p.ldo % 8 == 0) && (p.N % 8 == 0) &&
                          ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0);
      uint4* my_stage = reinterpret_cast<uint4*>(epi_stage) + quad * (32 * 8);
      // Two chunks of 16 accumulator columns are in flight: the TMEM load of chunk c + 1 is issued before chunk c is
      // processed, and a chunk's 16 bias values are fetched (four 16-byte loads, or guarded scalars at the edge) before
      // the wait, so that neither latency sits on the critical path of this warp.
      constexpr int NCH = BN / 16;
      auto load_bias = [&](int c, float (&bv)[16]) {
        const int col0 = n_blk * BN + c * 16;
        if (!add_bias) {
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
        const int col0 = n_blk * BN + c * 16;
        if (!staged && col0 >= p.N) return;  // warp-uniform
        float f[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          f[i] = fmaf(__uint_as_float(v[i]), p.alpha, bv[i]);
        }
        if (staged) {
          const int cu = (c * 2) % UNITS;  // first 16-byte unit of this chunk inside the staged row
          my_stage[lane * 8 + ((cu) ^ (lane & 7))] = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
          my_stage[lane * 8 + ((cu + 1) ^ (lane & 7))] = make_uint4(pack_bf16x2(f[8], f[9]), pack_bf16x2(f[10], f[11]), pack_bf16x2(f[12], f[13]), pack_bf16x2(f[14], f[15]));
          if (((c + 1) * 16) % GW != 0) return;  // group not complete yet
          __syncwarp();
          const int gcol0 = n_blk * BN + (c * 16 + 16 - GW);  // first column of the group
          const int row_base = m_blk * BM + quad * 32;
#pragma unroll
          for (int it = 0; it < (32 * UNITS) / 32; ++it) {
            const int idx = it * 32 + lane;
            const int r = idx / UNITS, u = idx % UNITS;
            const int grow = row_base + r, gcol = gcol0 + u * 8;
            if (grow < p.M && gcol < p.N) {
              const uint4 w = my_stage[r * 8 + (u ^ (r & 7))];
              const size_t eoff = (static_cast<size_t>(grow) * p.ldo + gcol) * 2;
              if (p.out_mode == 0) {
                *reinterpret_cast<uint4*>(reinterpret_cast<char*>(p.out) + eoff) = w;
              } else if (p.mc_out != 0) {
                multimem_st_v4(reinterpret_cast<char*>(p.mc_out) + p.slot_off + eoff, w.x, w.y, w.z, w.w);
              } else {
                for (int pr = 0; pr < p.world; ++pr)
                  *reinterpret_cast<uint4*>(reinterpret_cast<char*>(p.peer_out[pr]) + p.slot_off + eoff) = w;
              }
            }
          }
          __syncwarp();
          return;
        }
        if (!row_ok) return;
        const bool full = (col0 + 16 <= p.N);
        if (p.out_mode == 0) {
          __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(row) * p.ldo + col0;
          if (full && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
            uint4 w0 = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
            uint4 w1 = make_uint4(pack_bf16x2(f[8], f[9]), pack_bf16x2(f[10], f[11]), pack_bf16x2(f[12], f[13]), pack_bf16x2(f[14], f[15]));
            reinterpret_cast<uint4*>(o)[0] = w0;
            reinterpret_cast<uint4*>(o)[1] = w1;
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (col0 + i < p.N) o[i] = __float2bfloat16_rn(f[i]);
          }
        } else if (p.out_mode == 1) {
          float* o = reinterpret_cast<float*>(p.out) + static_cast<size_t>(row) * p.ldo + col0;
          if (full && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
              reinterpret_cast<float4*>(o)[i] = make_float4(f[4 * i], f[4 * i + 1], f[4 * i + 2], f[4 * i + 3]);
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (col0 + i < p.N) o[i] = f[i];
          }
        } else if (p.out_mode == 2) {
          float* o = reinterpret_cast<float*>(p.out) + static_cast<size_t>(row) * p.ldo + col0;
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (col0 + i < p.N) atomicAdd(o + i, f[i]);
        } else {
          // all-reduce fused into the epilogue, first half: this rank's partial tile goes into its own slot of every
          // rank's staging buffer with plain 16-byte stores (posted writes over NVLink; no atomics).  The sum over the
          // slots is taken locally by sb_allreduce_finish once every rank has stored.
          // (the launcher guarantees N % 16 == 0 and 16-byte aligned rows for this mode)
          const size_t off = p.slot_off + (static_cast<size_t>(row) * p.ldo + col0) * 2;
          const uint32_t w[8] = {pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]),
                                 pack_bf16x2(f[8], f[9]), pack_bf16x2(f[10], f[11]), pack_bf16x2(f[12], f[13]), pack_bf16x2(f[14], f[15])};
          if (p.mc_out != 0) {
            char* dst = reinterpret_cast<char*>(p.mc_out) + off;
            multimem_st_v4(dst, w[0], w[1], w[2], w[3]);
            multimem_st_v4(dst + 16, w[4], w[5], w[6], w[7]);
          } else {
            for (int r = 0; r < p.world; ++r) {
              uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<char*>(p.peer_out[r]) + off);
              dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
              dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
            }
          }
        }
      };
      uint32_t va[16], vb[16];
      float ba[16], bb[16];
      tmem_ld_x16(t_row, va);
      load_bias(0, ba);
#pragma unroll 1
      for (int c = 0; c < NCH; c += 2) {
        tmem_ld_wait();                                   // chunk c is in va
        if (c + 1 < NCH) {
          tmem_ld_x16(t_row + (c + 1) * 16, vb);
          load_bias(c + 1, bb);
        }
        process(c, va, ba);
        if (c + 1 < NCH) {
          tmem_ld_wait();                                 // chunk c + 1 is in vb
          if (c + 2 < NCH) {
            tmem_ld_x16(t_row + (c + 2) * 16, va);
            load_bias(c + 2, ba);
          }
          process(c + 1, vb, bb);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
    }
  }

  // Common exit.  After an abandoned wait, give copies that may still be in flight time to
  // land in this CTA's shared memory before it is released.
  __syncwarp();
  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------ host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// 2-D bf16 row-major tensor [outer, inner] with leading dimension ld (elements); box = {64, box_outer}.
static int make_map(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld,
                    uint32_t box_outer) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {64, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_ERROR_INVALID_CONTEXT) {
    // the driver entry point wants a current context, and a thread that has made no runtime call yet (an autograd worker
    // whose first CUDA work is this launch) has none bound: bind the device's primary context and encode again
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && cudaSetDevice(dev) == cudaSuccess && cudaFree(nullptr) == cudaSuccess)
      r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  if (r != CUDA_SUCCESS)   // rare and always a caller error: say which argument set the driver refused
    fprintf(stderr, "stacr_b200: cuTensorMapEncodeTiled failed (%d): ptr=%p inner=%llu outer=%llu ld=%llu box_outer=%u\n", static_cast<int>(r), ptr,
            static_cast<unsigned long long>(inner), static_cast<unsigned long long>(outer), static_cast<unsigned long long>(ld), box_outer);
  return r == CUDA_SUCCESS ? 0 : -2;
}

// The same encoder for the other translation units of the library.
int make_tensor_map_bf16(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t box_outer) {
  return make_map(map, ptr, inner, outer, ld, box_outer);
}

template <int BN, bool A_MN, bool B_MN>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int sms,
                       cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  static PerDeviceOnce once;
  bool* configured = once.slot();
  if (configured == nullptr) return -8;
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN>;
  if (!*configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    *configured = true;
  }
  const int num_m = (p.M + BM - 1) / BM, num_n = (p.N + BN - 1) / BN;
  const int total = num_m * num_n * p.splits;
  const int grid = total < sms ? total : sms;
  kern<<<grid, GEMM_THREADS, Cfg::SMEM_BYTES, stream>>>(ta, tb, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace sb

// D[M,N] = alpha * op(A) * op(B)^T + bias.
//   a_mn = 0: A is row-major [M, K] (ld = lda);  a_mn = 1: A is row-major [K, M].
//   b_mn = 0: B is row-major [N, K] (ld = ldb);  b_mn = 1: B is row-major [K, N].
//   out_mode 0 bf16 / 1 fp32 / 2 fp32 atomic add (required when splits > 1; caller zeroes out).
//   bn = tile width: 16, 32, 64, 128 or 256.
// Alignment: base pointers 16-byte aligned, lda/ldb multiples of 8 elements.
static int gemm_entry(const void* A, const void* B, void* out, const float* bias, int M, int N, int K, int lda, int ldb, int ldo,
                      int a_mn, int b_mn, int out_mode, int splits, int bn, float alpha, int sms, int* status, void* stream,
                      int world, unsigned long long mc_out, const unsigned long long* peer_out, unsigned long long slot_off) {
  using namespace sb;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda & 7) || (ldb & 7))
    return -3;
  if (splits > 1 && out_mode != 2) return -4;
  CUtensorMap ta, tb;
  int rc;
  if (a_mn) rc = make_map(&ta, A, M, K, lda, 64);
  else rc = make_map(&ta, A, K, M, lda, BM);
  if (rc) return rc;
  if (b_mn) rc = make_map(&tb, B, N, K, ldb, 64);
  else rc = make_map(&tb, B, K, N, ldb, bn);
  if (rc) return rc;
  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  const int num_kb = (K + BK - 1) / BK;
  if (splits < 1) splits = 1;
  if (splits > num_kb) splits = num_kb;
  p.kb_per = (num_kb + splits - 1) / splits;
  p.splits = (num_kb + p.kb_per - 1) / p.kb_per;
  p.ldo = ldo; p.out_mode = out_mode; p.alpha = alpha; p.out = out; p.bias = bias; p.status = status;
  p.world = world; p.mc_out = mc_out; p.slot_off = slot_off;
  for (int r = 0; r < 8; ++r) p.peer_out[r] = (peer_out != nullptr && r < world) ? peer_out[r] : 0ull;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
#define SB_DISPATCH(BN_)                                                              \
  if (bn == BN_) {                                                                     \
    if (!a_mn && !b_mn) return launch_gemm<BN_, false, false>(ta, tb, p, sms, st);     \
    if (!a_mn && b_mn) return launch_gemm<BN_, false, true>(ta, tb, p, sms, st);       \
    if (a_mn && !b_mn) return launch_gemm<BN_, true, false>(ta, tb, p, sms, st);       \
    return launch_gemm<BN_, true, true>(ta, tb, p, sms, st);                           \
  }
  SB_DISPATCH(256)
  SB_DISPATCH(128)
  SB_DISPATCH(64)
#undef SB_DISPATCH
  // Narrow tiles carry K-major B only (B is a small padded [bn, K] panel).
  if (b_mn) return -5;
  if (bn == 32) return a_mn ? launch_gemm<32, true, false>(ta, tb, p, sms, st) : launch_gemm<32, false, false>(ta, tb, p, sms, st);
  if (bn == 16) return a_mn ? launch_gemm<16, true, false>(ta, tb, p, sms, st) : launch_gemm<16, false, false>(ta, tb, p, sms, st);
  return -6;
}

extern "C" int sb_gemm_bf16(const void* A, const void* B, void* out, const float* bias, int M, int N, int K,
                            int lda, int ldb, int ldo, int a_mn, int b_mn, int out_mode, int splits,
                            int bn, float alpha, int sms, int* status, void* stream) {
  if (out_mode < 0 || out_mode > 2) return -7;
  return gemm_entry(A, B, out, bias, M, N, K, lda, ldb, ldo, a_mn, b_mn, out_mode, splits, bn, alpha, sms, status, stream, 1, 0ull, nullptr, 0ull);
}

// First half of a GEMM + all-reduce: every rank calls it with its partial operands and the epilogue stores the bf16
// tile into slot `rank` of the staging buffer of each of the `world` ranks (one multimem.st through the NVSwitch
// multicast address mc_out, or one plain store per peer pointer when mc_out == 0).  A staging buffer holds `world`
// slots of M x N bf16 (slot r at byte offset r * M * N * 2).  sb_allreduce_finish sums the slots once all ranks have
// stored.  peer_out is a HOST array of `world` (<= 8) staging addresses.  N % 16 == 0.  A bias (fp32, length N) is
// added to this rank's partial tile, so exactly one rank should pass it.
extern "C" int sb_gemm_bf16_allreduce(const void* A, const void* B, const float* bias, int M, int N, int K, int lda, int ldb,
                                      int a_mn, int b_mn, int bn, float alpha, int sms, int rank, int world, unsigned long long mc_out,
                                      const unsigned long long* peer_out, int* status, void* stream) {
  if (world < 1 || world > 8 || rank < 0 || rank >= world || (mc_out == 0 && peer_out == nullptr)) return -8;
  if (N % 16) return -9;
  const unsigned long long slot = static_cast<unsigned long long>(rank) * M * N * 2ull;
  void* out = reinterpret_cast<void*>(peer_out ? peer_out[rank] : mc_out);  // only its alignment is looked at
  return gemm_entry(A, B, out, bias, M, N, K, lda, ldb, N, a_mn, b_mn, 3, 1, bn, alpha, sms, status, stream, world, mc_out, peer_out, slot);
}
