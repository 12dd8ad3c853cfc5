// All-reduce over NVLink peer memory, written for gradient buffers that live in symmetric memory
// (every rank can address every rank's copy; optionally one NVSwitch multicast address maps all
// copies).  One kernel does start barrier -> reduce -> broadcast -> end barrier:
//
//   two-shot, peer loads/stores: rank r owns slice r of [lo, hi); for each 16-byte element of
//     its slice it loads the W copies (one local, W-1 over NVLink), adds, scales and stores the
//     result into all W copies.  Per rank (W-1)/W of the bytes cross NVLink in each direction.
//   multimem: the same slice ownership, but the W-way add is one `multimem.ld_reduce` executed
//     in the switch and the broadcast is one `multimem.st`.
//
// Barriers are epoch-tagged flag words in a second symmetric buffer: CTA b of rank A publishes
// flags[phase][b][A] = epoch into every peer with a system-scope release store, and waits with
// acquire loads until its own flags[phase][b][*] reach the epoch.  Every wait is bounded; on
// timeout the kernel records a status code and returns, and the host raises.
// The grid is at most one CTA per SM so all CTAs of all ranks are co-resident.
// Replaces the NCCL all-reduce that DistributedDataParallel issues for the reference
// (experiments/benchmarks/distributed_data.py:87-97 there).
#include "common.cuh"
#include <cstdlib>

namespace sb {

constexpr int MAX_RANKS = 16;
constexpr int MAX_CTAS = 160;

struct CommArgs {
  const unsigned long long* peer_ptrs;   // [world] base address of every rank's buffer (as mapped here)
  const unsigned long long* flag_ptrs;   // [world] base address of every rank's flag buffer
  unsigned long long mc_ptr;             // multicast address of the buffer (0 = none)
  int rank, world;
  long long lo, hi;                      // element range (fp32), 4-element aligned
  float scale;
  int epoch;
  int* status;
  unsigned long long wait_ns;            // how long a flag wait may last before the kernel gives up
  const int* epoch_ptr;                  // optional: the barrier epoch is read from device memory (CUDA-graph replays)
};

// The barrier epoch of this launch.  Kernel arguments are frozen when a step is captured into a CUDA graph, so a replayed
// collective reads its epoch from a device counter that a one-thread kernel in front of it advances (sb_epoch_bump).
__device__ __forceinline__ int epoch_of(const CommArgs& a) {
  return a.epoch_ptr ? *reinterpret_cast<const volatile int*>(a.epoch_ptr) : a.epoch;
}
__global__ void epoch_bump_kernel(int* counter) { *counter += 1; }

// Limit of the peer waits: 2 s unless STACR_WAIT_LIMIT_MS names another value (read once) or sb_comm_set_wait_limit_ns
// was called.  Jobs whose ranks can legitimately drift further apart (a first-use build, a rank-0-only checkpoint that is
// not fenced by a host barrier) raise it; tests that let a wait run out lower it.
static unsigned long long g_comm_wait_ns = 0;
static unsigned long long comm_wait_ns() {
  if (g_comm_wait_ns == 0) {
    unsigned long long ns = SB_WAIT_LIMIT_NS;
    if (const char* env = getenv("STACR_WAIT_LIMIT_MS")) {
      const long long ms = atoll(env);
      if (ms > 0) ns = static_cast<unsigned long long>(ms) * 1000000ull;
    }
    g_comm_wait_ns = ns;
  }
  return g_comm_wait_ns;
}

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// All threads of the CTA call this.  Returns false when a peer did not arrive in time.
__device__ bool rank_barrier(const CommArgs& a, int phase, int* s_fail) {
  __syncthreads();
  if (threadIdx.x < a.world) {
    const int peer = threadIdx.x;
    __threadfence_system();
    int* remote = reinterpret_cast<int*>(a.flag_ptrs[peer]) + (phase * MAX_CTAS + blockIdx.x) * MAX_RANKS + a.rank;
    const int epoch = epoch_of(a);
    st_release_sys(remote, epoch);
    const int* local = reinterpret_cast<const int*>(a.flag_ptrs[a.rank]) + (phase * MAX_CTAS + blockIdx.x) * MAX_RANKS + peer;
    const uint64_t t0 = globaltimer_ns();
    uint32_t polls = 0;
    while (ld_acquire_sys(local) < epoch) {
      if ((++polls & 255u) == 0u && globaltimer_ns() - t0 > a.wait_ns) {
        *s_fail = 1;
        if (a.status) atomicCAS(a.status, 0, ST_TIMEOUT_PEER_FLAG);
        break;
      }
    }
  }
  __syncthreads();
  return *s_fail == 0;
}

__device__ __forceinline__ void slice_of(const CommArgs& a, long long& begin, long long& end) {
  const long long vecs = (a.hi - a.lo) / 4;
  const long long per = (vecs + a.world - 1) / a.world;
  begin = min(vecs, per * a.rank);
  end = min(vecs, begin + per);
}

__global__ void __launch_bounds__(512) allreduce_two_shot_kernel(const CommArgs a) {
  __shared__ int s_fail;
  __shared__ unsigned long long s_peers[MAX_RANKS];
  if (threadIdx.x == 0) s_fail = 0;
  if (threadIdx.x < a.world) s_peers[threadIdx.x] = a.peer_ptrs[threadIdx.x];
  __syncthreads();
  if (!rank_barrier(a, 0, &s_fail)) return;
  long long begin, end;
  slice_of(a, begin, end);
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  constexpr int UNROLL = 8;  // independent 16-byte elements in flight per thread
  for (long long i0 = begin + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < end; i0 += stride * UNROLL) {
    float4 acc[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int p = 0; p < a.world; ++p) {
      const int src = (a.rank + p) % a.world;  // start at the local copy, spread peer traffic
      const float4* base = reinterpret_cast<const float4*>(s_peers[src]) + a.lo / 4;
      float4 v[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const long long i = i0 + u * stride;
        v[u] = i < end ? base[i] : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        acc[u].x += v[u].x; acc[u].y += v[u].y; acc[u].z += v[u].z; acc[u].w += v[u].w;
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      acc[u].x *= a.scale; acc[u].y *= a.scale; acc[u].z *= a.scale; acc[u].w *= a.scale;
    }
    for (int p = 0; p < a.world; ++p) {
      const int dst = (a.rank + p) % a.world;
      float4* base = reinterpret_cast<float4*>(s_peers[dst]) + a.lo / 4;
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const long long i = i0 + u * stride;
        if (i < end) base[i] = acc[u];
      }
    }
  }
  rank_barrier(a, 1, &s_fail);
}

__global__ void __launch_bounds__(512) allreduce_multimem_kernel(const CommArgs a) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  if (!rank_barrier(a, 0, &s_fail)) return;
  long long begin, end;
  slice_of(a, begin, end);
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  constexpr int UNROLL = 8;
  for (long long i0 = begin + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < end; i0 += stride * UNROLL) {
    float x[UNROLL], y[UNROLL], z[UNROLL], w[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long i = i0 + u * stride;
      if (i < end) {
        float* addr = reinterpret_cast<float*>(a.mc_ptr) + a.lo + i * 4;
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                     : "=f"(x[u]), "=f"(y[u]), "=f"(z[u]), "=f"(w[u])
                     : "l"(addr)
                     : "memory");
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long i = i0 + u * stride;
      if (i < end) {
        float* addr = reinterpret_cast<float*>(a.mc_ptr) + a.lo + i * 4;
        asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(x[u] * a.scale),
                     "f"(y[u] * a.scale), "f"(z[u] * a.scale), "f"(w[u] * a.scale)
                     : "memory");
      }
    }
  }
  rank_barrier(a, 1, &s_fail);
}

// bf16 all-reduce in place (sum, fp32 accumulation): [lo, hi) are bf16 element indices, multiples of 8.  Rank r owns the r-th
// of W equal runs of 16-byte vectors: it reduces them (in the switch through the multicast address, or with peer loads) and
// stores the result into every rank's copy.  Used for the tensor-parallel activations (sum of partial products).
__global__ void __launch_bounds__(512) allreduce_bf16_kernel(const CommArgs a) {
  __shared__ int s_fail;
  __shared__ unsigned long long s_peers[MAX_RANKS];
  if (threadIdx.x == 0) s_fail = 0;
  if (threadIdx.x < a.world) s_peers[threadIdx.x] = a.peer_ptrs[threadIdx.x];
  __syncthreads();
  if (!rank_barrier(a, 0, &s_fail)) return;
  const long long v0 = a.lo / 8, vecs = (a.hi - a.lo) / 8;
  const long long per = (vecs + a.world - 1) / a.world;
  const long long begin = v0 + min(vecs, per * a.rank), end = v0 + min(vecs, per * (a.rank + 1));
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  constexpr int UNROLL = 4;
  for (long long i0 = begin + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < end; i0 += stride * UNROLL) {
    uint4 r[UNROLL];
    if (a.mc_ptr != 0) {
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const long long i = i0 + u * stride;
        if (i < end) {
          const uint4* addr = reinterpret_cast<const uint4*>(a.mc_ptr) + i;
          asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                       : "=r"(r[u].x), "=r"(r[u].y), "=r"(r[u].z), "=r"(r[u].w)
                       : "l"(addr)
                       : "memory");
        }
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const long long i = i0 + u * stride;
        if (i < end) {
          uint4* addr = reinterpret_cast<uint4*>(a.mc_ptr) + i;
          asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(__uint_as_float(r[u].x)),
                       "f"(__uint_as_float(r[u].y)), "f"(__uint_as_float(r[u].z)), "f"(__uint_as_float(r[u].w))
                       : "memory");
        }
      }
    } else {
      float acc[UNROLL][8];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u)
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[u][k] = 0.f;
      for (int p = 0; p < a.world; ++p) {
        const uint4* base = reinterpret_cast<const uint4*>(s_peers[(a.rank + p) % a.world]);
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          const long long i = i0 + u * stride;
          if (i < end) {
            const uint4 raw = base[i];
            const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              acc[u][2 * k] += __uint_as_float(w[k] << 16);
              acc[u][2 * k + 1] += __uint_as_float(w[k] & 0xFFFF0000u);
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const long long i = i0 + u * stride;
        if (i < end) {
          const uint4 out = make_uint4(pack_bf16x2(acc[u][0], acc[u][1]), pack_bf16x2(acc[u][2], acc[u][3]), pack_bf16x2(acc[u][4], acc[u][5]),
                                       pack_bf16x2(acc[u][6], acc[u][7]));
          for (int p = 0; p < a.world; ++p) reinterpret_cast<uint4*>(s_peers[(a.rank + p) % a.world])[i] = out;
        }
      }
    }
  }
  rank_barrier(a, 1, &s_fail);
}

// Reduce-scatter with caller-chosen ownership: every rank reduces the part [own_lo, own_hi) of [lo, hi) that it owns
// (summing all ranks' copies, scaled) and stores the result into ITS OWN copy only.  Nothing is broadcast: the consumer
// of the reduced gradient is the owner's shard of the optimizer.  Half the NVLink traffic of the all-reduce above.
__global__ void __launch_bounds__(512) reduce_to_owner_kernel(const CommArgs a, long long own_lo, long long own_hi) {
  __shared__ int s_fail;
  __shared__ unsigned long long s_peers[MAX_RANKS];
  if (threadIdx.x == 0) s_fail = 0;
  if (threadIdx.x < a.world) s_peers[threadIdx.x] = a.peer_ptrs[threadIdx.x];
  __syncthreads();
  if (!rank_barrier(a, 0, &s_fail)) return;   // every rank's contribution to [lo, hi) is complete
  const long long b = (own_lo > a.lo ? own_lo : a.lo) / 4, e = (own_hi < a.hi ? own_hi : a.hi) / 4;   // 16-byte elements
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  float4* mine = reinterpret_cast<float4*>(s_peers[a.rank]);
  constexpr int UNROLL = 8;
  for (long long i0 = b + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < e; i0 += stride * UNROLL) {
    float4 acc[UNROLL];
    if (a.mc_ptr != 0) {
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const long long i = i0 + u * stride;
        acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < e) {
          const float* addr = reinterpret_cast<const float*>(a.mc_ptr) + i * 4;
          asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                       : "=f"(acc[u].x), "=f"(acc[u].y), "=f"(acc[u].z), "=f"(acc[u].w)
                       : "l"(addr)
                       : "memory");
        }
      }
    } else {
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int p = 0; p < a.world; ++p) {
        const int src = (a.rank + p) % a.world;
        const float4* base = reinterpret_cast<const float4*>(s_peers[src]);
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          const long long i = i0 + u * stride;
          if (i < e) {
            const float4 v = base[i];
            acc[u].x += v.x; acc[u].y += v.y; acc[u].z += v.z; acc[u].w += v.w;
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long i = i0 + u * stride;
      if (i < e) mine[i] = make_float4(acc[u].x * a.scale, acc[u].y * a.scale, acc[u].z * a.scale, acc[u].w * a.scale);
    }
  }
  rank_barrier(a, 1, &s_fail);   // no rank may overwrite its contribution while an owner is still reading it
}

// Every rank broadcasts its own slice of [lo, hi) (scaled) to all ranks: the second half of an all-reduce whose
// first half (the reduce-scatter) was done by the producing kernels with red.add into the owner's copy.
__global__ void __launch_bounds__(512) allgather_slices_kernel(const CommArgs a) {
  __shared__ int s_fail;
  __shared__ unsigned long long s_peers[MAX_RANKS];
  if (threadIdx.x == 0) s_fail = 0;
  if (threadIdx.x < a.world) s_peers[threadIdx.x] = a.peer_ptrs[threadIdx.x];
  __syncthreads();
  if (!rank_barrier(a, 0, &s_fail)) return;   // all ranks' producers have finished: the owner copies are complete
  long long begin, end;
  slice_of(a, begin, end);
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const float4* mine = reinterpret_cast<const float4*>(s_peers[a.rank]) + a.lo / 4;
  constexpr int UNROLL = 8;
  for (long long i0 = begin + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < end; i0 += stride * UNROLL) {
    float4 v[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long i = i0 + u * stride;
      v[u] = i < end ? mine[i] : make_float4(0.f, 0.f, 0.f, 0.f);
      v[u].x *= a.scale; v[u].y *= a.scale; v[u].z *= a.scale; v[u].w *= a.scale;
    }
    if (a.mc_ptr != 0) {
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const long long i = i0 + u * stride;
        if (i < end) {
          float* addr = reinterpret_cast<float*>(a.mc_ptr) + a.lo + i * 4;
          asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(v[u].x), "f"(v[u].y),
                       "f"(v[u].z), "f"(v[u].w)
                       : "memory");
        }
      }
    } else {
      for (int p = 0; p < a.world; ++p) {
        const int dst = (a.rank + p) % a.world;
        float4* base = reinterpret_cast<float4*>(s_peers[dst]) + a.lo / 4;
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          const long long i = i0 + u * stride;
          if (i < end) base[i] = v[u];
        }
      }
    }
  }
  rank_barrier(a, 1, &s_fail);
}

// Second half of a GEMM + all-reduce whose epilogue stored every rank's partial tile into that rank's slot of each
// rank's staging buffer: wait until all ranks have stored (flag barrier), then sum the `world` local slots in fp32 and
// write the bf16 result to `dst`.  One pass over local memory; nothing crosses NVLink here.
__global__ void __launch_bounds__(512) allreduce_finish_kernel(const CommArgs a, const __nv_bfloat16* __restrict__ staging,
                                                               __nv_bfloat16* __restrict__ dst, long long rows, int n) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  if (!rank_barrier(a, 0, &s_fail)) return;
  const long long total = rows * n / 8;  // 16-byte elements per slot
  const uint4* src = reinterpret_cast<const uint4*>(staging);
  uint4* out = reinterpret_cast<uint4*>(dst);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.f;
    for (int r = 0; r < a.world; ++r) {
      const uint4 raw = src[static_cast<long long>(r) * total + i];
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        acc[2 * k] += __uint_as_float(w[k] << 16);
        acc[2 * k + 1] += __uint_as_float(w[k] & 0xFFFF0000u);
      }
    }
    out[i] = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
  }
}

// A barrier across ranks as a kernel of its own (one CTA), on the third flag plane.
__global__ void __launch_bounds__(32) rank_barrier_kernel(const CommArgs a) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  rank_barrier(a, 2, &s_fail);
}

// One thread waits until *flag >= expected, for at most limit_ns; on expiry it records ST_TIMEOUT_PEER_FLAG and
// returns.  `observed` (optional) receives the last value read.
__global__ void flag_wait_kernel(const int* flag, int expected, unsigned long long limit_ns, int* status, int* observed) {
  const uint64_t t0 = globaltimer_ns();
  int v = ld_acquire_sys(flag);
  uint32_t polls = 0;
  while (v < expected) {
    if ((++polls & 63u) == 0u && globaltimer_ns() - t0 > limit_ns) {
      if (status) atomicCAS(status, 0, ST_TIMEOUT_PEER_FLAG);
      break;
    }
    v = ld_acquire_sys(flag);
  }
  if (observed) *observed = v;
}

__global__ void flag_set_kernel(int* flag, int value) {
  __threadfence_system();
  st_release_sys(flag, value);
}

// `sms` caps the grid: the reductions run next to compute kernels, and every CTA here takes an SM away from them, so
// the caller passes a small number (with 8 x 16 bytes in flight per thread a few dozen CTAs saturate the links).
static int comm_grid(long long vecs_per_rank, int sms) {
  int grid = static_cast<int>((vecs_per_rank + 511) / 512);
  const int cap = sms < MAX_CTAS ? sms : MAX_CTAS;
  if (grid > cap) grid = cap;
  return grid < 1 ? 1 : grid;
}

static int launch_allreduce(bool multimem, const CommArgs& a, int sms, cudaStream_t st) {
  if (a.world < 1 || a.world > MAX_RANKS) return -2;
  if ((a.lo & 3) || (a.hi & 3) || a.hi < a.lo) return -3;
  const long long vecs = (a.hi - a.lo) / 4 / (a.world > 0 ? a.world : 1);
  const int grid = comm_grid(vecs, sms);
  if (multimem) allreduce_multimem_kernel<<<grid, 512, 0, st>>>(a);
  else allreduce_two_shot_kernel<<<grid, 512, 0, st>>>(a);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace sb

extern "C" void sb_comm_set_wait_limit_ns(unsigned long long ns) { sb::g_comm_wait_ns = ns ? ns : SB_WAIT_LIMIT_NS; }
extern "C" unsigned long long sb_comm_wait_limit_ns() { return sb::comm_wait_ns(); }

// Advance a device-side epoch counter by one (stream-ordered; launch it in front of a collective that reads the counter).
extern "C" int sb_epoch_bump(int* counter, void* stream) {
  if (counter == nullptr) return -2;
  sb::epoch_bump_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(counter);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int sb_comm_flag_ints() { return 3 * sb::MAX_CTAS * sb::MAX_RANKS; }

extern "C" int sb_allreduce_two_shot(const void* peer_ptrs, const void* flag_ptrs, unsigned long long mc_ptr, int rank, int world,
                                     long long lo, long long hi, float scale, int epoch, const int* epoch_ptr, int sms, int* status, void* stream) {
  sb::CommArgs a{static_cast<const unsigned long long*>(peer_ptrs), static_cast<const unsigned long long*>(flag_ptrs), mc_ptr, rank,
                 world, lo, hi, scale, epoch, status, sb::comm_wait_ns(), epoch_ptr};
  return sb::launch_allreduce(false, a, sms, static_cast<cudaStream_t>(stream));
}

extern "C" int sb_allreduce_multimem(const void* peer_ptrs, const void* flag_ptrs, unsigned long long mc_ptr, int rank, int world,
                                     long long lo, long long hi, float scale, int epoch, const int* epoch_ptr, int sms, int* status, void* stream) {
  if (mc_ptr == 0) return -4;
  sb::CommArgs a{static_cast<const unsigned long long*>(peer_ptrs), static_cast<const unsigned long long*>(flag_ptrs), mc_ptr, rank,
                 world, lo, hi, scale, epoch, status, sb::comm_wait_ns(), epoch_ptr};
  return sb::launch_allreduce(true, a, sms, static_cast<cudaStream_t>(stream));
}

// Broadcast every rank's slice of [lo, hi) to all ranks (scaled).  mc_ptr != 0 selects the multicast store.
extern "C" int sb_allgather_slices(const void* peer_ptrs, const void* flag_ptrs, unsigned long long mc_ptr, int rank, int world,
                                   long long lo, long long hi, float scale, int epoch, const int* epoch_ptr, int sms, int* status, void* stream) {
  using namespace sb;
  if (world < 1 || world > MAX_RANKS) return -2;
  if ((lo & 3) || (hi & 3) || hi < lo) return -3;
  CommArgs a{static_cast<const unsigned long long*>(peer_ptrs), static_cast<const unsigned long long*>(flag_ptrs), mc_ptr, rank, world,
             lo, hi, scale, epoch, status, sb::comm_wait_ns(), epoch_ptr};
  const long long vecs = (hi - lo) / 4 / world;
  const int grid = comm_grid(vecs, sms);
  allgather_slices_kernel<<<grid, 512, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return static_cast<int>(cudaGetLastError());
}

// Reduce [lo, hi) across ranks into the owner's copy: this rank reduces [own_lo, own_hi) (clipped to [lo, hi); may be
// empty) and stores it locally.  mc_ptr != 0 selects the in-switch reduction.  All bounds are multiples of 4 elements.
extern "C" int sb_reduce_to_owner(const void* peer_ptrs, const void* flag_ptrs, unsigned long long mc_ptr, int rank, int world, long long lo,
                                  long long hi, long long own_lo, long long own_hi, float scale, int epoch, const int* epoch_ptr, int sms, int* status, void* stream) {
  using namespace sb;
  if (world < 1 || world > MAX_RANKS) return -2;
  if ((lo & 3) || (hi & 3) || (own_lo & 3) || (own_hi & 3) || hi < lo) return -3;
  CommArgs a{static_cast<const unsigned long long*>(peer_ptrs), static_cast<const unsigned long long*>(flag_ptrs), mc_ptr, rank, world,
             lo, hi, scale, epoch, status, sb::comm_wait_ns(), epoch_ptr};
  const long long b = own_lo > lo ? own_lo : lo, e = own_hi < hi ? own_hi : hi;
  const int grid = comm_grid(e > b ? (e - b) / 4 : 0, sms);
  reduce_to_owner_kernel<<<grid, 512, 0, static_cast<cudaStream_t>(stream)>>>(a, own_lo, own_hi);
  return static_cast<int>(cudaGetLastError());
}

// In-place bf16 sum over ranks of elements [lo, hi) (multiples of 8) of a symmetric bf16 buffer; mc_ptr != 0 selects the in-switch form.
extern "C" int sb_allreduce_bf16(const void* peer_ptrs, const void* flag_ptrs, unsigned long long mc_ptr, int rank, int world, long long lo,
                                 long long hi, int epoch, const int* epoch_ptr, int sms, int* status, void* stream) {
  using namespace sb;
  if (world < 1 || world > MAX_RANKS) return -2;
  if ((lo & 7) || (hi & 7) || hi < lo) return -3;
  CommArgs a{static_cast<const unsigned long long*>(peer_ptrs), static_cast<const unsigned long long*>(flag_ptrs), mc_ptr, rank, world,
             lo, hi, 1.f, epoch, status, sb::comm_wait_ns(), epoch_ptr};
  const int grid = comm_grid((hi - lo) / 8 / world, sms);
  allreduce_bf16_kernel<<<grid, 512, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int sb_rank_barrier(const void* flag_ptrs, int rank, int world, int epoch, const int* epoch_ptr, int* status, void* stream) {
  using namespace sb;
  if (world < 1 || world > MAX_RANKS) return -2;
  CommArgs a{nullptr, static_cast<const unsigned long long*>(flag_ptrs), 0ull, rank, world, 0, 0, 1.f, epoch, status, sb::comm_wait_ns(), epoch_ptr};
  rank_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return static_cast<int>(cudaGetLastError());
}

// Stream-ordered wait on a flag word with a time limit (nanoseconds, capped at 5 s).
extern "C" int sb_flag_wait(const int* flag, int expected, unsigned long long limit_ns, int* status, int* observed, void* stream) {
  if (flag == nullptr) return -2;
  if (limit_ns > 5000000000ull) limit_ns = 5000000000ull;
  sb::flag_wait_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(flag, expected, limit_ns, status, observed);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int sb_flag_set(int* flag, int value, void* stream) {
  if (flag == nullptr) return -2;
  sb::flag_set_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(flag, value);
  return static_cast<int>(cudaGetLastError());
}

// See allreduce_finish_kernel.  rows * n must be a multiple of 8; dst is a contiguous [rows, n] bf16 tensor.
extern "C" int sb_allreduce_finish(const void* flag_ptrs, int rank, int world, int epoch, const int* epoch_ptr, const void* staging, void* dst,
                                   long long rows, int n, int sms, int* status, void* stream) {
  using namespace sb;
  if (world < 1 || world > MAX_RANKS) return -2;
  if ((rows * n) % 8) return -3;
  CommArgs a{nullptr, static_cast<const unsigned long long*>(flag_ptrs), 0ull, rank, world, 0, 0, 1.f, epoch, status, sb::comm_wait_ns(), epoch_ptr};
  const int grid = comm_grid(rows * n / 8, sms);
  allreduce_finish_kernel<<<grid, 512, 0, static_cast<cudaStream_t>(stream)>>>(a, static_cast<const __nv_bfloat16*>(staging),
                                                                               static_cast<__nv_bfloat16*>(dst), rows, n);
  return static_cast<int>(cudaGetLastError());
}
