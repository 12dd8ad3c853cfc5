// Residual selection for the compressed linear layer.
//
// The residual E = X - C Q^T is never stored: every pass recomputes it from the bf16 input
// tile, the rank-r coefficients and the basis (r FMAs per element), which is cheaper than a
// round trip through HBM.  Exact top-k by magnitude is done as a radix select on the 15-bit
// bf16 magnitude of E:
//   pass 1  histogram of magnitudes (32768 bins, privatised in shared memory, one global
//           histogram per row chunk);
//   scan    per chunk, walk the histogram from the top to find the threshold bin and how many
//           entries of that bin are still needed (ties inside a bin are equal bf16 values, so
//           any subset is an exact top-k);
//   pass 2  recompute E, keep entries above the threshold (plus the needed ties), quantise
//           with the per-tensor scale amax/qmax known from the histogram, and append
//           (flat index, value) through a shared-memory staging buffer so that global
//           appends are one atomic per flush, not one per element.
// Replaces the chunked subtract + abs + torch.topk + cat + topk pipeline of the reference
// (stacr/layers.py:16-102 there) and its separate quantisation pass (stacr/quant.py:49-65).
#include "common.cuh"

namespace sb {

constexpr int NBINS = 32768;
constexpr int ROWS_UNROLL = 8;  // rows in flight per thread (memory-level parallelism)
constexpr int CS_ROWS = 256;    // coefficient rows staged in shared memory at a time

struct SelectParams {
  const __nv_bfloat16* x;   // [rows, n], leading dimension ldx
  const __nv_bfloat16* c;   // [rows, r] contiguous
  const __nv_bfloat16* q;   // [n, r] contiguous
  int rows, n, r, ldx;
  int chunk_rows;           // rows per selection chunk (== rows for a single global selection)
  int parts;                // CTAs per chunk
  unsigned int* hist;       // [nchunks, NBINS]
  // scan outputs / compaction inputs, one per chunk
  int* thr_bin;             // threshold bin
  int* thr_need;            // entries of the threshold bin still needed
  int* max_bin;             // largest non-empty bin
  int* tie_count;           // running count of accepted ties
  int* out_count;           // running count of appended entries
  const int* out_offset;    // first output slot of each chunk
  const int* quota;         // entries wanted per chunk
  int nchunks;
  int bits;                 // 0: bf16 values, 8: int8 values (int4 is packed from int8 afterwards)
  long long* out_idx64;     // flat indices (one of the two is used)
  int* out_idx32;
  void* out_val;            // bf16 or int8
  float* out_scale;         // scalar, written by the scan kernel
  int* status;
  const int* gate;          // optional [nchunks]: the exact passes skip chunks whose entry is 0 (NULL = run them all)
};

__device__ __forceinline__ float bf16_bits_to_float(unsigned short b) {
  return __uint_as_float(static_cast<uint32_t>(b) << 16);
}

// Raw bf16 loads of CPT consecutive columns (vectorised when the whole group is in range;
// the launcher guarantees 16-byte aligned rows) and of one coefficient row.
template <int CPT>
struct XVec { unsigned short v[CPT]; };

template <int CPT>
__device__ __forceinline__ XVec<CPT> load_x(const __nv_bfloat16* xrow, int col, int n) {
  XVec<CPT> out;
  if (col + CPT <= n) {
    if constexpr (CPT == 8) {
      *reinterpret_cast<uint4*>(out.v) = __ldg(reinterpret_cast<const uint4*>(xrow + col));
    } else if constexpr (CPT == 4) {
      *reinterpret_cast<uint2*>(out.v) = __ldg(reinterpret_cast<const uint2*>(xrow + col));
    } else {
      *reinterpret_cast<uint32_t*>(out.v) = __ldg(reinterpret_cast<const uint32_t*>(xrow + col));
    }
  } else {
#pragma unroll
    for (int i = 0; i < CPT; ++i) out.v[i] = (col + i < n) ? __bfloat16_as_ushort(xrow[col + i]) : 0;
  }
  return out;
}

template <int RP>
struct CVec { unsigned short v[RP]; };

template <int RP>
__device__ __forceinline__ CVec<RP> load_c(const __nv_bfloat16* crow, int r) {
  CVec<RP> out;
  if (r == RP) {  // rows are RP*2 bytes: 16-byte aligned for RP >= 8
#pragma unroll
    for (int j = 0; j < RP / 8; ++j)
      reinterpret_cast<uint4*>(out.v)[j] = __ldg(reinterpret_cast<const uint4*>(crow) + j);
  } else {
#pragma unroll
    for (int j = 0; j < RP; ++j) out.v[j] = (j < r) ? __bfloat16_as_ushort(crow[j]) : 0;
  }
  return out;
}

// Residual of CPT consecutive columns of one row, using register-resident basis rows.
template <int RP, int CPT>
__device__ __forceinline__ void residual_row(const XVec<CPT>& xv, const CVec<RP>& cv,
                                             const float (&qreg)[CPT][RP], float (&e)[CPT]) {
  float cf[RP];
#pragma unroll
  for (int j = 0; j < RP; ++j) cf[j] = bf16_bits_to_float(cv.v[j]);
#pragma unroll
  for (int i = 0; i < CPT; ++i) {
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < RP; ++j) acc = fmaf(cf[j], qreg[i][j], acc);
    e[i] = bf16_bits_to_float(xv.v[i]) - acc;
  }
}

template <int RP, int CPT>
__device__ __forceinline__ void load_q(const __nv_bfloat16* q, int r, int col, int n, float (&qreg)[CPT][RP]) {
#pragma unroll
  for (int i = 0; i < CPT; ++i) {
    if (r == RP && col + i < n) {  // a basis row is RP * 2 bytes: 16-byte aligned for RP >= 8
      const uint4* src = reinterpret_cast<const uint4*>(q + static_cast<size_t>(col + i) * RP);
#pragma unroll
      for (int v = 0; v < RP / 8; ++v) {
        const uint4 raw = __ldg(src + v);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          qreg[i][v * 8 + 2 * k] = __uint_as_float(w[k] << 16);
          qreg[i][v * 8 + 2 * k + 1] = __uint_as_float(w[k] & 0xFFFF0000u);
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < RP; ++j)
        qreg[i][j] = (col + i < n && j < r) ? __bfloat162float(q[static_cast<size_t>(col + i) * r + j]) : 0.f;
    }
  }
}

// Coefficient rows [row0, row1) of the slab as fp32 in shared memory, RP values per row (zero-padded past r).
// Called by every thread of the CTA; ends with a barrier.
template <int RP>
__device__ __forceinline__ void stage_coeff(const __nv_bfloat16* c, int r, int row0, int row1, float* s_c) {
  __syncthreads();  // the previous sub-slab is no longer being read
  const int total = (row1 - row0) * RP;
  for (int i = threadIdx.x; i < total; i += blockDim.x) {
    const int lr = i / RP, j = i - lr * RP;
    s_c[i] = (j < r) ? __bfloat162float(c[static_cast<size_t>(row0 + lr) * r + j]) : 0.f;
  }
  __syncthreads();
}

// Residual of CPT consecutive columns of one row; the coefficient row is read from shared memory (the address is
// the same for every lane that works on this row, so the loads are broadcasts).
template <int RP, int CPT>
__device__ __forceinline__ void residual_row_s(const XVec<CPT>& xv, const float* crow, const float (&qreg)[CPT][RP], float (&e)[CPT]) {
  float cf[RP];
#pragma unroll
  for (int v = 0; v < RP / 4; ++v) {
    const float4 t = reinterpret_cast<const float4*>(crow)[v];
    cf[4 * v] = t.x; cf[4 * v + 1] = t.y; cf[4 * v + 2] = t.z; cf[4 * v + 3] = t.w;
  }
#pragma unroll
  for (int i = 0; i < CPT; ++i) {
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < RP; ++j) acc = fmaf(cf[j], qreg[i][j], acc);
    e[i] = bf16_bits_to_float(xv.v[i]) - acc;
  }
}

// Work split shared by both passes: blockIdx.x = chunk * parts + part; a CTA walks its row
// slab with `rl` row lanes and `ctn` column threads (ctn * CPT covers a column block).
struct Slab {
  int chunk, row0, row1;
};
__device__ __forceinline__ Slab slab_of(const SelectParams& p) {
  Slab s;
  s.chunk = blockIdx.x / p.parts;
  const int part = blockIdx.x - s.chunk * p.parts;
  const int c0 = s.chunk * p.chunk_rows;
  const int c1 = min(p.rows, c0 + p.chunk_rows);
  const int len = c1 - c0;
  s.row0 = c0 + static_cast<int>((static_cast<long long>(len) * part) / p.parts);
  s.row1 = c0 + static_cast<int>((static_cast<long long>(len) * (part + 1)) / p.parts);
  return s;
}

template <int RP>
__global__ void __launch_bounds__(512, 1) residual_hist_kernel(const SelectParams p, int ctn, int rl) {
  constexpr int CPT = 64 / RP;
  extern __shared__ unsigned int sh_hist[];
  float* s_c = reinterpret_cast<float*>(sh_hist + NBINS);
  const Slab s = slab_of(p);
  if (p.gate && !p.gate[s.chunk]) return;
  for (int b = threadIdx.x; b < NBINS; b += blockDim.x) sh_hist[b] = 0;
  const int ct = threadIdx.x % ctn, lane_row = threadIdx.x / ctn;
  for (int sb0 = s.row0; sb0 < s.row1; sb0 += CS_ROWS) {
    const int sb1 = min(s.row1, sb0 + CS_ROWS);
    stage_coeff<RP>(p.c, p.r, sb0, sb1, s_c);
    for (int cb = 0; cb < p.n; cb += ctn * CPT) {
      const int col = cb + ct * CPT;
      if (col >= p.n || lane_row >= rl) continue;
      float qreg[CPT][RP];
      load_q<RP, CPT>(p.q, p.r, col, p.n, qreg);
      for (int row = sb0 + lane_row; row < sb1; row += rl * ROWS_UNROLL) {
        XVec<CPT> xv[ROWS_UNROLL];
#pragma unroll
        for (int u = 0; u < ROWS_UNROLL; ++u) {  // issue every load of the group before any use
          const int rr = row + u * rl;
          if (rr < sb1) xv[u] = load_x<CPT>(p.x + static_cast<size_t>(rr) * p.ldx, col, p.n);
        }
#pragma unroll
        for (int u = 0; u < ROWS_UNROLL; ++u) {
          const int rr = row + u * rl;
          if (rr >= sb1) continue;
          float e[CPT];
          residual_row_s<RP, CPT>(xv[u], s_c + (rr - sb0) * RP, qreg, e);
#pragma unroll
          for (int i = 0; i < CPT; ++i) {
            if (col + i < p.n) {
              unsigned short key = __bfloat16_as_ushort(__float2bfloat16_rn(e[i])) & 0x7FFF;
              atomicAdd(&sh_hist[key], 1u);
            }
          }
        }
      }
    }
  }
  __syncthreads();
  unsigned int* gh = p.hist + static_cast<size_t>(s.chunk) * NBINS;
  for (int b = threadIdx.x; b < NBINS; b += blockDim.x) {
    unsigned int v = sh_hist[b];
    if (v) atomicAdd(&gh[b], v);
  }
}

// One CTA per chunk: suffix scan over the histogram.
__global__ void __launch_bounds__(1024) residual_scan_kernel(const SelectParams p) {
  __shared__ unsigned int part[1024];
  __shared__ int s_maxbin;
  const int chunk = blockIdx.x;
  if (p.gate && !p.gate[chunk]) return;
  const unsigned int* gh = p.hist + static_cast<size_t>(chunk) * NBINS;
  const int t = threadIdx.x;
  constexpr int PER = NBINS / 1024;  // 32 bins per thread; thread t owns bins [t*PER, (t+1)*PER)
  unsigned int local[PER];
  unsigned int sum = 0;
  int my_max = -1;
#pragma unroll
  for (int v = 0; v < PER / 4; ++v) {  // 32 bins = eight 16-byte loads, all issued before the first use
    const uint4 raw = reinterpret_cast<const uint4*>(gh + t * PER)[v];
    local[4 * v] = raw.x; local[4 * v + 1] = raw.y; local[4 * v + 2] = raw.z; local[4 * v + 3] = raw.w;
  }
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    sum += local[i];
    if (local[i]) my_max = t * PER + i;
  }
  part[t] = sum;
  if (t == 0) s_maxbin = 0;
  __syncthreads();
  if (my_max >= 0) atomicMax(&s_maxbin, my_max);
  // suffix sums over threads (inclusive): suf[t] = sum_{u >= t} part[u]
  for (int off = 1; off < 1024; off <<= 1) {
    unsigned int add = (t + off < 1024) ? part[t + off] : 0u;
    __syncthreads();
    part[t] += add;
    __syncthreads();
  }
  const unsigned int k = static_cast<unsigned int>(p.quota[chunk]);
  const unsigned int above = (t + 1 < 1024) ? part[t + 1] : 0u;  // entries in bins owned by higher threads
  const unsigned int incl = part[t];
  if (k > 0 && above < k && incl >= k) {
    // the threshold bin is among this thread's bins; walk from its top bin down
    unsigned int run = above;
    for (int i = PER - 1; i >= 0; --i) {
      if (run + local[i] >= k) {
        p.thr_bin[chunk] = t * PER + i;
        p.thr_need[chunk] = static_cast<int>(k - run);
        break;
      }
      run += local[i];
    }
  }
  if (t == 0) {
    if (k == 0 || part[0] < k) {  // nothing wanted, or fewer entries than wanted: take everything
      p.thr_bin[chunk] = (k == 0) ? NBINS : -1;
      p.thr_need[chunk] = 0;
    }
    p.tie_count[chunk] = 0;
    p.out_count[chunk] = 0;
  }
  __syncthreads();
  if (t == 0) p.max_bin[chunk] = s_maxbin;
}

// Per-tensor scale from the largest magnitude over all chunks (runs after the scan).
__global__ void residual_scale_kernel(const SelectParams p) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    int mb = 0;
    for (int c = 0; c < p.nchunks; ++c) mb = max(mb, p.max_bin[c]);
    const float amax = bf16_bits_to_float(static_cast<unsigned short>(mb));
    const float qmax = (p.bits == 4) ? 7.f : 127.f;
    *p.out_scale = (p.bits == 0) ? 1.f : fmaxf(amax / qmax, 1.17549435e-38f);
  }
}

constexpr int MAX_DEVICES = 64;  // per-device launch configuration flags are indexed by the CUDA device ordinal
constexpr int WARP_CAP = 768;  // staged (index, value) pairs per warp between flushes (16 warps: 120 KB)

__device__ __forceinline__ void emit_entry(const SelectParams& p, int o, long long flat, unsigned short bits16,
                                           float inv_scale) {
  if (p.out_idx32) p.out_idx32[o] = static_cast<int>(flat);
  else p.out_idx64[o] = flat;
  if (p.bits == 0) {
    reinterpret_cast<unsigned short*>(p.out_val)[o] = bits16;
  } else {
    const float lo = (p.bits == 4) ? -8.f : -128.f, hi = (p.bits == 4) ? 7.f : 127.f;
    float qv = fminf(fmaxf(rintf(bf16_bits_to_float(bits16) * inv_scale), lo), hi);
    reinterpret_cast<signed char*>(p.out_val)[o] = static_cast<signed char>(qv);
  }
}

// bf16 bits of one residual entry, with exactly the arithmetic of residual_row_s (same operands, same order).
template <int RP>
__device__ __forceinline__ unsigned short residual_bits_at(const SelectParams& p, const float* crow, int rr, int c) {
  float acc = 0.f;
  const __nv_bfloat16* qrow = p.q + static_cast<size_t>(c) * p.r;
#pragma unroll
  for (int j = 0; j < RP; ++j) {
    const float qv = (j < p.r) ? __bfloat162float(qrow[j]) : 0.f;
    acc = fmaf(crow[j], qv, acc);
  }
  const float x = __bfloat162float(p.x[static_cast<size_t>(rr) * p.ldx + c]);
  return __bfloat16_as_ushort(__float2bfloat16_rn(x - acc));
}

// Pass 2.  The row loop only marks candidates: one compare of |e| against the lower edge of the threshold bin per
// element, collected in a 64-bit mask per thread.  The few marked entries (about the selection density) are then
// recomputed one by one to get their exact bf16 value, ties of the threshold bin are arbitrated, and the survivors
// are staged in the warp's own slice of shared memory (positions from a warp prefix sum, the running count lives
// in a register that all lanes agree on) and copied out with one global atomic per flush.  Warps never wait for
// one another inside the loop.
template <int RP>
__global__ void __launch_bounds__(512, 1) residual_compact_kernel(const SelectParams p, int ctn, int rl) {
  constexpr int CPT = 64 / RP;
  constexpr unsigned FULL = 0xffffffffu;
  extern __shared__ unsigned char sh_raw[];
  const int nwarps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  long long* st_idx_all = reinterpret_cast<long long*>(sh_raw);
  unsigned short* st_val_all = reinterpret_cast<unsigned short*>(st_idx_all + static_cast<size_t>(nwarps) * WARP_CAP);
  float* s_c = reinterpret_cast<float*>(sh_raw + static_cast<size_t>(16) * WARP_CAP * 10);
  long long* st_idx = st_idx_all + static_cast<size_t>(warp) * WARP_CAP;
  unsigned short* st_val = st_val_all + static_cast<size_t>(warp) * WARP_CAP;
  const Slab s = slab_of(p);
  if (p.gate && !p.gate[s.chunk]) return;
  const int thr = p.thr_bin[s.chunk];
  const int need = p.thr_need[s.chunk];
  const int quota = p.quota[s.chunk];
  const int obase = p.out_offset[s.chunk];
  const float inv_scale = 1.f / *p.out_scale;
  // every value that rounds to a magnitude >= thr is >= the midpoint between thr and the bf16 below it; values at
  // the midpoint itself may round down and are sorted out when the candidate is recomputed
  const float cut = thr > 0 ? 0.5f * (bf16_bits_to_float(static_cast<unsigned short>(thr)) + bf16_bits_to_float(static_cast<unsigned short>(thr - 1))) : 0.f;
  const int ct = threadIdx.x % ctn, lane_row = threadIdx.x / ctn;
  int wcnt = 0;  // entries staged by this warp (same value in every lane)

  auto flush = [&]() {  // whole warp
    const int cnt = min(wcnt, WARP_CAP);
    int base = 0;
    if (lane == 0 && cnt > 0) base = atomicAdd(&p.out_count[s.chunk], cnt);
    base = __shfl_sync(FULL, base, 0);
    __syncwarp();
    for (int i = lane; i < cnt; i += 32)
      if (base + i < quota) emit_entry(p, obase + base + i, st_idx[i], st_val[i], inv_scale);
    __syncwarp();
    wcnt = 0;
  };

  for (int sb0 = s.row0; sb0 < s.row1; sb0 += CS_ROWS) {
    const int sb1 = min(s.row1, sb0 + CS_ROWS);
    stage_coeff<RP>(p.c, p.r, sb0, sb1, s_c);
    for (int cb = 0; cb < p.n; cb += ctn * CPT) {
      const int col = cb + ct * CPT;
      const bool active = (col < p.n) && (lane_row < rl);
      float qreg[CPT][RP];
      if (active) load_q<RP, CPT>(p.q, p.r, col, p.n, qreg);
      const int step = rl * ROWS_UNROLL;
      const int iters = (sb1 - sb0 + step - 1) / step;  // the same for every thread: the warp votes below stay converged
      for (int it = 0; it < iters; ++it) {
        if (wcnt > WARP_CAP / 2) flush();
        const int row = sb0 + it * step + lane_row;
        XVec<CPT> xv[ROWS_UNROLL];
#pragma unroll
        for (int u = 0; u < ROWS_UNROLL; ++u) {
          const int rr = row + u * rl;
          if (active && rr < sb1) xv[u] = load_x<CPT>(p.x + static_cast<size_t>(rr) * p.ldx, col, p.n);
        }
        unsigned long long marks = 0;  // bit u * CPT + i: entry (row + u * rl, col + i) may belong to the selection
#pragma unroll
        for (int u = 0; u < ROWS_UNROLL; ++u) {
          const int rr = row + u * rl;
          if (active && rr < sb1) {
            float e[CPT];
            residual_row_s<RP, CPT>(xv[u], s_c + (rr - sb0) * RP, qreg, e);
#pragma unroll
            for (int i = 0; i < CPT; ++i)
              if (col + i < p.n && !(fabsf(e[i]) < cut)) marks |= 1ull << (u * CPT + i);
          }
        }
        if (__any_sync(FULL, marks != 0)) {
          // exact value of every candidate; entries below the bin and surplus ties are dropped
          unsigned long long todo = marks;
          while (todo) {
            const int b = __ffsll(static_cast<long long>(todo)) - 1;
            todo &= todo - 1;
            const int rr = row + (b / CPT) * rl, c = col + (b % CPT);
            const int key = residual_bits_at<RP>(p, s_c + (rr - sb0) * RP, rr, c) & 0x7FFF;
            bool take = key > thr;
            if (!take && key == thr && need > 0) {
              // ties are equal values: the first `need` askers win; stop asking once the bin is full
              if (*reinterpret_cast<volatile int*>(&p.tie_count[s.chunk]) < need) take = atomicAdd(&p.tie_count[s.chunk], 1) < need;
            }
            if (!take) marks &= ~(1ull << b);
          }
          const int mine = __popcll(marks);
          int incl = mine;
#pragma unroll
          for (int off = 1; off < 32; off <<= 1) {
            const int v = __shfl_up_sync(FULL, incl, off);
            if (lane >= off) incl += v;
          }
          const int total = __shfl_sync(FULL, incl, 31);
          int pos = wcnt + incl - mine;
          todo = marks;
          while (todo) {
            const int b = __ffsll(static_cast<long long>(todo)) - 1;
            todo &= todo - 1;
            const int rr = row + (b / CPT) * rl, c = col + (b % CPT);
            const unsigned short bits16 = residual_bits_at<RP>(p, s_c + (rr - sb0) * RP, rr, c);
            const long long flat = static_cast<long long>(rr) * p.n + c;
            if (pos < WARP_CAP) {
              st_idx[pos] = flat;
              st_val[pos] = bits16;
            } else {  // this warp's staging slice is full (very dense selection): append directly
              const int o = atomicAdd(&p.out_count[s.chunk], 1);
              if (o < quota) emit_entry(p, obase + o, flat, bits16, inv_scale);
            }
            ++pos;
          }
          wcnt += total;
          __syncwarp();
        }
      }
    }
  }
  flush();
}

// e[i] = X[idx] - C[row] . Q[col] for an explicit index list (uniform / block-sparse selectors).
__global__ void residual_gather_kernel(const __nv_bfloat16* x, const __nv_bfloat16* c, const __nv_bfloat16* q,
                                       int n, int r, int ldx, const long long* idx64, const int* idx32, long long count,
                                       __nv_bfloat16* out) {
  long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= count) return;
  const long long flat = idx64 ? idx64[i] : static_cast<long long>(idx32[i]);
  const long long row = flat / n;
  const int col = static_cast<int>(flat - row * n);
  float acc = 0.f;
  for (int j = 0; j < r; ++j)
    acc = fmaf(__bfloat162float(c[row * r + j]), __bfloat162float(q[static_cast<size_t>(col) * r + j]), acc);
  out[i] = __float2bfloat16_rn(__bfloat162float(x[row * ldx + col]) - acc);
}

// energy[row, b] = sum of squared (bf16-rounded) residuals over `bs` consecutive columns;
// bs is a power of two in [8, 256] dividing n.  A thread owns 8 consecutive columns for BE_ROWS rows: its 8 basis rows
// stay in registers, the coefficient rows of the CTA come from shared memory as broadcasts, X is read with one 16-byte
// load per row, and the bs / 8 lanes of a block are shuffle-reduced.
constexpr int BE_ROWS = 8;   // rows per CTA: small, so that a 4096-row activation gives every SM several CTAs (the kernel is latency-bound)

template <int RP>
__global__ void __launch_bounds__(256) residual_block_energy_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ c,
                                                                    const __nv_bfloat16* __restrict__ q, int rows, int n, int r, int ldx,
                                                                    int bs, float* __restrict__ energy) {
  __shared__ float s_c[BE_ROWS * RP];
  const int row0 = blockIdx.x * BE_ROWS;   // rows on the x dimension of the grid: it has no 65535 limit
  const int nrows = min(BE_ROWS, rows - row0);
  for (int i = threadIdx.x; i < BE_ROWS * RP; i += blockDim.x) {
    const int lr = i / RP, j = i - lr * RP;
    s_c[i] = (lr < nrows && j < r) ? __bfloat162float(c[static_cast<size_t>(row0 + lr) * r + j]) : 0.f;
  }
  __syncthreads();
  const int tpb = bs / 8;
  const int col = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  const bool live = col < n;  // n is a multiple of bs >= 8, so a live thread owns 8 valid columns
  float qreg[8][RP];
  if (RP == 8 && r == 8 && live && (reinterpret_cast<uintptr_t>(q) & 15) == 0) {
    // a basis row is 16 bytes: one vector load per column instead of eight 2-byte loads
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint4 raw = __ldg(reinterpret_cast<const uint4*>(q + static_cast<size_t>(col + i) * 8));
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        qreg[i][2 * k] = __uint_as_float(w[k] << 16);
        qreg[i][2 * k + 1] = __uint_as_float(w[k] & 0xFFFF0000u);
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < RP; ++j) qreg[i][j] = (live && j < r) ? __bfloat162float(q[static_cast<size_t>(col + i) * r + j]) : 0.f;
  }
  const bool vec = ((ldx & 7) == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
  // BE_UNROLL rows in flight per thread: with one load per row and iteration the kernel ran at DRAM latency (40 us for 10 MB)
  constexpr int BE_UNROLL = RP <= 8 ? 8 : (RP <= 16 ? 4 : 1);   // the basis rows already take 8 * RP registers
  for (int lr0 = 0; lr0 < nrows; lr0 += BE_UNROLL) {
    uint4 raw[BE_UNROLL];
#pragma unroll
    for (int u = 0; u < BE_UNROLL; ++u) {
      raw[u] = make_uint4(0u, 0u, 0u, 0u);
      if (live && lr0 + u < nrows) {
        const __nv_bfloat16* xr = x + static_cast<size_t>(row0 + lr0 + u) * ldx + col;
        if (vec) {
          raw[u] = __ldg(reinterpret_cast<const uint4*>(xr));
        } else {
          uint32_t w[4];
#pragma unroll
          for (int k = 0; k < 4; ++k)
            w[k] = static_cast<uint32_t>(__bfloat16_as_ushort(xr[2 * k])) | (static_cast<uint32_t>(__bfloat16_as_ushort(xr[2 * k + 1])) << 16);
          raw[u] = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < BE_UNROLL; ++u) {
      const int lr = lr0 + u;
      if (lr >= nrows) break;
      float sum = 0.f;
      if (live) {
        const uint32_t w[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
        float xv[8];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          xv[2 * k] = __uint_as_float(w[k] << 16);
          xv[2 * k + 1] = __uint_as_float(w[k] & 0xFFFF0000u);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float acc = 0.f;
#pragma unroll
          for (int j = 0; j < RP; ++j) acc = fmaf(s_c[lr * RP + j], qreg[i][j], acc);
          const float e = __bfloat162float(__float2bfloat16_rn(xv[i] - acc));
          sum = fmaf(e, e, sum);
        }
      }
      for (int off = 1; off < tpb; off <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
      if (live && (threadIdx.x % tpb) == 0) energy[static_cast<size_t>(row0 + lr) * (n / bs) + col / bs] = sum;
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Sampled-threshold selection: the same exact top-k with one full pass over X instead of two.
//
//   A  histogram of a stratified 1/16 sample of the residual (of every row, one 64-column line in 16, the
//      line offset rotating with the row, so that heavy rows and heavy columns are both represented); the
//      last CTA of a chunk to finish turns it into a *candidate* bin t_lo below which, by the sample's
//      estimate with a safety margin, none of the chunk's top-k entries lie;
//   C  the full pass: every entry whose magnitude reaches t_lo is appended (index, bf16 bits) to the
//      chunk's candidate list through per-warp staging, and counted in a second histogram; the last CTA of
//      a chunk finds the exact threshold bin and tie count among the candidates and checks that the
//      candidates really contain the top k (at least k of them at or above t_lo, list not overflowed);
//   E  compaction of the candidate list (a few hundred thousand entries, not the matrix) with the
//      quantisation fused, as in the exact compaction pass.
//
// A chunk whose check fails (an input the sample misjudged) is flagged, its first histogram is cleared,
// and the exact two-pass kernels, launched behind E with that flag as their gate, redo that chunk; for
// every other chunk they return at once.  The selection is therefore exact for every input; only its cost
// depends on the sample being representative.
// ------------------------------------------------------------------------------------------------
constexpr int SAMPLE_STRIDE = 16;
constexpr int SAMPLE_LINE = 64;
constexpr int SCAN_T = 256;  // threads that take part in a tail scan (NBINS / SCAN_T bins each)

struct Select2Params {
  SelectParams base;
  unsigned int* hist2;        // [nchunks, NBINS] histogram of the candidates, zeroed by the caller
  int* cand_bin;              // [nchunks] t_lo
  int* cand_count;            // [nchunks] candidates appended (may exceed the capacity: the excess was dropped)
  int* fallback;              // [nchunks] 1 = redo this chunk with the exact passes
  int* done_a;                // [nchunks] CTAs of pass A that have finished
  int* done_c;                // [nchunks] CTAs of pass C that have finished
  int* done_all;              // [1] CTAs of pass C that have finished, all chunks
  int* gmax;                  // [1] largest magnitude key seen
  const int* cand_off;        // [nchunks] first slot of the chunk's candidate list
  const int* cand_cap;        // [nchunks] its capacity
  const float* margin;        // [nchunks] safety factor on the sample's estimate
  long long* cand_idx;
  unsigned short* cand_val;
  float fixed_cut;            // >= 0: pass C lists every entry with |e| >= fixed_cut instead of using the sampled bin
};

// Whole CTA (blockDim.x >= SCAN_T).  Copies a chunk's histogram (written by other CTAs' atomics: read through L2) into
// shared memory with coalesced 16-byte loads and leaves in s_part[t] the number of entries in bins >= t * PER (inclusive
// suffix sums over SCAN_T segments of PER bins; s_part[0] is the total) and in s_out[2] the largest non-empty bin.
// A single thread walking 128 bins in global memory costs 128 dependent L2 round trips; from shared memory it is 2 us.
__device__ void hist_stage(const unsigned int* gh, unsigned int* sh, unsigned int* s_part, int* s_out) {
  constexpr int PER = NBINS / SCAN_T;
  const int t = threadIdx.x;
  const uint4* src = reinterpret_cast<const uint4*>(gh);
  uint4* dst = reinterpret_cast<uint4*>(sh);
#pragma unroll 4
  for (int i = t; i < NBINS / 4; i += blockDim.x) dst[i] = __ldcg(src + i);
  if (t == 0) s_out[2] = -1;
  __syncthreads();
  if (t < SCAN_T) {
    unsigned int sum = 0;
    int my_max = -1;
#pragma unroll 8
    for (int i = 0; i < PER; ++i) {
      const int ii = (i + t) & (PER - 1);  // rotate the start so that the lanes of a warp hit different banks
      const unsigned int v = sh[t * PER + ii];
      sum += v;
      if (v) my_max = max(my_max, t * PER + ii);
    }
    s_part[t] = sum;
    if (my_max >= 0) atomicMax(&s_out[2], my_max);
  }
  __syncthreads();
  for (int off = 1; off < SCAN_T; off <<= 1) {
    unsigned int add = 0;
    if (t < SCAN_T && t + off < SCAN_T) add = s_part[t + off];
    __syncthreads();
    if (t < SCAN_T) s_part[t] += add;
    __syncthreads();
  }
}

// After hist_stage: the largest bin b with count(bins >= b) >= k -> s_out[0], and how many entries of b are needed
// -> s_out[1].  k == 0 or fewer than k entries in total leave s_out[0] = -1.  Ends with a barrier.
__device__ void hist_locate(const unsigned int* sh, const unsigned int* s_part, unsigned int k, int* s_out) {
  constexpr int PER = NBINS / SCAN_T;
  const int t = threadIdx.x;
  if (t == 0) {
    s_out[0] = -1;
    s_out[1] = 0;
  }
  __syncthreads();
  if (t < SCAN_T) {
    const unsigned int above = (t + 1 < SCAN_T) ? s_part[t + 1] : 0u;
    const unsigned int incl = s_part[t];
    if (k > 0 && above < k && incl >= k) {
      unsigned int run = above;
      for (int i = PER - 1; i >= 0; --i) {
        const unsigned int cnt = sh[t * PER + i];
        if (run + cnt >= k) {
          s_out[0] = t * PER + i;
          s_out[1] = static_cast<int>(k - run);
          break;
        }
        run += cnt;
      }
    }
  }
  __syncthreads();
}

template <int RP>
__global__ void __launch_bounds__(512, 1) residual_sample_kernel(const Select2Params sp) {
  constexpr int CPT = 64 / RP;   // columns per thread; RP threads cover one 64-column line
  const SelectParams& p = sp.base;
  extern __shared__ unsigned int sh_hist[];
  __shared__ unsigned int s_part[SCAN_T];
  __shared__ int s_out[4];
  __shared__ int s_last;
  for (int b = threadIdx.x; b < NBINS; b += blockDim.x) sh_hist[b] = 0;
  const int chunk = blockIdx.x / p.parts, part = blockIdx.x - chunk * p.parts;
  const int c0 = chunk * p.chunk_rows, c1 = min(p.rows, c0 + p.chunk_rows);
  const int nlines = (p.n + SAMPLE_LINE - 1) / SAMPLE_LINE;
  // A group of RP threads owns one 64-column line position and a subset of the rows sampled there, so the basis rows of
  // its columns are loaded once and the row loads (4 in flight per thread) are independent of one another.
  constexpr int SU = 4;
  const int groups = blockDim.x / RP, gid = threadIdx.x / RP, sub = threadIdx.x - gid * RP;
  const int G = p.parts * groups;                       // groups working on this chunk
  const int nslots = G / nlines > 0 ? G / nlines : 1;   // row subsets per line position
  const int tasks = nlines * nslots;
  __syncthreads();
  for (int tk = part * groups + gid; tk < tasks; tk += G) {
    const int line = tk % nlines, slot = tk / nlines;
    const int col = line * SAMPLE_LINE + sub * CPT;
    if (col >= p.n) continue;
    float qreg[CPT][RP];
    load_q<RP, CPT>(p.q, p.r, col, p.n, qreg);
    const int first = c0 + ((SAMPLE_STRIDE - ((line + c0) % SAMPLE_STRIDE)) % SAMPLE_STRIDE) + slot * SAMPLE_STRIDE;
    const int step = SAMPLE_STRIDE * nslots;
    for (int row = first; row < c1; row += step * SU) {
      XVec<CPT> xv[SU];
      CVec<RP> cv[SU];
#pragma unroll
      for (int u = 0; u < SU; ++u) {
        const int rr = row + u * step;
        if (rr < c1) {
          xv[u] = load_x<CPT>(p.x + static_cast<size_t>(rr) * p.ldx, col, p.n);
          cv[u] = load_c<RP>(p.c + static_cast<size_t>(rr) * p.r, p.r);
        }
      }
#pragma unroll
      for (int u = 0; u < SU; ++u) {
        const int rr = row + u * step;
        if (rr >= c1) continue;
        float e[CPT];
        residual_row<RP, CPT>(xv[u], cv[u], qreg, e);
#pragma unroll
        for (int i = 0; i < CPT; ++i) {
          if (col + i < p.n) {
            const unsigned short key = __bfloat16_as_ushort(__float2bfloat16_rn(e[i])) & 0x7FFF;
            atomicAdd(&sh_hist[key], 1u);
          }
        }
      }
    }
  }
  __syncthreads();
  unsigned int* gh = p.hist + static_cast<size_t>(chunk) * NBINS;
  for (int b = threadIdx.x; b < NBINS; b += blockDim.x) {
    const unsigned int v = sh_hist[b];
    if (v) atomicAdd(&gh[b], v);
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(&sp.done_a[chunk], 1) == p.parts - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // the sample is complete: scale the wanted count to the sample, add the margin, find the candidate bin
  hist_stage(gh, sh_hist, s_part, s_out);
  const unsigned int sampled = s_part[0];
  const long long elems = static_cast<long long>(c1 - c0) * p.n;
  const int quota = p.quota[chunk];
  unsigned int want = 0;
  if (quota > 0 && elems > 0) {
    const double est = static_cast<double>(quota) * static_cast<double>(sampled) / static_cast<double>(elems);
    want = static_cast<unsigned int>(est * sp.margin[chunk]) + 8u;
  }
  hist_locate(sh_hist, s_part, want, s_out);
  if (threadIdx.x == 0) {
    // fewer sampled entries than wanted: every entry is a candidate (the list will overflow and the chunk falls back)
    sp.cand_bin[chunk] = quota <= 0 ? NBINS : (s_out[0] < 0 ? 0 : s_out[0]);
  }
}

// Tensor-core helpers of the full pass.  E = X - C Q^T for a 16-row x 8-column tile is one warp-level MMA with the
// negated coefficients as A, the basis as B and X itself as the incoming accumulator: rank 8 is exactly the K of
// m16n8k8, ranks up to 16 and 32 take one and two m16n8k16.  (The fifth-generation tcgen05 path needs K >= 16 operands
// in shared memory behind descriptors and its accumulator in tensor memory, which cannot be preloaded with X from global
// memory without a round trip through registers; for a K of 8 to 32 whose only purpose is to take 8 to 32 FMAs per element
// off the issue slots of a bandwidth-bound pass, the register-operand form is the right tool.)
__device__ __forceinline__ void mma_k8(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5}, {%6}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(b0));
}
__device__ __forceinline__ void mma_k16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// Two consecutive basis coefficients q[col, k], q[col, k + 1] as a bf16x2 word (zero past the rank or the last column).
__device__ __forceinline__ uint32_t q_pair(const __nv_bfloat16* q, int r, int n, int col, int k, bool vec) {
  if (col >= n) return 0u;
  const __nv_bfloat16* row = q + static_cast<size_t>(col) * r;
  if (vec) return __ldg(reinterpret_cast<const uint32_t*>(row + k));
  const uint32_t lo = (k < r) ? __bfloat16_as_ushort(row[k]) : 0u;
  const uint32_t hi = (k + 1 < r) ? __bfloat16_as_ushort(row[k + 1]) : 0u;
  return lo | (hi << 16);
}
__device__ __forceinline__ uint32_t word_of(const uint4& v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

// Pass C.  A warp owns 64-column blocks; for each it keeps the basis fragments in registers and walks the CTA's rows
// 32 at a time.  Within a block thread t of a quad owns columns [8t, 8t+8) and [32+8t, 32+8t+8) of each of its rows (two
// 16-byte loads per row), and the MMA's column index is mapped onto those physical columns, so the loads are full
// sectors and the accumulator registers already hold the thread's own columns.
//
// The tensor-core result only *detects*: a compare per element sets a bit in a per-thread mask (no branch in the tile
// loop).  After 32 rows the marked positions of the whole warp are enumerated into the warp's staging slice as
// (row, column) pairs with ballot prefix sums, and the lanes then recompute those few entries, one each, with the chained
// FMA arithmetic of the exact passes, so the stored values are bit-identical to theirs.  Detection uses a cut a little
// below the bin edge to absorb the difference between the two summation orders; the final threshold has to lie strictly
// above the candidate bin for the chunk to count as served, so an entry missed at the very edge can never matter.
template <int RP>
__global__ void __launch_bounds__(512, 1) residual_candidates_kernel(const Select2Params sp) {
  constexpr unsigned FULL = 0xffffffffu;
  constexpr int HW = RP / 2;     // 32-bit words per staged coefficient row
  constexpr int KB = RP / 8;     // basis registers per 8-column tile
  const SelectParams& p = sp.base;
  extern __shared__ unsigned char sh_raw[];
  __shared__ unsigned int s_part[SCAN_T];
  __shared__ int s_out[4];
  __shared__ int s_last;
  // Candidate magnitudes crowd into the few hundred bins just above the cut.  Counting them with global atomics makes
  // every CTA hammer the same few addresses (the hottest bin alone gets ~10^4 serialised updates); instead each CTA counts
  // a window of HWIN bins above the candidate bin in shared memory and adds its totals once at the end.
  constexpr int HWIN = 2048;
  __shared__ unsigned int s_win[HWIN];
  const int nwarps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const unsigned lane_lt = (1u << lane) - 1u;
  for (int b = threadIdx.x; b < HWIN; b += blockDim.x) s_win[b] = 0u;
  unsigned long long* st_rc_all = reinterpret_cast<unsigned long long*>(sh_raw);      // (row << 32) | column
  uint32_t* s_cb = reinterpret_cast<uint32_t*>(sh_raw + static_cast<size_t>(16) * WARP_CAP * 10);  // [CS_ROWS][HW] negated bf16 pairs
  unsigned long long* st_rc = st_rc_all + static_cast<size_t>(warp) * WARP_CAP;
  const Slab s = slab_of(p);
  const int t_lo = sp.cand_bin[s.chunk];
  const int cap = sp.cand_cap[s.chunk];
  const int cbase = sp.cand_off[s.chunk];
  unsigned int* h2 = sp.hist2 + static_cast<size_t>(s.chunk) * NBINS;
  // |e| below `cut` cannot round to a magnitude >= t_lo; detection compares against 0.998 of it
  float cut;
  if (t_lo >= NBINS) cut = __int_as_float(0x7f800000);   // nothing is wanted
  else if (t_lo > 0) cut = 0.5f * (bf16_bits_to_float(static_cast<unsigned short>(t_lo)) + bf16_bits_to_float(static_cast<unsigned short>(t_lo - 1)));
  else cut = 0.f;
  if (sp.fixed_cut >= 0.f) cut = sp.fixed_cut;
  const float detect = cut * 0.998f;
  const bool qvec = (p.r == RP);   // basis rows are RP * 2 bytes: pairs are 4-byte aligned
  int wbase = (t_lo >= NBINS) ? 0 : (t_lo > 0 ? t_lo - 1 : 0);   // first bin of the shared window
  if (sp.fixed_cut >= 0.f) {
    const int ck = __bfloat16_as_ushort(__float2bfloat16_rn(detect)) & 0x7FFF;
    wbase = ck > 0 ? ck - 1 : 0;
  }
  int lmax = 0;
  int wcnt = 0;                    // entries staged by this warp: the same value in every lane
  auto count_key = [&](int key) {
    const int w = key - wbase;
    if (w >= 0 && w < HWIN) atomicAdd(&s_win[w], 1u);
    else atomicAdd(&h2[key], 1u);
    lmax = max(lmax, key);
  };

  auto append = [&](long long flat, unsigned short b16) {  // one lane, straight to the list
    count_key(b16 & 0x7FFF);
    const int o = atomicAdd(&sp.cand_count[s.chunk], 1);
    if (o < cap) {
      sp.cand_idx[cbase + o] = flat;
      sp.cand_val[cbase + o] = b16;
    }
  };
  // bf16 bits of one residual entry with the arithmetic of the exact passes (same operands, same order)
  auto exact_bits = [&](int row, int col) -> unsigned short {
    const __nv_bfloat16* qrow = p.q + static_cast<size_t>(col) * p.r;
    const __nv_bfloat16* crow = p.c + static_cast<size_t>(row) * p.r;
    float cf[RP], qf[RP];
    if (qvec) {
#pragma unroll
      for (int v = 0; v < RP / 8; ++v) {
        const uint4 cw = __ldg(reinterpret_cast<const uint4*>(crow) + v), qw = __ldg(reinterpret_cast<const uint4*>(qrow) + v);
        const uint32_t c4[4] = {cw.x, cw.y, cw.z, cw.w}, q4[4] = {qw.x, qw.y, qw.z, qw.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          cf[8 * v + 2 * k] = __uint_as_float(c4[k] << 16);
          cf[8 * v + 2 * k + 1] = __uint_as_float(c4[k] & 0xFFFF0000u);
          qf[8 * v + 2 * k] = __uint_as_float(q4[k] << 16);
          qf[8 * v + 2 * k + 1] = __uint_as_float(q4[k] & 0xFFFF0000u);
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < RP; ++j) {
        cf[j] = (j < p.r) ? __bfloat162float(crow[j]) : 0.f;
        qf[j] = (j < p.r) ? __bfloat162float(qrow[j]) : 0.f;
      }
    }
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < RP; ++j) acc = fmaf(cf[j], qf[j], acc);
    const float x = __bfloat162float(p.x[static_cast<size_t>(row) * p.ldx + col]);
    return __bfloat16_as_ushort(__float2bfloat16_rn(x - acc));
  };
  auto flush = [&]() {  // whole warp, converged: recompute the staged positions exactly, count them, append them to the list
    __syncwarp();
    const int cnt = min(wcnt, WARP_CAP);
    if (cnt > 0) {
      int base = 0;
      if (lane == 0) base = atomicAdd(&sp.cand_count[s.chunk], cnt);
      base = __shfl_sync(FULL, base, 0);
      for (int i = lane; i < cnt; i += 32) {
        const unsigned long long rc = st_rc[i];
        const int row = static_cast<int>(rc >> 32), col = static_cast<int>(rc & 0xffffffffu);
        const unsigned short b16 = exact_bits(row, col);
        count_key(b16 & 0x7FFF);
        if (base + i < cap) {
          sp.cand_idx[cbase + base + i] = static_cast<long long>(row) * p.n + col;
          sp.cand_val[cbase + base + i] = b16;
        }
      }
    }
    __syncwarp();
    wcnt = 0;
  };

  const int nblocks = (p.n + 63) / 64;
  for (int sb0 = s.row0; sb0 < s.row1; sb0 += CS_ROWS) {
    const int sb1 = min(s.row1, sb0 + CS_ROWS);
    __syncthreads();  // the previous sub-slab's coefficients are no longer being read
    for (int i = threadIdx.x; i < CS_ROWS * HW; i += blockDim.x) {
      const int lr = i / HW, k = 2 * (i - lr * HW);
      const int row = sb0 + lr;
      uint32_t lo = 0u, hi = 0u;
      if (row < sb1) {
        const __nv_bfloat16* crow = p.c + static_cast<size_t>(row) * p.r;
        if (k < p.r) lo = __bfloat16_as_ushort(crow[k]);
        if (k + 1 < p.r) hi = __bfloat16_as_ushort(crow[k + 1]);
      }
      s_cb[i] = (lo | (hi << 16)) ^ 0x80008000u;  // A = -C
    }
    __syncthreads();
    const int npairs = (sb1 - sb0 + 31) / 32;
    for (int cb = warp; cb < nblocks; cb += nwarps) {
      const int n0 = cb * 64;
      uint32_t bq[8][KB];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        // the tile's column index g belongs to quad thread g / 2, element g % 2 of its j-th column pair
        const int pc = n0 + (j < 4 ? 8 * (g >> 1) + 2 * j : 32 + 8 * (g >> 1) + 2 * (j - 4)) + (g & 1);
#pragma unroll
        for (int kb = 0; kb < KB; ++kb) bq[j][kb] = q_pair(p.q, p.r, p.n, pc, 2 * t + 8 * kb, qvec);
      }
      const bool lo_ok = n0 + 8 * t + 8 <= p.n, hi_ok = n0 + 32 + 8 * t + 8 <= p.n;
      for (int sp2 = 0; sp2 < npairs; ++sp2) {
        if (wcnt > WARP_CAP / 2) flush();
        uint4 raw[2][4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int rtop = sb0 + sp2 * 32 + h * 16 + g, rbot = rtop + 8;
          const __nv_bfloat16* xt = p.x + static_cast<size_t>(rtop) * p.ldx + n0 + 8 * t;
          const __nv_bfloat16* xb = p.x + static_cast<size_t>(rbot) * p.ldx + n0 + 8 * t;
          const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
          raw[h][0] = (rtop < sb1 && lo_ok) ? __ldg(reinterpret_cast<const uint4*>(xt)) : zero;
          raw[h][1] = (rtop < sb1 && hi_ok) ? __ldg(reinterpret_cast<const uint4*>(xt + 32)) : zero;
          raw[h][2] = (rbot < sb1 && lo_ok) ? __ldg(reinterpret_cast<const uint4*>(xb)) : zero;
          raw[h][3] = (rbot < sb1 && hi_ok) ? __ldg(reinterpret_cast<const uint4*>(xb + 32)) : zero;
        }
        unsigned marks[2] = {0u, 0u};   // bit 4 * j + q of marks[h]: accumulator q of tile j of strip h reaches the cut
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int lr = sp2 * 32 + h * 16 + g;
          uint32_t a[RP / 4];
          if constexpr (RP == 8) {
            a[0] = s_cb[lr * HW + t];
            a[1] = s_cb[(lr + 8) * HW + t];
          } else {
#pragma unroll
            for (int ks = 0; ks < RP / 16; ++ks) {
              a[4 * ks + 0] = s_cb[lr * HW + 8 * ks + t];
              a[4 * ks + 1] = s_cb[(lr + 8) * HW + 8 * ks + t];
              a[4 * ks + 2] = s_cb[lr * HW + 8 * ks + t + 4];
              a[4 * ks + 3] = s_cb[(lr + 8) * HW + 8 * ks + t + 4];
            }
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint32_t wt = word_of(raw[h][j < 4 ? 0 : 1], j & 3);
            const uint32_t wb = word_of(raw[h][j < 4 ? 2 : 3], j & 3);
            float d[4] = {__uint_as_float(wt << 16), __uint_as_float(wt & 0xFFFF0000u), __uint_as_float(wb << 16), __uint_as_float(wb & 0xFFFF0000u)};
            if constexpr (RP == 8) {
              mma_k8(d, a[0], a[1], bq[j][0]);
            } else {
#pragma unroll
              for (int ks = 0; ks < RP / 16; ++ks) mma_k16(d, a[4 * ks], a[4 * ks + 1], a[4 * ks + 2], a[4 * ks + 3], bq[j][2 * ks], bq[j][2 * ks + 1]);
            }
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4)
              if (!(fabsf(d[q4]) < detect)) marks[h] |= 1u << (4 * j + q4);
          }
        }
        // enumerate the marked positions of the warp into its staging slice (their values are computed at the flush)
        unsigned long long m = static_cast<unsigned long long>(marks[0]) | (static_cast<unsigned long long>(marks[1]) << 32);
        while (__any_sync(FULL, m != 0ull)) {
          bool has = m != 0ull;
          int row = 0, col = 0;
          if (has) {
            const int bit = __ffsll(static_cast<long long>(m)) - 1;
            m &= m - 1ull;
            const int h = bit >> 5, j = (bit >> 2) & 7, q4 = bit & 3;
            row = sb0 + sp2 * 32 + h * 16 + g + ((q4 & 2) ? 8 : 0);
            col = n0 + (j < 4 ? 8 * t + 2 * j : 32 + 8 * t + 2 * (j - 4)) + (q4 & 1);
            has = row < sb1 && col < p.n;
          }
          const unsigned vm = __ballot_sync(FULL, has);
          const int pos = wcnt + __popc(vm & lane_lt);
          if (has) {
            if (pos < WARP_CAP) {
              st_rc[pos] = (static_cast<unsigned long long>(static_cast<unsigned>(row)) << 32) | static_cast<unsigned>(col);
            } else {  // staging slice full (a very dense stretch): this lane finishes its entry on its own
              append(static_cast<long long>(row) * p.n + col, exact_bits(row, col));
            }
          }
          wcnt = min(WARP_CAP, wcnt + __popc(vm));
        }
      }
    }
  }
  flush();
#pragma unroll
  for (int off = 16; off; off >>= 1) lmax = max(lmax, __shfl_xor_sync(FULL, lmax, off));
  if (lane == 0 && lmax > 0) atomicMax(sp.gmax, lmax);
  __syncthreads();
  for (int b = threadIdx.x; b < HWIN; b += blockDim.x) {
    const unsigned int v = s_win[b];
    if (v) atomicAdd(&h2[wbase + b], v);
  }

  // ---- tail: the last CTA of the chunk finds the exact threshold among the candidates; the last CTA of all sets the scale
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    s_last = (atomicAdd(&sp.done_c[s.chunk], 1) == p.parts - 1) ? 1 : 0;
    if (atomicAdd(sp.done_all, 1) == static_cast<int>(gridDim.x) - 1) {
      __threadfence();
      const int mb = *reinterpret_cast<volatile int*>(sp.gmax);
      const float amax = bf16_bits_to_float(static_cast<unsigned short>(mb));
      const float qmax = (p.bits == 4) ? 7.f : 127.f;
      *p.out_scale = (p.bits == 0) ? 1.f : fmaxf(amax / qmax, 1.17549435e-38f);
    }
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const int quota = p.quota[s.chunk];
  unsigned int* sh_hist = reinterpret_cast<unsigned int*>(sh_raw);  // the staging slices are idle now: 128 KB for the histogram
  hist_stage(h2, sh_hist, s_part, s_out);
  hist_locate(sh_hist, s_part, quota > 0 ? static_cast<unsigned int>(quota) : 0u, s_out);
  const int appended = *reinterpret_cast<volatile int*>(&sp.cand_count[s.chunk]);
  // served only when the threshold bin lies strictly above the candidate bin (whose lower part detection may have missed)
  const bool valid = quota <= 0 || (s_out[0] > t_lo && appended <= cap);
  if (threadIdx.x == 0) {
    p.thr_bin[s.chunk] = quota <= 0 ? NBINS : s_out[0];
    p.thr_need[s.chunk] = s_out[1];
    p.max_bin[s.chunk] = s_out[2] < 0 ? 0 : s_out[2];
    p.tie_count[s.chunk] = 0;
    p.out_count[s.chunk] = 0;
    sp.fallback[s.chunk] = valid ? 0 : 1;
  }
  if (!valid) {  // the exact passes will histogram this chunk from scratch
    unsigned int* gh = p.hist + static_cast<size_t>(s.chunk) * NBINS;
    for (int b = threadIdx.x; b < NBINS; b += blockDim.x) gh[b] = 0u;
  }
}

// Pass E: compaction of the candidate lists.  A CTA takes 1024 candidates at a time, decides, and reserves its output
// range with one atomic (the positions inside it come from a CTA-wide prefix sum).
constexpr int CE_ITEMS = 4;
__global__ void __launch_bounds__(256) candidates_compact_kernel(const Select2Params sp, int ctas_per_chunk) {
  constexpr unsigned FULL = 0xffffffffu;
  const SelectParams& p = sp.base;
  __shared__ int s_warp[8];
  __shared__ int s_base;
  const int chunk = blockIdx.x / ctas_per_chunk, part = blockIdx.x - chunk * ctas_per_chunk;
  if (sp.fallback[chunk]) return;
  const int thr = p.thr_bin[chunk], need = p.thr_need[chunk], quota = p.quota[chunk], obase = p.out_offset[chunk];
  const int count = min(sp.cand_count[chunk], sp.cand_cap[chunk]);
  const int cbase = sp.cand_off[chunk];
  const float inv_scale = 1.f / *p.out_scale;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int SPAN = 256 * CE_ITEMS;
  for (int base0 = part * SPAN; base0 < count; base0 += ctas_per_chunk * SPAN) {
    unsigned short b16[CE_ITEMS];
    bool take[CE_ITEMS];
    int mine = 0;
#pragma unroll
    for (int it = 0; it < CE_ITEMS; ++it) {
      const int i = base0 + it * 256 + static_cast<int>(threadIdx.x);
      take[it] = false;
      b16[it] = 0;
      if (i < count) {
        b16[it] = sp.cand_val[cbase + i];
        const int key = b16[it] & 0x7FFF;
        take[it] = key > thr;
        if (!take[it] && key == thr && need > 0) take[it] = atomicAdd(&p.tie_count[chunk], 1) < need;
      }
      mine += take[it] ? 1 : 0;
    }
    int incl = mine;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int v = __shfl_up_sync(FULL, incl, off);
      if (lane >= off) incl += v;
    }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    if (threadIdx.x == 0) {
      int total = 0;
      for (int w = 0; w < 8; ++w) {
        const int c = s_warp[w];
        s_warp[w] = total;
        total += c;
      }
      s_base = total > 0 ? atomicAdd(&p.out_count[chunk], total) : 0;
    }
    __syncthreads();
    int o = s_base + s_warp[warp] + incl - mine;
#pragma unroll
    for (int it = 0; it < CE_ITEMS; ++it) {
      if (take[it]) {
        const int i = base0 + it * 256 + static_cast<int>(threadIdx.x);
        if (o < quota) emit_entry(p, obase + o, sp.cand_idx[cbase + i], b16[it], inv_scale);
        ++o;
      }
    }
    __syncthreads();  // s_warp and s_base are rewritten by the next round
  }
}

template <int RP>
static int launch_select(const SelectParams& p, int phase, cudaStream_t st) {
  constexpr int CPT = 64 / RP;
  int ctn = (p.n + CPT - 1) / CPT;
  if (ctn > 512) ctn = 512;
  int rl = 512 / ctn;
  if (rl < 1) rl = 1;
  const int threads = ((ctn * rl + 31) / 32) * 32;
  const int grid = p.nchunks * p.parts;
  // the shared-memory opt-in is a per-device function attribute: remember it per device, not per process
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return -8;
  if (phase == 0) {
    static bool cfg[MAX_DEVICES] = {false};
    if (!cfg[dev]) {
      cudaError_t e = cudaFuncSetAttribute(residual_hist_kernel<RP>, cudaFuncAttributeMaxDynamicSharedMemorySize, NBINS * 4 + CS_ROWS * RP * 4);
      if (e != cudaSuccess) return static_cast<int>(e);
      cfg[dev] = true;
    }
    residual_hist_kernel<RP><<<grid, threads, NBINS * 4 + CS_ROWS * RP * 4, st>>>(p, ctn, rl);
  } else {
    const int smem = 16 * WARP_CAP * (8 + 2) + CS_ROWS * RP * 4;
    static bool cfg[MAX_DEVICES] = {false};
    if (!cfg[dev]) {
      cudaError_t e = cudaFuncSetAttribute(residual_compact_kernel<RP>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) return static_cast<int>(e);
      cfg[dev] = true;
    }
    residual_compact_kernel<RP><<<grid, threads, smem, st>>>(p, ctn, rl);
  }
  return static_cast<int>(cudaGetLastError());
}

template <int RP>
static int launch_candidates_only(const Select2Params& sp, cudaStream_t st) {
  const SelectParams& p = sp.base;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return -8;
  int smem_c = 16 * WARP_CAP * (8 + 2) + CS_ROWS * RP * 2;
  if (smem_c < NBINS * 4) smem_c = NBINS * 4;
  static bool cfg[MAX_DEVICES] = {false};
  if (!cfg[dev]) {
    cudaError_t e = cudaFuncSetAttribute(residual_candidates_kernel<RP>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_c);
    if (e != cudaSuccess) return static_cast<int>(e);
    cfg[dev] = true;
  }
  residual_candidates_kernel<RP><<<p.nchunks * p.parts, 512, smem_c, st>>>(sp);
  return static_cast<int>(cudaGetLastError());
}

template <int RP>
static int launch_sampled(const Select2Params& sp, int max_cap, cudaStream_t st) {
  const SelectParams& p = sp.base;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return -8;
  const int grid = p.nchunks * p.parts;
  const int smem_a = NBINS * 4;
  int smem_c = 16 * WARP_CAP * (8 + 2) + CS_ROWS * RP * 2;
  if (smem_c < NBINS * 4) smem_c = NBINS * 4;   // the tail scan stages the candidate histogram where the staging slices were
  static bool cfg[MAX_DEVICES] = {false};
  if (!cfg[dev]) {
    cudaError_t e = cudaFuncSetAttribute(residual_sample_kernel<RP>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_a);
    if (e != cudaSuccess) return static_cast<int>(e);
    e = cudaFuncSetAttribute(residual_candidates_kernel<RP>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_c);
    if (e != cudaSuccess) return static_cast<int>(e);
    cfg[dev] = true;
  }
  residual_sample_kernel<RP><<<grid, 512, smem_a, st>>>(sp);
  residual_candidates_kernel<RP><<<grid, 512, smem_c, st>>>(sp);
  int per_chunk = (max_cap + 256 * CE_ITEMS - 1) / (256 * CE_ITEMS);
  if (per_chunk < 1) per_chunk = 1;
  if (per_chunk > 2048) per_chunk = 2048;
  candidates_compact_kernel<<<p.nchunks * per_chunk, 256, 0, st>>>(sp, per_chunk);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace sb

// Exact top-k selection of the residual by magnitude, per row chunk.
//   work: int32 scratch of 6 * nchunks entries (thr_bin, thr_need, max_bin, tie_count, out_count);
//   hist: uint32 [nchunks, 32768], zeroed by the caller;
//   quota / out_offset: int32 [nchunks] on the device;
//   idx32 or idx64 (one non-null) and val (bf16 when bits == 0, int8 when bits == 8) have
//   sum(quota) entries; scale is one fp32.
extern "C" int sb_residual_topk(const void* x, const void* c, const void* q, int rows, int n, int r, int ldx,
                                int chunk_rows, int nchunks, int parts, void* hist, int* work, const int* quota,
                                const int* out_offset, int bits, int* idx32, long long* idx64, void* val,
                                float* scale, int* status, void* stream) {
  using namespace sb;
  if (rows <= 0 || n <= 0 || nchunks <= 0) return 0;
  if (r < 1 || r > 32) return -2;
  if ((ldx & 7) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(c) & 15)) return -3;
  SelectParams p;
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.c = static_cast<const __nv_bfloat16*>(c);
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.rows = rows; p.n = n; p.r = r; p.ldx = ldx;
  p.chunk_rows = chunk_rows; p.parts = parts; p.nchunks = nchunks;
  p.hist = static_cast<unsigned int*>(hist);
  p.thr_bin = work; p.thr_need = work + nchunks; p.max_bin = work + 2 * nchunks;
  p.tie_count = work + 3 * nchunks; p.out_count = work + 4 * nchunks;
  p.quota = quota; p.out_offset = out_offset;
  p.bits = bits; p.out_idx32 = idx32; p.out_idx64 = idx64; p.out_val = val; p.out_scale = scale;
  p.status = status;
  p.gate = nullptr;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int rc;
  const int rp = r <= 8 ? 8 : (r <= 16 ? 16 : 32);
  rc = rp == 8 ? launch_select<8>(p, 0, st) : rp == 16 ? launch_select<16>(p, 0, st) : launch_select<32>(p, 0, st);
  if (rc) return rc;
  residual_scan_kernel<<<nchunks, 1024, 0, st>>>(p);
  residual_scale_kernel<<<1, 32, 0, st>>>(p);
  rc = static_cast<int>(cudaGetLastError());
  if (rc) return rc;
  rc = rp == 8 ? launch_select<8>(p, 1, st) : rp == 16 ? launch_select<16>(p, 1, st) : launch_select<32>(p, 1, st);
  return rc;
}

// Sampled-threshold form of sb_residual_topk (see the comment above residual_sample_kernel).  Extra arguments:
//   hist2     uint32 [nchunks, 32768], zeroed by the caller like hist;
//   work      int32 [12 * nchunks + 2], zeroed by the caller;
//   cand_off / cand_cap  int32 [nchunks]: slot range of each chunk's candidate list inside cand_idx / cand_val;
//   margin    fp32 [nchunks]: safety factor applied to the sample's estimate of the candidate count;
//   cand_idx  int64 [sum cand_cap], cand_val uint16 [sum cand_cap]; max_cap = the largest cand_cap (sizes pass E's grid).
// n must be a multiple of 8 (16-byte row segments).
extern "C" int sb_residual_topk_sampled(const void* x, const void* c, const void* q, int rows, int n, int r, int ldx, int chunk_rows,
                                        int nchunks, int parts, void* hist, void* hist2, int* work, const int* quota,
                                        const int* out_offset, const int* cand_off, const int* cand_cap, const float* margin,
                                        long long* cand_idx, void* cand_val, int max_cap, int bits, int* idx32, long long* idx64,
                                        void* val, float* scale, int* status, void* stream) {
  using namespace sb;
  if (rows <= 0 || n <= 0 || nchunks <= 0) return 0;
  if (r < 1 || r > 32) return -2;
  if ((ldx & 7) || (n & 7) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(c) & 15)) return -3;
  Select2Params sp;
  SelectParams& p = sp.base;
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.c = static_cast<const __nv_bfloat16*>(c);
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.rows = rows; p.n = n; p.r = r; p.ldx = ldx;
  p.chunk_rows = chunk_rows; p.parts = parts; p.nchunks = nchunks;
  p.hist = static_cast<unsigned int*>(hist);
  p.thr_bin = work; p.thr_need = work + nchunks; p.max_bin = work + 2 * nchunks;
  p.tie_count = work + 3 * nchunks; p.out_count = work + 4 * nchunks;
  sp.cand_bin = work + 5 * nchunks; sp.cand_count = work + 6 * nchunks; sp.fallback = work + 7 * nchunks;
  sp.done_a = work + 8 * nchunks; sp.done_c = work + 9 * nchunks;
  sp.done_all = work + 12 * nchunks; sp.gmax = work + 12 * nchunks + 1;
  p.quota = quota; p.out_offset = out_offset;
  p.bits = bits; p.out_idx32 = idx32; p.out_idx64 = idx64; p.out_val = val; p.out_scale = scale;
  p.status = status;
  p.gate = sp.fallback;
  sp.hist2 = static_cast<unsigned int*>(hist2);
  sp.cand_off = cand_off; sp.cand_cap = cand_cap; sp.margin = margin;
  sp.cand_idx = cand_idx; sp.cand_val = static_cast<unsigned short*>(cand_val);
  sp.fixed_cut = -1.f;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int rp = r <= 8 ? 8 : (r <= 16 ? 16 : 32);
  int rc = rp == 8 ? launch_sampled<8>(sp, max_cap, st) : rp == 16 ? launch_sampled<16>(sp, max_cap, st) : launch_sampled<32>(sp, max_cap, st);
  if (rc) return rc;
  // exact passes, gated per chunk by the fallback flags (they return at once for chunks the sampled passes served)
  rc = rp == 8 ? launch_select<8>(p, 0, st) : rp == 16 ? launch_select<16>(p, 0, st) : launch_select<32>(p, 0, st);
  if (rc) return rc;
  residual_scan_kernel<<<nchunks, 1024, 0, st>>>(p);
  rc = static_cast<int>(cudaGetLastError());
  if (rc) return rc;
  return rp == 8 ? launch_select<8>(p, 1, st) : rp == 16 ? launch_select<16>(p, 1, st) : launch_select<32>(p, 1, st);
}

// Every residual entry with |e| >= cut, as (flat index, bf16 bits) pairs in cand_idx / cand_val (capacity cap; entries
// beyond it are counted but dropped).  work: int32 [14] zeroed by the caller, work[6] returns the number found;
// hist2: uint32 [32768] zeroed (receives the magnitude histogram of what was found); meta: int32 [4] = {0, 0, 0, cap}.
// One pass over X on the tensor-core residual kernel of the sampled selection; n % 8 == 0.
extern "C" int sb_residual_above(const void* x, const void* c, const void* q, int rows, int n, int r, int ldx, float cut, int parts, void* hist,
                                 void* hist2, int* work, const int* meta, long long* cand_idx, void* cand_val, float* scale, int* status,
                                 void* stream) {
  using namespace sb;
  if (rows <= 0 || n <= 0) return 0;
  if (r < 1 || r > 32 || cut < 0.f) return -2;
  if ((ldx & 7) || (n & 7) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(c) & 15)) return -3;
  Select2Params sp;
  SelectParams& p = sp.base;
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.c = static_cast<const __nv_bfloat16*>(c);
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.rows = rows; p.n = n; p.r = r; p.ldx = ldx;
  p.chunk_rows = rows; p.parts = parts; p.nchunks = 1;
  p.hist = static_cast<unsigned int*>(hist);
  p.thr_bin = work; p.thr_need = work + 1; p.max_bin = work + 2; p.tie_count = work + 3; p.out_count = work + 4;
  sp.cand_bin = work + 5; sp.cand_count = work + 6; sp.fallback = work + 7; sp.done_a = work + 8; sp.done_c = work + 9;
  sp.done_all = work + 12; sp.gmax = work + 13;
  p.quota = meta; p.out_offset = meta + 1;          // quota 0: the tail computes no threshold
  p.bits = 0; p.out_idx32 = nullptr; p.out_idx64 = nullptr; p.out_val = nullptr; p.out_scale = scale;
  p.status = status; p.gate = nullptr;
  sp.hist2 = static_cast<unsigned int*>(hist2);
  sp.cand_off = meta + 2; sp.cand_cap = meta + 3; sp.margin = nullptr;
  sp.cand_idx = cand_idx; sp.cand_val = static_cast<unsigned short*>(cand_val);
  sp.fixed_cut = cut;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int rp = r <= 8 ? 8 : (r <= 16 ? 16 : 32);
  return rp == 8 ? launch_candidates_only<8>(sp, st) : rp == 16 ? launch_candidates_only<16>(sp, st) : launch_candidates_only<32>(sp, st);
}

extern "C" int sb_residual_gather(const void* x, const void* c, const void* q, int n, int r, int ldx,
                                  const long long* idx64, const int* idx32, long long count, void* out, void* stream) {
  if (count <= 0) return 0;
  const int threads = 256;
  const long long blocks = (count + threads - 1) / threads;
  sb::residual_gather_kernel<<<static_cast<unsigned>(blocks), threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(c), static_cast<const __nv_bfloat16*>(q), n, r,
      ldx, idx64, idx32, count, static_cast<__nv_bfloat16*>(out));
  return static_cast<int>(cudaGetLastError());
}

extern "C" int sb_residual_block_energy(const void* x, const void* c, const void* q, int rows, int n, int r, int ldx,
                                        int bs, float* energy, void* stream) {
  if (rows <= 0) return 0;
  if (bs % 8 || bs > 256 || (bs & (bs - 1)) || n % bs) return -2;
  if (r < 1 || r > 32) return -2;
  dim3 grid((rows + sb::BE_ROWS - 1) / sb::BE_ROWS, (n / 8 + 255) / 256);
  const __nv_bfloat16* xb = static_cast<const __nv_bfloat16*>(x);
  const __nv_bfloat16* cb = static_cast<const __nv_bfloat16*>(c);
  const __nv_bfloat16* qb = static_cast<const __nv_bfloat16*>(q);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (r <= 8)
    sb::residual_block_energy_kernel<8><<<grid, 256, 0, st>>>(xb, cb, qb, rows, n, r, ldx, bs, energy);
  else if (r <= 16)
    sb::residual_block_energy_kernel<16><<<grid, 256, 0, st>>>(xb, cb, qb, rows, n, r, ldx, bs, energy);
  else
    sb::residual_block_energy_kernel<32><<<grid, 256, 0, st>>>(xb, cb, qb, rows, n, r, ldx, bs, energy);
  return static_cast<int>(cudaGetLastError());
}

// ------------------------------------------------------------------------------------------------
// Allocation-free variant (declared in stacr_noalloc.h).  Scratch lives in a file-scope device
// array; device code names it directly, host code must use the address obtained once per device
// from cudaGetSymbolAddress (the host-side name of a __device__ variable is not a device address).
// ------------------------------------------------------------------------------------------------
#include "stacr_noalloc.h"

namespace sb {

constexpr int NOALLOC_INTS_PER_CHUNK = 8;  // thr_bin, thr_need, max_bin, tie_count, out_count, quota, out_offset, pad
constexpr size_t NOALLOC_HIST_BYTES = static_cast<size_t>(SB_NOALLOC_MAX_CHUNKS) * NBINS * sizeof(unsigned int);
constexpr size_t NOALLOC_BYTES = NOALLOC_HIST_BYTES + SB_NOALLOC_MAX_CHUNKS * NOALLOC_INTS_PER_CHUNK * sizeof(int);

static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_BYTES];

__host__ __device__ inline int noalloc_chunk_quota(int rows, int chunk_rows, int quota_per_chunk, int chunk) {
  const int begin = chunk * chunk_rows;
  const int len = (rows - begin) < chunk_rows ? (rows - begin) : chunk_rows;
  if (len == chunk_rows) return quota_per_chunk;
  long long q = (static_cast<long long>(quota_per_chunk) * len + chunk_rows / 2) / chunk_rows;
  return q < 1 ? 1 : static_cast<int>(q);
}

// Clears the histogram bins and counters of the chunks in use and fills quota / out_offset.
__global__ void noalloc_prepare_kernel(int rows, int chunk_rows, int quota_per_chunk, int nchunks) {
  unsigned int* hist = reinterpret_cast<unsigned int*>(g_noalloc_scratch);
  int* ints = reinterpret_cast<int*>(g_noalloc_scratch + NOALLOC_HIST_BYTES);
  const size_t bins = static_cast<size_t>(nchunks) * NBINS;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < bins; i += static_cast<size_t>(gridDim.x) * blockDim.x)
    hist[i] = 0u;
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    int running = 0;
    for (int c = 0; c < nchunks; ++c) {
      const int quota = noalloc_chunk_quota(rows, chunk_rows, quota_per_chunk, c);
      for (int f = 0; f < 5; ++f) ints[f * SB_NOALLOC_MAX_CHUNKS + c] = 0;
      ints[5 * SB_NOALLOC_MAX_CHUNKS + c] = quota;
      ints[6 * SB_NOALLOC_MAX_CHUNKS + c] = running;
      running += quota;
    }
  }
}

// Device address of the scratch array for the current device, looked up on first use.
static int noalloc_scratch_for_current_device(unsigned char** out) {
  static unsigned char* cached[MAX_DEVICES] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= MAX_DEVICES) return -8;
  if (cached[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    cached[dev] = static_cast<unsigned char*>(ptr);
  }
  *out = cached[dev];
  return 0;
}

}  // namespace sb

extern "C" long long sb_residual_topk_noalloc_count(int rows, int chunk_rows, int quota_per_chunk) {
  if (rows <= 0 || chunk_rows <= 0 || quota_per_chunk < 0) return -1;
  const int nchunks = (rows + chunk_rows - 1) / chunk_rows;
  long long total = 0;
  for (int c = 0; c < nchunks; ++c) total += sb::noalloc_chunk_quota(rows, chunk_rows, quota_per_chunk, c);
  return total;
}

extern "C" int sb_residual_topk_noalloc(const void* x, const void* c, const void* q, int rows, int n, int r, int ldx,
                                        int chunk_rows, int quota_per_chunk, int bits, int* idx32, long long* idx64, void* val,
                                        float* scale, int* status, void* stream) {
  using namespace sb;
  if (rows <= 0 || n <= 0 || chunk_rows <= 0 || quota_per_chunk < 0) return -2;
  if (r < 1 || r > 32) return -2;
  if ((idx32 == nullptr) == (idx64 == nullptr)) return -2;
  // a chunk cannot yield more entries than it has: with a larger quota the tail of idx/val would stay unwritten
  if (static_cast<long long>(quota_per_chunk) > static_cast<long long>(chunk_rows) * n) return -2;
  if ((ldx & 7) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(c) & 15)) return -3;
  const int nchunks = (rows + chunk_rows - 1) / chunk_rows;
  if (nchunks > SB_NOALLOC_MAX_CHUNKS) return -7;  // larger than the built-in scratch: rejected, nothing launched
  unsigned char* scratch = nullptr;
  int rc = noalloc_scratch_for_current_device(&scratch);
  if (rc) return rc;
  int sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int* ints = reinterpret_cast<int*>(scratch + NOALLOC_HIST_BYTES);
  SelectParams p;
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.c = static_cast<const __nv_bfloat16*>(c);
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.rows = rows; p.n = n; p.r = r; p.ldx = ldx;
  p.chunk_rows = chunk_rows; p.nchunks = nchunks;
  p.parts = sms / nchunks > 0 ? sms / nchunks : 1;
  p.hist = reinterpret_cast<unsigned int*>(scratch);
  p.thr_bin = ints; p.thr_need = ints + SB_NOALLOC_MAX_CHUNKS; p.max_bin = ints + 2 * SB_NOALLOC_MAX_CHUNKS;
  p.tie_count = ints + 3 * SB_NOALLOC_MAX_CHUNKS; p.out_count = ints + 4 * SB_NOALLOC_MAX_CHUNKS;
  p.quota = ints + 5 * SB_NOALLOC_MAX_CHUNKS; p.out_offset = ints + 6 * SB_NOALLOC_MAX_CHUNKS;
  p.bits = bits; p.out_idx32 = idx32; p.out_idx64 = idx64; p.out_val = val; p.out_scale = scale; p.status = status;
  p.gate = nullptr;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  noalloc_prepare_kernel<<<64, 256, 0, st>>>(rows, chunk_rows, quota_per_chunk, nchunks);
  rc = static_cast<int>(cudaGetLastError());
  if (rc) return rc;
  const int rp = r <= 8 ? 8 : (r <= 16 ? 16 : 32);
  rc = rp == 8 ? launch_select<8>(p, 0, st) : rp == 16 ? launch_select<16>(p, 0, st) : launch_select<32>(p, 0, st);
  if (rc) return rc;
  residual_scan_kernel<<<nchunks, 1024, 0, st>>>(p);
  residual_scale_kernel<<<1, 32, 0, st>>>(p);
  rc = static_cast<int>(cudaGetLastError());
  if (rc) return rc;
  return rp == 8 ? launch_select<8>(p, 1, st) : rp == 16 ? launch_select<16>(p, 1, st) : launch_select<32>(p, 1, st);
}
