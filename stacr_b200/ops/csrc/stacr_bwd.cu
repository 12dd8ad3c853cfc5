// Factor-native weight gradient of the compressed linear layer:
//
//   dW[o, n] = sum_j T[o, j] Q[n, j]  +  sum_{(row, n, v) in S} v * dY[row, o]
//
// with T = dY^T C produced by the skinny tensor-core GEMM.  The sparse residual arrives as an
// unordered list of (flat index, value); it is bucketed by input feature n with a counting
// sort (count -> scan -> scatter) so that one CTA owns a strip of 8 features and accumulates
// whole output columns in registers: no atomics on dW, one coalesced write per element, and
// the rank-r expansion is fused into the same pass.  The dense X is never rebuilt.
// Replaces the COO build + coalesce + cuSPARSE SpMM + two library GEMMs of the reference
// (stacr/layers.py:173-196 there).
#include <cstdlib>

#include "common.cuh"

namespace sb {

__global__ void col_count_kernel(const int* idx32, const long long* idx64, long long nnz, int n, int* counts) {
  long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= nnz) return;
  const long long flat = idx64 ? idx64[i] : static_cast<long long>(idx32[i]);
  atomicAdd(&counts[static_cast<int>(flat % n)], 1);
}

// Exclusive scan of counts[0..n) into colptr[0..n]; also copies colptr into cursor. One CTA.
// With `parts` != NULL it also plans the weight-gradient kernel: a strip of 8 features whose entries exceed `target`
// is cut into parts[g] = ceil(entries / target) pieces; piece 0 belongs to the strip's own CTA, every further piece
// becomes an item (g, piece) of extra_items so that no CTA walks much more than `target` entries, however skewed
// the distribution of the residual over the features is.  extra_count <= nnz / target.
__global__ void __launch_bounds__(1024) col_scan_kernel(const int* counts, int n, int* colptr, int* cursor, int* parts,
                                                        int* extra_count, int2* extra_items, int target, int max_extra) {
  __shared__ int part[1024];
  const int t = threadIdx.x;
  const int per = (n + 1023) / 1024;
  const int lo = min(n, t * per), hi = min(n, lo + per);
  int sum = 0;
  for (int i = lo; i < hi; ++i) sum += counts[i];
  part[t] = sum;
  __syncthreads();
  for (int off = 1; off < 1024; off <<= 1) {
    int add = (t >= off) ? part[t - off] : 0;
    __syncthreads();
    part[t] += add;
    __syncthreads();
  }
  int run = part[t] - sum;  // exclusive prefix of this thread's range
  for (int i = lo; i < hi; ++i) {
    colptr[i] = run;
    cursor[i] = run;
    run += counts[i];
  }
  if (t == 1023) colptr[n] = part[1023];
  if (parts == nullptr) return;
  __syncthreads();  // colptr is complete and visible to the whole CTA
  const int groups = (n + 7) / 8;
  const int gper = (groups + 1023) / 1024;
  const int glo = min(groups, t * gper), ghi = min(groups, glo + gper);
  int extra = 0;
  for (int g = glo; g < ghi; ++g) {
    const int tot = colptr[min(n, 8 * g + 8)] - colptr[8 * g];
    const int pieces = max(1, (tot + target - 1) / target);
    parts[g] = pieces;
    extra += pieces - 1;
  }
  part[t] = extra;
  __syncthreads();
  for (int off = 1; off < 1024; off <<= 1) {
    int add = (t >= off) ? part[t - off] : 0;
    __syncthreads();
    part[t] += add;
    __syncthreads();
  }
  int slot = part[t] - extra;
  for (int g = glo; g < ghi; ++g) {
    const int pieces = parts[g];
    for (int piece = 1; piece < pieces; ++piece, ++slot)
      if (slot < max_extra) extra_items[slot] = make_int2(g, piece);
  }
  if (t == 1023) *extra_count = min(part[1023], max_extra);
}

__global__ void col_scatter_kernel(const int* idx32, const long long* idx64, long long nnz, int n, const void* val,
                                   int bits, const float* scale, int* cursor, int* rows_sorted, float* vals_sorted) {
  long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= nnz) return;
  const long long flat = idx64 ? idx64[i] : static_cast<long long>(idx32[i]);
  const int col = static_cast<int>(flat % n);
  const int row = static_cast<int>(flat / n);
  float v;
  if (bits == 0) {
    v = __bfloat162float(static_cast<const __nv_bfloat16*>(val)[i]);
  } else if (bits == 8) {
    v = static_cast<float>(static_cast<const signed char*>(val)[i]) * *scale;
  } else {  // two signed nibbles per byte, even element in the low half
    const unsigned char byte = static_cast<const unsigned char*>(val)[i >> 1];
    int nib = (i & 1) ? (byte >> 4) : (byte & 0x0F);
    if (nib > 7) nib -= 16;
    v = static_cast<float>(nib) * *scale;
  }
  const int slot = atomicAdd(&cursor[col], 1);
  rows_sorted[slot] = row;
  vals_sorted[slot] = v;
}

// Where the weight gradient goes when it is not a private tensor.
//   mode 1: accumulate into this GPU's flat gradient buffer (out[i] += v).
//   mode 2: data-parallel reduce-scatter fused into the epilogue.  The flat gradient buffers of all ranks are
//           symmetric memory; the fused region [region_lo, region_lo + 4 * per_vecs * world) is split into `world`
//           contiguous slices and every 16-byte element is added, with one `red.add.v4.f32`, into the copy held by the
//           rank that owns its slice (a peer store over NVLink, or a local one).  After all ranks have finished their
//           backward pass the owner holds the cross-rank sum of its slice; an all-gather kernel then broadcasts it.
struct DwSink {
  int mode;
  int world;
  float scale;
  long long param_off;   // element offset of this parameter inside the flat buffer (multiple of 4)
  long long region_lo;   // element offset of the fused region (multiple of 4)
  long long per_vecs;    // 16-byte elements per owner slice
  const unsigned long long* peer_ptrs;  // [world] base address of every rank's flat buffer, as mapped on this GPU
};

__device__ __forceinline__ void red_add_v4_sys(float* addr, float a, float b, float c, float d) {
  asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ void red_add_sys(float* addr, float a) {
  asm volatile("red.relaxed.sys.global.add.f32 [%0], %1;" ::"l"(addr), "f"(a) : "memory");
}

__device__ __forceinline__ void red_add_v4_gpu(float* addr, float a, float b, float c, float d) {
  asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// Destination of flat element `g` (g % 4 == 0 for the vector form) under mode 2.
__device__ __forceinline__ float* sink_owner_ptr(const DwSink& s, const unsigned long long* peers, long long g) {
  long long owner = ((g - s.region_lo) >> 2) / s.per_vecs;
  if (owner >= s.world) owner = s.world - 1;
  return reinterpret_cast<float*>(peers[owner]) + g;
}

// One CTA: 8 input features x (256 threads * 4) output features.
//   t  : [O, ldt] fp32 (T = dY^T C, first r columns valid)
//   q  : [N, r] fp32 basis
//   dy : [rows, O] bf16
// out[o, n] (transposed == 0, row-major [O, N]) or out[n, o] (transposed == 1, [N, O]).
__device__ __forceinline__ void st_v8_f32(float* dst, const float (&v)[8]) {
  asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]),
               "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7])
               : "memory");
}

// OPT output features per thread (4 or 8): a CTA covers 8 input features x 256 * OPT output features.  With OPT == 8 a
// gathered dY row is read 16 bytes per lane and the per-entry overhead (index, value, address) is spread over 8 FMAs.
//
// PHASE 0: one CTA per strip of 8 features writes the low-rank term plus piece 0 of the strip's entries.
// PHASE 1: one CTA per item of the plan (see col_scan_kernel) adds one further piece with vector reductions; it runs
//          after phase 0 in stream order, so the plain stores of phase 0 are never overtaken.
struct DwPlan {
  const int* parts;         // [ceil(n / 8)] pieces per strip (NULL: every strip is one piece)
  const int2* extra_items;  // (strip, piece) for pieces >= 1
  const int* extra_count;
};

template <typename OutT, int SINK, int OPT, int PHASE>
__global__ void __launch_bounds__(256) dw_fused_kernel(const float* __restrict__ t, int ldt, const float* __restrict__ q, int r,
                                                       const __nv_bfloat16* __restrict__ dy, int ldy, const int* __restrict__ colptr,
                                                       const int* __restrict__ rows_sorted, const float* __restrict__ vals_sorted,
                                                       int o_total, int n_total, int transposed, OutT* __restrict__ out,
                                                       const DwSink sink, const DwPlan plan) {
  int strip = blockIdx.x, piece = 0;
  if constexpr (PHASE == 1) {
    if (static_cast<int>(blockIdx.x) >= *plan.extra_count) return;
    const int2 item = plan.extra_items[blockIdx.x];
    strip = item.x;
    piece = item.y;
  }
  const int pieces = plan.parts ? plan.parts[strip] : 1;
  const int n0 = strip * 8;
  const int o0 = blockIdx.y * (256 * OPT) + threadIdx.x * OPT;
  const bool o_ok = o0 < o_total;  // O is a multiple of OPT (checked by the launcher)
  float acc[8][OPT];
  __shared__ float sq[8][32];
  __shared__ unsigned long long s_peers[16];
  if (SINK == 2 && threadIdx.x < sink.world && threadIdx.x < 16) s_peers[threadIdx.x] = sink.peer_ptrs[threadIdx.x];
  for (int i = threadIdx.x; i < 8 * 32; i += blockDim.x) {
    const int c = i >> 5, j = i & 31;
    sq[c][j] = (n0 + c < n_total && j < r) ? q[static_cast<size_t>(n0 + c) * r + j] : 0.f;
  }
  __syncthreads();
  if (!o_ok) return;
#pragma unroll
  for (int c = 0; c < 8; ++c)
#pragma unroll
    for (int i = 0; i < OPT; ++i) acc[c][i] = 0.f;
  if (PHASE == 0 && t != nullptr) {
    for (int j = 0; j < r; ++j) {
      float tv[OPT];
#pragma unroll
      for (int i = 0; i < OPT; ++i) tv[i] = t[static_cast<size_t>(o0 + i) * ldt + j];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const float qv = sq[c][j];
#pragma unroll
        for (int i = 0; i < OPT; ++i) acc[c][i] = fmaf(tv[i], qv, acc[c][i]);
      }
    }
  }
  if (colptr != nullptr) {
    const __nv_bfloat16* dy_o = dy + o0;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      if (n0 + c >= n_total) continue;
      const int c_beg = colptr[n0 + c], c_len = colptr[n0 + c + 1] - c_beg;
      const int beg = c_beg + static_cast<int>(static_cast<long long>(c_len) * piece / pieces);
      const int end = c_beg + static_cast<int>(static_cast<long long>(c_len) * (piece + 1) / pieces);
      // The dY row of an entry is only known after its row index is loaded; keep GATHER entries in
      // flight per thread so the kernel is bound by bandwidth rather than by one load latency.
      constexpr int GATHER = (OPT == 8) ? 4 : 8;
      for (int e = beg; e < end; e += GATHER) {
        int rr[GATHER];
        float vv[GATHER];
#pragma unroll
        for (int u = 0; u < GATHER; ++u) {
          const bool ok = e + u < end;
          rr[u] = ok ? __ldg(rows_sorted + e + u) : 0;
          vv[u] = ok ? __ldg(vals_sorted + e + u) : 0.f;
        }
        if constexpr (OPT == 8) {
          uint4 raw[GATHER];
#pragma unroll
          for (int u = 0; u < GATHER; ++u) raw[u] = __ldg(reinterpret_cast<const uint4*>(dy_o + static_cast<size_t>(rr[u]) * ldy));
#pragma unroll
          for (int u = 0; u < GATHER; ++u) {
            const uint32_t w[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              acc[c][2 * k] = fmaf(vv[u], __uint_as_float(w[k] << 16), acc[c][2 * k]);
              acc[c][2 * k + 1] = fmaf(vv[u], __uint_as_float(w[k] & 0xFFFF0000u), acc[c][2 * k + 1]);
            }
          }
        } else {
          uint2 raw[GATHER];
#pragma unroll
          for (int u = 0; u < GATHER; ++u) raw[u] = __ldg(reinterpret_cast<const uint2*>(dy_o + static_cast<size_t>(rr[u]) * ldy));
#pragma unroll
          for (int u = 0; u < GATHER; ++u) {
            acc[c][0] = fmaf(vv[u], __uint_as_float(raw[u].x << 16), acc[c][0]);
            acc[c][1] = fmaf(vv[u], __uint_as_float(raw[u].x & 0xFFFF0000u), acc[c][1]);
            acc[c][2] = fmaf(vv[u], __uint_as_float(raw[u].y << 16), acc[c][2]);
            acc[c][3] = fmaf(vv[u], __uint_as_float(raw[u].y & 0xFFFF0000u), acc[c][3]);
          }
        }
      }
    }
  }
  if constexpr (SINK != 0) {
    // out is the flat fp32 gradient buffer; the parameter starts at sink.param_off
#pragma unroll
    for (int c = 0; c < 8; ++c)
#pragma unroll
      for (int i = 0; i < OPT; ++i) acc[c][i] *= sink.scale;
    float* flat = reinterpret_cast<float*>(out);
    if (!transposed) {
      const bool vec = (n0 + 8 <= n_total) && ((n_total & 3) == 0);
#pragma unroll
      for (int i = 0; i < OPT; ++i) {
        const long long g = sink.param_off + static_cast<long long>(o0 + i) * n_total + n0;
        if (vec) {
          if constexpr (SINK == 1 && PHASE == 1) {
            red_add_v4_gpu(flat + g, acc[0][i], acc[1][i], acc[2][i], acc[3][i]);
            red_add_v4_gpu(flat + g + 4, acc[4][i], acc[5][i], acc[6][i], acc[7][i]);
          } else if constexpr (SINK == 1) {
            float4* dst = reinterpret_cast<float4*>(flat + g);
            float4 a = dst[0], b = dst[1];
            a.x += acc[0][i]; a.y += acc[1][i]; a.z += acc[2][i]; a.w += acc[3][i];
            b.x += acc[4][i]; b.y += acc[5][i]; b.z += acc[6][i]; b.w += acc[7][i];
            dst[0] = a;
            dst[1] = b;
          } else {
            red_add_v4_sys(sink_owner_ptr(sink, s_peers, g), acc[0][i], acc[1][i], acc[2][i], acc[3][i]);
            red_add_v4_sys(sink_owner_ptr(sink, s_peers, g + 4), acc[4][i], acc[5][i], acc[6][i], acc[7][i]);
          }
        } else {
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            if (n0 + c >= n_total) continue;
            if constexpr (SINK == 1 && PHASE == 1) atomicAdd(flat + g + c, acc[c][i]);
            else if constexpr (SINK == 1) flat[g + c] += acc[c][i];
            else red_add_sys(sink_owner_ptr(sink, s_peers, (g + c) & ~3LL) + ((g + c) & 3), acc[c][i]);
          }
        }
      }
    } else {
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        if (n0 + c >= n_total) continue;
#pragma unroll
        for (int h = 0; h < OPT / 4; ++h) {
          const long long g = sink.param_off + static_cast<long long>(n0 + c) * o_total + o0 + 4 * h;  // o0 % 4 == 0, O % 4 == 0
          if constexpr (SINK == 1 && PHASE == 1) {
            red_add_v4_gpu(flat + g, acc[c][4 * h], acc[c][4 * h + 1], acc[c][4 * h + 2], acc[c][4 * h + 3]);
          } else if constexpr (SINK == 1) {
            float4* dst = reinterpret_cast<float4*>(flat + g);
            float4 a = dst[0];
            a.x += acc[c][4 * h]; a.y += acc[c][4 * h + 1]; a.z += acc[c][4 * h + 2]; a.w += acc[c][4 * h + 3];
            dst[0] = a;
          } else {
            red_add_v4_sys(sink_owner_ptr(sink, s_peers, g), acc[c][4 * h], acc[c][4 * h + 1], acc[c][4 * h + 2], acc[c][4 * h + 3]);
          }
        }
      }
    }
    return;
  }
  if constexpr (PHASE == 1 && sizeof(OutT) == 4) {
    float* fout = reinterpret_cast<float*>(out);
    if (!transposed) {
      const bool vec = (n0 + 8 <= n_total) && ((n_total & 3) == 0);
#pragma unroll
      for (int i = 0; i < OPT; ++i) {
        float* dst = fout + static_cast<size_t>(o0 + i) * n_total + n0;
        if (vec) {
          red_add_v4_gpu(dst, acc[0][i], acc[1][i], acc[2][i], acc[3][i]);
          red_add_v4_gpu(dst + 4, acc[4][i], acc[5][i], acc[6][i], acc[7][i]);
        } else {
#pragma unroll
          for (int c = 0; c < 8; ++c)
            if (n0 + c < n_total) atomicAdd(dst + c, acc[c][i]);
        }
      }
    } else {
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        if (n0 + c >= n_total) continue;
        float* dst = fout + static_cast<size_t>(n0 + c) * o_total + o0;
#pragma unroll
        for (int h = 0; h < OPT / 4; ++h) red_add_v4_gpu(dst + 4 * h, acc[c][4 * h], acc[c][4 * h + 1], acc[c][4 * h + 2], acc[c][4 * h + 3]);
      }
    }
    return;
  }
  if (!transposed) {
    const bool vec = (n0 + 8 <= n_total) && ((n_total & 7) == 0);
#pragma unroll
    for (int i = 0; i < OPT; ++i) {
      OutT* dst = out + static_cast<size_t>(o0 + i) * n_total + n0;
      if (vec) {
        if constexpr (sizeof(OutT) == 4) {
          // one 32-byte store per row: a full sector, where two 16-byte stores would each be a partial write
          const float v[8] = {acc[0][i], acc[1][i], acc[2][i], acc[3][i], acc[4][i], acc[5][i], acc[6][i], acc[7][i]};
          if ((reinterpret_cast<uintptr_t>(dst) & 31) == 0) {
            st_v8_f32(reinterpret_cast<float*>(dst), v);
          } else {
            reinterpret_cast<float4*>(dst)[0] = make_float4(v[0], v[1], v[2], v[3]);
            reinterpret_cast<float4*>(dst)[1] = make_float4(v[4], v[5], v[6], v[7]);
          }
        } else {
          *reinterpret_cast<uint4*>(dst) = make_uint4(pack_bf16x2(acc[0][i], acc[1][i]), pack_bf16x2(acc[2][i], acc[3][i]),
                                                      pack_bf16x2(acc[4][i], acc[5][i]), pack_bf16x2(acc[6][i], acc[7][i]));
        }
      } else {
#pragma unroll
        for (int c = 0; c < 8; ++c)
          if (n0 + c < n_total) dst[c] = static_cast<OutT>(acc[c][i]);
      }
    }
  } else {
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      if (n0 + c >= n_total) continue;
      OutT* dst = out + static_cast<size_t>(n0 + c) * o_total + o0;
#pragma unroll
      for (int i = 0; i < OPT; ++i) dst[i] = static_cast<OutT>(acc[c][i]);
    }
  }
}

// colsum[o] = sum_rows dy[row, o]  (bias gradient).  A CTA owns 256 columns x a slab of 256 rows: its 8 warps take every
// eighth row (a warp reads 512 contiguous bytes of a row with 16-byte loads, 4 rows in flight), the warps' partial sums meet in
// shared memory, and one fp32 atomic per column and CTA goes out: 32 atomics per address for 8192 rows (more slabs made the
// same-address atomics the bottleneck, fewer CTAs left the SMs idle).
constexpr int CSUM_COLS = 256, CSUM_SLAB = 256, CSUM_UNROLL = 4;
__global__ void __launch_bounds__(256) colsum_kernel(const __nv_bfloat16* dy, int rows, int o_total, int ldy, int slab, float* out) {
  __shared__ float s_part[8][CSUM_COLS + 8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int o = blockIdx.x * CSUM_COLS + lane * 8;
  const int r0 = blockIdx.y * slab, r1 = min(rows, r0 + slab);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  const bool vec = (o + 8 <= o_total) && ((ldy & 7) == 0) && ((reinterpret_cast<uintptr_t>(dy) & 15) == 0);
  if (vec) {
    for (int row = r0 + warp; row < r1; row += 8 * CSUM_UNROLL) {
      uint4 raw[CSUM_UNROLL];
#pragma unroll
      for (int u = 0; u < CSUM_UNROLL; ++u)
        raw[u] = row + 8 * u < r1 ? __ldg(reinterpret_cast<const uint4*>(dy + static_cast<size_t>(row + 8 * u) * ldy + o)) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
      for (int u = 0; u < CSUM_UNROLL; ++u) {
        const uint32_t w[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          acc[2 * k] += __uint_as_float(w[k] << 16);
          acc[2 * k + 1] += __uint_as_float(w[k] & 0xFFFF0000u);
        }
      }
    }
  } else if (o < o_total) {
    for (int row = r0 + warp; row < r1; row += 8)
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (o + j < o_total) acc[j] += __bfloat162float(dy[static_cast<size_t>(row) * ldy + o + j]);
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) s_part[warp][lane * 8 + j] = acc[j];
  __syncthreads();
  const int col = blockIdx.x * CSUM_COLS + threadIdx.x;
  if (col < o_total) {
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) total += s_part[w][threadIdx.x];
    atomicAdd(out + col, total);
  }
}

// 8 output features per thread need 16-byte aligned dY rows and enough output features to fill the wider CTA.
static inline bool dw_wide(int o_total, int ldy, const void* dy) {
  return o_total >= 2048 && (o_total % 8) == 0 && (ldy % 8) == 0 && (reinterpret_cast<uintptr_t>(dy) & 15) == 0;
}

}  // namespace sb

// Target number of residual entries one weight-gradient CTA walks (see col_scan_kernel).
extern "C" int sb_dw_plan_target() {
  static int target = 0;
  if (target == 0) {
    const char* env = getenv("STACR_DW_TARGET");  // tuning knob; read once
    const int v = env ? atoi(env) : 0;
    target = (v >= 64 && v <= 65536) ? v : 256;
  }
  return target;
}

// Bucket the residual entries by input feature.  counts/cursor: int32 [n] scratch (counts zeroed by the
// caller); colptr: int32 [n+1]; rows_sorted/vals_sorted: [nnz].  plan (optional): int32 scratch of
// ceil(n / 8) + 1 + 2 * (nnz / sb_dw_plan_target()) entries that receives the work plan of sb_dw_fused*.
extern "C" int sb_residual_bucket(const int* idx32, const long long* idx64, long long nnz, int n, const void* val, int bits,
                                  const float* scale, int* counts, int* cursor, int* colptr, int* rows_sorted,
                                  float* vals_sorted, int* plan, void* stream) {
  using namespace sb;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int threads = 256;
  const unsigned blocks = static_cast<unsigned>((nnz + threads - 1) / threads);
  if (nnz > 0) col_count_kernel<<<blocks, threads, 0, st>>>(idx32, idx64, nnz, n, counts);
  const int groups = (n + 7) / 8;
  const int max_extra = static_cast<int>(nnz / sb_dw_plan_target());
  col_scan_kernel<<<1, 1024, 0, st>>>(counts, n, colptr, cursor, plan, plan ? plan + groups : nullptr,
                                      plan ? reinterpret_cast<int2*>(plan + groups + 1 + ((groups + 1) & 1)) : nullptr, sb_dw_plan_target(), max_extra);
  if (nnz > 0)
    col_scatter_kernel<<<blocks, threads, 0, st>>>(idx32, idx64, nnz, n, val, bits, scale, cursor, rows_sorted, vals_sorted);
  return static_cast<int>(cudaGetLastError());
}

namespace sb {

template <typename OutT, int SINK>
static int launch_dw(const float* t, int ldt, const float* q, int r, const void* dy, int ldy, const int* colptr, const int* rows_sorted,
                     const float* vals_sorted, int o_total, int n_total, int transposed, OutT* out, const DwSink& sink, const int* plan,
                     long long nnz, cudaStream_t st) {
  const __nv_bfloat16* dyp = static_cast<const __nv_bfloat16*>(dy);
  const bool wide = dw_wide(o_total, ldy, dy);
  const int groups = (n_total + 7) / 8;
  const unsigned gy = wide ? (o_total + 2047) / 2048 : (o_total + 1023) / 1024;
  DwPlan dp{nullptr, nullptr, nullptr};
  int max_extra = 0;
  if (plan != nullptr && colptr != nullptr && sizeof(OutT) == 4) {
    dp.parts = plan;
    dp.extra_count = plan + groups;
    dp.extra_items = reinterpret_cast<const int2*>(plan + groups + 1 + ((groups + 1) & 1));
    max_extra = static_cast<int>(nnz / sb_dw_plan_target());
  }
  dim3 grid(groups, gy);
  if (wide) dw_fused_kernel<OutT, SINK, 8, 0><<<grid, 256, 0, st>>>(t, ldt, q, r, dyp, ldy, colptr, rows_sorted, vals_sorted, o_total, n_total, transposed, out, sink, dp);
  else dw_fused_kernel<OutT, SINK, 4, 0><<<grid, 256, 0, st>>>(t, ldt, q, r, dyp, ldy, colptr, rows_sorted, vals_sorted, o_total, n_total, transposed, out, sink, dp);
  if (max_extra > 0) {
    dim3 grid1(max_extra, gy);
    if (wide) dw_fused_kernel<OutT, SINK, 8, 1><<<grid1, 256, 0, st>>>(t, ldt, q, r, dyp, ldy, colptr, rows_sorted, vals_sorted, o_total, n_total, transposed, out, sink, dp);
    else dw_fused_kernel<OutT, SINK, 4, 1><<<grid1, 256, 0, st>>>(t, ldt, q, r, dyp, ldy, colptr, rows_sorted, vals_sorted, o_total, n_total, transposed, out, sink, dp);
  }
  return static_cast<int>(cudaGetLastError());
}

}  // namespace sb

// dW = T Q^T + dY^T S, written as fp32 (out_bf16 == 0) or bf16.  Pass t == NULL to skip the low-rank
// term and colptr == NULL to skip the sparse term.  plan: the scratch filled by sb_residual_bucket (or NULL: one CTA
// per strip of 8 features walks all of the strip's entries); nnz: number of residual entries behind colptr.
extern "C" int sb_dw_fused(const float* t, int ldt, const float* q, int r, const void* dy, int ldy, const int* colptr,
                           const int* rows_sorted, const float* vals_sorted, int o_total, int n_total, int transposed,
                           int out_bf16, void* out, const int* plan, long long nnz, void* stream) {
  using namespace sb;
  if (o_total % 4 || (ldy & 3) || r > 32) return -2;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const DwSink none{};
  if (out_bf16)
    return launch_dw<__nv_bfloat16, 0>(t, ldt, q, r, dy, ldy, colptr, rows_sorted, vals_sorted, o_total, n_total, transposed,
                                       static_cast<__nv_bfloat16*>(out), none, nullptr, 0, st);
  return launch_dw<float, 0>(t, ldt, q, r, dy, ldy, colptr, rows_sorted, vals_sorted, o_total, n_total, transposed, static_cast<float*>(out),
                             none, plan, nnz, st);
}

// The same gradient, delivered into the flat fp32 gradient buffer `flat` instead of a private tensor.
//   mode 1: flat[param_off + i] += scale * dW[i]                       (this GPU only)
//   mode 2: owner_copy[param_off + i] += scale * dW[i] with one red.add per 16 bytes, where the owner of an element is
//           the rank whose slice of [region_lo, region_lo + 4 * per_vecs * world) holds it; peer_ptrs (device array of
//           `world` addresses) maps every rank's flat buffer.  The parameter must lie inside the region.
extern "C" int sb_dw_fused_sink(const float* t, int ldt, const float* q, int r, const void* dy, int ldy, const int* colptr,
                                const int* rows_sorted, const float* vals_sorted, int o_total, int n_total, int transposed,
                                float* flat, int mode, float scale, long long param_off, long long region_lo, long long per_vecs,
                                int world, const void* peer_ptrs, const int* plan, long long nnz, void* stream) {
  using namespace sb;
  if (o_total % 4 || (ldy & 3) || r > 32) return -2;
  if ((param_off & 3) || mode < 1 || mode > 2) return -3;
  if (mode == 2) {
    if (peer_ptrs == nullptr || world < 1 || world > 16 || per_vecs < 1 || (region_lo & 3) || param_off < region_lo) return -4;
    const long long last = param_off + static_cast<long long>(o_total) * n_total;
    if (last > region_lo + 4 * per_vecs * world) return -5;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const DwSink sink{mode, world, scale, param_off, region_lo, per_vecs, static_cast<const unsigned long long*>(peer_ptrs)};
  if (mode == 1)
    return launch_dw<float, 1>(t, ldt, q, r, dy, ldy, colptr, rows_sorted, vals_sorted, o_total, n_total, transposed, flat, sink, plan, nnz, st);
  return launch_dw<float, 2>(t, ldt, q, r, dy, ldy, colptr, rows_sorted, vals_sorted, o_total, n_total, transposed, flat, sink, plan, nnz, st);
}

extern "C" int sb_colsum_bf16(const void* dy, int rows, int o_total, int ldy, float* out, void* stream) {
  using namespace sb;
  if (rows <= 0 || o_total <= 0) return 0;
  int slab = sb::CSUM_SLAB;
  while ((rows + slab - 1) / slab > 65535) slab *= 2;   // grid.y limit
  dim3 grid((o_total + sb::CSUM_COLS - 1) / sb::CSUM_COLS, (rows + slab - 1) / slab);
  sb::colsum_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(dy), rows, o_total, ldy, slab, out);
  return static_cast<int>(cudaGetLastError());
}
