// Device-side encodings of the sparse residual's index stream, and the small per-tensor codecs of the adaptive engine.
//
//   CSR    flat = row * n + col entries are grouped by row with a counting sort (row histogram, one-CTA scan for the
//          row pointers, scatter with a per-row cursor); the narrow column ids, the gather order and its inverse come
//          out of the scatter.  Order inside a row is whatever the scatter produced: CSR does not need it sorted.
//   delta  the CSR grouping followed by an in-row sort (one CTA per row, bitonic network in shared memory on
//          (column, source position) keys) yields the globally sorted stream; gaps are first differences.
//   int8 / int4 codecs with a per-tensor scale (clamped symmetric range, int4 stored offset by 8, two per byte), and the
//          sum of squares used for the Pythagoras residual energy.
// These replace the argsort + bincount + cumsum and sort + diff pipelines of the reference
// (stacr/index_compression.py:134-272, stacr/adaptive.py:44-135,1341-1346 there).
#include "common.cuh"

namespace sb {

__device__ __forceinline__ long long load_flat(const int* i32, const long long* i64, long long i) {
  return i32 ? static_cast<long long>(i32[i]) : i64[i];
}

__global__ void __launch_bounds__(256) row_count_kernel(const int* i32, const long long* i64, long long nnz, int n, int rows,
                                                        int* counts, int* bad) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nnz; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long flat = load_flat(i32, i64, i);
    const long long row = flat / n;
    if (flat < 0 || row >= rows) {
      atomicAdd(bad, 1);
      continue;
    }
    atomicAdd(&counts[row], 1);
  }
}

// row_ptr[0] = 0, row_ptr[r + 1] = row_ptr[r] + counts[r]; cursor[r] = row_ptr[r].  One CTA of 1024 threads walks the rows
// in blocks of 1024 with a running carry.
__global__ void __launch_bounds__(1024) row_scan_kernel(const int* counts, int rows, int* row_ptr, int* cursor) {
  __shared__ int s_warp[32];
  __shared__ int s_carry;
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  if (t == 0) {
    s_carry = 0;
    row_ptr[0] = 0;
  }
  __syncthreads();
  for (int base = 0; base < rows; base += 1024) {
    const int r = base + t;
    const int v = r < rows ? counts[r] : 0;
    int incl = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int u = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += u;
    }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      int w = s_warp[lane];
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, w, off);
        if (lane >= off) w += u;
      }
      s_warp[lane] = w;
    }
    __syncthreads();
    const int carry = s_carry;
    const int before = carry + (warp ? s_warp[warp - 1] : 0) + incl - v;
    if (r < rows) {
      cursor[r] = before;
      row_ptr[r + 1] = before + v;
    }
    __syncthreads();
    if (t == 1023) s_carry = carry + s_warp[31];
    __syncthreads();
  }
}

template <typename ColT>
__global__ void __launch_bounds__(256) row_scatter_kernel(const int* i32, const long long* i64, long long nnz, int n, int rows,
                                                          int* cursor, ColT* cols, int* order, int* inverse) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nnz; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long flat = load_flat(i32, i64, i);
    const long long row = flat / n;
    if (flat < 0 || row >= rows) continue;
    const int pos = atomicAdd(&cursor[row], 1);
    cols[pos] = static_cast<ColT>(flat - row * n);
    if (order) order[pos] = static_cast<int>(i);
    if (inverse) inverse[i] = pos;
  }
}

// One CTA per row: sort the row's (column, source position) pairs by column.  Rows longer than SORT_CAP are left as
// they are and counted in `unsorted` (the caller then falls back to a library sort for this tensor).
constexpr int SORT_CAP = 4096;

__global__ void __launch_bounds__(256) row_sort_kernel(const int* row_ptr, int rows, int* cols, int* order, int* inverse, int* unsorted) {
  __shared__ unsigned long long keys[SORT_CAP];
  const int row = blockIdx.x;
  if (row >= rows) return;
  const int lo = row_ptr[row], m = row_ptr[row + 1] - lo;
  if (m <= 1) return;
  if (m > SORT_CAP) {
    if (threadIdx.x == 0) atomicAdd(unsorted, 1);
    return;
  }
  int pow2 = 1;
  while (pow2 < m) pow2 <<= 1;
  for (int i = threadIdx.x; i < pow2; i += blockDim.x)
    keys[i] = i < m ? ((static_cast<unsigned long long>(static_cast<unsigned int>(cols[lo + i])) << 32) | static_cast<unsigned int>(order[lo + i]))
                    : ~0ull;
  __syncthreads();
  for (int size = 2; size <= pow2; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int i = threadIdx.x; i < pow2 / 2; i += blockDim.x) {
        const int a = 2 * i - (i & (stride - 1));   // lower index of the pair
        const int b = a + stride;
        const bool up = ((a & size) == 0);
        const unsigned long long ka = keys[a], kb = keys[b];
        if ((ka > kb) == up) {
          keys[a] = kb;
          keys[b] = ka;
        }
      }
      __syncthreads();
    }
  }
  for (int i = threadIdx.x; i < m; i += blockDim.x) {
    const unsigned long long k = keys[i];
    const int src = static_cast<int>(k & 0xffffffffu);
    cols[lo + i] = static_cast<int>(k >> 32);
    order[lo + i] = src;
    if (inverse) inverse[src] = lo + i;
  }
}

// sorted_flat[i] = row(i) * n + cols[i] for a row-grouped, in-row sorted stream; gaps[i] = sorted[i + 1] - sorted[i];
// *max_gap = largest gap (for the caller's choice of the gap width); base[0] = sorted[0].
__global__ void __launch_bounds__(256) delta_kernel(const int* row_ptr, int rows, const int* cols, long long nnz, int n, long long* gaps,
                                                    long long* base, unsigned long long* max_gap) {
  // entry i belongs to the row r with row_ptr[r] <= i < row_ptr[r + 1]: binary search per entry
  unsigned long long local_max = 0;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nnz; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    auto flat_at = [&](long long e) {
      int lo = 0, hi = rows;  // first r with row_ptr[r + 1] > e
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (row_ptr[mid + 1] > e) hi = mid;
        else lo = mid + 1;
      }
      return static_cast<long long>(lo) * n + cols[e];
    };
    const long long cur = flat_at(i);
    if (i == 0) base[0] = cur;
    if (i + 1 < nnz) {
      const long long g = flat_at(i + 1) - cur;
      gaps[i] = g;
      if (static_cast<unsigned long long>(g) > local_max) local_max = static_cast<unsigned long long>(g);
    }
  }
  if (local_max) atomicMax(max_gap, local_max);
}

// ------------------------------------------------------------------------------------------------ per-tensor codecs
template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// out[0] = max |x| (as the bits of a non-negative float, so integer atomicMax orders it), out[1] += sum x^2.
template <typename T>
__global__ void __launch_bounds__(256) amax_sumsq_kernel(const T* x, long long numel, unsigned int* amax_bits, float* sumsq) {
  float m = 0.f, s = 0.f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < numel; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float v = to_f32<T>(x[i]);
    m = fmaxf(m, fabsf(v));
    s = fmaf(v, v, s);
  }
#pragma unroll
  for (int off = 16; off; off >>= 1) {
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    s += __shfl_xor_sync(0xffffffffu, s, off);
  }
  __shared__ float sm[8], ss[8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    sm[warp] = m;
    ss[warp] = s;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) {
      m = fmaxf(m, sm[w]);
      s += ss[w];
    }
    if (amax_bits) atomicMax(amax_bits, __float_as_uint(m));
    if (sumsq) atomicAdd(sumsq, s);
  }
}

// Symmetric quantisation with the scale amax / qmax taken from amax_bits (scale 1 when the tensor is all zero).
// bits == 8: out[i] = clamp(rint(x / scale), -127, 127) as int8.  bits == 4: two codes per byte, (q + 8) with the even
// element in the low nibble; an odd tail is padded with the code of zero.
template <typename T>
__global__ void __launch_bounds__(256) quantize_kernel(const T* x, long long numel, int bits, const unsigned int* amax_bits, float* scale_out,
                                                       unsigned char* out) {
  const float amax = __uint_as_float(*amax_bits);
  const float qmax = bits == 4 ? 7.f : 127.f;
  const float scale = amax > 0.f ? fmaxf(amax / qmax, 1.17549435e-38f) : 1.f;
  if (blockIdx.x == 0 && threadIdx.x == 0) *scale_out = scale;
  const float inv = 1.f / scale;
  if (bits == 8) {
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < numel; i += static_cast<long long>(gridDim.x) * blockDim.x)
      reinterpret_cast<signed char*>(out)[i] = static_cast<signed char>(fminf(fmaxf(rintf(to_f32<T>(x[i]) * inv), -127.f), 127.f));
  } else {
    const long long pairs = (numel + 1) / 2;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < pairs; i += static_cast<long long>(gridDim.x) * blockDim.x) {
      const float a = to_f32<T>(x[2 * i]);
      const float b = (2 * i + 1 < numel) ? to_f32<T>(x[2 * i + 1]) : 0.f;
      const int qa = static_cast<int>(fminf(fmaxf(rintf(a * inv), -7.f), 7.f)) + 8;
      const int qb = static_cast<int>(fminf(fmaxf(rintf(b * inv), -7.f), 7.f)) + 8;
      out[i] = static_cast<unsigned char>(qa | (qb << 4));
    }
  }
}

// dst[i, :] = src[index[i], :] (gather) or dst[index[i], :] = src[i, :] (scatter) for rows of `width` bf16 values,
// width % 8 == 0: the mask-aware compaction of padded batches.
__global__ void __launch_bounds__(256) move_rows_kernel(const uint4* src, uint4* dst, const long long* index, long long count, int vecs, int scatter) {
  const long long total = count * vecs;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vecs;
    const int v = static_cast<int>(i - r * vecs);
    const long long other = index[r];
    if (scatter) dst[other * vecs + v] = src[i];
    else dst[i] = src[other * vecs + v];
  }
}

// Per-row symmetric int8 codec of a [rows, r] coefficient matrix (r <= 64): scale[row] = max(|row|) / 127 (at least the
// smallest normal float), q = clamp(rint(x / scale), -127, 127).  One thread per row.
template <typename T>
__global__ void __launch_bounds__(256) quantize_rows_kernel(const T* x, long long rows, int r, int ldx, signed char* q, float* scale) {
  for (long long row = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; row < rows; row += static_cast<long long>(gridDim.x) * blockDim.x) {
    const T* xr = x + row * ldx;
    float amax = 0.f;
    for (int j = 0; j < r; ++j) amax = fmaxf(amax, fabsf(to_f32<T>(xr[j])));
    const float sc = fmaxf(amax / 127.f, 1.17549435e-38f);
    scale[row] = sc;
    const float inv = 1.f / sc;
    for (int j = 0; j < r; ++j) q[row * r + j] = static_cast<signed char>(fminf(fmaxf(rintf(to_f32<T>(xr[j]) * inv), -127.f), 127.f));
  }
}

// out[row, j] = bf16(q[row, j] * scale[row])
__global__ void __launch_bounds__(256) dequantize_rows_kernel(const signed char* q, const float* scale, long long rows, int r, __nv_bfloat16* out) {
  const long long total = rows * r;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * blockDim.x)
    out[i] = __float2bfloat16_rn(static_cast<float>(q[i]) * scale[i / r]);
}

static inline unsigned grid_for(long long work, int threads, int cap) {
  long long g = (work + threads - 1) / threads;
  if (g > cap) g = cap;
  return static_cast<unsigned>(g < 1 ? 1 : g);
}

}  // namespace sb

// Group the entries by row.  counts [rows] zeroed by the caller; cursor [rows]; row_ptr [rows + 1]; cols int16 (col16) or
// int32 (col32), exactly one non-NULL; order / inverse int32 [nnz] (either may be NULL); bad [1] zeroed, receives the number
// of entries outside the matrix (they are skipped).  nnz < 2^31.
extern "C" int sb_csr_pack(const int* idx32, const long long* idx64, long long nnz, int rows, int n, int* counts, int* cursor, int* row_ptr,
                           short* col16, int* col32, int* order, int* inverse, int* bad, void* stream) {
  using namespace sb;
  if (nnz <= 0 || rows <= 0 || n <= 0) return nnz == 0 ? 0 : -2;
  if ((idx32 == nullptr) == (idx64 == nullptr)) return -2;
  if ((col16 == nullptr) == (col32 == nullptr)) return -2;
  if (nnz >= 2147483647LL) return -3;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = grid_for(nnz, 256, 2048);
  row_count_kernel<<<grid, 256, 0, st>>>(idx32, idx64, nnz, n, rows, counts, bad);
  row_scan_kernel<<<1, 1024, 0, st>>>(counts, rows, row_ptr, cursor);
  if (col16) row_scatter_kernel<short><<<grid, 256, 0, st>>>(idx32, idx64, nnz, n, rows, cursor, col16, order, inverse);
  else row_scatter_kernel<int><<<grid, 256, 0, st>>>(idx32, idx64, nnz, n, rows, cursor, col32, order, inverse);
  return static_cast<int>(cudaGetLastError());
}

// After sb_csr_pack with int32 columns and an order array: sort every row by column (rows of more than 4096 entries are
// counted in unsorted[0] and left alone) and emit the first differences of the sorted flat stream.
extern "C" int sb_delta_pack(const int* row_ptr, int rows, int n, long long nnz, int* col32, int* order, int* inverse, long long* gaps,
                             long long* base, unsigned long long* max_gap, int* unsorted, void* stream) {
  using namespace sb;
  if (nnz <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  row_sort_kernel<<<rows, 256, 0, st>>>(row_ptr, rows, col32, order, inverse, unsorted);
  delta_kernel<<<grid_for(nnz, 256, 2048), 256, 0, st>>>(row_ptr, rows, col32, nnz, n, gaps, base, max_gap);
  return static_cast<int>(cudaGetLastError());
}

// stats[0] (as uint bits) = max |x|, stats[1] += sum x^2; stats zeroed by the caller.  is_bf16 selects the element type.
extern "C" int sb_amax_sumsq(const void* x, long long numel, int is_bf16, void* stats, void* stream) {
  using namespace sb;
  if (numel <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  unsigned int* amax = static_cast<unsigned int*>(stats);
  float* sumsq = reinterpret_cast<float*>(amax + 1);
  const unsigned grid = grid_for(numel, 256 * 8, 1184);
  if (is_bf16) amax_sumsq_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), numel, amax, sumsq);
  else amax_sumsq_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(x), numel, amax, sumsq);
  return static_cast<int>(cudaGetLastError());
}

// Quantise with the amax a previous sb_amax_sumsq left in stats[0]; scale_out receives the scale.
extern "C" int sb_quantize_sym(const void* x, long long numel, int is_bf16, int bits, const void* stats, float* scale_out, void* out, void* stream) {
  using namespace sb;
  if (numel <= 0) return 0;
  if (bits != 4 && bits != 8) return -2;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned int* amax = static_cast<const unsigned int*>(stats);
  const unsigned grid = grid_for(numel, 256 * 4, 1184);
  if (is_bf16) quantize_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), numel, bits, amax, scale_out, static_cast<unsigned char*>(out));
  else quantize_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(x), numel, bits, amax, scale_out, static_cast<unsigned char*>(out));
  return static_cast<int>(cudaGetLastError());
}

// Row gather (scatter = 0) or scatter (scatter = 1) of bf16 rows of `width` values (width % 8 == 0, 16-byte aligned bases).
extern "C" int sb_move_rows(const void* src, void* dst, const long long* index, long long count, int width, int scatter, void* stream) {
  using namespace sb;
  if (count <= 0) return 0;
  if (width % 8 || (reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 15)) return -3;
  const int vecs = width / 8;
  move_rows_kernel<<<grid_for(count * vecs, 256, 1184 * 2), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), static_cast<uint4*>(dst), index, count, vecs, scatter);
  return static_cast<int>(cudaGetLastError());
}

// Per-row int8 quantisation of fp32 or bf16 x[rows, r] (leading dimension ldx): q int8 [rows, r] contiguous, scale fp32 [rows].
extern "C" int sb_quantize_rows_int8(const void* x, int is_bf16, long long rows, int r, int ldx, void* q, float* scale, void* stream) {
  using namespace sb;
  if (rows <= 0 || r <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = grid_for(rows, 256, 1184);
  if (is_bf16) quantize_rows_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), rows, r, ldx, static_cast<signed char*>(q), scale);
  else quantize_rows_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(x), rows, r, ldx, static_cast<signed char*>(q), scale);
  return static_cast<int>(cudaGetLastError());
}

// bf16 out[rows, r] = q * scale[row].
extern "C" int sb_dequantize_rows_int8(const void* q, const float* scale, long long rows, int r, void* out, void* stream) {
  using namespace sb;
  if (rows <= 0 || r <= 0) return 0;
  dequantize_rows_kernel<<<grid_for(rows * r, 256, 1184), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const signed char*>(q), scale, rows, r, static_cast<__nv_bfloat16*>(out));
  return static_cast<int>(cudaGetLastError());
}
