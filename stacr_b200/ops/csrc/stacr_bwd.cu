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
#include "common.cuh"

namespace sb {

__global__ void col_count_kernel(const int* idx32, const long long* idx64, long long nnz, int n, int* counts) {
  long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= nnz) return;
  const long long flat = idx64 ? idx64[i] : static_cast<long long>(idx32[i]);
  atomicAdd(&counts[static_cast<int>(flat % n)], 1);
}

// Exclusive scan of counts[0..n) into colptr[0..n]; also copies colptr into cursor. One CTA.
__global__ void __launch_bounds__(1024) col_scan_kernel(const int* counts, int n, int* colptr, int* cursor) {
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

// One CTA: 8 input features x (256 threads * 4) output features.
//   t  : [O, ldt] fp32 (T = dY^T C, first r columns valid)
//   q  : [N, r] fp32 basis
//   dy : [rows, O] bf16
// out[o, n] (transposed == 0, row-major [O, N]) or out[n, o] (transposed == 1, [N, O]).
template <typename OutT>
__global__ void __launch_bounds__(256) dw_fused_kernel(const float* __restrict__ t, int ldt, const float* __restrict__ q, int r,
                                                       const __nv_bfloat16* __restrict__ dy, int ldy, const int* __restrict__ colptr,
                                                       const int* __restrict__ rows_sorted, const float* __restrict__ vals_sorted,
                                                       int o_total, int n_total, int transposed, OutT* __restrict__ out) {
  const int n0 = blockIdx.x * 8;
  const int o0 = blockIdx.y * 1024 + threadIdx.x * 4;
  const bool o_ok = o0 < o_total;  // O is a multiple of 4 (checked by the launcher)
  float acc[8][4];
  __shared__ float sq[8][32];
  for (int i = threadIdx.x; i < 8 * 32; i += blockDim.x) {
    const int c = i >> 5, j = i & 31;
    sq[c][j] = (n0 + c < n_total && j < r) ? q[static_cast<size_t>(n0 + c) * r + j] : 0.f;
  }
  __syncthreads();
  if (!o_ok) return;
#pragma unroll
  for (int c = 0; c < 8; ++c)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[c][i] = 0.f;
  if (t != nullptr) {
    for (int j = 0; j < r; ++j) {
      float tv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) tv[i] = t[static_cast<size_t>(o0 + i) * ldt + j];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const float qv = sq[c][j];
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[c][i] = fmaf(tv[i], qv, acc[c][i]);
      }
    }
  }
  if (colptr != nullptr) {
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      if (n0 + c >= n_total) continue;
      const int beg = colptr[n0 + c], end = colptr[n0 + c + 1];
      // The dY row of an entry is only known after its row index is loaded; keep GATHER entries in
      // flight per thread so the kernel is bound by bandwidth rather than by one load latency.
      constexpr int GATHER = 8;
      for (int e = beg; e < end; e += GATHER) {
        int rr[GATHER];
        float vv[GATHER];
        uint2 raw[GATHER];
#pragma unroll
        for (int u = 0; u < GATHER; ++u) {
          const bool ok = e + u < end;
          rr[u] = ok ? __ldg(rows_sorted + e + u) : 0;
          vv[u] = ok ? __ldg(vals_sorted + e + u) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < GATHER; ++u)
          raw[u] = __ldg(reinterpret_cast<const uint2*>(dy + static_cast<size_t>(rr[u]) * ldy + o0));
#pragma unroll
        for (int u = 0; u < GATHER; ++u) {
          const __nv_bfloat162 p0 = *reinterpret_cast<const __nv_bfloat162*>(&raw[u].x);
          const __nv_bfloat162 p1 = *reinterpret_cast<const __nv_bfloat162*>(&raw[u].y);
          acc[c][0] = fmaf(vv[u], __low2float(p0), acc[c][0]);
          acc[c][1] = fmaf(vv[u], __high2float(p0), acc[c][1]);
          acc[c][2] = fmaf(vv[u], __low2float(p1), acc[c][2]);
          acc[c][3] = fmaf(vv[u], __high2float(p1), acc[c][3]);
        }
      }
    }
  }
  if (!transposed) {
    const bool vec = (n0 + 8 <= n_total) && ((n_total & 7) == 0);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      OutT* dst = out + static_cast<size_t>(o0 + i) * n_total + n0;
      if (vec) {
        if constexpr (sizeof(OutT) == 4) {
          reinterpret_cast<float4*>(dst)[0] = make_float4(acc[0][i], acc[1][i], acc[2][i], acc[3][i]);
          reinterpret_cast<float4*>(dst)[1] = make_float4(acc[4][i], acc[5][i], acc[6][i], acc[7][i]);
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
      for (int i = 0; i < 4; ++i) dst[i] = static_cast<OutT>(acc[c][i]);
    }
  }
}

// colsum[o] = sum_rows dy[row, o]  (bias gradient); fp32 atomics over row slabs.
__global__ void __launch_bounds__(256) colsum_kernel(const __nv_bfloat16* dy, int rows, int o_total, int ldy, int slab,
                                                     float* out) {
  const int o = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (o >= o_total) return;
  const int r0 = blockIdx.y * slab, r1 = min(rows, r0 + slab);
  float a = 0.f, b = 0.f;
  for (int row = r0; row < r1; ++row) {
    const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(dy + static_cast<size_t>(row) * ldy + o);
    a += __low2float(v);
    b += __high2float(v);
  }
  atomicAdd(out + o, a);
  if (o + 1 < o_total) atomicAdd(out + o + 1, b);
}

}  // namespace sb

// Bucket the residual entries by input feature.  counts/cursor: int32 [n] scratch (counts zeroed by the
// caller); colptr: int32 [n+1]; rows_sorted/vals_sorted: [nnz].
extern "C" int sb_residual_bucket(const int* idx32, const long long* idx64, long long nnz, int n, const void* val, int bits,
                                  const float* scale, int* counts, int* cursor, int* colptr, int* rows_sorted,
                                  float* vals_sorted, void* stream) {
  using namespace sb;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int threads = 256;
  const unsigned blocks = static_cast<unsigned>((nnz + threads - 1) / threads);
  if (nnz > 0) col_count_kernel<<<blocks, threads, 0, st>>>(idx32, idx64, nnz, n, counts);
  col_scan_kernel<<<1, 1024, 0, st>>>(counts, n, colptr, cursor);
  if (nnz > 0)
    col_scatter_kernel<<<blocks, threads, 0, st>>>(idx32, idx64, nnz, n, val, bits, scale, cursor, rows_sorted, vals_sorted);
  return static_cast<int>(cudaGetLastError());
}

// dW = T Q^T + dY^T S, written as fp32 (out_bf16 == 0) or bf16.  Pass t == NULL to skip the low-rank
// term and colptr == NULL to skip the sparse term.
extern "C" int sb_dw_fused(const float* t, int ldt, const float* q, int r, const void* dy, int ldy, const int* colptr,
                           const int* rows_sorted, const float* vals_sorted, int o_total, int n_total, int transposed,
                           int out_bf16, void* out, void* stream) {
  using namespace sb;
  if (o_total % 4 || (ldy & 3) || r > 32) return -2;
  dim3 grid((n_total + 7) / 8, (o_total + 1023) / 1024);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (out_bf16)
    dw_fused_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(t, ldt, q, r, static_cast<const __nv_bfloat16*>(dy), ldy, colptr,
                                                         rows_sorted, vals_sorted, o_total, n_total, transposed,
                                                         static_cast<__nv_bfloat16*>(out));
  else
    dw_fused_kernel<float><<<grid, 256, 0, st>>>(t, ldt, q, r, static_cast<const __nv_bfloat16*>(dy), ldy, colptr, rows_sorted,
                                                 vals_sorted, o_total, n_total, transposed, static_cast<float*>(out));
  return static_cast<int>(cudaGetLastError());
}

extern "C" int sb_colsum_bf16(const void* dy, int rows, int o_total, int ldy, float* out, void* stream) {
  using namespace sb;
  if (rows <= 0 || o_total <= 0) return 0;
  if (ldy & 1) return -2;
  const int slab = 256;
  dim3 grid((o_total / 2 + 255) / 256 + 1, (rows + slab - 1) / slab);
  colsum_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(dy), rows, o_total, ldy,
                                                                      slab, out);
  return static_cast<int>(cudaGetLastError());
}
