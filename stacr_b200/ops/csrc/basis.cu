// Basis maintenance on the device: the Oja subspace step followed by CholeskyQR2 in one kernel (the
// operands are N x r with r <= 32, a few hundred KB at most).  Rank <= 8 runs as a thread-block cluster
// of up to 8 CTAs: every thread keeps its rows of Q in registers from the Oja step to the final store, and
// the three r x r Gram matrices are reduced through distributed shared memory.  Larger ranks use one CTA.
//
//   A = Q + lr * (G / n - Q * (S / n)),   G = X^T Y (from the skinny tensor-core GEMM),
//                                         S = Y^T Y (reduced here from Y),
//   Q' = A R^-1 with R^T R = A^T A, applied twice.
//
// A is a small perturbation of an orthonormal matrix, so its Gram matrix is close to the
// identity and CholeskyQR2 reaches fp32 orthogonality; the subspace equals the one a
// Householder QR returns (column signs may differ, which cancels in C Q^T).
// Outputs: the fp32 basis, a bf16 copy [N, r] and a zero-padded bf16 transpose [rpad, N]
// that the projection GEMM reads as its K-major B operand.
// Replaces four library GEMMs and a cuSOLVER QR per step (stacr/layers.py:350-353 and
// stacr/oja.py:8-11 of the reference project).
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace sb {

constexpr int RMAX = 32;

// gram[i][j] = sum_rows f(a[row, i]) * f(a[row, j]) over `count` rows of an [count, lda] matrix, where
// f rounds to bf16 when `round_bf16` is set (so that the same rounded values are used as in the
// tensor-core product they are compared with).  Row i of the Gram matrix is reduced per pass:
// per-thread partial sums -> warp shuffles -> one shared-memory partial per warp.
template <int RP>
__device__ void block_gram(const float* a, int count, int lda, int r, bool round_bf16, float* gram, float* partial /*[32][RP]*/) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int i = 0; i < r; ++i) {
    float acc[RP];
#pragma unroll
    for (int j = 0; j < RP; ++j) acc[j] = 0.f;
    for (int row = threadIdx.x; row < count; row += blockDim.x) {
      const float* ar = a + static_cast<size_t>(row) * lda;
      float ai = ar[i];
      if (round_bf16) ai = __bfloat162float(__float2bfloat16_rn(ai));
#pragma unroll
      for (int j = 0; j < RP; ++j) {
        if (j <= i) {
          float aj = ar[j];
          if (round_bf16) aj = __bfloat162float(__float2bfloat16_rn(aj));
          acc[j] = fmaf(ai, aj, acc[j]);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < RP; ++j) {
      if (j <= i) {
        float v = acc[j];
        for (int off = 16; off; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        if (lane == 0) partial[warp * RP + j] = v;
      }
    }
    __syncthreads();
    if (threadIdx.x <= i) {
      float total = 0.f;
      for (int w = 0; w < nwarps; ++w) total += partial[w * RP + threadIdx.x];
      gram[i * RMAX + threadIdx.x] = total;
      gram[threadIdx.x * RMAX + i] = total;
    }
    __syncthreads();
  }
}

// Rank <= 8 fast path: all 36 entries of the upper triangle in one pass over the rows.
__device__ void block_gram8(const float* a, int count, int lda, int r, bool round_bf16, float* gram, float* partial /*[32][36]*/) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  float acc[36];
#pragma unroll
  for (int k = 0; k < 36; ++k) acc[k] = 0.f;
  for (int row = threadIdx.x; row < count; row += blockDim.x) {
    const float* ar = a + static_cast<size_t>(row) * lda;
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      v[j] = (j < r) ? ar[j] : 0.f;
      if (round_bf16) v[j] = __bfloat162float(__float2bfloat16_rn(v[j]));
    }
    int k = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j <= i; ++j) {
        acc[k] = fmaf(v[i], v[j], acc[k]);
        ++k;
      }
  }
#pragma unroll
  for (int k = 0; k < 36; ++k) {
    float v = acc[k];
    for (int off = 16; off; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    if (lane == 0) partial[warp * 36 + k] = v;
  }
  __syncthreads();
  if (threadIdx.x < 36) {
    float total = 0.f;
    for (int w = 0; w < nwarps; ++w) total += partial[w * 36 + threadIdx.x];
    int i = 0, base = 0;
    while (base + i + 1 <= static_cast<int>(threadIdx.x)) {
      base += i + 1;
      ++i;
    }
    const int j = threadIdx.x - base;
    gram[i * RMAX + j] = total;
    gram[j * RMAX + i] = total;
  }
  __syncthreads();
}

// In-place upper Cholesky factor R (R^T R = G) and its inverse, by thread 0.  Returns false in
// shared flag when a pivot is not positive.
__device__ void chol_and_invert(float* g, float* rinv, int r, int* ok) {
  if (threadIdx.x == 0) {
    *ok = 1;
    // g <- R (upper), row by row
    for (int i = 0; i < r; ++i) {
      float d = g[i * RMAX + i];
      for (int k = 0; k < i; ++k) d -= g[k * RMAX + i] * g[k * RMAX + i];
      if (!(d > 1e-20f)) {
        *ok = 0;
        d = 1.f;
      }
      const float rii = sqrtf(d);
      g[i * RMAX + i] = rii;
      for (int j = i + 1; j < r; ++j) {
        float v = g[i * RMAX + j];
        for (int k = 0; k < i; ++k) v -= g[k * RMAX + i] * g[k * RMAX + j];
        g[i * RMAX + j] = v / rii;
      }
      for (int j = 0; j < i; ++j) g[i * RMAX + j] = 0.f;
    }
    // rinv <- R^-1 (upper) by back substitution
    for (int j = 0; j < r; ++j) {
      for (int i = 0; i < r; ++i) rinv[i * RMAX + j] = 0.f;
      rinv[j * RMAX + j] = 1.f / g[j * RMAX + j];
      for (int i = j - 1; i >= 0; --i) {
        float v = 0.f;
        for (int k = i + 1; k <= j; ++k) v += g[i * RMAX + k] * rinv[k * RMAX + j];
        rinv[i * RMAX + j] = -v / g[i * RMAX + i];
      }
    }
  }
  __syncthreads();
}

template <int RP>
__global__ void __launch_bounds__(1024) oja_update_kernel(const float* q_in, const float* g, int ldg, const float* y, int ldy,
                                                          int rows, int n, int r, float lr, float* q_out,
                                                          __nv_bfloat16* q_bf16, __nv_bfloat16* qt_bf16, int rpad, int* status) {
  __shared__ float s_mat[RMAX * RMAX];
  __shared__ float s_inv[RMAX * RMAX];
  __shared__ float scratch[32 * (RP > 36 ? RP : 36)];
  __shared__ int s_ok;
  const float inv_n = 1.f / fmaxf(1.f, static_cast<float>(rows));
  if (lr != 0.f && g != nullptr) {
    if (RP == 8) block_gram8(y, rows, ldy, r, true, s_mat, scratch);  // S = Y^T Y
    else block_gram<RP>(y, rows, ldy, r, true, s_mat, scratch);
    for (int row = threadIdx.x; row < n; row += blockDim.x) {
      float qrow[RP];
      for (int j = 0; j < r; ++j) qrow[j] = q_in[static_cast<size_t>(row) * r + j];
      for (int j = 0; j < r; ++j) {
        float qs = 0.f;
        for (int k = 0; k < r; ++k) qs = fmaf(qrow[k], s_mat[k * RMAX + j], qs);
        q_out[static_cast<size_t>(row) * r + j] = qrow[j] + lr * inv_n * (g[static_cast<size_t>(row) * ldg + j] - qs);
      }
    }
  } else {
    for (int i = threadIdx.x; i < n * r; i += blockDim.x) q_out[i] = q_in[i];
  }
  __syncthreads();
  for (int pass = 0; pass < 2; ++pass) {
    if (RP == 8) block_gram8(q_out, n, r, r, false, s_mat, scratch);
    else block_gram<RP>(q_out, n, r, r, false, s_mat, scratch);
    chol_and_invert(s_mat, s_inv, r, &s_ok);
    if (!s_ok) {
      if (threadIdx.x == 0 && status) atomicCAS(status, 0, ST_BAD_ARGUMENT);
      break;
    }
    for (int row = threadIdx.x; row < n; row += blockDim.x) {
      float a[RP];
      for (int j = 0; j < r; ++j) a[j] = q_out[static_cast<size_t>(row) * r + j];
      for (int j = 0; j < r; ++j) {
        float v = 0.f;
        for (int k = 0; k <= j; ++k) v = fmaf(a[k], s_inv[k * RMAX + j], v);
        q_out[static_cast<size_t>(row) * r + j] = v;
      }
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < n * r; i += blockDim.x) {
    const float v = q_out[i];
    if (q_bf16) q_bf16[i] = __float2bfloat16_rn(v);
  }
  if (qt_bf16) {
    for (int i = threadIdx.x; i < n * rpad; i += blockDim.x) {
      const int j = i / n, row = i - j * n;
      qt_bf16[i] = (j < r) ? __float2bfloat16_rn(q_out[static_cast<size_t>(row) * r + j]) : __float2bfloat16_rn(0.f);
    }
  }
}


// Upper Cholesky factor of an 8 x 8 Gram matrix and its inverse, entirely in the registers of one thread (every loop
// has compile-time bounds, so the arrays never touch memory).  Unused trailing rows/columns (r < 8) are treated as
// identity.  The result goes to rinv (shared, row stride RMAX).
__device__ __forceinline__ bool chol_and_invert8_regs(const float* g_sh, float* rinv_sh, int r) {
  float a[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) a[i][j] = (i < r && j < r) ? g_sh[i * RMAX + j] : (i == j ? 1.f : 0.f);
  bool ok = true;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float d = a[i][i];
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (k < i) d -= a[k][i] * a[k][i];
    if (!(d > 1e-20f)) {
      ok = false;
      d = 1.f;
    }
    const float rii = sqrtf(d), inv = 1.f / rii;
    a[i][i] = rii;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (j > i) {
        float v = a[i][j];
#pragma unroll
        for (int k = 0; k < 8; ++k)
          if (k < i) v -= a[k][i] * a[k][j];
        a[i][j] = v * inv;
      }
    }
  }
  float x[8][8];  // R^-1, upper triangular, by back substitution column by column
#pragma unroll
  for (int j = 0; j < 8; ++j) {
#pragma unroll
    for (int i = 7; i >= 0; --i) {
      if (i > j) {
        x[i][j] = 0.f;
      } else if (i == j) {
        x[i][j] = 1.f / a[j][j];
      } else {
        float v = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k)
          if (k > i && k <= j) v += a[i][k] * x[k][j];
        x[i][j] = -v / a[i][i];
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) rinv_sh[i * RMAX + j] = x[i][j];
  return ok;
}

// ---------------------------------------------------------------------------------------------------------
// Cluster version for r <= 8.
constexpr int OJA_ROWS_PT = 4;  // basis rows per thread: n <= cluster size * 1024 * 4

__device__ __forceinline__ void accumulate_upper8(const float (&v)[8], float (&acc)[36]) {
  int k = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j <= i; ++j) {
      acc[k] = fmaf(v[i], v[j], acc[k]);
      ++k;
    }
}

// acc (36 upper-triangle sums of this thread) -> symmetric r x r total over the whole cluster in s_gram.
// s_part must be zero on entry and is zero again on exit.
// One round of a reduce-scatter across the warp: of N_IN values per lane, the lanes with bit `OFF` clear keep the first N_OUT,
// the others the rest, each adding what its partner (lane ^ OFF) held of the kept half.
template <int N_IN, int N_OUT, int OFF>
__device__ __forceinline__ void scatter_round(const float (&in)[N_IN], float (&out)[N_OUT], int lane) {
  const bool hi = (lane & OFF) != 0;
#pragma unroll
  for (int i = 0; i < N_OUT; ++i) {
    const float lo_v = in[i];
    const float hi_v = (i + N_OUT < N_IN) ? in[i + N_OUT] : 0.f;
    out[i] = (hi ? hi_v : lo_v) + __shfl_xor_sync(0xffffffffu, hi ? lo_v : hi_v, OFF);
  }
}

__device__ void cluster_gram8(cg::cluster_group& cluster, const float (&acc)[36], float* s_part, float* s_gram) {
  const int lane = threadIdx.x & 31;
  // 36 sums per lane -> at most 2 finished sums per lane in 37 shuffles (a butterfly that halves the values it carries at
  // every step) instead of 36 x 5: the shuffle unit moves one warp per clock per SM, and 32 warps x 180 shuffles per Gram
  // matrix, three matrices per update, was most of this kernel's 43 us.
  float a18[18], a9[9], a5[5], a3[3], a2[2];
  scatter_round<36, 18, 16>(acc, a18, lane);
  scatter_round<18, 9, 8>(a18, a9, lane);
  scatter_round<9, 5, 4>(a9, a5, lane);
  scatter_round<5, 3, 2>(a5, a3, lane);
  scatter_round<3, 2, 1>(a3, a2, lane);
  {
    const int b4 = (lane >> 4) & 1, b3 = (lane >> 3) & 1, b2 = (lane >> 2) & 1, b1 = (lane >> 1) & 1, b0 = lane & 1;
    const int l3 = b2 ? 4 : 5;                       // values this lane's group still carried after each uneven split
    const int l4 = b1 ? l3 - 3 : 3;
    const int l5 = b0 ? l4 - 2 : (l4 < 2 ? l4 : 2);
    const int base = 18 * b4 + 9 * b3 + 5 * b2 + 3 * b1 + 2 * b0;
    if (0 < l5) atomicAdd(&s_part[base], a2[0]);
    if (1 < l5) atomicAdd(&s_part[base + 1], a2[1]);
  }
  cluster.sync();  // every CTA's partial is complete
  if (threadIdx.x < 36) {
    float total = 0.f;
    const int nb = static_cast<int>(cluster.num_blocks());
    for (int b = 0; b < nb; ++b) total += cluster.map_shared_rank(s_part, b)[threadIdx.x];
    int i = 0, base = 0;
    while (base + i + 1 <= static_cast<int>(threadIdx.x)) {
      base += i + 1;
      ++i;
    }
    const int j = threadIdx.x - base;
    s_gram[i * RMAX + j] = total;
    s_gram[j * RMAX + i] = total;
  }
  cluster.sync();  // every CTA has read every partial
  if (threadIdx.x < 36) s_part[threadIdx.x] = 0.f;
  __syncthreads();
}

template <int ROWS_PT>
__global__ void __launch_bounds__(1024) oja_update_cluster8_kernel(const float* __restrict__ q_in, const float* __restrict__ g, int ldg,
                                                                   const float* __restrict__ y, int ldy, int rows, int n, int r, float lr,
                                                                   float* __restrict__ q_out, __nv_bfloat16* __restrict__ q_bf16,
                                                                   __nv_bfloat16* __restrict__ qt_bf16, int rpad, int* status) {
  cg::cluster_group cluster = cg::this_cluster();
  __shared__ float s_part[36];
  __shared__ float s_mat[RMAX * RMAX];
  __shared__ float s_inv[RMAX * RMAX];
  __shared__ int s_ok;
  if (threadIdx.x < 36) s_part[threadIdx.x] = 0.f;
  __syncthreads();
  const int gthreads = static_cast<int>(cluster.num_blocks()) * blockDim.x;
  const int gtid = static_cast<int>(cluster.block_rank()) * blockDim.x + threadIdx.x;
  const float inv_n = 1.f / fmaxf(1.f, static_cast<float>(rows));
  float qrow[ROWS_PT][8];
#pragma unroll
  for (int t = 0; t < ROWS_PT; ++t) {
    const int row = gtid + t * gthreads;
    if (r == 8 && row < n) {  // a row is 32 bytes: two 16-byte loads
      const float4 lo = reinterpret_cast<const float4*>(q_in + static_cast<size_t>(row) * 8)[0];
      const float4 hi = reinterpret_cast<const float4*>(q_in + static_cast<size_t>(row) * 8)[1];
      qrow[t][0] = lo.x; qrow[t][1] = lo.y; qrow[t][2] = lo.z; qrow[t][3] = lo.w;
      qrow[t][4] = hi.x; qrow[t][5] = hi.y; qrow[t][6] = hi.z; qrow[t][7] = hi.w;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) qrow[t][j] = (row < n && j < r) ? q_in[static_cast<size_t>(row) * r + j] : 0.f;
    }
  }
  if (lr != 0.f && g != nullptr) {
    float acc[36];
#pragma unroll
    for (int k = 0; k < 36; ++k) acc[k] = 0.f;
    for (int row = gtid; row < rows; row += gthreads) {  // S = Y^T Y on the bf16-rounded coefficients
      const float* yr = y + static_cast<size_t>(row) * ldy;
      float v[8];
      if ((ldy & 3) == 0) {  // rows are 16-byte aligned: two vector loads, then mask the columns past r
        const float4 lo = reinterpret_cast<const float4*>(yr)[0];
        const float4 hi = reinterpret_cast<const float4*>(yr)[1];
        v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w; v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = (j < r) ? yr[j] : 0.f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = (j < r) ? __bfloat162float(__float2bfloat16_rn(v[j])) : 0.f;
      accumulate_upper8(v, acc);
    }
    cluster_gram8(cluster, acc, s_part, s_mat);
#pragma unroll
    for (int t = 0; t < ROWS_PT; ++t) {
      const int row = gtid + t * gthreads;
      if (row >= n) continue;
      float next[8], gv[8];
      const float* gr = g + static_cast<size_t>(row) * ldg;
      if ((ldg & 3) == 0) {  // rows are 16-byte aligned: two vector loads
        const float4 lo = reinterpret_cast<const float4*>(gr)[0], hi = reinterpret_cast<const float4*>(gr)[1];
        gv[0] = lo.x; gv[1] = lo.y; gv[2] = lo.z; gv[3] = lo.w; gv[4] = hi.x; gv[5] = hi.y; gv[6] = hi.z; gv[7] = hi.w;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) gv[j] = (j < r) ? gr[j] : 0.f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float qs = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) qs = fmaf(qrow[t][k], s_mat[k * RMAX + j], qs);
        next[j] = (j < r) ? qrow[t][j] + lr * inv_n * (gv[j] - qs) : 0.f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) qrow[t][j] = next[j];
    }
  }
  for (int pass = 0; pass < 2; ++pass) {  // CholeskyQR2
    float acc[36];
#pragma unroll
    for (int k = 0; k < 36; ++k) acc[k] = 0.f;
#pragma unroll
    for (int t = 0; t < ROWS_PT; ++t) accumulate_upper8(qrow[t], acc);  // rows past n are zero
    cluster_gram8(cluster, acc, s_part, s_mat);
    if (threadIdx.x == 0) s_ok = chol_and_invert8_regs(s_mat, s_inv, r) ? 1 : 0;  // the same numbers in every CTA: uniform outcome
    __syncthreads();
    if (!s_ok) {
      if (threadIdx.x == 0 && status) atomicCAS(status, 0, ST_BAD_ARGUMENT);
      break;
    }
#pragma unroll
    for (int t = 0; t < ROWS_PT; ++t) {
      float next[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float v = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k)
          if (k <= j && j < r) v = fmaf(qrow[t][k], s_inv[k * RMAX + j], v);
        next[j] = v;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) qrow[t][j] = next[j];
    }
    __syncthreads();
  }
#pragma unroll
  for (int t = 0; t < ROWS_PT; ++t) {
    const int row = gtid + t * gthreads;
    if (row >= n) continue;
    if (r == 8) {  // a row is 32 bytes of fp32 and 16 bytes of bf16: vector stores
      float4* qo = reinterpret_cast<float4*>(q_out + static_cast<size_t>(row) * 8);
      qo[0] = make_float4(qrow[t][0], qrow[t][1], qrow[t][2], qrow[t][3]);
      qo[1] = make_float4(qrow[t][4], qrow[t][5], qrow[t][6], qrow[t][7]);
      if (q_bf16)
        *reinterpret_cast<uint4*>(q_bf16 + static_cast<size_t>(row) * 8) =
            make_uint4(pack_bf16x2(qrow[t][0], qrow[t][1]), pack_bf16x2(qrow[t][2], qrow[t][3]), pack_bf16x2(qrow[t][4], qrow[t][5]),
                       pack_bf16x2(qrow[t][6], qrow[t][7]));
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (j < r) {
          q_out[static_cast<size_t>(row) * r + j] = qrow[t][j];
          if (q_bf16) q_bf16[static_cast<size_t>(row) * r + j] = __float2bfloat16_rn(qrow[t][j]);
        }
      }
    }
    if (qt_bf16) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (j < rpad) qt_bf16[static_cast<size_t>(j) * n + row] = __float2bfloat16_rn(j < r ? qrow[t][j] : 0.f);
      for (int j = 8; j < rpad; ++j) qt_bf16[static_cast<size_t>(j) * n + row] = __float2bfloat16_rn(0.f);
    }
  }
  cluster.sync();  // no CTA leaves while a peer may still read its shared memory
}

}  // namespace sb

// Q' = orth(Q + lr (G/rows - Q (Y^T Y)/rows)).  g: [n, ldg] fp32; y: [rows, ldy] fp32 (both may be NULL
// with lr == 0 to only re-orthonormalise and refresh the bf16 copies).  q_out must not alias q_in.
namespace sb {

// ------------------------------------------------------------------------------------------------
// Small dense algebra for the basis initialisation (no library solver): orthonormalisation of a tall thin matrix by
// modified Gram-Schmidt with re-orthogonalisation, the Gram matrix of a tall thin matrix, and the eigen-decomposition of
// a symmetric matrix of order <= 32 by cyclic Jacobi rotations.  One-off work per layer; written for robustness (the
// iterates of a subspace iteration are close to collinear, which breaks Cholesky-based orthonormalisation in fp32).
// ------------------------------------------------------------------------------------------------
constexpr int SMALL_W = 32;

// In place: columns of a[n, w] (row-major, leading dimension lda) become orthonormal.  One CTA of 1024 threads.
// For every column: two rounds of (coefficients against all previous columns in ONE block reduction, subtract), then
// normalise.  A column that vanishes (rank deficiency) is replaced by a unit vector orthogonalised the same way.
__global__ void __launch_bounds__(1024) mgs_qr_kernel(float* a, int n, int w, int lda) {
  __shared__ float s_red[32][SMALL_W + 1];
  __shared__ float s_coef[SMALL_W + 1];
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  for (int j = 0; j < w; ++j) {
    for (int attempt = 0; attempt < 2; ++attempt) {
      for (int round = 0; round < 2; ++round) {
        // coefficients c[i] = <a_i, a_j> for i < j, and the squared norm of a_j in slot j
        float part[SMALL_W + 1];
#pragma unroll
        for (int i = 0; i <= SMALL_W; ++i) part[i] = 0.f;
        for (int row = t; row < n; row += blockDim.x) {
          const float v = a[static_cast<size_t>(row) * lda + j];
#pragma unroll
          for (int i = 0; i < SMALL_W; ++i)
            if (i < j) part[i] = fmaf(a[static_cast<size_t>(row) * lda + i], v, part[i]);
          part[SMALL_W] = fmaf(v, v, part[SMALL_W]);
        }
#pragma unroll
        for (int i = 0; i <= SMALL_W; ++i) {
          float v = part[i];
#pragma unroll
          for (int off = 16; off; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
          if (lane == 0) s_red[warp][i] = v;
        }
        __syncthreads();
        if (t <= SMALL_W) {
          float v = 0.f;
          for (int k = 0; k < 32; ++k) v += s_red[k][t];
          s_coef[t] = v;
        }
        __syncthreads();
        for (int row = t; row < n; row += blockDim.x) {
          float v = a[static_cast<size_t>(row) * lda + j];
          for (int i = 0; i < j; ++i) v = fmaf(-s_coef[i], a[static_cast<size_t>(row) * lda + i], v);
          a[static_cast<size_t>(row) * lda + j] = v;
        }
        __syncthreads();
      }
      // norm after the two rounds
      float nn = 0.f;
      for (int row = t; row < n; row += blockDim.x) {
        const float v = a[static_cast<size_t>(row) * lda + j];
        nn = fmaf(v, v, nn);
      }
#pragma unroll
      for (int off = 16; off; off >>= 1) nn += __shfl_xor_sync(0xffffffffu, nn, off);
      if (lane == 0) s_red[warp][0] = nn;
      __syncthreads();
      if (t == 0) {
        float v = 0.f;
        for (int k = 0; k < 32; ++k) v += s_red[k][0];
        s_coef[0] = v;
      }
      __syncthreads();
      const float norm2 = s_coef[0];
      __syncthreads();
      if (norm2 > 1e-20f) {
        const float inv = rsqrtf(norm2);
        for (int row = t; row < n; row += blockDim.x) a[static_cast<size_t>(row) * lda + j] *= inv;
        __syncthreads();
        break;
      }
      // the column vanished: restart it from the unit vector e_(j mod n) and orthogonalise again
      for (int row = t; row < n; row += blockDim.x) a[static_cast<size_t>(row) * lda + j] = (row == j % n) ? 1.f : 0.f;
      __syncthreads();
    }
  }
}

// out[w, w] += a^T a for a[rows, w] (row-major, lda), w <= 32; out zeroed by the caller.  CTA (32 x 32 threads) per row slab.
__global__ void __launch_bounds__(1024) gram_small_kernel(const float* a, int rows, int w, int lda, int slab, double* out) {
  const int i = threadIdx.y, j = threadIdx.x;
  const int r0 = blockIdx.x * slab, r1 = min(rows, r0 + slab);
  double acc = 0.0;
  if (i < w && j < w)
    for (int row = r0; row < r1; ++row) acc += static_cast<double>(a[static_cast<size_t>(row) * lda + i]) * static_cast<double>(a[static_cast<size_t>(row) * lda + j]);
  if (i < w && j < w) atomicAdd(out + i * w + j, acc);
}

// Eigen-decomposition of the symmetric matrix m[w, w] (fp64, row-major), w <= 32, by cyclic Jacobi rotations in one warp
// (lane k owns row k of the working matrix and of the accumulated rotations).  Eigenvalues in descending order in
// evals[w]; the matching eigenvectors are the COLUMNS of evecs[w, w].
__global__ void __launch_bounds__(32) jacobi_eig_kernel(const double* m, int w, double* evals, double* evecs) {
  __shared__ double A[SMALL_W][SMALL_W + 1];
  __shared__ double V[SMALL_W][SMALL_W + 1];
  __shared__ int order[SMALL_W];
  const int k = threadIdx.x;
  for (int j = 0; j < w; ++j) {
    if (k < w) {
      A[k][j] = 0.5 * (m[k * w + j] + m[j * w + k]);
      V[k][j] = (k == j) ? 1.0 : 0.0;
    }
  }
  __syncwarp();
  for (int sweep = 0; sweep < 30; ++sweep) {
    double off = 0.0;
    if (k < w)
      for (int j = 0; j < w; ++j)
        if (j != k) off += A[k][j] * A[k][j];
#pragma unroll
    for (int o = 16; o; o >>= 1) off += __shfl_xor_sync(0xffffffffu, off, o);
    double diag = (k < w) ? fabs(A[k][k]) : 0.0;
#pragma unroll
    for (int o = 16; o; o >>= 1) diag = fmax(diag, __shfl_xor_sync(0xffffffffu, diag, o));
    if (off <= 1e-28 * diag * diag + 1e-300) break;
    for (int p = 0; p < w - 1; ++p) {
      for (int q = p + 1; q < w; ++q) {
        const double apq = A[p][q];
        double c = 1.0, s = 0.0;
        if (fabs(apq) > 1e-300) {
          const double theta = (A[q][q] - A[p][p]) / (2.0 * apq);
          const double tt = (theta >= 0.0 ? 1.0 : -1.0) / (fabs(theta) + sqrt(theta * theta + 1.0));
          c = 1.0 / sqrt(tt * tt + 1.0);
          s = tt * c;
        }
        __syncwarp();
        if (k < w) {  // columns p and q of A and V, row k
          const double akp = A[k][p], akq = A[k][q];
          A[k][p] = c * akp - s * akq;
          A[k][q] = s * akp + c * akq;
          const double vkp = V[k][p], vkq = V[k][q];
          V[k][p] = c * vkp - s * vkq;
          V[k][q] = s * vkp + c * vkq;
        }
        __syncwarp();
        if (k < w) {  // rows p and q of A, column k
          const double apk = A[p][k], aqk = A[q][k];
          A[p][k] = c * apk - s * aqk;
          A[q][k] = s * apk + c * aqk;
        }
        __syncwarp();
      }
    }
  }
  if (k == 0) {  // selection sort of the diagonal, descending
    for (int i = 0; i < w; ++i) order[i] = i;
    for (int i = 0; i < w; ++i)
      for (int j = i + 1; j < w; ++j)
        if (A[order[j]][order[j]] > A[order[i]][order[i]]) {
          const int tmp = order[i];
          order[i] = order[j];
          order[j] = tmp;
        }
  }
  __syncwarp();
  if (k < w) {
    evals[k] = A[order[k]][order[k]];
    for (int j = 0; j < w; ++j) evecs[k * w + j] = V[k][order[j]];
  }
}

}  // namespace sb

// Orthonormalise the columns of fp32 a[n, w] in place (w <= 32).
extern "C" int sb_mgs_qr(float* a, int n, int w, int lda, void* stream) {
  if (n <= 0 || w <= 0) return 0;
  if (w > sb::SMALL_W) return -2;
  sb::mgs_qr_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(a, n, w, lda);
  return static_cast<int>(cudaGetLastError());
}

// out (fp64 [w, w], zeroed by the caller) += a^T a for fp32 a[rows, w], w <= 32.
extern "C" int sb_gram_small(const float* a, int rows, int w, int lda, double* out, void* stream) {
  if (rows <= 0 || w <= 0) return 0;
  if (w > sb::SMALL_W) return -2;
  const int slab = 256;
  sb::gram_small_kernel<<<(rows + slab - 1) / slab, dim3(32, 32), 0, static_cast<cudaStream_t>(stream)>>>(a, rows, w, lda, slab, out);
  return static_cast<int>(cudaGetLastError());
}

// Symmetric eigen-decomposition of fp64 m[w, w], w <= 32: evals descending, eigenvectors in the columns of evecs.
extern "C" int sb_jacobi_eig(const double* m, int w, double* evals, double* evecs, void* stream) {
  if (w <= 0) return 0;
  if (w > sb::SMALL_W) return -2;
  sb::jacobi_eig_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(m, w, evals, evecs);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int sb_oja_update(const float* q_in, const float* g, int ldg, const float* y, int ldy, int rows, int n, int r,
                             float lr, float* q_out, void* q_bf16, void* qt_bf16, int rpad, int* status, void* stream) {
  if (r < 1 || r > sb::RMAX) return -2;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  __nv_bfloat16* qb = static_cast<__nv_bfloat16*>(q_bf16);
  __nv_bfloat16* qt = static_cast<__nv_bfloat16*>(qt_bf16);
  if (r <= 8 && n <= 8 * 1024 * sb::OJA_ROWS_PT) {
    const int want = (n > rows ? n : rows);
    unsigned csize = 1;
    while (csize < 8 && static_cast<int>(csize) * 1024 < want) csize <<= 1;
    while (static_cast<long long>(csize) * 1024 * sb::OJA_ROWS_PT < n) csize <<= 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(csize, 1, 1);
    cfg.blockDim = dim3(1024, 1, 1);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = csize;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (static_cast<long long>(csize) * 1024 >= n)
      return static_cast<int>(cudaLaunchKernelEx(&cfg, sb::oja_update_cluster8_kernel<1>, q_in, g, ldg, y, ldy, rows, n, r, lr, q_out, qb, qt, rpad, status));
    return static_cast<int>(cudaLaunchKernelEx(&cfg, sb::oja_update_cluster8_kernel<sb::OJA_ROWS_PT>, q_in, g, ldg, y, ldy, rows, n, r, lr, q_out, qb, qt, rpad, status));
  }
  if (r <= 8) sb::oja_update_kernel<8><<<1, 1024, 0, st>>>(q_in, g, ldg, y, ldy, rows, n, r, lr, q_out, qb, qt, rpad, status);
  else if (r <= 16) sb::oja_update_kernel<16><<<1, 1024, 0, st>>>(q_in, g, ldg, y, ldy, rows, n, r, lr, q_out, qb, qt, rpad, status);
  else sb::oja_update_kernel<32><<<1, 1024, 0, st>>>(q_in, g, ldg, y, ldy, rows, n, r, lr, q_out, qb, qt, rpad, status);
  return static_cast<int>(cudaGetLastError());
}
