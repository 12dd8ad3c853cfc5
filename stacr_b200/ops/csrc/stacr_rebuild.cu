// Transient reconstruction of a compressed layer input for the tensor-core weight gradient:
//
//   Xhat[row, n] = bf16( sum_j C[row, j] Q[n, j] )          (rebuild_lowrank_kernel)
//   Xhat[row, n] = bf16( Xhat[row, n] + v )  for (row, n, v) in S   (rebuild_scatter_kernel)
//
// The saved factors stay what they are (coefficients, basis, sparse residual); Xhat lives only while one layer's
// backward runs, in a buffer that every layer reuses, and is the MN-major operand of dW = dY^T Xhat on the
// CTA-pair GEMM.  At a 0.5 % residual the gather form of the weight gradient moves nnz * out * 2 bytes
// (1.4 GB for an 8192-wide MLP layer); the dense product is 0.27 TFLOP, which the tensor cores finish sooner.
// Indices of S are unique, so the scatter needs no atomics.  Replaces the COO build + coalesce + cuSPARSE SpMM
// of the reference (stacr/layers.py:173-196 there) on large layers.
#include "common.cuh"

namespace sb {

constexpr int RB_COLS = 8;       // columns per thread: one 16-byte store
constexpr int RB_ROWS = 64;      // rows per CTA: the thread's 8 basis rows are loaded once and reused for all of them
constexpr int RB_THREADS = 128;  // 1024 columns per CTA
constexpr int RB_RMAX = 32;

template <int RP>
__global__ void __launch_bounds__(RB_THREADS) rebuild_lowrank_kernel(const __nv_bfloat16* __restrict__ c, const float* __restrict__ q, int r, int rows,
                                                              int n, __nv_bfloat16* __restrict__ out, int ldo) {
  __shared__ __align__(16) float s_c[RB_ROWS * RP];
  const int row0 = blockIdx.y * RB_ROWS;
  const int nrows = min(RB_ROWS, rows - row0);
  for (int i = threadIdx.x; i < RB_ROWS * RP; i += blockDim.x) {
    const int lr = i / RP, j = i - lr * RP;
    s_c[i] = (lr < nrows && j < r) ? __bfloat162float(c[static_cast<size_t>(row0 + lr) * r + j]) : 0.f;
  }
  __syncthreads();
  const int col0 = (blockIdx.x * blockDim.x + threadIdx.x) * RB_COLS;
  if (col0 >= n) return;
  float qreg[RB_COLS][RP];
  if (r == RP && col0 + RB_COLS <= n && ((reinterpret_cast<uintptr_t>(q) & 15) == 0)) {
    // a basis row is RP floats = RP / 4 16-byte vectors; the thread's 8 rows are one contiguous block
    const float4* src = reinterpret_cast<const float4*>(q + static_cast<size_t>(col0) * RP);
#pragma unroll
    for (int i = 0; i < RB_COLS; ++i)
#pragma unroll
      for (int v = 0; v < RP / 4; ++v) {
        const float4 t = __ldg(src + i * (RP / 4) + v);
        qreg[i][4 * v] = t.x; qreg[i][4 * v + 1] = t.y; qreg[i][4 * v + 2] = t.z; qreg[i][4 * v + 3] = t.w;
      }
  } else {
#pragma unroll
    for (int i = 0; i < RB_COLS; ++i)
#pragma unroll
      for (int j = 0; j < RP; ++j) qreg[i][j] = (col0 + i < n && j < r) ? __ldg(q + static_cast<size_t>(col0 + i) * r + j) : 0.f;
  }
  const bool vec = (col0 + RB_COLS <= n) && ((ldo & 7) == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
  for (int lr = 0; lr < nrows; ++lr) {
    float acc[RB_COLS];
#pragma unroll
    for (int i = 0; i < RB_COLS; ++i) acc[i] = 0.f;
#pragma unroll
    for (int v = 0; v < RP / 4; ++v) {
      const float4 cv = *reinterpret_cast<const float4*>(s_c + lr * RP + 4 * v);  // same address for the whole warp: a broadcast
      const float cj[4] = {cv.x, cv.y, cv.z, cv.w};
#pragma unroll
      for (int k = 0; k < 4; ++k)
#pragma unroll
        for (int i = 0; i < RB_COLS; ++i) acc[i] = fmaf(cj[k], qreg[i][4 * v + k], acc[i]);
    }
    __nv_bfloat16* o = out + static_cast<size_t>(row0 + lr) * ldo + col0;
    if (vec) {
      *reinterpret_cast<uint4*>(o) = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]),
                                                pack_bf16x2(acc[6], acc[7]));
    } else {
#pragma unroll
      for (int i = 0; i < RB_COLS; ++i)
        if (col0 + i < n) o[i] = __float2bfloat16_rn(acc[i]);
    }
  }
}

__global__ void rebuild_scatter_kernel(const int* __restrict__ idx32, const long long* __restrict__ idx64, long long nnz, int n, long long total,
                                       const void* __restrict__ val, int bits, const float* __restrict__ scale, __nv_bfloat16* __restrict__ out,
                                       int ldo) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= nnz) return;
  const long long flat = idx64 ? idx64[i] : static_cast<long long>(idx32[i]);
  if (flat < 0 || flat >= total) return;  // an index outside the tensor is ignored, never written
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
  __nv_bfloat16* o = out + (flat / n) * ldo + (flat % n);
  *o = __float2bfloat16_rn(__bfloat162float(*o) + v);
}

}  // namespace sb

// out[rows, n] (leading dimension ldo, bf16) = C Q^T, then the residual entries are added in place.
//   c: bf16 [rows, r] contiguous;  q: fp32 [n, r] contiguous;  idx32 xor idx64: nnz flat positions row * n + col (unique);
//   val: bf16 (bits 0), int8 codes (bits 8) or packed signed nibbles (bits 4) with *scale.
extern "C" int sb_rebuild_input(const void* c, const float* q, int r, int rows, int n, const int* idx32, const long long* idx64, long long nnz,
                                const void* val, int bits, const float* scale, void* out, int ldo, void* stream) {
  using namespace sb;
  if (rows <= 0 || n <= 0) return 0;
  if (r < 1 || r > RB_RMAX || ldo < n) return -2;
  if (nnz > 0 && ((idx32 == nullptr) == (idx64 == nullptr))) return -2;
  if (nnz > 0 && bits != 0 && bits != 4 && bits != 8) return -2;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const dim3 grid((n + RB_THREADS * RB_COLS - 1) / (RB_THREADS * RB_COLS), (rows + RB_ROWS - 1) / RB_ROWS);
  const __nv_bfloat16* cb = static_cast<const __nv_bfloat16*>(c);
  __nv_bfloat16* ob = static_cast<__nv_bfloat16*>(out);
  if (r <= 8)
    rebuild_lowrank_kernel<8><<<grid, RB_THREADS, 0, st>>>(cb, q, r, rows, n, ob, ldo);
  else if (r <= 16)
    rebuild_lowrank_kernel<16><<<grid, RB_THREADS, 0, st>>>(cb, q, r, rows, n, ob, ldo);
  else
    rebuild_lowrank_kernel<32><<<grid, RB_THREADS, 0, st>>>(cb, q, r, rows, n, ob, ldo);
  if (nnz > 0) {
    const int threads = 256;
    const long long blocks = (nnz + threads - 1) / threads;
    rebuild_scatter_kernel<<<static_cast<unsigned>(blocks), threads, 0, st>>>(idx32, idx64, nnz, n, static_cast<long long>(rows) * n, val, bits, scale,
                                                                            ob, ldo);
  }
  return static_cast<int>(cudaGetLastError());
}
