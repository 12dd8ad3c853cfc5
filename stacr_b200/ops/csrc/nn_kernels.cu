// Bandwidth-bound model ops for bf16 training on sm_100a: LayerNorm forward/backward (fp32
// statistics kept per row), GELU forward/backward (erf and tanh forms), and a fused softmax
// cross-entropy whose forward pass also writes the logit gradient, so the logits are read
// twice and written once in total.  All loads and stores are 16-byte vectors.
// These replace the ATen LayerNorm / GELU / log-softmax + NLL kernels the reference reaches
// through the Hugging Face model code it trains.
#include "common.cuh"

namespace sb {

__device__ __forceinline__ void unpack8(const uint4& raw, float (&f)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __low2float(p[i]);
    f[2 * i + 1] = __high2float(p[i]);
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  return make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int off = 16; off; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int off = 16; off; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
  return v;
}

// ---------------------------------------------------------------------------- LayerNorm
// One warp per row; the row (n <= 16384, n % 8 == 0) lives in registers: MAXV vectors of 8 per lane.
// With a second (gamma2, beta2, y2) the same statistics feed a second affine output: the two normalisations of a
// parallel-residual block (attention and MLP branch read the same x) cost one read of x.
template <int MAXV>
__global__ void __launch_bounds__(256) layernorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ gamma,
                                                            const float* __restrict__ beta, int rows, int n, float eps,
                                                            __nv_bfloat16* __restrict__ y, float* __restrict__ mean_out,
                                                            float* __restrict__ rstd_out, const float* __restrict__ gamma2 = nullptr,
                                                            const float* __restrict__ beta2 = nullptr,
                                                            __nv_bfloat16* __restrict__ y2 = nullptr) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int nvec = n >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * n);
  uint4 raw[MAXV];   // the row stays packed (half the registers of its fp32 form) and is unpacked once per pass
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int vi = lane + i * 32;
    if (vi < nvec) {
      raw[i] = __ldg(xr + vi);
      float v[8];
      unpack8(raw[i], v);
#pragma unroll
      for (int j = 0; j < 8; ++j) sum += v[j];
    }
  }
  const float mean = warp_sum(sum) / n;
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    if (lane + i * 32 < nvec) {
      float v[8];
      unpack8(raw[i], v);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float d = v[j] - mean;
        sq = fmaf(d, d, sq);
      }
    }
  }
  const float rstd = rsqrtf(warp_sum(sq) / n + eps);
  if (lane == 0) {
    mean_out[row] = mean;
    rstd_out[row] = rstd;
  }
  uint4* yr = reinterpret_cast<uint4*>(y + static_cast<size_t>(row) * n);
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int vi = lane + i * 32;
    if (vi < nvec) {
      float o[8];
      const float4 g0 = __ldg(reinterpret_cast<const float4*>(gamma) + vi * 2), g1 = __ldg(reinterpret_cast<const float4*>(gamma) + vi * 2 + 1);
      const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
      float b[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      if (beta) {
        const float4 b0 = __ldg(reinterpret_cast<const float4*>(beta) + vi * 2), b1 = __ldg(reinterpret_cast<const float4*>(beta) + vi * 2 + 1);
        b[0] = b0.x; b[1] = b0.y; b[2] = b0.z; b[3] = b0.w; b[4] = b1.x; b[5] = b1.y; b[6] = b1.z; b[7] = b1.w;
      }
#pragma unroll
      float v[8];
      unpack8(raw[i], v);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = (v[j] - mean) * rstd * g[j] + b[j];
      yr[vi] = pack8(o);
      if (y2) {
        const float4 h0 = __ldg(reinterpret_cast<const float4*>(gamma2) + vi * 2), h1 = __ldg(reinterpret_cast<const float4*>(gamma2) + vi * 2 + 1);
        const float g2[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
        float b2[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (beta2) {
          const float4 c0 = __ldg(reinterpret_cast<const float4*>(beta2) + vi * 2), c1 = __ldg(reinterpret_cast<const float4*>(beta2) + vi * 2 + 1);
          b2[0] = c0.x; b2[1] = c0.y; b2[2] = c0.z; b2[3] = c0.w; b2[4] = c1.x; b2[5] = c1.y; b2[6] = c1.z; b2[7] = c1.w;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = (v[j] - mean) * rstd * g2[j] + b2[j];
        reinterpret_cast<uint4*>(y2 + static_cast<size_t>(row) * n)[vi] = pack8(o);
      }
    }
  }
}

// dx per row: one warp per row, two passes, the second re-reading the row from L1 / L2 (see layernorm_bwd_dx2_kernel).
template <int MAXV>
__global__ void __launch_bounds__(256) layernorm_bwd_dx_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                                               const float* __restrict__ gamma, const float* __restrict__ mean,
                                                               const float* __restrict__ rstd, int rows, int n,
                                                               __nv_bfloat16* __restrict__ dx) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int nvec = n >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * n);
  const uint4* dr = reinterpret_cast<const uint4*>(dy + static_cast<size_t>(row) * n);
  const float4* gv = reinterpret_cast<const float4*>(gamma);
  const float mu = mean[row], rs = rstd[row];
  float s1 = 0.f, s2 = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int vi = lane + i * 32;
    if (vi < nvec) {
      float xv[8], dv[8];
      unpack8(__ldg(xr + vi), xv);
      unpack8(__ldg(dr + vi), dv);
      const float4 g0 = __ldg(gv + vi * 2), g1 = __ldg(gv + vi * 2 + 1);
      const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float dg = dv[j] * g[j];
        s1 += dg;
        s2 = fmaf(dg, (xv[j] - mu) * rs, s2);
      }
    }
  }
  s1 = warp_sum(s1) / n;
  s2 = warp_sum(s2) / n;
  uint4* dxr = reinterpret_cast<uint4*>(dx + static_cast<size_t>(row) * n);
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int vi = lane + i * 32;
    if (vi < nvec) {
      float xv[8], dv[8], o[8];
      unpack8(__ldg(xr + vi), xv);
      unpack8(__ldg(dr + vi), dv);
      const float4 g0 = __ldg(gv + vi * 2), g1 = __ldg(gv + vi * 2 + 1);
      const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = rs * (dv[j] * g[j] - s1 - (xv[j] - mu) * rs * s2);
      dxr[vi] = pack8(o);
    }
  }
}

// dx of two normalisations of the same x plus a residual gradient, in one pass:
//   dx = LNbwd(dy1; gamma1) + LNbwd(dy2; gamma2) + res
// (x + f(LN1(x)) + g(LN2(x)): the three gradient streams that meet at x).  One warp per row.
template <int MAXV>
__global__ void __launch_bounds__(256) layernorm_bwd_dx2_kernel(const __nv_bfloat16* __restrict__ dy1, const __nv_bfloat16* __restrict__ dy2,
                                                                const __nv_bfloat16* __restrict__ res, const __nv_bfloat16* __restrict__ x,
                                                                const float* __restrict__ gamma1, const float* __restrict__ gamma2,
                                                                const float* __restrict__ mean, const float* __restrict__ rstd, int rows, int n,
                                                                __nv_bfloat16* __restrict__ dx) {
  // Two passes over the row, the second re-reading it (from L1 / L2: the same warp has just touched those lines) instead of
  // keeping three operands of the row in registers: 243 registers allowed one 8-warp CTA per SM and the kernel ran at a third
  // of the memory bandwidth; at ~64 registers four CTAs are resident and their phases overlap.
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int nvec = n >> 3;
  const size_t off = static_cast<size_t>(row) * n;
  const uint4* xr = reinterpret_cast<const uint4*>(x + off);
  const uint4* d1 = reinterpret_cast<const uint4*>(dy1 + off);
  const uint4* d2 = reinterpret_cast<const uint4*>(dy2 + off);
  const float4* g1v = reinterpret_cast<const float4*>(gamma1);
  const float4* g2v = reinterpret_cast<const float4*>(gamma2);
  const float mu = mean[row], rs = rstd[row];
  float a1 = 0.f, a2 = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int vi = lane + i * 32;
    if (vi < nvec) {
      float xv[8], u[8], w[8];
      unpack8(__ldg(xr + vi), xv);
      unpack8(__ldg(d1 + vi), u);
      unpack8(__ldg(d2 + vi), w);
      const float4 g0 = __ldg(g1v + vi * 2), g1 = __ldg(g1v + vi * 2 + 1), h0 = __ldg(g2v + vi * 2), h1 = __ldg(g2v + vi * 2 + 1);
      const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
      const float h[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        // the two backward formulas are linear in (sum, sum * xhat): the moments of both branches add
        const float t = fmaf(u[j], g[j], w[j] * h[j]);
        a1 += t;
        a2 = fmaf(t, (xv[j] - mu) * rs, a2);
      }
    }
  }
  const float s1 = warp_sum(a1) / n;
  const float s2 = warp_sum(a2) / n;
  uint4* dxr = reinterpret_cast<uint4*>(dx + off);
  const uint4* rr = res ? reinterpret_cast<const uint4*>(res + off) : nullptr;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int vi = lane + i * 32;
    if (vi < nvec) {
      float xv[8], u[8], w[8], o[8], r[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      unpack8(__ldg(xr + vi), xv);
      unpack8(__ldg(d1 + vi), u);
      unpack8(__ldg(d2 + vi), w);
      if (rr) unpack8(__ldg(rr + vi), r);
      const float4 g0 = __ldg(g1v + vi * 2), g1 = __ldg(g1v + vi * 2 + 1), h0 = __ldg(g2v + vi * 2), h1 = __ldg(g2v + vi * 2 + 1);
      const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
      const float h[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = fmaf(rs, fmaf(u[j], g[j], w[j] * h[j]) - s1 - (xv[j] - mu) * rs * s2, r[j]);
      dxr[vi] = pack8(o);
    }
  }
}

// out = a + b + c on contiguous bf16 (numel % 8 == 0): the residual sum of a parallel block in one pass.
__global__ void __launch_bounds__(256) add3_kernel(const uint4* __restrict__ a, const uint4* __restrict__ b, const uint4* __restrict__ c,
                                                   uint4* __restrict__ out, size_t nvec) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < nvec; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    float x[8], y[8], z[8];
    unpack8(__ldg(a + i), x);
    unpack8(__ldg(b + i), y);
    unpack8(__ldg(c + i), z);
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] = x[j] + y[j] + z[j];
    out[i] = pack8(x);
  }
}

// dgamma[c] = sum_rows dy * xhat, dbeta[c] = sum_rows dy.  CTA = 64 columns x a slab of rows; 8 column
// threads x 32 row lanes; lanes reduce through shared memory, one atomic per column per CTA.
__global__ void __launch_bounds__(256) layernorm_bwd_params_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                                                   const float* __restrict__ mean, const float* __restrict__ rstd,
                                                                   int rows, int n, int slab, float* __restrict__ dgamma,
                                                                   float* __restrict__ dbeta) {
  __shared__ float s_g[32][65], s_b[32][65];
  const int tx = threadIdx.x & 7, ty = threadIdx.x >> 3;
  const int col = blockIdx.x * 64 + tx * 8;
  const int r0 = blockIdx.y * slab, r1 = min(rows, r0 + slab);
  float ag[8] = {0, 0, 0, 0, 0, 0, 0, 0}, ab[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (col < n) {
    for (int row = r0 + ty; row < r1; row += 32) {
      float xv[8], dv[8];
      unpack8(__ldg(reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * n + col)), xv);
      unpack8(__ldg(reinterpret_cast<const uint4*>(dy + static_cast<size_t>(row) * n + col)), dv);
      const float mu = mean[row], rs = rstd[row];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        ag[j] = fmaf(dv[j], (xv[j] - mu) * rs, ag[j]);
        ab[j] += dv[j];
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    s_g[ty][tx * 8 + j] = ag[j];
    s_b[ty][tx * 8 + j] = ab[j];
  }
  __syncthreads();
  if (threadIdx.x < 64 && blockIdx.x * 64 + threadIdx.x < n) {
    float g = 0.f, b = 0.f;
#pragma unroll
    for (int r = 0; r < 32; ++r) {
      g += s_g[r][threadIdx.x];
      b += s_b[r][threadIdx.x];
    }
    atomicAdd(dgamma + blockIdx.x * 64 + threadIdx.x, g);
    atomicAdd(dbeta + blockIdx.x * 64 + threadIdx.x, b);
  }
}

// ---------------------------------------------------------------------------- GELU
// The exact (erf) form is evaluated through the normal tail Phi(-|x|) = 0.5 * P(t) * exp(-x^2 / 2), t = 1 / (1 + p |x| / sqrt 2),
// with the five-term rational fit of Abramowitz & Stegun 7.1.26 (absolute error 1.5e-7, far below bf16 resolution; the
// tail is formed without cancellation, so large negative inputs keep their relative accuracy).  The exponential is the
// one the derivative needs for the density, so forward costs one ex2 and one reciprocal and backward no more than that:
// with the library erff the two kernels were bound by instruction issue, not by memory.
struct GeluParts { float cdf, e; };
__device__ __forceinline__ GeluParts gelu_parts(float x) {
  const float ax = fabsf(x);
  const float t = __frcp_rn(fmaf(0.3275911f * 0.70710678118654752f, ax, 1.f));
  const float poly = t * fmaf(t, fmaf(t, fmaf(t, fmaf(t, 1.061405429f, -1.453152027f), 1.421413741f), -0.284496736f), 0.254829592f);
  GeluParts g;
  g.e = __expf(-0.5f * x * x);
  const float tail = 0.5f * poly * g.e;
  g.cdf = x >= 0.f ? 1.f - tail : tail;
  return g;
}
__device__ __forceinline__ float gelu_f(float x, bool tanh_form) {
  if (tanh_form) {
    const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    return 0.5f * x * (1.f + tanhf(u));
  }
  return x * gelu_parts(x).cdf;
}
__device__ __forceinline__ float gelu_grad_f(float x, bool tanh_form) {
  if (tanh_form) {
    const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    const float t = tanhf(u);
    const float du = 0.7978845608028654f * (1.f + 3.f * 0.044715f * x * x);
    return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * du;
  }
  const GeluParts g = gelu_parts(x);
  return fmaf(x * 0.3989422804014327f, g.e, g.cdf);
}

constexpr int GELU_UNROLL = 4;  // independent 16-byte loads in flight per thread and operand

__global__ void __launch_bounds__(256) gelu_fwd_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, size_t nvec, int tanh_form) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x * GELU_UNROLL;
  for (size_t i0 = static_cast<size_t>(blockIdx.x) * blockDim.x * GELU_UNROLL + threadIdx.x; i0 < nvec; i0 += stride) {
    uint4 raw[GELU_UNROLL];
#pragma unroll
    for (int u = 0; u < GELU_UNROLL; ++u) {
      const size_t i = i0 + static_cast<size_t>(u) * blockDim.x;
      if (i < nvec) raw[u] = __ldg(x + i);
    }
#pragma unroll
    for (int u = 0; u < GELU_UNROLL; ++u) {
      const size_t i = i0 + static_cast<size_t>(u) * blockDim.x;
      if (i < nvec) {
        float v[8];
        unpack8(raw[u], v);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = gelu_f(v[j], tanh_form);
        y[i] = pack8(v);
      }
    }
  }
}
__global__ void __launch_bounds__(256) gelu_bwd_kernel(const uint4* __restrict__ dy, const uint4* __restrict__ x, uint4* __restrict__ dx,
                                                       size_t nvec, int tanh_form) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x * GELU_UNROLL;
  for (size_t i0 = static_cast<size_t>(blockIdx.x) * blockDim.x * GELU_UNROLL + threadIdx.x; i0 < nvec; i0 += stride) {
    uint4 rx[GELU_UNROLL], rd[GELU_UNROLL];
#pragma unroll
    for (int u = 0; u < GELU_UNROLL; ++u) {
      const size_t i = i0 + static_cast<size_t>(u) * blockDim.x;
      if (i < nvec) {
        rx[u] = __ldg(x + i);
        rd[u] = __ldg(dy + i);
      }
    }
#pragma unroll
    for (int u = 0; u < GELU_UNROLL; ++u) {
      const size_t i = i0 + static_cast<size_t>(u) * blockDim.x;
      if (i < nvec) {
        float v[8], d[8];
        unpack8(rx[u], v);
        unpack8(rd[u], d);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = d[j] * gelu_grad_f(v[j], tanh_form);
        dx[i] = pack8(v);
      }
    }
  }
}

// The same derivative on a [rows, n] matrix (n % 8 == 0), which also leaves the column sums of the bf16 result in
// `colsum` (fp32, zeroed by the caller): the gradient of the bias of the linear layer that fed the activation, for which
// a separate pass over the freshly written matrix would otherwise be made.  A thread owns 8 consecutive columns over a
// slab of rows; its partial sums stay in registers and leave as 8 atomics per slab.
__global__ void __launch_bounds__(256) gelu_bwd_colsum_kernel(const uint4* __restrict__ dy, const uint4* __restrict__ x, uint4* __restrict__ dx,
                                                              int rows, int nvecs, int slab, int tanh_form, float* __restrict__ colsum) {
  const int cv = blockIdx.x * blockDim.x + threadIdx.x;
  if (cv >= nvecs) return;
  const int r0 = blockIdx.y * slab, r1 = min(rows, r0 + slab);
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  for (int row = r0; row < r1; row += GELU_UNROLL) {
    uint4 rx[GELU_UNROLL], rd[GELU_UNROLL];
#pragma unroll
    for (int u = 0; u < GELU_UNROLL; ++u) {
      if (row + u < r1) {
        const size_t i = static_cast<size_t>(row + u) * nvecs + cv;
        rx[u] = __ldg(x + i);
        rd[u] = __ldg(dy + i);
      }
    }
#pragma unroll
    for (int u = 0; u < GELU_UNROLL; ++u) {
      if (row + u < r1) {
        float v[8], d[8];
        unpack8(rx[u], v);
        unpack8(rd[u], d);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = d[j] * gelu_grad_f(v[j], tanh_form);
        const uint4 packed = pack8(v);
        dx[static_cast<size_t>(row + u) * nvecs + cv] = packed;
        float o[8];
        unpack8(packed, o);  // sum what was stored (the rounded values), as a later pass over the stored matrix would
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += o[j];
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) atomicAdd(colsum + static_cast<size_t>(cv) * 8 + j, acc[j]);
}

// ---------------------------------------------------------------------------- embedding
// out[t, :] = table[ids[t], :] as bf16, from a bf16 table (the optimizer's shadow copy) or an fp32 one; width % 8 == 0.
// Ids outside [0, vocab) produce a zero row and set *bad.
template <typename T>
__global__ void __launch_bounds__(256) embedding_fwd_kernel(const T* __restrict__ table, const long long* __restrict__ ids, long long tokens,
                                                            int width, int vocab, uint4* __restrict__ out, int* bad) {
  const int vecs = width >> 3;
  const long long total = tokens * vecs;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long tkn = i / vecs;
    const int v = static_cast<int>(i - tkn * vecs);
    const long long id = ids[tkn];
    if (id < 0 || id >= vocab) {
      if (v == 0) atomicAdd(bad, 1);
      out[i] = make_uint4(0u, 0u, 0u, 0u);
      continue;
    }
    if constexpr (sizeof(T) == 2) {
      out[i] = __ldg(reinterpret_cast<const uint4*>(table + id * width) + v);
    } else {
      const float4* src = reinterpret_cast<const float4*>(table + id * width) + 2 * v;
      const float4 a = __ldg(src), b = __ldg(src + 1);
      out[i] = make_uint4(pack_bf16x2(a.x, a.y), pack_bf16x2(a.z, a.w), pack_bf16x2(b.x, b.y), pack_bf16x2(b.z, b.w));
    }
  }
}

// grad_table[ids[t], :] += dy[t, :] (fp32 accumulation with atomics; the caller zeroes grad_table).  Rows of padding_idx
// and out-of-range ids receive nothing.
__global__ void __launch_bounds__(256) embedding_bwd_kernel(const uint4* __restrict__ dy, const long long* __restrict__ ids, long long tokens,
                                                            int width, int vocab, long long padding_idx, float* __restrict__ grad_table) {
  const int vecs = width >> 3;
  const long long total = tokens * vecs;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long tkn = i / vecs;
    const int v = static_cast<int>(i - tkn * vecs);
    const long long id = ids[tkn];
    if (id < 0 || id >= vocab || id == padding_idx) continue;
    float f[8];
    unpack8(__ldg(dy + i), f);
    float* dst = grad_table + id * width + v * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(dst + j, f[j]);
  }
}

// ---------------------------------------------------------------------------- cross-entropy
// One CTA per row.  Pass 1: running max and sum of exponentials (online softmax); pass 2 writes
// dlogits = (softmax - onehot) * inv_valid and the row loss.  Rows with target == -100 get zeros.
__global__ void __launch_bounds__(512) cross_entropy_kernel(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ target,
                                                            int v, const float* __restrict__ inv_valid, __nv_bfloat16* __restrict__ dlogits,
                                                            float* __restrict__ row_loss, float* __restrict__ row_lse) {
  __shared__ float s_m[16], s_s[16];
  __shared__ float s_max, s_lse;
  const int row = blockIdx.x;
  const long long tgt = target[row];
  const int nvec = v >> 3;
  const uint4* lr = reinterpret_cast<const uint4*>(logits + static_cast<size_t>(row) * v);
  uint4* dr = reinterpret_cast<uint4*>(dlogits + static_cast<size_t>(row) * v);
  if (tgt < 0) {  // ignored row
    if (dlogits != nullptr)
      for (int i = threadIdx.x; i < nvec; i += blockDim.x) dr[i] = make_uint4(0, 0, 0, 0);
    if (threadIdx.x == 0) {
      row_loss[row] = 0.f;
      if (row_lse) row_lse[row] = 0.f;
    }
    return;
  }
  float m = -INFINITY, s = 0.f;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    float f[8];
    unpack8(__ldg(lr + i), f);
    float lm = f[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
    const float nm = fmaxf(m, lm);
    float add = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) add += __expf(f[j] - nm);
    s = s * __expf(m - nm) + add;
    m = nm;
  }
  const float wm = warp_max(m);
  s = warp_sum(m == -INFINITY ? 0.f : s * __expf(m - wm));  // a thread that saw no element has m = -inf: exp(-inf + inf) would be NaN
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    s_m[warp] = wm;
    s_s[warp] = s;
  }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    float mm = lane < nw ? s_m[lane] : -INFINITY;
    float ss = lane < nw ? s_s[lane] : 0.f;
    const float gm = warp_max(mm);
    ss = warp_sum(mm == -INFINITY ? 0.f : ss * __expf(mm - gm));
    if (lane == 0) {
      s_max = gm;
      s_lse = gm + __logf(ss);
    }
  }
  __syncthreads();
  const float lse = s_lse;
  if (dlogits == nullptr) {  // loss only: the gradient is produced by cross_entropy_bwd_kernel when (and if) it is asked for
    if (threadIdx.x == 0) {
      row_loss[row] = lse - __bfloat162float(logits[static_cast<size_t>(row) * v + tgt]);
      if (row_lse) row_lse[row] = lse;
    }
    return;
  }
  const float scale = *inv_valid;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    float f[8];
    unpack8(__ldg(lr + i), f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float p = __expf(f[j] - lse);
      if (i * 8 + j == tgt) {
        row_loss[row] = lse - f[j];
        p -= 1.f;
      }
      f[j] = p * scale;
    }
    dr[i] = pack8(f);
  }
}

// dlogits = (softmax(logits) - onehot(target)) * inv_valid * dloss from the saved row log-sum-exp: one read of the logits
// and one write, with the upstream scalar gradient folded in (no separate scaling pass over a [rows, vocab] tensor).
__global__ void __launch_bounds__(512) cross_entropy_bwd_kernel(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ target,
                                                                int v, const float* __restrict__ row_lse, const float* __restrict__ inv_valid,
                                                                const float* __restrict__ dloss, __nv_bfloat16* __restrict__ dlogits) {
  const int row = blockIdx.x;
  const long long tgt = target[row];
  const int nvec = v >> 3;
  const uint4* lr = reinterpret_cast<const uint4*>(logits + static_cast<size_t>(row) * v);
  uint4* dr = reinterpret_cast<uint4*>(dlogits + static_cast<size_t>(row) * v);
  if (tgt < 0) {
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) dr[i] = make_uint4(0, 0, 0, 0);
    return;
  }
  const float lse = row_lse[row];
  const float scale = *inv_valid * *dloss;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    float f[8];
    unpack8(__ldg(lr + i), f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float p = __expf(f[j] - lse);
      if (i * 8 + j == tgt) p -= 1.f;
      f[j] = p * scale;
    }
    dr[i] = pack8(f);
  }
}

// ---------------------------------------------------------------------------- rotary embedding
// In-place NeoX-style rotation of the first `rot` dims of the q and k parts of a fused qkv tensor
// [tokens, heads, 3 * head_dim] (token t is at position t % seq).  out1 = x1 cos - s x2 sin,
// out2 = x2 cos + s x1 sin with s = +1 (forward) or -1 (backward: the transpose of a rotation).
// One thread rotates 8 pairs (two 16-byte vectors).
__global__ void __launch_bounds__(256) rotary_qk_kernel(__nv_bfloat16* __restrict__ qkv, const float* __restrict__ cos_t,
                                                        const float* __restrict__ sin_t, long long tokens, int seq, int heads,
                                                        int head_dim, int rot, float sign) {
  const int half = rot >> 1;
  const int groups = half >> 3;  // 8-pair groups per (token, head, q|k)
  const long long total = tokens * heads * 2 * groups;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int g = static_cast<int>(i % groups);
    long long rest = i / groups;
    const int which = static_cast<int>(rest % 2);
    rest /= 2;
    const int head = static_cast<int>(rest % heads);
    const long long tok = rest / heads;
    const int pos = static_cast<int>(tok % seq);
    __nv_bfloat16* base = qkv + (tok * heads + head) * 3 * static_cast<long long>(head_dim) + which * head_dim + g * 8;
    float a[8], b[8];
    unpack8(*reinterpret_cast<const uint4*>(base), a);
    unpack8(*reinterpret_cast<const uint4*>(base + half), b);
    const float* cr = cos_t + static_cast<size_t>(pos) * half + g * 8;
    const float* sr = sin_t + static_cast<size_t>(pos) * half + g * 8;
    float o1[8], o2[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float c = __ldg(cr + j), sn = sign * __ldg(sr + j);
      o1[j] = a[j] * c - b[j] * sn;
      o2[j] = b[j] * c + a[j] * sn;
    }
    *reinterpret_cast<uint4*>(base) = pack8(o1);
    *reinterpret_cast<uint4*>(base + half) = pack8(o2);
  }
}

// ---------------------------------------------------------------------------- cast
__global__ void __launch_bounds__(256) cast_f32_bf16_kernel(const float4* __restrict__ src, uint2* __restrict__ dst, size_t nvec4) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < nvec4; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const float4 v = __ldg(src + i);
    dst[i] = make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
  }
}

template <int MAXV>
static int ln_fwd_launch(const void* x, const float* g, const float* b, int rows, int n, float eps, void* y, float* mean, float* rstd,
                         cudaStream_t st) {
  const int wpb = 8;
  layernorm_fwd_kernel<MAXV><<<(rows + wpb - 1) / wpb, wpb * 32, 0, st>>>(static_cast<const __nv_bfloat16*>(x), g, b, rows, n, eps,
                                                                          static_cast<__nv_bfloat16*>(y), mean, rstd);
  return static_cast<int>(cudaGetLastError());
}
template <int MAXV>
static int ln_fwd2_launch(const void* x, const float* g1, const float* b1, const float* g2, const float* b2, int rows, int n, float eps, void* y1,
                          void* y2, float* mean, float* rstd, cudaStream_t st) {
  const int wpb = 8;
  layernorm_fwd_kernel<MAXV><<<(rows + wpb - 1) / wpb, wpb * 32, 0, st>>>(static_cast<const __nv_bfloat16*>(x), g1, b1, rows, n, eps,
                                                                          static_cast<__nv_bfloat16*>(y1), mean, rstd, g2, b2,
                                                                          static_cast<__nv_bfloat16*>(y2));
  return static_cast<int>(cudaGetLastError());
}
static void ln_params_launch(const void* dy, const void* x, const float* mean, const float* rstd, int rows, int n, float* dg, float* db, int sms,
                             cudaStream_t st);
template <int MAXV>
static int ln_bwd2_launch(const void* dy1, const void* dy2, const void* res, const void* x, const float* g1, const float* g2, const float* mean,
                          const float* rstd, int rows, int n, void* dx, float* dg1, float* db1, float* dg2, float* db2, int sms, cudaStream_t st) {
  const int wpb = 8;
  layernorm_bwd_dx2_kernel<MAXV><<<(rows + wpb - 1) / wpb, wpb * 32, 0, st>>>(
      static_cast<const __nv_bfloat16*>(dy1), static_cast<const __nv_bfloat16*>(dy2), static_cast<const __nv_bfloat16*>(res),
      static_cast<const __nv_bfloat16*>(x), g1, g2, mean, rstd, rows, n, static_cast<__nv_bfloat16*>(dx));
  ln_params_launch(dy1, x, mean, rstd, rows, n, dg1, db1, sms, st);
  ln_params_launch(dy2, x, mean, rstd, rows, n, dg2, db2, sms, st);
  return static_cast<int>(cudaGetLastError());
}
template <int MAXV>
static int ln_bwd_launch(const void* dy, const void* x, const float* g, const float* mean, const float* rstd, int rows, int n, void* dx,
                         float* dg, float* db, int sms, cudaStream_t st) {
  const int wpb = 8;
  layernorm_bwd_dx_kernel<MAXV><<<(rows + wpb - 1) / wpb, wpb * 32, 0, st>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x), g, mean, rstd, rows, n, static_cast<__nv_bfloat16*>(dx));
  ln_params_launch(dy, x, mean, rstd, rows, n, dg, db, sms, st);
  return static_cast<int>(cudaGetLastError());
}
static void ln_params_launch(const void* dy, const void* x, const float* mean, const float* rstd, int rows, int n, float* dg, float* db, int sms,
                             cudaStream_t st) {
  const int colblocks = (n + 63) / 64;
  int slabs = (sms * 4 + colblocks - 1) / colblocks;
  if (slabs < 1) slabs = 1;
  int slab = (rows + slabs - 1) / slabs;
  if (slab < 32) slab = 32;
  dim3 grid(colblocks, (rows + slab - 1) / slab);
  layernorm_bwd_params_kernel<<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x), mean, rstd,
                                                    rows, n, slab, dg, db);
}

}  // namespace sb

// y = LayerNorm(x) * gamma + beta for bf16 x [rows, n] (n % 8 == 0, n <= 4096); gamma/beta fp32.
extern "C" int sb_layernorm_fwd(const void* x, const float* gamma, const float* beta, int rows, int n, float eps, void* y,
                                float* mean, float* rstd, void* stream) {
  using namespace sb;
  if (rows <= 0) return 0;
  if (n % 8 || n > 4096) return -2;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int nv = (n / 8 + 31) / 32;
  if (nv <= 4) return ln_fwd_launch<4>(x, gamma, beta, rows, n, eps, y, mean, rstd, st);
  if (nv <= 8) return ln_fwd_launch<8>(x, gamma, beta, rows, n, eps, y, mean, rstd, st);
  if (nv <= 16) return ln_fwd_launch<16>(x, gamma, beta, rows, n, eps, y, mean, rstd, st);
  return -3;
}

// dx bf16; dgamma/dbeta fp32 [n], zeroed by the caller.
extern "C" int sb_layernorm_bwd(const void* dy, const void* x, const float* gamma, const float* mean, const float* rstd, int rows,
                                int n, void* dx, float* dgamma, float* dbeta, int sms, void* stream) {
  using namespace sb;
  if (rows <= 0) return 0;
  if (n % 8 || n > 4096) return -2;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int nv = (n / 8 + 31) / 32;
  if (nv <= 4) return ln_bwd_launch<4>(dy, x, gamma, mean, rstd, rows, n, dx, dgamma, dbeta, sms, st);
  if (nv <= 8) return ln_bwd_launch<8>(dy, x, gamma, mean, rstd, rows, n, dx, dgamma, dbeta, sms, st);
  if (nv <= 16) return ln_bwd_launch<16>(dy, x, gamma, mean, rstd, rows, n, dx, dgamma, dbeta, sms, st);
  return -3;
}

// Two affine outputs of one normalisation (see layernorm_fwd_kernel).
extern "C" int sb_layernorm_fwd2(const void* x, const float* gamma1, const float* beta1, const float* gamma2, const float* beta2, int rows, int n,
                                 float eps, void* y1, void* y2, float* mean, float* rstd, void* stream) {
  using namespace sb;
  if (rows <= 0) return 0;
  if (n % 8 || n > 4096) return -2;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int nv = (n / 8 + 31) / 32;
  if (nv <= 4) return ln_fwd2_launch<4>(x, gamma1, beta1, gamma2, beta2, rows, n, eps, y1, y2, mean, rstd, st);
  if (nv <= 8) return ln_fwd2_launch<8>(x, gamma1, beta1, gamma2, beta2, rows, n, eps, y1, y2, mean, rstd, st);
  if (nv <= 16) return ln_fwd2_launch<16>(x, gamma1, beta1, gamma2, beta2, rows, n, eps, y1, y2, mean, rstd, st);
  return -3;
}

// dx = LNbwd(dy1) + LNbwd(dy2) + res (res may be null); the four parameter gradients are fp32 [n], zeroed by the caller.
extern "C" int sb_layernorm_bwd2(const void* dy1, const void* dy2, const void* res, const void* x, const float* gamma1, const float* gamma2,
                                 const float* mean, const float* rstd, int rows, int n, void* dx, float* dgamma1, float* dbeta1, float* dgamma2,
                                 float* dbeta2, int sms, void* stream) {
  using namespace sb;
  if (rows <= 0) return 0;
  if (n % 8 || n > 4096) return -2;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int nv = (n / 8 + 31) / 32;
  if (nv <= 4) return ln_bwd2_launch<4>(dy1, dy2, res, x, gamma1, gamma2, mean, rstd, rows, n, dx, dgamma1, dbeta1, dgamma2, dbeta2, sms, st);
  if (nv <= 8) return ln_bwd2_launch<8>(dy1, dy2, res, x, gamma1, gamma2, mean, rstd, rows, n, dx, dgamma1, dbeta1, dgamma2, dbeta2, sms, st);
  return -3;
}

extern "C" int sb_add3(const void* a, const void* b, const void* c, void* out, long long numel, int sms, void* stream) {
  if (numel <= 0) return 0;
  if (numel % 8) return -2;
  const size_t nvec = static_cast<size_t>(numel / 8);
  size_t blocks = (nvec + 255) / 256;
  if (blocks > static_cast<size_t>(sms) * 16) blocks = static_cast<size_t>(sms) * 16;
  sb::add3_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(a), static_cast<const uint4*>(b), static_cast<const uint4*>(c), static_cast<uint4*>(out), nvec);
  return static_cast<int>(cudaGetLastError());
}

static inline unsigned gelu_blocks(size_t nvec, int sms) {
  size_t blocks = (nvec + 256 * sb::GELU_UNROLL - 1) / (256 * sb::GELU_UNROLL);
  if (blocks > static_cast<size_t>(sms) * 8) blocks = static_cast<size_t>(sms) * 8;
  return static_cast<unsigned>(blocks < 1 ? 1 : blocks);
}

extern "C" int sb_gelu_fwd(const void* x, void* y, long long numel, int tanh_form, int sms, void* stream) {
  if (numel <= 0) return 0;
  if (numel % 8) return -2;
  const size_t nvec = static_cast<size_t>(numel / 8);
  sb::gelu_fwd_kernel<<<gelu_blocks(nvec, sms), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(x), static_cast<uint4*>(y), nvec, tanh_form);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int sb_gelu_bwd(const void* dy, const void* x, void* dx, long long numel, int tanh_form, int sms, void* stream) {
  if (numel <= 0) return 0;
  if (numel % 8) return -2;
  const size_t nvec = static_cast<size_t>(numel / 8);
  sb::gelu_bwd_kernel<<<gelu_blocks(nvec, sms), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(dy), static_cast<const uint4*>(x), static_cast<uint4*>(dx), nvec, tanh_form);
  return static_cast<int>(cudaGetLastError());
}

// dx = dy * gelu'(x) on contiguous bf16 [rows, n] (n % 8 == 0) and colsum[n] += column sums of dx (fp32; the caller zeroes it).
extern "C" int sb_gelu_bwd_colsum(const void* dy, const void* x, void* dx, int rows, int n, int tanh_form, float* colsum, int sms,
                                  void* stream) {
  if (rows <= 0 || n <= 0) return 0;
  if (n % 8) return -2;
  const int nvecs = n / 8;
  const int col_blocks = (nvecs + 255) / 256;
  int slabs = (sms * 8 + col_blocks - 1) / col_blocks;
  if (slabs > (rows + 7) / 8) slabs = (rows + 7) / 8;   // at least 8 rows per slab: 8 atomics pay for 64 elements or more
  if (slabs < 1) slabs = 1;
  if (slabs > 65535) slabs = 65535;
  const int slab = (rows + slabs - 1) / slabs;
  dim3 grid(col_blocks, (rows + slab - 1) / slab);
  sb::gelu_bwd_colsum_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(dy), static_cast<const uint4*>(x), static_cast<uint4*>(dx), rows, nvecs, slab, tanh_form, colsum);
  return static_cast<int>(cudaGetLastError());
}

// Row losses and dlogits for bf16 logits [rows, v] (v % 8 == 0); inv_valid = 1 / (#targets != -100) on the device.
// dlogits == NULL: losses (and, when row_lse != NULL, the row log-sum-exp for sb_cross_entropy_bwd) only.
extern "C" int sb_cross_entropy(const void* logits, const long long* target, int rows, int v, const float* inv_valid, void* dlogits,
                                float* row_loss, float* row_lse, void* stream) {
  if (rows <= 0) return 0;
  if (v % 8) return -2;
  sb::cross_entropy_kernel<<<rows, 512, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(logits), target, v, inv_valid, static_cast<__nv_bfloat16*>(dlogits), row_loss, row_lse);
  return static_cast<int>(cudaGetLastError());
}

// dlogits (may alias logits) = (softmax - onehot) * inv_valid * dloss; inv_valid and dloss are device scalars.
extern "C" int sb_cross_entropy_bwd(const void* logits, const long long* target, int rows, int v, const float* row_lse, const float* inv_valid,
                                    const float* dloss, void* dlogits, void* stream) {
  if (rows <= 0) return 0;
  if (v % 8) return -2;
  sb::cross_entropy_bwd_kernel<<<rows, 512, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(logits), target, v, row_lse, inv_valid, dloss, static_cast<__nv_bfloat16*>(dlogits));
  return static_cast<int>(cudaGetLastError());
}

extern "C" int sb_cast_f32_bf16(const float* src, void* dst, long long numel, int sms, void* stream) {
  if (numel <= 0) return 0;
  if (numel % 4) return -2;
  const size_t nvec = static_cast<size_t>(numel / 4);
  size_t blocks = (nvec + 255) / 256;
  if (blocks > static_cast<size_t>(sms) * 16) blocks = static_cast<size_t>(sms) * 16;
  sb::cast_f32_bf16_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const float4*>(src), static_cast<uint2*>(dst), nvec);
  return static_cast<int>(cudaGetLastError());
}

// Row lookup into bf16 output; table_is_bf16 selects the table's element type.  width % 8 == 0.
extern "C" int sb_embedding_fwd(const void* table, int table_is_bf16, const long long* ids, long long tokens, int width, int vocab, void* out,
                                int* bad, int sms, void* stream) {
  if (tokens <= 0) return 0;
  if (width % 8) return -2;
  const long long total = tokens * (width / 8);
  long long blocks = (total + 255) / 256;
  if (blocks > static_cast<long long>(sms) * 16) blocks = static_cast<long long>(sms) * 16;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (table_is_bf16)
    sb::embedding_fwd_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(table), ids, tokens, width,
                                                                                          vocab, static_cast<uint4*>(out), bad);
  else
    sb::embedding_fwd_kernel<float><<<static_cast<unsigned>(blocks), 256, 0, st>>>(static_cast<const float*>(table), ids, tokens, width, vocab,
                                                                                  static_cast<uint4*>(out), bad);
  return static_cast<int>(cudaGetLastError());
}

// Scatter-add of bf16 output-gradient rows into an fp32 table gradient (zeroed by the caller).
extern "C" int sb_embedding_bwd(const void* dy, const long long* ids, long long tokens, int width, int vocab, long long padding_idx,
                                float* grad_table, int sms, void* stream) {
  if (tokens <= 0) return 0;
  if (width % 8) return -2;
  const long long total = tokens * (width / 8);
  long long blocks = (total + 255) / 256;
  if (blocks > static_cast<long long>(sms) * 16) blocks = static_cast<long long>(sms) * 16;
  sb::embedding_bwd_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(dy), ids, tokens, width, vocab, padding_idx, grad_table);
  return static_cast<int>(cudaGetLastError());
}

// In-place rotary embedding on the q and k parts of qkv [tokens, heads, 3*head_dim] bf16; rot % 16 == 0, head_dim % 8 == 0.
extern "C" int sb_rotary_qk(void* qkv, const float* cos_t, const float* sin_t, long long tokens, int seq, int heads, int head_dim,
                            int rot, float sign, int sms, void* stream) {
  if (tokens <= 0) return 0;
  if (rot % 16 || head_dim % 8 || rot > head_dim) return -2;
  const long long total = tokens * heads * 2 * (rot / 16);
  long long blocks = (total + 255) / 256;
  if (blocks > static_cast<long long>(sms) * 16) blocks = static_cast<long long>(sms) * 16;
  sb::rotary_qk_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(qkv), cos_t, sin_t, tokens, seq, heads, head_dim, rot, sign);
  return static_cast<int>(cudaGetLastError());
}
