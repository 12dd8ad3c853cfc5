// Optimizer steps as single multi-tensor launches.
//
// A step descriptor table lives on the device: one entry per 2048-element chunk naming the
// tensor and the chunk's offset, so one launch covers every parameter regardless of how many
// tensors there are.  Two kernels:
//   * AdamW with fp32 moments (decoupled weight decay, bias correction), optionally writing a
//     bf16 shadow copy of the updated weight for the next forward;
//   * AdamW with 8-bit block-wise moments: 256-element blocks, one fp32 absmax per block and
//     moment, power-law companded codes (signed square-root code for the first moment,
//     unsigned fourth-root code for the second), so small magnitudes keep relative precision.
// The 8-bit layout follows the block-wise design of the optimizer the reference obtains from an
// external library (stacr/protocols/baselines/bnb_optimizer.py:61-176 there; tensors smaller
// than 4096 elements keep fp32 state).
#include "common.cuh"

namespace sb {

struct TensorDesc {
  float* param;
  const float* grad;
  float* m;
  float* v;
  __nv_bfloat16* shadow;  // optional bf16 copy of param
  unsigned char* m8;      // 8-bit states (8-bit kernel only)
  unsigned char* v8;
  float* m_absmax;
  float* v_absmax;
  long long numel;
  // NVSwitch multicast address of the bf16 copy (0 = none).  When set, the updated weight is stored through it, so the
  // store itself delivers the value to every rank's copy: a rank that updates only its shard of the parameters leaves
  // all ranks' bf16 weights current without a separate all-gather.  Requires 16-byte aligned full vectors.
  unsigned long long shadow_mc;
};

__device__ __forceinline__ void store_shadow(const TensorDesc& t, long long i0, const float (&p)[8]) {
  const uint4 w = make_uint4(pack_bf16x2(p[0], p[1]), pack_bf16x2(p[2], p[3]), pack_bf16x2(p[4], p[5]), pack_bf16x2(p[6], p[7]));
  if (t.shadow_mc) {
    __nv_bfloat16* addr = reinterpret_cast<__nv_bfloat16*>(t.shadow_mc) + i0;
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(__uint_as_float(w.x)), "f"(__uint_as_float(w.y)),
                 "f"(__uint_as_float(w.z)), "f"(__uint_as_float(w.w))
                 : "memory");
  } else {
    *reinterpret_cast<uint4*>(t.shadow + i0) = w;
  }
}

struct ChunkDesc {
  int tensor;
  int pad;
  long long offset;
};

constexpr int CHUNK = 2048;

struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay, bias1, bias2, grad_scale;
};

// Hyper-parameters from device memory when the step is replayed from a CUDA graph: kernel arguments are frozen at capture
// time, the eight floats behind `hyper` are refreshed by a small copy in front of every replay.
__device__ __forceinline__ AdamArgs resolve_args(AdamArgs a, const float* hyper) {
  if (hyper) {
    a.lr = hyper[0]; a.beta1 = hyper[1]; a.beta2 = hyper[2]; a.eps = hyper[3];
    a.weight_decay = hyper[4]; a.bias1 = hyper[5]; a.bias2 = hyper[6]; a.grad_scale = hyper[7];
  }
  return a;
}

__global__ void __launch_bounds__(256) adamw_fp32_kernel(const TensorDesc* __restrict__ tensors, const ChunkDesc* __restrict__ chunks,
                                                         AdamArgs a0, const float* __restrict__ hyper) {
  const AdamArgs a = resolve_args(a0, hyper);
  const ChunkDesc c = chunks[blockIdx.x];
  const TensorDesc t = tensors[c.tensor];
  const long long end = min(t.numel, c.offset + CHUNK);
  for (long long i = c.offset + threadIdx.x; i < end; i += blockDim.x) {
    const float g = t.grad[i] * a.grad_scale;
    float p = t.param[i];
    const float m = a.beta1 * t.m[i] + (1.f - a.beta1) * g;
    const float v = a.beta2 * t.v[i] + (1.f - a.beta2) * g * g;
    t.m[i] = m;
    t.v[i] = v;
    p -= a.lr * a.weight_decay * p;
    p -= a.lr * (m / a.bias1) / (sqrtf(v / a.bias2) + a.eps);
    t.param[i] = p;
    if (t.shadow) t.shadow[i] = __float2bfloat16_rn(p);
  }
}

// 8-bit code <-> float through the mantissa: 0x4B0000cc is 2^23 + c exactly, and adding 1.5 * 2^23 to a value in [0, 2^22)
// rounds it to nearest-even into the low mantissa bits (what rintf + a conversion would give).
__device__ __forceinline__ float byte_to_float(unsigned char c) { return __uint_as_float(0x4B000000u | c) - 8388608.f; }
__device__ __forceinline__ unsigned char float_to_byte(float x) { return static_cast<unsigned char>(__float_as_uint(x + 12582912.f) & 0xFFu); }

// Code formats: m -> 128 + round(127 * sign(m) * sqrt(|m| / absmax)), v -> round(255 * (v / absmax)^(1/4)), one absmax pair per
// 256-element block.

// One warp = one 256-element quantisation block (8 consecutive elements per lane, 16-byte
// loads/stores, absmax by warp shuffles only); one CTA of 8 warps = one 2048-element chunk.
__global__ void __launch_bounds__(256, 4) adamw_8bit_kernel(const TensorDesc* __restrict__ tensors, const ChunkDesc* __restrict__ chunks,
                                                         AdamArgs a0, const float* __restrict__ hyper) {
  const AdamArgs a = resolve_args(a0, hyper);
  const ChunkDesc c = chunks[blockIdx.x];
  const TensorDesc t = tensors[c.tensor];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long base = c.offset + static_cast<long long>(warp) * 256;
  if (base >= t.numel) return;
  const long long i0 = base + lane * 8;
  const long long qb = base / 256;
  const bool vec = (i0 + 8 <= t.numel) && ((reinterpret_cast<uintptr_t>(t.param + i0) & 15) == 0) &&
                   ((reinterpret_cast<uintptr_t>(t.grad + i0) & 15) == 0);
  float p[8], g[8], m[8], v[8];
  unsigned char cm[8], cv[8];
  const bool q8 = t.m8 != nullptr;
  if (vec) {
    *reinterpret_cast<float4*>(p) = *reinterpret_cast<const float4*>(t.param + i0);
    *reinterpret_cast<float4*>(p + 4) = *reinterpret_cast<const float4*>(t.param + i0 + 4);
    *reinterpret_cast<float4*>(g) = __ldg(reinterpret_cast<const float4*>(t.grad + i0));
    *reinterpret_cast<float4*>(g + 4) = __ldg(reinterpret_cast<const float4*>(t.grad + i0 + 4));
    if (q8) {
      *reinterpret_cast<uint2*>(cm) = *reinterpret_cast<const uint2*>(t.m8 + i0);
      *reinterpret_cast<uint2*>(cv) = *reinterpret_cast<const uint2*>(t.v8 + i0);
    } else {
      *reinterpret_cast<float4*>(m) = *reinterpret_cast<const float4*>(t.m + i0);
      *reinterpret_cast<float4*>(m + 4) = *reinterpret_cast<const float4*>(t.m + i0 + 4);
      *reinterpret_cast<float4*>(v) = *reinterpret_cast<const float4*>(t.v + i0);
      *reinterpret_cast<float4*>(v + 4) = *reinterpret_cast<const float4*>(t.v + i0 + 4);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const bool ok = i0 + j < t.numel;
      p[j] = ok ? t.param[i0 + j] : 0.f;
      g[j] = ok ? t.grad[i0 + j] : 0.f;
      if (q8) {
        cm[j] = ok ? t.m8[i0 + j] : 128;
        cv[j] = ok ? t.v8[i0 + j] : 0;
      } else {
        m[j] = ok ? t.m[i0 + j] : 0.f;
        v[j] = ok ? t.v[i0 + j] : 0.f;
      }
    }
  }
  // The special-function pipe (conversions, roots, reciprocals: 16 per clock per SM) is as scarce here as DRAM bandwidth, so
  // the 8-bit path spends four of its operations per element instead of nine: codes become floats and back through the
  // mantissa (no int<->float conversion), sqrt(v) is shared by the update and the encoder, and the encoders' divisions by the
  // block maximum are one rsqrt per block.
  if (q8) {
    const float sm = t.m_absmax[qb] * (1.f / (127.f * 127.f)), sv = t.v_absmax[qb] * (1.f / (255.f * 255.f * 255.f * 255.f));
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float cf = byte_to_float(cm[j]) - 128.f;
      m[j] = cf * fabsf(cf) * sm;                       // sign(c) * (|c| / 127)^2 * absmax
      const float vf = byte_to_float(cv[j]);
      const float v2 = vf * vf;
      v[j] = v2 * v2 * sv;                              // (c / 255)^4 * absmax
    }
  }
  float am = 0.f, rmax = 0.f, r[8];
  const float inv_b1 = 1.f / a.bias1, rs_b2 = rsqrtf(a.bias2), decay = 1.f - a.lr * a.weight_decay;
  const float step1 = a.lr * inv_b1;  // one reciprocal per element instead of three divisions
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float gj = g[j] * a.grad_scale;
    m[j] = a.beta1 * m[j] + (1.f - a.beta1) * gj;
    v[j] = a.beta2 * v[j] + (1.f - a.beta2) * gj * gj;
    r[j] = sqrtf(v[j]);
    p[j] = p[j] * decay - step1 * m[j] * __frcp_rn(fmaf(r[j], rs_b2, a.eps));
    if (i0 + j < t.numel) {
      am = fmaxf(am, fabsf(m[j]));
      rmax = fmaxf(rmax, r[j]);
    }
  }
  if (q8) {
#pragma unroll
    for (int off = 16; off; off >>= 1) {
      am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, off));
      rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, off));
    }
    const float rs_am = am > 0.f ? rsqrtf(am) * 127.f : 0.f, rs_r = rmax > 0.f ? rsqrtf(rmax) * 255.f : 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      cm[j] = float_to_byte(128.f + copysignf(fminf(sqrtf(fabsf(m[j])) * rs_am, 127.f), m[j]));   // sqrt(|m| / absmax)
      cv[j] = float_to_byte(fminf(sqrtf(r[j]) * rs_r, 255.f));                                    // (v / absmax)^(1/4)
    }
    if (lane == 0) {
      t.m_absmax[qb] = am;
      t.v_absmax[qb] = rmax * rmax;
    }
  }
  if (vec) {
    *reinterpret_cast<float4*>(t.param + i0) = *reinterpret_cast<const float4*>(p);
    *reinterpret_cast<float4*>(t.param + i0 + 4) = *reinterpret_cast<const float4*>(p + 4);
    if (t.shadow) store_shadow(t, i0, p);
    if (q8) {
      *reinterpret_cast<uint2*>(t.m8 + i0) = *reinterpret_cast<const uint2*>(cm);
      *reinterpret_cast<uint2*>(t.v8 + i0) = *reinterpret_cast<const uint2*>(cv);
    } else {
      *reinterpret_cast<float4*>(t.m + i0) = *reinterpret_cast<const float4*>(m);
      *reinterpret_cast<float4*>(t.m + i0 + 4) = *reinterpret_cast<const float4*>(m + 4);
      *reinterpret_cast<float4*>(t.v + i0) = *reinterpret_cast<const float4*>(v);
      *reinterpret_cast<float4*>(t.v + i0 + 4) = *reinterpret_cast<const float4*>(v + 4);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (i0 + j >= t.numel) continue;
      t.param[i0 + j] = p[j];
      if (t.shadow) t.shadow[i0 + j] = __float2bfloat16_rn(p[j]);
      if (q8) {
        t.m8[i0 + j] = cm[j];
        t.v8[i0 + j] = cv[j];
      } else {
        t.m[i0 + j] = m[j];
        t.v[i0 + j] = v[j];
      }
    }
  }
}

// sum of squares of every gradient (for clipping): one partial per chunk block, atomically added.
__global__ void __launch_bounds__(256) grad_sqnorm_kernel(const TensorDesc* __restrict__ tensors, const ChunkDesc* __restrict__ chunks,
                                                          float* __restrict__ out) {
  __shared__ float red[8];
  const ChunkDesc c = chunks[blockIdx.x];
  const TensorDesc t = tensors[c.tensor];
  const long long end = min(t.numel, c.offset + CHUNK);
  float s = 0.f;
  for (long long i = c.offset + threadIdx.x; i < end; i += blockDim.x) {
    const float g = t.grad[i];
    s = fmaf(g, g, s);
  }
  for (int off = 16; off; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float total = 0.f;
    for (int w = 0; w < 8; ++w) total += red[w];
    atomicAdd(out, total);
  }
}

}  // namespace sb

extern "C" int sb_tensor_desc_size() { return static_cast<int>(sizeof(sb::TensorDesc)); }
extern "C" int sb_chunk_desc_size() { return static_cast<int>(sizeof(sb::ChunkDesc)); }
extern "C" int sb_optim_chunk() { return sb::CHUNK; }

extern "C" int sb_adamw_step(const void* tensors, const void* chunks, int n_chunks, int eight_bit, float lr, float beta1, float beta2,
                             float eps, float weight_decay, float bias1, float bias2, float grad_scale, const float* hyper, void* stream) {
  using namespace sb;
  if (n_chunks <= 0) return 0;
  AdamArgs a{lr, beta1, beta2, eps, weight_decay, bias1, bias2, grad_scale};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (eight_bit)
    adamw_8bit_kernel<<<n_chunks, 256, 0, st>>>(static_cast<const TensorDesc*>(tensors), static_cast<const ChunkDesc*>(chunks), a, hyper);
  else
    adamw_fp32_kernel<<<n_chunks, 256, 0, st>>>(static_cast<const TensorDesc*>(tensors), static_cast<const ChunkDesc*>(chunks), a, hyper);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int sb_grad_sqnorm(const void* tensors, const void* chunks, int n_chunks, float* out, void* stream) {
  using namespace sb;
  if (n_chunks <= 0) return 0;
  grad_sqnorm_kernel<<<n_chunks, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const TensorDesc*>(tensors),
                                                                              static_cast<const ChunkDesc*>(chunks), out);
  return static_cast<int>(cudaGetLastError());
}
