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
};

struct ChunkDesc {
  int tensor;
  int pad;
  long long offset;
};

constexpr int CHUNK = 2048;

struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay, bias1, bias2, grad_scale;
};

__global__ void __launch_bounds__(256) adamw_fp32_kernel(const TensorDesc* __restrict__ tensors, const ChunkDesc* __restrict__ chunks,
                                                         AdamArgs a) {
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

__device__ __forceinline__ float decode_m(unsigned char c, float amax) {
  const float s = (static_cast<float>(c) - 128.f) * (1.f / 127.f);
  return copysignf(s * s, s) * amax;
}
__device__ __forceinline__ unsigned char encode_m(float m, float amax) {
  if (amax <= 0.f) return 128;
  const float s = sqrtf(fminf(fabsf(m) / amax, 1.f));
  return static_cast<unsigned char>(128.f + rintf(copysignf(s, m) * 127.f));
}
__device__ __forceinline__ float decode_v(unsigned char c, float amax) {
  const float s = static_cast<float>(c) * (1.f / 255.f);
  return s * s * s * s * amax;
}
__device__ __forceinline__ unsigned char encode_v(float v, float amax) {
  if (amax <= 0.f) return 0;
  return static_cast<unsigned char>(rintf(sqrtf(sqrtf(fminf(v / amax, 1.f))) * 255.f));
}

// One CTA (256 threads) = one 256-element quantisation block; CHUNK/256 blocks per chunk.
__global__ void __launch_bounds__(256) adamw_8bit_kernel(const TensorDesc* __restrict__ tensors, const ChunkDesc* __restrict__ chunks,
                                                         AdamArgs a) {
  __shared__ float red_m[8], red_v[8];
  const ChunkDesc c = chunks[blockIdx.x / (CHUNK / 256)];
  const TensorDesc t = tensors[c.tensor];
  const long long base = c.offset + static_cast<long long>(blockIdx.x % (CHUNK / 256)) * 256;
  if (base >= t.numel) return;
  const long long i = base + threadIdx.x;
  const bool ok = i < t.numel;
  const long long qb = base / 256;
  float m = 0.f, v = 0.f, p = 0.f;
  if (ok) {
    const float g = t.grad[i] * a.grad_scale;
    p = t.param[i];
    if (t.m8) {
      m = decode_m(t.m8[i], t.m_absmax[qb]);
      v = decode_v(t.v8[i], t.v_absmax[qb]);
    } else {
      m = t.m[i];
      v = t.v[i];
    }
    m = a.beta1 * m + (1.f - a.beta1) * g;
    v = a.beta2 * v + (1.f - a.beta2) * g * g;
    p -= a.lr * a.weight_decay * p;
    p -= a.lr * (m / a.bias1) / (sqrtf(v / a.bias2) + a.eps);
    t.param[i] = p;
    if (t.shadow) t.shadow[i] = __float2bfloat16_rn(p);
  }
  if (!t.m8) {
    if (ok) {
      t.m[i] = m;
      t.v[i] = v;
    }
    return;
  }
  float am = fabsf(m), av = v;
  for (int off = 16; off; off >>= 1) {
    am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, off));
    av = fmaxf(av, __shfl_xor_sync(0xffffffffu, av, off));
  }
  if ((threadIdx.x & 31) == 0) {
    red_m[threadIdx.x >> 5] = am;
    red_v[threadIdx.x >> 5] = av;
  }
  __syncthreads();
  am = red_m[0];
  av = red_v[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) {
    am = fmaxf(am, red_m[w]);
    av = fmaxf(av, red_v[w]);
  }
  if (ok) {
    t.m8[i] = encode_m(m, am);
    t.v8[i] = encode_v(v, av);
  }
  if (threadIdx.x == 0) {
    t.m_absmax[qb] = am;
    t.v_absmax[qb] = av;
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
                             float eps, float weight_decay, float bias1, float bias2, float grad_scale, void* stream) {
  using namespace sb;
  if (n_chunks <= 0) return 0;
  AdamArgs a{lr, beta1, beta2, eps, weight_decay, bias1, bias2, grad_scale};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (eight_bit)
    adamw_8bit_kernel<<<n_chunks * (CHUNK / 256), 256, 0, st>>>(static_cast<const TensorDesc*>(tensors), static_cast<const ChunkDesc*>(chunks), a);
  else
    adamw_fp32_kernel<<<n_chunks, 256, 0, st>>>(static_cast<const TensorDesc*>(tensors), static_cast<const ChunkDesc*>(chunks), a);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int sb_grad_sqnorm(const void* tensors, const void* chunks, int n_chunks, float* out, void* stream) {
  using namespace sb;
  if (n_chunks <= 0) return 0;
  grad_sqnorm_kernel<<<n_chunks, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const TensorDesc*>(tensors),
                                                                              static_cast<const ChunkDesc*>(chunks), out);
  return static_cast<int>(cudaGetLastError());
}
