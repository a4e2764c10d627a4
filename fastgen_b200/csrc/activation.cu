// Elementwise pieces around the products:
//  * fg_bias_act: x[t, f] = act(x[t, f] + bias[f]) in place, for a dense feed-forward
//    down(act(up x)); act is the exact (erf) GELU, the tanh GELU
//    0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))), the squared ReLU max(z, 0)^2, or nothing (bias only).  Float32
//    arithmetic, one rounding.
//  * fg_scale_softcap: logits[r, v] = cap * tanh(logits[r, v] * scale / cap) in place (float32);
//    cap <= 0 leaves the scaling alone.
#include "common.cuh"

namespace {

enum { ACT_NONE = 0, ACT_GELU_ERF = 1, ACT_GELU_TANH = 2, ACT_RELU2 = 3 };

__device__ __forceinline__ float activate(float z, int act) {
  if (act == ACT_GELU_ERF) return 0.5f * z * (1.f + erff(z * 0.70710678118654752440f));
  if (act == ACT_GELU_TANH) return 0.5f * z * (1.f + tanhf(0.79788456080286535588f * (z + 0.044715f * z * z * z)));
  if (act == ACT_RELU2) return z > 0.f ? z * z : 0.f;
  return z;
}

template <typename T>
__global__ void bias_act_kernel(T* x, const T* __restrict__ bias, int width, size_t total, int act) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    float v = to_f32<T>(x[i]);
    if (bias != nullptr) v = to_f32<T>(from_f32<T>(v + to_f32<T>(bias[i % width])));
    x[i] = from_f32<T>(activate(v, act));
  }
}

// bfloat16 rows whose width is a multiple of 8, no bias: eight elements (16 bytes) a thread
__global__ void __launch_bounds__(256) act_bf16x8_kernel(uint4* x, size_t pieces, int act) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < pieces; i += stride) {
    uint4 raw = x[i];
    __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 v = __bfloat1622float2(h2[k]);
      h2[k] = __floats2bfloat162_rn(activate(v.x, act), activate(v.y, act));
    }
    x[i] = raw;
  }
}

__global__ void scale_softcap_kernel(float* x, size_t total, float scale, float cap) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    float v = x[i] * scale;
    if (cap > 0.f) v = cap * tanhf(v / cap);
    x[i] = v;
  }
}

int grid_for(size_t items, int threads) {
  size_t blocks = (items + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  return (int)blocks;
}

}  // namespace

extern "C" int fg_bias_act(void* x, const void* bias, int dtype, int n_rows, int width, int act, cudaStream_t stream) {
  const size_t total = (size_t)n_rows * width;
  if (total == 0) return 0;
  FG_CHECK_ARG(act >= ACT_NONE && act <= ACT_RELU2, "fg_bias_act: unknown activation %d", act);
  const int threads = 256;
  if (dtype == FG_BF16 && bias == nullptr && total % 8 == 0 && ((uintptr_t)x & 15) == 0)
    act_bf16x8_kernel<<<grid_for(total / 8, threads), threads, 0, stream>>>((uint4*)x, total / 8, act);
  else if (dtype == FG_BF16)
    bias_act_kernel<__nv_bfloat16><<<grid_for(total, threads), threads, 0, stream>>>(
        (__nv_bfloat16*)x, (const __nv_bfloat16*)bias, width, total, act);
  else if (dtype == FG_F32)
    bias_act_kernel<float><<<grid_for(total, threads), threads, 0, stream>>>((float*)x, (const float*)bias, width,
                                                                            total, act);
  else
    FG_CHECK_ARG(false, "fg_bias_act: bad dtype %d", dtype);
  FG_CHECK_LAUNCH("fg_bias_act");
  return 0;
}

extern "C" int fg_scale_softcap(float* x, int n_rows, int width, float scale, float cap, cudaStream_t stream) {
  const size_t total = (size_t)n_rows * width;
  if (total == 0) return 0;
  scale_softcap_kernel<<<grid_for(total, 256), 256, 0, stream>>>(x, total, scale, cap);
  FG_CHECK_LAUNCH("fg_scale_softcap");
  return 0;
}

// x[t, h, :] *= sigmoid(gate[t, h]) in place: a head's output multiplied by a gate of its own (one
// number a token and head), float32 arithmetic, one rounding.  x: [T, heads * head_dim] with a row
// stride; gate: a row-strided view [T, heads] of the same type.  Tokens of slot < 0 are padding.
template <typename T>
__global__ void __launch_bounds__(256)
head_gate_kernel(T* x, long x_stride, const T* __restrict__ gate, long gate_stride, const int* __restrict__ req,
                 int heads, int head_dim) {
  const int t = blockIdx.x;
  if (req != nullptr && req[t] < 0) return;
  const int width = heads * head_dim;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float g = to_f32<T>(gate[(size_t)t * gate_stride + i / head_dim]);
    T* p = x + (size_t)t * x_stride + i;
    *p = from_f32<T>(to_f32<T>(*p) * (1.f / (1.f + expf(-g))));
  }
}

// The same in 16-byte pieces of bfloat16: a thread a piece (eight columns of one head), one gate a piece.
__global__ void __launch_bounds__(256)
head_gate_bf16x8_kernel(__nv_bfloat16* x, long x_stride, const __nv_bfloat16* __restrict__ gate, long gate_stride,
                        const int* __restrict__ req, int n_tokens, int heads, int head_dim) {
  const int pieces = heads * head_dim / 8;  // a row's
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long)n_tokens * pieces) return;
  const int t = (int)(idx / pieces), piece = (int)(idx - (long)t * pieces);
  if (req != nullptr && req[t] < 0) return;
  const float g = __bfloat162float(gate[(size_t)t * gate_stride + piece * 8 / head_dim]);
  const float s = 1.f / (1.f + expf(-g));
  uint4* p = reinterpret_cast<uint4*>(x + (size_t)t * x_stride + piece * 8);
  uint4 raw = *p;
  __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __bfloat1622float2(h2[i]);
    h2[i] = __floats2bfloat162_rn(v.x * s, v.y * s);
  }
  *p = raw;
}

extern "C" int fg_head_gate(void* x, long x_stride, const void* gate, long gate_stride, int dtype, const int* req,
                            int n_tokens, int heads, int head_dim, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  if (dtype == FG_BF16 && head_dim % 8 == 0 && x_stride % 8 == 0 && ((uintptr_t)x & 15) == 0) {
    const long n = (long)n_tokens * heads * head_dim / 8;
    head_gate_bf16x8_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(
        (__nv_bfloat16*)x, x_stride, (const __nv_bfloat16*)gate, gate_stride, req, n_tokens, heads, head_dim);
    FG_CHECK_LAUNCH("fg_head_gate");
    return 0;
  }
  if (dtype == FG_F32)
    head_gate_kernel<float><<<n_tokens, 256, 0, stream>>>((float*)x, x_stride, (const float*)gate, gate_stride, req,
                                                          heads, head_dim);
  else if (dtype == FG_BF16)
    head_gate_kernel<__nv_bfloat16><<<n_tokens, 256, 0, stream>>>((__nv_bfloat16*)x, x_stride,
                                                                  (const __nv_bfloat16*)gate, gate_stride, req, heads,
                                                                  head_dim);
  else
    FG_CHECK_ARG(false, "fg_head_gate: bad dtype %d", dtype);
  FG_CHECK_LAUNCH("fg_head_gate");
  return 0;
}
