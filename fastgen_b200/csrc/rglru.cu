// The real-gated linear recurrent unit (the recurrence of Griffin's recurrent block) in float32.
//
// Per channel c, with u the convolved input branch, raw gate sums gr and gi (block-diagonal maps of u),
// their biases, and a learned lam:
//
//   r = sigmoid(gr + b_r);  i = sigmoid(gi + b_i);  a = exp(-decay * r * softplus(lam))   (decay = 8)
//   S <- a * S + sqrt(1 - a^2) * i * u          (from S = 0 also for a sequence's first token)
//   out = S * y                                  (y: the other branch, already activated)
//
// Two kernels.  The first computes a and the input term b = sqrt(1 - a^2) i u of every (token, channel)
// side by side: nothing there depends on the state.  The second is the chain S <- a S + b, a thread a
// (sequence, channel), token by token, so that a prompt cut anywhere gives the same sums in the same
// order; its loads are issued eight tokens ahead of the chain.  The state is one float32 per channel in
// the request's slot (zero at admission); seq_slot < 0 is padding that touches nothing.
#include "common.cuh"

namespace {

// gates: [blocks, T, 2 * bw] (a block's r sums, then its i sums), of type TG.  u: [T, width] of type TU.
// coef: float32 [T, 2, width] (a, then b).  neg_rate[c] = -decay * softplus(lam[c]).
template <typename TG, typename TU>
__global__ void __launch_bounds__(256)
rglru_coef_kernel(const TG* __restrict__ gates, const TU* __restrict__ u, long u_stride,
                  const float* __restrict__ bias_r, const float* __restrict__ bias_i,
                  const float* __restrict__ neg_rate, float* __restrict__ coef, const int* __restrict__ req,
                  int n_tokens, int width, int bw) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long)n_tokens * width) return;
  const int t = (int)(idx / width), c = (int)(idx % width);
  if (req[t] < 0) return;
  const int b = c / bw, j = c - b * bw;
  const TG* g = gates + ((size_t)b * n_tokens + t) * 2 * bw;
  const float r = 1.f / (1.f + expf(-(to_f32<TG>(g[j]) + bias_r[c])));
  const float i = 1.f / (1.f + expf(-(to_f32<TG>(g[bw + j]) + bias_i[c])));
  const float log_a = neg_rate[c] * r;
  const float a = expf(log_a);
  // 1 - a^2 = -expm1(2 log a): no cancellation where a is close to 1
  const float root = sqrtf(-expm1f(2.f * log_a));
  coef[(size_t)t * 2 * width + c] = a;
  coef[(size_t)t * 2 * width + width + c] = root * i * to_f32<TU>(u[(size_t)t * u_stride + c]);
}

template <typename T>
__global__ void __launch_bounds__(128)
rglru_chain_kernel(const float* __restrict__ coef, const T* __restrict__ y, long y_stride, T* __restrict__ out,
                   long out_stride, float* __restrict__ state, long state_stride, long state_offset,
                   const int* __restrict__ seq_slot, const int* __restrict__ seq_start, int width) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x, s = blockIdx.y;
  const int slot = seq_slot[s];
  if (c >= width || slot < 0) return;
  const int t0 = seq_start[s], t1 = seq_start[s + 1];
  float* sp = state + (size_t)slot * state_stride + state_offset + c;
  float S = *sp;
  constexpr int U = 8;
  for (int t = t0; t < t1; t += U) {
    float a[U], b[U], yy[U];
#pragma unroll
    for (int k = 0; k < U; ++k) {
      const int tt = min(t + k, t1 - 1);
      a[k] = coef[(size_t)tt * 2 * width + c];
      b[k] = coef[(size_t)tt * 2 * width + width + c];
      yy[k] = to_f32<T>(y[(size_t)tt * y_stride + c]);
    }
#pragma unroll
    for (int k = 0; k < U; ++k) {
      if (t + k >= t1) break;
      S = fmaf(a[k], S, b[k]);
      out[(size_t)(t + k) * out_stride + c] = from_f32<T>(S * yy[k]);
    }
  }
  *sp = S;
}

}  // namespace

// gates: [blocks, T, 2 bw] of gate_dtype; u: [T, width] of u_dtype (row stride u_stride); y and out of
// dtype; coef: float32 scratch [T, 2, width].
extern "C" int fg_rglru_scan(const void* gates, int gate_dtype, const void* u, long u_stride, int u_dtype,
                             const float* bias_r, const float* bias_i, const float* neg_rate, float* coef,
                             const void* y, long y_stride, void* out, long out_stride, int dtype, float* state,
                             long state_stride, long state_offset, const int* req, const int* seq_slot,
                             const int* seq_start, int n_tokens, int n_seqs, int width, int blocks,
                             cudaStream_t stream) {
  if (n_tokens == 0 || n_seqs == 0) return 0;
  FG_CHECK_ARG(width > 0 && blocks > 0 && width % blocks == 0, "fg_rglru_scan: %d channels in %d blocks", width, blocks);
  FG_CHECK_ARG(n_seqs <= 65535, "fg_rglru_scan: too many sequences");
  const int bw = width / blocks;
  const long n = (long)n_tokens * width;
  const unsigned grid = (unsigned)((n + 255) / 256);
#define FG_COEF(TG, TU)                                                                                             \
  rglru_coef_kernel<TG, TU><<<grid, 256, 0, stream>>>((const TG*)gates, (const TU*)u, u_stride, bias_r, bias_i, neg_rate, \
                                                      coef, req, n_tokens, width, bw)
  if (gate_dtype == FG_F32 && u_dtype == FG_F32) FG_COEF(float, float);
  else if (gate_dtype == FG_F32 && u_dtype == FG_BF16) FG_COEF(float, __nv_bfloat16);
  else if (gate_dtype == FG_BF16 && u_dtype == FG_F32) FG_COEF(__nv_bfloat16, float);
  else if (gate_dtype == FG_BF16 && u_dtype == FG_BF16) FG_COEF(__nv_bfloat16, __nv_bfloat16);
  else FG_CHECK_ARG(false, "fg_rglru_scan: bad dtypes %d, %d", gate_dtype, u_dtype);
#undef FG_COEF
  FG_CHECK_LAUNCH("fg_rglru_scan (coefficients)");
  const dim3 cgrid((width + 127) / 128, n_seqs);
  if (dtype == FG_F32)
    rglru_chain_kernel<float><<<cgrid, 128, 0, stream>>>(coef, (const float*)y, y_stride, (float*)out, out_stride, state,
                                                         state_stride, state_offset, seq_slot, seq_start, width);
  else if (dtype == FG_BF16)
    rglru_chain_kernel<__nv_bfloat16><<<cgrid, 128, 0, stream>>>(coef, (const __nv_bfloat16*)y, y_stride,
                                                                 (__nv_bfloat16*)out, out_stride, state, state_stride,
                                                                 state_offset, seq_slot, seq_start, width);
  else
    FG_CHECK_ARG(false, "fg_rglru_scan: bad dtype %d", dtype);
  FG_CHECK_LAUNCH("fg_rglru_scan");
  return 0;
}
