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

// The same chain with its operands staged through shared memory: a block of four warps works on 32
// channels of one sequence.  All threads start the asynchronous copies of the next stage of RC_TOK
// tokens (16-byte pieces of the coefficients' and y's rows, as many in flight as there are), warp 0 runs
// the chain over the stage that has landed, and all store its outputs in 16-byte pieces: the chain never
// waits for global memory.  Arithmetic and order per channel are those of the kernel above (bitwise the
// same results).  Needs a width that is a multiple of 32 and 16-byte aligned rows.
constexpr int RC_CH = 32, RC_TOK = 64, RC_THREADS = 128;

__device__ __forceinline__ void rc_copy16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src)
               : "memory");
}

template <typename T>
constexpr size_t rc_smem_bytes() {
  return 2 * RC_TOK * RC_CH * (2 * sizeof(float) + 2 * sizeof(T));
}

template <typename T>
__global__ void __launch_bounds__(RC_THREADS)
rglru_chain_staged_kernel(const float* __restrict__ coef, const T* __restrict__ y, long y_stride, T* __restrict__ out,
                          long out_stride, float* __restrict__ state, long state_stride, long state_offset,
                          const int* __restrict__ seq_slot, const int* __restrict__ seq_start, int width) {
  extern __shared__ __align__(16) unsigned char rc_smem[];
  float(*as)[RC_TOK][RC_CH] = reinterpret_cast<float(*)[RC_TOK][RC_CH]>(rc_smem);
  float(*bs)[RC_TOK][RC_CH] = as + 2;
  T(*yr)[RC_TOK][RC_CH] = reinterpret_cast<T(*)[RC_TOK][RC_CH]>(bs + 2);
  T(*os)[RC_TOK][RC_CH] = yr + 2;
  constexpr int FP = RC_CH * sizeof(float) / 16;  // pieces of a row of coefficients
  constexpr int YP = RC_CH * sizeof(T) / 16;      // pieces of a row of y (and of the outputs)
  constexpr int YE = 16 / sizeof(T);
  const int s = blockIdx.y, c0 = blockIdx.x * RC_CH;
  const int slot = seq_slot[s];
  if (slot < 0) return;
  const int t0 = seq_start[s], t1 = seq_start[s + 1];
  if (t1 <= t0) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n_stages = (t1 - t0 + RC_TOK - 1) / RC_TOK;
  auto fetch = [&](int stage) {
    const int ts = t0 + stage * RC_TOK, nt = min(RC_TOK, t1 - ts), buf = stage & 1;
    for (int i = tid; i < nt * FP; i += RC_THREADS) {
      const int tt = i / FP, piece = i - tt * FP;
      const float* src = coef + (size_t)(ts + tt) * 2 * width + c0 + piece * 4;
      rc_copy16(&as[buf][tt][piece * 4], src);
      rc_copy16(&bs[buf][tt][piece * 4], src + width);
    }
    for (int i = tid; i < nt * YP; i += RC_THREADS) {
      const int tt = i / YP, piece = i - tt * YP;
      rc_copy16(&yr[buf][tt][piece * YE], y + (size_t)(ts + tt) * y_stride + c0 + piece * YE);
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };
  float* sp = state + (size_t)slot * state_stride + state_offset + c0 + lane;
  float S = warp == 0 ? *sp : 0.f;
  fetch(0);
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");
  __syncthreads();
  for (int stage = 0; stage < n_stages; ++stage) {
    const int ts = t0 + stage * RC_TOK, nt = min(RC_TOK, t1 - ts), buf = stage & 1;
    if (stage + 1 < n_stages) fetch(stage + 1);
    if (warp == 0) {
#pragma unroll 8
      for (int tt = 0; tt < nt; ++tt) {
        S = fmaf(as[buf][tt][lane], S, bs[buf][tt][lane]);
        os[buf][tt][lane] = from_f32<T>(S * to_f32<T>(yr[buf][tt][lane]));
      }
    }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();
    // (this stage's outputs leave while the next stage is walked: they have a buffer of their own)
    for (int i = tid; i < nt * YP; i += RC_THREADS) {
      const int tt = i / YP, piece = i - tt * YP;
      *reinterpret_cast<uint4*>(out + (size_t)(ts + tt) * out_stride + c0 + piece * YE) =
          *reinterpret_cast<const uint4*>(&os[buf][tt][piece * YE]);
    }
  }
  if (warp == 0) *sp = S;
}

template <typename T>
int launch_chain(const float* coef, const T* y, long y_stride, T* out, long out_stride, float* state, long state_stride,
                 long state_offset, const int* seq_slot, const int* seq_start, int n_tokens, int n_seqs, int width,
                 cudaStream_t stream) {
  constexpr int YE = 16 / (int)sizeof(T);
  const bool staged = width % RC_CH == 0 && y_stride % YE == 0 && out_stride % YE == 0 && ((uintptr_t)y & 15) == 0 &&
                      ((uintptr_t)out & 15) == 0 && ((uintptr_t)coef & 15) == 0;
  if (n_tokens <= 2 * n_seqs || !staged) {
    // a token or two a sequence: nothing to stage (and rows that cannot be copied in 16-byte pieces)
    const dim3 cgrid((width + 127) / 128, n_seqs);
    rglru_chain_kernel<T><<<cgrid, 128, 0, stream>>>(coef, y, y_stride, out, out_stride, state, state_stride, state_offset,
                                                     seq_slot, seq_start, width);
  } else {
    constexpr size_t smem = rc_smem_bytes<T>();
    static bool attr_set = false;
    if (!attr_set) {
      cudaError_t e = cudaFuncSetAttribute(rglru_chain_staged_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      FG_CHECK_ARG(e == cudaSuccess, "fg_rglru_scan: shared memory: %s", cudaGetErrorString(e));
      attr_set = true;
    }
    const dim3 cgrid((width + RC_CH - 1) / RC_CH, n_seqs);
    rglru_chain_staged_kernel<T><<<cgrid, RC_THREADS, smem, stream>>>(coef, y, y_stride, out, out_stride, state, state_stride,
                                                                      state_offset, seq_slot, seq_start, width);
  }
  FG_CHECK_LAUNCH("fg_rglru_scan");
  return 0;
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
  if (dtype == FG_F32)
    return launch_chain(coef, (const float*)y, y_stride, (float*)out, out_stride, state, state_stride, state_offset, seq_slot,
                        seq_start, n_tokens, n_seqs, width, stream);
  if (dtype == FG_BF16)
    return launch_chain(coef, (const __nv_bfloat16*)y, y_stride, (__nv_bfloat16*)out, out_stride, state, state_stride,
                        state_offset, seq_slot, seq_start, n_tokens, n_seqs, width, stream);
  FG_CHECK_ARG(false, "fg_rglru_scan: bad dtype %d", dtype);
  return 0;
}
