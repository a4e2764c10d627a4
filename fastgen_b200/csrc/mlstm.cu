// The matrix memory with exponential gates (the mLSTM of xLSTM), token by token in float32.
//
// Per head, with q (already times dim^-1/2), k of `d` numbers and v of `dv`, a log input gate i and a
// log forget gate f, and a running maximum m that starts at ZERO (not at minus infinity):
//
//   i = cap * tanh((i_raw + b_i) / cap);   f = logsigmoid(cap * tanh((f_raw + b_f) / cap))
//   m' = max(f + m, i);   S <- exp(f + m - m') S + exp(i - m') k v^T;   n likewise with k alone
//   o = S^T q / (max(|n . q|, exp(-m')) + 1e-6)
//
// n is kept as one more column of S (the column of a value that is always 1), so the recurrence is
// one kernel over dv + 1 columns and the division happens where the output is normed.
//
// A request's state is one float32 row per slot: [heads][dv + 1][d] (a column's rows side by side, as
// the threads hold them; column dv is n), then [heads] running maxima.  It is zero at admission.  A
// step may bring a sequence any number of tokens; sequences are consecutive runs of tokens with one
// slot (seq_slot < 0: padding that touches nothing).
//
// Three kernels: the gates of every token side by side (nothing here depends on the state), the chain
// of running maxima (an addition and a maximum a token), and the recurrence itself, which runs token
// by token so that its sums do not depend on how a prompt was cut or on what else is in the batch.
// A fourth divides, norms per head and gates the read-out.
#include "common.cuh"

namespace {

__device__ __forceinline__ float log_sigmoid(float z) {
  // -softplus(-z), exact at both ends
  return z < -30.f ? z : -log1pf(expf(-z));
}

// ---- gates ------------------------------------------------------------------------------------------
// gates: float32 [T, 2 heads] raw sums (input gates, then forget gates), replaced in place by the
// capped log gates i and f.
__global__ void mlstm_gates_kernel(float* __restrict__ gates, const float* __restrict__ bias,
                                   const int* __restrict__ req, int n_tokens, int heads, float cap) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long)n_tokens * 2 * heads) return;
  const int t = (int)(idx / (2 * heads)), j = (int)(idx % (2 * heads));
  if (req[t] < 0) return;
  const float z = cap * tanhf((gates[idx] + bias[j]) / cap);
  gates[idx] = j < heads ? z : log_sigmoid(z);
}

// ---- the chain of running maxima ------------------------------------------------------------------
// A thread a (sequence, head).  coef[t, h] = (f + m - m', i - m', -m'): the logarithms of what the
// recurrence multiplies S by, multiplies k v^T by, and of the floor of the denominator.
__global__ void mlstm_maxima_kernel(const float* __restrict__ gates, float* __restrict__ coef,
                                    float* __restrict__ state, long state_stride, long m_offset,
                                    const int* __restrict__ seq_slot, const int* __restrict__ seq_start, int n_seqs,
                                    int heads) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_seqs * heads) return;
  const int s = idx / heads, h = idx % heads;
  const int slot = seq_slot[s];
  if (slot < 0) return;
  const int t0 = seq_start[s], t1 = seq_start[s + 1];
  float* mp = state + (size_t)slot * state_stride + m_offset + h;
  float m = *mp;
  constexpr int U = 8;
  for (int t = t0; t < t1; t += U) {
    float gi[U], gf[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int tt = min(t + u, t1 - 1);
      gi[u] = gates[(size_t)tt * 2 * heads + h];
      gf[u] = gates[(size_t)tt * 2 * heads + heads + h];
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (t + u >= t1) break;
      const float mn = fmaxf(gf[u] + m, gi[u]);
      float* c = coef + ((size_t)(t + u) * heads + h) * 3;
      c[0] = gf[u] + m - mn;
      c[1] = gi[u] - mn;
      c[2] = -mn;
      m = mn;
    }
  }
  *mp = m;
}

// ---- the recurrence ---------------------------------------------------------------------------------
// A block works on (sequence, head, MS_COLS columns of dv + 1); MS_LANES threads share a column, each
// with every MS_LANES-th row of the state in registers (NPT rows a thread; rows beyond d are zero and
// meet zero q and k).  Tokens are staged through shared memory 32 (large heads: 8) at a time.
constexpr int MS_COLS = 16;
constexpr int MS_LANES = 8;
constexpr int MS_THREADS = MS_COLS * MS_LANES;

template <typename T, int NPT>
__global__ void __launch_bounds__(MS_THREADS)
mlstm_scan_kernel(const T* __restrict__ q, long q_stride, const T* __restrict__ k, long k_stride,
                  const T* __restrict__ v, long v_stride, const float* __restrict__ coef, float* __restrict__ y,
                  long y_stride, float* __restrict__ state, long state_stride, const int* __restrict__ seq_slot,
                  const int* __restrict__ seq_start, int heads, int d, int dv, float q_scale) {
  constexpr int DP = NPT * MS_LANES;  // padded rows
  constexpr int MS_TOKENS = NPT > 16 ? 8 : 32;  // tokens a stage: the stage's q and k fit 32 KiB
  __shared__ float qs[MS_TOKENS][DP];
  __shared__ float ks[MS_TOKENS][DP];
  __shared__ float vs[MS_TOKENS][MS_COLS];  // value times exp(i - m')
  __shared__ float keep[MS_TOKENS];
  __shared__ float ys[MS_TOKENS][MS_COLS];
  const int s = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * MS_COLS;
  const int slot = seq_slot[s];
  if (slot < 0) return;
  const int t0 = seq_start[s], t1 = seq_start[s + 1];
  if (t1 <= t0) return;
  const int tid = threadIdx.x, lane = tid % MS_LANES, cl = tid / MS_LANES;
  const int col = c0 + cl;
  const bool live = col <= dv;  // column dv is n
  float* sp = state + (size_t)slot * state_stride + ((size_t)h * (dv + 1) + min(col, dv)) * d;
  float S[NPT];
#pragma unroll
  for (int i = 0; i < NPT; ++i) {
    const int r = lane + MS_LANES * i;
    S[i] = (live && r < d) ? sp[r] : 0.f;
  }
  for (int ts = t0; ts < t1; ts += MS_TOKENS) {
    const int nt = min(MS_TOKENS, t1 - ts);
    __syncthreads();  // the stage before has been read
    for (int i = tid; i < nt * DP; i += MS_THREADS) {
      const int tt = i / DP, r = i - tt * DP;
      float qv = 0.f, kv = 0.f;
      if (r < d) {
        qv = to_f32<T>(q[(size_t)(ts + tt) * q_stride + (size_t)h * d + r]) * q_scale;
        kv = to_f32<T>(k[(size_t)(ts + tt) * k_stride + (size_t)h * d + r]);
      }
      qs[tt][r] = qv;
      ks[tt][r] = kv;
    }
    for (int i = tid; i < nt * MS_COLS; i += MS_THREADS) {
      const int tt = i / MS_COLS, c = c0 + (i - tt * MS_COLS);
      const float w = expf(coef[((size_t)(ts + tt) * heads + h) * 3 + 1]);
      float vv = 0.f;
      if (c < dv) vv = to_f32<T>(v[(size_t)(ts + tt) * v_stride + (size_t)h * dv + c]) * w;
      else if (c == dv) vv = w;
      vs[tt][i - tt * MS_COLS] = vv;
    }
    for (int i = tid; i < nt; i += MS_THREADS) keep[i] = expf(coef[((size_t)(ts + i) * heads + h) * 3]);
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float kp = keep[tt], vv = vs[tt][cl];
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < NPT; ++i) {
        S[i] = fmaf(kp, S[i], ks[tt][lane + MS_LANES * i] * vv);
        acc = fmaf(S[i], qs[tt][lane + MS_LANES * i], acc);
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      acc += __shfl_xor_sync(0xffffffffu, acc, 4);
      if (lane == 0) ys[tt][cl] = acc;
    }
    __syncthreads();
    for (int i = tid; i < nt * MS_COLS; i += MS_THREADS) {
      const int tt = i / MS_COLS, c = c0 + (i - tt * MS_COLS);
      if (c <= dv) y[(size_t)(ts + tt) * y_stride + (size_t)h * (dv + 1) + c] = ys[tt][i - tt * MS_COLS];
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
      const int r = lane + MS_LANES * i;
      if (r < d) sp[r] = S[i];
    }
  }
}

// ---- division, norm per head, gate ------------------------------------------------------------------
// y: float32 [T, heads * (dv + 1)] (a head's dv sums, then n . q).  out[t, h, :] = o / rms(o) * w[h, :] *
// sigmoid(z[t, h, :]) with o = y / (max(|n . q|, exp(coef[t, h, 2])) + 1e-6).  A warp a (token, head).
template <typename T>
__global__ void __launch_bounds__(128)
mlstm_out_kernel(const float* __restrict__ y, long y_stride, const float* __restrict__ coef, const T* __restrict__ z,
                 long z_stride, const float* __restrict__ w, T* __restrict__ out, long out_stride,
                 const int* __restrict__ req, int n_tokens, int heads, int dv, float eps) {
  const long item = (long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (item >= (long)n_tokens * heads) return;
  const int t = (int)(item / heads), h = (int)(item % heads), lane = threadIdx.x & 31;
  if (req[t] < 0) return;
  const float* row = y + (size_t)t * y_stride + (size_t)h * (dv + 1);
  const float den = fmaxf(fabsf(row[dv]), expf(coef[((size_t)t * heads + h) * 3 + 2])) + 1e-6f;
  float ss = 0.f;
  for (int j = lane; j < dv; j += 32) {
    const float o = row[j] / den;
    ss = fmaf(o, o, ss);
  }
  ss = warp_sum(ss);
  const float rstd = 1.f / sqrtf(ss / (float)dv + eps);
  for (int j = lane; j < dv; j += 32) {
    const float o = row[j] / den;
    const float g = to_f32<T>(z[(size_t)t * z_stride + (size_t)h * dv + j]);
    out[(size_t)t * out_stride + (size_t)h * dv + j] = from_f32<T>(o * rstd * w[(size_t)h * dv + j] / (1.f + expf(-g)));
  }
}

template <typename T>
int launch_scan(const T* q, long qs, const T* k, long ks, const T* v, long vs, const float* coef, float* y, long ys,
                float* state, long ss, const int* seq_slot, const int* seq_start, int n_seqs, int heads, int d, int dv,
                float q_scale, cudaStream_t stream) {
  const dim3 grid((dv + 1 + MS_COLS - 1) / MS_COLS, heads, n_seqs);
#define FG_MS(NPT)                                                                                                  \
  mlstm_scan_kernel<T, NPT><<<grid, MS_THREADS, 0, stream>>>(q, qs, k, ks, v, vs, coef, y, ys, state, ss, seq_slot, \
                                                             seq_start, heads, d, dv, q_scale)
  if (d <= 32) FG_MS(4);
  else if (d <= 64) FG_MS(8);
  else if (d <= 128) FG_MS(16);
  else FG_MS(32);
#undef FG_MS
  FG_CHECK_LAUNCH("fg_mlstm_scan");
  return 0;
}

}  // namespace

extern "C" long long fg_mlstm_state_floats(int heads, int d, int dv) { return (long long)heads * (dv + 1) * d + heads; }

// gates: float32 [T, 2 heads] raw sums, overwritten with the log gates.  q, k, v: row-strided views of the
// compute type.  coef: float32 scratch [T, heads, 3].  y: float32 [T, heads * (dv + 1)].
extern "C" int fg_mlstm_scan(float* gates, const float* gate_bias, float cap, const void* q, long q_stride, const void* k,
                             long k_stride, const void* v, long v_stride, int dtype, float* coef, float* y,
                             long y_stride, float* state, long state_stride, const int* req, const int* seq_slot,
                             const int* seq_start, int n_tokens, int n_seqs, int heads, int d, int dv, float q_scale,
                             cudaStream_t stream) {
  if (n_tokens == 0 || n_seqs == 0) return 0;
  FG_CHECK_ARG(heads > 0 && d > 0 && d <= 256 && dv > 0 && cap > 0.f, "fg_mlstm_scan: %d heads of %d x %d", heads, d, dv);
  FG_CHECK_ARG(n_seqs <= 65535 && heads <= 65535, "fg_mlstm_scan: too many sequences or heads");
  const long n = (long)n_tokens * 2 * heads;
  mlstm_gates_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(gates, gate_bias, req, n_tokens, heads, cap);
  FG_CHECK_LAUNCH("fg_mlstm_scan (gates)");
  const long m_offset = (long)heads * (dv + 1) * d;
  mlstm_maxima_kernel<<<(n_seqs * heads + 63) / 64, 64, 0, stream>>>(gates, coef, state, state_stride, m_offset,
                                                                      seq_slot, seq_start, n_seqs, heads);
  FG_CHECK_LAUNCH("fg_mlstm_scan (maxima)");
  if (dtype == FG_F32)
    return launch_scan((const float*)q, q_stride, (const float*)k, k_stride, (const float*)v, v_stride, coef, y,
                       y_stride, state, state_stride, seq_slot, seq_start, n_seqs, heads, d, dv, q_scale, stream);
  if (dtype == FG_BF16)
    return launch_scan((const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k, k_stride, (const __nv_bfloat16*)v,
                       v_stride, coef, y, y_stride, state, state_stride, seq_slot, seq_start, n_seqs, heads, d, dv,
                       q_scale, stream);
  FG_CHECK_ARG(false, "fg_mlstm_scan: bad dtype %d", dtype);
  return 0;
}

extern "C" int fg_mlstm_out(const float* y, long y_stride, const float* coef, const void* z, long z_stride, int dtype,
                            const float* w, void* out, long out_stride, const int* req, int n_tokens, int heads, int dv,
                            float eps, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  const long items = (long)n_tokens * heads;
  const unsigned grid = (unsigned)((items + 3) / 4);
  if (dtype == FG_F32)
    mlstm_out_kernel<float><<<grid, 128, 0, stream>>>(y, y_stride, coef, (const float*)z, z_stride, w, (float*)out,
                                                      out_stride, req, n_tokens, heads, dv, eps);
  else if (dtype == FG_BF16)
    mlstm_out_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>(y, y_stride, coef, (const __nv_bfloat16*)z, z_stride, w,
                                                              (__nv_bfloat16*)out, out_stride, req, n_tokens, heads, dv,
                                                              eps);
  else
    FG_CHECK_ARG(false, "fg_mlstm_out: bad dtype %d", dtype);
  FG_CHECK_LAUNCH("fg_mlstm_out");
  return 0;
}
