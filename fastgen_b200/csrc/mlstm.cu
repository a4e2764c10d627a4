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
// of running maxima (an addition and a maximum a token, fed from shared memory), and the recurrence itself, which runs token
// by token so that its sums do not depend on how a prompt was cut or on what else is in the batch.
// A fourth divides, norms per head and gates the read-out.
#include "common.cuh"

namespace {

// The values of one 16-byte piece of a row.
template <typename T>
struct Piece;
template <>
struct Piece<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void unpack(const uint4& raw, float (&v)[4]) {
    v[0] = __uint_as_float(raw.x); v[1] = __uint_as_float(raw.y); v[2] = __uint_as_float(raw.z); v[3] = __uint_as_float(raw.w);
  }
};
template <>
struct Piece<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(const uint4& raw, float (&v)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
};

__device__ __forceinline__ float log_sigmoid(float z) {
  // -softplus(-z), exact at both ends
  return z < -30.f ? z : -log1pf(expf(-z));
}

// ---- gates ------------------------------------------------------------------------------------------
// gates: float32 [T, 2 heads] raw sums (input gates, then forget gates), replaced in place by the
// capped log gates i and f.
__device__ __forceinline__ float log_gate(float raw, float bias, float cap, bool forget) {
  const float z = cap * tanhf((raw + bias) / cap);
  return forget ? log_sigmoid(z) : z;
}

__global__ void mlstm_gates_kernel(float* __restrict__ gates, const float* __restrict__ bias,
                                   const int* __restrict__ req, int n_tokens, int heads, float cap) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long)n_tokens * 2 * heads) return;
  const int t = (int)(idx / (2 * heads)), j = (int)(idx % (2 * heads));
  if (req[t] < 0) return;
  gates[idx] = log_gate(gates[idx], bias[j], cap, j >= heads);
}

// ---- the chain of running maxima ------------------------------------------------------------------
// A block a sequence.  A stretch of tokens' gates comes into shared memory side by side (one contiguous
// run of global memory), thread h walks head h's chain over the stretch, and the stretch's coefficients
// leave side by side: the chain itself never waits for global memory.
// coef[t, h] = (f + m - m', i - m', -m'): the logarithms of what the recurrence multiplies S by, multiplies
// k v^T by, and of the floor of the denominator.
constexpr int MX_THREADS = 128;

__global__ void __launch_bounds__(MX_THREADS)
mlstm_maxima_kernel(const float* __restrict__ gates, float* __restrict__ coef, float* __restrict__ state,
                    long state_stride, long m_offset, const int* __restrict__ seq_slot,
                    const int* __restrict__ seq_start, int heads, int stretch, const float* __restrict__ raw_bias,
                    float cap) {
  // raw_bias: null, or the gates are still raw sums and become log gates on their way in (steps of a few
  // tokens, which then need no kernel of their own for that)
  extern __shared__ float mx_smem[];
  float* g = mx_smem;                        // [stretch][2 heads]
  float* c = g + (size_t)stretch * 2 * heads;  // [stretch][heads][3]
  const int s = blockIdx.x, tid = threadIdx.x;
  const int slot = seq_slot[s];
  if (slot < 0) return;
  const int t0 = seq_start[s], t1 = seq_start[s + 1];
  float* mp = state + (size_t)slot * state_stride + m_offset;
  // (more heads than threads: a thread walks several chains)
  for (int h0 = 0; h0 < heads; h0 += MX_THREADS) {
    const int h = h0 + tid;
    float m = h < heads ? mp[h] : 0.f;
    for (int ts = t0; ts < t1; ts += stretch) {
      const int nt = min(stretch, t1 - ts);
      __syncthreads();
      for (int i = tid; i < nt * 2 * heads; i += MX_THREADS) {
        float v = gates[(size_t)ts * 2 * heads + i];
        if (raw_bias != nullptr) {
          const int j = i % (2 * heads);
          v = log_gate(v, raw_bias[j], cap, j >= heads);
        }
        g[i] = v;
      }
      __syncthreads();
      if (h < heads) {
        // eight tokens' gates are read before their chain is walked: the chain is an addition and a
        // maximum a token and must not wait for shared memory
        constexpr int U = 8;
        for (int t8 = 0; t8 < nt; t8 += U) {
          float gi[U], gf[U];
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const int tt = min(t8 + u, nt - 1);
            gi[u] = g[tt * 2 * heads + h];
            gf[u] = g[tt * 2 * heads + heads + h];
          }
#pragma unroll
          for (int u = 0; u < U; ++u) {
            if (t8 + u < nt) {
              const float mn = fmaxf(gf[u] + m, gi[u]);
              float* o = c + ((size_t)(t8 + u) * heads + h) * 3;
              o[0] = gf[u] + m - mn;
              o[1] = gi[u] - mn;
              o[2] = -mn;
              m = mn;
            }
          }
        }
      }
      __syncthreads();
      if (h0 == 0 && heads <= MX_THREADS) {
        for (int i = tid; i < nt * 3 * heads; i += MX_THREADS) coef[(size_t)ts * 3 * heads + i] = c[i];
      } else {
        for (int i = tid; i < nt * 3 * heads; i += MX_THREADS) {
          const int hh = (i / 3) % heads;
          if (hh >= h0 && hh < h0 + MX_THREADS) coef[(size_t)ts * 3 * heads + i] = c[i];
        }
      }
    }
    if (h < heads) mp[h] = m;
  }
}

// ---- the recurrence ---------------------------------------------------------------------------------
// A block works on (sequence, head, MS_COLS columns of dv + 1); MS_LANES threads share a column, each
// with every MS_LANES-th row of the state in registers (NPT rows a thread; rows beyond d are zero and
// meet zero q and k).  Tokens are staged through shared memory in two buffers: while the block's four
// computing warps walk a stage, its two fetching warps bring the next one (q times its scale, k, the
// values times exp(i - m'), the decays exp(f + m - m')), so the chain does not wait for global memory.
constexpr int MS_COLS = 16;
constexpr int MS_LANES = 8;
constexpr int MS_COMPUTE = MS_COLS * MS_LANES;
constexpr int MS_FETCH = 64;
constexpr int MS_THREADS = MS_COMPUTE + MS_FETCH;

template <typename T, int NPT>
__global__ void __launch_bounds__(MS_THREADS)
mlstm_scan_kernel(const T* __restrict__ q, long q_stride, const T* __restrict__ k, long k_stride,
                  const T* __restrict__ v, long v_stride, const float* __restrict__ coef, float* __restrict__ y,
                  long y_stride, float* __restrict__ state, long state_stride, const int* __restrict__ seq_slot,
                  const int* __restrict__ seq_start, int heads, int d, int dv, float q_scale, bool vec) {
  // vec: the rows of q and k can be read in 16-byte pieces (the launch has checked sizes and alignment)
  constexpr int DP = NPT * MS_LANES;                        // padded rows
  constexpr int MS_TOKENS = DP >= 64 ? 2048 / DP : 32;      // tokens a stage: two stages of q and k fit 32 KiB
  __shared__ float qs[2][MS_TOKENS][DP];
  __shared__ float ks[2][MS_TOKENS][DP];
  __shared__ float vs[2][MS_TOKENS][MS_COLS];  // value times exp(i - m')
  __shared__ float keep[2][MS_TOKENS];
  __shared__ float ys[2][MS_TOKENS][MS_COLS];
  const int s = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * MS_COLS;
  const int slot = seq_slot[s];
  if (slot < 0) return;
  const int t0 = seq_start[s], t1 = seq_start[s + 1];
  if (t1 <= t0) return;
  const int tid = threadIdx.x, lane = tid % MS_LANES, cl = tid / MS_LANES;
  const bool computes = tid < MS_COMPUTE;
  const int col = c0 + cl;
  const bool live = computes && col <= dv;  // column dv is n
  float* sp = state + (size_t)slot * state_stride + ((size_t)h * (dv + 1) + min(col, dv)) * d;
  float S[NPT];
#pragma unroll
  for (int i = 0; i < NPT; ++i) {
    const int r = lane + MS_LANES * i;
    S[i] = (live && r < d) ? sp[r] : 0.f;
  }
  const int n_stages = (t1 - t0 + MS_TOKENS - 1) / MS_TOKENS;
  if (vec) {
    // the pieces never reach the rows beyond d: those are zero for good
    for (int i = tid; i < 2 * MS_TOKENS * DP; i += MS_THREADS) {
      (&qs[0][0][0])[i] = 0.f;
      (&ks[0][0][0])[i] = 0.f;
    }
    __syncthreads();
  }
  auto fetch = [&](int stage, int first, int step) {
    const int ts = t0 + stage * MS_TOKENS, nt = min(MS_TOKENS, t1 - ts), buf = stage & 1;
    if (vec) {
      // 16-byte pieces, four of q and four of k in flight a thread before any is unpacked
      constexpr int VE = Piece<T>::N;
      const int cpr = d / VE, n = nt * cpr;
      for (int base = first; base < n; base += 4 * step) {
        uint4 qa[4], ka[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int i = base + u * step;
          if (i < n) {
            const int tt = i / cpr, r0 = (i - tt * cpr) * VE;
            qa[u] = *reinterpret_cast<const uint4*>(q + (size_t)(ts + tt) * q_stride + (size_t)h * d + r0);
            ka[u] = *reinterpret_cast<const uint4*>(k + (size_t)(ts + tt) * k_stride + (size_t)h * d + r0);
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int i = base + u * step;
          if (i < n) {
            const int tt = i / cpr, r0 = (i - tt * cpr) * VE;
            float qv[VE], kv[VE];
            Piece<T>::unpack(qa[u], qv);
            Piece<T>::unpack(ka[u], kv);
#pragma unroll
            for (int j = 0; j < VE; ++j) {
              qs[buf][tt][r0 + j] = qv[j] * q_scale;
              ks[buf][tt][r0 + j] = kv[j];
            }
          }
        }
      }
    } else {
#pragma unroll 4
      for (int i = first; i < nt * DP; i += step) {
        const int tt = i / DP, r = i - tt * DP;
        float qv = 0.f, kv = 0.f;
        if (r < d) {
          qv = to_f32<T>(q[(size_t)(ts + tt) * q_stride + (size_t)h * d + r]) * q_scale;
          kv = to_f32<T>(k[(size_t)(ts + tt) * k_stride + (size_t)h * d + r]);
        }
        qs[buf][tt][r] = qv;
        ks[buf][tt][r] = kv;
      }
    }
    for (int i = first; i < nt * MS_COLS; i += step) {
      const int tt = i / MS_COLS, c = c0 + (i - tt * MS_COLS);
      const float w = expf(coef[((size_t)(ts + tt) * heads + h) * 3 + 1]);
      float vv = 0.f;
      if (c < dv) vv = to_f32<T>(v[(size_t)(ts + tt) * v_stride + (size_t)h * dv + c]) * w;
      else if (c == dv) vv = w;
      vs[buf][tt][i - tt * MS_COLS] = vv;
    }
    for (int i = first; i < nt; i += step) keep[buf][i] = expf(coef[((size_t)(ts + i) * heads + h) * 3]);
  };
  fetch(0, tid, MS_THREADS);
  __syncthreads();
  for (int stage = 0; stage < n_stages; ++stage) {
    const int ts = t0 + stage * MS_TOKENS, nt = min(MS_TOKENS, t1 - ts), buf = stage & 1;
    if (computes) {
      // (unrolled: a token's sums over the lanes do not hold up the next token's update of S)
#pragma unroll 4
      for (int tt = 0; tt < nt; ++tt) {
        const float kp = keep[buf][tt], vv = vs[buf][tt][cl];
        float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
        for (int i = 0; i < NPT; i += 2) {
          S[i] = fmaf(kp, S[i], ks[buf][tt][lane + MS_LANES * i] * vv);
          acc0 = fmaf(S[i], qs[buf][tt][lane + MS_LANES * i], acc0);
          S[i + 1] = fmaf(kp, S[i + 1], ks[buf][tt][lane + MS_LANES * (i + 1)] * vv);
          acc1 = fmaf(S[i + 1], qs[buf][tt][lane + MS_LANES * (i + 1)], acc1);
        }
        float acc = acc0 + acc1;
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        acc += __shfl_xor_sync(0xffffffffu, acc, 4);
        if (lane == 0) ys[buf][tt][cl] = acc;
      }
    } else if (stage + 1 < n_stages) {
      fetch(stage + 1, tid - MS_COMPUTE, MS_FETCH);
    }
    __syncthreads();
    // (this stage's outputs leave while the next stage is walked: they have a buffer of their own)
    for (int i = tid; i < nt * MS_COLS; i += MS_THREADS) {
      const int tt = i / MS_COLS, c = c0 + (i - tt * MS_COLS);
      if (c <= dv) y[(size_t)(ts + tt) * y_stride + (size_t)h * (dv + 1) + c] = ys[buf][tt][i - tt * MS_COLS];
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
  constexpr int VE = 16 / (int)sizeof(T);
  const bool vec = d % VE == 0 && qs % VE == 0 && ks % VE == 0 && ((uintptr_t)q & 15) == 0 && ((uintptr_t)k & 15) == 0;
#define FG_MS(NPT)                                                                                                  \
  mlstm_scan_kernel<T, NPT><<<grid, MS_THREADS, 0, stream>>>(q, qs, k, ks, v, vs, coef, y, ys, state, ss, seq_slot, \
                                                             seq_start, heads, d, dv, q_scale, vec)
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

// gates: float32 [T, 2 heads] raw sums (steps of many tokens overwrite them with the log gates).  q, k, v: row-strided views of the
// compute type.  coef: float32 scratch [T, heads, 3].  y: float32 [T, heads * (dv + 1)].
extern "C" int fg_mlstm_scan(float* gates, const float* gate_bias, float cap, const void* q, long q_stride, const void* k,
                             long k_stride, const void* v, long v_stride, int dtype, float* coef, float* y,
                             long y_stride, float* state, long state_stride, const int* req, const int* seq_slot,
                             const int* seq_start, int n_tokens, int n_seqs, int heads, int d, int dv, float q_scale,
                             cudaStream_t stream) {
  if (n_tokens == 0 || n_seqs == 0) return 0;
  FG_CHECK_ARG(heads > 0 && d > 0 && d <= 256 && dv > 0 && cap > 0.f, "fg_mlstm_scan: %d heads of %d x %d", heads, d, dv);
  FG_CHECK_ARG(n_seqs <= 65535 && heads <= 65535, "fg_mlstm_scan: too many sequences or heads");
  // many tokens: the gates of all tokens side by side first; few: on their way into the chain's kernel
  const bool few = n_tokens <= 4 * n_seqs;
  if (!few) {
    const long n = (long)n_tokens * 2 * heads;
    mlstm_gates_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(gates, gate_bias, req, n_tokens, heads, cap);
    FG_CHECK_LAUNCH("fg_mlstm_scan (gates)");
  }
  const long m_offset = (long)heads * (dv + 1) * d;
  // a stretch of tokens whose gates and coefficients fit 40 KiB of shared memory
  int stretch = (40 * 1024 / 4) / (5 * heads);
  stretch = stretch < 1 ? 1 : (stretch > 256 ? 256 : stretch);
  FG_CHECK_ARG(5 * heads * 4 <= 40 * 1024, "fg_mlstm_scan: %d heads are too many", heads);
  mlstm_maxima_kernel<<<n_seqs, MX_THREADS, (size_t)stretch * 5 * heads * sizeof(float), stream>>>(
      gates, coef, state, state_stride, m_offset, seq_slot, seq_start, heads, stretch, few ? gate_bias : nullptr, cap);
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
