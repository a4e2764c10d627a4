// The state-space mixer (Mamba-2 form): short causal convolution with SiLU, the recurrence
// over a per-head matrix state, and the gated norm of its output.
//
// The mixer's input projection gives, per token, a row [z | x | B | C | dt] (inner, inner,
// groups*N, groups*N, heads columns).  x, B and C ("xBC", `channels` columns) pass the
// convolution; then, per head h with group g = h / (heads / groups), in float32:
//
//   dt = softplus(dt_raw + dt_bias[h]);   a = exp(-exp(A_log[h]) * dt)
//   S <- a * S + dt * B x^T      (S is N x P, P the head's value size)
//   y = S^T C + D[h] * x
//
// A request's state lives in one float32 row per slot: [heads, P, N] for S (a column's rows side
// by side, as the recurrence's threads hold them), then
// [taps-1, channels] for the convolution's last inputs (oldest first).  It is zero at
// admission, which is also "zeros before the start" for the convolution.  A step may bring a
// sequence any number of tokens; sequences are consecutive runs of tokens with one slot, and
// tokens of slot < 0 are padding that touches nothing.
//
// The recurrence runs token by token, so its sums do not depend on how a prompt was cut or
// what else is in the batch.
#include "common.cuh"

// ---- convolution + SiLU ---------------------------------------------------------------------
// out[t, c] = silu(bias[c] + sum_k w[c, k] * in[t - (taps-1-k), c]); inputs before the step's
// first token of the sequence come from the state.
constexpr int CONV_THREADS = 128;
constexpr int CONV_MAX_TAPS = 8;

// A thread computes one channel of four consecutive tokens.  Nothing here waits for anything
// else: the slots of the tokens around them are read first, then all the taps' inputs (from the
// step's tokens, or from the state where a sequence's part of the step began less than taps-1
// tokens ago), and neighbouring threads' re-reads hit the cache.
constexpr int CONV_TOKENS = 4;

// TO: the output's type; SILU: whether the sum passes SiLU (else it is stored as it is).
template <typename T, typename TO, bool SILU>
__global__ void __launch_bounds__(CONV_THREADS)
conv_silu_kernel(const T* __restrict__ in, long in_stride, TO* __restrict__ out, long out_stride,
                 const float* __restrict__ w, const float* __restrict__ bias, const float* __restrict__ state,
                 long state_stride, long conv_offset, const int* __restrict__ req, int n_tokens, int channels,
                 int taps) {
  const int c = blockIdx.y * CONV_THREADS + threadIdx.x;
  if (c >= channels) return;
  const int t0 = blockIdx.x * CONV_TOKENS;
  constexpr int BACK = CONV_MAX_TAPS - 1;
  int rq[CONV_TOKENS + BACK];  // rq[j]: the slot of token t0 - BACK + j
#pragma unroll
  for (int j = 0; j < CONV_TOKENS + BACK; ++j) {
    const int t = t0 - BACK + j;
    rq[j] = (t >= 0 && t < n_tokens) ? req[t] : -1;
  }
  float wk[CONV_MAX_TAPS];
#pragma unroll
  for (int k = 0; k < CONV_MAX_TAPS; ++k) wk[k] = k < taps ? w[(size_t)c * taps + k] : 0.f;
  const float bc = bias ? bias[c] : 0.f;
  float v[CONV_TOKENS][CONV_MAX_TAPS];
#pragma unroll
  for (int u = 0; u < CONV_TOKENS; ++u) {
    const int t = t0 + u, slot = rq[u + BACK];
    // how many of the taps-1 tokens before t the step itself brings
    int have = 0;
#pragma unroll
    for (int b = 1; b <= BACK; ++b)
      if (have == b - 1 && b <= taps - 1 && rq[u + BACK - b] == slot) have = b;
#pragma unroll
    for (int k = 0; k < CONV_MAX_TAPS; ++k) {
      v[u][k] = 0.f;
      if (slot >= 0 && k < taps) {
        const int back = taps - 1 - k;  // this tap meets the input `back` tokens ago
        v[u][k] = back <= have ? to_f32<T>(in[(size_t)(t - back) * in_stride + c])
                               : state[(size_t)slot * state_stride + conv_offset +
                                       (size_t)(taps - 1 + have - back) * channels + c];
      }
    }
  }
#pragma unroll
  for (int u = 0; u < CONV_TOKENS; ++u) {
    if (rq[u + BACK] < 0) continue;
    float acc = bc;
#pragma unroll
    for (int k = 0; k < CONV_MAX_TAPS; ++k)
      if (k < taps) acc = fmaf(wk[k], v[u][k], acc);
    out[(size_t)(t0 + u) * out_stride + c] = from_f32<TO>(SILU ? acc / (1.f + expf(-acc)) : acc);
  }
}

// The state's convolution inputs after the step: the last taps-1 of (old inputs, new inputs).
template <typename T>
__global__ void __launch_bounds__(CONV_THREADS)
conv_state_kernel(const T* __restrict__ in, long in_stride, float* __restrict__ state, long state_stride,
                  long conv_offset, const int* __restrict__ seq_slot, const int* __restrict__ seq_start,
                  int channels, int taps) {
  const int c = blockIdx.y * CONV_THREADS + threadIdx.x;
  const int slot = seq_slot[blockIdx.x];
  if (c >= channels || slot < 0) return;
  const int start = seq_start[blockIdx.x], n = seq_start[blockIdx.x + 1] - start;
  float* st = state + (size_t)slot * state_stride + conv_offset;
  // ascending k: entry k + n is read before any write reaches it
  for (int k = 0; k < taps - 1; ++k) {
    const int j = n - (taps - 1) + k;
    const float v = j >= 0 ? to_f32<T>(in[(size_t)(start + j) * in_stride + c]) : st[(size_t)(k + n) * channels + c];
    st[(size_t)k * channels + c] = v;
  }
}

// ---- the recurrence ---------------------------------------------------------------------------
// A block works on (sequence, head, 16 columns of P); LANES threads share a column p, each with
// every LANES-th row n of the state in registers (8 threads a column for small states, a warp a
// column from 64 rows on: the recurrence has heads * P * N independent chains and nothing else
// to fill the GPU with).  Tokens are staged through shared
// memory sixteen at a time in two buffers: while a stage is computed, the next one's B, C and x
// arrive by asynchronous copies and its raw step sizes wait in a register.
constexpr int SCAN_PB = 16;      // columns of P a block
constexpr int SCAN_TOKENS = 16;  // tokens a stage
constexpr int SCAN_GROUP = 8;    // tokens whose sums are reduced together

__device__ __forceinline__ void cp_async_4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src)
               : "memory");
}

template <typename T, int NPT, int SCAN_LANES>
__global__ void __launch_bounds__(SCAN_PB * SCAN_LANES)
ssm_scan_kernel(const float* __restrict__ xbc, long xbc_stride, const T* __restrict__ dt_raw, long dt_stride,
                const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ d_skip,
                float* __restrict__ y, long y_stride, float* __restrict__ state, long state_stride,
                const int* __restrict__ seq_slot, const int* __restrict__ seq_start, int heads, int groups,
                int N, int P) {
  constexpr int SCAN_THREADS = SCAN_PB * SCAN_LANES;
  extern __shared__ float smem[];
  const int stage_floats = 2 * SCAN_TOKENS * N + SCAN_TOKENS * SCAN_PB + 2 * SCAN_TOKENS;
  auto Bs = [&](int buf) { return smem + buf * stage_floats; };               // [SCAN_TOKENS][N]
  auto Cs = [&](int buf) { return Bs(buf) + SCAN_TOKENS * N; };               // [SCAN_TOKENS][N]
  auto xs = [&](int buf) { return Cs(buf) + SCAN_TOKENS * N; };               // [SCAN_TOKENS][SCAN_PB]
  auto dts = [&](int buf) { return xs(buf) + SCAN_TOKENS * SCAN_PB; };        // [SCAN_TOKENS]
  auto decs = [&](int buf) { return dts(buf) + SCAN_TOKENS; };                // [SCAN_TOKENS]

  const int slot = seq_slot[blockIdx.x];
  if (slot < 0) return;
  const int start = seq_start[blockIdx.x], n_tok = seq_start[blockIdx.x + 1] - start;
  if (n_tok <= 0) return;
  const int h = blockIdx.y, g = h / (heads / groups);
  const int p0 = blockIdx.z * SCAN_PB;
  const int tid = threadIdx.x;
  const int pl = tid / SCAN_LANES, lane = tid % SCAN_LANES;
  const int p = p0 + pl;
  const bool p_ok = p < P;
  const int inner = heads * P;
  const float bias = dt_bias[h];
  const float a = -expf(a_log[h]);
  const float dsk = d_skip[h];

  float* S = state + (size_t)slot * state_stride + (size_t)h * N * P;
  float s[NPT];
#pragma unroll
  for (int i = 0; i < NPT; ++i) {
    const int n = lane + SCAN_LANES * i;
    s[i] = (p_ok && n < N) ? S[(size_t)p * N + n] : 0.f;
  }

  const int n_stages = (n_tok + SCAN_TOKENS - 1) / SCAN_TOKENS;
  auto issue = [&](int k) {
    const int buf = k & 1, t0 = k * SCAN_TOKENS, nt = min(SCAN_TOKENS, n_tok - t0);
    float *bs = Bs(buf), *cs = Cs(buf), *xx = xs(buf);
    for (int i = tid; i < nt * N; i += SCAN_THREADS) {
      const int tt = i / N, n = i - tt * N;
      const float* row = xbc + (size_t)(start + t0 + tt) * xbc_stride + inner + g * N + n;
      cp_async_4(bs + i, row);
      cp_async_4(cs + i, row + groups * N);
    }
    for (int i = tid; i < nt * SCAN_PB; i += SCAN_THREADS) {
      const int tt = i / SCAN_PB, pp = i - tt * SCAN_PB;
      if (p0 + pp < P) cp_async_4(xx + i, xbc + (size_t)(start + t0 + tt) * xbc_stride + h * P + p0 + pp);
      else xx[i] = 0.f;
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };
  auto raw_dt = [&](int k) {
    const int t = k * SCAN_TOKENS + tid;
    return (tid < SCAN_TOKENS && t < n_tok) ? to_f32<T>(dt_raw[(size_t)(start + t) * dt_stride + h]) : 0.f;
  };
  issue(0);
  float dtr = raw_dt(0);

  for (int k = 0; k < n_stages; ++k) {
    const int buf = k & 1, t0 = k * SCAN_TOKENS, nt = min(SCAN_TOKENS, n_tok - t0);
    if (tid < nt) {
      const float v = dtr + bias;
      const float dt = v > 20.f ? v : log1pf(expf(v));
      dts(buf)[tid] = dt;
      decs(buf)[tid] = expf(a * dt);
    }
    if (k + 1 < n_stages) {
      issue(k + 1);
      dtr = raw_dt(k + 1);
      asm volatile("cp.async.wait_group 1;\n" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    }
    __syncthreads();
    const float *bs = Bs(buf), *cs = Cs(buf), *xx = xs(buf), *dd = dts(buf), *de = decs(buf);
    // eight tokens at a time: their sums over the state's rows are reduced across the column's
    // threads together, and thread j of the column stores token j's output
    for (int tt0 = 0; tt0 < nt; tt0 += SCAN_GROUP) {
      float acc[SCAN_GROUP];
#pragma unroll
      for (int u = 0; u < SCAN_GROUP; ++u) {
        const int tt = tt0 + u;
        float a0 = 0.f, a1 = 0.f;
        if (tt < nt) {
          const float dec = de[tt];
          const float dx = dd[tt] * xx[tt * SCAN_PB + pl];
#pragma unroll
          for (int i = 0; i < NPT; ++i) {
            const int n = lane + SCAN_LANES * i;
            if (n < N) {
              s[i] = fmaf(dec, s[i], bs[tt * N + n] * dx);
              if (i & 1) a1 = fmaf(s[i], cs[tt * N + n], a1);
              else a0 = fmaf(s[i], cs[tt * N + n], a0);
            }
          }
        }
        acc[u] = a0 + a1;
      }
#pragma unroll
      for (int o = SCAN_LANES / 2; o > 0; o >>= 1)
#pragma unroll
        for (int u = 0; u < SCAN_GROUP; ++u) acc[u] += __shfl_xor_sync(0xffffffffu, acc[u], o);
      float mine = 0.f;
#pragma unroll
      for (int u = 0; u < SCAN_GROUP; ++u)
        if (lane == u) mine = acc[u];
      const int tt = tt0 + lane;
      if (lane < SCAN_GROUP && tt < nt && p_ok) y[(size_t)(start + t0 + tt) * y_stride + h * P + p] = fmaf(dsk, xx[tt * SCAN_PB + pl], mine);
    }
    __syncthreads();  // the stage is read to its end before the copies after next overwrite it
  }
#pragma unroll
  for (int i = 0; i < NPT; ++i) {
    const int n = lane + SCAN_LANES * i;
    if (p_ok && n < N) S[(size_t)p * N + n] = s[i];
  }
}

// ---- the recurrence, states of 64, 128 or 256 rows ------------------------------------------------
// The same recurrence with fewer instructions a state element: N = 32 * NPT is a compile-time
// number (no bounds to test, every address an immediate), B and C of a token sit side by side in
// shared memory (one 8-byte load brings both), a warp owns two columns of P (a loaded pair serves
// both), and the sums of 8 tokens x 2 columns over the state's rows are reduced by halving
// exchanges (16 shuffles for the 16 sums) that leave sum k in lanes 2k and 2k + 1.
constexpr int TS_COLS = 2;                       // columns of P a warp
constexpr int TS_WARPS = SCAN_PB / TS_COLS;      // warps a block
constexpr int TS_THREADS = 32 * TS_WARPS;

template <typename T, int NPT>
__global__ void __launch_bounds__(TS_THREADS)
ssm_scan_tiled_kernel(const float* __restrict__ xbc, long xbc_stride, const T* __restrict__ dt_raw, long dt_stride,
                      const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                      const float* __restrict__ d_skip, float* __restrict__ y, long y_stride,
                      float* __restrict__ state, long state_stride, const int* __restrict__ seq_slot,
                      const int* __restrict__ seq_start, int heads, int groups, int P) {
  constexpr int N = 32 * NPT;
  constexpr int STAGE = 2 * SCAN_TOKENS * N + SCAN_TOKENS * SCAN_PB + 2 * SCAN_TOKENS;  // floats
  extern __shared__ __align__(16) float smem[];
  auto BC = [&](int buf) { return reinterpret_cast<float2*>(smem + buf * STAGE); };      // [TOKENS][N] (B, C)
  auto xs = [&](int buf) { return smem + buf * STAGE + 2 * SCAN_TOKENS * N; };           // [TOKENS][SCAN_PB]
  auto dts = [&](int buf) { return xs(buf) + SCAN_TOKENS * SCAN_PB; };
  auto decs = [&](int buf) { return dts(buf) + SCAN_TOKENS; };

  const int slot = seq_slot[blockIdx.x];
  if (slot < 0) return;
  const int start = seq_start[blockIdx.x], n_tok = seq_start[blockIdx.x + 1] - start;
  if (n_tok <= 0) return;
  const int h = blockIdx.y, g = h / (heads / groups);
  const int p0 = blockIdx.z * SCAN_PB;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int pc = p0 + TS_COLS * warp;  // this warp's first column
  const int inner = heads * P;
  const float bias = dt_bias[h];
  const float a = -expf(a_log[h]);
  const float dsk = d_skip[h];

  float* S = state + (size_t)slot * state_stride + (size_t)h * N * P;
  float s[TS_COLS][NPT];
#pragma unroll
  for (int c = 0; c < TS_COLS; ++c)
#pragma unroll
    for (int i = 0; i < NPT; ++i) s[c][i] = pc + c < P ? S[(size_t)(pc + c) * N + lane + 32 * i] : 0.f;

  const int n_stages = (n_tok + SCAN_TOKENS - 1) / SCAN_TOKENS;
  auto issue = [&](int k) {
    const int buf = k & 1, t0 = k * SCAN_TOKENS, nt = min(SCAN_TOKENS, n_tok - t0);
    float* bc = smem + buf * STAGE;
    float* xx = xs(buf);
    for (int i = tid; i < nt * N; i += TS_THREADS) {
      const int tt = i / N, n = i - tt * N;
      const float* row = xbc + (size_t)(start + t0 + tt) * xbc_stride + inner + g * N + n;
      cp_async_4(bc + 2 * i, row);
      cp_async_4(bc + 2 * i + 1, row + groups * N);
    }
    for (int i = tid; i < nt * SCAN_PB; i += TS_THREADS) {
      const int tt = i / SCAN_PB, pp = i - tt * SCAN_PB;
      if (p0 + pp < P) cp_async_4(xx + i, xbc + (size_t)(start + t0 + tt) * xbc_stride + h * P + p0 + pp);
      else xx[i] = 0.f;
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };
  auto raw_dt = [&](int k) {
    const int t = k * SCAN_TOKENS + tid;
    return (tid < SCAN_TOKENS && t < n_tok) ? to_f32<T>(dt_raw[(size_t)(start + t) * dt_stride + h]) : 0.f;
  };
  issue(0);
  float dtr = raw_dt(0);

  for (int k = 0; k < n_stages; ++k) {
    const int buf = k & 1, t0 = k * SCAN_TOKENS, nt = min(SCAN_TOKENS, n_tok - t0);
    if (tid < nt) {
      const float v = dtr + bias;
      const float dt = v > 20.f ? v : log1pf(expf(v));
      dts(buf)[tid] = dt;
      decs(buf)[tid] = expf(a * dt);
    }
    if (k + 1 < n_stages) {
      issue(k + 1);
      dtr = raw_dt(k + 1);
      asm volatile("cp.async.wait_group 1;\n" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    }
    __syncthreads();
    const float2* bc = BC(buf);
    const float *xx = xs(buf), *dd = dts(buf), *de = decs(buf);
    for (int tt0 = 0; tt0 < nt; tt0 += SCAN_GROUP) {
      float acc[TS_COLS * SCAN_GROUP];  // [column][token of the group]
#pragma unroll
      for (int u = 0; u < SCAN_GROUP; ++u) {
        const int tt = tt0 + u;
        float a0 = 0.f, a1 = 0.f;
        if (tt < nt) {
          const float dec = de[tt], dtv = dd[tt];
          const float2 xv = *reinterpret_cast<const float2*>(xx + tt * SCAN_PB + TS_COLS * warp);
          const float dx0 = dtv * xv.x, dx1 = dtv * xv.y;
#pragma unroll
          for (int i = 0; i < NPT; ++i) {
            const float2 v = bc[tt * N + lane + 32 * i];
            s[0][i] = fmaf(dec, s[0][i], v.x * dx0);
            a0 = fmaf(s[0][i], v.y, a0);
            s[1][i] = fmaf(dec, s[1][i], v.x * dx1);
            a1 = fmaf(s[1][i], v.y, a1);
          }
        }
        acc[u] = a0;
        acc[SCAN_GROUP + u] = a1;
      }
      // halving exchanges: after the step with mask m a lane keeps the half of its sums that its
      // bit m chooses, with the partner's share added
#pragma unroll
      for (int half = TS_COLS * SCAN_GROUP / 2, mask = 16; half >= 1; half >>= 1, mask >>= 1) {
        const bool upper = (lane & mask) != 0;
#pragma unroll
        for (int j = 0; j < half; ++j) {
          const float send = upper ? acc[j] : acc[j + half];
          const float keep = upper ? acc[j + half] : acc[j];
          acc[j] = keep + __shfl_xor_sync(0xffffffffu, send, mask);
        }
      }
      acc[0] += __shfl_xor_sync(0xffffffffu, acc[0], 1);  // (16 sums use the masks 16, 8, 4, 2)
      const int kidx = (lane >> 1) & 15, c = kidx >> 3, tt = tt0 + (kidx & 7);
      if (!(lane & 1) && tt < nt && pc + c < P)
        y[(size_t)(start + t0 + tt) * y_stride + h * P + pc + c] =
            fmaf(dsk, xx[tt * SCAN_PB + TS_COLS * warp + c], acc[0]);
    }
    __syncthreads();  // the stage is read to its end before the copies after next overwrite it
  }
#pragma unroll
  for (int c = 0; c < TS_COLS; ++c)
#pragma unroll
    for (int i = 0; i < NPT; ++i)
      if (pc + c < P) S[(size_t)(pc + c) * N + lane + 32 * i] = s[c][i];
}

// ---- gate, then RMS norm in equal parts ---------------------------------------------------------
// out[t, part] = v * rsqrt(mean(v^2) + eps) * w with v = y * silu(z) over the part's columns.
constexpr int GN_THREADS = 256;

template <typename T>
__global__ void __launch_bounds__(GN_THREADS)
gated_part_norm_kernel(const float* __restrict__ y, long y_stride, const T* __restrict__ z, long z_stride,
                       const float* __restrict__ w, T* __restrict__ out, long out_stride, const int* __restrict__ req,
                       int part, float eps) {
  __shared__ float scratch[32];
  const int t = blockIdx.x, c0 = blockIdx.y * part;
  if (req[t] < 0) return;
  const float* yr = y + (size_t)t * y_stride + c0;
  const T* zr = z + (size_t)t * z_stride + c0;
  float ss = 0.f;
  for (int d = threadIdx.x; d < part; d += GN_THREADS) {
    const float zv = to_f32<T>(zr[d]);
    const float v = yr[d] * (zv / (1.f + expf(-zv)));
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float rstd = 1.f / sqrtf(ss / (float)part + eps);
  for (int d = threadIdx.x; d < part; d += GN_THREADS) {
    const float zv = to_f32<T>(zr[d]);
    const float v = yr[d] * (zv / (1.f + expf(-zv)));
    out[(size_t)t * out_stride + c0 + d] = from_f32<T>(v * rstd * w[c0 + d]);
  }
}

// Parts of up to 1,024 columns: a warp a (token, part), the part's values in registers between the
// sum of squares and the scaling, so y and z are read once.
constexpr int GW_WARPS = 8;
constexpr int GW_ITEMS = 32;

template <typename T>
__global__ void __launch_bounds__(GW_WARPS * 32)
gated_part_norm_warp_kernel(const float* __restrict__ y, long y_stride, const T* __restrict__ z, long z_stride,
                            const float* __restrict__ w, T* __restrict__ out, long out_stride,
                            const int* __restrict__ req, int n_tokens, int parts, int part, float eps) {
  const int lane = threadIdx.x & 31;
  const long item = (long)blockIdx.x * GW_WARPS + (threadIdx.x >> 5);
  if (item >= (long)n_tokens * parts) return;
  const int t = item / parts, c0 = (item - (long)t * parts) * part;
  if (req[t] < 0) return;
  const float* yr = y + (size_t)t * y_stride + c0;
  const T* zr = z + (size_t)t * z_stride + c0;
  float v[GW_ITEMS];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < GW_ITEMS; ++i) {
    const int d = lane + 32 * i;
    v[i] = 0.f;
    if (d < part) {
      const float zv = to_f32<T>(zr[d]);
      v[i] = yr[d] * (zv / (1.f + expf(-zv)));
    }
    ss += v[i] * v[i];
  }
  ss = warp_sum(ss);
  const float rstd = 1.f / sqrtf(ss / (float)part + eps);
#pragma unroll
  for (int i = 0; i < GW_ITEMS; ++i) {
    const int d = lane + 32 * i;
    if (d < part) out[(size_t)t * out_stride + c0 + d] = from_f32<T>(v[i] * rstd * w[c0 + d]);
  }
}

// ---- C interface -----------------------------------------------------------------------------------

// A causal convolution over time per channel, from and into the state's last inputs, with a choice
// of activation (act 1: SiLU, 0: none) and of the output's type (out_dtype).
template <typename T, typename TO>
static int launch_time_conv(const T* in, long proj_stride, TO* out, long out_stride, const float* w, const float* bias,
                            float* state, long state_stride, long conv_offset, const int* req, const int* seq_slot,
                            const int* seq_start, int n_tokens, int n_seqs, int channels, int taps, int act,
                            cudaStream_t stream) {
  const dim3 grid((n_tokens + CONV_TOKENS - 1) / CONV_TOKENS, (channels + CONV_THREADS - 1) / CONV_THREADS);
  const dim3 sgrid(n_seqs, grid.y);
  if (act)
    conv_silu_kernel<T, TO, true><<<grid, CONV_THREADS, 0, stream>>>(in, proj_stride, out, out_stride, w, bias, state,
                                                                     state_stride, conv_offset, req, n_tokens, channels,
                                                                     taps);
  else
    conv_silu_kernel<T, TO, false><<<grid, CONV_THREADS, 0, stream>>>(in, proj_stride, out, out_stride, w, bias, state,
                                                                      state_stride, conv_offset, req, n_tokens,
                                                                      channels, taps);
  FG_CHECK_LAUNCH("fg_time_conv");
  if (taps > 1)
    conv_state_kernel<T><<<sgrid, CONV_THREADS, 0, stream>>>(in, proj_stride, state, state_stride, conv_offset, seq_slot,
                                                             seq_start, channels, taps);
  FG_CHECK_LAUNCH("fg_time_conv (state)");
  return 0;
}

extern "C" int fg_time_conv(const void* proj, long proj_stride, long offset, int dtype, void* out, long out_stride,
                            int out_dtype, const float* w, const float* bias, float* state, long state_stride,
                            long conv_offset, const int* req, const int* seq_slot, const int* seq_start, int n_tokens,
                            int n_seqs, int channels, int taps, int act, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  FG_CHECK_ARG(taps >= 1 && taps <= CONV_MAX_TAPS, "fg_time_conv: %d taps (1 to %d)", taps, CONV_MAX_TAPS);
  FG_CHECK_ARG((dtype == FG_F32 || dtype == FG_BF16) && (out_dtype == FG_F32 || out_dtype == dtype),
               "fg_time_conv: types %d -> %d", dtype, out_dtype);
#define FG_CONV_ARGS w, bias, state, state_stride, conv_offset, req, seq_slot, seq_start, n_tokens, n_seqs, channels, taps, act, stream
  if (dtype == FG_F32)
    return launch_time_conv((const float*)proj + offset, proj_stride, (float*)out, out_stride, FG_CONV_ARGS);
  if (out_dtype == FG_F32)
    return launch_time_conv((const __nv_bfloat16*)proj + offset, proj_stride, (float*)out, out_stride, FG_CONV_ARGS);
  return launch_time_conv((const __nv_bfloat16*)proj + offset, proj_stride, (__nv_bfloat16*)out, out_stride, FG_CONV_ARGS);
#undef FG_CONV_ARGS
}

extern "C" int fg_mamba2_conv(const void* proj, long proj_stride, long xbc_offset, int dtype, float* out,
                              long out_stride, const float* w, const float* bias, float* state, long state_stride,
                              long conv_offset, const int* req, const int* seq_slot, const int* seq_start,
                              int n_tokens, int n_seqs, int channels, int taps, cudaStream_t stream) {
  return fg_time_conv(proj, proj_stride, xbc_offset, dtype, out, out_stride, FG_F32, w, bias, state, state_stride,
                      conv_offset, req, seq_slot, seq_start, n_tokens, n_seqs, channels, taps, 1, stream);
}

template <typename T>
static int launch_scan(const float* xbc, long xbc_stride, const T* dt_raw, long dt_stride, const float* dt_bias,
                       const float* a_log, const float* d_skip, float* y, long y_stride, float* state, long state_stride,
                       const int* seq_slot, const int* seq_start, int n_seqs, int heads, int groups, int N, int P,
                       cudaStream_t stream) {
  const dim3 grid(n_seqs, heads, (P + SCAN_PB - 1) / SCAN_PB);
  const size_t smem = 2 * sizeof(float) * (size_t)(2 * SCAN_TOKENS * N + SCAN_TOKENS * SCAN_PB + 2 * SCAN_TOKENS);
  if (N == 64 || N == 128 || N == 256) {
    const size_t tsmem = 2 * sizeof(float) * (size_t)(2 * SCAN_TOKENS * N + SCAN_TOKENS * SCAN_PB + 2 * SCAN_TOKENS);
#define TILED(NPT)                                                                                              \
  do {                                                                                                          \
    auto kern = ssm_scan_tiled_kernel<T, NPT>;                                                                  \
    if (tsmem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tsmem); \
    kern<<<grid, TS_THREADS, tsmem, stream>>>(xbc, xbc_stride, dt_raw, dt_stride, dt_bias, a_log, d_skip, y,    \
                                              y_stride, state, state_stride, seq_slot, seq_start, heads,        \
                                              groups, P);                                                       \
  } while (0)
    if (N == 64) TILED(2);
    else if (N == 128) TILED(4);
    else TILED(8);
#undef TILED
    return 0;
  }
  const int lanes = N >= 64 ? 32 : 8;
  const int npt = (N + lanes - 1) / lanes;
#define SCAN(NPT, LANES)                                                                                        \
  do {                                                                                                          \
    auto kern = ssm_scan_kernel<T, NPT, LANES>;                                                                 \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
    kern<<<grid, SCAN_PB * LANES, smem, stream>>>(xbc, xbc_stride, dt_raw, dt_stride, dt_bias, a_log, d_skip, y, \
                                                  y_stride, state, state_stride, seq_slot, seq_start, heads,    \
                                                  groups, N, P);                                                \
  } while (0)
  if (lanes == 32) {
    if (npt <= 2) SCAN(2, 32);
    else if (npt <= 4) SCAN(4, 32);
    else SCAN(8, 32);
  } else {
    if (npt <= 1) SCAN(1, 8);
    else if (npt <= 2) SCAN(2, 8);
    else if (npt <= 4) SCAN(4, 8);
    else SCAN(8, 8);
  }
#undef SCAN
  return 0;
}

extern "C" int fg_mamba2_scan(const float* xbc, long xbc_stride, const void* proj, long proj_stride, long dt_offset,
                              int dtype, const float* dt_bias, const float* a_log, const float* d_skip, float* y,
                              long y_stride, float* state, long state_stride, const int* seq_slot,
                              const int* seq_start, int n_seqs, int heads, int groups, int N, int P,
                              cudaStream_t stream) {
  if (n_seqs == 0) return 0;
  FG_CHECK_ARG(heads > 0 && groups > 0 && heads % groups == 0 && N > 0 && P > 0,
               "fg_mamba2_scan: bad sizes heads=%d groups=%d N=%d P=%d", heads, groups, N, P);
  int rc;
  if (dtype == FG_F32)
    rc = launch_scan<float>(xbc, xbc_stride, (const float*)proj + dt_offset, proj_stride, dt_bias,
                            a_log, d_skip, y, y_stride, state, state_stride, seq_slot,
                            seq_start, n_seqs, heads, groups, N, P, stream);
  else if (dtype == FG_BF16)
    rc = launch_scan<__nv_bfloat16>(xbc, xbc_stride, (const __nv_bfloat16*)proj + dt_offset, proj_stride,
                                    dt_bias, a_log, d_skip, y, y_stride, state, state_stride, seq_slot,
                                    seq_start, n_seqs, heads, groups, N, P, stream);
  else
    FG_CHECK_ARG(false, "fg_mamba2_scan: bad dtype %d", dtype);
  if (rc) return rc;
  FG_CHECK_LAUNCH("fg_mamba2_scan");
  return 0;
}

extern "C" int fg_gated_part_norm(const float* y, long y_stride, const void* z, long z_stride, int dtype,
                                  const float* w, void* out, long out_stride, const int* req, int n_tokens, int width,
                                  int parts, float eps, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  FG_CHECK_ARG(parts > 0 && width % parts == 0, "fg_gated_part_norm: %d columns in %d parts", width, parts);
  const dim3 grid(n_tokens, parts);
  const int part = width / parts;
  if (part <= 32 * GW_ITEMS) {
    const long items = (long)n_tokens * parts;
    const int blocks = (int)((items + GW_WARPS - 1) / GW_WARPS);
    if (dtype == FG_F32)
      gated_part_norm_warp_kernel<float><<<blocks, GW_WARPS * 32, 0, stream>>>(
          y, y_stride, (const float*)z, z_stride, w, (float*)out, out_stride, req, n_tokens, parts, part, eps);
    else if (dtype == FG_BF16)
      gated_part_norm_warp_kernel<__nv_bfloat16><<<blocks, GW_WARPS * 32, 0, stream>>>(
          y, y_stride, (const __nv_bfloat16*)z, z_stride, w, (__nv_bfloat16*)out, out_stride, req, n_tokens, parts,
          part, eps);
    else
      FG_CHECK_ARG(false, "fg_gated_part_norm: bad dtype %d", dtype);
    FG_CHECK_LAUNCH("fg_gated_part_norm");
    return 0;
  }
  if (dtype == FG_F32)
    gated_part_norm_kernel<float><<<grid, GN_THREADS, 0, stream>>>(y, y_stride, (const float*)z, z_stride,
                                                                    w, (float*)out, out_stride, req,
                                                                    width / parts, eps);
  else if (dtype == FG_BF16)
    gated_part_norm_kernel<__nv_bfloat16><<<grid, GN_THREADS, 0, stream>>>(
        y, y_stride, (const __nv_bfloat16*)z, z_stride, w, (__nv_bfloat16*)out, out_stride, req,
        width / parts, eps);
  else
    FG_CHECK_ARG(false, "fg_gated_part_norm: bad dtype %d", dtype);
  FG_CHECK_LAUNCH("fg_gated_part_norm");
  return 0;
}
