// The gated delta rule: a matrix state per head that forgets per key channel and is corrected
// towards each new value.  Per head, with q, k unit vectors (q also times d^-1/2), a decay
// g in (0, 1)^d, a step size beta and the value v, in float32 and in this order:
//
//     S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q          (S is [d, dv])
//
// The read-out sees the token's own write.  With R = diag(g) S_old, o = R^T q + u (k . q): both
// sums over the rows of the old state are formed side by side and k . q comes with the token.
//
// A block of eight warps works on (sequence, head, a run of the state's columns).  A column's rows
// are spread over LPC lanes, RPL rows a lane in registers (in runs of four, so that a lane reads
// its part of k, g and q as 16-byte words); a warp holds 32 / LPC columns.  The sums over a column's
// rows end in log2(LPC) exchanges, which is what a token's step waits for: the recurrence is a
// chain from token to token, and its length, not the arithmetic, sets the time.  Tokens are staged
// eight at a time through two buffers in shared memory: warp w prepares token w of a stage (unit
// norms, k . q, the decay exp(-exp(A) softplus(a + bias)), sigmoid of the step size: all float32)
// from values it fetched into registers while the stage before was computed; whole stages run
// unrolled, so that a token's operands are read while the one before it is reduced.  The
// recurrence runs token by token, so prompt portions, single tokens and mixed batches take this
// kernel and give the same numbers however a prompt is cut.  The state of a slot is
// [heads][dv][d] float32 (a column's rows side by side), zero at admission.
#include "common.cuh"

constexpr int DELTA_WARPS = 8;
constexpr int DELTA_TOKENS = 8;  // tokens a stage (one warp prepares each)
constexpr int DELTA_THREADS = DELTA_WARPS * 32;
static_assert(DELTA_TOKENS == DELTA_WARPS, "warp w prepares token w of a stage");

__device__ __forceinline__ float softplus_f32(float z) { return z > 20.f ? z : log1pf(expf(z)); }

template <typename TA, int LPC, int RPL>
__global__ void __launch_bounds__(DELTA_THREADS)
delta_scan_kernel(const float* qkv, long qkv_stride, const TA* a, long a_stride, const TA* b, long b_stride,
                  const float* __restrict__ dt_bias, const float* __restrict__ a_log, float* __restrict__ out,
                  long out_stride, float* __restrict__ state, long state_stride, const int* __restrict__ seq_slot,
                  const int* __restrict__ seq_start, int n_heads, int n_kv_heads, int d, int dv) {
  constexpr int DP = LPC * RPL;           // rows, padded
  constexpr int NRP = DP / 32;            // rows a lane prepares
  constexpr int CPW = 32 / LPC;           // columns a warp
  constexpr int COLS = DELTA_WARPS * CPW; // columns a block
  constexpr int NV = (COLS + 31) / 32;
  static_assert(DP % 32 == 0 && RPL % 4 == 0, "rows in runs of four, a multiple of 32 in all");
  extern __shared__ __align__(16) float smem[];
  // per buffer: q[TOK][DP], k[TOK][DP], g[TOK][DP], v[TOK][COLS], beta[TOK], kq[TOK]
  constexpr int BUF = DELTA_TOKENS * (3 * DP + COLS + 2);
  const int slot = seq_slot[blockIdx.z];
  if (slot < 0) return;
  const int start = seq_start[blockIdx.z], n = seq_start[blockIdx.z + 1] - start;
  if (n <= 0) return;
  const int h = blockIdx.y, hk = h / (n_heads / n_kv_heads);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane % LPC, cw = warp * CPW + lane / LPC;  // the lane's part of a column; its column in the block
  const int col0 = blockIdx.x * COLS, j = col0 + cw;
  const bool live_col = j < dv;
  const int q_off = hk * d, k_off = (n_kv_heads + hk) * d, v_off = 2 * n_kv_heads * d + h * dv;
  const float rate = expf(a_log[h]);
  const float q_scale = 1.f / sqrtf((float)d);

  // the lane's rows: 4 (sub + LPC jj) + e for jj < RPL / 4, e < 4
  float S[RPL];
  float* st = state + (size_t)slot * state_stride + ((size_t)h * dv + (live_col ? j : 0)) * d;
#pragma unroll
  for (int i = 0; i < RPL; ++i) {
    const int r = 4 * (sub + LPC * (i >> 2)) + (i & 3);
    S[i] = (live_col && r < d) ? st[r] : 0.f;
  }
  float bias_r[NRP];
#pragma unroll
  for (int i = 0; i < NRP; ++i) {
    const int r = lane + 32 * i;
    bias_r[i] = r < d ? dt_bias[h * d + r] : 0.f;
  }

  // what warp `warp` fetches for its token of the next stage
  float fq[NRP], fk[NRP], fa[NRP], fv[NV], fb = 0.f;
  auto fetch = [&](int stage) {
    const int t = stage * DELTA_TOKENS + warp;
    const bool live = t < n;
    const size_t row = (size_t)(start + (live ? t : 0));
#pragma unroll
    for (int i = 0; i < NRP; ++i) {
      const int r = lane + 32 * i;
      const bool ok = live && r < d;
      fq[i] = ok ? qkv[row * qkv_stride + q_off + r] : 0.f;
      fk[i] = ok ? qkv[row * qkv_stride + k_off + r] : 0.f;
      fa[i] = ok ? to_f32<TA>(a[row * a_stride + h * d + r]) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = lane + 32 * i;
      fv[i] = (live && c < COLS && col0 + c < dv) ? qkv[row * qkv_stride + v_off + col0 + c] : 0.f;
    }
    fb = live ? to_f32<TA>(b[row * b_stride + h]) : 0.f;
  };
  auto prepare = [&](float* buf) {
    float* sq = buf + warp * DP;
    float* sk = buf + DELTA_TOKENS * DP + warp * DP;
    float* sg = buf + 2 * DELTA_TOKENS * DP + warp * DP;
    float* sv = buf + 3 * DELTA_TOKENS * DP;
    float* sbeta = sv + DELTA_TOKENS * COLS;
    float* skq = sbeta + DELTA_TOKENS;
    float ssq = 0.f, ssk = 0.f;
#pragma unroll
    for (int i = 0; i < NRP; ++i) {
      ssq = fmaf(fq[i], fq[i], ssq);
      ssk = fmaf(fk[i], fk[i], ssk);
    }
    ssq = warp_sum(ssq);
    ssk = warp_sum(ssk);
    const float rq = q_scale / sqrtf(ssq + 1e-6f), rk = 1.f / sqrtf(ssk + 1e-6f);
    float kq = 0.f;
#pragma unroll
    for (int i = 0; i < NRP; ++i) {
      const float qn = fq[i] * rq, kn = fk[i] * rk;
      kq = fmaf(qn, kn, kq);
      sq[lane + 32 * i] = qn;
      sk[lane + 32 * i] = kn;
      // rows beyond d: k and q are zero there, and so is the state
      sg[lane + 32 * i] = expf(-rate * softplus_f32(fa[i] + bias_r[i]));
    }
    kq = warp_sum(kq);
#pragma unroll
    for (int i = 0; i < NV; ++i)
      if (lane + 32 * i < COLS) sv[warp * COLS + lane + 32 * i] = fv[i];
    if (lane == 0) {
      sbeta[warp] = 1.f / (1.f + expf(-fb));
      skq[warp] = kq;
    }
  };

  // one token of the recurrence, its operands at `buf` (token tt of the stage)
  auto step = [&](const float* buf, int tt, size_t out_row) {
    const float4* sq = reinterpret_cast<const float4*>(buf + tt * DP);
    const float4* sk = reinterpret_cast<const float4*>(buf + DELTA_TOKENS * DP + tt * DP);
    const float4* sg = reinterpret_cast<const float4*>(buf + 2 * DELTA_TOKENS * DP + tt * DP);
    const float* sv = buf + 3 * DELTA_TOKENS * DP;
    const float* sbeta = sv + DELTA_TOKENS * COLS;
    const float* skq = sbeta + DELTA_TOKENS;
    float kr[RPL];
    float rk2[2] = {0.f, 0.f}, rq2[2] = {0.f, 0.f};
#pragma unroll
    for (int jj = 0; jj < RPL / 4; ++jj) {
      const float4 kv = sk[sub + LPC * jj], gv = sg[sub + LPC * jj], qv = sq[sub + LPC * jj];
      const float ke[4] = {kv.x, kv.y, kv.z, kv.w}, ge[4] = {gv.x, gv.y, gv.z, gv.w}, qe[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = 4 * jj + e;
        kr[i] = ke[e];
        S[i] *= ge[e];
        rk2[e & 1] = fmaf(S[i], ke[e], rk2[e & 1]);
        rq2[e & 1] = fmaf(S[i], qe[e], rq2[e & 1]);
      }
    }
    float rk_sum = rk2[0] + rk2[1], rq_sum = rq2[0] + rq2[1];
#pragma unroll
    for (int o = LPC / 2; o > 0; o >>= 1) {
      rk_sum += __shfl_xor_sync(0xffffffffu, rk_sum, o);
      rq_sum += __shfl_xor_sync(0xffffffffu, rq_sum, o);
    }
    const float u = sbeta[tt] * (sv[tt * COLS + cw] - rk_sum);
#pragma unroll
    for (int i = 0; i < RPL; ++i) S[i] = fmaf(kr[i], u, S[i]);
    if (sub == 0 && live_col) out[out_row * out_stride + h * dv + j] = fmaf(u, skq[tt], rq_sum);
  };

  const int n_stages = (n + DELTA_TOKENS - 1) / DELTA_TOKENS;
  fetch(0);
  for (int stage = 0; stage < n_stages; ++stage) {
    float* buf = smem + (stage & 1) * BUF;
    prepare(buf);
    __syncthreads();
    if (stage + 1 < n_stages) fetch(stage + 1);
    const int n_tok = min(DELTA_TOKENS, n - stage * DELTA_TOKENS);
    const size_t row0 = (size_t)start + (size_t)stage * DELTA_TOKENS;
    if (n_tok == DELTA_TOKENS) {
#pragma unroll
      for (int tt = 0; tt < DELTA_TOKENS; ++tt) step(buf, tt, row0 + tt);
    } else {
      for (int tt = 0; tt < n_tok; ++tt) step(buf, tt, row0 + tt);
    }
  }
  if (live_col) {
#pragma unroll
    for (int i = 0; i < RPL; ++i) {
      const int r = 4 * (sub + LPC * (i >> 2)) + (i & 3);
      if (r < d) st[r] = S[i];
    }
  }
}

template <typename TA>
static int launch_scan(cudaStream_t stream, const float* qkv, long qkv_stride, const TA* a, long a_stride, const TA* b,
                       long b_stride, const float* dt_bias, const float* a_log, float* out, long out_stride,
                       float* state, long state_stride, const int* seq_slot, const int* seq_start, int n_seqs,
                       int n_heads, int n_kv_heads, int d, int dv) {
#define CASE(LPC, RPL)                                                                                         \
  {                                                                                                            \
    constexpr int COLS = DELTA_WARPS * (32 / LPC);                                                             \
    const size_t smem = 2 * DELTA_TOKENS * (3 * LPC * RPL + COLS + 2) * sizeof(float);                          \
    auto kern = delta_scan_kernel<TA, LPC, RPL>;                                                                \
    if (smem > 48 * 1024) {                                                                                     \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
      FG_CHECK_ARG(e == cudaSuccess, "fg_delta_scan: shared memory: %s", cudaGetErrorString(e));                \
    }                                                                                                           \
    dim3 grid((dv + COLS - 1) / COLS, n_heads, n_seqs);                                                         \
    kern<<<grid, DELTA_THREADS, smem, stream>>>(qkv, qkv_stride, a, a_stride, b, b_stride, dt_bias, a_log, out, \
                                                out_stride, state, state_stride, seq_slot, seq_start, n_heads,  \
                                                n_kv_heads, d, dv);                                             \
  }
  if (d <= 32) CASE(4, 8)
  else if (d <= 64) CASE(8, 8)
  else if (d <= 128) CASE(8, 16)
  else if (d <= 256) CASE(16, 16)
  else FG_CHECK_ARG(false, "fg_delta_scan: key size %d (up to 256)", d);
#undef CASE
  return 0;
}

// qkv: float32 [T, q (kv heads x d) | k (kv heads x d) | v (heads x dv)], the convolutions' outputs.
// a: [T, heads x d] decay logits and b: [T, .] step-size logits (column h of row t at b[t * b_stride + h]),
// both of `dtype`.  dt_bias: float32 [heads x d]; a_log: float32 [heads].  out: float32 [T, heads x dv].
// state: float32 [slots, state_stride], a slot's first heads * dv * d numbers.
extern "C" int fg_delta_scan(const float* qkv, long qkv_stride, const void* a, long a_stride, const void* b,
                             long b_stride, int dtype, const float* dt_bias, const float* a_log, float* out,
                             long out_stride, float* state, long state_stride, const int* seq_slot,
                             const int* seq_start, int n_seqs, int n_heads, int n_kv_heads, int d, int dv,
                             cudaStream_t stream) {
  if (n_seqs == 0) return 0;
  FG_CHECK_ARG(n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0, "fg_delta_scan: %d heads over %d key heads",
               n_heads, n_kv_heads);
  FG_CHECK_ARG(d >= 1 && d <= 256 && dv >= 1, "fg_delta_scan: key size %d (1 to 256), value size %d", d, dv);
  FG_CHECK_ARG(n_heads <= 65535 && n_seqs <= 65535, "fg_delta_scan: too many heads or sequences");
  int rc;
  if (dtype == FG_F32)
    rc = launch_scan<float>(stream, qkv, qkv_stride, (const float*)a, a_stride, (const float*)b, b_stride, dt_bias,
                            a_log, out, out_stride, state, state_stride, seq_slot, seq_start, n_seqs, n_heads,
                            n_kv_heads, d, dv);
  else if (dtype == FG_BF16)
    rc = launch_scan<__nv_bfloat16>(stream, qkv, qkv_stride, (const __nv_bfloat16*)a, a_stride,
                                    (const __nv_bfloat16*)b, b_stride, dt_bias, a_log, out, out_stride, state,
                                    state_stride, seq_slot, seq_start, n_seqs, n_heads, n_kv_heads, d, dv);
  else
    FG_CHECK_ARG(false, "fg_delta_scan: bad dtype %d", dtype);
  if (rc != 0) return rc;
  FG_CHECK_LAUNCH("fg_delta_scan");
  return 0;
}

// ---- the read-out's norm and gate -------------------------------------------------------------
// out[t, h, :] = o[t, h, :] * rsqrt(mean(o[t, h, :]^2) + eps) * w[:] * sigmoid(z[t, h, :]); a warp a
// (token, head), float32 arithmetic, one rounding.
template <typename TZ>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float* o, long o_stride, const TZ* z, long z_stride, const float* __restrict__ w,
                      TZ* __restrict__ out, long out_stride, const int* __restrict__ req, int n_tokens, int n_heads,
                      int dv, float eps) {
  const int item = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (item >= n_tokens * n_heads) return;
  const int t = item / n_heads, h = item - t * n_heads;
  if (req[t] < 0) return;
  const float* src = o + (size_t)t * o_stride + h * dv;
  float ss = 0.f;
  for (int c = lane; c < dv; c += 32) ss = fmaf(src[c], src[c], ss);
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / (float)dv + eps);
  for (int c = lane; c < dv; c += 32) {
    const float gate = 1.f / (1.f + expf(-to_f32<TZ>(z[(size_t)t * z_stride + h * dv + c])));
    out[(size_t)t * out_stride + h * dv + c] = from_f32<TZ>(src[c] * rstd * w[c] * gate);
  }
}

extern "C" int fg_head_norm_gate(const float* o, long o_stride, const void* z, long z_stride, int dtype,
                                 const float* w, void* out, long out_stride, const int* req, int n_tokens,
                                 int n_heads, int dv, float eps, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  const int blocks = (n_tokens * n_heads + 3) / 4;
  if (dtype == FG_F32)
    head_norm_gate_kernel<float><<<blocks, 128, 0, stream>>>(o, o_stride, (const float*)z, z_stride, w, (float*)out,
                                                             out_stride, req, n_tokens, n_heads, dv, eps);
  else if (dtype == FG_BF16)
    head_norm_gate_kernel<__nv_bfloat16><<<blocks, 128, 0, stream>>>(o, o_stride, (const __nv_bfloat16*)z, z_stride, w,
                                                                     (__nv_bfloat16*)out, out_stride, req, n_tokens,
                                                                     n_heads, dv, eps);
  else
    FG_CHECK_ARG(false, "fg_head_norm_gate: bad dtype %d", dtype);
  FG_CHECK_LAUNCH("fg_head_norm_gate");
  return 0;
}
