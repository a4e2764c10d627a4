// The gated delta rule: a matrix state per head that forgets per key channel and is corrected
// towards each new value.  Per head, with q, k unit vectors (q also times d^-1/2), a decay
// g in (0, 1)^d, a step size beta and the value v, in float32 and in this order:
//
//     S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q          (S is [d, dv])
//
// The read-out sees the token's own write.  With R = diag(g) S_old, o = R^T q + u (k . q): both
// sums over the rows of the old state are formed side by side and k . q comes with the token.
//
// A block works on (sequence, head, DELTA_COLS columns of the state): a warp owns one column,
// a lane every 32nd row of it in registers.  Tokens are staged eight at a time through two
// buffers in shared memory: warp w prepares token w of a stage (unit norms, k . q, the decay
// exp(-exp(A) softplus(a + bias)), sigmoid of the step size: all float32) from values it
// fetched into registers while the stage before was computed.  The recurrence runs token by
// token, so prompt portions, single tokens and mixed batches take this kernel and give the
// same numbers however a prompt is cut.  The state of a slot is [heads][dv][d] float32 (a
// column's rows side by side), zero at admission.
#include "common.cuh"

constexpr int DELTA_COLS = 8;    // columns of the state a block (one warp each)
constexpr int DELTA_TOKENS = 8;  // tokens a stage (one warp prepares each)
constexpr int DELTA_THREADS = DELTA_COLS * 32;
static_assert(DELTA_TOKENS == DELTA_COLS, "warp w prepares token w of a stage");

__device__ __forceinline__ float softplus_f32(float z) { return z > 20.f ? z : log1pf(expf(z)); }

template <typename TA, int NR>
__global__ void __launch_bounds__(DELTA_THREADS)
delta_scan_kernel(const float* qkv, long qkv_stride, const TA* a, long a_stride, const TA* b, long b_stride,
                  const float* __restrict__ dt_bias, const float* __restrict__ a_log, float* __restrict__ out,
                  long out_stride, float* __restrict__ state, long state_stride, const int* __restrict__ seq_slot,
                  const int* __restrict__ seq_start, int n_heads, int n_kv_heads, int d, int dv) {
  constexpr int DP = 32 * NR;  // rows, padded
  extern __shared__ float smem[];
  // per buffer: q[TOK][DP], k[TOK][DP], g[TOK][DP], v[TOK][COLS], beta[TOK], kq[TOK]
  constexpr int BUF = DELTA_TOKENS * (3 * DP + DELTA_COLS + 2);
  const int slot = seq_slot[blockIdx.z];
  if (slot < 0) return;
  const int start = seq_start[blockIdx.z], n = seq_start[blockIdx.z + 1] - start;
  if (n <= 0) return;
  const int h = blockIdx.y, hk = h / (n_heads / n_kv_heads);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col0 = blockIdx.x * DELTA_COLS, j = col0 + warp;
  const int q_off = hk * d, k_off = (n_kv_heads + hk) * d, v_off = 2 * n_kv_heads * d + h * dv;
  const float rate = expf(a_log[h]);
  const float q_scale = 1.f / sqrtf((float)d);

  float S[NR];
  float* st = state + (size_t)slot * state_stride + ((size_t)h * dv + j) * d;
#pragma unroll
  for (int i = 0; i < NR; ++i) {
    const int r = lane + 32 * i;
    S[i] = (j < dv && r < d) ? st[r] : 0.f;
  }
  float bias_r[NR];
#pragma unroll
  for (int i = 0; i < NR; ++i) {
    const int r = lane + 32 * i;
    bias_r[i] = r < d ? dt_bias[h * d + r] : 0.f;
  }

  // what warp `warp` fetches for its token of the next stage
  float fq[NR], fk[NR], fa[NR], fv = 0.f, fb = 0.f;
  auto fetch = [&](int stage) {
    const int t = stage * DELTA_TOKENS + warp;
    const bool live = t < n;
    const size_t row = (size_t)(start + (live ? t : 0));
#pragma unroll
    for (int i = 0; i < NR; ++i) {
      const int r = lane + 32 * i;
      const bool ok = live && r < d;
      fq[i] = ok ? qkv[row * qkv_stride + q_off + r] : 0.f;
      fk[i] = ok ? qkv[row * qkv_stride + k_off + r] : 0.f;
      fa[i] = ok ? to_f32<TA>(a[row * a_stride + h * d + r]) : 0.f;
    }
    fv = (live && lane < DELTA_COLS && col0 + lane < dv) ? qkv[row * qkv_stride + v_off + col0 + lane] : 0.f;
    fb = live ? to_f32<TA>(b[row * b_stride + h]) : 0.f;
  };
  auto prepare = [&](float* buf) {
    float* sq = buf + warp * DP;
    float* sk = buf + DELTA_TOKENS * DP + warp * DP;
    float* sg = buf + 2 * DELTA_TOKENS * DP + warp * DP;
    float* sv = buf + 3 * DELTA_TOKENS * DP;
    float* sbeta = sv + DELTA_TOKENS * DELTA_COLS;
    float* skq = sbeta + DELTA_TOKENS;
    float ssq = 0.f, ssk = 0.f;
#pragma unroll
    for (int i = 0; i < NR; ++i) {
      ssq = fmaf(fq[i], fq[i], ssq);
      ssk = fmaf(fk[i], fk[i], ssk);
    }
    ssq = warp_sum(ssq);
    ssk = warp_sum(ssk);
    const float rq = q_scale / sqrtf(ssq + 1e-6f), rk = 1.f / sqrtf(ssk + 1e-6f);
    float kq = 0.f;
#pragma unroll
    for (int i = 0; i < NR; ++i) {
      const float qn = fq[i] * rq, kn = fk[i] * rk;
      kq = fmaf(qn, kn, kq);
      sq[lane + 32 * i] = qn;
      sk[lane + 32 * i] = kn;
      sg[lane + 32 * i] = expf(-rate * softplus_f32(fa[i] + bias_r[i]));
    }
    kq = warp_sum(kq);
    if (lane < DELTA_COLS) sv[warp * DELTA_COLS + lane] = fv;
    if (lane == 0) {
      sbeta[warp] = 1.f / (1.f + expf(-fb));
      skq[warp] = kq;
    }
  };

  const int n_stages = (n + DELTA_TOKENS - 1) / DELTA_TOKENS;
  fetch(0);
  for (int stage = 0; stage < n_stages; ++stage) {
    float* buf = smem + (stage & 1) * BUF;
    prepare(buf);
    __syncthreads();
    if (stage + 1 < n_stages) fetch(stage + 1);
    if (j < dv) {
      const float* sq = buf;
      const float* sk = buf + DELTA_TOKENS * DP;
      const float* sg = buf + 2 * DELTA_TOKENS * DP;
      const float* sv = buf + 3 * DELTA_TOKENS * DP;
      const float* sbeta = sv + DELTA_TOKENS * DELTA_COLS;
      const float* skq = sbeta + DELTA_TOKENS;
      const int n_tok = min(DELTA_TOKENS, n - stage * DELTA_TOKENS);
      for (int tt = 0; tt < n_tok; ++tt) {
        float kr[NR];
        float rk_sum = 0.f, rq_sum = 0.f;
#pragma unroll
        for (int i = 0; i < NR; ++i) {
          const int r = lane + 32 * i;
          kr[i] = sk[tt * DP + r];
          S[i] *= sg[tt * DP + r];
          rk_sum = fmaf(S[i], kr[i], rk_sum);
          rq_sum = fmaf(S[i], sq[tt * DP + r], rq_sum);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          rk_sum += __shfl_xor_sync(0xffffffffu, rk_sum, o);
          rq_sum += __shfl_xor_sync(0xffffffffu, rq_sum, o);
        }
        const float u = sbeta[tt] * (sv[tt * DELTA_COLS + warp] - rk_sum);
#pragma unroll
        for (int i = 0; i < NR; ++i) S[i] = fmaf(kr[i], u, S[i]);
        if (lane == 0) out[(size_t)(start + stage * DELTA_TOKENS + tt) * out_stride + h * dv + j] = fmaf(u, skq[tt], rq_sum);
      }
    }
  }
  if (j < dv) {
#pragma unroll
    for (int i = 0; i < NR; ++i) {
      const int r = lane + 32 * i;
      if (r < d) st[r] = S[i];
    }
  }
}

template <typename TA>
static int launch_scan(int nr, dim3 grid, cudaStream_t stream, const float* qkv, long qkv_stride, const TA* a,
                       long a_stride, const TA* b, long b_stride, const float* dt_bias, const float* a_log, float* out,
                       long out_stride, float* state, long state_stride, const int* seq_slot, const int* seq_start,
                       int n_heads, int n_kv_heads, int d, int dv) {
#define CASE(NR)                                                                                               \
  case NR: {                                                                                                   \
    const size_t smem = 2 * DELTA_TOKENS * (3 * 32 * NR + DELTA_COLS + 2) * sizeof(float);                      \
    auto kern = delta_scan_kernel<TA, NR>;                                                                      \
    if (smem > 48 * 1024) {                                                                                     \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
      FG_CHECK_ARG(e == cudaSuccess, "fg_delta_scan: shared memory: %s", cudaGetErrorString(e));                \
    }                                                                                                           \
    kern<<<grid, DELTA_THREADS, smem, stream>>>(qkv, qkv_stride, a, a_stride, b, b_stride, dt_bias, a_log, out, \
                                                out_stride, state, state_stride, seq_slot, seq_start, n_heads,  \
                                                n_kv_heads, d, dv);                                             \
  } break
  switch (nr) {
    CASE(1); CASE(2); CASE(3); CASE(4); CASE(5); CASE(6); CASE(7); CASE(8);
    default: FG_CHECK_ARG(false, "fg_delta_scan: key size %d (up to 256)", d);
  }
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
  dim3 grid((dv + DELTA_COLS - 1) / DELTA_COLS, n_heads, n_seqs);
  const int nr = (d + 31) / 32;
  int rc;
  if (dtype == FG_F32)
    rc = launch_scan<float>(nr, grid, stream, qkv, qkv_stride, (const float*)a, a_stride, (const float*)b, b_stride,
                            dt_bias, a_log, out, out_stride, state, state_stride, seq_slot, seq_start, n_heads,
                            n_kv_heads, d, dv);
  else if (dtype == FG_BF16)
    rc = launch_scan<__nv_bfloat16>(nr, grid, stream, qkv, qkv_stride, (const __nv_bfloat16*)a, a_stride,
                                    (const __nv_bfloat16*)b, b_stride, dt_bias, a_log, out, out_stride, state,
                                    state_stride, seq_slot, seq_start, n_heads, n_kv_heads, d, dv);
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
