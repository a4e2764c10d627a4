// The gated delta rule: a matrix state per head that forgets per key channel and is corrected
// towards each new value.  Per head, with q, k unit vectors (q also times d^-1/2), a decay
// g in (0, 1)^d, a step size beta and the value v, in float32 and in this order:
//
//     S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q          (S is [d, dv])
//
// The read-out sees the token's own write.  With R = diag(g) S_old, o = R^T q + u (k . q): both
// sums over the rows of the old state are formed side by side and k . q comes with the token.
//
// Two kernels.  The first prepares every token by itself (a warp a (token, head)): unit norms,
// k . q, the decay exp(-exp(A) softplus(a + bias)) per key channel, sigmoid of the step size, all
// float32, written as padded float32 rows that the second can copy in 16-byte words:
//   qn, kn [T, kv heads, DP]; rec [T, heads, DP + 4] = the decay's DP numbers, beta, k . q, 0, 0;
//   vp [T, heads, DVP]        (DP: d rounded up to the kernel's row count, DVP: dv up to a multiple of 4)
// The second runs the recurrence, which is a chain from token to token whose length, not the
// arithmetic, sets the time, so nothing else is left in it.  A block of eight warps works on
// (sequence, head, a run of the state's columns).  A column's rows are spread over LPC lanes, RPL
// rows a lane in registers (in runs of four: a lane reads its part of k, g and q as 16-byte words);
// a warp holds 32 / LPC columns and the sums over a column's rows end in log2(LPC) exchanges.
// (Measured at key size 64, 2,048 tokens: 16 lanes x 4 rows 536 us, 32 x 4 591 us, 8 x 8 601 us, 2 x 32 669 us.)
// Tokens arrive eight at a time through a ring of cp.async buffers, several stages ahead; whole
// stages run unrolled, so that a token's operands are read while the one before it is reduced.
// The recurrence runs token by token, so prompt portions, single tokens and mixed batches take
// these kernels and give the same numbers however a prompt is cut.  The state of a slot is
// [heads][dv][d] float32 (a column's rows side by side), zero at admission.
#include "common.cuh"

constexpr int DELTA_WARPS = 8;
constexpr int DELTA_TOKENS = 8;  // tokens a stage
constexpr int DELTA_STAGES = 4;  // buffers of the ring
constexpr int DELTA_THREADS = DELTA_WARPS * 32;
constexpr int DELTA_MAX_NRP = 8;  // key sizes up to 256

__device__ __forceinline__ float softplus_f32(float z) { return z > 20.f ? z : log1pf(expf(z)); }

template <typename TA>
__global__ void __launch_bounds__(128)
delta_prepare_kernel(const float* qkv, long qkv_stride, const TA* a, long a_stride, const TA* b, long b_stride,
                     const float* __restrict__ dt_bias, const float* __restrict__ a_log, const int* __restrict__ req,
                     float* __restrict__ qn, float* __restrict__ kn, float* __restrict__ rec, float* __restrict__ vp,
                     int n_tokens, int n_heads, int n_kv_heads, int d, int dv, int DP, int DVP) {
  const int item = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (item >= n_tokens * n_heads) return;
  const int t = item / n_heads, h = item - t * n_heads;
  if (req[t] < 0) return;
  const int group = n_heads / n_kv_heads, hk = h / group;
  const float* row = qkv + (size_t)t * qkv_stride;
  const int q_off = hk * d, k_off = (n_kv_heads + hk) * d, v_off = 2 * n_kv_heads * d + h * dv;
  const int nrp = DP / 32;
  float fq[DELTA_MAX_NRP], fk[DELTA_MAX_NRP];
  float ssq = 0.f, ssk = 0.f;
#pragma unroll
  for (int i = 0; i < DELTA_MAX_NRP; ++i) {
    const int r = lane + 32 * i;
    const bool ok = i < nrp && r < d;
    fq[i] = ok ? row[q_off + r] : 0.f;
    fk[i] = ok ? row[k_off + r] : 0.f;
    ssq = fmaf(fq[i], fq[i], ssq);
    ssk = fmaf(fk[i], fk[i], ssk);
  }
  ssq = warp_sum(ssq);
  ssk = warp_sum(ssk);
  const float rq = (1.f / sqrtf((float)d)) / sqrtf(ssq + 1e-6f), rk = 1.f / sqrtf(ssk + 1e-6f);
  const float rate = expf(a_log[h]);
  float* rec_row = rec + ((size_t)t * n_heads + h) * (DP + 4);
  const bool first = h == hk * group;  // the group's first head writes the group's q and k
  float* qn_row = qn + ((size_t)t * n_kv_heads + hk) * DP;
  float* kn_row = kn + ((size_t)t * n_kv_heads + hk) * DP;
  float kq = 0.f;
#pragma unroll
  for (int i = 0; i < DELTA_MAX_NRP; ++i) {
    const int r = lane + 32 * i;
    if (i < nrp) {
      const float qv = fq[i] * rq, kv = fk[i] * rk;
      kq = fmaf(qv, kv, kq);
      if (first) {
        qn_row[r] = qv;
        kn_row[r] = kv;
      }
      // rows beyond d: k and q are zero there, and so is the state
      rec_row[r] = r < d ? expf(-rate * softplus_f32(to_f32<TA>(a[(size_t)t * a_stride + h * d + r]) + dt_bias[h * d + r])) : 0.f;
    }
  }
  kq = warp_sum(kq);
  if (lane < 4) {
    const float beta = 1.f / (1.f + expf(-to_f32<TA>(b[(size_t)t * b_stride + h])));
    rec_row[DP + lane] = lane == 0 ? beta : (lane == 1 ? kq : 0.f);
  }
  float* vp_row = vp + ((size_t)t * n_heads + h) * DVP;
  for (int c = lane; c < DVP; c += 32) vp_row[c] = c < dv ? row[v_off + c] : 0.f;
}

__device__ __forceinline__ void delta_copy16(float* dst, const float* src, bool pred) {
  const int bytes = pred ? 16 : 0;  // 0: the 16 bytes are zero-filled, nothing is read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src),
               "r"(bytes) : "memory");
}

template <int LPC, int RPL>
__global__ void __launch_bounds__(DELTA_THREADS)
delta_scan_kernel(const float* __restrict__ qn, const float* __restrict__ kn, const float* __restrict__ rec,
                  const float* __restrict__ vp, float* __restrict__ out, long out_stride, float* __restrict__ state,
                  long state_stride, const int* __restrict__ seq_slot, const int* __restrict__ seq_start, int n_heads,
                  int n_kv_heads, int d, int dv, int DVP) {
  constexpr int DP = LPC * RPL;            // rows, padded
  constexpr int CPW = 32 / LPC;            // columns a warp
  constexpr int COLS = DELTA_WARPS * CPW;  // columns a block
  constexpr int REC = DP + 4;
  static_assert(DP % 32 == 0 && RPL % 4 == 0 && COLS % 4 == 0, "rows in runs of four, a multiple of 32 in all");
  extern __shared__ __align__(16) float smem[];
  // per token of a buffer: q[DP], k[DP], rec[DP + 4] (g, beta, k . q), v[COLS]
  constexpr int TOKF = 3 * DP + 4 + COLS;
  constexpr int BUF = DELTA_TOKENS * TOKF;
  constexpr int CHUNKS = TOKF / 4;  // 16-byte words a token
  const int slot = seq_slot[blockIdx.z];
  if (slot < 0) return;
  const int start = seq_start[blockIdx.z], n = seq_start[blockIdx.z + 1] - start;
  if (n <= 0) return;
  const int h = blockIdx.y, hk = h / (n_heads / n_kv_heads);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane % LPC, cw = warp * CPW + lane / LPC;  // the lane's part of a column; its column in the block
  const int col0 = blockIdx.x * COLS, j = col0 + cw;
  const bool live_col = j < dv;

  // the lane's rows: 4 (sub + LPC jj) + e for jj < RPL / 4, e < 4
  float S[RPL];
  float* st = state + (size_t)slot * state_stride + ((size_t)h * dv + (live_col ? j : 0)) * d;
#pragma unroll
  for (int i = 0; i < RPL; ++i) {
    const int r = 4 * (sub + LPC * (i >> 2)) + (i & 3);
    S[i] = (live_col && r < d) ? st[r] : 0.f;
  }

  // the copies of one stage: every thread takes 16-byte words of the stage's tokens in turn
  auto issue = [&](int stage) {
    float* buf = smem + (stage % DELTA_STAGES) * BUF;
    for (int c = threadIdx.x; c < DELTA_TOKENS * CHUNKS; c += DELTA_THREADS) {
      const int tt = c / CHUNKS, w = c - tt * CHUNKS, t = stage * DELTA_TOKENS + tt;
      const bool live = t < n;
      const size_t tok = (size_t)(start + (live ? t : 0));
      const float* src;
      bool ok = live;
      if (w < DP / 4) {
        src = qn + (tok * n_kv_heads + hk) * DP + 4 * w;
      } else if (w < 2 * (DP / 4)) {
        src = kn + (tok * n_kv_heads + hk) * DP + 4 * (w - DP / 4);
      } else if (w < 2 * (DP / 4) + REC / 4) {
        src = rec + (tok * n_heads + h) * REC + 4 * (w - 2 * (DP / 4));
      } else {
        const int c4 = 4 * (w - 2 * (DP / 4) - REC / 4);
        ok = live && col0 + c4 < DVP;
        src = vp + (tok * n_heads + h) * DVP + (ok ? col0 + c4 : 0);
      }
      delta_copy16(buf + tt * TOKF + 4 * w, src, ok);
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };

  // one token of the recurrence, its operands at `tokp`
  auto step = [&](const float* tokp, size_t out_row) {
    const float4* sq = reinterpret_cast<const float4*>(tokp);
    const float4* sk = reinterpret_cast<const float4*>(tokp + DP);
    const float4* sg = reinterpret_cast<const float4*>(tokp + 2 * DP);
    const float beta = tokp[3 * DP], kq = tokp[3 * DP + 1], v = tokp[3 * DP + 4 + cw];
    float kr[RPL];
    float rk2[4] = {0.f, 0.f, 0.f, 0.f}, rq2[4] = {0.f, 0.f, 0.f, 0.f};  // four chains a sum: a lane's rows are many
#pragma unroll
    for (int jj = 0; jj < RPL / 4; ++jj) {
      const float4 kv = sk[sub + LPC * jj], gv = sg[sub + LPC * jj], qv = sq[sub + LPC * jj];
      const float ke[4] = {kv.x, kv.y, kv.z, kv.w}, ge[4] = {gv.x, gv.y, gv.z, gv.w}, qe[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = 4 * jj + e;
        kr[i] = ke[e];
        S[i] *= ge[e];
        rk2[e] = fmaf(S[i], ke[e], rk2[e]);
        rq2[e] = fmaf(S[i], qe[e], rq2[e]);
      }
    }
    float rk_sum = (rk2[0] + rk2[1]) + (rk2[2] + rk2[3]), rq_sum = (rq2[0] + rq2[1]) + (rq2[2] + rq2[3]);
#pragma unroll
    for (int o = LPC / 2; o > 0; o >>= 1) {
      rk_sum += __shfl_xor_sync(0xffffffffu, rk_sum, o);
      rq_sum += __shfl_xor_sync(0xffffffffu, rq_sum, o);
    }
    const float u = beta * (v - rk_sum);
#pragma unroll
    for (int i = 0; i < RPL; ++i) S[i] = fmaf(kr[i], u, S[i]);
    if (sub == 0 && live_col) out[out_row * out_stride + h * dv + j] = fmaf(u, kq, rq_sum);
  };

  const int n_stages = (n + DELTA_TOKENS - 1) / DELTA_TOKENS;
#pragma unroll
  for (int s = 0; s < DELTA_STAGES - 1; ++s) {
    if (s < n_stages) issue(s);
    else asm volatile("cp.async.commit_group;\n" ::: "memory");
  }
  for (int stage = 0; stage < n_stages; ++stage) {
    // this stage's copies have landed (the groups after it may be in flight), for every thread
    asm volatile("cp.async.wait_group %0;\n" ::"n"(DELTA_STAGES - 2) : "memory");
    __syncthreads();
    // the buffer of the stage before this one is free now: fill it with the stage three ahead
    if (stage + DELTA_STAGES - 1 < n_stages) issue(stage + DELTA_STAGES - 1);
    else asm volatile("cp.async.commit_group;\n" ::: "memory");
    const float* buf = smem + (stage % DELTA_STAGES) * BUF;
    const int n_tok = min(DELTA_TOKENS, n - stage * DELTA_TOKENS);
    const size_t row0 = (size_t)start + (size_t)stage * DELTA_TOKENS;
    if (n_tok == DELTA_TOKENS) {
#pragma unroll
      for (int tt = 0; tt < DELTA_TOKENS; ++tt) step(buf + tt * TOKF, row0 + tt);
    } else {
      for (int tt = 0; tt < n_tok; ++tt) step(buf + tt * TOKF, row0 + tt);
    }
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");
  if (live_col) {
#pragma unroll
    for (int i = 0; i < RPL; ++i) {
      const int r = 4 * (sub + LPC * (i >> 2)) + (i & 3);
      if (r < d) st[r] = S[i];
    }
  }
}

// rows of the prepared arrays for key size d (the row count of the kernel that takes it)
static int delta_rows(int d) { return d <= 32 ? 32 : d <= 64 ? 64 : d <= 128 ? 128 : 256; }

static int launch_scan(cudaStream_t stream, const float* qn, const float* kn, const float* rec, const float* vp,
                       float* out, long out_stride, float* state, long state_stride, const int* seq_slot,
                       const int* seq_start, int n_seqs, int n_heads, int n_kv_heads, int d, int dv, int DVP) {
#define CASE(LPC, RPL)                                                                                         \
  {                                                                                                            \
    constexpr int COLS = DELTA_WARPS * (32 / LPC);                                                             \
    const size_t smem = (size_t)DELTA_STAGES * DELTA_TOKENS * (3 * LPC * RPL + 4 + COLS) * sizeof(float);       \
    auto kern = delta_scan_kernel<LPC, RPL>;                                                                    \
    if (smem > 48 * 1024) {                                                                                     \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
      FG_CHECK_ARG(e == cudaSuccess, "fg_delta_scan: shared memory: %s", cudaGetErrorString(e));                \
    }                                                                                                           \
    dim3 grid((dv + COLS - 1) / COLS, n_heads, n_seqs);                                                         \
    kern<<<grid, DELTA_THREADS, smem, stream>>>(qn, kn, rec, vp, out, out_stride, state, state_stride, seq_slot, \
                                                seq_start, n_heads, n_kv_heads, d, dv, DVP);                    \
  }
  if (d <= 32) CASE(8, 4)
  else if (d <= 64) CASE(16, 4)
  else if (d <= 128) CASE(16, 8)
  else CASE(16, 16)
#undef CASE
  return 0;
}

// floats of the scratch that fg_delta_scan needs for `n_tokens` tokens
extern "C" long fg_delta_scan_scratch_floats(int n_tokens, int n_heads, int n_kv_heads, int d, int dv) {
  const long DP = delta_rows(d), DVP = (dv + 3) / 4 * 4;
  return (long)n_tokens * (2 * n_kv_heads * DP + n_heads * (DP + 4) + n_heads * DVP);
}

// qkv: float32 [T, q (kv heads x d) | k (kv heads x d) | v (heads x dv)], the convolutions' outputs.
// a: [T, heads x d] decay logits and b: [T, .] step-size logits (column h of row t at b[t * b_stride + h]),
// both of `dtype`.  dt_bias: float32 [heads x d]; a_log: float32 [heads].  out: float32 [T, heads x dv].
// state: float32 [slots, state_stride], a slot's first heads * dv * d numbers.
extern "C" int fg_delta_scan(const float* qkv, long qkv_stride, const void* a, long a_stride, const void* b,
                             long b_stride, int dtype, const float* dt_bias, const float* a_log, float* out,
                             long out_stride, float* state, long state_stride, const int* seq_slot,
                             const int* seq_start, int n_seqs, const int* req, int n_tokens, float* scratch,
                             int n_heads, int n_kv_heads, int d, int dv, cudaStream_t stream) {
  if (n_seqs == 0 || n_tokens == 0) return 0;
  FG_CHECK_ARG(n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0, "fg_delta_scan: %d heads over %d key heads",
               n_heads, n_kv_heads);
  FG_CHECK_ARG(d >= 1 && d <= 256 && dv >= 1, "fg_delta_scan: key size %d (1 to 256), value size %d", d, dv);
  FG_CHECK_ARG(n_heads <= 65535 && n_seqs <= 65535, "fg_delta_scan: too many heads or sequences");
  FG_CHECK_ARG(scratch != nullptr && ((uintptr_t)scratch & 15) == 0, "fg_delta_scan: scratch missing or unaligned");
  const int DP = delta_rows(d), DVP = (dv + 3) / 4 * 4;
  float* qn = scratch;
  float* kn = qn + (size_t)n_tokens * n_kv_heads * DP;
  float* rec = kn + (size_t)n_tokens * n_kv_heads * DP;
  float* vp = rec + (size_t)n_tokens * n_heads * (DP + 4);
  const int blocks = (int)(((long)n_tokens * n_heads + 3) / 4);
  if (dtype == FG_F32)
    delta_prepare_kernel<float><<<blocks, 128, 0, stream>>>(qkv, qkv_stride, (const float*)a, a_stride, (const float*)b,
                                                            b_stride, dt_bias, a_log, req, qn, kn, rec, vp, n_tokens,
                                                            n_heads, n_kv_heads, d, dv, DP, DVP);
  else if (dtype == FG_BF16)
    delta_prepare_kernel<__nv_bfloat16><<<blocks, 128, 0, stream>>>(
        qkv, qkv_stride, (const __nv_bfloat16*)a, a_stride, (const __nv_bfloat16*)b, b_stride, dt_bias, a_log, req, qn,
        kn, rec, vp, n_tokens, n_heads, n_kv_heads, d, dv, DP, DVP);
  else
    FG_CHECK_ARG(false, "fg_delta_scan: bad dtype %d", dtype);
  FG_CHECK_LAUNCH("fg_delta_scan (prepare)");
  const int rc = launch_scan(stream, qn, kn, rec, vp, out, out_stride, state, state_stride, seq_slot, seq_start, n_seqs,
                             n_heads, n_kv_heads, d, dv, DVP);
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
