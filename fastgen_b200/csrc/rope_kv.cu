// Rotary position encoding of queries and keys fused with the write of keys
// and values into their cache pages.
//
// Replaces apply_rope x2 (fastgen/kernels/rope.py:57-89) and paged_memcpy x2
// (fastgen/kernels/paged_memcpy.py:57-76) of fastgen/forward.py:449-460.
//   angle = float(pos) * freqs[j]                      (float32 product)
//   x[2j]   = re * cos(angle) - im * sin(angle)
//   x[2j+1] = im * cos(angle) + re * sin(angle)        (precise sinf/cosf)
// Queries are rotated in place.  Keys are rotated and stored, values copied, to
//   slot = block_table[req, pos / page] * page + pos % page
// of a pool laid out [n_pages, n_kv_heads, page, head_dim], so that the
// [page, head_dim] tile of one head is contiguous.
// Tokens whose request index is negative are padding: nothing is written.
#include "common.cuh"

constexpr int ROPE_THREADS = 128;

// An adjacent pair as one access (4 bytes of bfloat16, 8 of float32) when the
// launch found every pair aligned, else as two.
template <typename T>
__device__ __forceinline__ float2 load_pair(const T* p, bool vec);
template <>
__device__ __forceinline__ float2 load_pair<float>(const float* p, bool vec) {
  if (vec) return *reinterpret_cast<const float2*>(p);
  return make_float2(p[0], p[1]);
}
template <>
__device__ __forceinline__ float2 load_pair<__nv_bfloat16>(const __nv_bfloat16* p, bool vec) {
  if (vec) return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
  return make_float2(__bfloat162float(p[0]), __bfloat162float(p[1]));
}
template <typename T>
__device__ __forceinline__ void store_pair(T* p, float2 v, bool vec);
template <>
__device__ __forceinline__ void store_pair<float>(float* p, float2 v, bool vec) {
  if (vec) *reinterpret_cast<float2*>(p) = v;
  else { p[0] = v.x; p[1] = v.y; }
}
template <>
__device__ __forceinline__ void store_pair<__nv_bfloat16>(__nv_bfloat16* p, float2 v, bool vec) {
  if (vec) *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v.x, v.y);
  else { p[0] = __float2bfloat16_rn(v.x); p[1] = __float2bfloat16_rn(v.y); }
}

// A thread owns one pair index j of one token: it computes sin and cos of the
// token's angle for j once and walks the heads (queries, then keys, then values)
// that its block is given: blockIdx.x is the token, blockIdx.y a slice of the
// heads (few tokens get more slices, so that the GPU is still filled).
template <typename T>
__global__ void __launch_bounds__(ROPE_THREADS)
rope_kv_kernel(T* __restrict__ q, int q_stride, const T* __restrict__ k, int k_stride,
               const T* __restrict__ v, int v_stride, const int* __restrict__ pos,
               const int* __restrict__ req, const float* __restrict__ freqs,
               const float* __restrict__ v_freqs, T* __restrict__ k_pages, T* __restrict__ v_pages, const int* __restrict__ block_table, int table_width,
               int page_size, int n_pages, int n_heads, int n_kv_heads, int head_dim, int* status,
               bool vec, int heads_per_block, const float* rstd, const float* __restrict__ qn_w,
               const float* __restrict__ kn_w, int rstd_heads) {
  const int t = blockIdx.x;
  const int r = req[t];
  if (r < 0) return;
  const int half = head_dim >> 1;
  const int lanes = ROPE_THREADS / half > 0 ? ROPE_THREADS / half : 1;  // heads walked side by side
  const int j = threadIdx.x % half, lane_head = threadIdx.x / half;
  if (lane_head >= lanes) return;
  const int p = pos[t];
  const int n_kv = (k != nullptr) ? n_kv_heads : 0;
  const int total = n_heads + 2 * n_kv;  // heads in the order q..., k..., v...
  const int h_end = min(total, (int)(blockIdx.y + 1) * heads_per_block);
  float s = 0.f, c = 1.f, sv = 0.f, cv = 1.f;
  // queries and keys normed over their whole projection: the token's two factors; with rstd_heads
  // (= query heads + key heads) every head of the token has a factor of its own
  const float rq = rstd && !rstd_heads ? rstd[2 * t] : 1.f, rk = rstd && !rstd_heads ? rstd[2 * t + 1] : 1.f;
  if (freqs != nullptr) sincosf((float)p * freqs[j], &s, &c);
  if (v_freqs != nullptr) sincosf((float)p * v_freqs[j], &sv, &cv);
  size_t slot = 0;
  bool have_slot = false;
  for (int h = blockIdx.y * heads_per_block + lane_head; h < h_end; h += lanes) {
    if (h < n_heads) {
      T* x = q + (size_t)t * q_stride + h * head_dim + 2 * j;
      float2 val = load_pair<T>(x, vec);
      if (rstd != nullptr) {
        const float f = rstd_heads ? rstd[(size_t)t * rstd_heads + h] : rq;
        val.x *= f * (qn_w ? qn_w[h * head_dim + 2 * j] : 1.f);
        val.y *= f * (qn_w ? qn_w[h * head_dim + 2 * j + 1] : 1.f);
      }
      store_pair<T>(x, make_float2(val.x * c - val.y * s, val.y * c + val.x * s), vec);
      continue;
    }
    if (!have_slot) {
      const int logical = p / page_size;
      const int page = (logical < table_width) ? block_table[(size_t)r * table_width + logical] : -1;
      if (page < 0 || page >= n_pages) {
        if (status) atomicOr(status, FG_STATUS_BAD_PAGE);
        return;
      }
      slot = (size_t)page * n_kv_heads * page_size + (p - logical * page_size);
      have_slot = true;
    }
    const bool is_v = h >= n_heads + n_kv;
    const int g = h - n_heads - (is_v ? n_kv : 0);
    const size_t dst = (slot + (size_t)g * page_size) * head_dim + 2 * j;
    if (is_v) {
      const T* x = v + (size_t)t * v_stride + g * head_dim + 2 * j;
      const float2 val = load_pair<T>(x, vec);
      // values turn by their own table when they have one (cv = 1, sv = 0: a copy)
      store_pair<T>(v_pages + dst, make_float2(val.x * cv - val.y * sv, val.y * cv + val.x * sv), vec);
    } else {
      const T* x = k + (size_t)t * k_stride + g * head_dim + 2 * j;
      float2 val = load_pair<T>(x, vec);
      if (rstd != nullptr) {
        const float f = rstd_heads ? rstd[(size_t)t * rstd_heads + n_heads + g] : rk;
        val.x *= f * (kn_w ? kn_w[g * head_dim + 2 * j] : 1.f);
        val.y *= f * (kn_w ? kn_w[g * head_dim + 2 * j + 1] : 1.f);
      }
      store_pair<T>(k_pages + dst, make_float2(val.x * c - val.y * s, val.y * c + val.x * s), vec);
    }
  }
}

// bfloat16 with 16-byte accesses: a thread owns four adjacent pairs (8 elements) of one
// token, computes their four angles once and walks the heads, several heads in flight.
// Needs head_dim % 8 == 0 and 16-byte aligned rows.
constexpr int ROPE_UNROLL = 4;

__global__ void __launch_bounds__(ROPE_THREADS)
rope_kv_bf16x8_kernel(__nv_bfloat16* __restrict__ q, int q_stride, const __nv_bfloat16* __restrict__ k, int k_stride,
                      const __nv_bfloat16* __restrict__ v, int v_stride, const int* __restrict__ pos,
                      const int* __restrict__ req, const float* __restrict__ freqs,
                      const float* __restrict__ v_freqs, __nv_bfloat16* __restrict__ k_pages, __nv_bfloat16* __restrict__ v_pages,
                      const int* __restrict__ block_table, int table_width, int page_size, int n_pages,
                      int n_heads, int n_kv_heads, int head_dim, int* status, int heads_per_block,
                      const float* rstd, const float* __restrict__ qn_w, const float* __restrict__ kn_w,
                      int rstd_heads) {
  const int t = blockIdx.x;
  const int r = req[t];
  if (r < 0) return;
  const int pieces = head_dim >> 3;                 // 16-byte pieces a head
  const int lanes = ROPE_THREADS / pieces;          // heads walked side by side
  const int piece = threadIdx.x % pieces, lane_head = threadIdx.x / pieces;
  if (lane_head >= lanes) return;
  const int p = pos[t];
  const int n_kv = (k != nullptr) ? n_kv_heads : 0;
  const int total = n_heads + 2 * n_kv;  // heads in the order q..., k..., v...
  const int h_end = min(total, (int)(blockIdx.y + 1) * heads_per_block);
  float sn[4], cs[4], snv[4], csv[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    sn[i] = snv[i] = 0.f;
    cs[i] = csv[i] = 1.f;
    if (freqs != nullptr) sincosf((float)p * freqs[piece * 4 + i], &sn[i], &cs[i]);
    if (v_freqs != nullptr) sincosf((float)p * v_freqs[piece * 4 + i], &snv[i], &csv[i]);
  }
  size_t slot = 0;
  if (n_kv > 0) {
    const int logical = p / page_size;
    const int page = (logical < table_width) ? block_table[(size_t)r * table_width + logical] : -1;
    if (page < 0 || page >= n_pages) {
      if (status) atomicOr(status, FG_STATUS_BAD_PAGE);
      return;
    }
    slot = (size_t)page * n_kv_heads * page_size + (p - logical * page_size);
  }
  const float rq = rstd && !rstd_heads ? rstd[2 * t] : 1.f, rk = rstd && !rstd_heads ? rstd[2 * t + 1] : 1.f;
  // nw: the eight norm weights of this piece of the head (null: ones), r: the factor of the token
  // (or of this head of the token)
  auto rotate = [&](uint4 raw, const float* nw, float r) {
    __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 val = __bfloat1622float2(h2[i]);
      if (rstd != nullptr) {
        val.x *= r * (nw ? nw[2 * i] : 1.f);
        val.y *= r * (nw ? nw[2 * i + 1] : 1.f);
      }
      h2[i] = __floats2bfloat162_rn(val.x * cs[i] - val.y * sn[i], val.y * cs[i] + val.x * sn[i]);
    }
    return raw;
  };
  auto rotate_v = [&](uint4 raw) {
    __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 val = __bfloat1622float2(h2[i]);
      h2[i] = __floats2bfloat162_rn(val.x * csv[i] - val.y * snv[i], val.y * csv[i] + val.x * snv[i]);
    }
    return raw;
  };
  for (int h0 = blockIdx.y * heads_per_block + lane_head; h0 < h_end; h0 += lanes * ROPE_UNROLL) {
    uint4 raw[ROPE_UNROLL];
    // the loads of several heads first, then their rotations and stores
#pragma unroll
    for (int u = 0; u < ROPE_UNROLL; ++u) {
      const int h = h0 + u * lanes;
      if (h >= h_end) continue;
      const __nv_bfloat16* src;
      if (h < n_heads) src = q + (size_t)t * q_stride + h * head_dim;
      else if (h < n_heads + n_kv) src = k + (size_t)t * k_stride + (h - n_heads) * head_dim;
      else src = v + (size_t)t * v_stride + (h - n_heads - n_kv) * head_dim;
      raw[u] = *reinterpret_cast<const uint4*>(src + piece * 8);
    }
#pragma unroll
    for (int u = 0; u < ROPE_UNROLL; ++u) {
      const int h = h0 + u * lanes;
      if (h >= h_end) continue;
      if (h < n_heads) {
        *reinterpret_cast<uint4*>(q + (size_t)t * q_stride + h * head_dim + piece * 8) =
            rotate(raw[u], qn_w ? qn_w + h * head_dim + piece * 8 : nullptr,
                   rstd_heads ? rstd[(size_t)t * rstd_heads + h] : rq);
        continue;
      }
      const bool is_v = h >= n_heads + n_kv;
      const int g = h - n_heads - (is_v ? n_kv : 0);
      const size_t dst = (slot + (size_t)g * page_size) * head_dim + piece * 8;
      *reinterpret_cast<uint4*>((is_v ? v_pages : k_pages) + dst) =
          is_v ? (v_freqs != nullptr ? rotate_v(raw[u]) : raw[u])
               : rotate(raw[u], kn_w ? kn_w + g * head_dim + piece * 8 : nullptr,
                        rstd_heads ? rstd[(size_t)t * rstd_heads + n_heads + g] : rk);
    }
  }
}

// The factors of a norm of queries and keys over their whole projection: for every token
// out[2t] = rsqrt(sum of squares of its nq query columns / count_q + eps) and out[2t+1] the same of
// its nk key columns (count: the columns that are not padding; padding columns hold zeros).
template <typename T>
__global__ void __launch_bounds__(128)
qk_rstd_kernel(const T* q, long q_stride, int nq, float count_q, const T* k, long k_stride, int nk, float count_k,
               const int* __restrict__ req, float eps, float* __restrict__ out) {
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  if (req[t] < 0) return;
  float sq = 0.f, sk = 0.f;
  for (int d = threadIdx.x; d < nq; d += blockDim.x) {
    const float v = to_f32<T>(q[(size_t)t * q_stride + d]);
    sq = fmaf(v, v, sq);
  }
  for (int d = threadIdx.x; d < nk; d += blockDim.x) {
    const float v = to_f32<T>(k[(size_t)t * k_stride + d]);
    sk = fmaf(v, v, sk);
  }
  sq = block_sum(sq, scratch);
  sk = block_sum(sk, scratch);
  if (threadIdx.x == 0) {
    out[2 * t] = rsqrtf(sq / count_q + eps);
    out[2 * t + 1] = nk > 0 ? rsqrtf(sk / count_k + eps) : 1.f;
  }
}

extern "C" int fg_qk_rstd(const void* q, long q_stride, int nq, int count_q, const void* k, long k_stride, int nk,
                          int count_k, int dtype, const int* req, float eps, float* out, int n_tokens,
                          cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  FG_CHECK_ARG(nq > 0 && count_q > 0 && (nk == 0 || (k != nullptr && count_k > 0)), "fg_qk_rstd: bad sizes");
  if (dtype == FG_F32)
    qk_rstd_kernel<float><<<n_tokens, 128, 0, stream>>>((const float*)q, q_stride, nq, (float)count_q, (const float*)k,
                                                        k_stride, nk, (float)count_k, req, eps, out);
  else
    qk_rstd_kernel<__nv_bfloat16><<<n_tokens, 128, 0, stream>>>((const __nv_bfloat16*)q, q_stride, nq, (float)count_q,
                                                                (const __nv_bfloat16*)k, k_stride, nk, (float)count_k,
                                                                req, eps, out);
  FG_CHECK_LAUNCH("fg_qk_rstd");
  return 0;
}

// Per-head factors of queries and keys: out[t, h] for the token's query heads, then its key heads.
// With `norm` a head's factor is rsqrt(mean of its first `real_dim` columns squared + eps) (an RMS norm
// per head; the head's padding columns hold zeros); with temp_every > 0 a query head's factor is also
// multiplied by 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1) at position p: a query temperature
// that grows in steps with the position.  A warp a (token, head).
template <typename T>
__global__ void __launch_bounds__(128)
qk_head_factors_kernel(const T* q, long q_stride, const T* k, long k_stride, int n_heads, int n_kv_heads,
                       int head_dim, int real_dim, int norm, float eps, float temp_coef, int temp_every,
                       const int* __restrict__ pos, const int* __restrict__ req, float* __restrict__ out, int n_tokens) {
  const int heads = n_heads + n_kv_heads;
  const long item = (long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (item >= (long)n_tokens * heads) return;
  const int t = (int)(item / heads), h = (int)(item % heads), lane = threadIdx.x & 31;
  if (req[t] < 0) return;
  float f = 1.f;
  if (norm) {
    const T* x = h < n_heads ? q + (size_t)t * q_stride + (size_t)h * head_dim
                             : k + (size_t)t * k_stride + (size_t)(h - n_heads) * head_dim;
    float ss = 0.f;
    for (int d = lane; d < real_dim; d += 32) {
      const float v = to_f32<T>(x[d]);
      ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    f = rsqrtf(ss / (float)real_dim + eps);
  }
  if (temp_every > 0 && h < n_heads) f *= 1.f + temp_coef * logf((float)((pos[t] + 1) / temp_every) + 1.f);
  if (lane == 0) out[(size_t)t * heads + h] = f;
}

// The same for bfloat16 rows that can be read in 16-byte pieces: eight lanes a (token, head), a piece of
// eight columns a lane and round.
__global__ void __launch_bounds__(128)
qk_head_factors_bf16x8_kernel(const __nv_bfloat16* q, long q_stride, const __nv_bfloat16* k, long k_stride, int n_heads,
                              int n_kv_heads, int head_dim, int real_dim, int norm, float eps, float temp_coef,
                              int temp_every, const int* __restrict__ pos, const int* __restrict__ req,
                              float* __restrict__ out, int n_tokens) {
  const int heads = n_heads + n_kv_heads;
  const long item = ((long)blockIdx.x * 128 + threadIdx.x) >> 3;
  const int lane = threadIdx.x & 7;
  const bool live = item < (long)n_tokens * heads;
  const int t = live ? (int)(item / heads) : 0, h = live ? (int)(item % heads) : 0;
  const bool active = live && req[t] >= 0;
  float f = 1.f;
  if (norm) {
    float ss = 0.f;
    if (active) {
      const __nv_bfloat16* x = h < n_heads ? q + (size_t)t * q_stride + (size_t)h * head_dim
                                           : k + (size_t)t * k_stride + (size_t)(h - n_heads) * head_dim;
      for (int d = lane * 8; d < real_dim; d += 64) {
        const uint4 raw = *reinterpret_cast<const uint4*>(x + d);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 v = __bfloat1622float2(h2[i]);
          ss = fmaf(v.x, v.x, ss);
          ss = fmaf(v.y, v.y, ss);
        }
      }
    }
    ss += __shfl_xor_sync(0xffffffffu, ss, 1);
    ss += __shfl_xor_sync(0xffffffffu, ss, 2);
    ss += __shfl_xor_sync(0xffffffffu, ss, 4);
    f = rsqrtf(ss / (float)real_dim + eps);
  }
  if (!active) return;
  if (temp_every > 0 && h < n_heads) f *= 1.f + temp_coef * logf((float)((pos[t] + 1) / temp_every) + 1.f);
  if (lane == 0) out[(size_t)t * heads + h] = f;
}

extern "C" int fg_qk_head_factors(const void* q, long q_stride, const void* k, long k_stride, int dtype, int n_heads,
                                  int n_kv_heads, int head_dim, int real_dim, int norm, float eps, float temp_coef,
                                  int temp_every, const int* pos, const int* req, float* out, int n_tokens,
                                  cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  if (dtype == FG_BF16 && head_dim % 8 == 0 && real_dim % 8 == 0 && q_stride % 8 == 0 && k_stride % 8 == 0 &&
      ((uintptr_t)q & 15) == 0 && (k == nullptr || ((uintptr_t)k & 15) == 0)) {
    const long lanes = (long)n_tokens * (n_heads + n_kv_heads) * 8;
    qk_head_factors_bf16x8_kernel<<<(unsigned)((lanes + 127) / 128), 128, 0, stream>>>(
        (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k, k_stride, n_heads, n_kv_heads, head_dim, real_dim, norm,
        eps, temp_coef, temp_every, pos, req, out, n_tokens);
    FG_CHECK_LAUNCH("fg_qk_head_factors");
    return 0;
  }
  FG_CHECK_ARG(n_heads > 0 && n_kv_heads >= 0 && real_dim > 0 && real_dim <= head_dim && (n_kv_heads == 0 || k || !norm),
               "fg_qk_head_factors: bad sizes");
  const long items = (long)n_tokens * (n_heads + n_kv_heads);
  const unsigned grid = (unsigned)((items + 3) / 4);
  if (dtype == FG_F32)
    qk_head_factors_kernel<float><<<grid, 128, 0, stream>>>((const float*)q, q_stride, (const float*)k, k_stride,
                                                            n_heads, n_kv_heads, head_dim, real_dim, norm, eps,
                                                            temp_coef, temp_every, pos, req, out, n_tokens);
  else
    qk_head_factors_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>(
        (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k, k_stride, n_heads, n_kv_heads, head_dim, real_dim,
        norm, eps, temp_coef, temp_every, pos, req, out, n_tokens);
  FG_CHECK_LAUNCH("fg_qk_head_factors");
  return 0;
}

// q: [T, n_heads*head_dim] with row stride q_stride (elements), rotated in place.
// k, v: [T, n_kv_heads*head_dim] with their strides, or both null (queries only).
// freqs: float32 [head_dim/2] or null for no rotation of queries and keys; v_freqs: the same
// for values, which are rotated by their own position on their way into the page (null: copied).
extern "C" int fg_rope_kv_write(void* q, int q_stride, const void* k, int k_stride, const void* v,
                                int v_stride, int dtype, const int* pos, const int* req,
                                const float* freqs, const float* v_freqs, void* k_pages, void* v_pages,
                                const int* block_table, int table_width, int page_size, int n_pages,
                                int n_tokens, int n_heads, int n_kv_heads, int head_dim, int* status,
                                const float* rstd, const float* qn_w, const float* kn_w, int rstd_heads,
                                cudaStream_t stream) {
  // rstd: null, or float32 factors by which queries and keys are multiplied before they turn: [T, 2]
  // (a token's queries, its keys) when rstd_heads is 0, else [T, rstd_heads] with rstd_heads = n_heads +
  // n_kv_heads (every query head, then every key head).  qn_w / kn_w: per-column weights that join the
  // factors, or null for ones.
  if (n_tokens == 0) return 0;
  FG_CHECK_ARG(rstd_heads == 0 || (rstd != nullptr && rstd_heads == n_heads + n_kv_heads),
               "fg_rope_kv_write: %d factors a token for %d + %d heads", rstd_heads, n_heads, n_kv_heads);
  FG_CHECK_ARG(head_dim > 0 && head_dim % 2 == 0, "fg_rope_kv_write: head_dim %d must be even", head_dim);
  FG_CHECK_ARG((k == nullptr) == (v == nullptr), "fg_rope_kv_write: k and v must both be given or both null");
  FG_CHECK_ARG(k == nullptr || (k_pages && v_pages && block_table && page_size > 0),
               "fg_rope_kv_write: cache arguments missing");
  FG_CHECK_ARG(head_dim / 2 <= ROPE_THREADS, "fg_rope_kv_write: head size %d is too large", head_dim);
  const int total_heads = n_heads + (k ? 2 * n_kv_heads : 0);
  // many tokens: one block a token; few tokens: slices of heads, so that there are enough blocks
  int slices = n_tokens >= 1024 ? 1 : (n_tokens >= 128 ? 4 : 16);
  if (slices > total_heads) slices = total_heads;
  const int ipt = (total_heads + slices - 1) / slices;  // heads per block
  const dim3 grid(n_tokens, (total_heads + ipt - 1) / ipt);
  const int threads = ROPE_THREADS;
  FG_CHECK_ARG(grid.y <= 65535, "fg_rope_kv_write: too many heads");
  const size_t pair = dtype == FG_F32 ? 8 : 4;
  const auto ok = [&](const void* p, int stride) { return p == nullptr || (((uintptr_t)p % pair) == 0 && stride % 2 == 0); };
  const bool vec = ok(q, q_stride) && ok(k, k_stride) && ok(v, v_stride) && ok(k_pages, 0) && ok(v_pages, 0);
  const auto ok16 = [&](const void* p, int stride) { return p == nullptr || (((uintptr_t)p & 15) == 0 && stride % 8 == 0); };
  if (dtype == FG_BF16 && head_dim % 8 == 0 && head_dim / 8 <= ROPE_THREADS && ok16(q, q_stride) && ok16(k, k_stride) &&
      ok16(v, v_stride) && ok16(k_pages, 0) && ok16(v_pages, 0)) {
    rope_kv_bf16x8_kernel<<<grid, threads, 0, stream>>>(
        (__nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k, k_stride, (const __nv_bfloat16*)v, v_stride, pos, req,
        freqs, v_freqs, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, block_table, table_width, page_size,
        n_pages, n_heads, n_kv_heads, head_dim, status, ipt, rstd, qn_w, kn_w, rstd_heads);
    FG_CHECK_LAUNCH("fg_rope_kv_write");
    return 0;
  }
  if (dtype == FG_F32)
    rope_kv_kernel<float><<<grid, threads, 0, stream>>>(
        (float*)q, q_stride, (const float*)k, k_stride, (const float*)v, v_stride, pos, req, freqs, v_freqs,
        (float*)k_pages, (float*)v_pages, block_table, table_width, page_size, n_pages, n_heads,
        n_kv_heads, head_dim, status, vec, ipt, rstd, qn_w, kn_w, rstd_heads);
  else if (dtype == FG_BF16)
    rope_kv_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>(
        (__nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k, k_stride, (const __nv_bfloat16*)v,
        v_stride, pos, req, freqs, v_freqs, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, block_table,
        table_width, page_size, n_pages, n_heads, n_kv_heads, head_dim, status, vec, ipt, rstd, qn_w, kn_w, rstd_heads);
  else
    FG_CHECK_ARG(false, "fg_rope_kv_write: bad dtype %d", dtype);
  FG_CHECK_LAUNCH("fg_rope_kv_write");
  return 0;
}
