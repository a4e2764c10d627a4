// Feed-forward with routed experts: every token goes through `top` of `n_experts` small gated
// feed-forwards and their outputs are summed with the router's weights.
//
//   fg_moe_logits  the router's logits x W^T in float32 (W float32, x of either type): a warp a token.
//   fg_moe_route   scores s = softmax(logits) (float32); the experts with the largest s + correction
//                  are chosen; their weights are their s, as they are (or divided by their sum).
//   fg_moe_plan    sorts the (token, choice) pairs by expert (stable: ascending pair index within an
//                  expert) and cuts every expert's rows into tiles of `tile_rows`.  Everything stays on
//                  the device: the products below are launched for the most tiles there can be and
//                  their surplus blocks leave at once, so a step can be captured in a graph.
//   fg_moe_gemm    out[r, :] = x[row(r), :] W[e(r)]^T over the sorted rows r, float32 sums in ascending
//                  k in one accumulator (the value of a row does not depend on the batch around it);
//                  with two weight stacks the result is silu(x W1^T) * (x W3^T).  This is the product of
//                  the float32 mode and of sizes the tensor-core kernel does not take.
//   fg_moe_gemm_mma the same product in bfloat16 on the tensor cores.
//   fg_moe_combine ff[t, :] = sum_k weight[t, k] * y[row of (t, k), :], ascending k.
#include "common.cuh"

// ---- the router's logits ---------------------------------------------------------------------
// logits[t, e] = sum_k x[t, k] w[e, k] in float32: a block of four warps a token, eight experts at a
// time.  A thread sums runs of eight consecutive k (read as 16-byte words, all of an expert group's
// loads in flight before the first sum: the router's matrix comes from memory at every step and a
// chain of dependent loads would be all latency) in ascending order; the threads' sums meet in a fixed
// exchange tree and the four warps' in ascending order, so a token's logits do not depend on the
// batch around it.  K that is no multiple of eight, or unaligned rows, go element by element.
constexpr int LOGITS_GROUP = 8;
constexpr int LOGITS_THREADS = 128;

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(LOGITS_THREADS)
moe_logits_kernel(const T* x, long ldx, const float* __restrict__ w, long ldw, float* __restrict__ logits,
                  const int* __restrict__ req, int n_experts, int K) {
  __shared__ float part[LOGITS_THREADS / 32][LOGITS_GROUP];
  const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (req != nullptr && req[t] < 0) return;
  const T* row = x + (size_t)t * ldx;
  for (int e0 = 0; e0 < n_experts; e0 += LOGITS_GROUP) {
    float acc[LOGITS_GROUP];
#pragma unroll
    for (int j = 0; j < LOGITS_GROUP; ++j) acc[j] = 0.f;
    if (VEC) {
      for (int k = tid * 8; k < K; k += LOGITS_THREADS * 8) {
        float xv[8], wv[LOGITS_GROUP][8];
        load8<T>(row + k, xv);
#pragma unroll
        for (int j = 0; j < LOGITS_GROUP; ++j) {
          // (experts beyond the last read the last one's row again and are dropped below)
          const int e = min(e0 + j, n_experts - 1);
          load8<float>(w + (size_t)e * ldw + k, wv[j]);
        }
#pragma unroll
        for (int j = 0; j < LOGITS_GROUP; ++j)
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[j] = fmaf(xv[i], wv[j][i], acc[j]);
      }
    } else {
      for (int k = tid; k < K; k += LOGITS_THREADS) {
        const float xv = to_f32<T>(row[k]);
#pragma unroll
        for (int j = 0; j < LOGITS_GROUP; ++j)
          if (e0 + j < n_experts) acc[j] = fmaf(xv, w[(size_t)(e0 + j) * ldw + k], acc[j]);
      }
    }
#pragma unroll
    for (int j = 0; j < LOGITS_GROUP; ++j) {
      const float total = warp_sum(acc[j]);
      if (lane == 0) part[warp][j] = total;
    }
    __syncthreads();
    if (tid < LOGITS_GROUP && e0 + tid < n_experts) {
      float total = part[0][tid];
#pragma unroll
      for (int i = 1; i < LOGITS_THREADS / 32; ++i) total += part[i][tid];
      logits[(size_t)t * n_experts + e0 + tid] = total;
    }
    __syncthreads();
  }
}

extern "C" int fg_moe_logits(const void* x, int dtype, long ldx, const float* w, long ldw, float* logits,
                             const int* req, int n_tokens, int n_experts, int K, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  FG_CHECK_ARG(n_experts >= 1 && K >= 1, "fg_moe_logits: %d experts over %d inputs", n_experts, K);
  FG_CHECK_ARG(dtype == FG_F32 || dtype == FG_BF16, "fg_moe_logits: bad dtype %d", dtype);
  const long x_words = dtype == FG_F32 ? 4 : 8;  // elements of 16 bytes
  const bool vec = K % 8 == 0 && ((uintptr_t)x & 15) == 0 && ldx % x_words == 0 && ((uintptr_t)w & 15) == 0 && ldw % 4 == 0;
#define LAUNCH(T, VEC)                                                                                             \
  moe_logits_kernel<T, VEC><<<n_tokens, LOGITS_THREADS, 0, stream>>>((const T*)x, ldx, w, ldw, logits, req, n_experts, K)
  if (dtype == FG_F32) {
    if (vec) LAUNCH(float, true); else LAUNCH(float, false);
  } else {
    if (vec) LAUNCH(__nv_bfloat16, true); else LAUNCH(__nv_bfloat16, false);
  }
#undef LAUNCH
  FG_CHECK_LAUNCH("fg_moe_logits");
  return 0;
}

constexpr int ROUTE_MAX_PER_LANE = 8;  // up to 256 experts

__global__ void __launch_bounds__(128)
moe_route_kernel(const float* logits, const float* __restrict__ correction, int* __restrict__ ids,
                 float* __restrict__ weights, const int* __restrict__ req, int n_tokens, int n_experts, int top,
                 int renormalize) {
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= n_tokens) return;
  if (req[t] < 0) {
    for (int k = lane; k < top; k += 32) {
      ids[(size_t)t * top + k] = -1;
      weights[(size_t)t * top + k] = 0.f;
    }
    return;
  }
  float z[ROUTE_MAX_PER_LANE], s[ROUTE_MAX_PER_LANE], c[ROUTE_MAX_PER_LANE];
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    z[i] = e < n_experts ? logits[(size_t)t * n_experts + e] : -INFINITY;
    m = fmaxf(m, z[i]);
  }
  m = warp_max(m);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i) {
    s[i] = lane + 32 * i < n_experts ? expf(z[i] - m) : 0.f;
    sum += s[i];
  }
  sum = warp_sum(sum);
#pragma unroll
  for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    s[i] = s[i] / sum;
    c[i] = e < n_experts ? s[i] + (correction ? correction[e] : 0.f) : -INFINITY;
  }
  for (int k = 0; k < top; ++k) {
    // the largest choice score left; equal scores go to the lower index
    float best = -INFINITY, best_s = 0.f;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (e < n_experts && (c[i] > best || (c[i] == best && e < best_e))) {
        best = c[i];
        best_e = e;
        best_s = s[i];
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      const float os = __shfl_xor_sync(0xffffffffu, best_s, o);
      if (ob > best || (ob == best && oe < best_e)) {
        best = ob;
        best_e = oe;
        best_s = os;
      }
    }
    if (lane == 0) {
      ids[(size_t)t * top + k] = best_e;
      weights[(size_t)t * top + k] = best_s;
    }
#pragma unroll
    for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i)
      if (lane + 32 * i == best_e) c[i] = -INFINITY;
  }
  if (renormalize) {
    // the chosen experts' weights divided by their sum (ascending choice)
    __syncwarp();
    float total = 0.f;
    for (int k = 0; k < top; ++k) total += weights[(size_t)t * top + k];
    __syncwarp();
    for (int k = lane; k < top; k += 32) weights[(size_t)t * top + k] /= total;
  }
}

extern "C" int fg_moe_route(const float* logits, const float* correction, int* ids, float* weights, const int* req,
                            int n_tokens, int n_experts, int top, int renormalize, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  FG_CHECK_ARG(n_experts >= 1 && n_experts <= 32 * ROUTE_MAX_PER_LANE, "fg_moe_route: %d experts (1 to %d)",
               n_experts, 32 * ROUTE_MAX_PER_LANE);
  FG_CHECK_ARG(top >= 1 && top <= n_experts, "fg_moe_route: %d of %d experts", top, n_experts);
  moe_route_kernel<<<(n_tokens + 3) / 4, 128, 0, stream>>>(logits, correction, ids, weights, req, n_tokens, n_experts,
                                                           top, renormalize);
  FG_CHECK_LAUNCH("fg_moe_route");
  return 0;
}

// ---- choice among groups of experts, sigmoid scores ------------------------------------------------
// kind 0: scores s = softmax(logits); kind 1: s = sigmoid(logits).  With n_groups > 0 the experts form
// n_groups equal groups of neighbours; a group's score is the sum of its `group_top` largest scores, and
// only experts of the `keep_groups` best groups (equal ones: the lower index) can be chosen.  The `top`
// experts with the largest s + correction among those are chosen (equal ones: the lower index); their
// weights are their s, divided with `renormalize` by (their sum + renorm_eps), then times weight_scale.
// A warp a token; the scores pass through the warp's row of shared memory.
constexpr int ROUTE_WARPS = 4;

__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_route_groups_kernel(const float* logits, const float* __restrict__ correction, int* __restrict__ ids,
                        float* __restrict__ weights, const int* __restrict__ req, int n_tokens, int n_experts, int top,
                        int kind, int n_groups, int keep_groups, int group_top, int renormalize, float renorm_eps,
                        float weight_scale) {
  __shared__ float s_s[ROUTE_WARPS][32 * ROUTE_MAX_PER_LANE];
  __shared__ float g_s[ROUTE_WARPS][32 * ROUTE_MAX_PER_LANE];
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * ROUTE_WARPS + w;
  if (t >= n_tokens) return;
  if (req[t] < 0) {
    for (int k = lane; k < top; k += 32) {
      ids[(size_t)t * top + k] = -1;
      weights[(size_t)t * top + k] = 0.f;
    }
    return;
  }
  float s[ROUTE_MAX_PER_LANE], c[ROUTE_MAX_PER_LANE];
  if (kind == 0) {
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      s[i] = e < n_experts ? logits[(size_t)t * n_experts + e] : -INFINITY;
      m = fmaxf(m, s[i]);
    }
    m = warp_max(m);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i) {
      s[i] = lane + 32 * i < n_experts ? expf(s[i] - m) : 0.f;
      sum += s[i];
    }
    sum = warp_sum(sum);
#pragma unroll
    for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i) s[i] = s[i] / sum;
  } else {
#pragma unroll
    for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      s[i] = e < n_experts ? 1.f / (1.f + expf(-logits[(size_t)t * n_experts + e])) : 0.f;
    }
  }
#pragma unroll
  for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    c[i] = e < n_experts ? s[i] + (correction ? correction[e] : 0.f) : -INFINITY;
    if (e < n_experts) s_s[w][e] = s[i];
  }
  if (n_groups > 0) {
    __syncwarp();
    const int per = n_experts / n_groups;
    // a group's score: its group_top largest scores added, largest first
    for (int gi = lane; gi < n_groups; gi += 32) {
      float total = 0.f;
      float last = INFINITY;
      int last_e = -1;
      for (int k = 0; k < group_top && k < per; ++k) {
        // the largest score below (last, last_e) in the order (score descending, index ascending)
        float best = -INFINITY;
        int best_e = -1;
        for (int j = 0; j < per; ++j) {
          const float v = s_s[w][gi * per + j];
          const bool after = v < last || (v == last && j > last_e);
          if (after && (v > best || best_e < 0)) {
            best = v;
            best_e = j;
          }
        }
        if (best_e < 0) break;
        total += best;
        last = best;
        last_e = best_e;
      }
      g_s[w][gi] = total;
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (e >= n_experts) continue;
      const int gi = e / per;
      const float mine = g_s[w][gi];
      int rank = 0;  // groups ahead of this one
      for (int o = 0; o < n_groups; ++o) {
        const float v = g_s[w][o];
        rank += (v > mine || (v == mine && o < gi)) ? 1 : 0;
      }
      if (rank >= keep_groups) c[i] = -INFINITY;
    }
  }
  float total = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY, best_s = 0.f;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (e < n_experts && (c[i] > best || (c[i] == best && e < best_e))) {
        best = c[i];
        best_e = e;
        best_s = s[i];
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      const float os = __shfl_xor_sync(0xffffffffu, best_s, o);
      if (ob > best || (ob == best && oe < best_e)) {
        best = ob;
        best_e = oe;
        best_s = os;
      }
    }
    total += best_s;  // every lane holds the same sum, in ascending choice
    if (lane == 0) {
      ids[(size_t)t * top + k] = best_e;
      weights[(size_t)t * top + k] = best_s;
    }
#pragma unroll
    for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i)
      if (lane + 32 * i == best_e) c[i] = -INFINITY;
  }
  __syncwarp();
  if (renormalize || weight_scale != 1.f)
    for (int k = lane; k < top; k += 32) {
      const float wgt = weights[(size_t)t * top + k];
      weights[(size_t)t * top + k] = (renormalize ? wgt / (total + renorm_eps) : wgt) * weight_scale;
    }
}

extern "C" int fg_moe_route_groups(const float* logits, const float* correction, int* ids, float* weights,
                                   const int* req, int n_tokens, int n_experts, int top, int kind, int n_groups,
                                   int keep_groups, int group_top, int renormalize, float renorm_eps,
                                   float weight_scale, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  FG_CHECK_ARG(n_experts >= 1 && n_experts <= 32 * ROUTE_MAX_PER_LANE, "fg_moe_route_groups: %d experts (1 to %d)",
               n_experts, 32 * ROUTE_MAX_PER_LANE);
  FG_CHECK_ARG(top >= 1 && top <= n_experts, "fg_moe_route_groups: %d of %d experts", top, n_experts);
  FG_CHECK_ARG(kind == 0 || kind == 1, "fg_moe_route_groups: unknown kind of score %d", kind);
  if (n_groups > 0) {
    FG_CHECK_ARG(n_experts % n_groups == 0 && keep_groups >= 1 && keep_groups <= n_groups && group_top >= 1,
                 "fg_moe_route_groups: %d experts in %d groups of which %d", n_experts, n_groups, keep_groups);
    FG_CHECK_ARG(keep_groups * (n_experts / n_groups) >= top, "fg_moe_route_groups: %d groups cannot hold %d experts",
                 keep_groups, top);
  }
  moe_route_groups_kernel<<<(n_tokens + ROUTE_WARPS - 1) / ROUTE_WARPS, ROUTE_WARPS * 32, 0, stream>>>(
      logits, correction, ids, weights, req, n_tokens, n_experts, top, kind, n_groups, keep_groups, group_top,
      renormalize, renorm_eps, weight_scale);
  FG_CHECK_LAUNCH("fg_moe_route_groups");
  return 0;
}

// ---- the plan -----------------------------------------------------------------------------------
// One block.  A warp takes experts w, w + 32, ...: it walks all pairs 32 at a time and counts (first
// pass) or places (second pass) those of its expert, in ascending pair order.
constexpr int PLAN_THREADS = 1024;
constexpr int PLAN_MAX_EXPERTS = 256;

__global__ void __launch_bounds__(PLAN_THREADS)
moe_plan_kernel(const int* __restrict__ ids, int n_pairs, int n_experts, int tile_rows, int* __restrict__ row_pair,
                int* __restrict__ pair_row, int* __restrict__ tile_expert, int* __restrict__ tile_row0,
                int* __restrict__ tile_n, int* __restrict__ n_tiles, int max_tiles, int* __restrict__ expert_end) {
  __shared__ int count[PLAN_MAX_EXPERTS], offset[PLAN_MAX_EXPERTS + 1], tile0[PLAN_MAX_EXPERTS + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int e = warp; e < n_experts; e += PLAN_THREADS / 32) {
    int c = 0;
    for (int base = 0; base < n_pairs; base += 32) {
      const int p = base + lane;
      c += __popc(__ballot_sync(0xffffffffu, p < n_pairs && ids[p] == e));
    }
    if (lane == 0) count[e] = c;
  }
  for (int p = threadIdx.x; p < n_pairs; p += PLAN_THREADS)
    if (ids[p] < 0 || ids[p] >= n_experts) pair_row[p] = -1;  // padding: belongs to no expert
  __syncthreads();
  if (threadIdx.x == 0) {
    int rows = 0, tiles = 0;
    for (int e = 0; e < n_experts; ++e) {
      offset[e] = rows;
      tile0[e] = tiles;
      rows += count[e];
      tiles += (count[e] + tile_rows - 1) / tile_rows;
    }
    offset[n_experts] = rows;
    tile0[n_experts] = tiles;
    *n_tiles = tiles < max_tiles ? tiles : max_tiles;
  }
  __syncthreads();
  if (expert_end != nullptr)
    for (int e = threadIdx.x; e < n_experts; e += PLAN_THREADS) expert_end[e] = offset[e + 1];
  for (int e = warp; e < n_experts; e += PLAN_THREADS / 32) {
    int placed = 0;
    for (int base = 0; base < n_pairs; base += 32) {
      const int p = base + lane;
      const bool mine = p < n_pairs && ids[p] == e;
      const unsigned mask = __ballot_sync(0xffffffffu, mine);
      if (mine) {
        const int r = offset[e] + placed + __popc(mask & ((1u << lane) - 1u));
        row_pair[r] = p;
        pair_row[p] = r;
      }
      placed += __popc(mask);
    }
    const int tiles = tile0[e + 1] - tile0[e];
    for (int i = lane; i < tiles; i += 32) {
      const int slot = tile0[e] + i;
      if (slot < max_tiles) {
        tile_expert[slot] = e;
        tile_row0[slot] = offset[e] + i * tile_rows;
        tile_n[slot] = min(tile_rows, count[e] - i * tile_rows);
      }
    }
  }
}

extern "C" int fg_moe_plan(const int* ids, int n_pairs, int n_experts, int tile_rows, int* row_pair, int* pair_row,
                           int* tile_expert, int* tile_row0, int* tile_n, int* n_tiles, int max_tiles,
                           int* expert_end, cudaStream_t stream) {
  FG_CHECK_ARG(n_experts >= 1 && n_experts <= PLAN_MAX_EXPERTS, "fg_moe_plan: %d experts (1 to %d)", n_experts,
               PLAN_MAX_EXPERTS);
  FG_CHECK_ARG(tile_rows > 0 && max_tiles >= (n_pairs + tile_rows - 1) / tile_rows + n_experts - 1,
               "fg_moe_plan: room for %d tiles is too little", max_tiles);
  moe_plan_kernel<<<1, PLAN_THREADS, 0, stream>>>(ids, n_pairs, n_experts, tile_rows, row_pair, pair_row, tile_expert,
                                                  tile_row0, tile_n, n_tiles, max_tiles, expert_end);
  FG_CHECK_LAUNCH("fg_moe_plan");
  return 0;
}

// ---- the sorted rows, gathered -----------------------------------------------------------------
// xs[r, :] = x[row_pair[r] / top, :] for the rows that the plan filled (r < expert_end[last]); a
// block a row.  For products that want one expert's rows side by side in memory.
template <typename T>
__global__ void __launch_bounds__(128)
moe_gather_kernel(const T* x, long ldx, T* __restrict__ xs, long lds, const int* __restrict__ row_pair,
                  const int* __restrict__ expert_end, int n_experts, int top, int K, int vec) {
  const int r = blockIdx.x;
  if (r >= expert_end[n_experts - 1]) return;
  const T* src = x + (size_t)(row_pair[r] / top) * ldx;
  T* dst = xs + (size_t)r * lds;
  if (vec) {
    const int words = K * (int)sizeof(T) / 16;
    for (int c = threadIdx.x; c < words; c += blockDim.x)
      reinterpret_cast<uint4*>(dst)[c] = reinterpret_cast<const uint4*>(src)[c];
  } else {
    for (int c = threadIdx.x; c < K; c += blockDim.x) dst[c] = src[c];
  }
}

extern "C" int fg_moe_gather(const void* x, long ldx, void* xs, long lds, int dtype, const int* row_pair,
                             const int* expert_end, int n_experts, int top, int n_pairs, int K, cudaStream_t stream) {
  if (n_pairs == 0) return 0;
  FG_CHECK_ARG(dtype == FG_F32 || dtype == FG_BF16, "fg_moe_gather: bad dtype %d", dtype);
  const int size = dtype == FG_F32 ? 4 : 2;
  const int vec = (K * size) % 16 == 0 && (ldx * size) % 16 == 0 && (lds * size) % 16 == 0 && ((uintptr_t)x & 15) == 0 &&
                  ((uintptr_t)xs & 15) == 0;
  if (dtype == FG_F32)
    moe_gather_kernel<float><<<n_pairs, 128, 0, stream>>>((const float*)x, ldx, (float*)xs, lds, row_pair, expert_end,
                                                          n_experts, top, K, vec);
  else
    moe_gather_kernel<__nv_bfloat16><<<n_pairs, 128, 0, stream>>>((const __nv_bfloat16*)x, ldx, (__nv_bfloat16*)xs, lds,
                                                                  row_pair, expert_end, n_experts, top, K, vec);
  FG_CHECK_LAUNCH("fg_moe_gather");
  return 0;
}

// ---- the products, float32 sums --------------------------------------------------------------------
namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;  // 256 threads, 4x4 outputs each
}

// x: [., K] rows of the left operand; row r of the sorted list reads x row (GATHER ? row_pair[r] / top : r).
// w1 (and w3 when GATED): [experts, N, K], expert e at w + e * w_stride.  out: [sorted rows, N].
template <typename T, bool GATED>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(const T* x, long ldx, const T* __restrict__ w1, const T* __restrict__ w3, long w_stride, T* __restrict__ out, long ldo,
                int N, int K, const int* __restrict__ row_pair, int top, const int* __restrict__ tile_expert,
                const int* __restrict__ tile_row0, const int* __restrict__ tile_n, const int* __restrict__ n_tiles) {
  if ((int)blockIdx.y >= *n_tiles) return;
  __shared__ float As[BK][BM + 4];
  __shared__ float W1s[BK][BN + 4];
  __shared__ float W3s[GATED ? BK : 1][BN + 4];
  __shared__ int src_row[BM];
  const int e = tile_expert[blockIdx.y], row0 = tile_row0[blockIdx.y], rows = tile_n[blockIdx.y];
  const int tid = threadIdx.x;
  if (tid < BM) {
    int r = -1;
    if (tid < rows) r = row_pair != nullptr ? row_pair[row0 + tid] / top : row0 + tid;
    src_row[tid] = r;
  }
  __syncthreads();
  const int tx = tid & 15, ty = tid >> 4;
  const int n0 = blockIdx.x * BN;
  const T* W1 = w1 + (size_t)e * w_stride;
  const T* W3 = GATED ? w3 + (size_t)e * w_stride : nullptr;
  float acc[TM][TN], acc3[GATED ? TM : 1][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      acc[i][j] = 0.f;
      if (GATED) acc3[i][j] = 0.f;
    }
  const int lr = tid >> 2, lk = (tid & 3) * 4;
  const int a_row = src_row[lr];
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int kk = k0 + lk + u;
      const int wn = n0 + lr;
      As[lk + u][lr] = (a_row >= 0 && kk < K) ? to_f32<T>(x[(size_t)a_row * ldx + kk]) : 0.f;
      W1s[lk + u][lr] = (wn < N && kk < K) ? to_f32<T>(W1[(size_t)wn * K + kk]) : 0.f;
      if (GATED) W3s[lk + u][lr] = (wn < N && kk < K) ? to_f32<T>(W3[(size_t)wn * K + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN], b3[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) {
        b[j] = W1s[kk][tx * TN + j];
        if (GATED) b3[j] = W3s[kk][tx * TN + j];
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
          acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
          if (GATED) acc3[i][j] = fmaf(a[i], b3[j], acc3[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = ty * TM + i;
    if (m >= rows) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (GATED) v = v / (1.f + expf(-v)) * acc3[i][j];
      out[(size_t)(row0 + m) * ldo + n] = from_f32<T>(v);
    }
  }
}

extern "C" int fg_moe_gemm_tile_rows() { return BM; }

extern "C" int fg_moe_gemm(const void* x, long ldx, const void* w1, const void* w3, long w_stride, void* out, long ldo, int dtype,
                           int N, int K, const int* row_pair, int top, const int* tile_expert, const int* tile_row0,
                           const int* tile_n, const int* n_tiles, int max_tiles, cudaStream_t stream) {
  if (max_tiles == 0 || N == 0) return 0;
  FG_CHECK_ARG(K > 0 && max_tiles <= 65535, "fg_moe_gemm: bad sizes K=%d tiles=%d", K, max_tiles);
  dim3 grid((N + BN - 1) / BN, max_tiles);
#define LAUNCH(T, GATED)                                                                                         \
  moe_gemm_kernel<T, GATED><<<grid, 256, 0, stream>>>((const T*)x, ldx, (const T*)w1, (const T*)w3, w_stride, (T*)out, ldo, N, K, \
                                                      row_pair, top, tile_expert, tile_row0, tile_n, n_tiles)
  if (dtype == FG_F32) {
    if (w3) LAUNCH(float, true); else LAUNCH(float, false);
  } else if (dtype == FG_BF16) {
    if (w3) LAUNCH(__nv_bfloat16, true); else LAUNCH(__nv_bfloat16, false);
  } else {
    FG_CHECK_ARG(false, "fg_moe_gemm: bad dtype %d", dtype);
  }
#undef LAUNCH
  FG_CHECK_LAUNCH("fg_moe_gemm");
  return 0;
}

// ---- the products on the tensor cores (bfloat16) ------------------------------------------------------
// The same tiles of one expert's rows, mma.sync m16n8k16 with float32 accumulators: a block of four
// warps makes MM rows x MN columns (warp w rows 16w .. 16w + 15), K in steps of MK through four
// cp.async buffers (three steps in flight while one is multiplied: with a few rows the product is
// a stream of the experts' matrices from memory, and the bytes in flight set its rate).  A row's sums run over k in the same order whatever else is in its tile, so
// its value does not depend on the batch.  Rows are gathered by the plan (x row = row_pair / top)
// as they are copied; rows and columns beyond the tile's are zero-filled and never stored.
// Needs K a multiple of 8 and 16-byte aligned rows (the caller checks).
namespace {
constexpr int MM = 64, MN = 64, MK = 64, MLD = MK + 8;  // rows of 144 bytes: ldmatrix without bank conflicts
constexpr int MST = 4;                                    // buffers
constexpr int MKC = MK / 8;                               // 16-byte words a row of a step

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void copy_16(void* dst, const void* src, bool pred) {
  const int bytes = pred ? 16 : 0;  // 0: the 16 bytes are zero-filled, nothing is read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void copy_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void copy_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }
__device__ __forceinline__ void load_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
}  // namespace

template <bool GATED>
__global__ void __launch_bounds__(128)
moe_gemm_mma_kernel(const __nv_bfloat16* x, long ldx, const __nv_bfloat16* __restrict__ w1,
                    const __nv_bfloat16* __restrict__ w3, long w_stride, __nv_bfloat16* __restrict__ out, long ldo, int N, int K,
                    const int* __restrict__ row_pair, int top, const int* __restrict__ tile_expert,
                    const int* __restrict__ tile_row0, const int* __restrict__ tile_n,
                    const int* __restrict__ n_tiles) {
  if ((int)blockIdx.y >= *n_tiles) return;
  extern __shared__ __align__(16) unsigned char moe_smem[];
  typedef __nv_bfloat16 (*Tile)[MM][MLD];  // MM == MN
  Tile As = reinterpret_cast<Tile>(moe_smem);
  Tile W1s = As + MST;
  Tile W3s = W1s + MST;  // (only with GATED)
  __shared__ int src_row[MM];
  const int e = tile_expert[blockIdx.y], row0 = tile_row0[blockIdx.y], rows = tile_n[blockIdx.y];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid < MM) {
    int r = -1;
    if (tid < rows) r = row_pair != nullptr ? row_pair[row0 + tid] / top : row0 + tid;
    src_row[tid] = r;
  }
  __syncthreads();
  const int n0 = blockIdx.x * MN;
  const __nv_bfloat16* W1 = w1 + (size_t)e * w_stride;
  const __nv_bfloat16* W3 = GATED ? w3 + (size_t)e * w_stride : nullptr;

  auto load = [&](int buf, int k0) {
#pragma unroll
    for (int i = 0; i < (MM * MKC) / 128; ++i) {
      const int c = tid + i * 128, r = c / MKC, col = (c % MKC) * 8, kk = k0 + col;
      const int a_row = src_row[r];
      const bool a_ok = a_row >= 0 && kk < K;
      copy_16(&As[buf][r][col], a_ok ? x + (size_t)a_row * ldx + kk : x, a_ok);
      const bool w_ok = n0 + r < N && kk < K;
      const size_t w_off = w_ok ? (size_t)(n0 + r) * K + kk : 0;
      copy_16(&W1s[buf][r][col], W1 + w_off, w_ok);
      if (GATED) copy_16(&W3s[buf][r][col], W3 + w_off, w_ok);
    }
    copy_commit();
  };

  float acc[MN / 8][4], acc3[GATED ? MN / 8 : 1][4];
#pragma unroll
  for (int nt = 0; nt < MN / 8; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      acc[nt][i] = 0.f;
      if (GATED) acc3[nt][i] = 0.f;
    }

  const int steps = (K + MK - 1) / MK;
#pragma unroll
  for (int s = 0; s < MST - 1; ++s) {
    if (s < steps) load(s, s * MK); else copy_commit();
  }
  for (int s = 0; s < steps; ++s) {
    const int buf = s % MST;
    // the buffer of step s - 1 is free since the barrier that closed it: fill it with step s + MST - 1
    if (s + MST - 1 < steps) load((s + MST - 1) % MST, (s + MST - 1) * MK); else copy_commit();
    copy_wait<MST - 1>();
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < MK; kk += 16) {
      uint32_t a[4];
      load_x4(a, &As[buf][warp * 16 + (lane & 15)][kk + ((lane >> 4) << 3)]);
#pragma unroll
      for (int np = 0; np < MN / 16; ++np) {
        uint32_t b[4];
        const int n = np * 16 + (lane & 7) + ((lane >> 4) << 3);
        const int k = kk + (((lane >> 3) & 1) << 3);
        load_x4(b, &W1s[buf][n][k]);
        mma_bf16(acc[2 * np], a, b[0], b[1]);
        mma_bf16(acc[2 * np + 1], a, b[2], b[3]);
        if (GATED) {
          load_x4(b, &W3s[buf][n][k]);
          mma_bf16(acc3[2 * np], a, b[0], b[1]);
          mma_bf16(acc3[2 * np + 1], a, b[2], b[3]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int nt = 0; nt < MN / 8; ++nt)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int m = warp * 16 + (lane >> 2) + half * 8;
      const int n = n0 + nt * 8 + (lane & 3) * 2;
      if (m >= rows || n >= N) continue;
      float v0 = acc[nt][half * 2], v1 = acc[nt][half * 2 + 1];
      if (GATED) {
        v0 = v0 / (1.f + expf(-v0)) * acc3[nt][half * 2];
        v1 = v1 / (1.f + expf(-v1)) * acc3[nt][half * 2 + 1];
      }
      __nv_bfloat16* dst = out + (size_t)(row0 + m) * ldo + n;
      dst[0] = __float2bfloat16(v0);
      if (n + 1 < N) dst[1] = __float2bfloat16(v1);
    }
}

extern "C" int fg_moe_mma_tile_rows() { return MM; }

extern "C" int fg_moe_gemm_mma(const void* x, long ldx, const void* w1, const void* w3, long w_stride, void* out, long ldo, int N,
                               int K, const int* row_pair, int top, const int* tile_expert, const int* tile_row0,
                               const int* tile_n, const int* n_tiles, int max_tiles, cudaStream_t stream) {
  if (max_tiles == 0 || N == 0) return 0;
  FG_CHECK_ARG(K > 0 && K % 8 == 0 && ldx % 8 == 0 && max_tiles <= 65535,
               "fg_moe_gemm_mma: bad sizes K=%d ldx=%ld tiles=%d", K, ldx, max_tiles);
  dim3 grid((N + MN - 1) / MN, max_tiles);
  typedef const __nv_bfloat16* P;
  const size_t tile = sizeof(__nv_bfloat16) * MM * MLD, smem3 = 3 * MST * tile, smem2 = 2 * MST * tile;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(moe_gemm_mma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem3);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(moe_gemm_mma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
    FG_CHECK_ARG(e == cudaSuccess, "fg_moe_gemm_mma: shared memory: %s", cudaGetErrorString(e));
    attr_set = true;
  }
  if (w3)
    moe_gemm_mma_kernel<true><<<grid, 128, smem3, stream>>>((P)x, ldx, (P)w1, (P)w3, w_stride, (__nv_bfloat16*)out, ldo, N, K, row_pair,
                                                        top, tile_expert, tile_row0, tile_n, n_tiles);
  else
    moe_gemm_mma_kernel<false><<<grid, 128, smem2, stream>>>((P)x, ldx, (P)w1, nullptr, w_stride, (__nv_bfloat16*)out, ldo, N, K,
                                                         row_pair, top, tile_expert, tile_row0, tile_n, n_tiles);
  FG_CHECK_LAUNCH("fg_moe_gemm_mma");
  return 0;
}

// ---- the weighted sum of a token's experts ----------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const T* y, long ldy, const float* weights, const int* pair_row, T* __restrict__ out, long ldo,
                   int dim, int top) {
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < dim; c += blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k) {
      const int r = pair_row[(size_t)t * top + k];
      if (r >= 0) acc = fmaf(weights[(size_t)t * top + k], to_f32<T>(y[(size_t)r * ldy + c]), acc);
    }
    out[(size_t)t * ldo + c] = from_f32<T>(acc);
  }
}

extern "C" int fg_moe_combine(const void* y, long ldy, const float* weights, const int* pair_row, void* out, long ldo,
                              int dtype, int n_tokens, int dim, int top, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  if (dtype == FG_F32)
    moe_combine_kernel<float><<<n_tokens, 256, 0, stream>>>((const float*)y, ldy, weights, pair_row, (float*)out, ldo,
                                                            dim, top);
  else if (dtype == FG_BF16)
    moe_combine_kernel<__nv_bfloat16><<<n_tokens, 256, 0, stream>>>((const __nv_bfloat16*)y, ldy, weights, pair_row,
                                                                    (__nv_bfloat16*)out, ldo, dim, top);
  else
    FG_CHECK_ARG(false, "fg_moe_combine: bad dtype %d", dtype);
  FG_CHECK_LAUNCH("fg_moe_combine");
  return 0;
}
