// RMS norm fused with a residual sum of several summands:
//   h[t,:] += row[:] + sum_i coef[i] * delta_i[t,:]      (float32, h stored back)
//   out[t,:] = h[t,:] * rsqrt(mean(h^2) + eps) * (w[:] or 1 + w[:])
// The summands are what the sub-layers of a block left pending (two mixers side by side and a
// feed-forward that read the same norm, each with its own multiple); `row` is a vector that
// joins every token's stream (the step vector of a pass over a run of layers).  One block per
// row of h; the order of the row's reduction depends only on dim.
#include "common.cuh"

constexpr int SUM_MAX_TERMS = 4;
constexpr int SUM_THREADS = 256;

struct SumTerms {
  const void* delta[SUM_MAX_TERMS];
  float coef[SUM_MAX_TERMS];
  int n;
};

template <typename TD, typename TO, bool VEC>
__global__ void __launch_bounds__(SUM_THREADS)
rmsnorm_sum_kernel(float* h, SumTerms terms, const float* __restrict__ row, const void* __restrict__ w, int w_dtype,
                   int one_plus, TO* __restrict__ out, const int* __restrict__ rows, int dim, float eps) {
  __shared__ float scratch[32];
  extern __shared__ float kept[];  // the row of h after the sum, between the two passes
  pdl_trigger();
  const size_t base = (size_t)(rows ? rows[blockIdx.x] : blockIdx.x) * dim;
  const size_t obase = (size_t)blockIdx.x * dim;
  const bool store_h = rows == nullptr && (terms.n > 0 || row != nullptr);
  pdl_wait();
  float ss = 0.f;
  if (VEC) {
    for (int d = threadIdx.x * 4; d < dim; d += SUM_THREADS * 4) {
      float4 v = *reinterpret_cast<const float4*>(h + base + d);
      if (row != nullptr) {
        const float4 r = *reinterpret_cast<const float4*>(row + d);
        v.x += r.x; v.y += r.y; v.z += r.z; v.w += r.w;
      }
      for (int i = 0; i < terms.n; ++i) {
        const TD* p = static_cast<const TD*>(terms.delta[i]) + base + d;
        const float c = terms.coef[i];
        v.x = fmaf(c, to_f32<TD>(p[0]), v.x); v.y = fmaf(c, to_f32<TD>(p[1]), v.y);
        v.z = fmaf(c, to_f32<TD>(p[2]), v.z); v.w = fmaf(c, to_f32<TD>(p[3]), v.w);
      }
      if (store_h) *reinterpret_cast<float4*>(h + base + d) = v;
      *reinterpret_cast<float4*>(kept + d) = v;
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
  } else {
    for (int d = threadIdx.x; d < dim; d += SUM_THREADS) {
      float v = h[base + d];
      if (row != nullptr) v += row[d];
      for (int i = 0; i < terms.n; ++i) v = fmaf(terms.coef[i], to_f32<TD>(static_cast<const TD*>(terms.delta[i])[base + d]), v);
      if (store_h) h[base + d] = v;
      kept[d] = v;
      ss += v * v;
    }
  }
  if (out == nullptr) return;
  if (w == nullptr) {
    // no norm: the summed row itself, in the output's type (the input of a product that reads the stream)
    __syncthreads();
    for (int d = threadIdx.x; d < dim; d += SUM_THREADS) out[obase + d] = from_f32<TO>(kept[d]);
    return;
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)dim + eps);
  const float plus = one_plus ? 1.f : 0.f;
  for (int d = threadIdx.x; d < dim; d += SUM_THREADS)
    out[obase + d] = from_f32<TO>(kept[d] * rstd * (plus + load_as_f32(w, w_dtype, d)));
}

// h: float32 [T, dim].  deltas: n_terms pointers to [T, dim] tensors of delta_dtype, with their
// multiples.  row: float32 [dim] or null.  out: [n_rows, dim] of out_dtype, or null (the sum only); with
// out and no weight the summed rows are stored in out as they are (no norm).
// rows: null, or n_rows indices into h and the summands to gather (h is then left as it was).
extern "C" int fg_rmsnorm_sum(float* h, const void* const* deltas, const float* coefs, int n_terms, int delta_dtype,
                              const float* row, const void* w, int w_dtype, int one_plus, void* out, int out_dtype,
                              const int* rows, int n_rows, int dim, float eps, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  FG_CHECK_ARG(dim > 0 && dim <= 48 * 1024 / 4, "fg_rmsnorm_sum: bad dim %d", dim);
  FG_CHECK_ARG(n_terms >= 0 && n_terms <= SUM_MAX_TERMS, "fg_rmsnorm_sum: %d summands (at most %d)", n_terms,
               SUM_MAX_TERMS);
  SumTerms terms;
  terms.n = n_terms;
  bool vec = dim % 4 == 0 && ((uintptr_t)h & 15) == 0 && (row == nullptr || ((uintptr_t)row & 15) == 0);
  for (int i = 0; i < SUM_MAX_TERMS; ++i) {
    terms.delta[i] = i < n_terms ? deltas[i] : nullptr;
    terms.coef[i] = i < n_terms ? coefs[i] : 0.f;
  }
  const size_t smem = (size_t)dim * sizeof(float);
#define LAUNCH(TD, TO)                                                                                      \
  do {                                                                                                      \
    if (vec)                                                                                                \
      fg_launch_pdl(rmsnorm_sum_kernel<TD, TO, true>, dim3(n_rows), dim3(SUM_THREADS), smem, stream, h, terms, row, \
                    w, w_dtype, one_plus, (TO*)out, rows, dim, eps);                                        \
    else                                                                                                    \
      fg_launch_pdl(rmsnorm_sum_kernel<TD, TO, false>, dim3(n_rows), dim3(SUM_THREADS), smem, stream, h, terms, row, \
                    w, w_dtype, one_plus, (TO*)out, rows, dim, eps);                                        \
  } while (0)
  const int key = (n_terms ? delta_dtype : FG_F32) * 2 + (out ? out_dtype : FG_F32);
  switch (key) {
    case 0: LAUNCH(float, float); break;
    case 1: LAUNCH(float, __nv_bfloat16); break;
    case 2: LAUNCH(__nv_bfloat16, float); break;
    case 3: LAUNCH(__nv_bfloat16, __nv_bfloat16); break;
    default: FG_CHECK_ARG(false, "fg_rmsnorm_sum: bad dtypes");
  }
#undef LAUNCH
  FG_CHECK_LAUNCH("fg_rmsnorm_sum");
  return 0;
}
