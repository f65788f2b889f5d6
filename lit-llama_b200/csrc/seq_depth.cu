// Norms with a bias, the residual step of layers that read a learned average over the results of all earlier layers,
// and ungated feed-forward activations.  Sums, means and the average are f32; `act_t` is only the storage type of
// sublayer results, weights and the normed output.
#include "seq_common.cuh"

namespace b2l {

constexpr int DEPTH_THREADS = 256;

// mean and 1 / sqrt(variance + eps) (layer norm) or 0 and 1 / sqrt(mean square + eps) (RMS norm) of a row held as
// `n` register values per thread.  Two passes over the registers: the variance is the mean of the squared deviations.
template <int EPT>
__device__ __forceinline__ void row_moments(const float (&v)[EPT], int D, int kind, float eps, float* red, float& mean, float& rinv) {
  mean = 0.f;
  if (kind == B2L_SEQ_NORM_LAYER) {
    float s = 0.f;
#pragma unroll
    for (int e = 0; e < EPT; ++e) s += v[e];                       // entries beyond D are 0
    mean = block_sum(s, red) / (float)D;
    __syncthreads();
  }
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < EPT; ++e) {
    const int i = threadIdx.x + e * DEPTH_THREADS;
    const float d = i < D ? v[e] - mean : 0.f;
    ss += d * d;
  }
  ss = block_sum(ss, red);
  rinv = 1.0f / sqrtf(ss / (float)D + eps);
}

template <typename act_t, int EPT>
__global__ void __launch_bounds__(DEPTH_THREADS) seq_norm_kernel(const float* __restrict__ x, const act_t* __restrict__ w,
                                                                 const act_t* __restrict__ b, int kind, float eps,
                                                                 act_t* __restrict__ out, const int* __restrict__ rows, int D) {
  __shared__ float red[32];
  const int r = rows ? rows[blockIdx.x] : blockIdx.x;
  const float* xr = x + (size_t)r * D;
  float v[EPT];
#pragma unroll
  for (int e = 0; e < EPT; ++e) {
    const int i = threadIdx.x + e * DEPTH_THREADS;
    v[e] = i < D ? xr[i] : 0.f;
  }
  float mean, rinv;
  row_moments<EPT>(v, D, kind, eps, red, mean, rinv);
  act_t* o = out + (size_t)blockIdx.x * D;
#pragma unroll
  for (int e = 0; e < EPT; ++e) {
    const int i = threadIdx.x + e * DEPTH_THREADS;
    if (i < D) st_act(o, i, (v[e] - mean) * rinv * ld_act(w, i) + (b ? ld_act(b, i) : 0.f));
  }
}

// Rows wider than the register form takes: three passes over global memory.
template <typename act_t>
__global__ void __launch_bounds__(DEPTH_THREADS) seq_norm_wide_kernel(const float* __restrict__ x, const act_t* __restrict__ w,
                                                                      const act_t* __restrict__ b, int kind, float eps,
                                                                      act_t* __restrict__ out, const int* __restrict__ rows, int D) {
  __shared__ float red[32];
  const int r = rows ? rows[blockIdx.x] : blockIdx.x;
  const float* xr = x + (size_t)r * D;
  float mean = 0.f;
  if (kind == B2L_SEQ_NORM_LAYER) {
    float s = 0.f;
    for (int i = threadIdx.x; i < D; i += DEPTH_THREADS) s += xr[i];
    mean = block_sum(s, red) / (float)D;
    __syncthreads();
  }
  float ss = 0.f;
  for (int i = threadIdx.x; i < D; i += DEPTH_THREADS) ss += (xr[i] - mean) * (xr[i] - mean);
  ss = block_sum(ss, red);
  const float rinv = 1.0f / sqrtf(ss / (float)D + eps);
  act_t* o = out + (size_t)blockIdx.x * D;
  for (int i = threadIdx.x; i < D; i += DEPTH_THREADS) st_act(o, i, (xr[i] - mean) * rinv * ld_act(w, i) + (b ? ld_act(b, i) : 0.f));
}

// One CTA per token: own result = x_in + y1 + y2 -> hist[n_hist-1]; x_out = sum_j avg[j] hist[j]; h = norm(x_out).
// The row stays in registers from the sum to the normed output; the earlier entries of hist are each read once.
template <typename act_t, int EPT>
__global__ void __launch_bounds__(DEPTH_THREADS) seq_depth_step_kernel(const act_t* __restrict__ y1, const act_t* __restrict__ y2,
                                                                       const float* x_in, float* __restrict__ hist, int n_hist,
                                                                       const float* __restrict__ avg, float* x_out,
                                                                       const act_t* __restrict__ wn, const act_t* __restrict__ bn, int kind,
                                                                       float eps, act_t* __restrict__ h, int T, int D) {
  __shared__ float red[32];
  const size_t row = (size_t)blockIdx.x * D, plane = (size_t)T * D;
  float v[EPT];
  float* own = hist + (size_t)(n_hist - 1) * plane + row;
  if (y1) {
#pragma unroll
    for (int e = 0; e < EPT; ++e) {
      const int i = threadIdx.x + e * DEPTH_THREADS;
      v[e] = 0.f;
      if (i < D) {
        float add = ld_act(y1, row + i);
        if (y2) add += ld_act(y2, row + i);
        v[e] = x_in[row + i] + add;
        own[i] = v[e];
      }
    }
  } else {
#pragma unroll
    for (int e = 0; e < EPT; ++e) {
      const int i = threadIdx.x + e * DEPTH_THREADS;
      v[e] = i < D ? own[i] : 0.f;
    }
  }
  if (avg) {
    const float last = avg[n_hist - 1];
#pragma unroll
    for (int e = 0; e < EPT; ++e) v[e] *= last;
    for (int j = 0; j + 1 < n_hist; ++j) {
      const float a = avg[j];
      const float* hj = hist + (size_t)j * plane + row;
#pragma unroll
      for (int e = 0; e < EPT; ++e) {
        const int i = threadIdx.x + e * DEPTH_THREADS;
        if (i < D) v[e] = fmaf(a, hj[i], v[e]);
      }
    }
  }
  if (x_out) {
#pragma unroll
    for (int e = 0; e < EPT; ++e) {
      const int i = threadIdx.x + e * DEPTH_THREADS;
      if (i < D) x_out[row + i] = v[e];
    }
  }
  if (wn == nullptr) return;
  float mean, rinv;
  row_moments<EPT>(v, D, kind, eps, red, mean, rinv);
#pragma unroll
  for (int e = 0; e < EPT; ++e) {
    const int i = threadIdx.x + e * DEPTH_THREADS;
    if (i < D) st_act(h, row + i, (v[e] - mean) * rinv * ld_act(wn, i) + (bn ? ld_act(bn, i) : 0.f));
  }
}

// exp(z) - 1 - z for z <= 0 without the cancellation of the plain form: the series z^2/2 + ... + z^7/5040 near zero (its
// first missing term is below 2^-23 of the sum for |z| < 1/4), exp(z) - 1 - z elsewhere, where the difference is at least
// 0.028 and an absolute error of 1e-7 is at most 4e-6 of it.  No branch: both forms are a handful of operations.
__device__ __forceinline__ float expm1_minus_z(float z) {
  const float series = z * z * fmaf(z, fmaf(z, fmaf(z, fmaf(z, fmaf(z, 1.0f / 5040.0f, 1.0f / 720.0f), 1.0f / 120.0f), 1.0f / 24.0f), 1.0f / 6.0f), 0.5f);
  const float plain = (expf(z) - 1.0f) - z;
  return z > -0.25f ? series : plain;
}

__device__ __forceinline__ float unary_act(float z, int act, float a, float b) {
  switch (act) {
    case B2L_SEQ_ACT_GELU_TANH: return gelu_tanh_f(z);
    case B2L_SEQ_ACT_SILU: return silu_f(z);
    case B2L_SEQ_ACT_SIGMOID: return sigmoid_f(z);
    case B2L_SEQ_ACT_XIELU: return (z > 0.f ? a * z * z : b * expm1_minus_z(fminf(z, 0.f))) + 0.5f * z;
    default: return z;
  }
}

template <typename act_t>
__global__ void seq_unary_act_kernel(const act_t* __restrict__ in, int ldin, act_t* __restrict__ out, int ldout, int F, int act,
                                     const float* __restrict__ coef) {
  const float a = coef ? coef[0] : 0.f, b = coef ? coef[1] : 0.f;
  const act_t* p = in + (size_t)blockIdx.x * ldin;
  act_t* q = out + (size_t)blockIdx.x * ldout;
  for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < F; j += gridDim.y * blockDim.x) st_act(q, j, unary_act(ld_act(p, j), act, a, b));
}

// 16-byte form: eight bf16 or four f32 numbers per load (F and the leading dimensions multiples of that, aligned pointers).
template <typename act_t>
__global__ void seq_unary_act_vec_kernel(const act_t* __restrict__ in, int ldin, act_t* __restrict__ out, int ldout, int F, int act,
                                         const float* __restrict__ coef) {
  constexpr int PER = 16 / sizeof(act_t);
  const float a = coef ? coef[0] : 0.f, b = coef ? coef[1] : 0.f;
  const act_t* p = in + (size_t)blockIdx.x * ldin;
  act_t* q = out + (size_t)blockIdx.x * ldout;
  for (int j = (blockIdx.y * blockDim.x + threadIdx.x) * PER; j < F; j += gridDim.y * blockDim.x * PER) {
    const uint4 u = *reinterpret_cast<const uint4*>(p + j);
    uint4 r;
    if (sizeof(act_t) == 2) {
      const uint32_t uw[4] = {u.x, u.y, u.z, u.w};
      uint32_t rw[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const __nv_bfloat162 t = __floats2bfloat162_rn(unary_act(__uint_as_float(uw[k] << 16), act, a, b),
                                                       unary_act(__uint_as_float(uw[k] & 0xffff0000u), act, a, b));
        rw[k] = *reinterpret_cast<const uint32_t*>(&t);
      }
      r = make_uint4(rw[0], rw[1], rw[2], rw[3]);
    } else {
      r.x = __float_as_uint(unary_act(__uint_as_float(u.x), act, a, b));
      r.y = __float_as_uint(unary_act(__uint_as_float(u.y), act, a, b));
      r.z = __float_as_uint(unary_act(__uint_as_float(u.z), act, a, b));
      r.w = __float_as_uint(unary_act(__uint_as_float(u.w), act, a, b));
    }
    *reinterpret_cast<uint4*>(q + j) = r;
  }
}

}  // namespace b2l

using namespace b2l;

extern "C" int b2l_seq_norm(const float* x, const void* w, const void* b, int kind, float eps, void* out, const int* rows, int n_rows,
                            int D, int act_dtype, b2l_stream_t stream) {
  B2L_CHECK_ARG(x && w && out, "b2l_seq_norm: null pointer");
  B2L_CHECK_ARG(kind == B2L_SEQ_NORM_RMS || kind == B2L_SEQ_NORM_LAYER, "b2l_seq_norm: unknown norm %d", kind);
  B2L_CHECK_ARG(n_rows >= 0 && D > 0, "b2l_seq_norm: bad size");
  if (n_rows == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
#define B2L_NORM_ARGS x, (const act_t*)w, (const act_t*)b, kind, eps, (act_t*)out, rows, D
  B2L_SEQ_DISPATCH(act_dtype, {
    if (D <= 1 * DEPTH_THREADS) seq_norm_kernel<act_t, 1><<<n_rows, DEPTH_THREADS, 0, s>>>(B2L_NORM_ARGS);
    else if (D <= 4 * DEPTH_THREADS) seq_norm_kernel<act_t, 4><<<n_rows, DEPTH_THREADS, 0, s>>>(B2L_NORM_ARGS);
    else if (D <= 8 * DEPTH_THREADS) seq_norm_kernel<act_t, 8><<<n_rows, DEPTH_THREADS, 0, s>>>(B2L_NORM_ARGS);
    else if (D <= 16 * DEPTH_THREADS) seq_norm_kernel<act_t, 16><<<n_rows, DEPTH_THREADS, 0, s>>>(B2L_NORM_ARGS);
    else seq_norm_wide_kernel<act_t><<<n_rows, DEPTH_THREADS, 0, s>>>(B2L_NORM_ARGS);
  });
#undef B2L_NORM_ARGS
  B2L_LAUNCH_CHECK("seq_norm_kernel");
  return 0;
}

extern "C" int b2l_seq_depth_step(const void* y1, const void* y2, const float* x_in, float* hist, int n_hist, const float* avg,
                                  float* x_out, const void* w_next, const void* b_next, int norm_kind, float eps, void* h, int T, int D,
                                  int act_dtype, b2l_stream_t stream) {
  B2L_CHECK_ARG(hist != nullptr && n_hist >= 1, "b2l_seq_depth_step: no history");
  B2L_CHECK_ARG(y1 != nullptr || y2 == nullptr, "b2l_seq_depth_step: a second result without the first");
  B2L_CHECK_ARG(y1 == nullptr || x_in != nullptr, "b2l_seq_depth_step: results without the layer's input");
  B2L_CHECK_ARG((w_next == nullptr) == (h == nullptr) && (w_next != nullptr || b_next == nullptr), "b2l_seq_depth_step: a norm needs its weight and its output");
  B2L_CHECK_ARG(norm_kind == B2L_SEQ_NORM_RMS || norm_kind == B2L_SEQ_NORM_LAYER, "b2l_seq_depth_step: unknown norm %d", norm_kind);
  B2L_CHECK_ARG(T >= 0 && D > 0, "b2l_seq_depth_step: bad size");
  B2L_CHECK_SUPPORTED(D <= 16 * DEPTH_THREADS, "b2l_seq_depth_step: width %d above %d", D, 16 * DEPTH_THREADS);
  if (T == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
#define B2L_DEPTH_ARGS (const act_t*)y1, (const act_t*)y2, x_in, hist, n_hist, avg, x_out, (const act_t*)w_next, (const act_t*)b_next, norm_kind, eps, (act_t*)h, T, D
  B2L_SEQ_DISPATCH(act_dtype, {
    if (D <= 1 * DEPTH_THREADS) seq_depth_step_kernel<act_t, 1><<<T, DEPTH_THREADS, 0, s>>>(B2L_DEPTH_ARGS);
    else if (D <= 4 * DEPTH_THREADS) seq_depth_step_kernel<act_t, 4><<<T, DEPTH_THREADS, 0, s>>>(B2L_DEPTH_ARGS);
    else if (D <= 8 * DEPTH_THREADS) seq_depth_step_kernel<act_t, 8><<<T, DEPTH_THREADS, 0, s>>>(B2L_DEPTH_ARGS);
    else seq_depth_step_kernel<act_t, 16><<<T, DEPTH_THREADS, 0, s>>>(B2L_DEPTH_ARGS);
  });
#undef B2L_DEPTH_ARGS
  B2L_LAUNCH_CHECK("seq_depth_step_kernel");
  return 0;
}

extern "C" int b2l_seq_unary_act(const void* in, int ldin, void* out, int ldout, int T, int F, int act, const float* coef, int act_dtype,
                                 b2l_stream_t stream) {
  B2L_CHECK_ARG(in && out, "b2l_seq_unary_act: null pointer");
  B2L_CHECK_ARG(T >= 0 && F > 0 && ldin >= F && ldout >= F, "b2l_seq_unary_act: bad size");
  B2L_CHECK_ARG(act == B2L_SEQ_ACT_GELU_TANH || act == B2L_SEQ_ACT_SILU || act == B2L_SEQ_ACT_SIGMOID || act == B2L_SEQ_ACT_XIELU,
                "b2l_seq_unary_act: unknown activation %d", act);
  B2L_CHECK_ARG(act != B2L_SEQ_ACT_XIELU || coef != nullptr, "b2l_seq_unary_act: xIELU without its two coefficients");
  if (T == 0) return 0;
  B2L_SEQ_DISPATCH(act_dtype, {
    const int per = 16 / (int)sizeof(act_t);
    const bool vec = F % per == 0 && ldin % per == 0 && ldout % per == 0 && (((uintptr_t)in | (uintptr_t)out) & 15) == 0;
    if (vec) {
      dim3 grid((unsigned)T, (unsigned)std::min((F / per + 255) / 256, 64));
      seq_unary_act_vec_kernel<act_t><<<grid, 256, 0, (cudaStream_t)stream>>>((const act_t*)in, ldin, (act_t*)out, ldout, F, act, coef);
    } else {
      dim3 grid((unsigned)T, (unsigned)std::min((F + 255) / 256, 64));
      seq_unary_act_kernel<act_t><<<grid, 256, 0, (cudaStream_t)stream>>>((const act_t*)in, ldin, (act_t*)out, ldout, F, act, coef);
    }
  });
  B2L_LAUNCH_CHECK("seq_unary_act_kernel");
  return 0;
}
