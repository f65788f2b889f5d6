// Row-wise and element-wise mechanisms of the sequence mixers: embedding into an f32 residual stream, RMS norms
// (pre, post + residual + next pre fused), gated activations, short causal convolution with carried inputs, unit
// norms, decay factors, grouped read-out norm with its gate.  All arithmetic is f32; `act_t` is only the storage
// type of projection outputs and weights.
#include "seq_common.cuh"

namespace b2l {

template <typename act_t, typename idx_t>
__global__ void seq_embed_kernel(const idx_t* __restrict__ tok, const act_t* __restrict__ table, float scale,
                                 float* __restrict__ x, int D, int vocab) {
  long long t = (long long)tok[blockIdx.x];
  if (t < 0 || t >= vocab) t = 0;
  const act_t* src = table + (size_t)t * D;
  float* dst = x + (size_t)blockIdx.x * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x) dst[i] = ld_act(src, i) * scale;
}

template <typename act_t>
__global__ void __launch_bounds__(256) seq_rmsnorm_kernel(const float* __restrict__ x, const act_t* __restrict__ w, float eps,
                                                          act_t* __restrict__ out, const int* __restrict__ rows, int D) {
  __shared__ float red[32];
  const int r = rows ? rows[blockIdx.x] : blockIdx.x;
  const float* xr = x + (size_t)r * D;
  act_t* o = out + (size_t)blockIdx.x * D;
  float ss = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) ss += xr[i] * xr[i];
  ss = block_sum(ss, red);
  const float rinv = 1.0f / sqrtf(ss / (float)D + eps);
  for (int i = threadIdx.x; i < D; i += blockDim.x) st_act(o, i, xr[i] * rinv * ld_act(w, i));
}

// x += rmsnorm(y) * w_post; optionally h = rmsnorm(x) * w_next.  One CTA per row; the updated row stays in
// registers between the two passes when it fits (D <= 256 * 8), else it is re-read.
template <typename act_t>
__global__ void __launch_bounds__(256) seq_norm_add_norm_kernel(const act_t* __restrict__ y, const act_t* __restrict__ wp, float eps,
                                                                float* __restrict__ x, const act_t* __restrict__ wn,
                                                                act_t* __restrict__ h, int D) {
  __shared__ float red[32];
  const act_t* yr = y + (size_t)blockIdx.x * D;
  float* xr = x + (size_t)blockIdx.x * D;
  float ss = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    const float v = ld_act(yr, i);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float rinv = 1.0f / sqrtf(ss / (float)D + eps);
  float s2 = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    const float v = xr[i] + ld_act(yr, i) * rinv * ld_act(wp, i);
    xr[i] = v;
    s2 += v * v;
  }
  if (wn == nullptr) return;
  s2 = block_sum(s2, red);
  const float r2 = 1.0f / sqrtf(s2 / (float)D + eps);
  act_t* hr = h + (size_t)blockIdx.x * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x) st_act(hr, i, xr[i] * r2 * ld_act(wn, i));   // own writes: visible to this thread
}

// The same with the row held in registers (D <= 256 * EPT): every operand is requested before the first reduction, so
// a single-token step pays one memory latency instead of three.
template <typename act_t, int EPT>
__global__ void __launch_bounds__(256) seq_norm_add_norm_reg_kernel(const act_t* __restrict__ y, const act_t* __restrict__ wp, float eps,
                                                                    float* __restrict__ x, const act_t* __restrict__ wn,
                                                                    act_t* __restrict__ h, int D) {
  __shared__ float red[32];
  const act_t* yr = y + (size_t)blockIdx.x * D;
  float* xr = x + (size_t)blockIdx.x * D;
  float yv[EPT], xv[EPT], pv[EPT], nv[EPT];
#pragma unroll
  for (int e = 0; e < EPT; ++e) {
    const int i = threadIdx.x + e * 256;
    const bool in = i < D;
    yv[e] = in ? ld_act(yr, i) : 0.f;
    xv[e] = in ? xr[i] : 0.f;
    pv[e] = in ? ld_act(wp, i) : 0.f;
    nv[e] = (in && wn) ? ld_act(wn, i) : 0.f;
  }
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < EPT; ++e) ss += yv[e] * yv[e];
  ss = block_sum(ss, red);
  const float rinv = 1.0f / sqrtf(ss / (float)D + eps);
  float s2 = 0.f;
#pragma unroll
  for (int e = 0; e < EPT; ++e) {
    const int i = threadIdx.x + e * 256;
    xv[e] += yv[e] * rinv * pv[e];
    if (i < D) xr[i] = xv[e];
    s2 += xv[e] * xv[e];
  }
  if (wn == nullptr) return;
  s2 = block_sum(s2, red);
  const float r2 = 1.0f / sqrtf(s2 / (float)D + eps);
  act_t* hr = h + (size_t)blockIdx.x * D;
#pragma unroll
  for (int e = 0; e < EPT; ++e) {
    const int i = threadIdx.x + e * 256;
    if (i < D) st_act(hr, i, xv[e] * r2 * nv[e]);
  }
}

// Moved to seq_common.cuh: gated_pair(a, b, act, limit) = act(a) * b, or the clamped unit.

// 16-byte form (F and ldgu multiples of 8 elements, aligned pointers): eight bf16 or four f32 numbers per load.
template <typename act_t>
__global__ void seq_gated_act_vec_kernel(const act_t* __restrict__ gu, int ldgu, act_t* __restrict__ out, int F, int act, float limit) {
  constexpr int PER = 16 / sizeof(act_t);
  const act_t* g = gu + (size_t)blockIdx.x * ldgu;
  act_t* o = out + (size_t)blockIdx.x * F;
  for (int j = (blockIdx.y * blockDim.x + threadIdx.x) * PER; j < F; j += gridDim.y * blockDim.x * PER) {
    const uint4 a4 = *reinterpret_cast<const uint4*>(g + j), b4 = *reinterpret_cast<const uint4*>(g + F + j);
    uint4 r4;
    if (sizeof(act_t) == 2) {
      const uint32_t aw[4] = {a4.x, a4.y, a4.z, a4.w}, bw[4] = {b4.x, b4.y, b4.z, b4.w};
      uint32_t rw[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float lo = gated_pair(__uint_as_float(aw[q] << 16), __uint_as_float(bw[q] << 16), act, limit);
        const float hi = gated_pair(__uint_as_float(aw[q] & 0xffff0000u), __uint_as_float(bw[q] & 0xffff0000u), act, limit);
        const __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
        rw[q] = *reinterpret_cast<const uint32_t*>(&t);
      }
      r4 = make_uint4(rw[0], rw[1], rw[2], rw[3]);
    } else {
      r4.x = __float_as_uint(gated_pair(__uint_as_float(a4.x), __uint_as_float(b4.x), act, limit));
      r4.y = __float_as_uint(gated_pair(__uint_as_float(a4.y), __uint_as_float(b4.y), act, limit));
      r4.z = __float_as_uint(gated_pair(__uint_as_float(a4.z), __uint_as_float(b4.z), act, limit));
      r4.w = __float_as_uint(gated_pair(__uint_as_float(a4.w), __uint_as_float(b4.w), act, limit));
    }
    *reinterpret_cast<uint4*>(o + j) = r4;
  }
}

template <typename act_t>
__global__ void seq_gated_act_kernel(const act_t* __restrict__ gu, int ldgu, act_t* __restrict__ out, int F, int act, float limit) {
  const act_t* g = gu + (size_t)blockIdx.x * ldgu;
  act_t* o = out + (size_t)blockIdx.x * F;
  for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < F; j += gridDim.y * blockDim.x) {
    const float a = ld_act(g, j), b = ld_act(g, (size_t)F + j);
    st_act(o, j, gated_pair(a, b, act, limit));
  }
}

// Causal convolution + silu.  Thread = one channel over a tile of CONV_TT tokens with a sliding window in registers.
// Tile 0 reads the carried inputs; with a single tile the same thread also advances the state (no race); with
// several tiles seq_conv_state_kernel advances it in a second launch.
constexpr int CONV_TT = 32;
constexpr int CONV_MAX_TAPS = 8;
template <typename act_t>
__global__ void seq_conv_silu_kernel(const act_t* __restrict__ in, int ldin, const act_t* __restrict__ w,
                                     const act_t* __restrict__ bias, act_t* __restrict__ state, const int* __restrict__ meta,
                                     float* __restrict__ out, int ldout, int T, int C, int taps, int update_state) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int t0 = blockIdx.y * CONV_TT, t1 = min(T, t0 + CONV_TT);
  act_t* st = state + (size_t)meta[0] * (taps - 1) * C;
  float wr[CONV_MAX_TAPS], win[CONV_MAX_TAPS];   // win[j] = input at t - (taps-1) + j
#pragma unroll
  for (int j = 0; j < CONV_MAX_TAPS; ++j) wr[j] = j < taps ? ld_act(w, (size_t)c * taps + j) : 0.f;
  const float b = bias ? ld_act(bias, c) : 0.f;
#pragma unroll
  for (int j = 0; j < CONV_MAX_TAPS; ++j) {
    win[j] = 0.f;
    if (j < taps - 1) {
      const int t = t0 - (taps - 1) + j;   // input index relative to the portion
      win[j] = t >= 0 ? ld_act(in, (size_t)t * ldin + c) : ld_act(st, (size_t)(taps - 1 + t) * C + c);
    }
  }
  for (int t = t0; t < t1; ++t) {
    const float cur = ld_act(in, (size_t)t * ldin + c);
    float acc = b;
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; ++j) {
      if (j < taps - 1) acc += wr[j] * win[j];
    }
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; ++j) {
      if (j == taps - 1) acc += wr[j] * cur;
    }
    out[(size_t)t * ldout + c] = silu_f(acc);
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS - 1; ++j) {
      if (j < taps - 2) win[j] = win[j + 1];
    }
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; ++j) {
      if (j == taps - 2) win[j] = cur;
    }
  }
  if (update_state) {   // single tile: win[] now holds the last taps-1 inputs of the sequence
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; ++j) {
      if (j < taps - 1) st_act(st, (size_t)j * C + c, win[j]);
    }
  }
}

// state <- the last taps-1 inputs after T >= taps-1 new tokens (multi-tile launches only).
template <typename act_t>
__global__ void seq_conv_state_kernel(const act_t* __restrict__ in, int ldin, act_t* __restrict__ state,
                                      const int* __restrict__ meta, int T, int C, int taps) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  act_t* st = state + (size_t)meta[0] * (taps - 1) * C;
  for (int j = 0; j < taps - 1; ++j) st[(size_t)j * C + c] = in[(size_t)(T - (taps - 1) + j) * ldin + c];
}

template <typename act_t>
__global__ void seq_cast_f32_kernel(const act_t* __restrict__ in, int ldin, float* __restrict__ out, int ldout, int n) {
  const act_t* p = in + (size_t)blockIdx.x * ldin;
  float* q = out + (size_t)blockIdx.x * ldout;
  for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < n; j += gridDim.y * blockDim.x) q[j] = ld_act(p, j);
}

// One warp per (token, head): x * mult / sqrt(sum x^2 + eps), in place.
__global__ void seq_unit_norm_kernel(float* __restrict__ x, int ld, int n_groups, int heads, int size, float eps, float mult) {
  const int g = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (g >= n_groups) return;
  float* p = x + (size_t)(g / heads) * ld + (size_t)(g % heads) * size;
  float ss = 0.f;
  for (int i = lane; i < size; i += 32) ss += p[i] * p[i];
  ss = warp_sum(ss);
  const float r = mult / sqrtf(ss + eps);
  for (int i = lane; i < size; i += 32) p[i] *= r;
}

template <typename act_t>
__global__ void seq_decay_kernel(const act_t* __restrict__ a, int lda, const act_t* __restrict__ bias,
                                 const act_t* __restrict__ A_log, int mode, float inv_tau, float* __restrict__ out,
                                 float* __restrict__ dt_out, int heads, int size) {
  const int n = heads * size;
  const act_t* ar = a + (size_t)blockIdx.x * lda;
  for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < n; j += gridDim.y * blockDim.x) {
    const float z = ld_act(ar, j) + (bias ? ld_act(bias, j) : 0.f);
    float r;
    if (mode == B2L_SEQ_DECAY_EXP_SOFTPLUS) {
      const float dt = softplus_f(z);
      if (dt_out) dt_out[(size_t)blockIdx.x * n + j] = dt;
      r = expf(-expf(ld_act(A_log, j / size)) * dt);
    } else {
      // sigmoid(z)^(1/tau) = exp(-softplus(-z) / tau): no underflow of the sigmoid for very negative z
      r = expf(-softplus_f(-z) * inv_tau);
    }
    out[(size_t)blockIdx.x * n + j] = r;
  }
}

// One warp per (token, group).
template <typename act_t>
__global__ void seq_group_norm_gate_kernel(const float* __restrict__ o, int ldo, const act_t* __restrict__ w, int w_shared,
                                           const act_t* __restrict__ gate, int ldg, int gate_act, int gate_first, float eps,
                                           float out_mult, act_t* __restrict__ out, int ldout, int n_rows, int groups, int group) {
  const int id = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (id >= n_rows * groups) return;
  const int t = id / groups, g = id % groups;
  const float* p = o + (size_t)t * ldo + (size_t)g * group;
  const act_t* gp = gate ? gate + (size_t)t * ldg + (size_t)g * group : nullptr;
  auto gate_of = [&](int i) {
    const float z = ld_act(gp, i);
    return gate_act == B2L_SEQ_ACT_SILU ? silu_f(z) : (gate_act == B2L_SEQ_ACT_SIGMOID ? sigmoid_f(z) : gelu_tanh_f(z));
  };
  float ss = 0.f;
  for (int i = lane; i < group; i += 32) {
    float v = p[i];
    if (gp && gate_first) v *= gate_of(i);
    ss += v * v;
  }
  ss = warp_sum(ss);
  const float r = out_mult / sqrtf(ss / (float)group + eps);
  act_t* q = out + (size_t)t * ldout + (size_t)g * group;
  for (int i = lane; i < group; i += 32) {
    float v = p[i];
    if (gp && gate_first) v *= gate_of(i);
    v = v * r * ld_act(w, w_shared ? i : g * group + i);
    if (gp && !gate_first) v *= gate_of(i);
    st_act(q, i, v);
  }
}

// The same for large groups (a whole layer's channels normalised together): one CTA per (token, group).
template <typename act_t>
__global__ void __launch_bounds__(256) seq_group_norm_gate_block_kernel(const float* __restrict__ o, int ldo, const act_t* __restrict__ w, int w_shared,
                                                                        const act_t* __restrict__ gate, int ldg, int gate_act, int gate_first,
                                                                        float eps, float out_mult, act_t* __restrict__ out, int ldout, int groups,
                                                                        int group) {
  __shared__ float red[32];
  const int t = blockIdx.x / groups, g = blockIdx.x % groups;
  const float* p = o + (size_t)t * ldo + (size_t)g * group;
  const act_t* gp = gate ? gate + (size_t)t * ldg + (size_t)g * group : nullptr;
  auto gate_of = [&](int i) {
    const float z = ld_act(gp, i);
    return gate_act == B2L_SEQ_ACT_SILU ? silu_f(z) : (gate_act == B2L_SEQ_ACT_SIGMOID ? sigmoid_f(z) : gelu_tanh_f(z));
  };
  float ss = 0.f;
  for (int i = threadIdx.x; i < group; i += blockDim.x) {
    float v = p[i];
    if (gp && gate_first) v *= gate_of(i);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float r = out_mult / sqrtf(ss / (float)group + eps);
  act_t* q = out + (size_t)t * ldout + (size_t)g * group;
  for (int i = threadIdx.x; i < group; i += blockDim.x) {
    float v = p[i];
    if (gp && gate_first) v *= gate_of(i);
    v = v * r * ld_act(w, w_shared ? i : g * group + i);
    if (gp && !gate_first) v *= gate_of(i);
    st_act(q, i, v);
  }
}

// Per-head RMS norm + partial rotation.  One warp per (token, head).
template <typename act_t, typename out_t>
__global__ void seq_headnorm_rope_kernel(const act_t* __restrict__ x, int ldx, const act_t* __restrict__ w, float eps,
                                         const float* __restrict__ freq, int rot_dims, float rot_mult,
                                         const int* __restrict__ meta, out_t* __restrict__ out, int n_rows, int heads, int size) {
  const int id = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (id >= n_rows * heads) return;
  const int t = id / heads, hd = id % heads;
  const act_t* p = x + (size_t)t * ldx + (size_t)hd * size;
  out_t* q = out + ((size_t)t * heads + hd) * size;
  float r = 1.f;
  if (w) {
    float ss = 0.f;
    for (int i = lane; i < size; i += 32) {
      const float v = ld_act(p, i);
      ss += v * v;
    }
    ss = warp_sum(ss);
    r = 1.0f / sqrtf(ss / (float)size + eps);
  }
  const float pos = (float)(meta[1] + t);
  const int half = rot_dims / 2;
  for (int i = lane; i < half; i += 32) {
    const float u = ld_act(p, i) * r * (w ? ld_act(w, i) : 1.f);
    const float v = ld_act(p, i + half) * r * (w ? ld_act(w, i + half) : 1.f);
    float s, c;
    sincosf(pos * freq[i], &s, &c);
    s *= rot_mult;
    c *= rot_mult;
    st_act(q, i, u * c - v * s);
    st_act(q, i + half, v * c + u * s);
  }
  for (int i = rot_dims + lane; i < size; i += 32) st_act(q, i, ld_act(p, i) * r * (w ? ld_act(w, i) : 1.f));
}

}  // namespace b2l

using namespace b2l;

extern "C" int b2l_seq_embed(const void* tokens, int tokens_i64, const void* table, int act_dtype, float scale, float* x,
                             int T, int D, int vocab, b2l_stream_t stream) {
  B2L_CHECK_ARG(tokens && table && x, "b2l_seq_embed: null pointer");
  B2L_CHECK_ARG(T >= 0 && D > 0 && vocab > 0, "b2l_seq_embed: bad size");
  if (T == 0) return 0;
  B2L_SEQ_DISPATCH(act_dtype, {
    if (tokens_i64)
      seq_embed_kernel<act_t, long long><<<T, 128, 0, (cudaStream_t)stream>>>((const long long*)tokens, (const act_t*)table, scale, x, D, vocab);
    else
      seq_embed_kernel<act_t, int><<<T, 128, 0, (cudaStream_t)stream>>>((const int*)tokens, (const act_t*)table, scale, x, D, vocab);
  });
  B2L_LAUNCH_CHECK("seq_embed_kernel");
  return 0;
}

extern "C" int b2l_seq_rmsnorm(const float* x, const void* w, float eps, void* out, const int* rows, int n_rows, int D,
                               int act_dtype, b2l_stream_t stream) {
  B2L_CHECK_ARG(x && w && out, "b2l_seq_rmsnorm: null pointer");
  B2L_CHECK_ARG(n_rows >= 0 && D > 0, "b2l_seq_rmsnorm: bad size");
  if (n_rows == 0) return 0;
  B2L_SEQ_DISPATCH(act_dtype, (seq_rmsnorm_kernel<act_t><<<n_rows, 256, 0, (cudaStream_t)stream>>>(x, (const act_t*)w, eps, (act_t*)out, rows, D)));
  B2L_LAUNCH_CHECK("seq_rmsnorm_kernel");
  return 0;
}

extern "C" int b2l_seq_norm_add_norm(const void* y, const void* w_post, float eps, float* x, const void* w_next, void* h,
                                     int T, int D, int act_dtype, b2l_stream_t stream) {
  B2L_CHECK_ARG(y && w_post && x, "b2l_seq_norm_add_norm: null pointer");
  B2L_CHECK_ARG((w_next == nullptr) == (h == nullptr), "b2l_seq_norm_add_norm: w_next and h go together");
  B2L_CHECK_ARG(T >= 0 && D > 0, "b2l_seq_norm_add_norm: bad size");
  if (T == 0) return 0;
#define B2L_NAN_ARGS (const act_t*)y, (const act_t*)w_post, eps, x, (const act_t*)w_next, (act_t*)h, D
  B2L_SEQ_DISPATCH(act_dtype, {
    cudaStream_t s_ = (cudaStream_t)stream;
    if (D <= 1024) seq_norm_add_norm_reg_kernel<act_t, 4><<<T, 256, 0, s_>>>(B2L_NAN_ARGS);
    else if (D <= 2048) seq_norm_add_norm_reg_kernel<act_t, 8><<<T, 256, 0, s_>>>(B2L_NAN_ARGS);
    else if (D <= 4096) seq_norm_add_norm_reg_kernel<act_t, 16><<<T, 256, 0, s_>>>(B2L_NAN_ARGS);
    else seq_norm_add_norm_kernel<act_t><<<T, 256, 0, s_>>>(B2L_NAN_ARGS);
  });
#undef B2L_NAN_ARGS
  B2L_LAUNCH_CHECK("seq_norm_add_norm_kernel");
  return 0;
}

extern "C" int b2l_seq_gated_act(const void* gu, int ldgu, void* out, int T, int F, int act, float limit, int act_dtype, b2l_stream_t stream) {
  B2L_CHECK_ARG(gu && out, "b2l_seq_gated_act: null pointer");
  B2L_CHECK_ARG(T >= 0 && F > 0 && ldgu >= 2 * F, "b2l_seq_gated_act: bad size");
  B2L_CHECK_ARG(act >= 0 && act <= 3, "b2l_seq_gated_act: unknown activation %d", act);
  B2L_CHECK_ARG(act != B2L_SEQ_ACT_CLAMPED_SWISH || limit > 0.f, "b2l_seq_gated_act: the clamped unit needs a positive limit");
  if (T == 0) return 0;
  const bool vec = F % 8 == 0 && ldgu % 8 == 0 && (((uintptr_t)gu | (uintptr_t)out) & 15) == 0;
  B2L_SEQ_DISPATCH(act_dtype, {
    if (vec) {
      const int per = 16 / (int)sizeof(act_t);
      dim3 grid((unsigned)T, (unsigned)std::min((F / per + 255) / 256, 64));
      seq_gated_act_vec_kernel<act_t><<<grid, 256, 0, (cudaStream_t)stream>>>((const act_t*)gu, ldgu, (act_t*)out, F, act, limit);
    } else {
      dim3 grid((unsigned)T, (unsigned)std::min((F + 255) / 256, 64));
      seq_gated_act_kernel<act_t><<<grid, 256, 0, (cudaStream_t)stream>>>((const act_t*)gu, ldgu, (act_t*)out, F, act, limit);
    }
  });
  B2L_LAUNCH_CHECK("seq_gated_act_kernel");
  return 0;
}

extern "C" int b2l_seq_conv_silu(const void* in, int ldin, const void* w, const void* bias, void* state, const int* meta,
                                 float* out, int ldout, int T, int C, int taps, int act_dtype, b2l_stream_t stream) {
  B2L_CHECK_ARG(in && w && (state || taps == 1) && meta && out, "b2l_seq_conv_silu: null pointer");
  B2L_CHECK_ARG(T >= 0 && C > 0 && ldin >= C && ldout >= C, "b2l_seq_conv_silu: bad size");
  B2L_CHECK_SUPPORTED(taps >= 1 && taps <= CONV_MAX_TAPS, "b2l_seq_conv_silu: taps %d outside 1..%d", taps, CONV_MAX_TAPS);
  if (T == 0) return 0;
  const int tiles = (T + CONV_TT - 1) / CONV_TT;
  dim3 grid((unsigned)((C + 127) / 128), (unsigned)tiles);
  B2L_SEQ_DISPATCH(act_dtype, {
    seq_conv_silu_kernel<act_t><<<grid, 128, 0, (cudaStream_t)stream>>>((const act_t*)in, ldin, (const act_t*)w, (const act_t*)bias,
                                                                        (act_t*)state, meta, out, ldout, T, C, taps, tiles == 1);
    if (tiles > 1 && taps > 1)   // T > CONV_TT >= taps - 1: the new state comes from the portion alone
      seq_conv_state_kernel<act_t><<<(C + 127) / 128, 128, 0, (cudaStream_t)stream>>>((const act_t*)in, ldin, (act_t*)state, meta, T, C, taps);
  });
  B2L_LAUNCH_CHECK("seq_conv_silu_kernel");
  return 0;
}

extern "C" int b2l_seq_cast_f32(const void* in, int ldin, float* out, int ldout, int T, int n, int act_dtype, b2l_stream_t stream) {
  B2L_CHECK_ARG(in && out, "b2l_seq_cast_f32: null pointer");
  B2L_CHECK_ARG(T >= 0 && n > 0 && ldin >= n && ldout >= n, "b2l_seq_cast_f32: bad size");
  if (T == 0) return 0;
  dim3 grid((unsigned)T, (unsigned)std::min((n + 255) / 256, 64));
  B2L_SEQ_DISPATCH(act_dtype, (seq_cast_f32_kernel<act_t><<<grid, 256, 0, (cudaStream_t)stream>>>((const act_t*)in, ldin, out, ldout, n)));
  B2L_LAUNCH_CHECK("seq_cast_f32_kernel");
  return 0;
}

extern "C" int b2l_seq_unit_norm(float* x, int ld, int T, int heads, int size, float eps, float mult, b2l_stream_t stream) {
  B2L_CHECK_ARG(x != nullptr, "b2l_seq_unit_norm: null pointer");
  B2L_CHECK_ARG(T >= 0 && heads > 0 && size > 0 && ld >= heads * size, "b2l_seq_unit_norm: bad size");
  if (T == 0) return 0;
  const int n = T * heads;
  seq_unit_norm_kernel<<<(n + 3) / 4, 128, 0, (cudaStream_t)stream>>>(x, ld, n, heads, size, eps, mult);
  B2L_LAUNCH_CHECK("seq_unit_norm_kernel");
  return 0;
}

extern "C" int b2l_seq_decay(const void* a, int lda, const void* bias, const void* A_log, int mode, float tau, float* out,
                             float* dt_out, int T, int heads, int size, int act_dtype, b2l_stream_t stream) {
  B2L_CHECK_ARG(a && out, "b2l_seq_decay: null pointer");
  B2L_CHECK_ARG(T >= 0 && heads > 0 && size > 0 && lda >= heads * size, "b2l_seq_decay: bad size");
  B2L_CHECK_ARG(mode == B2L_SEQ_DECAY_SIGMOID_ROOT || (mode == B2L_SEQ_DECAY_EXP_SOFTPLUS && A_log), "b2l_seq_decay: bad mode or no A_log");
  B2L_CHECK_ARG(mode != B2L_SEQ_DECAY_SIGMOID_ROOT || tau > 0.f, "b2l_seq_decay: tau must be positive");
  if (T == 0) return 0;
  const int n = heads * size;
  dim3 grid((unsigned)T, (unsigned)std::min((n + 255) / 256, 64));
  B2L_SEQ_DISPATCH(act_dtype, (seq_decay_kernel<act_t><<<grid, 256, 0, (cudaStream_t)stream>>>(
                                  (const act_t*)a, lda, (const act_t*)bias, (const act_t*)A_log, mode, mode == B2L_SEQ_DECAY_SIGMOID_ROOT ? 1.0f / tau : 0.f,
                                  out, dt_out, heads, size)));
  B2L_LAUNCH_CHECK("seq_decay_kernel");
  return 0;
}

extern "C" int b2l_seq_group_norm_gate(const float* o, int ldo, const void* w, int w_shared, const void* gate, int ldg,
                                       int gate_act, int gate_first, float eps, float out_mult, void* out, int ldout, int T,
                                       int n, int group, int act_dtype, b2l_stream_t stream) {
  B2L_CHECK_ARG(o && w && out, "b2l_seq_group_norm_gate: null pointer");
  B2L_CHECK_ARG(T >= 0 && n > 0 && group > 0 && n % group == 0 && ldo >= n && ldout >= n, "b2l_seq_group_norm_gate: bad size");
  if (T == 0) return 0;
  const int ids = T * (n / group);
  B2L_SEQ_DISPATCH(act_dtype, {
    if (group >= 512)
      seq_group_norm_gate_block_kernel<act_t><<<ids, 256, 0, (cudaStream_t)stream>>>(
          o, ldo, (const act_t*)w, w_shared, (const act_t*)gate, ldg, gate_act, gate_first, eps, out_mult, (act_t*)out, ldout, n / group, group);
    else
      seq_group_norm_gate_kernel<act_t><<<(ids + 3) / 4, 128, 0, (cudaStream_t)stream>>>(
          o, ldo, (const act_t*)w, w_shared, (const act_t*)gate, ldg, gate_act, gate_first, eps, out_mult, (act_t*)out, ldout, T, n / group, group);
  });
  B2L_LAUNCH_CHECK("seq_group_norm_gate_kernel");
  return 0;
}

extern "C" int b2l_seq_headnorm_rope(const void* x, int ldx, const void* w, float eps, const float* freq, int rot_dims,
                                     float rot_mult, const int* meta, void* out, int out_f32, int T, int heads, int size,
                                     int act_dtype, b2l_stream_t stream) {
  B2L_CHECK_ARG(x && meta && out, "b2l_seq_headnorm_rope: null pointer");
  B2L_CHECK_ARG(T >= 0 && heads > 0 && size > 0 && ldx >= heads * size, "b2l_seq_headnorm_rope: bad size");
  B2L_CHECK_ARG(rot_dims >= 0 && rot_dims <= size && rot_dims % 2 == 0 && (rot_dims == 0 || freq), "b2l_seq_headnorm_rope: bad rotation");
  if (T == 0) return 0;
  const int ids = T * heads;
  B2L_SEQ_DISPATCH(act_dtype, {
    if (out_f32)
      seq_headnorm_rope_kernel<act_t, float><<<(ids + 3) / 4, 128, 0, (cudaStream_t)stream>>>(
          (const act_t*)x, ldx, (const act_t*)w, eps, freq, rot_dims, rot_mult, meta, (float*)out, T, heads, size);
    else
      seq_headnorm_rope_kernel<act_t, act_t><<<(ids + 3) / 4, 128, 0, (cudaStream_t)stream>>>(
          (const act_t*)x, ldx, (const act_t*)w, eps, freq, rot_dims, rot_mult, meta, (act_t*)out, T, heads, size);
  });
  B2L_LAUNCH_CHECK("seq_headnorm_rope_kernel");
  return 0;
}

// ---- residual streams with two sublayers on the same input ----
namespace b2l {

// x += y1 + y2 (each may be null), then up to two RMS norms of the new row with weights stored around `w_offset`
// (h = x / rms(x) * (w_offset + w)): a layer whose mixer and feed-forward read the same x with a norm each.  `rows`
// picks the rows (out row r <- x row rows[r]) when nothing is added.  One CTA per row; the sum is f32.
template <typename act_t>
__global__ void __launch_bounds__(256) seq_add_norm2_kernel(const act_t* __restrict__ y1, const act_t* __restrict__ y2, float* __restrict__ x,
                                                            const act_t* __restrict__ w1, act_t* __restrict__ h1,
                                                            const act_t* __restrict__ w2, act_t* __restrict__ h2, float w_offset, float eps,
                                                            const int* __restrict__ rows, int D) {
  __shared__ float red[32];
  const int r = rows ? rows[blockIdx.x] : blockIdx.x;
  float* xr = x + (size_t)r * D;
  float ss = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float v = xr[i];
    if (y1) {
      float add = ld_act(y1, (size_t)r * D + i);
      if (y2) add += ld_act(y2, (size_t)r * D + i);
      v += add;
      xr[i] = v;
    }
    ss += v * v;
  }
  if (w1 == nullptr) return;
  ss = block_sum(ss, red);
  const float rinv = 1.0f / sqrtf(ss / (float)D + eps);
  for (int i = threadIdx.x; i < D; i += blockDim.x) {       // own writes of xr: visible to this thread
    const float v = xr[i] * rinv;
    st_act(h1, (size_t)blockIdx.x * D + i, v * (w_offset + ld_act(w1, i)));
    if (w2) st_act(h2, (size_t)blockIdx.x * D + i, v * (w_offset + ld_act(w2, i)));
  }
}

__global__ void seq_softcap_kernel(float* __restrict__ z, size_t n, float cap) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) z[i] = cap * tanhf(z[i] / cap);
}

}  // namespace b2l

extern "C" int b2l_seq_add_norm2(const void* y1, const void* y2, float* x, const void* w1, void* h1, const void* w2, void* h2,
                                 float w_offset, float eps, const int* rows, int n_rows, int D, int act_dtype, b2l_stream_t stream) {
  B2L_CHECK_ARG(x != nullptr && (y1 != nullptr || y2 == nullptr), "b2l_seq_add_norm2: null pointer");
  B2L_CHECK_ARG((w1 == nullptr) == (h1 == nullptr) && (w2 == nullptr) == (h2 == nullptr) && (w1 != nullptr || w2 == nullptr),
                "b2l_seq_add_norm2: every norm needs its weight and its output, the second norm needs the first");
  B2L_CHECK_ARG(rows == nullptr || y1 == nullptr, "b2l_seq_add_norm2: rows are picked only when nothing is added");
  B2L_CHECK_ARG(n_rows >= 0 && D > 0, "b2l_seq_add_norm2: bad size");
  if (n_rows == 0 || (y1 == nullptr && w1 == nullptr)) return 0;
  B2L_SEQ_DISPATCH(act_dtype, {
    seq_add_norm2_kernel<act_t><<<n_rows, 256, 0, (cudaStream_t)stream>>>((const act_t*)y1, (const act_t*)y2, x, (const act_t*)w1, (act_t*)h1,
                                                                         (const act_t*)w2, (act_t*)h2, w_offset, eps, rows, D);
  });
  B2L_LAUNCH_CHECK("seq_add_norm2_kernel");
  return 0;
}

extern "C" int b2l_seq_softcap(float* z, size_t n, float cap, b2l_stream_t stream) {
  B2L_CHECK_ARG(z != nullptr && cap > 0.f, "b2l_seq_softcap: null pointer or cap <= 0");
  if (n == 0) return 0;
  const int grid = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
  b2l::seq_softcap_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(z, n, cap);
  B2L_LAUNCH_CHECK("seq_softcap_kernel");
  return 0;
}
