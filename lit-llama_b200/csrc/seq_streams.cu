// Several residual streams (hyper-connections), a hashed token-pair embedding beside the token embedding, and the
// preparation of attention operands from one stacked projection: RMS norm of queries and keys (over the whole
// projection or per head), partial rotation, and the mixing of values with those of an earlier layer.
// All arithmetic is f32; `act_t` is only the storage type of projection outputs and weights.
#include "seq_common.cuh"

namespace b2l {

constexpr int HC_MAX_STREAMS = 16;

// x[t, s, :] = table[token[t]] * scale + pair[row(t)] for every stream s, with
//   row(t) = (previous token * mul_prev + token[t] * mul_cur) mod buckets, and row `buckets` at position 0.
// The previous token of the portion's first token is the sequence's state (int32 per slot); the CTA of token 0 reads
// it and then stores the portion's last token there, so no other CTA touches the state.
template <typename act_t, typename idx_t>
__global__ void seq_embed_pair_kernel(const idx_t* __restrict__ tok, const act_t* __restrict__ table, const act_t* __restrict__ pair,
                                      float scale, int* __restrict__ prev_state, const int* __restrict__ meta, long long mul_prev,
                                      long long mul_cur, int buckets, float* __restrict__ x, int T, int D, int vocab, int streams) {
  const int t = blockIdx.x;
  long long cur = (long long)tok[t];
  if (cur < 0 || cur >= vocab) cur = 0;
  long long row = -1;
  if (pair != nullptr) {
    __shared__ long long s_prev;
    if (threadIdx.x == 0) {
      long long prev;
      if (t > 0) {
        prev = (long long)tok[t - 1];
        if (prev < 0 || prev >= vocab) prev = 0;
      } else {
        prev = meta[1] > 0 ? (long long)prev_state[meta[0]] : -1;
        long long last = (long long)tok[T - 1];
        if (last < 0 || last >= vocab) last = 0;
        prev_state[meta[0]] = (int)last;
      }
      s_prev = prev;
    }
    __syncthreads();
    const long long prev = s_prev;
    // (prev * mul_prev + cur * mul_cur) mod buckets with every factor reduced first: no overflow for any multiplier
    const long long b = buckets;
    row = prev < 0 ? b : ((prev % b) * (mul_prev % b) + (cur % b) * (mul_cur % b)) % b;
  }
  const act_t* src = table + (size_t)cur * D;
  const act_t* add = row >= 0 ? pair + (size_t)row * D : nullptr;
  float* dst = x + (size_t)t * streams * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float v = ld_act(src, i) * scale;
    if (add) v += ld_act(add, i);
    for (int s = 0; s < streams; ++s) dst[(size_t)s * D + i] = v;
  }
}

// One sublayer's step on S residual streams X [rows][S][D] (f32), one CTA per row:
//   write (y given):        X_t <- sum_s mix[s, t] X_s + out[t] y           (all streams at once from the old ones)
//   read  (w_next given):   h = rmsnorm(sum_s in_next[s] X_s) * w_next      (of the new streams)
// `rows` picks the rows that are read when nothing is written (h row r <- X row rows[r]).  The mixed row u stays in
// shared memory between the sum of squares and the scaling.
template <typename act_t, int S>
__global__ void __launch_bounds__(256) seq_hc_step_kernel(const act_t* __restrict__ y, float* __restrict__ X, const float* __restrict__ mix,
                                                          const float* __restrict__ outw, const float* __restrict__ in_next,
                                                          const act_t* __restrict__ w_next, act_t* __restrict__ h, float eps,
                                                          const int* __restrict__ rows, int D, int s_rt) {
  extern __shared__ float hc_u[];
  __shared__ float red[32];
  const int n_s = S > 0 ? S : s_rt;
  const int r = rows ? rows[blockIdx.x] : blockIdx.x;
  float* xr = X + (size_t)r * n_s * D;
  float m[HC_MAX_STREAMS * HC_MAX_STREAMS], o[HC_MAX_STREAMS], a[HC_MAX_STREAMS];
#pragma unroll
  for (int s = 0; s < HC_MAX_STREAMS; ++s) {
    if (s >= n_s) break;
    o[s] = y ? outw[s] : 0.f;
    a[s] = in_next ? in_next[s] : 0.f;
#pragma unroll
    for (int t = 0; t < HC_MAX_STREAMS; ++t) {
      if (t >= n_s) break;
      m[s * HC_MAX_STREAMS + t] = y ? mix[s * n_s + t] : 0.f;
    }
  }
  float ss = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float xs[HC_MAX_STREAMS];
#pragma unroll
    for (int s = 0; s < HC_MAX_STREAMS; ++s) {
      if (s >= n_s) break;
      xs[s] = xr[(size_t)s * D + i];
    }
    float u = 0.f;
    if (y) {
      const float yv = ld_act(y, (size_t)r * D + i);
#pragma unroll
      for (int t = 0; t < HC_MAX_STREAMS; ++t) {
        if (t >= n_s) break;
        float v = o[t] * yv;
#pragma unroll
        for (int s = 0; s < HC_MAX_STREAMS; ++s) {
          if (s >= n_s) break;
          v = fmaf(m[s * HC_MAX_STREAMS + t], xs[s], v);
        }
        xr[(size_t)t * D + i] = v;
        u = fmaf(a[t], v, u);
      }
    } else {
#pragma unroll
      for (int s = 0; s < HC_MAX_STREAMS; ++s) {
        if (s >= n_s) break;
        u = fmaf(a[s], xs[s], u);
      }
    }
    if (w_next) {
      hc_u[i] = u;
      ss += u * u;
    }
  }
  if (w_next == nullptr) return;
  ss = block_sum(ss, red);
  const float rinv = 1.0f / sqrtf(ss / (float)D + eps);
  act_t* hr = h + (size_t)blockIdx.x * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x) st_act(hr, i, hc_u[i] * rinv * ld_act(w_next, i));     // own writes of hc_u
}

// out[t, :] = sum_s X[t, s, :]  (diagnostics: the residual stream as one vector).
__global__ void seq_hc_sum_kernel(const float* __restrict__ X, float* __restrict__ out, int D, int n_s) {
  const float* xr = X + (size_t)blockIdx.x * n_s * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float v = 0.f;
    for (int s = 0; s < n_s; ++s) v += xr[(size_t)s * D + i];
    out[(size_t)blockIdx.x * D + i] = v;
  }
}

__global__ void seq_scale_kernel(float* __restrict__ z, size_t n, float mult) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) z[i] *= mult;
}

// Attention operands of one token from the stacked projection row, one CTA per token.
//   q_out (f32) and k_out (act): RMS norm (whole_row: over all heads*K entries with a weight of that size; else per
//   head with a weight of K entries shared by the heads; no weight: no norm), then rotation of the first rot_dims
//   entries of every head (entry i with entry i + rot_dims/2) by the angle (pos0 + t) * freq[i].
//   v_out (act): (1 - lambda) v + lambda v_first when v_first is given (lambda read on the device), else not written.
template <typename act_t>
__global__ void __launch_bounds__(256) seq_qkv_prep_kernel(b2l_seq_qkv_prep_args a) {
  __shared__ float red[32];
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const act_t* row = (const act_t*)a.proj + (size_t)t * a.ld;
  const float pos = (float)(a.meta[1] + t);
  const int half = a.rot_dims / 2, K = a.K;
  for (int which = 0; which < 2; ++which) {
    const act_t* x = row + (which == 0 ? a.q_off : a.k_off);
    const act_t* w = (const act_t*)(which == 0 ? a.q_norm : a.k_norm);
    const int heads = which == 0 ? a.heads : a.kv_heads;
    float r_row = 1.f;
    if (w && a.whole_row) {
      float ss = 0.f;
      for (int i = threadIdx.x; i < heads * K; i += blockDim.x) {
        const float v = ld_act(x, i);
        ss += v * v;
      }
      ss = block_sum(ss, red);
      r_row = 1.0f / sqrtf(ss / (float)(heads * K) + a.eps);
    }
    for (int hd = warp; hd < heads; hd += nw) {
      const act_t* p = x + (size_t)hd * K;
      const act_t* wh = w ? (a.whole_row ? w + (size_t)hd * K : w) : nullptr;
      float r = r_row;
      if (w && !a.whole_row) {
        float ss = 0.f;
        for (int i = lane; i < K; i += 32) {
          const float v = ld_act(p, i);
          ss += v * v;
        }
        ss = warp_sum(ss);
        r = 1.0f / sqrtf(ss / (float)K + a.eps);
      }
      float* qo = a.q_out + ((size_t)t * heads + hd) * K;
      act_t* ko = (act_t*)a.k_out + ((size_t)t * heads + hd) * K;
      for (int i = lane; i < half; i += 32) {
        const float u = ld_act(p, i) * r * (wh ? ld_act(wh, i) : 1.f);
        const float v = ld_act(p, i + half) * r * (wh ? ld_act(wh, i + half) : 1.f);
        float s, c;
        sincosf(pos * a.freq[i], &s, &c);
        s *= a.rot_mult;
        c *= a.rot_mult;
        if (which == 0) {
          qo[i] = u * c - v * s;
          qo[i + half] = v * c + u * s;
        } else {
          st_act(ko, i, u * c - v * s);
          st_act(ko, i + half, v * c + u * s);
        }
      }
      for (int i = a.rot_dims + lane; i < K; i += 32) {
        const float v = ld_act(p, i) * r * (wh ? ld_act(wh, i) : 1.f);
        if (which == 0) qo[i] = v;
        else st_act(ko, i, v);
      }
    }
  }
  if (a.v_first != nullptr) {
    const float lam = ld_act((const act_t*)a.lambda, 0);
    const act_t* v = row + a.v_off;
    const act_t* vf = (const act_t*)a.v_first + (size_t)t * a.ldvf;
    act_t* vo = (act_t*)a.v_out + (size_t)t * a.kv_heads * a.V;
    for (int i = threadIdx.x; i < a.kv_heads * a.V; i += blockDim.x) st_act(vo, i, (1.f - lam) * ld_act(v, i) + lam * ld_act(vf, i));
  }
}

}  // namespace b2l

using namespace b2l;

extern "C" int b2l_seq_embed_pair(const void* tokens, int tokens_i64, const void* table, const void* pair_table, float scale,
                                  int* prev_state, const int* meta, long long mul_prev, long long mul_cur, int buckets, float* x, int T,
                                  int D, int vocab, int streams, int act_dtype, b2l_stream_t stream) {
  B2L_CHECK_ARG(tokens && table && x, "b2l_seq_embed_pair: null pointer");
  B2L_CHECK_ARG(pair_table == nullptr || (prev_state && meta && buckets > 0 && mul_prev >= 0 && mul_cur >= 0),
                "b2l_seq_embed_pair: the pair table needs its state, the slot and position pair and a positive bucket count");
  B2L_CHECK_ARG(T >= 0 && D > 0 && vocab > 0 && streams >= 1, "b2l_seq_embed_pair: bad size");
  if (T == 0) return 0;
  cudaStream_t s_ = (cudaStream_t)stream;
  B2L_SEQ_DISPATCH(act_dtype, {
    if (tokens_i64)
      seq_embed_pair_kernel<act_t, long long><<<T, 128, 0, s_>>>((const long long*)tokens, (const act_t*)table, (const act_t*)pair_table, scale,
                                                                  prev_state, meta, mul_prev, mul_cur, buckets, x, T, D, vocab, streams);
    else
      seq_embed_pair_kernel<act_t, int><<<T, 128, 0, s_>>>((const int*)tokens, (const act_t*)table, (const act_t*)pair_table, scale, prev_state,
                                                            meta, mul_prev, mul_cur, buckets, x, T, D, vocab, streams);
  });
  B2L_LAUNCH_CHECK("seq_embed_pair_kernel");
  return 0;
}

extern "C" int b2l_seq_hc_step(const void* y, float* X, const float* mix, const float* out_w, const float* in_next, const void* w_next,
                               void* h, float eps, const int* rows, int n_rows, int D, int streams, int act_dtype, b2l_stream_t stream) {
  B2L_CHECK_ARG(X != nullptr, "b2l_seq_hc_step: null pointer");
  B2L_CHECK_ARG((y == nullptr) == (mix == nullptr) && (y == nullptr) == (out_w == nullptr), "b2l_seq_hc_step: y, mix and out_w go together");
  B2L_CHECK_ARG((w_next == nullptr) == (h == nullptr) && (w_next == nullptr) == (in_next == nullptr),
                "b2l_seq_hc_step: in_next, w_next and h go together");
  B2L_CHECK_ARG(rows == nullptr || y == nullptr, "b2l_seq_hc_step: rows are picked only when nothing is written");
  B2L_CHECK_ARG(n_rows >= 0 && D > 0 && streams >= 1, "b2l_seq_hc_step: bad size");
  B2L_CHECK_SUPPORTED(streams <= HC_MAX_STREAMS, "b2l_seq_hc_step: %d streams, at most %d", streams, HC_MAX_STREAMS);
  if (n_rows == 0 || (y == nullptr && w_next == nullptr)) return 0;
  const size_t smem = w_next ? sizeof(float) * (size_t)D : 0;
  B2L_CHECK_SUPPORTED(smem <= 200 * 1024, "b2l_seq_hc_step: width %d too large", D);
  static DynSmemCache cache[2 * 9];
  cudaStream_t s_ = (cudaStream_t)stream;
#define B2L_HC_ARGS (const act_t*)y, X, mix, out_w, in_next, (const act_t*)w_next, (act_t*)h, eps, rows, D, streams
#define B2L_HC_LAUNCH(SV, slot)                                                                                   \
  do {                                                                                                            \
    const int rc_ = ensure_dyn_smem(seq_hc_step_kernel<act_t, SV>, smem, cache[(sizeof(act_t) == 2 ? 0 : 9) + slot]); \
    if (rc_ != 0) return rc_;                                                                                     \
    seq_hc_step_kernel<act_t, SV><<<n_rows, 256, smem, s_>>>(B2L_HC_ARGS);                                         \
  } while (0)
  B2L_SEQ_DISPATCH(act_dtype, {
    switch (streams) {          // the usual stream counts are compiled with their loops unrolled
      case 1: B2L_HC_LAUNCH(1, 0); break;
      case 2: B2L_HC_LAUNCH(2, 1); break;
      case 3: B2L_HC_LAUNCH(3, 2); break;
      case 4: B2L_HC_LAUNCH(4, 3); break;
      case 5: B2L_HC_LAUNCH(5, 4); break;
      case 6: B2L_HC_LAUNCH(6, 5); break;
      case 7: B2L_HC_LAUNCH(7, 6); break;
      case 8: B2L_HC_LAUNCH(8, 7); break;
      default: B2L_HC_LAUNCH(0, 8); break;     // more streams: loops with run-time bounds
    }
  });
#undef B2L_HC_LAUNCH
#undef B2L_HC_ARGS
  B2L_LAUNCH_CHECK("seq_hc_step_kernel");
  return 0;
}

extern "C" int b2l_seq_hc_sum(const float* X, float* out, int T, int D, int streams, b2l_stream_t stream) {
  B2L_CHECK_ARG(X && out && T >= 0 && D > 0 && streams >= 1, "b2l_seq_hc_sum: null pointer or bad size");
  if (T == 0) return 0;
  seq_hc_sum_kernel<<<T, 256, 0, (cudaStream_t)stream>>>(X, out, D, streams);
  B2L_LAUNCH_CHECK("seq_hc_sum_kernel");
  return 0;
}

extern "C" int b2l_seq_scale(float* z, size_t n, float mult, b2l_stream_t stream) {
  B2L_CHECK_ARG(z != nullptr, "b2l_seq_scale: null pointer");
  if (n == 0) return 0;
  const int grid = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
  seq_scale_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(z, n, mult);
  B2L_LAUNCH_CHECK("seq_scale_kernel");
  return 0;
}

extern "C" int b2l_seq_qkv_prep(const b2l_seq_qkv_prep_args* a, b2l_stream_t stream) {
  B2L_CHECK_ARG(a != nullptr, "b2l_seq_qkv_prep: null argument block");
  B2L_CHECK_ARG(a->proj && a->meta && a->q_out && a->k_out, "b2l_seq_qkv_prep: null pointer");
  B2L_CHECK_ARG(a->T >= 0 && a->heads > 0 && a->kv_heads > 0 && a->K > 0 && a->V > 0, "b2l_seq_qkv_prep: bad size");
  B2L_CHECK_ARG(a->rot_dims >= 0 && a->rot_dims <= a->K && a->rot_dims % 2 == 0 && (a->rot_dims == 0 || a->freq), "b2l_seq_qkv_prep: bad rotation");
  B2L_CHECK_ARG((a->v_first == nullptr) || (a->v_out && a->lambda), "b2l_seq_qkv_prep: value mixing needs lambda and an output");
  if (a->T == 0) return 0;
  B2L_SEQ_DISPATCH(a->act_dtype, (seq_qkv_prep_kernel<act_t><<<a->T, 256, 0, (cudaStream_t)stream>>>(*a)));
  B2L_LAUNCH_CHECK("seq_qkv_prep_kernel");
  return 0;
}
