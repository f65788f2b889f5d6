// Mixture-of-experts feed-forward: the router (softmax or sigmoid scores, a selection bias that only steers the choice,
// groups of neighbouring experts of which only the best may be chosen, top-k, weights renormalised over the chosen or
// the scores themselves; the weight scales an expert's output or its input), the
// expert products for a handful of tokens with the expert index read on the device (a captured single-token step
// replays for any routing), and the sort / gather / combine around the per-expert library products of long portions.
// Experts with index >= n_real are identities: their output is the input itself.
#include <climits>

#include "seq_common.cuh"

namespace b2l {

struct Best {
  float v;
  int i;
};
__device__ __forceinline__ Best better(Best a, Best b) { return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a; }
__device__ __forceinline__ Best warp_best(Best x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best y;
    y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
    y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
    x = better(x, y);
  }
  return x;
}

// The router of one token by one warp, from its logits zr[n] (global or shared).  s[n] (scores), c[n] (choice
// scores) and g[groups] are the warp's shared scratch.
__device__ __forceinline__ void route_token(const float* zr, const float* __restrict__ corr, int n, int groups, int keep, int top,
                                            int score_fn, int renorm, int group_top, float weight_scale, int* __restrict__ idx_t, float* __restrict__ wgt_t, float* s, float* c,
                                            float* g, int lane) {
  if (score_fn == B2L_SEQ_SCORE_SIGMOID) {
    for (int i = lane; i < n; i += 32) {
      s[i] = sigmoid_f(zr[i]);
      c[i] = s[i] + (corr ? corr[i] : 0.f);
    }
  } else {
    float mx = -INFINITY;
    for (int i = lane; i < n; i += 32) mx = fmaxf(mx, zr[i]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int i = lane; i < n; i += 32) {
      const float e = expf(zr[i] - mx);
      s[i] = e;
      sum += e;
    }
    sum = warp_sum(sum);
    for (int i = lane; i < n; i += 32) {
      s[i] = s[i] / sum;
      c[i] = s[i] + (corr ? corr[i] : 0.f);
    }
  }
  __syncwarp();
  if (groups > 1 && keep < groups) {
    const int per = n / groups;
    for (int q = lane; q < groups; q += 32) {
      if (group_top <= 1) {                           // a group is worth its largest choice score
        float b = -INFINITY;
        for (int i = 0; i < per; ++i) b = fmaxf(b, c[q * per + i]);
        g[q] = b;
      } else {                                        // ... or the sum of its group_top largest: pick them one by one
        float sum = 0.f, last = INFINITY;
        int last_i = -1;
        for (int k = 0; k < group_top && k < per; ++k) {
          float b = -INFINITY;
          int bi = -1;
          for (int i = 0; i < per; ++i) {
            const float v = c[q * per + i];
            const bool after = v < last || (v == last && i > last_i);       // not yet picked, in the order (value down, index up)
            if (after && (bi < 0 || v > b)) { b = v; bi = i; }
          }
          sum += b;
          last = b;
          last_i = bi;
        }
        g[q] = sum;
      }
    }
    __syncwarp();
    for (int k = 0; k < keep; ++k) {                // the best `keep` groups get the mark +inf
      Best b{-INFINITY, INT_MAX};
      for (int q = lane; q < groups; q += 32)
        if (g[q] != INFINITY) b = better(b, Best{g[q], q});
      b = warp_best(b);
      if (lane == 0 && b.i != INT_MAX) g[b.i] = INFINITY;
      __syncwarp();
    }
    for (int i = lane; i < n; i += 32)
      if (g[i / per] != INFINITY) c[i] = -INFINITY;
    __syncwarp();
  }
  float total = 0.f;
  for (int k = 0; k < top; ++k) {
    Best b{-INFINITY, INT_MAX};
    for (int i = lane; i < n; i += 32)
      if (!isnan(c[i])) b = better(b, Best{c[i], i});
    b = warp_best(b);
    const int e = b.i == INT_MAX ? 0 : b.i;
    if (lane == 0) {
      idx_t[k] = e;
      c[e] = NAN;                                   // chosen: out of the next rounds
    }
    total += s[e];
    __syncwarp();
  }
  for (int k = lane; k < top; k += 32) wgt_t[k] = (renorm ? s[idx_t[k]] / (total + 1e-20f) : s[idx_t[k]]) * weight_scale;
}

// One warp per token.  Shared per warp: s[n], c[n], g[groups].
__global__ void seq_moe_route_kernel(const float* __restrict__ z, int ldz, const float* __restrict__ corr, int n, int groups, int keep,
                                     int top, int score_fn, int renorm, int group_top, float weight_scale, int* __restrict__ idx, float* __restrict__ wgt, int T) {
  extern __shared__ float route_smem[];
  const int wpc = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * wpc + warp;
  if (t >= T) return;
  float* s = route_smem + (size_t)warp * (2 * n + groups);
  route_token(z + (size_t)t * ldz, corr, n, groups, keep, top, score_fn, renorm, group_top, weight_scale, idx + (size_t)t * top, wgt + (size_t)t * top, s, s + n, s + 2 * n,
              lane);
}

// Dot product of a weight row with a vector in shared memory (f32); the warp's lanes stride the row.
template <typename act_t>
__device__ __forceinline__ float row_dot(const act_t* __restrict__ w, const float* __restrict__ x, int n, int lane, bool vec) {
  float acc = 0.f;
  if (vec) {                                         // 16-byte loads: n a multiple of 8 (bf16) / 4 (f32), aligned rows
    constexpr int PER = 16 / sizeof(act_t);
    for (int i = lane * PER; i < n; i += 32 * PER) {
      const uint4 u = *reinterpret_cast<const uint4*>(w + i);
      if (sizeof(act_t) == 2) {
        const uint32_t ww[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          acc = fmaf(__uint_as_float(ww[q] << 16), x[i + 2 * q], acc);
          acc = fmaf(__uint_as_float(ww[q] & 0xffff0000u), x[i + 2 * q + 1], acc);
        }
      } else {
        acc = fmaf(__uint_as_float(u.x), x[i], acc);
        acc = fmaf(__uint_as_float(u.y), x[i + 1], acc);
        acc = fmaf(__uint_as_float(u.z), x[i + 2], acc);
        acc = fmaf(__uint_as_float(u.w), x[i + 3], acc);
      }
    }
  } else {
    for (int i = lane; i < n; i += 32) acc = fmaf(ld_act(w, i), x[i], acc);
  }
  return warp_sum(acc);
}

// Router of a few tokens in one launch: the logits W_router h_t (f32 accumulation of exact products; a warp per
// router row) and the routing.  One CTA per token.  Shared: x[D], z[n], s[n], c[n], g[groups].
template <typename act_t>
__global__ void __launch_bounds__(1024) seq_moe_route_fused_kernel(const act_t* __restrict__ h, int ldh, const act_t* __restrict__ wr,
                                                                  const float* __restrict__ corr, int D, int n, int groups, int keep, int top,
                                                                  int score_fn, int renorm, int group_top, float weight_scale,
                                                                  int* __restrict__ idx, float* __restrict__ wgt, int vec) {
  extern __shared__ float route_smem[];
  float* x = route_smem;
  float* z = x + D;
  const int t = blockIdx.x, wpc = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < D; i += blockDim.x) x[i] = ld_act(h, (size_t)t * ldh + i);
  __syncthreads();
  for (int r = warp; r < n; r += wpc) {
    const float v = row_dot(wr + (size_t)r * D, x, D, lane, vec);
    if (lane == 0) z[r] = v;
  }
  __syncthreads();
  if (warp == 0)
    route_token(z, corr, n, groups, keep, top, score_fn, renorm, group_top, weight_scale, idx + (size_t)t * top, wgt + (size_t)t * top, z + n, z + 2 * n, z + 3 * n, lane);
}

// mid[a, j] = gated(W_gate[e] x, W_up[e] x) for assignment a = t * top + k, e = idx[a], x = h_t or (in_scale given) the
// storage-type rounding of in_scale[a] * h_t.  grid (N, ff chunks).
template <typename act_t>
__global__ void __launch_bounds__(256) seq_moe_up_kernel(const act_t* __restrict__ h, int ldh, const act_t* __restrict__ wgu,
                                                         const int* __restrict__ idx, const float* __restrict__ in_scale,
                                                         act_t* __restrict__ mid, int D, int ff, int n_real, int top, int act, float limit,
                                                         int vec) {
  extern __shared__ float moe_x[];
  const int a = blockIdx.x, e = idx[a];
  if (e >= n_real) return;
  const act_t* hr = h + (size_t)(a / top) * ldh;
  if (in_scale) {
    const float w = in_scale[a];
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
      act_t tmp[1];
      st_act(tmp, 0, w * ld_act(hr, i));
      moe_x[i] = ld_act(tmp, 0);
    }
  } else {
    for (int i = threadIdx.x; i < D; i += blockDim.x) moe_x[i] = ld_act(hr, i);
  }
  __syncthreads();
  const int wpc = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const act_t* w = wgu + (size_t)e * 2 * ff * D;
  for (int j = blockIdx.y * wpc + warp; j < ff; j += gridDim.y * wpc) {
    const float gv = row_dot(w + (size_t)j * D, moe_x, D, lane, vec);
    const float uv = row_dot(w + (size_t)(ff + j) * D, moe_x, D, lane, vec);
    if (lane == 0) {
      // both halves pass through the storage type, as the two-product form does
      act_t tmp[2];
      st_act(tmp, 0, gv);
      st_act(tmp, 1, uv);
      st_act(mid, (size_t)a * ff + j, gated_pair(ld_act(tmp, 0), ld_act(tmp, 1), act, limit));
    }
  }
}

// y[t, i] = sum_k w[t, k] * (e < n_real ? W_down[e][i, :] . mid[a, :] : h[t, i]).  grid (T, D chunks).
template <typename act_t>
__global__ void __launch_bounds__(256) seq_moe_down_kernel(const act_t* __restrict__ mid, const act_t* __restrict__ wd,
                                                           const int* __restrict__ idx, const float* __restrict__ wgt,
                                                           const float* __restrict__ in_scale, const act_t* __restrict__ h, int ldh,
                                                           act_t* __restrict__ y, int ldy, int D, int ff, int n_real, int top, int vec) {
  extern __shared__ float moe_x[];
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < top * ff; i += blockDim.x) {
    const int k = i / ff;
    moe_x[i] = idx[(size_t)t * top + k] < n_real ? ld_act(mid, ((size_t)t * top + k) * ff + (i % ff)) : 0.f;
  }
  __syncthreads();
  const int wpc = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = blockIdx.y * wpc + warp; i < D; i += gridDim.y * wpc) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k) {
      const int e = idx[(size_t)t * top + k];
      const float wk = wgt ? wgt[(size_t)t * top + k] : 1.f;
      float v;
      if (e < n_real) {
        v = row_dot(wd + ((size_t)e * D + i) * ff, moe_x + (size_t)k * ff, ff, lane, vec);
        act_t tmp[1];
        st_act(tmp, 0, v);                              // an expert's output in the storage type
        v = ld_act(tmp, 0);
      } else {
        v = ld_act(h, (size_t)t * ldh + i) * ((wgt || in_scale == nullptr) ? 1.f : in_scale[(size_t)t * top + k]);
      }
      acc = fmaf(wk, v, acc);
    }
    if (lane == 0) st_act(y, (size_t)t * ldy + i, acc);
  }
}

// ---- long portions: assignments sorted by expert around per-expert library products ----
__global__ void seq_moe_count_kernel(const int* __restrict__ idx, int N, int n_real, int* __restrict__ counts) {
  const int a = blockIdx.x * blockDim.x + threadIdx.x;
  if (a < N && idx[a] < n_real) atomicAdd(&counts[idx[a]], 1);
}
__global__ void seq_moe_scan_kernel(const int* counts, int n_real, int* __restrict__ offsets, int* cursor) {   // counts may be cursor
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < n_real; ++e) {
      const int c = counts[e];
      offsets[e] = at;
      cursor[e] = at;
      at += c;
    }
    offsets[n_real] = at;
  }
}
__global__ void seq_moe_fill_kernel(const int* __restrict__ idx, int N, int n_real, int* __restrict__ cursor, int* __restrict__ perm,
                                    int* __restrict__ inv) {
  const int a = blockIdx.x * blockDim.x + threadIdx.x;
  if (a >= N) return;
  const int e = idx[a];
  if (e >= n_real) {
    inv[a] = -1;
    return;
  }
  const int p = atomicAdd(&cursor[e], 1);
  perm[p] = a;
  inv[a] = p;
}
// xg[p, :] = h[perm[p] / top, :] for p < offsets[n_real].  One CTA per row.
template <typename act_t>
__global__ void seq_moe_gather_kernel(const act_t* __restrict__ h, int ldh, const int* __restrict__ perm, const int* __restrict__ n_rows,
                                      const float* __restrict__ row_scale, int top, act_t* __restrict__ xg, int D) {
  const int p = blockIdx.x;
  if (p >= *n_rows) return;
  const act_t* src = h + (size_t)(perm[p] / top) * ldh;
  act_t* dst = xg + (size_t)p * D;
  if (row_scale) {
    const float w = row_scale[perm[p]];
    for (int i = threadIdx.x; i < D; i += blockDim.x) st_act(dst, i, w * ld_act(src, i));
  } else {
    for (int i = threadIdx.x; i < D; i += blockDim.x) dst[i] = src[i];
  }
}
// y[t, i] = sum_k w[t, k] * (inv[a] >= 0 ? yg[inv[a], i] : h[t, i]).  One CTA per token.
template <typename act_t>
__global__ void seq_moe_combine_kernel(const act_t* __restrict__ yg, const int* __restrict__ inv, const float* __restrict__ wgt,
                                       const act_t* __restrict__ h, int ldh, act_t* __restrict__ y, int ldy, int D, int top) {
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k) {
      const int p = inv[(size_t)t * top + k];
      const float v = p >= 0 ? ld_act(yg, (size_t)p * D + i) : ld_act(h, (size_t)t * ldh + i);
      acc = fmaf(wgt ? wgt[(size_t)t * top + k] : 1.f, v, acc);
    }
    st_act(y, (size_t)t * ldy + i, acc);
  }
}

static DynSmemCache g_moe_smem[4];

}  // namespace b2l

using namespace b2l;

extern "C" int b2l_seq_moe_route(const float* logits, int ld, const float* correction, int n, int groups, int keep, int top, int score_fn,
                                 int renormalize, int group_top, float weight_scale, int* idx, float* weights, int T, b2l_stream_t stream) {
  B2L_CHECK_ARG(logits && idx && weights, "b2l_seq_moe_route: null pointer");
  B2L_CHECK_ARG(group_top >= 1, "b2l_seq_moe_route: a group's score needs at least its largest member");
  B2L_CHECK_ARG(T >= 0 && n > 0 && ld >= n && top > 0 && top <= n && groups >= 1 && n % groups == 0 && keep >= 1 && keep <= groups,
                "b2l_seq_moe_route: bad size");
  B2L_CHECK_ARG((long long)keep * (n / groups) >= top, "b2l_seq_moe_route: the kept groups hold fewer than `top` experts");
  B2L_CHECK_ARG(score_fn == B2L_SEQ_SCORE_SOFTMAX || score_fn == B2L_SEQ_SCORE_SIGMOID, "b2l_seq_moe_route: unknown score function %d", score_fn);
  if (T == 0) return 0;
  const int wpc = 4;
  const size_t smem = sizeof(float) * wpc * (2 * (size_t)n + groups);
  B2L_CHECK_SUPPORTED(smem <= 48 * 1024, "b2l_seq_moe_route: %d experts need %zu bytes of shared memory", n, smem);
  seq_moe_route_kernel<<<(T + wpc - 1) / wpc, wpc * 32, smem, (cudaStream_t)stream>>>(logits, ld, correction, n, groups, keep, top, score_fn, renormalize,
                                                                                          group_top, weight_scale, idx, weights, T);
  B2L_LAUNCH_CHECK("seq_moe_route_kernel");
  return 0;
}

static inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

extern "C" int b2l_seq_moe_route_fused(const void* h, int ldh, const void* w_router, const float* correction, int D, int n, int groups,
                                       int keep, int top, int score_fn, int renormalize, int group_top, float weight_scale, int* idx,
                                       float* weights, int T, int act_dtype, b2l_stream_t stream) {
  B2L_CHECK_ARG(h && w_router && idx && weights, "b2l_seq_moe_route_fused: null pointer");
  B2L_CHECK_ARG(group_top >= 1, "b2l_seq_moe_route_fused: a group's score needs at least its largest member");
  B2L_CHECK_ARG(T >= 0 && D > 0 && ldh >= D && n > 0 && top > 0 && top <= n && groups >= 1 && n % groups == 0 && keep >= 1 && keep <= groups,
                "b2l_seq_moe_route_fused: bad size");
  B2L_CHECK_ARG((long long)keep * (n / groups) >= top, "b2l_seq_moe_route_fused: the kept groups hold fewer than `top` experts");
  B2L_CHECK_ARG(score_fn == B2L_SEQ_SCORE_SOFTMAX || score_fn == B2L_SEQ_SCORE_SIGMOID, "b2l_seq_moe_route_fused: unknown score function %d", score_fn);
  if (T == 0) return 0;
  const size_t smem = sizeof(float) * ((size_t)D + 3 * (size_t)n + groups);
  B2L_CHECK_SUPPORTED(smem <= 200 * 1024, "b2l_seq_moe_route_fused: width %d and %d experts need %zu bytes of shared memory", D, n, smem);
  static DynSmemCache cache[2];
  B2L_SEQ_DISPATCH(act_dtype, {
    constexpr int PER = 16 / sizeof(act_t);
    const int vec = (D % PER == 0 && al16(w_router)) ? 1 : 0;
    const int rc = ensure_dyn_smem(seq_moe_route_fused_kernel<act_t>, smem, cache[sizeof(act_t) == 2 ? 0 : 1]);
    if (rc != 0) return rc;
    seq_moe_route_fused_kernel<act_t><<<T, n >= 32 ? 1024 : 32 * ((n + 3) / 4 * 4 > 8 ? (n + 3) / 4 * 4 : 8), smem, (cudaStream_t)stream>>>((const act_t*)h, ldh, (const act_t*)w_router, correction, D, n, groups,
                                                                             keep, top, score_fn, renormalize, group_top, weight_scale, idx, weights, vec);
  });
  B2L_LAUNCH_CHECK("seq_moe_route_fused_kernel");
  return 0;
}

extern "C" int b2l_seq_moe_experts_small(const void* h, int ldh, const void* w_gate_up, const void* w_down, const int* idx,
                                         const float* weights, void* mid, void* y, int ldy, int T, int D, int ff, int n_real,
                                         int top, int act, float limit, int weight_input, int act_dtype, b2l_stream_t stream) {
  B2L_CHECK_ARG(h && idx && weights && mid && y && (n_real == 0 || (w_gate_up && w_down)), "b2l_seq_moe_experts_small: null pointer");
  B2L_CHECK_ARG(T >= 0 && D > 0 && ff > 0 && top > 0 && n_real >= 0 && ldh >= D && ldy >= D, "b2l_seq_moe_experts_small: bad size");
  B2L_CHECK_ARG(act >= 0 && act <= 3 && (act != B2L_SEQ_ACT_CLAMPED_SWISH || limit > 0.f), "b2l_seq_moe_experts_small: bad activation");
  if (T == 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t smem_up = sizeof(float) * (size_t)D, smem_dn = sizeof(float) * (size_t)top * ff;
  B2L_CHECK_SUPPORTED(smem_up <= 200 * 1024 && smem_dn <= 200 * 1024, "b2l_seq_moe_experts_small: width %d or top * ff %d too large", D, top * ff);
  B2L_SEQ_DISPATCH(act_dtype, {
    constexpr int PER = 16 / sizeof(act_t);
    const int vec_up = (D % PER == 0 && al16(w_gate_up)) ? 1 : 0;
    const int vec_dn = (ff % PER == 0 && al16(w_down)) ? 1 : 0;
    int rc = ensure_dyn_smem(seq_moe_up_kernel<act_t>, smem_up, g_moe_smem[sizeof(act_t) == 2 ? 0 : 1]);
    if (rc != 0) return rc;
    rc = ensure_dyn_smem(seq_moe_down_kernel<act_t>, smem_dn, g_moe_smem[sizeof(act_t) == 2 ? 2 : 3]);
    if (rc != 0) return rc;
    if (n_real > 0)
      seq_moe_up_kernel<act_t><<<dim3(T * top, (ff + 7) / 8), 256, smem_up, st>>>((const act_t*)h, ldh, (const act_t*)w_gate_up, idx,
                                                                                   weight_input ? weights : nullptr, (act_t*)mid, D, ff, n_real,
                                                                                   top, act, limit, vec_up);
    seq_moe_down_kernel<act_t><<<dim3(T, (D + 7) / 8), 256, smem_dn, st>>>((const act_t*)mid, (const act_t*)w_down, idx,
                                                                            weight_input ? nullptr : weights, weight_input ? weights : nullptr,
                                                                            (const act_t*)h, ldh, (act_t*)y, ldy, D, ff, n_real, top, vec_dn);
  });
  B2L_LAUNCH_CHECK("seq_moe_up_kernel / seq_moe_down_kernel");
  return 0;
}

extern "C" int b2l_seq_moe_sort(const int* idx, int N, int n_real, int* offsets, int* cursor, int* perm, int* inv, b2l_stream_t stream) {
  B2L_CHECK_ARG(idx && offsets && cursor && perm && inv, "b2l_seq_moe_sort: null pointer");
  B2L_CHECK_ARG(N >= 0 && n_real >= 0, "b2l_seq_moe_sort: bad size");
  cudaStream_t st = (cudaStream_t)stream;
  B2L_CUDA(cudaMemsetAsync(cursor, 0, sizeof(int) * (size_t)(n_real + 1), st));
  if (N > 0) seq_moe_count_kernel<<<(N + 255) / 256, 256, 0, st>>>(idx, N, n_real, cursor);
  // counts live in `cursor` until the scan has read them: the scan reads entry e before it overwrites it
  seq_moe_scan_kernel<<<1, 32, 0, st>>>(cursor, n_real, offsets, cursor);
  if (N > 0) seq_moe_fill_kernel<<<(N + 255) / 256, 256, 0, st>>>(idx, N, n_real, cursor, perm, inv);
  B2L_LAUNCH_CHECK("seq_moe_sort kernels");
  return 0;
}

extern "C" int b2l_seq_moe_gather(const void* h, int ldh, const int* perm, const int* n_rows, const float* row_scale, int top, void* xg,
                                  int N, int D, int act_dtype, b2l_stream_t stream) {
  B2L_CHECK_ARG(h && perm && n_rows && xg, "b2l_seq_moe_gather: null pointer");
  B2L_CHECK_ARG(N >= 0 && D > 0 && top > 0 && ldh >= D, "b2l_seq_moe_gather: bad size");
  if (N == 0) return 0;
  B2L_SEQ_DISPATCH(act_dtype, {
    seq_moe_gather_kernel<act_t><<<N, 128, 0, (cudaStream_t)stream>>>((const act_t*)h, ldh, perm, n_rows, row_scale, top, (act_t*)xg, D);
  });
  B2L_LAUNCH_CHECK("seq_moe_gather_kernel");
  return 0;
}

extern "C" int b2l_seq_moe_combine(const void* yg, const int* inv, const float* weights, const void* h, int ldh, void* y, int ldy,
                                   int T, int D, int top, int act_dtype, b2l_stream_t stream) {
  B2L_CHECK_ARG(yg && inv && h && y, "b2l_seq_moe_combine: null pointer");
  B2L_CHECK_ARG(T >= 0 && D > 0 && top > 0 && ldh >= D && ldy >= D, "b2l_seq_moe_combine: bad size");
  if (T == 0) return 0;
  B2L_SEQ_DISPATCH(act_dtype, {
    seq_moe_combine_kernel<act_t><<<T, 256, 0, (cudaStream_t)stream>>>((const act_t*)yg, inv, weights, (const act_t*)h, ldh, (act_t*)y, ldy, D, top);
  });
  B2L_LAUNCH_CHECK("seq_moe_combine_kernel");
  return 0;
}
