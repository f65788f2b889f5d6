// Attention operands through a short causal convolution: one launch takes the stacked projection [q | k | v] of a
// portion, convolves every channel over time (the last taps-1 projected rows of the sequence are carried per slot),
// rotates the heads of q and k by position and writes q as f32, k and v in the storage type.
// A thread owns the two channels of one rotation pair, (2i, 2i+1) or (i, i + rot_dims/2) inside a head, or two
// neighbouring channels where nothing is rotated, over a tile of tokens, with both sliding windows in registers.
#include "seq_common.cuh"

namespace b2l {

constexpr int CR_TT = 8;             // tokens per tile (at least the most taps - 1: a later tile never reads the carried rows)
constexpr int CR_MAX_TAPS = 8;
constexpr int CR_THREADS = 128;

template <typename act_t>
__global__ void __launch_bounds__(CR_THREADS) seq_conv_rope_kernel(b2l_seq_conv_rope_args a, int update_state) {
  const int pi = blockIdx.x * CR_THREADS + threadIdx.x;
  if (2 * pi >= a.C) return;
  const int col = a.c_off + 2 * pi;
  const int nq = a.q_heads * a.K, nk = a.k_off >= 0 ? a.k_heads * a.K : 0, nv = a.k_off >= 0 ? a.n_v : 0;
  int region = -1, base = 0;                                    // 0 q, 1 k, 2 v; base: first column of the region
  if (col >= a.q_off && col < a.q_off + nq) { region = 0; base = a.q_off; }
  else if (nk && col >= a.k_off && col < a.k_off + nk) { region = 1; base = a.k_off; }
  else if (nv && col >= a.v_off && col < a.v_off + nv) { region = 2; base = a.v_off; }
  if (region < 0) return;                                       // a gap between the parts: zero rows of the projection
  int ca = col, cb = col + 1, fi = -1;
  if (region < 2 && a.rot_dims > 0) {
    const int d = (col - base) % a.K, head0 = col - d, ph = d >> 1, half = a.rot_dims >> 1;
    if (ph < half) {
      fi = ph;
      if (!a.interleaved) { ca = head0 + ph; cb = head0 + ph + half; }
    }
  }
  const act_t* in = (const act_t*)a.proj;
  const act_t* w = (const act_t*)a.w;
  const int taps = a.taps, C = a.C, ra = ca - a.c_off, rb = cb - a.c_off;
  const int slot = a.meta[0], pos0 = a.meta[1];
  act_t* st = (act_t*)a.state + (size_t)slot * (taps - 1) * C;
  const int t0 = blockIdx.y * CR_TT, t1 = min(a.T, t0 + CR_TT);
  float wa[CR_MAX_TAPS], wb[CR_MAX_TAPS], xa[CR_MAX_TAPS], xb[CR_MAX_TAPS];      // x?[j] = input at t - (taps-1) + j
#pragma unroll
  for (int j = 0; j < CR_MAX_TAPS; ++j) {
    wa[j] = j < taps ? ld_act(w, (size_t)ra * taps + j) : 0.f;
    wb[j] = j < taps ? ld_act(w, (size_t)rb * taps + j) : 0.f;
    xa[j] = xb[j] = 0.f;
    if (j < taps - 1) {
      const int t = t0 - (taps - 1) + j;
      xa[j] = t >= 0 ? ld_act(in, (size_t)t * a.ld + ca) : ld_act(st, (size_t)(taps - 1 + t) * C + ra);
      xb[j] = t >= 0 ? ld_act(in, (size_t)t * a.ld + cb) : ld_act(st, (size_t)(taps - 1 + t) * C + rb);
    }
  }
  const float f = fi >= 0 ? a.freq[fi] : 0.f;
  for (int t = t0; t < t1; ++t) {
    const float ua = ld_act(in, (size_t)t * a.ld + ca), ub = ld_act(in, (size_t)t * a.ld + cb);
    float ya = 0.f, yb = 0.f;
#pragma unroll
    for (int j = 0; j < CR_MAX_TAPS; ++j) {
      if (j < taps - 1) {
        ya = fmaf(wa[j], xa[j], ya);
        yb = fmaf(wb[j], xb[j], yb);
      }
    }
#pragma unroll
    for (int j = 0; j < CR_MAX_TAPS; ++j) {
      if (j == taps - 1) {
        ya = fmaf(wa[j], ua, ya);
        yb = fmaf(wb[j], ub, yb);
      }
    }
    if (fi >= 0) {
      float s, c;
      sincosf((float)(pos0 + t) * f, &s, &c);
      s *= a.rot_mult;
      c *= a.rot_mult;
      const float u = ya, v = yb;
      ya = u * c - v * s;
      yb = v * c + u * s;
    }
    if (region == 0) {
      a.q_out[(size_t)t * nq + (ca - base)] = ya;
      a.q_out[(size_t)t * nq + (cb - base)] = yb;
    } else if (region == 1) {
      st_act((act_t*)a.k_out, (size_t)t * nk + (ca - base), ya);
      st_act((act_t*)a.k_out, (size_t)t * nk + (cb - base), yb);
    } else {
      st_act((act_t*)a.v_out, (size_t)t * nv + (ca - base), ya);
      st_act((act_t*)a.v_out, (size_t)t * nv + (cb - base), yb);
    }
#pragma unroll
    for (int j = 0; j < CR_MAX_TAPS - 1; ++j) {
      if (j < taps - 2) {
        xa[j] = xa[j + 1];
        xb[j] = xb[j + 1];
      }
    }
#pragma unroll
    for (int j = 0; j < CR_MAX_TAPS; ++j) {
      if (j == taps - 2) {
        xa[j] = ua;
        xb[j] = ub;
      }
    }
  }
  if (update_state) {            // a single tile: the windows now hold the last taps-1 rows of the sequence
#pragma unroll
    for (int j = 0; j < CR_MAX_TAPS; ++j) {
      if (j < taps - 1) {
        st_act(st, (size_t)j * C + ra, xa[j]);
        st_act(st, (size_t)j * C + rb, xb[j]);
      }
    }
  }
}

// state <- the last taps-1 projected rows after T >= taps-1 new tokens (launches of several tiles only).
template <typename act_t>
__global__ void seq_conv_rope_state_kernel(const act_t* __restrict__ in, int ld, act_t* __restrict__ state, const int* __restrict__ meta,
                                           int T, int C, int taps) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  act_t* st = state + (size_t)meta[0] * (taps - 1) * C;
  for (int j = 0; j < taps - 1; ++j) st[(size_t)j * C + c] = in[(size_t)(T - (taps - 1) + j) * ld + c];
}

}  // namespace b2l

using namespace b2l;

extern "C" int b2l_seq_conv_rope(const b2l_seq_conv_rope_args* a, b2l_stream_t stream) {
  B2L_CHECK_ARG(a != nullptr, "b2l_seq_conv_rope: null argument block");
  B2L_CHECK_ARG(a->proj && a->w && (a->state || a->taps == 1) && a->meta && a->q_out, "b2l_seq_conv_rope: null pointer");
  B2L_CHECK_ARG(a->k_off < 0 || (a->k_out && a->v_out), "b2l_seq_conv_rope: keys and values without their outputs");
  B2L_CHECK_ARG(a->T >= 0 && a->C > 0 && a->c_off >= 0 && a->ld >= a->c_off + a->C && a->q_heads > 0 && a->K > 0, "b2l_seq_conv_rope: bad size");
  B2L_CHECK_SUPPORTED(a->taps >= 1 && a->taps <= CR_MAX_TAPS, "b2l_seq_conv_rope: taps %d outside 1..%d", a->taps, CR_MAX_TAPS);
  B2L_CHECK_ARG(a->K % 2 == 0 && a->C % 2 == 0 && a->c_off % 2 == 0 && a->q_off % 2 == 0 && (a->k_off < 0 || (a->k_off % 2 == 0 && a->v_off % 2 == 0 && a->n_v % 2 == 0)),
                "b2l_seq_conv_rope: head size, channel count and offsets must be even");
  B2L_CHECK_ARG(a->q_off >= a->c_off && a->q_off + a->q_heads * a->K <= a->c_off + a->C, "b2l_seq_conv_rope: q outside the convolved channels");
  B2L_CHECK_ARG(a->k_off < 0 || (a->k_heads > 0 && a->n_v > 0 && a->k_off >= a->c_off && a->k_off + a->k_heads * a->K <= a->c_off + a->C &&
                                 a->v_off >= a->c_off && a->v_off + a->n_v <= a->c_off + a->C), "b2l_seq_conv_rope: k or v outside the convolved channels");
  B2L_CHECK_ARG(a->rot_dims >= 0 && a->rot_dims <= a->K && a->rot_dims % 2 == 0 && (a->rot_dims == 0 || a->freq), "b2l_seq_conv_rope: bad rotation");
  if (a->T == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int tiles = (a->T + CR_TT - 1) / CR_TT;
  dim3 grid((unsigned)((a->C / 2 + CR_THREADS - 1) / CR_THREADS), (unsigned)tiles);
  B2L_SEQ_DISPATCH(a->act_dtype, {
    seq_conv_rope_kernel<act_t><<<grid, CR_THREADS, 0, s>>>(*a, tiles == 1);
    if (tiles > 1 && a->taps > 1)      // T > CR_TT >= taps - 1: the new state comes from the portion alone
      seq_conv_rope_state_kernel<act_t><<<(a->C + 127) / 128, 128, 0, s>>>((const act_t*)a->proj + a->c_off, a->ld, (act_t*)a->state, a->meta, a->T, a->C, a->taps);
  });
  B2L_LAUNCH_CHECK("seq_conv_rope_kernel");
  return 0;
}
