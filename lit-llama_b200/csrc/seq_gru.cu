// Gated recurrence on every channel by itself (minGRU): the gates read only the current token, so a portion is a
// first-order linear recurrence S_t = a_t S_(t-1) + b_t per channel with a_t = 1 - z_t, b_t = z_t c_t.
//   sequential form (decoding, short portions): a thread per channel walks the tokens; the loads of the next tokens do
//     not depend on the state, so they are issued ahead of the dependent multiply-adds;
//   chunked form (long portions): (1) every chunk's product of a and its end state from zero, (2) one pass over the
//     chunks per channel that turns those into every chunk's start state and advances the carried state, (3) every
//     chunk again from its start state, writing the gated outputs.
// Gates, candidates and the state are f32; only the projections arrive in the storage type.
#include "seq_common.cuh"

namespace b2l {

constexpr int GRU_THREADS = 128;
constexpr int GRU_CHUNK = 64;        // tokens per chunk of the chunked form
constexpr int GRU_AHEAD = 8;         // tokens whose operands are loaded together

__device__ __forceinline__ void gru_terms(float pz, float px, float& a, float& b) {
  const float z = sigmoid_f(pz);
  const float c = px >= 0.f ? px + 0.5f : sigmoid_f(px);
  a = 1.0f - z;
  b = z * c;
}

// MODE 0: the whole portion from the carried state, outputs, new carried state.
// MODE 1: chunk blockIdx.y from zero: work[chunk][0] = product of a, work[chunk][1] = end state.
// MODE 2: chunk blockIdx.y from its start state work[chunk][0]: outputs.
template <typename act_t, int MODE>
__global__ void __launch_bounds__(GRU_THREADS) seq_mingru_kernel(const act_t* __restrict__ proj, int ld, int z_off, int x_off, int g_off,
                                                                float* __restrict__ state, const int* __restrict__ meta,
                                                                act_t* __restrict__ out, int ldo, float* __restrict__ work, int T, int width) {
  const int c = blockIdx.x * GRU_THREADS + threadIdx.x;
  if (c >= width) return;
  const int t0 = MODE == 0 ? 0 : blockIdx.y * GRU_CHUNK, t1 = MODE == 0 ? T : min(T, t0 + GRU_CHUNK);
  float* st = state + (size_t)meta[0] * width;
  float* wk = work + (size_t)blockIdx.y * 2 * width;
  float s = MODE == 0 ? st[c] : (MODE == 1 ? 0.f : wk[c]);
  float prod = 1.f;
  for (int tb = t0; tb < t1; tb += GRU_AHEAD) {
    float pz[GRU_AHEAD], px[GRU_AHEAD], pg[GRU_AHEAD];
#pragma unroll
    for (int u = 0; u < GRU_AHEAD; ++u) {
      const int t = min(tb + u, t1 - 1);
      const act_t* row = proj + (size_t)t * ld;
      pz[u] = ld_act(row, z_off + c);
      px[u] = ld_act(row, x_off + c);
      pg[u] = (MODE != 1 && g_off >= 0) ? ld_act(row, g_off + c) : 0.f;
    }
#pragma unroll
    for (int u = 0; u < GRU_AHEAD; ++u) {
      if (tb + u < t1) {
        float a, b;
        gru_terms(pz[u], px[u], a, b);
        s = fmaf(a, s, b);
        if (MODE == 1) prod *= a;
        else st_act(out, (size_t)(tb + u) * ldo + c, g_off >= 0 ? s * silu_f(pg[u]) : s);
      }
    }
  }
  if (MODE == 0) st[c] = s;
  if (MODE == 1) {
    wk[c] = prod;
    wk[width + c] = s;
  }
}

// Per channel over the chunks: work[chunk][0] <- the chunk's start state; the carried state advances past the portion.
__global__ void __launch_bounds__(GRU_THREADS) seq_mingru_combine_kernel(float* __restrict__ state, const int* __restrict__ meta,
                                                                        float* __restrict__ work, int n_chunks, int width) {
  const int c = blockIdx.x * GRU_THREADS + threadIdx.x;
  if (c >= width) return;
  float* st = state + (size_t)meta[0] * width;
  float s = st[c];
  for (int k = 0; k < n_chunks; ++k) {
    float* wk = work + (size_t)k * 2 * width;
    const float a = wk[c], b = wk[width + c];
    wk[c] = s;
    s = fmaf(a, s, b);
  }
  st[c] = s;
}

}  // namespace b2l

using namespace b2l;

extern "C" int b2l_seq_mingru_chunks(int T) { return T >= 4 * GRU_CHUNK ? (T + GRU_CHUNK - 1) / GRU_CHUNK : 1; }

extern "C" int b2l_seq_mingru(const void* proj, int ld, int z_off, int x_off, int g_off, float* state, const int* meta, void* out, int ldo,
                              float* work, int n_chunks, int T, int width, int act_dtype, b2l_stream_t stream) {
  B2L_CHECK_ARG(proj && state && meta && out, "b2l_seq_mingru: null pointer");
  B2L_CHECK_ARG(T >= 0 && width > 0 && z_off >= 0 && x_off >= 0 && ld >= z_off + width && ld >= x_off + width && (g_off < 0 || ld >= g_off + width) &&
                    ldo >= width, "b2l_seq_mingru: bad size");
  B2L_CHECK_ARG(n_chunks >= 1 && (n_chunks == 1 || (work != nullptr && n_chunks == (T + GRU_CHUNK - 1) / GRU_CHUNK)),
                "b2l_seq_mingru: %d chunks for %d tokens (chunks of %d), or no work space", n_chunks, T, GRU_CHUNK);
  if (T == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const unsigned gx = (unsigned)((width + GRU_THREADS - 1) / GRU_THREADS);
#define B2L_GRU_ARGS (const act_t*)proj, ld, z_off, x_off, g_off, state, meta, (act_t*)out, ldo, work, T, width
  B2L_SEQ_DISPATCH(act_dtype, {
    if (n_chunks == 1) {
      seq_mingru_kernel<act_t, 0><<<gx, GRU_THREADS, 0, s>>>(B2L_GRU_ARGS);
    } else {
      seq_mingru_kernel<act_t, 1><<<dim3(gx, (unsigned)n_chunks), GRU_THREADS, 0, s>>>(B2L_GRU_ARGS);
      seq_mingru_combine_kernel<<<gx, GRU_THREADS, 0, s>>>(state, meta, work, n_chunks, width);
      seq_mingru_kernel<act_t, 2><<<dim3(gx, (unsigned)n_chunks), GRU_THREADS, 0, s>>>(B2L_GRU_ARGS);
    }
  });
#undef B2L_GRU_ARGS
  B2L_LAUNCH_CHECK("seq_mingru_kernel");
  return 0;
}
