// Latent attention: keys and values of every head are linear images of one cached latent vector per position, plus
// one rotated key part shared by all heads.  Only [latent | rotated key] is cached.  One kernel serves two forms:
//  - latent ("absorbed") form, for single tokens and short portions: with q' = W_uk^T q_unrotated per head,
//        score(i, j) = (q'_i . c_j + q_rot_i . k_rot_j) * scale,     o'_i = sum_j weight(i, j) c_j,
//    and the caller maps o' to the value space (W_uv) afterwards.  All heads of all queries are rows over the same
//    cached rows, so one key tile in shared memory serves every row of a CTA and the cache is read once;
//  - expanded form, for long portions: the caller expands [value_h | key_h] of every cached position with one
//    product, and every head attends over its own rows plus the shared rotated part: 3-4 times fewer operations
//    per (query, key) pair when the latent is several times wider than a head.
// Softmax has one learned sink per head in the denominator (exp(sink_h), no key, no value) when a sink is given.  With
// a window a row sees its own position and the window - 1 before it; a CTA then walks only the keys between the first
// key of its first row and the last key of its last row.  Scores, weights and accumulators are f32.
#include <climits>

#include "seq_common.cuh"

namespace b2l {

// A general partial rotation.  Per head of `size` entries: entries [off, off + rot_dims) are rotated by the angle
// (pos0 + t) * freq[i], pairs (2i, 2i+1) when interleaved, else (i, i + rot_dims/2); everything is multiplied by
// `mult` afterwards.  Heads start every hsx (input) / hso (output) elements.  One warp per (token, head).
template <typename in_t, typename out_t>
__global__ void seq_rope_kernel(const in_t* __restrict__ x, int ldx, const float* __restrict__ freq, int rot_dims, int interleaved,
                                int off, float mult, float rot_mult, const int* __restrict__ meta, out_t* __restrict__ out, int ldo, int n_rows, int heads,
                                int size, int hsx, int hso) {
  const int id = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (id >= n_rows * heads) return;
  const int t = id / heads, hd = id % heads;
  const in_t* p = x + (size_t)t * ldx + (size_t)hd * hsx;
  out_t* q = out + (size_t)t * ldo + (size_t)hd * hso;
  const float pos = (float)(meta[1] + t);
  const int half = rot_dims / 2;
  for (int i = lane; i < off; i += 32) st_act(q, i, ld_act(p, i) * mult);
  for (int i = lane; i < half; i += 32) {
    const int iu = off + (interleaved ? 2 * i : i), iv = off + (interleaved ? 2 * i + 1 : i + half);
    const float u = ld_act(p, iu), v = ld_act(p, iv);
    float s, c;
    sincosf(pos * freq[i], &s, &c);
    s *= rot_mult;
    c *= rot_mult;
    st_act(q, iu, (u * c - v * s) * mult);
    st_act(q, iv, (v * c + u * s) * mult);
  }
  for (int i = off + rot_dims + lane; i < size; i += 32) st_act(q, i, ld_act(p, i) * mult);
}

// One CTA per token of the portion, on the f32 product [W_dq ; W_dkv] h:
//   cq  = rmsnorm(proj[q_off : q_off + q_rank]) * wq                       -> cq (act), input of the query up-projection
//   c   = rmsnorm(proj[kv_off : kv_off + rank]) * wkv                      -> cache[slot][pos][0 : rank]
//   k_r = rotate(proj[kv_off + rank : kv_off + rank + rot_dim])            -> cache[slot][pos][rank : rank + rot_dim]
template <typename act_t>
__global__ void __launch_bounds__(128) seq_latent_prep_kernel(const float* __restrict__ proj, int ld, int q_off, int q_rank,
                                                              const act_t* __restrict__ wq, act_t* __restrict__ cq, int kv_off, int rank,
                                                              const act_t* __restrict__ wkv, int rot_dim, const float* __restrict__ freq,
                                                              int rot_dims, int interleaved, float rot_mult, float eps,
                                                              const int* __restrict__ meta, act_t* __restrict__ cache, int max_pos) {
  __shared__ float red[32];
  const int t = blockIdx.x;
  const float* row = proj + (size_t)t * ld;
  {
    const float* a = row + q_off;
    float ss = 0.f;
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x) ss += a[i] * a[i];
    ss = block_sum(ss, red);
    const float r = 1.0f / sqrtf(ss / (float)q_rank + eps);
    act_t* o = cq + (size_t)t * q_rank;
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x) st_act(o, i, a[i] * r * ld_act(wq, i));
  }
  const int slot = meta[0], pos = meta[1] + t;
  const float* a = row + kv_off;
  float ss = 0.f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) ss += a[i] * a[i];
  ss = block_sum(ss, red);
  if (pos < 0 || pos >= max_pos) return;      // the pool never hands out such a position
  const float r = 1.0f / sqrtf(ss / (float)rank + eps);
  act_t* dst = cache + ((size_t)slot * max_pos + pos) * (size_t)(rank + rot_dim);
  for (int i = threadIdx.x; i < rank; i += blockDim.x) st_act(dst, i, a[i] * r * ld_act(wkv, i));
  const float* b = a + rank;
  const int half = rot_dims / 2;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const int iu = interleaved ? 2 * i : i, iv = interleaved ? 2 * i + 1 : i + half;
    float s, c;
    sincosf((float)pos * freq[i], &s, &c);
    s *= rot_mult;
    c *= rot_mult;
    st_act(dst, rank + iu, b[iu] * c - b[iv] * s);
    st_act(dst, rank + iv, b[iv] * c + b[iu] * s);
  }
  for (int i = rot_dims + threadIdx.x; i < rot_dim; i += blockDim.x) st_act(dst, rank + i, b[i]);
}

constexpr int LAT_RW = 4;       // rows (query, head) per warp
constexpr int LAT_BN = 32;      // keys per tile: one per lane
constexpr int LAT_LDK = 33;     // padded key count of the transposed tile
constexpr int LAT_THREADS = 256;

// A key row is [A (n_a entries) | B (n_b entries)]: A per key group, B shared by all groups (the rotated key part).
// Scores use the entries from score_off on, values are the first vdim entries of A.  Two uses:
//   latent form:   one group, A = cached latent, B = cached rotated key, score_off 0, vdim = rank, every head of every
//                  query is a row over the same keys (heads_per_group = heads);
//   expanded form: a group per head (grid.z), A = [value_h | unrotated key_h] expanded from the latent for this call,
//                  score_off = vdim, heads_per_group = 1.
// Rows of a group: r = t * heads_per_group + (h % heads_per_group).  The first `row_warps` warps own LAT_RW
// consecutive rows each, every warp of the CTA helps to load key tiles; grid.y splits the keys.
// Shared: kT[Kp][33] (the key tile transposed, f32), qs[rows][Qp], ps[rows][32].  Scores: lane j owns key j of the
// tile (q read as broadcast float4, kT conflict-free).  Values: lane owns value entries lane + 32 i (weights read
// as broadcast float4, kT with stride 33 conflict-free).
template <typename act_t, int VI>
__global__ void __launch_bounds__(LAT_THREADS, VI <= 4 ? 3 : 1) seq_latent_attention_kernel(b2l_seq_latent_attn_args a, int row_warps) {
  extern __shared__ __align__(16) float lat_smem[];
  const int Kall = a.n_a + a.n_b, Kp = (Kall + 3) & ~3;
  const int s0 = a.score_off & ~3, Qp = Kp - s0;                       // scores run over d in [s0, Kp), q is zero below score_off
  const int nw = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hpg = a.heads_per_group, group = blockIdx.z;
  const int rows_cta = row_warps * LAT_RW, R = a.T * hpg;
  float* kT = lat_smem;
  float* qs = kT + (size_t)Kp * LAT_LDK;
  float* ps = qs + (size_t)rows_cta * Qp;
  const int slot = a.meta[0], pos0 = a.meta[1];
  const int row0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * rows_cta;      // the rows with the most keys start first
  const act_t* key_a = reinterpret_cast<const act_t*>(a.key_a) + (size_t)slot * a.slot_stride_a + (size_t)group * a.hska;
  const act_t* key_b = reinterpret_cast<const act_t*>(a.key_b) + (size_t)slot * a.slot_stride_b;

  // queries of this CTA's rows -> shared (zero beyond the row count, below score_off and in the padding)
  for (int i = threadIdx.x; i < rows_cta * Qp; i += blockDim.x) {
    const int rl = i / Qp, d = s0 + i % Qp, r = row0 + rl;
    float v = 0.f;
    if (r < R && d >= a.score_off && d < Kall) {
      const int t = r / hpg, h = group * hpg + r % hpg;
      v = d < a.n_a ? a.q_a[(size_t)t * a.ldqa_t + (size_t)h * a.ldqa_h + (d - a.score_off)]
                    : a.q_b[(size_t)t * a.ldqb_t + (size_t)h * a.ldqb_h + (d - a.n_a)];
    }
    qs[i] = v;
  }
  for (int i = threadIdx.x; i < (Kp - Kall) * LAT_LDK; i += blockDim.x) kT[(size_t)Kall * LAT_LDK + i] = 0.f;

  // key range of this CTA and split
  const int last_row = min(row0 + rows_cta, R) - 1;
  const int n_keys = pos0 + last_row / hpg + 1;                     // keys k_first .. n_keys-1 are visible to some row of the CTA
  const int k_first = a.window > 0 ? max(0, pos0 + row0 / hpg - a.window + 1) : 0;
  int per = (n_keys - k_first + (int)gridDim.y - 1) / (int)gridDim.y;
  per = (per + LAT_BN - 1) / LAT_BN * LAT_BN;
  const int j_begin = min(n_keys, k_first + (int)blockIdx.y * per), j_end = min(n_keys, j_begin + per);

  int lim[LAT_RW];                                                  // last visible key of each row (-1: no such row)
  float m[LAT_RW], l[LAT_RW], acc[LAT_RW][VI];
#pragma unroll
  for (int r = 0; r < LAT_RW; ++r) {
    const int row = row0 + warp * LAT_RW + r;
    lim[r] = (warp < row_warps && row < R) ? pos0 + row / hpg : -1;
    m[r] = -INFINITY;
    l[r] = 0.f;
#pragma unroll
    for (int i = 0; i < VI; ++i) acc[r][i] = 0.f;
  }
  const int warp_lim = max(max(lim[0], lim[1]), max(lim[2], lim[3]));
  int first[LAT_RW];                                                // first visible key of each row
#pragma unroll
  for (int r = 0; r < LAT_RW; ++r) first[r] = (a.window > 0 && lim[r] >= 0) ? max(0, lim[r] - a.window + 1) : 0;
  int warp_first = INT_MAX;                                         // of the warp's rows that exist
#pragma unroll
  for (int r = 0; r < LAT_RW; ++r)
    if (lim[r] >= 0) warp_first = min(warp_first, first[r]);
  const int wq = min(warp, row_warps - 1);                          // loader-only warps never read these
  const float* qw = qs + (size_t)wq * LAT_RW * Qp;
  float* pw = ps + (size_t)wq * LAT_RW * LAT_BN;

  for (int jt = j_begin; jt < j_end; jt += LAT_BN) {
    __syncthreads();                                                // the previous tile is consumed (and qs is written)
    const int nk = min(LAT_BN, j_end - jt);
    {
      // a warp loads LAT_BN / 8 key rows, lanes along the rows; the loads of all its rows are issued together, before
      // the first store, so a tile costs a few memory latencies instead of one per row
      constexpr int KPW = LAT_BN / (LAT_THREADS / 32);
      const act_t* pa[KPW];
      const act_t* pb[KPW];
      bool ok[KPW];
#pragma unroll
      for (int u = 0; u < KPW; ++u) {
        const int j = warp + u * (LAT_THREADS / 32);
        ok[u] = j < nk;
        pa[u] = key_a + (size_t)(jt + (ok[u] ? j : 0)) * a.ldka;
        pb[u] = key_b + (size_t)(jt + (ok[u] ? j : 0)) * a.ldkb;
      }
#pragma unroll 4
      for (int d = lane; d < a.n_a; d += 32) {
        float v[KPW];
#pragma unroll
        for (int u = 0; u < KPW; ++u) v[u] = ld_act(pa[u], d);
#pragma unroll
        for (int u = 0; u < KPW; ++u) kT[(size_t)d * LAT_LDK + warp + u * (LAT_THREADS / 32)] = ok[u] ? v[u] : 0.f;
      }
#pragma unroll 2
      for (int d = lane; d < a.n_b; d += 32) {
        float v[KPW];
#pragma unroll
        for (int u = 0; u < KPW; ++u) v[u] = ld_act(pb[u], d);
#pragma unroll
        for (int u = 0; u < KPW; ++u) kT[(size_t)(a.n_a + d) * LAT_LDK + warp + u * (LAT_THREADS / 32)] = ok[u] ? v[u] : 0.f;
      }
    }
    __syncthreads();
    if (jt > warp_lim || jt + LAT_BN <= warp_first) continue;       // every key of the tile lies after or before this warp's rows
    float s[LAT_RW] = {0.f, 0.f, 0.f, 0.f}, s2[LAT_RW] = {0.f, 0.f, 0.f, 0.f};     // two chains per row: the FMAs of one hide the other's latency
    int d = s0;
    for (; d + 8 <= Kp; d += 8) {
      float k[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) k[u] = kT[(size_t)(d + u) * LAT_LDK + lane];
#pragma unroll
      for (int r = 0; r < LAT_RW; ++r) {
        const float4 qa = *reinterpret_cast<const float4*>(qw + (size_t)r * Qp + (d - s0));
        const float4 qb = *reinterpret_cast<const float4*>(qw + (size_t)r * Qp + (d - s0) + 4);
        s[r] = fmaf(qa.x, k[0], fmaf(qa.y, k[1], fmaf(qa.z, k[2], fmaf(qa.w, k[3], s[r]))));
        s2[r] = fmaf(qb.x, k[4], fmaf(qb.y, k[5], fmaf(qb.z, k[6], fmaf(qb.w, k[7], s2[r]))));
      }
    }
    for (; d < Kp; d += 4) {
      const float k0 = kT[(size_t)d * LAT_LDK + lane], k1 = kT[(size_t)(d + 1) * LAT_LDK + lane];
      const float k2 = kT[(size_t)(d + 2) * LAT_LDK + lane], k3 = kT[(size_t)(d + 3) * LAT_LDK + lane];
#pragma unroll
      for (int r = 0; r < LAT_RW; ++r) {
        const float4 q4 = *reinterpret_cast<const float4*>(qw + (size_t)r * Qp + (d - s0));
        s[r] = fmaf(q4.x, k0, fmaf(q4.y, k1, fmaf(q4.z, k2, fmaf(q4.w, k3, s[r]))));
      }
    }
#pragma unroll
    for (int r = 0; r < LAT_RW; ++r) s[r] += s2[r];
    const int j = jt + lane;
#pragma unroll
    for (int r = 0; r < LAT_RW; ++r) {
      const bool seen = lane < nk && j <= lim[r] && j >= first[r];
      const float sc = seen ? s[r] * a.scale : -INFINITY;
      const float mn = fmaxf(m[r], warp_max(sc));
      float p = 0.f, corr = 1.f;
      if (mn > -INFINITY) {
        p = seen ? expf(sc - mn) : 0.f;
        corr = expf(m[r] - mn);                                     // m = -inf: 0
      }
      l[r] = l[r] * corr + warp_sum(p);
      m[r] = mn;
#pragma unroll
      for (int i = 0; i < VI; ++i) acc[r][i] *= corr;
      pw[r * LAT_BN + lane] = p;
    }
    __syncwarp();
#pragma unroll 2
    for (int jj = 0; jj < LAT_BN; jj += 4) {
      float4 p4[LAT_RW];
#pragma unroll
      for (int r = 0; r < LAT_RW; ++r) p4[r] = *reinterpret_cast<const float4*>(pw + r * LAT_BN + jj);
#pragma unroll
      for (int i = 0; i < VI; ++i) {
        const int v = lane + 32 * i;
        if (v < a.vdim) {
          const float* kv = kT + (size_t)v * LAT_LDK + jj;
          const float c0 = kv[0], c1 = kv[1], c2 = kv[2], c3 = kv[3];
#pragma unroll
          for (int r = 0; r < LAT_RW; ++r)
            acc[r][i] = fmaf(p4[r].x, c0, fmaf(p4[r].y, c1, fmaf(p4[r].z, c2, fmaf(p4[r].w, c3, acc[r][i]))));
        }
      }
    }
    __syncwarp();
  }

  if (warp >= row_warps) return;
#pragma unroll
  for (int r = 0; r < LAT_RW; ++r) {
    const int row = row0 + warp * LAT_RW + r;
    if (row >= R) continue;
    const int t = row / hpg, h = group * hpg + row % hpg;
    if (gridDim.y == 1) {
      const float sink = a.sink ? a.sink[h] : -INFINITY;            // without a sink every row sees its own key: m is finite
      const float M = fmaxf(m[r], sink);
      const float e = expf(m[r] - M);                               // m = -inf (no key): 0
      const float inv = e / (l[r] * e + (a.sink ? expf(sink - M) : 0.f));
      act_t* o = reinterpret_cast<act_t*>(a.out) + (size_t)t * a.ldo + (size_t)h * a.vdim;
#pragma unroll
      for (int i = 0; i < VI; ++i) {
        const int v = lane + 32 * i;
        if (v < a.vdim) st_act(o, v, acc[r][i] * inv);
      }
    } else {
      float* w = a.work + ((size_t)blockIdx.y * a.T * a.heads + (size_t)t * a.heads + h) * (size_t)(a.vdim + 2);
      if (lane == 0) {
        w[0] = m[r];
        w[1] = l[r];
      }
#pragma unroll
      for (int i = 0; i < VI; ++i) {
        const int v = lane + 32 * i;
        if (v < a.vdim) w[2 + v] = acc[r][i];
      }
    }
  }
}

// Merges the key splits of a row and adds the sink.  One CTA per row (t, h): warp 0 turns every split's running
// maximum and sum into one factor exp(m_s - M) / denominator, then the threads own value entries and add the
// splits' accumulators with independent loads.
template <typename act_t>
__global__ void __launch_bounds__(256) seq_latent_combine_kernel(const float* __restrict__ work, const float* __restrict__ sink,
                                                                 act_t* __restrict__ out, int ldo, int R, int heads, int vdim, int splits) {
  extern __shared__ float comb_f[];                      // [splits]
  const int row = blockIdx.x, t = row / heads, h = row % heads;
  const size_t stride = (size_t)(vdim + 2);
  const float* w0 = work + (size_t)row * stride;
  const size_t sstep = (size_t)R * stride;
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    const float sk = sink ? sink[h] : -INFINITY;
    float M = sk;
    for (int s = lane; s < splits; s += 32) M = fmaxf(M, w0[(size_t)s * sstep]);
    M = warp_max(M);
    float den = 0.f;
    for (int s = lane; s < splits; s += 32) {
      const float m = w0[(size_t)s * sstep];
      const float f = m > -INFINITY ? expf(m - M) : 0.f;
      comb_f[s] = f;
      den += f * w0[(size_t)s * sstep + 1];
    }
    den = warp_sum(den) + (sink ? expf(sk - M) : 0.f);
    const float inv = 1.0f / den;
    for (int s = lane; s < splits; s += 32) comb_f[s] *= inv;
  }
  __syncthreads();
  act_t* o = out + (size_t)t * ldo + (size_t)h * vdim;
  for (int v = threadIdx.x; v < vdim; v += blockDim.x) {
    float acc = 0.f;
#pragma unroll 16
    for (int s = 0; s < splits; ++s) {
      acc = fmaf(w0[(size_t)s * sstep + 2 + v], comb_f[s], acc);            // an empty split wrote zeros and has factor 0
    }
    st_act(o, v, acc);
  }
}

static DynSmemCache g_lat_smem[8];

template <typename act_t, int VI>
static int launch_latent(const b2l_seq_latent_attn_args& a, int row_warps, size_t smem, int cache_id, cudaStream_t st) {
  auto kern = seq_latent_attention_kernel<act_t, VI>;
  if (smem > 48 * 1024) {
    const int rc = ensure_dyn_smem(kern, smem, g_lat_smem[cache_id]);
    if (rc != 0) return rc;
  }
  const int R = a.T * a.heads_per_group, rows_cta = row_warps * LAT_RW;
  kern<<<dim3((R + rows_cta - 1) / rows_cta, a.splits, a.heads / a.heads_per_group), LAT_THREADS, smem, st>>>(a, row_warps);
  return 0;
}

}  // namespace b2l

using namespace b2l;

extern "C" int b2l_seq_rope(const void* x, int ldx, int in_f32, const float* freq, int rot_dims, int interleaved, int rot_off,
                            float mult, float rot_mult, const int* meta, void* out, int ldo, int out_f32, int T, int heads, int size,
                            int hsx, int hso, int act_dtype, b2l_stream_t stream) {
  B2L_CHECK_ARG(x && meta && out, "b2l_seq_rope: null pointer");
  B2L_CHECK_ARG(T >= 0 && heads > 0 && size > 0 && hsx >= size && hso >= size && ldx >= (heads - 1) * hsx + size && ldo >= (heads - 1) * hso + size,
                "b2l_seq_rope: bad size");
  B2L_CHECK_ARG(rot_dims >= 0 && rot_off >= 0 && rot_off + rot_dims <= size && rot_dims % 2 == 0 && (rot_dims == 0 || freq),
                "b2l_seq_rope: bad rotation");
  if (T == 0) return 0;
  const int ids = T * heads, grid = (ids + 3) / 4;
  cudaStream_t st = (cudaStream_t)stream;
#define B2L_ROPE_GO(IN, OUT) \
  seq_rope_kernel<IN, OUT><<<grid, 128, 0, st>>>((const IN*)x, ldx, freq, rot_dims, interleaved, rot_off, mult, rot_mult, meta, (OUT*)out, ldo, T, heads, size, hsx, hso)
  B2L_SEQ_DISPATCH(act_dtype, {
    if (in_f32 && out_f32) B2L_ROPE_GO(float, float);
    else if (in_f32) B2L_ROPE_GO(float, act_t);
    else if (out_f32) B2L_ROPE_GO(act_t, float);
    else B2L_ROPE_GO(act_t, act_t);
  });
#undef B2L_ROPE_GO
  B2L_LAUNCH_CHECK("seq_rope_kernel");
  return 0;
}

extern "C" int b2l_seq_latent_prep(const float* proj, int ld, int q_off, int q_rank, const void* w_q, void* cq, int kv_off,
                                   int rank, const void* w_kv, int rot_dim, const float* freq, int rot_dims, int interleaved,
                                   float rot_mult, float eps, const int* meta, void* cache, int max_pos, int T, int act_dtype,
                                   b2l_stream_t stream) {
  B2L_CHECK_ARG(proj && w_q && cq && w_kv && meta && cache, "b2l_seq_latent_prep: null pointer");
  B2L_CHECK_ARG(T >= 0 && q_rank > 0 && rank > 0 && rot_dim >= 0 && max_pos > 0 && q_off >= 0 && kv_off >= 0 && ld >= q_off + q_rank &&
                    ld >= kv_off + rank + rot_dim, "b2l_seq_latent_prep: bad size");
  B2L_CHECK_ARG(rot_dims >= 0 && rot_dims <= rot_dim && rot_dims % 2 == 0 && (rot_dims == 0 || freq), "b2l_seq_latent_prep: bad rotation");
  if (T == 0) return 0;
  B2L_SEQ_DISPATCH(act_dtype, {
    seq_latent_prep_kernel<act_t><<<T, 128, 0, (cudaStream_t)stream>>>(proj, ld, q_off, q_rank, (const act_t*)w_q, (act_t*)cq, kv_off, rank,
                                                                      (const act_t*)w_kv, rot_dim, freq, rot_dims, interleaved, rot_mult, eps, meta,
                                                                      (act_t*)cache, max_pos);
  });
  B2L_LAUNCH_CHECK("seq_latent_prep_kernel");
  return 0;
}

extern "C" int b2l_seq_latent_attention_warps(int T, int heads_per_group) {
  const int rows = T * heads_per_group;
  int w = (rows + LAT_RW - 1) / LAT_RW;
  return w < 1 ? 1 : (w > 8 ? 8 : w);
}

extern "C" int b2l_seq_latent_attention(const b2l_seq_latent_attn_args* a, b2l_stream_t stream) {
  B2L_CHECK_ARG(a != nullptr, "b2l_seq_latent_attention: null args");
  B2L_CHECK_ARG(a->q_a && a->key_a && a->meta && a->out && (a->n_b == 0 || (a->q_b && a->key_b)), "b2l_seq_latent_attention: null pointer");
  B2L_CHECK_ARG(a->window >= 0, "b2l_seq_latent_attention: negative window");
  B2L_CHECK_ARG(a->T >= 0 && a->heads > 0 && a->heads_per_group > 0 && a->heads % a->heads_per_group == 0 && a->n_a > 0 && a->n_b >= 0 &&
                    a->vdim > 0 && a->vdim <= a->n_a && a->score_off >= 0 && a->score_off < a->n_a + a->n_b && a->score_off <= a->n_a &&
                    a->splits >= 1 && a->ldo >= a->heads * a->vdim, "b2l_seq_latent_attention: bad size");
  B2L_CHECK_ARG(a->splits == 1 || a->work, "b2l_seq_latent_attention: key splits need a workspace");
  B2L_CHECK_SUPPORTED(a->splits <= 4096, "b2l_seq_latent_attention: %d key splits > 4096", a->splits);
  B2L_CHECK_SUPPORTED(a->vdim <= 512, "b2l_seq_latent_attention: value size %d > 512", a->vdim);
  if (a->T == 0) return 0;
  const int row_warps = b2l_seq_latent_attention_warps(a->T, a->heads_per_group);
  const int Kall = a->n_a + a->n_b, Kp = (Kall + 3) & ~3, Qp = Kp - (a->score_off & ~3);
  const size_t smem = sizeof(float) * ((size_t)Kp * LAT_LDK + (size_t)row_warps * LAT_RW * Qp + (size_t)row_warps * LAT_RW * LAT_BN);
  B2L_CHECK_SUPPORTED(smem <= 220 * 1024, "b2l_seq_latent_attention: key size %d needs %zu bytes of shared memory", Kall, smem);
  cudaStream_t st = (cudaStream_t)stream;
  int rc = 0;
  B2L_SEQ_DISPATCH(a->act_dtype, {
    const int base = sizeof(act_t) == 2 ? 0 : 4;
    if (a->vdim <= 64) rc = launch_latent<act_t, 2>(*a, row_warps, smem, base + 0, st);
    else if (a->vdim <= 128) rc = launch_latent<act_t, 4>(*a, row_warps, smem, base + 1, st);
    else if (a->vdim <= 256) rc = launch_latent<act_t, 8>(*a, row_warps, smem, base + 2, st);
    else rc = launch_latent<act_t, 16>(*a, row_warps, smem, base + 3, st);
  });
  if (rc != 0) return rc;
  B2L_LAUNCH_CHECK("seq_latent_attention_kernel");
  if (a->splits > 1) {
    const int R = a->T * a->heads;
    B2L_SEQ_DISPATCH(a->act_dtype, {
      seq_latent_combine_kernel<act_t><<<R, a->vdim > 128 ? 256 : 128, sizeof(float) * a->splits, st>>>(a->work, a->sink, (act_t*)a->out, a->ldo, R, a->heads, a->vdim, a->splits);
    });
    B2L_LAUNCH_CHECK("seq_latent_combine_kernel");
  }
  return 0;
}
