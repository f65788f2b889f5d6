// Local causal softmax attention with an optional sink term, score soft-capping, grouped key/value heads, a sigmoid
// output gate (one per head or one per channel) and a ring cache of `block` positions.  Two kinds of locality:
//   block-local (window == 0): a query at position p sees keys j <= p with j / block == p / block;
//   sliding window (window > 0): it sees the keys p - window + 1 .. p (itself and the window - 1 positions before it).
// Either way a sequence never needs more than `block` cached positions: entry p % block of the ring.  Keys of the portion being processed are read from the fresh
// projections (k_new / v_new), older ones of the same block from the ring; the ring is advanced AFTER the
// attention kernel (a second kernel in the same call), so a portion longer than a block cannot overwrite what it
// still has to read.
//
// warp kernel (single tokens, and shapes the tiled kernel does not take): WPQ warps per (query, head).  A warp takes batches of 32 consecutive keys: each lane scores one
// key (q from shared memory, its key row by 16-byte loads), the batch maximum and the weights go through shuffles,
// and the value rows are accumulated with lanes over value channels.  Scores, weights and accumulators are f32.
//
// Several maps over the same values (maps > 1): every query head and every key head carries `maps` score vectors of K
// entries; each map is a softmax attention of its own and is handled as a head of its own ("virtual head" h = real
// head * maps + map) that reads key map (h % maps) of its key/value head and that head's values.  The maps' outputs are
// stored side by side; combining them (for instance the difference of two maps) is the caller's next kernel.
#include "seq_common.cuh"

namespace b2l {

constexpr int ATT_VMAX = 8;   // value channels per lane: V <= 256

// Key head and value head of (virtual) query head h.
__device__ __forceinline__ void kv_heads_of(const b2l_seq_attn_args& a, int h, int& gk, int& gv) {
  const int maps = a.maps > 1 ? a.maps : 1;
  const int hr = h / maps;
  gv = hr / ((a.heads / maps) / a.kv_heads);
  gk = gv * maps + (h - hr * maps);
}

template <typename act_t>
__device__ __forceinline__ void st_out(const b2l_seq_attn_args& a, size_t i, float v) {
  if (a.out_f32) reinterpret_cast<float*>(a.out)[i] = v;
  else st_act(reinterpret_cast<act_t*>(a.out), i, v);
}

// The first position a query at position p sees.
__device__ __forceinline__ int first_visible(const b2l_seq_attn_args& a, int p) {
  return a.window > 0 ? max(0, p - a.window + 1) : (p / a.block) * a.block;
}

template <typename act_t>
__device__ __forceinline__ float dot_row(const float* __restrict__ q, const act_t* __restrict__ k, int K, bool vec);

template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const float* __restrict__ q, const __nv_bfloat16* __restrict__ k, int K, bool vec) {
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  if (vec) {
#pragma unroll 4
    for (int i = 0; i < K; i += 8) {
      const uint4 w = *reinterpret_cast<const uint4*>(k + i);
      const float4 qa = *reinterpret_cast<const float4*>(q + i), qb = *reinterpret_cast<const float4*>(q + i + 4);
      s0 = fmaf(__uint_as_float(w.x << 16), qa.x, s0); s1 = fmaf(__uint_as_float(w.x & 0xffff0000u), qa.y, s1);
      s2 = fmaf(__uint_as_float(w.y << 16), qa.z, s2); s3 = fmaf(__uint_as_float(w.y & 0xffff0000u), qa.w, s3);
      s0 = fmaf(__uint_as_float(w.z << 16), qb.x, s0); s1 = fmaf(__uint_as_float(w.z & 0xffff0000u), qb.y, s1);
      s2 = fmaf(__uint_as_float(w.w << 16), qb.z, s2); s3 = fmaf(__uint_as_float(w.w & 0xffff0000u), qb.w, s3);
    }
  } else {
    for (int i = 0; i < K; ++i) s0 = fmaf(__bfloat162float(k[i]), q[i], s0);
  }
  return (s0 + s1) + (s2 + s3);
}

template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ q, const float* __restrict__ k, int K, bool vec) {
  float s0 = 0.f, s1 = 0.f;
  if (vec) {
    for (int i = 0; i < K; i += 4) {
      const float4 w = *reinterpret_cast<const float4*>(k + i), qa = *reinterpret_cast<const float4*>(q + i);
      s0 = fmaf(w.x, qa.x, s0); s1 = fmaf(w.y, qa.y, s1);
      s0 = fmaf(w.z, qa.z, s0); s1 = fmaf(w.w, qa.w, s1);
    }
  } else {
    for (int i = 0; i < K; ++i) s0 = fmaf(k[i], q[i], s0);
  }
  return s0 + s1;
}

template <typename act_t, int WPQ>
__global__ void __launch_bounds__(WPQ > 4 ? 32 * WPQ : 128) seq_block_attention_kernel(b2l_seq_attn_args a, int vec) {
  extern __shared__ float smem[];
  constexpr int NW = WPQ > 4 ? WPQ : 4;              // warps per CTA
  constexpr int QPC = NW / WPQ;                      // (query, head) pairs per CTA
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int K = a.K, V = a.V, Kpad = (K + 3) & ~3;
  float* sq = smem;                                  // [QPC][Kpad]
  float* sm = sq + QPC * Kpad;                       // merge area [NW][2 + 32 * ATT_VMAX]

  const int pair = blockIdx.x * QPC + warp / WPQ, sub = warp % WPQ;
  const bool live = pair < a.T * a.heads;
  const int t = live ? pair / a.heads : 0, h = live ? pair % a.heads : 0;
  int gk, gv;
  kv_heads_of(a, h, gk, gv);
  const int kh = a.kv_heads * (a.maps > 1 ? a.maps : 1);
  const int slot = a.meta[0], pos0 = a.meta[1];
  const int p = pos0 + t, c0 = first_visible(a, p);

  float* myq = sq + (warp / WPQ) * Kpad;
  if (live && sub == 0)
    for (int i = lane; i < K; i += 32) myq[i] = a.q[((size_t)t * a.heads + h) * K + i];
  __syncthreads();

  const act_t* kn = (const act_t*)a.k_new;
  const act_t* vn = (const act_t*)a.v_new;
  const act_t* ck = (const act_t*)a.cache_k + (size_t)slot * a.block * kh * K;
  const act_t* cv = (const act_t*)a.cache_v + (size_t)slot * a.block * a.kv_heads * V;

  float m = a.has_sink ? 0.f : -INFINITY, l = (a.has_sink && sub == 0) ? 1.f : 0.f;
  float acc[ATT_VMAX];
#pragma unroll
  for (int c = 0; c < ATT_VMAX; ++c) acc[c] = 0.f;

  if (live) {
    for (int jb = c0 + sub * 32; jb <= p; jb += 32 * WPQ) {
      const int j = jb + lane;
      float s = -INFINITY;
      if (j <= p) {
        const act_t* kr = j >= pos0 ? kn + ((size_t)(j - pos0) * kh + gk) * K
                                    : ck + ((size_t)(j % a.block) * kh + gk) * K;
        s = dot_row<act_t>(myq, kr, K, vec != 0) * a.scale;
        if (a.softcap > 0.f) s = a.softcap * tanhf(s / a.softcap);
      }
      const float mn = fmaxf(m, warp_max(s));
      const float corr = expf(m - mn);                 // m = -inf only before the first batch without a sink: acc and l are 0
      const float w = j <= p ? expf(s - mn) : 0.f;
      l = l * (m == -INFINITY ? 0.f : corr) + warp_sum(w);
#pragma unroll
      for (int c = 0; c < ATT_VMAX; ++c) acc[c] *= (m == -INFINITY ? 0.f : corr);
      m = mn;
      const int nb = min(32, p - jb + 1);
#pragma unroll 8
      for (int jj = 0; jj < 32; ++jj) {
        const float wj = __shfl_sync(0xffffffffu, w, jj);      // 0 beyond the last key of the batch
        const int jv = jb + min(jj, nb - 1);                    // a valid row for the masked tail (weight 0)
        const act_t* vr = jv >= pos0 ? vn + (size_t)(jv - pos0) * a.ldv + (size_t)gv * V
                                     : cv + ((size_t)(jv % a.block) * a.kv_heads + gv) * V;
#pragma unroll
        for (int c = 0; c < ATT_VMAX; ++c) {
          const int ch = c * 32 + lane;
          if (ch < V) acc[c] = fmaf(wj, ld_act(vr, ch), acc[c]);
        }
      }
    }
  }

  if (WPQ > 1) {   // merge the partial softmaxes of the WPQ warps of this pair (QPC == 1)
    float* mine = sm + warp * (2 + ATT_VMAX * 32);
    if (lane == 0) { mine[0] = m; mine[1] = l; }
#pragma unroll
    for (int c = 0; c < ATT_VMAX; ++c) mine[2 + c * 32 + lane] = acc[c];
    __syncthreads();
    if (warp != 0) return;
    float M = -INFINITY;
    for (int w = 0; w < WPQ; ++w) M = fmaxf(M, sm[w * (2 + ATT_VMAX * 32)]);
    l = 0.f;
#pragma unroll
    for (int c = 0; c < ATT_VMAX; ++c) acc[c] = 0.f;
    for (int w = 0; w < WPQ; ++w) {
      const float* o = sm + w * (2 + ATT_VMAX * 32);
      const float f = o[0] == -INFINITY ? 0.f : expf(o[0] - M);
      l += o[1] * f;
#pragma unroll
      for (int c = 0; c < ATT_VMAX; ++c) acc[c] += o[2 + c * 32 + lane] * f;
    }
  }
  if (!live) return;
  float f = a.out_mult / l;
  const act_t* gate = (const act_t*)a.gate + (size_t)t * a.ldg;
  if (a.gate && !a.gate_per_channel) f *= sigmoid_f(ld_act(gate, h));
  const size_t o = (size_t)t * a.ldo + (size_t)h * V;
#pragma unroll
  for (int c = 0; c < ATT_VMAX; ++c) {
    const int ch = c * 32 + lane;
    if (ch < V) st_out<act_t>(a, o + ch, acc[c] * f * ((a.gate && a.gate_per_channel) ? sigmoid_f(ld_act(gate, (size_t)h * V + ch)) : 1.f));
  }
}

// ---- a few queries (decoding): a CTA takes DEC_CK consecutive keys of one query for ALL query heads of one key/value
// group, so a cached row is read once per group: keys and values of the chunk arrive in shared memory by 16-byte
// asynchronous copies (plain loads for odd sizes), the scores of (head, key) pairs are spread over the threads with padded
// key rows (conflict-free 16-byte reads), a warp per head forms the chunk's softmax, and the value product gives one
// output channel of one head per thread.  Every chunk writes {max, sum, weighted values} to the work space and a second
// kernel merges the chunks of a (query, head), adds the sink, applies the gate and stores.  The grid covers the most keys
// a query can see (the window or the block), not the position, so a captured single-token step replays anywhere.
constexpr int DEC_CK = 64, DEC_THREADS = 128;

__device__ __forceinline__ void dec_cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void dec_cp_wait_all() {
  asm volatile("cp.async.commit_group;" ::: "memory");
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

template <typename act_t>
__global__ void __launch_bounds__(DEC_THREADS) seq_attention_chunk_kernel(b2l_seq_attn_args a, int n_chunks, int vec) {
  extern __shared__ __align__(16) unsigned char dec_smem[];
  constexpr int PER = 16 / (int)sizeof(act_t);
  const int maps = a.maps > 1 ? a.maps : 1;
  const int K = a.K, KR = K * maps, V = a.V, Kpa = KR + PER, hpg = a.heads / a.kv_heads;      // a key row holds the maps side by side
  const int Vp = (V + PER - 1) / PER * PER;
  act_t* sK = reinterpret_cast<act_t*>(dec_smem);                 // [DEC_CK][Kpa]
  act_t* sV = sK + DEC_CK * Kpa;                                  // [DEC_CK][Vp]
  float* sQ = reinterpret_cast<float*>(sV + DEC_CK * Vp);         // [hpg][K]
  float* sS = sQ + hpg * K;                                       // [hpg][DEC_CK]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c = blockIdx.x, g = blockIdx.y, t = blockIdx.z;
  const int slot = a.meta[0], pos0 = a.meta[1];
  const int p = pos0 + t, lo = first_visible(a, p) + c * DEC_CK;
  const int nv = min(DEC_CK, p - lo + 1);                         // keys of this chunk that the query sees
  float* part = a.work + ((size_t)(t * a.heads + g * hpg) * n_chunks + c) * (V + 2);      // head hq: + hq * n_chunks * (V + 2)
  if (a.T == 1 && c == 0 && !a.no_append) {
    // A single token appends itself to the ring here: its entry p % block holds a position that no query of this call
    // sees (one ring turn back), and the chunks read the token's own key and value from k_new / v_new.
    act_t* rk = (act_t*)a.cache_k + (((size_t)slot * a.block + p % a.block) * a.kv_heads + g) * KR;
    act_t* rv = (act_t*)a.cache_v + (((size_t)slot * a.block + p % a.block) * a.kv_heads + g) * a.V;
    const act_t* nk = (const act_t*)a.k_new + (size_t)g * KR;
    const act_t* nvv = (const act_t*)a.v_new + (size_t)g * a.V;
    for (int i = threadIdx.x; i < KR; i += DEC_THREADS) rk[i] = nk[i];
    for (int i = threadIdx.x; i < a.V; i += DEC_THREADS) rv[i] = nvv[i];
  }
  if (nv <= 0) {
    for (int hq = tid; hq < hpg; hq += DEC_THREADS) {
      part[(size_t)hq * n_chunks * (V + 2)] = -INFINITY;
      part[(size_t)hq * n_chunks * (V + 2) + 1] = 0.f;
    }
    return;
  }
  const act_t* kn = (const act_t*)a.k_new;
  const act_t* vn = (const act_t*)a.v_new;
  const act_t* ck = (const act_t*)a.cache_k + (size_t)slot * a.block * a.kv_heads * KR;
  const act_t* cv = (const act_t*)a.cache_v + (size_t)slot * a.block * a.kv_heads * V;
  if (vec) {
    const int kc = KR / PER, vc = V / PER;
    for (int i = tid; i < nv * kc; i += DEC_THREADS) {
      const int r = i / kc, e = (i - r * kc) * PER, j = lo + r;
      dec_cp_async16(sK + r * Kpa + e, j >= pos0 ? kn + ((size_t)(j - pos0) * a.kv_heads + g) * KR + e : ck + ((size_t)(j % a.block) * a.kv_heads + g) * KR + e);
    }
    for (int i = tid; i < nv * vc; i += DEC_THREADS) {
      const int r = i / vc, e = (i - r * vc) * PER, j = lo + r;
      dec_cp_async16(sV + r * Vp + e, j >= pos0 ? vn + (size_t)(j - pos0) * a.ldv + (size_t)g * V + e : cv + ((size_t)(j % a.block) * a.kv_heads + g) * V + e);
    }
  } else {
    for (int i = tid; i < nv * KR; i += DEC_THREADS) {
      const int r = i / KR, e = i - r * KR, j = lo + r;
      sK[r * Kpa + e] = j >= pos0 ? kn[((size_t)(j - pos0) * a.kv_heads + g) * KR + e] : ck[((size_t)(j % a.block) * a.kv_heads + g) * KR + e];
    }
    for (int i = tid; i < nv * V; i += DEC_THREADS) {
      const int r = i / V, e = i - r * V, j = lo + r;
      sV[r * Vp + e] = j >= pos0 ? vn[(size_t)(j - pos0) * a.ldv + (size_t)g * V + e] : cv[((size_t)(j % a.block) * a.kv_heads + g) * V + e];
    }
  }
  for (int i = tid; i < hpg * K; i += DEC_THREADS) sQ[i] = a.q[((size_t)t * a.heads + (size_t)g * hpg) * K + i];
  dec_cp_wait_all();
  __syncthreads();
  for (int i = tid; i < hpg * DEC_CK; i += DEC_THREADS) {          // a warp: 32 consecutive keys of one head
    const int hq = i / DEC_CK, r = i - hq * DEC_CK;
    float sc = -INFINITY;
    if (r < nv) {
      sc = dot_row<act_t>(sQ + hq * K, sK + r * Kpa + (hq % maps) * K, K, vec != 0) * a.scale;      // the group's first head is a multiple of maps
      if (a.softcap > 0.f) sc = a.softcap * tanhf(sc / a.softcap);
    }
    sS[i] = sc;
  }
  __syncthreads();
  for (int hq = warp; hq < hpg; hq += DEC_THREADS / 32) {
    float* row = sS + hq * DEC_CK;
    float m = -INFINITY;
    for (int r = lane; r < DEC_CK; r += 32) m = fmaxf(m, row[r]);
    m = warp_max(m);                                             // finite: the chunk has at least one visible key
    float l = 0.f;
    for (int r = lane; r < DEC_CK; r += 32) {
      const float w = r < nv ? expf(row[r] - m) : 0.f;
      row[r] = w;
      l += w;
    }
    l = warp_sum(l);
    if (lane == 0) {
      part[(size_t)hq * n_chunks * (V + 2)] = m;
      part[(size_t)hq * n_chunks * (V + 2) + 1] = l;
    }
  }
  __syncthreads();
  for (int i = tid; i < hpg * V; i += DEC_THREADS) {
    const int hq = i / V, ch = i - hq * V;
    const float* w = sS + hq * DEC_CK;
    float acc0 = 0.f, acc1 = 0.f;
    int r = 0;
    for (; r + 1 < nv; r += 2) {
      acc0 = fmaf(w[r], ld_act(sV, (size_t)r * Vp + ch), acc0);
      acc1 = fmaf(w[r + 1], ld_act(sV, (size_t)(r + 1) * Vp + ch), acc1);
    }
    if (r < nv) acc0 = fmaf(w[r], ld_act(sV, (size_t)r * Vp + ch), acc0);
    part[(size_t)hq * n_chunks * (V + 2) + 2 + ch] = acc0 + acc1;
  }
}

// out[t, h] = gate * out_mult * sum_c e^(m_c - M) acc_c / (sink e^(-M) + sum_c e^(m_c - M) l_c): one CTA per (query, head).
// The chunk factors go through shared memory, so the loads of the channel sums do not wait for one another.
constexpr int MERGE_THREADS = 128;

// The merged, normalised output channels `ch = tid + 128 i` of one (query, virtual head) row into val[i]; the sink and
// out_mult are applied, gates are not.  Ends with every thread past its reads of merge_f and red.
__device__ __forceinline__ void merge_row(const b2l_seq_attn_args& a, const float* __restrict__ part, int n_chunks, float* merge_f, float* red,
                                          float (&val)[ATT_VMAX * 32 / MERGE_THREADS]) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, V = a.V;
  float M = a.has_sink ? 0.f : -INFINITY;
  for (int c = tid; c < n_chunks; c += MERGE_THREADS) M = fmaxf(M, part[(size_t)c * (V + 2)]);
  M = warp_max(M);
  if (lane == 0) red[warp] = M;
  __syncthreads();
#pragma unroll
  for (int w = 0; w < MERGE_THREADS / 32; ++w) M = fmaxf(M, red[w]);
  __syncthreads();
  float l = 0.f;
  for (int c = tid; c < n_chunks; c += MERGE_THREADS) {
    const float m = part[(size_t)c * (V + 2)];
    const float f = m == -INFINITY ? 0.f : expf(m - M);
    merge_f[c] = f;
    if (f != 0.f) l += part[(size_t)c * (V + 2) + 1] * f;
  }
  l = warp_sum(l);
  if (lane == 0) red[warp] = l;
  __syncthreads();
  l = 0.f;
#pragma unroll
  for (int w = 0; w < MERGE_THREADS / 32; ++w) l += red[w];
  if (a.has_sink) l += expf(0.f - M);
  const float f = a.out_mult / l;
#pragma unroll
  for (int i = 0; i < ATT_VMAX * 32 / MERGE_THREADS; ++i) {
    const int ch = tid + i * MERGE_THREADS;
    val[i] = 0.f;
    if (ch >= V) continue;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    int c = 0;
    for (; c + 4 <= n_chunks; c += 4) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float fc = merge_f[c + u];
        const float v = fc != 0.f ? part[(size_t)(c + u) * (V + 2) + 2 + ch] : 0.f;      // an empty chunk wrote nothing there
        acc[u] = fmaf(v, fc, acc[u]);
      }
    }
    for (; c < n_chunks; ++c) {
      const float fc = merge_f[c];
      if (fc != 0.f) acc[0] = fmaf(part[(size_t)c * (V + 2) + 2 + ch], fc, acc[0]);
    }
    val[i] = ((acc[0] + acc[1]) + (acc[2] + acc[3])) * f;
  }
  __syncthreads();
}

// DIFF == false: one CTA per (query, virtual head): merge, gate, store.
// DIFF == true (two maps per head and a differential read-out asked for): one CTA per (query, real head) merges both maps
// and stores (a_0 - lambda a_1) / rms * mult in the activation type: the maps never go through memory.
template <typename act_t, bool DIFF>
__global__ void __launch_bounds__(MERGE_THREADS) seq_attention_merge_kernel(b2l_seq_attn_args a, int n_chunks) {
  extern __shared__ float merge_f[];                 // [n_chunks]
  __shared__ float red[MERGE_THREADS / 32];
  constexpr int CPT = ATT_VMAX * 32 / MERGE_THREADS;  // channels per thread
  const int tid = threadIdx.x, V = a.V;
  if (!DIFF) {
    const int pair = blockIdx.x, t = pair / a.heads, h = pair - t * a.heads;
    float val[CPT];
    merge_row(a, a.work + (size_t)pair * n_chunks * (V + 2), n_chunks, merge_f, red, val);
    const act_t* gate = (const act_t*)a.gate + (size_t)t * a.ldg;
    const float g = (a.gate && !a.gate_per_channel) ? sigmoid_f(ld_act(gate, h)) : 1.f;
    const size_t o = (size_t)t * a.ldo + (size_t)h * V;
#pragma unroll
    for (int i = 0; i < CPT; ++i) {
      const int ch = tid + i * MERGE_THREADS;
      if (ch < V) st_out<act_t>(a, o + ch, val[i] * g * ((a.gate && a.gate_per_channel) ? sigmoid_f(ld_act(gate, (size_t)h * V + ch)) : 1.f));
    }
  } else {
    const int real = a.heads / 2, t = blockIdx.x / real, hr = blockIdx.x - t * real;
    float v0[CPT], v1[CPT];
    merge_row(a, a.work + (size_t)(t * a.heads + 2 * hr) * n_chunks * (V + 2), n_chunks, merge_f, red, v0);
    merge_row(a, a.work + (size_t)(t * a.heads + 2 * hr + 1) * n_chunks * (V + 2), n_chunks, merge_f, red, v1);
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < CPT; ++i) {
      v0[i] -= a.diff_lambda * v1[i];                 // channels beyond V are 0 in both
      ss += v0[i] * v0[i];
    }
    ss = warp_sum(ss);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    ss = 0.f;
#pragma unroll
    for (int w = 0; w < MERGE_THREADS / 32; ++w) ss += red[w];
    const float r = a.diff_mult / sqrtf(ss / (float)V + a.diff_eps);
    act_t* o = (act_t*)a.diff_out + (size_t)t * a.ldd + (size_t)hr * V;
#pragma unroll
    for (int i = 0; i < CPT; ++i) {
      const int ch = tid + i * MERGE_THREADS;
      if (ch < V) st_act(o, ch, v0[i] * r);
    }
  }
}

template <typename act_t>
static size_t chunk_smem_bytes(const b2l_seq_attn_args* a) {
  const int per = 16 / (int)sizeof(act_t), hpg = a->heads / a->kv_heads;
  const int Vp = (a->V + per - 1) / per * per;
  const int KR = a->K * (a->maps > 1 ? a->maps : 1);
  return sizeof(act_t) * ((size_t)DEC_CK * (KR + per) + (size_t)DEC_CK * Vp) + sizeof(float) * ((size_t)hpg * a->K + (size_t)hpg * DEC_CK);
}
static int chunk_count(const b2l_seq_attn_args* a) { return ((a->window > 0 ? a->window : a->block) + DEC_CK - 1) / DEC_CK; }
static bool few_queries(const b2l_seq_attn_args* a) { return a->T * a->heads < 2 * sm_count(); }
static DynSmemCache g_chunk_smem[2];

// ---- prompt portions: a CTA computes TQ queries of one head against key tiles of TK positions, SGEMM style.
// Scores: thread (ty, tx) holds queries ty + 16 i and keys tx + 8 j (4 x 4) with q and k rows read as float4 from
// padded shared memory; the 8 lanes of a ty group share their rows' maxima and sums by shuffles; the weights go
// through shared memory into the value product, where the same thread holds its 4 queries x V/8 value channels.
// All in f32 on the CUDA cores: the design wants scores and weights in 32-bit, which the tensor cores do not give.
constexpr int TQ = 64, TK = 32, TILE_THREADS = 128;

template <typename act_t>
__device__ __forceinline__ float4 ld4_act(const act_t* p);
template <>
__device__ __forceinline__ float4 ld4_act<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <>
__device__ __forceinline__ float4 ld4_act<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 w = *reinterpret_cast<const uint2*>(p);
  return make_float4(__uint_as_float(w.x << 16), __uint_as_float(w.x & 0xffff0000u), __uint_as_float(w.y << 16), __uint_as_float(w.y & 0xffff0000u));
}

__device__ __forceinline__ void att_cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void att_cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void att_cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Key and value tiles stay in their storage type in shared memory (converted when read) and arrive by cp.async, one
// tile ahead of the arithmetic: rows of K*sizeof + 16 bytes keep the 8 key rows of a ty group on distinct banks.
template <typename act_t, int VC>
__global__ void __launch_bounds__(TILE_THREADS) seq_block_attention_tile_kernel(b2l_seq_attn_args a) {
  extern __shared__ __align__(16) float smem[];
  constexpr int PER = 16 / (int)sizeof(act_t);            // elements per 16 bytes
  const int K = a.K, V = a.V, Kp = K + 4, Kpa = K + PER;    // 32 (VC - 1) < V <= 32 VC, V a multiple of 4
  float* sQ = smem;                                       // [TQ][Kp] f32
  float* sP = sQ + TQ * Kp;                               // [TQ][TK + 1]
  act_t* sKb = reinterpret_cast<act_t*>(sP + TQ * (TK + 1) + 3);   // 2 x [TK][Kpa]
  sKb = reinterpret_cast<act_t*>((reinterpret_cast<uintptr_t>(sKb)) & ~(uintptr_t)15);
  act_t* sVb = sKb + 2 * TK * Kpa;                        // 2 x [TK][V]
  const int tid = threadIdx.x, ty = tid >> 3, tx = tid & 7;
  const int h = blockIdx.y, kh = a.kv_heads * (a.maps > 1 ? a.maps : 1);
  int gk, gv;
  kv_heads_of(a, h, gk, gv);
  const int qt = gridDim.x - 1 - blockIdx.x;              // the longest tiles (last queries of a block) start first
  const int t_first = qt * TQ, nq = min(TQ, a.T - t_first);
  const int slot = a.meta[0], pos0 = a.meta[1];
  const int p_first = pos0 + t_first, p_last = p_first + nq - 1;
  const int j_begin = first_visible(a, p_first);
  const bool vlast = tx * 4 + 32 * (VC - 1) < V;          // this thread's last group of 4 value channels exists

  const act_t* kn = (const act_t*)a.k_new;
  const act_t* vn = (const act_t*)a.v_new;
  const act_t* ck = (const act_t*)a.cache_k + (size_t)slot * a.block * kh * K;
  const act_t* cv = (const act_t*)a.cache_v + (size_t)slot * a.block * a.kv_heads * V;

  auto issue_tile = [&](int jb, int buf) {
    act_t* dK = sKb + buf * TK * Kpa;
    act_t* dV = sVb + buf * TK * V;
    const int kc = K / PER, vc = V / PER;                 // 16-byte pieces per row
    for (int i = tid; i < TK * kc; i += TILE_THREADS) {
      const int r = i / kc, c = (i - r * kc) * PER, j = jb + r;
      if (j <= p_last) {
        const int e = j % a.block;
        att_cp_async16(dK + r * Kpa + c, j >= pos0 ? kn + ((size_t)(j - pos0) * kh + gk) * K + c : ck + ((size_t)e * kh + gk) * K + c);
      } else {
        *reinterpret_cast<uint4*>(dK + r * Kpa + c) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    for (int i = tid; i < TK * vc; i += TILE_THREADS) {
      const int r = i / vc, c = (i - r * vc) * PER, j = jb + r;
      if (j <= p_last) {
        const int e = j % a.block;
        att_cp_async16(dV + r * V + c, j >= pos0 ? vn + (size_t)(j - pos0) * a.ldv + (size_t)gv * V + c : cv + ((size_t)e * a.kv_heads + gv) * V + c);
      } else {
        *reinterpret_cast<uint4*>(dV + r * V + c) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    att_cp_commit();
  };

  issue_tile(j_begin, 0);
  const int K4 = K >> 2;
  for (int i = tid; i < TQ * K4; i += TILE_THREADS) {
    const int r = i / K4, c = (i - r * K4) << 2;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < nq) v = *reinterpret_cast<const float4*>(a.q + ((size_t)(t_first + r) * a.heads + h) * K + c);
    *reinterpret_cast<float4*>(sQ + r * Kp + c) = v;
  }

  float m[4], l[4], acc[4][VC][4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    m[i] = a.has_sink ? 0.f : -INFINITY;
    l[i] = a.has_sink ? 1.f : 0.f;
#pragma unroll
    for (int c = 0; c < VC; ++c) acc[i][c][0] = acc[i][c][1] = acc[i][c][2] = acc[i][c][3] = 0.f;
  }

  int buf = 0;
  for (int jb = j_begin; jb <= p_last; jb += TK, buf ^= 1) {
    if (jb + TK <= p_last) {
      issue_tile(jb + TK, buf ^ 1);
      att_cp_wait<1>();
    } else {
      att_cp_wait<0>();
    }
    __syncthreads();                   // tile jb (and, the first time, sQ) is visible to every thread
    const act_t* sK = sKb + buf * TK * Kpa;
    const act_t* sV = sVb + buf * TK * V;

    float s[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
    for (int c = 0; c < K; c += 4) {
      float4 qv[4], kv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) qv[i] = *reinterpret_cast<const float4*>(sQ + (ty + 16 * i) * Kp + c);
#pragma unroll
      for (int j = 0; j < 4; ++j) kv[j] = ld4_act<act_t>(sK + (tx + 8 * j) * Kpa + c);
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          s[i][j] = fmaf(qv[i].x, kv[j].x, s[i][j]);
          s[i][j] = fmaf(qv[i].y, kv[j].y, s[i][j]);
          s[i][j] = fmaf(qv[i].z, kv[j].z, s[i][j]);
          s[i][j] = fmaf(qv[i].w, kv[j].w, s[i][j]);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int p = p_first + ty + 16 * i;          // this row's position (rows beyond nq are never stored)
      const int c0 = first_visible(a, p);
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int key = jb + tx + 8 * j;
        float v = s[i][j] * a.scale;
        if (a.softcap > 0.f) v = a.softcap * tanhf(v / a.softcap);
        v = (key <= p && key >= c0) ? v : -INFINITY;
        s[i][j] = v;
        mx = fmaxf(mx, v);
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
      const float mn = fmaxf(m[i], mx);
      const float corr = (mn == -INFINITY) ? 1.f : expf(m[i] - mn);
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float w = (s[i][j] == -INFINITY) ? 0.f : expf(s[i][j] - mn);
        sP[(ty + 16 * i) * (TK + 1) + tx + 8 * j] = w;
        sum += w;
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      sum += __shfl_xor_sync(0xffffffffu, sum, 4);
      l[i] = l[i] * corr + sum;
      m[i] = mn;
#pragma unroll
      for (int c = 0; c < VC; ++c) {
        acc[i][c][0] *= corr; acc[i][c][1] *= corr; acc[i][c][2] *= corr; acc[i][c][3] *= corr;
      }
    }
    __syncwarp();                      // a row's weights are written and read by the 8 lanes of one ty group
    const int nk = min(TK, p_last - jb + 1);
    for (int j = 0; j < nk; ++j) {
      float w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) w[i] = sP[(ty + 16 * i) * (TK + 1) + j];
#pragma unroll
      for (int c = 0; c < VC; ++c) {
        if (c == VC - 1 && !vlast) break;
        const float4 v = ld4_act<act_t>(sV + j * V + tx * 4 + 32 * c);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          acc[i][c][0] = fmaf(w[i], v.x, acc[i][c][0]); acc[i][c][1] = fmaf(w[i], v.y, acc[i][c][1]);
          acc[i][c][2] = fmaf(w[i], v.z, acc[i][c][2]); acc[i][c][3] = fmaf(w[i], v.w, acc[i][c][3]);
        }
      }
    }
    __syncthreads();                   // this tile's buffers and sP may be overwritten
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = ty + 16 * i;
    if (r >= nq) continue;
    const int t = t_first + r;
    float f = a.out_mult / l[i];
    const act_t* gate = (const act_t*)a.gate + (size_t)t * a.ldg;
    if (a.gate && !a.gate_per_channel) f *= sigmoid_f(ld_act(gate, h));
    const size_t o = (size_t)t * a.ldo + (size_t)h * V;
#pragma unroll
    for (int c = 0; c < VC; ++c) {
      const int ch = tx * 4 + 32 * c;
      if (c == VC - 1 && !vlast) break;
      float gq[4] = {f, f, f, f};
      if (a.gate && a.gate_per_channel) {
        const float4 gv = ld4_act<act_t>(gate + (size_t)h * V + ch);      // 16-byte aligned rows of 4-channel groups: checked by the launcher
        gq[0] *= sigmoid_f(gv.x); gq[1] *= sigmoid_f(gv.y); gq[2] *= sigmoid_f(gv.z); gq[3] *= sigmoid_f(gv.w);
      }
      st_out<act_t>(a, o + ch + 0, acc[i][c][0] * gq[0]); st_out<act_t>(a, o + ch + 1, acc[i][c][1] * gq[1]);
      st_out<act_t>(a, o + ch + 2, acc[i][c][2] * gq[2]); st_out<act_t>(a, o + ch + 3, acc[i][c][3] * gq[3]);
    }
  }
}

template <typename act_t>
static size_t tile_smem_bytes(int K, int V) {
  const int per = 16 / (int)sizeof(act_t);
  return sizeof(float) * ((size_t)TQ * (K + 4) + (size_t)TQ * (TK + 1) + 4) + sizeof(act_t) * 2 * ((size_t)TK * (K + per) + (size_t)TK * V) + 16;
}

static DynSmemCache g_tile_smem[8];

template <typename act_t, int VC>
static int launch_tile(const b2l_seq_attn_args* a, cudaStream_t s, int cache_slot) {
  const size_t smem = tile_smem_bytes<act_t>(a->K, a->V);
  int rc = ensure_dyn_smem(seq_block_attention_tile_kernel<act_t, VC>, smem, g_tile_smem[cache_slot]);
  if (rc) return rc;
  dim3 grid((unsigned)((a->T + TQ - 1) / TQ), (unsigned)a->heads);
  seq_block_attention_tile_kernel<act_t, VC><<<grid, TILE_THREADS, smem, s>>>(*a);
  return 0;
}

// ring[p % block] <- token p for the portion's tokens in the block of its last token (block-local) or for its last
// `block` tokens (sliding window).
template <typename act_t>
__global__ void seq_ring_append_kernel(b2l_seq_attn_args a) {
  const int slot = a.meta[0], pos0 = a.meta[1];
  const int last = pos0 + a.T - 1;
  const int first = max(pos0, a.window > 0 ? last - a.block + 1 : (last / a.block) * a.block);
  const int p = first + blockIdx.x;
  if (p > last) return;
  const int t = p - pos0, e = p % a.block;
  const int nk = a.kv_heads * (a.maps > 1 ? a.maps : 1) * a.K, nv = a.kv_heads * a.V;
  const act_t* kn = (const act_t*)a.k_new + (size_t)t * nk;
  const act_t* vn = (const act_t*)a.v_new + (size_t)t * a.ldv;
  act_t* ck = (act_t*)a.cache_k + ((size_t)slot * a.block + e) * nk;
  act_t* cv = (act_t*)a.cache_v + ((size_t)slot * a.block + e) * nv;
  for (int i = threadIdx.x; i < nk; i += blockDim.x) ck[i] = kn[i];
  for (int i = threadIdx.x; i < nv; i += blockDim.x) cv[i] = vn[i];
}

// Differential read-out: one warp per (token, head): o = a0 - lambda a1, divided by its root mean square, times mult.
template <typename act_t>
__global__ void seq_diff_combine_kernel(const float* __restrict__ a, int lda, float lambda, float eps, float mult, act_t* __restrict__ out,
                                        int ldo, int n_rows, int heads, int V) {
  const int id = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (id >= n_rows * heads) return;
  const int t = id / heads, h = id - t * heads;
  const float* p = a + (size_t)t * lda + (size_t)h * 2 * V;
  float o[ATT_VMAX], ss = 0.f;
#pragma unroll
  for (int c = 0; c < ATT_VMAX; ++c) {
    const int ch = c * 32 + lane;
    o[c] = ch < V ? p[ch] - lambda * p[V + ch] : 0.f;
    ss += o[c] * o[c];
  }
  ss = warp_sum(ss);
  const float r = mult / sqrtf(ss / (float)V + eps);
  act_t* q = out + (size_t)t * ldo + (size_t)h * V;
#pragma unroll
  for (int c = 0; c < ATT_VMAX; ++c) {
    const int ch = c * 32 + lane;
    if (ch < V) st_act(q, ch, o[c] * r);
  }
}

}  // namespace b2l

using namespace b2l;

extern "C" int b2l_seq_diff_combine(const float* a, int lda, float lambda, float eps, float mult, void* out, int ldo, int T, int heads, int V,
                                    int act_dtype, b2l_stream_t stream) {
  B2L_CHECK_ARG(a && out, "b2l_seq_diff_combine: null pointer");
  B2L_CHECK_ARG(T >= 0 && heads > 0 && V > 0 && lda >= heads * 2 * V && ldo >= heads * V, "b2l_seq_diff_combine: bad size");
  B2L_CHECK_SUPPORTED(V <= ATT_VMAX * 32, "b2l_seq_diff_combine: value size %d above %d", V, ATT_VMAX * 32);
  if (T == 0) return 0;
  const int ids = T * heads;
  B2L_SEQ_DISPATCH(act_dtype, (seq_diff_combine_kernel<act_t><<<(ids + 3) / 4, 128, 0, (cudaStream_t)stream>>>(a, lda, lambda, eps, mult, (act_t*)out, ldo, T, heads, V)));
  B2L_LAUNCH_CHECK("seq_diff_combine_kernel");
  return 0;
}

extern "C" int b2l_seq_block_attention(const b2l_seq_attn_args* a, b2l_stream_t stream) {
  B2L_CHECK_ARG(a != nullptr, "b2l_seq_block_attention: null argument block");
  B2L_CHECK_ARG(a->q && a->k_new && a->v_new && a->cache_k && a->cache_v && a->meta && a->out, "b2l_seq_block_attention: null pointer");
  B2L_CHECK_ARG(a->T >= 0 && a->heads > 0 && a->kv_heads > 0 && a->K > 0 && a->V > 0 && a->block > 0, "b2l_seq_block_attention: bad size");
  B2L_CHECK_ARG(a->maps >= 0 && a->heads % (a->kv_heads * (a->maps > 1 ? a->maps : 1)) == 0,
                "b2l_seq_block_attention: heads %d not a multiple of kv_heads %d times maps %d", a->heads, a->kv_heads, a->maps);
  B2L_CHECK_ARG(!(a->gate && a->out_f32), "b2l_seq_block_attention: a gated output is stored in the activation type");
  B2L_CHECK_ARG(a->diff_out == nullptr || (a->maps == 2 && a->out_f32 && !a->gate && a->ldd >= a->heads / 2 * a->V && a->ldo >= a->heads * a->V),
                "b2l_seq_block_attention: the differential read-out wants two maps per head, f32 maps in `out` and no gate");
  B2L_CHECK_ARG(a->window >= 0 && (a->window == 0 || a->block >= a->window), "b2l_seq_block_attention: a ring of %d positions cannot serve a window of %d",
                a->block, a->window);
  B2L_CHECK_SUPPORTED(a->V <= ATT_VMAX * 32, "b2l_seq_block_attention: value size %d above %d", a->V, ATT_VMAX * 32);
  B2L_CHECK_ARG(a->act_dtype == B2L_BF16 || a->act_dtype == B2L_F32, "b2l_seq_block_attention: act_dtype %d unsupported", a->act_dtype);
  if (a->T == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const size_t esz = a->act_dtype == B2L_BF16 ? 2 : 4;
  const int vec = ((a->K * esz) % 16 == 0) && (((uintptr_t)a->k_new | (uintptr_t)a->cache_k) % 16 == 0) && (a->K % 8 == 0 || esz == 4);
  const int pairs = a->T * a->heads;
  const int Kpad = (a->K + 3) & ~3;
  const bool split = few_queries(a);                  // few queries (decoding)
  const size_t chunk_smem = a->act_dtype == B2L_BF16 ? chunk_smem_bytes<__nv_bfloat16>(a) : chunk_smem_bytes<float>(a);
  if (split && a->work != nullptr && chunk_smem <= 200 * 1024 && chunk_count(a) <= 8192) {     // chunks of keys in parallel, then a merge
    const int n_chunks = chunk_count(a);
    B2L_CHECK_ARG((size_t)a->work_floats >= (size_t)pairs * n_chunks * (a->V + 2), "b2l_seq_block_attention: work space of %d floats, %zu needed",
                  a->work_floats, (size_t)pairs * n_chunks * (a->V + 2));
    const int per = 16 / (int)esz;
    const int vec16 = (a->K % per == 0 && a->V % per == 0 && a->ldv % per == 0 &&
                       (((uintptr_t)a->k_new | (uintptr_t)a->v_new | (uintptr_t)a->cache_k | (uintptr_t)a->cache_v | (uintptr_t)a->q) % 16) == 0) ? 1 : 0;
    dim3 grid((unsigned)n_chunks, (unsigned)a->kv_heads, (unsigned)a->T);
    if (a->act_dtype == B2L_BF16) {
      int rc = ensure_dyn_smem(seq_attention_chunk_kernel<__nv_bfloat16>, chunk_smem, g_chunk_smem[0]);
      if (rc) return rc;
      seq_attention_chunk_kernel<__nv_bfloat16><<<grid, DEC_THREADS, chunk_smem, s>>>(*a, n_chunks, vec16);
      if (a->diff_out) seq_attention_merge_kernel<__nv_bfloat16, true><<<pairs / 2, MERGE_THREADS, sizeof(float) * n_chunks, s>>>(*a, n_chunks);
      else seq_attention_merge_kernel<__nv_bfloat16, false><<<pairs, MERGE_THREADS, sizeof(float) * n_chunks, s>>>(*a, n_chunks);
    } else {
      int rc = ensure_dyn_smem(seq_attention_chunk_kernel<float>, chunk_smem, g_chunk_smem[1]);
      if (rc) return rc;
      seq_attention_chunk_kernel<float><<<grid, DEC_THREADS, chunk_smem, s>>>(*a, n_chunks, vec16);
      if (a->diff_out) seq_attention_merge_kernel<float, true><<<pairs / 2, MERGE_THREADS, sizeof(float) * n_chunks, s>>>(*a, n_chunks);
      else seq_attention_merge_kernel<float, false><<<pairs, MERGE_THREADS, sizeof(float) * n_chunks, s>>>(*a, n_chunks);
    }
    B2L_LAUNCH_CHECK("seq_attention_chunk_kernel");
    if (a->T == 1 || a->no_append) return 0;        // a single token was appended by its first chunk
    const int n_app0 = std::min(a->T, a->block);
    if (a->act_dtype == B2L_BF16) seq_ring_append_kernel<__nv_bfloat16><<<n_app0, 128, 0, s>>>(*a);
    else seq_ring_append_kernel<float><<<n_app0, 128, 0, s>>>(*a);
    B2L_LAUNCH_CHECK("seq_ring_append_kernel");
    return 0;
  }
  const size_t smem = sizeof(float) * ((size_t)(split ? 1 : 4) * Kpad + (split ? 16 : 4) * (2 + ATT_VMAX * 32));
  B2L_CHECK_SUPPORTED(smem <= 48 * 1024, "b2l_seq_block_attention: key size %d too large", a->K);
  const bool al = (((uintptr_t)a->q | (uintptr_t)a->k_new | (uintptr_t)a->v_new | (uintptr_t)a->cache_k | (uintptr_t)a->cache_v) % 16) == 0;
  const size_t tile_smem = a->act_dtype == B2L_BF16 ? tile_smem_bytes<__nv_bfloat16>(a->K, a->V) : tile_smem_bytes<float>(a->K, a->V);
  const bool gate_ok = !(a->gate && a->gate_per_channel) || (((uintptr_t)a->gate % 16) == 0 && (a->ldg * esz) % 16 == 0);
  const bool tile = !split && a->T >= 16 && al && (a->K * esz) % 16 == 0 && (a->V * esz) % 16 == 0 && a->V % 4 == 0 && a->V <= 128 &&
                    (a->ldv * esz) % 16 == 0 && gate_ok && tile_smem <= 200 * 1024;
  if (tile) {
    const int vc = (a->V + 31) / 32;
    int rc = 0;
    if (a->act_dtype == B2L_BF16)
      rc = vc == 1 ? launch_tile<__nv_bfloat16, 1>(a, s, 0) : vc == 2 ? launch_tile<__nv_bfloat16, 2>(a, s, 1)
         : vc == 3 ? launch_tile<__nv_bfloat16, 3>(a, s, 2) : launch_tile<__nv_bfloat16, 4>(a, s, 3);
    else
      rc = vc == 1 ? launch_tile<float, 1>(a, s, 4) : vc == 2 ? launch_tile<float, 2>(a, s, 5)
         : vc == 3 ? launch_tile<float, 3>(a, s, 6) : launch_tile<float, 4>(a, s, 7);
    if (rc) return rc;
  } else if (a->act_dtype == B2L_BF16) {
    if (split) seq_block_attention_kernel<__nv_bfloat16, 16><<<pairs, 512, smem, s>>>(*a, vec);
    else seq_block_attention_kernel<__nv_bfloat16, 1><<<(pairs + 3) / 4, 128, smem, s>>>(*a, vec);
  } else {
    if (split) seq_block_attention_kernel<float, 16><<<pairs, 512, smem, s>>>(*a, vec);
    else seq_block_attention_kernel<float, 1><<<(pairs + 3) / 4, 128, smem, s>>>(*a, vec);
  }
  B2L_LAUNCH_CHECK("seq_block_attention_kernel");
  if (a->diff_out) {                                  // the read-out of the two maps, from the f32 maps in `out`
    const int ids = a->T * (a->heads / 2);
    B2L_SEQ_DISPATCH(a->act_dtype, (seq_diff_combine_kernel<act_t><<<(ids + 3) / 4, 128, 0, s>>>((const float*)a->out, a->ldo, a->diff_lambda, a->diff_eps, a->diff_mult,
                                                                                                   (act_t*)a->diff_out, a->ldd, a->T, a->heads / 2, a->V)));
    B2L_LAUNCH_CHECK("seq_diff_combine_kernel");
  }
  if (a->no_append) return 0;
  const int n_app = std::min(a->T, a->block);
  if (a->act_dtype == B2L_BF16) seq_ring_append_kernel<__nv_bfloat16><<<n_app, 128, 0, s>>>(*a);
  else seq_ring_append_kernel<float><<<n_app, 128, 0, s>>>(*a);
  B2L_LAUNCH_CHECK("seq_ring_append_kernel");
  return 0;
}

extern "C" long long b2l_seq_block_attention_work_floats(const b2l_seq_attn_args* a) {
  if (a == nullptr || a->T <= 0 || a->heads <= 0 || a->kv_heads <= 0 || a->V <= 0 || a->block <= 0) return 0;
  if (!few_queries(a)) return 0;
  return (long long)a->T * a->heads * chunk_count(a) * (a->V + 2);
}
