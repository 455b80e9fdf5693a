// Attention over a paged cache of latents: every position keeps one vector [c ; kr] of
// C + R numbers shared by all heads, c a normalised low-rank latent from which keys and values
// would be projected, kr a rotated key part.  The query side absorbs the key projection
// (q_lat = W_uk^T q), so a head's score is (q_lat . c + q_rot . kr) * scale and its output the
// weighted sum of the latents themselves, projected to values afterwards.  Options: a sliding
// window (query at p sees p - window < j <= p) and a learned sink per head, a number that joins
// the softmax's denominator as exp(sink) with no key, no value and no scaling.
//
// Kernels: the preparation of a step's rows (two RMS norms with plain weights, the rotation of
// the shared key part, by halves or by neighbouring pairs, the write into the page slots), the rotation of the queries' rotated
// parts, and the attention itself.  Scores, softmax weights, angles and norms are 32-bit;
// T says how the cache and the outputs that feed matrix products are stored.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kKeys = 32;   // keys per tile, aligned to absolute positions: the sum's order does not depend on the cut

// ---- rows of a step: query latent, cached latent, rotated shared key ---------------------------
// proj [tokens, ld] floats: [0, Q) the query's low-rank projection, [Q, Q + C) the latent's,
// [Q + C, Q + C + R) the shared key part.  cq (T) = rmsnorm(first) * wq; the cache row of the
// token's slot = [rmsnorm(second) * wc ; rotate(third)].
template <typename T>
__global__ void __launch_bounds__(kThreads) latent_prep_kernel(T* __restrict__ cq, T* __restrict__ cache,
                                                               const float* __restrict__ proj, int ld, int Q, int C,
                                                               int R, const T* __restrict__ wq, const T* __restrict__ wc,
                                                               const int* __restrict__ positions,
                                                               const float* __restrict__ inv_freq, int rot_dims,
                                                               const int* __restrict__ slots, long long n_slots,
                                                               float eps, int pairs) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const float* row = proj + (size_t)t * ld;
  float sq = 0.f, sc = 0.f;
  for (int i = threadIdx.x; i < Q; i += kThreads) sq += row[i] * row[i];
  for (int i = threadIdx.x; i < C; i += kThreads) sc += row[Q + i] * row[Q + i];
  sq = block_sum(sq, scratch);
  sc = block_sum(sc, scratch);
  const float iq = Q > 0 ? 1.0f / sqrtf(sq / (float)Q + eps) : 0.f, ic = 1.0f / sqrtf(sc / (float)C + eps);
  for (int i = threadIdx.x; i < Q; i += kThreads) cq[(size_t)t * Q + i] = from_f32<T>(row[i] * iq * to_f32(wq[i]));
  if (cache == nullptr) return;
  const long long slot = slots[t];
  if (slot == -1) return;      // a row of padding: its latent goes nowhere
  if (slot < 0 || slot >= n_slots) {
    if (threadIdx.x == 0) lab_set_error(LAB_ERR_PAGE_RANGE);
    return;
  }
  T* dst = cache + (size_t)slot * (C + R);
  for (int i = threadIdx.x; i < C; i += kThreads) dst[i] = from_f32<T>(row[Q + i] * ic * to_f32(wc[i]));
  const float pos = (float)positions[t];
  const int half = rot_dims / 2;
  const float* kr = row + Q + C;
  for (int i = threadIdx.x; i < R; i += kThreads) {
    float v = kr[i];
    if (i < rot_dims) {
      // entry f of the frequencies turns the pair (f, f + half), or with `pairs` the neighbours (2f, 2f + 1)
      const int f = pairs ? i >> 1 : (i < half ? i : i - half);
      const bool first = pairs ? !(i & 1) : i < half;
      const float ang = pos * inv_freq[f];
      const float cs = cosf(ang), sn = sinf(ang);
      float lo, hi;
      rope_rotate(kr[pairs ? 2 * f : f], kr[pairs ? 2 * f + 1 : f + half], cs, sn, lo, hi);
      v = first ? lo : hi;
    }
    dst[C + i] = from_f32<T>(v);
  }
}

// ---- the queries' rotated parts ---------------------------------------------------------------
// q (T) [tokens, heads, q_head] (a head: D plain entries, R to rotate, then padding) -> q_cat (float)
// [tokens, heads, C + R]: columns [C, C + R) get the rotated R entries of each head (the first C columns
// are the absorbed product's).  With `in_place`, the rotated entries also replace the stored ones in q
// (rounded to T), for kernels that read q itself; q_cat may then be null.
template <typename T>
__global__ void __launch_bounds__(kThreads) latent_q_rope_kernel(float* __restrict__ q_cat, T* __restrict__ q,
                                                                 int heads, int D, int R, int C, int q_head,
                                                                 const int* __restrict__ positions,
                                                                 const float* __restrict__ inv_freq, int rot_dims,
                                                                 int in_place, int pairs) {
  extern __shared__ float rotated[];      // [heads * R]
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const float pos = (float)positions[t];
  const int half = rot_dims / 2;
  for (int idx = threadIdx.x; idx < heads * R; idx += kThreads) {
    const int h = idx / R, i = idx % R;
    const T* src = q + ((size_t)t * heads + h) * q_head + D;
    float v = to_f32(src[i]);
    if (i < rot_dims) {
      const int f = pairs ? i >> 1 : (i < half ? i : i - half);
      const bool first = pairs ? !(i & 1) : i < half;
      const float ang = pos * inv_freq[f];
      const float cs = cosf(ang), sn = sinf(ang);
      float lo, hi;
      rope_rotate(to_f32(src[pairs ? 2 * f : f]), to_f32(src[pairs ? 2 * f + 1 : f + half]), cs, sn, lo, hi);
      v = first ? lo : hi;
    }
    if (q_cat != nullptr) q_cat[((size_t)t * heads + h) * (C + R) + C + i] = v;
    rotated[idx] = v;
  }
  if (!in_place) return;
  __syncthreads();       // every pair has been read before any of it is replaced
  for (int idx = threadIdx.x; idx < heads * R; idx += kThreads)
    q[((size_t)t * heads + idx / R) * q_head + D + idx % R] = from_f32<T>(rotated[idx]);
}

// ---- keys and values for the tensor-core attention of prompts' portions ------------------------
// Requests that bring many tokens attend in the plain form: keys [W_uk c ; kr] and values W_uv c per head,
// projected up for the step from the latents the rows can see, into scratch pools that have the cache's own
// page numbering (so the kernel walks the step's block table as it is).
// `meta` [selected requests][4]: request index in the step, first key position, number of keys, first row
// in the compact list.  Gather: compact row i <- the latent c of its key, and slot_of[i] <- its cache slot.
template <typename T>
__global__ void __launch_bounds__(128) latent_gather_kernel(T* __restrict__ compact, int* __restrict__ slot_of,
                                                            const T* __restrict__ cache, const int* __restrict__ meta,
                                                            const int* __restrict__ block_table, int bt_width, int C,
                                                            int W, int page_size, int num_pages) {
  pdl_trigger();
  pdl_wait();
  const int* mt = meta + 4 * blockIdx.y;
  const int req = mt[0], lo = mt[1], count = mt[2], base = mt[3];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kk = blockIdx.x * 4 + warp;
  if (kk >= count) return;
  const int pos = lo + kk;
  const int page = block_table[(size_t)req * bt_width + pos / page_size];
  if (page < 0 || page >= num_pages) {
    if (lane == 0) lab_set_error(LAB_ERR_PAGE_RANGE);
    return;
  }
  const int slot = page * page_size + pos % page_size;
  if (lane == 0) slot_of[base + kk] = slot;
  const T* src = cache + (size_t)slot * W;
  T* dst = compact + (size_t)(base + kk) * C;
  for (int c = lane; c < C; c += 32) dst[c] = src[c];
}

// Scatter: projected [rows, heads * D + heads * V] (keys' plain parts, then values) and the cached
// rotated part -> k_pool, v_pool [pages, heads, page_size, HD]: k = [plain ; kr ; 0], v = [value ; 0].
template <typename T>
__global__ void __launch_bounds__(kThreads) latent_scatter_kernel(T* __restrict__ k_pool, T* __restrict__ v_pool,
                                                                  const T* __restrict__ projected,
                                                                  const int* __restrict__ slot_of,
                                                                  const T* __restrict__ cache, int heads, int D, int R,
                                                                  int V, int C, int HD, int page_size) {
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x;
  const int slot = slot_of[i];
  const int page = slot / page_size, off = slot % page_size;
  const T* row = projected + (size_t)i * heads * (D + V);
  const T* kr = cache + (size_t)slot * (C + R) + C;
  for (int idx = threadIdx.x; idx < heads * HD; idx += kThreads) {
    const int h = idx / HD, c = idx % HD;
    const size_t at = (((size_t)page * heads + h) * page_size + off) * HD + c;
    k_pool[at] = c < D ? row[h * D + c] : (c < D + R ? kr[c - D] : from_f32<T>(0.f));
    v_pool[at] = c < V ? row[heads * D + h * V + c] : from_f32<T>(0.f);
  }
}

__device__ __forceinline__ float2 load_pair(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 load_pair(const __nv_bfloat16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}

// ---- attention ------------------------------------------------------------------------------------
// One CTA takes up to QT consecutive rows of one request with HG of its heads (all of them where
// shared memory allows): the tiles of keys it stages in shared memory serve every (row, head) pair.  A warp owns pairs; a lane owns a key of
// the tile for the scores and columns of the output for the weighted sum.  Running maximum, sum
// and output of a pair live in shared memory; the sink opens them (maximum = sink, sum = 1).
struct LatentParams {
  void* out;              // [tokens, heads * C] of T
  const float* q;         // [tokens, heads, C + R]
  const void* cache;      // [pages * page_size, C + R] of T
  const float* sink;      // [heads] or null
  const int* q_start;
  const int* pos0;
  const int* kv_len;      // a request that holds nothing (padding of a padded batch) gets zeros
  const int* block_table;
  int bt_width, heads, C, W, page_size, num_pages, window, QT, HG;
  int below;              // > 0: only requests that bring fewer rows than this (others are served elsewhere)
  int splits;             // > 1 (steps of single tokens only): blockIdx.x takes a share of the keys' tiles and
  float* part;            // leaves (maximum, sum, unnormalised output) here for the merge kernel
  float scale;
};

template <typename T>
__global__ void __launch_bounds__(kThreads) latent_attention_kernel(LatentParams p) {
  extern __shared__ float smem[];
  pdl_trigger();
  pdl_wait();
  const int req = blockIdx.y;
  const int split = p.splits > 1 ? blockIdx.x : 0, row_block = p.splits > 1 ? 0 : blockIdx.x;
  const int first = p.q_start[req] + row_block * p.QT;
  const int n = min(p.QT, p.q_start[req + 1] - first);
  if (n <= 0 || (p.below > 0 && p.q_start[req + 1] - p.q_start[req] >= p.below)) return;
  const int C = p.C, W = p.W, KW = W + 1;
  const int h0 = blockIdx.z * p.HG, H = min(p.HG, p.heads - h0);     // this CTA's heads: h0 .. h0 + H - 1
  const int pairs = n * H;
  if (p.kv_len[req] <= 0) {
    if (p.splits > 1) {
      // shares of nothing: the merge kernel writes the zeros
      for (int i = threadIdx.x; i < pairs * (C + 2); i += kThreads) {
        const int pair = i / (C + 2), c = i % (C + 2);
        p.part[(((size_t)req * p.heads + h0 + pair) * p.splits + split) * (C + 2) + c] = c == 0 ? -INFINITY : 0.f;
      }
    } else {
      T* zero = (T*)p.out;
      for (int i = threadIdx.x; i < pairs * C; i += kThreads)
        zero[((size_t)(first + (i / C) / H) * p.heads + h0 + (i / C) % H) * C + i % C] = from_f32<T>(0.f);
    }
    return;
  }
  float* qs = smem;                                  // [QT * HG][W]
  float* keys = qs + (size_t)p.QT * p.HG * W;        // [kKeys][W + 1]
  float* acc = keys + kKeys * KW;                    // [QT * HG][C]
  float* run_m = acc + (size_t)p.QT * p.HG * C;      // [QT * HG]
  float* run_l = run_m + p.QT * p.HG;
  float* probs = run_l + p.QT * p.HG;                // [kWarps][kKeys]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const T* cache = (const T*)p.cache;

  const int p_first = p.pos0[req] + row_block * p.QT, p_last = p_first + n - 1;
  const int lo = p.window > 0 ? max(0, p_first - p.window + 1) : 0;
  for (int i = tid; i < pairs * W; i += kThreads) {
    const int pair = i / W, c = i % W;
    qs[i] = p.q[((size_t)(first + pair / H) * p.heads + h0 + pair % H) * W + c];
  }
  for (int i = tid; i < pairs * C; i += kThreads) acc[i] = 0.f;
  const bool with_sink = p.sink != nullptr && split == 0;      // the sink joins one share of the keys only
  for (int i = tid; i < pairs; i += kThreads) {
    run_m[i] = with_sink ? p.sink[h0 + i % H] : -INFINITY;
    run_l[i] = with_sink ? 1.f : 0.f;
  }
  const int* table = p.block_table + (size_t)req * p.bt_width;

  int tile_lo = lo / kKeys, tile_hi = p_last / kKeys;
  if (p.splits > 1) {
    const int per = (tile_hi - tile_lo + p.splits) / p.splits;
    tile_lo += split * per;
    tile_hi = min(tile_hi, tile_lo + per - 1);
  }
  constexpr int kPerWarp = kKeys / kWarps;      // keys of a tile each warp brings in
  for (int tile = tile_lo; tile <= tile_hi; ++tile) {
    __syncthreads();       // the previous tile's readers are done (and the set-up above is visible)
    const T* src[kPerWarp];
#pragma unroll
    for (int e = 0; e < kPerWarp; ++e) {
      const int pos = tile * kKeys + warp * kPerWarp + e;
      src[e] = nullptr;
      if (pos >= lo && pos <= p_last) {
        const int page = table[pos / p.page_size];
        if (page < 0 || page >= p.num_pages) {
          if (lane == 0) lab_set_error(LAB_ERR_PAGE_RANGE);
        } else {
          src[e] = cache + ((size_t)page * p.page_size + pos % p.page_size) * W;
        }
      }
    }
    if ((W & 1) == 0) {
      // two entries a load, the loads of a warp's keys in flight together
      for (int c = 2 * lane; c < W; c += 64) {
        float2 v[kPerWarp];
#pragma unroll
        for (int e = 0; e < kPerWarp; ++e) v[e] = src[e] != nullptr ? load_pair(src[e] + c) : make_float2(0.f, 0.f);
#pragma unroll
        for (int e = 0; e < kPerWarp; ++e) {
          keys[(warp * kPerWarp + e) * KW + c] = v[e].x;
          keys[(warp * kPerWarp + e) * KW + c + 1] = v[e].y;
        }
      }
    } else {
      for (int c = lane; c < W; c += 32)
#pragma unroll
        for (int e = 0; e < kPerWarp; ++e)
          keys[(warp * kPerWarp + e) * KW + c] = src[e] != nullptr ? to_f32(src[e][c]) : 0.f;
    }
    __syncthreads();
    for (int pair = warp; pair < pairs; pair += kWarps) {
      const int qpos = p_first + pair / H;
      const int kpos = tile * kKeys + lane;
      const bool seen = kpos <= qpos && kpos >= lo && (p.window <= 0 || qpos - kpos < p.window);
      float s = -INFINITY;
      if (seen) {
        const float* qv = qs + (size_t)pair * W;
        const float* kv = keys + lane * KW;
        float dot = 0.f;
        for (int c = 0; c < W; ++c) dot = fmaf(qv[c], kv[c], dot);
        s = dot * p.scale;
      }
      const float tile_max = warp_max(s);
      if (tile_max == -INFINITY) continue;           // the whole tile lies outside this row's reach
      const float m_old = run_m[pair];
      const float m_new = fmaxf(m_old, tile_max);
      const float corr = expf(m_old - m_new);        // m_old = -inf only without a sink: then 0
      const float pj = seen ? expf(s - m_new) : 0.f;
      const float sum = warp_sum(pj);
      __syncwarp();
      probs[warp * kKeys + lane] = pj;
      if (lane == 0) {
        run_m[pair] = m_new;
        run_l[pair] = run_l[pair] * corr + sum;
      }
      __syncwarp();
      const float* pw = probs + warp * kKeys;
      for (int c = lane; c < C; c += 32) {
        float a = acc[(size_t)pair * C + c] * corr;
#pragma unroll 8
        for (int jk = 0; jk < kKeys; ++jk) a = fmaf(pw[jk], keys[jk * KW + c], a);
        acc[(size_t)pair * C + c] = a;
      }
    }
  }
  __syncthreads();
  if (p.splits > 1) {
    // one row per request here: pair = head.  [request][head][split][maximum, sum, output[C]]
    for (int i = tid; i < pairs * (C + 2); i += kThreads) {
      const int pair = i / (C + 2), c = i % (C + 2);
      float* dst = p.part + (((size_t)req * p.heads + h0 + pair) * p.splits + split) * (C + 2);
      dst[c] = c == 0 ? run_m[pair] : (c == 1 ? run_l[pair] : acc[(size_t)pair * C + c - 2]);
    }
    return;
  }
  T* out = (T*)p.out;
  for (int i = tid; i < pairs * C; i += kThreads) {
    const int pair = i / C, c = i % C;
    out[((size_t)(first + pair / H) * p.heads + h0 + pair % H) * C + c] = from_f32<T>(acc[i] / run_l[pair]);
  }
}

// The shares of a single-token request's keys, merged in ascending order of the shares.
template <typename T>
__global__ void __launch_bounds__(128) latent_merge_kernel(T* __restrict__ out, const float* __restrict__ part,
                                                           const int* __restrict__ q_start, int heads, int C,
                                                           int splits, int below) {
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.x, req = blockIdx.y;
  const int rows = q_start[req + 1] - q_start[req];
  if (rows <= 0 || (below > 0 && rows >= below)) return;
  const float* mine = part + ((size_t)req * heads + h) * splits * (C + 2);
  // every share's weight once, in shared memory (a loop of dependent loads costs a latency per share)
  __shared__ float weight[64];
  if (threadIdx.x < 64) {
    const float m = threadIdx.x < splits ? mine[(size_t)threadIdx.x * (C + 2)] : -INFINITY;
    float big = m;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) big = fmaxf(big, __shfl_xor_sync(0xffffffffu, big, o));
    weight[threadIdx.x] = big;      // the warp's maximum for now
  }
  __syncthreads();
  const float big = fmaxf(weight[0], weight[32]);
  __syncthreads();
  if (threadIdx.x < 64) {
    const float m = threadIdx.x < splits ? mine[(size_t)threadIdx.x * (C + 2)] : -INFINITY;
    weight[threadIdx.x] = m == -INFINITY ? 0.f : expf(m - big);
  }
  __syncthreads();
  float total = 0.f;
  for (int s = 0; s < splits; ++s) total += weight[s] * mine[(size_t)s * (C + 2) + 1];
  for (int c = threadIdx.x; c < C; c += 128) {
    float a = 0.f;
    for (int s0 = 0; s0 < splits; s0 += 8) {
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = s0 + j < splits ? mine[(size_t)(s0 + j) * (C + 2) + 2 + c] : 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) a = fmaf(s0 + j < splits ? weight[s0 + j] : 0.f, v[j], a);
    }
    out[((size_t)q_start[req] * heads + h) * C + c] = from_f32<T>(total > 0.f ? a / total : 0.f);
  }
}

size_t attention_smem(int QT, int H, int C, int W) {
  return sizeof(float) * ((size_t)QT * H * W + (size_t)kKeys * (W + 1) + (size_t)QT * H * C + 2 * (size_t)QT * H +
                          kWarps * kKeys);
}

// Rows and heads one CTA takes: all heads and up to 8 rows while that fits 96 KB of shared memory (two
// CTAs an SM); a step of single tokens takes a warp's worth of heads per CTA, so that more CTAs share the
// keys' stream; heads are halved further while a CTA's share exceeds 200 KB.
bool attention_shape(int heads, int C, int W, int max_q, int* qt_out, int* hg_out) {
  int hg = max_q <= 1 ? (heads < kWarps ? heads : kWarps) : heads;
  int qt = 8;
  while (qt > 1 && (attention_smem(qt, hg, C, W) > 96 * 1024 || qt / 2 >= max_q)) qt /= 2;
  while (hg > 1 && attention_smem(qt, hg, C, W) > 200 * 1024) hg = (hg + 1) / 2;
  if (attention_smem(qt, hg, C, W) > 200 * 1024) return false;
  *qt_out = qt;
  *hg_out = hg;
  return true;
}

}  // namespace

LAB_EXPORT int lab_latent_prep(void* cq, void* cache, const float* proj, int ld, int Q, int C, int R, const void* wq,
                               const void* wc, const int* positions, const float* inv_freq, int rot_dims,
                               const int* slots, long long n_slots, int tokens, float eps, int pairs, int dtype,
                               cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (dtype == LAB_F32)
    lab_launch(latent_prep_kernel<float>, dim3(tokens), dim3(kThreads), 0, stream, (float*)cq, (float*)cache, proj, ld,
               Q, C, R, (const float*)wq, (const float*)wc, positions, inv_freq, rot_dims, slots, n_slots, eps, pairs);
  else
    lab_launch(latent_prep_kernel<__nv_bfloat16>, dim3(tokens), dim3(kThreads), 0, stream, (__nv_bfloat16*)cq,
               (__nv_bfloat16*)cache, proj, ld, Q, C, R, (const __nv_bfloat16*)wq, (const __nv_bfloat16*)wc, positions,
               inv_freq, rot_dims, slots, n_slots, eps, pairs);
  LAB_LAUNCH_CHECK();
}

LAB_EXPORT int lab_latent_q_rope(float* q_cat, void* q, int tokens, int heads, int D, int R, int C, int q_head,
                                 const int* positions, const float* inv_freq, int rot_dims, int in_place, int pairs,
                                 int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  const size_t smem = sizeof(float) * (size_t)heads * R;
  if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
  if (dtype == LAB_F32)
    lab_launch(latent_q_rope_kernel<float>, dim3(tokens), dim3(kThreads), smem, stream, q_cat, (float*)q, heads, D, R, C,
               q_head, positions, inv_freq, rot_dims, in_place, pairs);
  else
    lab_launch(latent_q_rope_kernel<__nv_bfloat16>, dim3(tokens), dim3(kThreads), smem, stream, q_cat,
               (__nv_bfloat16*)q, heads, D, R, C, q_head, positions, inv_freq, rot_dims, in_place, pairs);
  LAB_LAUNCH_CHECK();
}

// bfloat16 only: the tensor-core attention these feed takes nothing else.
LAB_EXPORT int lab_latent_gather(void* compact, int* slot_of, const void* cache, const int* meta, int n_selected,
                                 int max_count, const int* block_table, int bt_width, int C, int W, int page_size,
                                 int num_pages, cudaStream_t stream) {
  if (n_selected <= 0 || max_count <= 0) return 0;
  lab_launch(latent_gather_kernel<__nv_bfloat16>, dim3((max_count + 3) / 4, n_selected), dim3(128), 0, stream,
             (__nv_bfloat16*)compact, slot_of, (const __nv_bfloat16*)cache, meta, block_table, bt_width, C, W,
             page_size, num_pages);
  LAB_LAUNCH_CHECK();
}

LAB_EXPORT int lab_latent_scatter(void* k_pool, void* v_pool, const void* projected, const int* slot_of,
                                  const void* cache, int rows, int heads, int D, int R, int V, int C, int HD,
                                  int page_size, cudaStream_t stream) {
  if (rows <= 0) return 0;
  lab_launch(latent_scatter_kernel<__nv_bfloat16>, dim3(rows), dim3(kThreads), 0, stream, (__nv_bfloat16*)k_pool,
             (__nv_bfloat16*)v_pool, (const __nv_bfloat16*)projected, slot_of, (const __nv_bfloat16*)cache, heads, D, R,
             V, C, HD, page_size);
  LAB_LAUNCH_CHECK();
}

// Rows of a request that one CTA takes (0: a single head's row does not fit shared memory).
LAB_EXPORT int lab_latent_attention_rows(int heads, int C, int W, int max_q) {
  int qt = 0, hg = 0;
  return attention_shape(heads, C, W, max_q, &qt, &hg) ? qt : 0;
}

LAB_EXPORT int lab_latent_attention(void* out, const float* q, const void* cache, const float* sink,
                                    const int* q_start, const int* pos0, const int* kv_len, const int* block_table,
                                    int bt_width,
                                    int n_requests, int max_q, int heads, int C, int W, int page_size, int num_pages,
                                    int window, float scale, int below, int splits, float* part, int dtype,
                                    cudaStream_t stream) {
  if (n_requests <= 0 || max_q <= 0) return 0;
  if (splits > 1 && (max_q != 1 || part == nullptr)) return (int)cudaErrorInvalidValue;
  LatentParams p;
  p.below = below;
  p.splits = splits < 1 ? 1 : splits;
  p.part = part;
  p.out = out; p.q = q; p.cache = cache; p.sink = sink; p.q_start = q_start; p.pos0 = pos0; p.kv_len = kv_len;
  p.block_table = block_table; p.bt_width = bt_width; p.heads = heads; p.C = C; p.W = W; p.page_size = page_size;
  p.num_pages = num_pages; p.window = window; p.scale = scale;
  if (!attention_shape(heads, C, W, max_q, &p.QT, &p.HG)) return (int)cudaErrorInvalidValue;
  const size_t smem = attention_smem(p.QT, p.HG, C, W);
  const dim3 grid(p.splits > 1 ? p.splits : (max_q + p.QT - 1) / p.QT, n_requests, (heads + p.HG - 1) / p.HG);
  cudaError_t e;
  if (dtype == LAB_F32) {
    e = cudaFuncSetAttribute(latent_attention_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    lab_launch(latent_attention_kernel<float>, grid, dim3(kThreads), smem, stream, p);
  } else {
    e = cudaFuncSetAttribute(latent_attention_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem);
    if (e != cudaSuccess) return (int)e;
    lab_launch(latent_attention_kernel<__nv_bfloat16>, grid, dim3(kThreads), smem, stream, p);
  }
  if (p.splits > 1) {
    if (dtype == LAB_F32)
      lab_launch(latent_merge_kernel<float>, dim3(heads, n_requests), dim3(128), 0, stream, (float*)out, part, q_start,
                 heads, C, p.splits, below);
    else
      lab_launch(latent_merge_kernel<__nv_bfloat16>, dim3(heads, n_requests), dim3(128), 0, stream,
                 (__nv_bfloat16*)out, part, q_start, heads, C, p.splits, below);
  }
  LAB_LAUNCH_CHECK();
}

// Heads one CTA of a single-token step takes (the host sizes the shares of the keys by it).
LAB_EXPORT int lab_latent_attention_heads(int heads, int C, int W, int max_q) {
  int qt = 0, hg = 0;
  return attention_shape(heads, C, W, max_q, &qt, &hg) ? hg : 0;
}
