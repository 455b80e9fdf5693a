// Rotary positions on neighbouring pairs, fused with the sum of the projection's partial products, its
// bias, the rounding of q and the write of keys and values into their page slots.
//
// proj [tokens, ld] floats (or `splits` such partial products `split_stride` floats apart, summed in
// ascending order): q heads at columns [0, n_q * dim), key heads from column k_at on (n_kv * dim), value
// heads from column v_at on (n_kv * vdim).  v_at == k_at means that the values are the keys as projected,
// before the rotation (a design without a value matrix).  bias [same columns] or null.
//
// Of every q and k head the first rot_dims entries turn: the pair (2i, 2i + 1) by the angle
// position * inv_freq[i] (32-bit position, angle, cosine and sine); later entries pass unchanged.
// q goes out in the storage type, `head` entries a head (zeros beyond dim); k and v go to the row's slot
// of caches [slots, n_kv, page, head] (zeros beyond dim and vdim), unless slots is null (a call that
// only reads the cache) or the row's slot is -1 (a row of padding).
#include "common.cuh"

namespace {
constexpr int kThreads = 256;

struct RopePairsParams {
  const float* proj;
  long long split_stride;
  int splits, ld, k_at, v_at;
  const int* positions;
  const float* inv_freq;
  const int* slots;
  long long n_slots;     // rows of the caches: pages * page size
  int n_q, n_kv, dim, vdim, head, rot_dims, page_size;
};

__device__ __forceinline__ float summed(const RopePairsParams& p, size_t at) {
  float v = p.proj[at];
  for (int s = 1; s < p.splits; ++s) v += p.proj[at + (size_t)s * p.split_stride];
  return v;
}

// the entry e of a head that starts at column `col` of row t, with bias, rotated where it must be
template <typename T>
__device__ __forceinline__ float rotated_entry(const RopePairsParams& p, const T* bias, size_t row, int col, int e,
                                               float pos, bool rotate) {
  float v = summed(p, row + col + e) + (bias != nullptr ? to_f32(bias[col + e]) : 0.f);
  if (!rotate || e >= p.rot_dims) return v;
  const int mate = e ^ 1;
  const float w = summed(p, row + col + mate) + (bias != nullptr ? to_f32(bias[col + mate]) : 0.f);
  const float ang = pos * p.inv_freq[e >> 1];
  const float cs = cosf(ang), sn = sinf(ang);
  // even entry: u cos - v sin; odd entry: v cos + u sin
  return (e & 1) ? __fmaf_rn(v, cs, __fmul_rn(w, sn)) : __fmaf_rn(v, cs, -__fmul_rn(w, sn));
}

template <typename T>
__global__ void __launch_bounds__(kThreads) rope_pairs_store_kernel(T* __restrict__ q_out, T* __restrict__ cache_k,
                                                                    T* __restrict__ cache_v,
                                                                    const T* __restrict__ bias, RopePairsParams p) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const size_t row = (size_t)t * p.ld;
  const float pos = (float)p.positions[t];
  const int HD = p.head;
  for (int i = threadIdx.x; i < p.n_q * HD; i += kThreads) {
    const int h = i / HD, e = i % HD;
    q_out[(size_t)t * p.n_q * HD + i] = from_f32<T>(e < p.dim ? rotated_entry(p, bias, row, h * p.dim, e, pos, true) : 0.f);
  }
  if (p.slots == nullptr) return;
  const long long slot = p.slots[t];
  if (slot == -1) return;
  if (slot < 0 || slot >= p.n_slots) {
    if (threadIdx.x == 0) lab_set_error(LAB_ERR_PAGE_RANGE);
    return;
  }
  const long long page = slot / p.page_size, off = slot % p.page_size;
  for (int i = threadIdx.x; i < p.n_kv * HD; i += kThreads) {
    const int g = i / HD, e = i % HD;
    const size_t at = (((size_t)page * p.n_kv + g) * p.page_size + off) * HD + e;
    cache_k[at] = from_f32<T>(e < p.dim ? rotated_entry(p, bias, row, p.k_at + g * p.dim, e, pos, true) : 0.f);
    cache_v[at] = from_f32<T>(e < p.vdim ? rotated_entry(p, bias, row, p.v_at + g * p.vdim, e, pos, false) : 0.f);
  }
}

// ---- the same, with a norm per head and a temperature on q ------------------------------------------
// After the rotation every q and k head may be divided by its root mean square over `dim` (eps inside the
// root) and multiplied by a weight of `dim` entries that all heads share (null: no weight); then q is
// multiplied by a number per head (`q_head_scale`, null: 1) and by 1 + coef * ln(floor((pos + 1) / every) + 1)
// (`every` 0: 1).  One warp per (row, head), a head's entries over the lanes.
struct HeadPrepParams {
  float norm_eps;          // <= 0: no norm
  const float* q_head_scale;
  float temp_coef;
  int temp_every;
};

template <typename T>
__global__ void __launch_bounds__(kThreads) head_prep_store_kernel(T* __restrict__ q_out, T* __restrict__ cache_k,
                                                                   T* __restrict__ cache_v, const T* __restrict__ bias,
                                                                   const T* __restrict__ q_norm_w,
                                                                   const T* __restrict__ k_norm_w, RopePairsParams p,
                                                                   HeadPrepParams hp, int tokens) {
  pdl_trigger();
  pdl_wait();
  constexpr int kPerLane = 8;      // heads of up to 256 entries
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int units = p.n_q + 2 * p.n_kv;
  const long long unit = (long long)blockIdx.x * (kThreads / 32) + warp;
  if (unit >= (long long)tokens * units) return;
  const int t = (int)(unit / units), u = (int)(unit - (long long)t * units);
  const size_t row = (size_t)t * p.ld;
  const int ipos = p.positions[t];
  const float pos = (float)ipos;
  const int HD = p.head;
  const bool is_q = u < p.n_q, is_v = u >= p.n_q + p.n_kv;
  const int g = is_q ? u : (is_v ? u - p.n_q - p.n_kv : u - p.n_q);
  T* dst;
  if (is_q) {
    dst = q_out + ((size_t)t * p.n_q + g) * HD;
  } else {
    if (p.slots == nullptr) return;
    const long long slot = p.slots[t];
    if (slot == -1) return;
    if (slot < 0 || slot >= p.n_slots) {
      if (lane == 0) lab_set_error(LAB_ERR_PAGE_RANGE);
      return;
    }
    const long long page = slot / p.page_size, off = slot % p.page_size;
    dst = (is_v ? cache_v : cache_k) + (((size_t)page * p.n_kv + g) * p.page_size + off) * HD;
  }
  if (is_v) {
    for (int e = lane; e < HD; e += 32)
      dst[e] = from_f32<T>(e < p.vdim ? rotated_entry(p, bias, row, p.v_at + g * p.vdim, e, pos, false) : 0.f);
    return;
  }
  const int col = is_q ? g * p.dim : p.k_at + g * p.dim;
  float val[kPerLane], ss = 0.f;
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) {
    const int e = lane + 32 * i;
    val[i] = e < p.dim ? rotated_entry(p, bias, row, col, e, pos, true) : 0.f;
    ss = fmaf(val[i], val[i], ss);
  }
  float mult = 1.f;
  if (hp.norm_eps > 0.f) mult = 1.0f / sqrtf(warp_sum(ss) / (float)p.dim + hp.norm_eps);
  const T* w = is_q ? q_norm_w : k_norm_w;
  float after = 1.f;
  if (is_q) {
    if (hp.q_head_scale != nullptr) after = hp.q_head_scale[g];
    if (hp.temp_every > 0) after *= 1.f + hp.temp_coef * logf((float)((ipos + 1) / hp.temp_every) + 1.f);
  }
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) {
    const int e = lane + 32 * i;
    if (e >= HD) break;
    float v = val[i] * mult;
    if (w != nullptr && e < p.dim) v *= to_f32(w[e]);
    dst[e] = from_f32<T>(v * after);
  }
}
}  // namespace

LAB_EXPORT int lab_rope_pairs_store(void* q_out, void* cache_k, void* cache_v, const float* proj, int splits,
                                    long long split_stride, int ld, int k_at, int v_at, const void* bias,
                                    const int* positions, const float* inv_freq, int rot_dims, const int* slots,
                                    long long n_slots, int tokens, int n_q, int n_kv, int dim, int vdim, int head,
                                    int page_size, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (rot_dims < 0 || rot_dims % 2 || rot_dims > dim || dim > head || vdim > head || splits < 1 || page_size < 1)
    return (int)cudaErrorInvalidValue;
  RopePairsParams p;
  p.proj = proj; p.split_stride = split_stride; p.splits = splits; p.ld = ld; p.k_at = k_at; p.v_at = v_at;
  p.positions = positions; p.inv_freq = inv_freq; p.slots = slots; p.n_slots = n_slots; p.n_q = n_q; p.n_kv = n_kv;
  p.dim = dim; p.vdim = vdim; p.head = head; p.rot_dims = rot_dims; p.page_size = page_size;
  if (dtype == LAB_F32)
    lab_launch(rope_pairs_store_kernel<float>, dim3(tokens), dim3(kThreads), 0, stream, (float*)q_out, (float*)cache_k,
               (float*)cache_v, (const float*)bias, p);
  else
    lab_launch(rope_pairs_store_kernel<__nv_bfloat16>, dim3(tokens), dim3(kThreads), 0, stream, (__nv_bfloat16*)q_out,
               (__nv_bfloat16*)cache_k, (__nv_bfloat16*)cache_v, (const __nv_bfloat16*)bias, p);
  LAB_LAUNCH_CHECK();
}


// As lab_rope_pairs_store, with the norm per head (norm_eps > 0; weights q_norm_w, k_norm_w of `dim` entries or
// null) and q's temperatures (q_head_scale [n_q] floats or null; temp_every > 0: 1 + temp_coef * ln(floor((pos + 1)
// / temp_every) + 1)).  rot_dims may be 0: no rotation.
LAB_EXPORT int lab_head_prep_store(void* q_out, void* cache_k, void* cache_v, const float* proj, int splits,
                                   long long split_stride, int ld, int k_at, int v_at, const void* bias,
                                   const int* positions, const float* inv_freq, int rot_dims, const int* slots,
                                   long long n_slots, int tokens, int n_q, int n_kv, int dim, int vdim, int head,
                                   int page_size, float norm_eps, const void* q_norm_w, const void* k_norm_w,
                                   const float* q_head_scale, float temp_coef, int temp_every, int dtype,
                                   cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (rot_dims < 0 || rot_dims % 2 || rot_dims > dim || dim > head || vdim > head || splits < 1 || page_size < 1 ||
      head > 256 || temp_every < 0)
    return (int)cudaErrorInvalidValue;
  RopePairsParams p;
  p.proj = proj; p.split_stride = split_stride; p.splits = splits; p.ld = ld; p.k_at = k_at; p.v_at = v_at;
  p.positions = positions; p.inv_freq = inv_freq; p.slots = slots; p.n_slots = n_slots; p.n_q = n_q; p.n_kv = n_kv;
  p.dim = dim; p.vdim = vdim; p.head = head; p.rot_dims = rot_dims; p.page_size = page_size;
  HeadPrepParams hp;
  hp.norm_eps = norm_eps; hp.q_head_scale = q_head_scale; hp.temp_coef = temp_coef; hp.temp_every = temp_every;
  const long long units = (long long)tokens * (n_q + 2 * n_kv);
  const int blocks = (int)((units + kThreads / 32 - 1) / (kThreads / 32));
  if (dtype == LAB_F32)
    lab_launch(head_prep_store_kernel<float>, dim3(blocks), dim3(kThreads), 0, stream, (float*)q_out, (float*)cache_k,
               (float*)cache_v, (const float*)bias, (const float*)q_norm_w, (const float*)k_norm_w, p, hp, tokens);
  else
    lab_launch(head_prep_store_kernel<__nv_bfloat16>, dim3(blocks), dim3(kThreads), 0, stream, (__nv_bfloat16*)q_out,
               (__nv_bfloat16*)cache_k, (__nv_bfloat16*)cache_v, (const __nv_bfloat16*)bias,
               (const __nv_bfloat16*)q_norm_w, (const __nv_bfloat16*)k_norm_w, p, hp, tokens);
  LAB_LAUNCH_CHECK();
}
