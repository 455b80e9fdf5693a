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
