// Row-wise operators for models whose residual stream is kept in 32-bit floats whatever the
// storage type T of weights and activations is: embedding with a norm, RMS norms that read the
// 32-bit stream (one or two at once, gain w or 1 + w), embedding with a learned position, the sum
// x += norm(product) of blocks that norm a sublayer's output, token shift with a per-request previous
// row, the block's sum into the stream with per-channel scales (alone, or as the opening of the
// next block's norms, as the 16-bit stream's add + norm kernel has it), concatenation for a re-entry
// projection, and a soft cap on logits.  All arithmetic is 32-bit; T only says how weights are
// stored and how outputs that feed a matrix product are rounded.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;

// Sum of split-K partial products p[s * stride + at], s ascending.  The loads of eight splits are issued
// before the first add: a loop whose every load feeds the next add runs one memory latency per split.
__device__ __forceinline__ float sum_splits(const float* __restrict__ p, int splits, long long stride, size_t at) {
  float total = 0.f;
  for (int s0 = 0; s0 < splits; s0 += 8) {
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = s0 + j < splits ? p[(s0 + j) * stride + at] : 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) total += v[j];
  }
  return total;
}

// ---- embedding + norm ---------------------------------------------------------------------
// out[t] = table[id_t] / rms(table[id_t]) * (offset + w)
template <typename T>
__global__ void __launch_bounds__(kThreads) embed_norm_kernel(float* __restrict__ out, const T* __restrict__ table,
                                                              const int* __restrict__ ids, const T* __restrict__ w,
                                                              int hidden, int vocab, float eps, float offset) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  id = min(max(id, 0), vocab - 1);
  const T* row = table + (size_t)id * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += kThreads) {
    const float v = to_f32(row[i]);
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += kThreads)
    out[(size_t)t * hidden + i] = to_f32(row[i]) * inv * (offset + to_f32(w[i]));
}

// ---- one or two norms of the same 32-bit row ----------------------------------------------
// out_a (32-bit) = x / rms(x) * (offset + wa); out_b (T) = x / rms(x) * (offset + wb).
// With `rows`, output row i comes from x[rows[i]].
template <typename T>
__global__ void __launch_bounds__(kThreads) norm_stream_kernel(float* __restrict__ out_a, T* __restrict__ out_b,
                                                               const float* __restrict__ x, const T* __restrict__ wa,
                                                               const T* __restrict__ wb, const int* __restrict__ rows,
                                                               int n_in, int hidden, float eps, float offset) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  int src = t;
  if (rows != nullptr) {
    src = rows[t];
    if (src < 0 || src >= n_in) {
      if (threadIdx.x == 0) lab_set_error(LAB_ERR_ROW_RANGE);
      return;
    }
  }
  const float* row = x + (size_t)src * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += kThreads) {
    const float v = row[i];
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += kThreads) {
    const float v = row[i] * inv;
    if (out_a != nullptr) out_a[(size_t)t * hidden + i] = v * (offset + to_f32(wa[i]));
    if (out_b != nullptr) out_b[(size_t)t * hidden + i] = from_f32<T>(v * (offset + to_f32(wb[i])));
  }
}

// ---- token shift ----------------------------------------------------------------------------
// h[t] = n[t] + (prev - n[t]) * mix, prev = n[t - 1] within a request's rows, the request's kept
// row for its first row of the step (zeros at position 0).  The block of a request's first row
// also puts the request's last row of this step in its place, after it has read the old one, so
// no other block reads what it overwrites.
template <typename T>
__global__ void __launch_bounds__(kThreads) token_shift_kernel(T* __restrict__ out, const float* __restrict__ normed,
                                                               const T* __restrict__ mix, float* __restrict__ kept,
                                                               const int* __restrict__ row_req,
                                                               const int* __restrict__ q_start,
                                                               const int* __restrict__ pos0,
                                                               const int* __restrict__ state_slot, int hidden,
                                                               int n_slots, int write) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int r = row_req[t];
  const int first = q_start[r], last = q_start[r + 1] - 1;
  const int slot = state_slot[r];
  if (slot == -1) {      // a row of padding (a request of length zero in a padded batch): zeros, no state
    for (int i = threadIdx.x; i < hidden; i += kThreads) out[(size_t)t * hidden + i] = from_f32<T>(0.f);
    return;
  }
  if (slot < 0 || slot >= n_slots) {
    if (threadIdx.x == 0) lab_set_error(LAB_ERR_PAGE_RANGE);
    return;
  }
  const float* cur = normed + (size_t)t * hidden;
  float* keep = kept + (size_t)slot * hidden;
  const bool opens = t == first;
  const bool from_kept = opens && pos0[r] > 0;
  const float* prev = opens ? keep : cur - hidden;
  for (int i = threadIdx.x; i < hidden; i += kThreads) {
    const float c = cur[i];
    const float p = (opens && !from_kept) ? 0.f : prev[i];
    out[(size_t)t * hidden + i] = from_f32<T>(c + (p - c) * to_f32(mix[i]));
    if (opens && write) keep[i] = normed[(size_t)last * hidden + i];
  }
}

// ---- the block's sum into the stream ------------------------------------------------------
// x[t] += mult * (sa * a[t] + sb * b[t]); a and b are 32-bit products [tokens, hidden] or split-K
// partial products [splits, tokens, hidden] summed here in ascending order; b may be absent.
template <typename T>
__global__ void __launch_bounds__(kThreads) stream_add_kernel(float* __restrict__ x, const float* __restrict__ a,
                                                              int a_splits, const float* __restrict__ b, int b_splits,
                                                              const T* __restrict__ sa, const T* __restrict__ sb,
                                                              long long n, int hidden, long long split_stride,
                                                              float mult) {
  pdl_trigger();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * kThreads + threadIdx.x; i < n; i += (long long)gridDim.x * kThreads) {
    const int c = (int)(i % hidden);
    float total = sum_splits(a, a_splits, split_stride, (size_t)i) * to_f32(sa[c]);
    if (b != nullptr) total += sum_splits(b, b_splits, split_stride, (size_t)i) * to_f32(sb[c]);
    x[i] += mult * total;
  }
}

// ---- the block's sum and the norms that follow it, in one pass --------------------------------
// v = x[src] + mult * (sa * a[src] + sb * b[src]) (a, b as above); without `rows` v replaces x[t]; then
// out_a (32-bit) = v / rms(v) * (offset + wa) and out_b (T) = v / rms(v) * (offset + wb).  With `rows`,
// output row t comes from row rows[t] and x is left as it is (the final norm at the wanted rows).
template <typename T>
__global__ void __launch_bounds__(1024) stream_add_norm_kernel(
    float* __restrict__ out_a, T* __restrict__ out_b, float* __restrict__ x, const float* __restrict__ a, int a_splits,
    const float* __restrict__ b, int b_splits, const T* __restrict__ sa, const T* __restrict__ sb,
    long long split_stride, float mult, const T* __restrict__ wa, const T* __restrict__ wb,
    const int* __restrict__ rows, int n_in, int hidden, float eps, float offset) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  int src = t;
  if (rows != nullptr) {
    src = rows[t];
    if (src < 0 || src >= n_in) {
      if (threadIdx.x == 0) lab_set_error(LAB_ERR_ROW_RANGE);
      return;
    }
  }
  const size_t base = (size_t)src * hidden;
  auto value = [&](int i) {
    float total = sum_splits(a, a_splits, split_stride, base + i) * to_f32(sa[i]);
    if (b != nullptr) total += sum_splits(b, b_splits, split_stride, base + i) * to_f32(sb[i]);
    return x[base + i] + mult * total;
  };
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = value(i);
    if (rows == nullptr) x[base + i] = v;      // the same thread reads it back below
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = (rows == nullptr ? x[base + i] : value(i)) * inv;
    if (out_a != nullptr) out_a[(size_t)t * hidden + i] = v * (offset + to_f32(wa[i]));
    if (out_b != nullptr) out_b[(size_t)t * hidden + i] = from_f32<T>(v * (offset + to_f32(wb[i])));
  }
}

// ---- embedding + learned position ---------------------------------------------------------
// out[t] = table[id_t] * scale + positions[p_t] as a 32-bit row.
template <typename T>
__global__ void __launch_bounds__(kThreads) embed_position_kernel(float* __restrict__ out,
                                                                  const T* __restrict__ table,
                                                                  const T* __restrict__ pos_table,
                                                                  const int* __restrict__ ids,
                                                                  const int* __restrict__ positions, int hidden,
                                                                  int vocab, int max_positions, float scale) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t], p = pos_table != nullptr ? positions[t] : 0;
  id = min(max(id, 0), vocab - 1);
  const T* row = table + (size_t)id * hidden;
  if (pos_table == nullptr) {      // no learned positions: the table's row as a 32-bit row
    for (int i = threadIdx.x; i < hidden; i += kThreads) out[(size_t)t * hidden + i] = to_f32(row[i]) * scale;
    return;
  }
  if (p >= max_positions && threadIdx.x == 0) lab_set_error(LAB_ERR_ROW_RANGE);
  p = min(max(p, 0), max_positions - 1);
  const T* prow = pos_table + (size_t)p * hidden;
  for (int i = threadIdx.x; i < hidden; i += kThreads)
    out[(size_t)t * hidden + i] = to_f32(row[i]) * scale + to_f32(prow[i]);
}

// ---- x += norm(product): the sum that closes a sublayer whose *output* is normed ----------------
// y = a[t] (+ bias), a a 32-bit product [tokens, hidden] or split-K partial products summed in ascending
// order; x[t] += y / rms(y) * w; and (if asked) the new x[t] rounded to T, for the product that reads
// the stream next, or, with `w_next`, the new x[t] normed once more: x[t] / rms(x[t]) * w_next, rounded (the
// norm that opens the next sublayer, in the same pass).
template <typename T>
__global__ void __launch_bounds__(1024) stream_norm_add_kernel(float* __restrict__ x, T* __restrict__ copy,
                                                               const float* __restrict__ a, int a_splits,
                                                               long long split_stride, const T* __restrict__ bias,
                                                               const T* __restrict__ w, int hidden, float eps,
                                                               const T* __restrict__ w_next) {
  __shared__ float scratch[32];
  extern __shared__ float row[];      // [hidden]: the product's row, summed once
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const size_t base = (size_t)t * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = sum_splits(a, a_splits, split_stride, base + i);
    if (bias != nullptr) v += to_f32(bias[i]);
    row[i] = v;
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
  float s2 = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = x[base + i] + row[i] * inv * to_f32(w[i]);
    x[base + i] = v;
    if (w_next != nullptr) {
      row[i] = v;
      s2 += v * v;
    } else if (copy != nullptr) {
      copy[base + i] = from_f32<T>(v);
    }
  }
  if (w_next == nullptr || copy == nullptr) return;
  s2 = block_sum(s2, scratch);
  const float inv2 = 1.0f / sqrtf(s2 / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) copy[base + i] = from_f32<T>(row[i] * inv2 * to_f32(w_next[i]));
}

// ---- the stream rounded to T ------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads) stream_round_kernel(T* __restrict__ out, const float* __restrict__ x,
                                                                long long n) {
  pdl_trigger();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * kThreads + threadIdx.x; i < n; i += (long long)gridDim.x * kThreads)
    out[i] = from_f32<T>(x[i]);
}

// ---- out = ca * a + cb * b over 32-bit products (or split-K partial products) -------------------
__global__ void __launch_bounds__(kThreads) weighted_sum_kernel(float* __restrict__ out, const float* __restrict__ a,
                                                                int a_splits, const float* __restrict__ b, int b_splits,
                                                                long long n, float ca, float cb) {
  pdl_trigger();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * kThreads + threadIdx.x; i < n; i += (long long)gridDim.x * kThreads)
    out[i] = ca * sum_splits(a, a_splits, n, (size_t)i) + cb * sum_splits(b, b_splits, n, (size_t)i);
}

// ---- [x; x0] rounded to T -------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads) concat_kernel(T* __restrict__ out, const float* __restrict__ x,
                                                          const float* __restrict__ x0, long long tokens, int hidden) {
  pdl_trigger();
  pdl_wait();
  const long long n = tokens * 2 * hidden;
  for (long long i = (long long)blockIdx.x * kThreads + threadIdx.x; i < n; i += (long long)gridDim.x * kThreads) {
    const long long t = i / (2 * hidden);
    const int c = (int)(i % (2 * hidden));
    out[i] = from_f32<T>(c < hidden ? x[t * hidden + c] : x0[t * hidden + c - hidden]);
  }
}

// ---- logits <- cap * tanh(logits / cap) -----------------------------------------------------
__global__ void __launch_bounds__(kThreads) softcap_kernel(float* __restrict__ logits, long long n, float cap) {
  pdl_trigger();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * kThreads + threadIdx.x; i < n; i += (long long)gridDim.x * kThreads)
    logits[i] = cap * tanhf(logits[i] / cap);
}

int blocks_for(long long n) { return (int)((n + kThreads - 1) / kThreads < 148 * 8 ? (n + kThreads - 1) / kThreads : 148 * 8); }

}  // namespace

LAB_EXPORT int lab_embed_norm(float* out, const void* table, const int* ids, const void* w, int tokens, int hidden,
                              int vocab, float eps, float offset, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (dtype == LAB_F32)
    lab_launch(embed_norm_kernel<float>, dim3(tokens), dim3(kThreads), 0, stream, out, (const float*)table, ids,
               (const float*)w, hidden, vocab, eps, offset);
  else
    lab_launch(embed_norm_kernel<__nv_bfloat16>, dim3(tokens), dim3(kThreads), 0, stream, out,
               (const __nv_bfloat16*)table, ids, (const __nv_bfloat16*)w, hidden, vocab, eps, offset);
  LAB_LAUNCH_CHECK();
}

LAB_EXPORT int lab_norm_stream(float* out_a, void* out_b, const float* x, const void* wa, const void* wb,
                               const int* rows, int n_out, int n_in, int hidden, float eps, float offset, int dtype,
                               cudaStream_t stream) {
  if (n_out <= 0) return 0;
  if (dtype == LAB_F32)
    lab_launch(norm_stream_kernel<float>, dim3(n_out), dim3(kThreads), 0, stream, out_a, (float*)out_b, x,
               (const float*)wa, (const float*)wb, rows, n_in, hidden, eps, offset);
  else
    lab_launch(norm_stream_kernel<__nv_bfloat16>, dim3(n_out), dim3(kThreads), 0, stream, out_a, (__nv_bfloat16*)out_b,
               x, (const __nv_bfloat16*)wa, (const __nv_bfloat16*)wb, rows, n_in, hidden, eps, offset);
  LAB_LAUNCH_CHECK();
}

LAB_EXPORT int lab_token_shift(void* out, const float* normed, const void* mix, float* kept, const int* row_req,
                               const int* q_start, const int* pos0, const int* state_slot, int tokens, int hidden,
                               int n_slots, int write, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (dtype == LAB_F32)
    lab_launch(token_shift_kernel<float>, dim3(tokens), dim3(kThreads), 0, stream, (float*)out, normed,
               (const float*)mix, kept, row_req, q_start, pos0, state_slot, hidden, n_slots, write);
  else
    lab_launch(token_shift_kernel<__nv_bfloat16>, dim3(tokens), dim3(kThreads), 0, stream, (__nv_bfloat16*)out, normed,
               (const __nv_bfloat16*)mix, kept, row_req, q_start, pos0, state_slot, hidden, n_slots, write);
  LAB_LAUNCH_CHECK();
}

LAB_EXPORT int lab_stream_add(float* x, const float* a, int a_splits, const float* b, int b_splits, const void* sa,
                              const void* sb, long long tokens, int hidden, float mult, int dtype,
                              cudaStream_t stream) {
  const long long n = tokens * hidden;
  if (n <= 0) return 0;
  if (dtype == LAB_F32)
    lab_launch(stream_add_kernel<float>, dim3(blocks_for(n)), dim3(kThreads), 0, stream, x, a, a_splits, b, b_splits,
               (const float*)sa, (const float*)sb, n, hidden, n, mult);
  else
    lab_launch(stream_add_kernel<__nv_bfloat16>, dim3(blocks_for(n)), dim3(kThreads), 0, stream, x, a, a_splits, b,
               b_splits, (const __nv_bfloat16*)sa, (const __nv_bfloat16*)sb, n, hidden, n, mult);
  LAB_LAUNCH_CHECK();
}

LAB_EXPORT int lab_stream_add_norm(float* out_a, void* out_b, float* x, const float* a, int a_splits, const float* b,
                                   int b_splits, const void* sa, const void* sb, float mult, const void* wa,
                                   const void* wb, const int* rows, int n_out, int n_in, int hidden, float eps,
                                   float offset, int dtype, cudaStream_t stream) {
  if (n_out <= 0) return 0;
  const long long stride = (long long)n_in * hidden;
  // few rows (a decode step): an element a thread, so that a row's loads are all in flight at once
  const int threads = n_out <= 64 ? (hidden >= 1024 ? 1024 : (hidden + 31) / 32 * 32) : kThreads;
  if (dtype == LAB_F32)
    lab_launch(stream_add_norm_kernel<float>, dim3(n_out), dim3(threads), 0, stream, out_a, (float*)out_b, x, a,
               a_splits, b, b_splits, (const float*)sa, (const float*)sb, stride, mult, (const float*)wa,
               (const float*)wb, rows, n_in, hidden, eps, offset);
  else
    lab_launch(stream_add_norm_kernel<__nv_bfloat16>, dim3(n_out), dim3(threads), 0, stream, out_a,
               (__nv_bfloat16*)out_b, x, a, a_splits, b, b_splits, (const __nv_bfloat16*)sa, (const __nv_bfloat16*)sb,
               stride, mult, (const __nv_bfloat16*)wa, (const __nv_bfloat16*)wb, rows, n_in, hidden, eps, offset);
  LAB_LAUNCH_CHECK();
}

LAB_EXPORT int lab_embed_position(float* out, const void* table, const void* pos_table, const int* ids,
                                  const int* positions, int tokens, int hidden, int vocab, int max_positions, float scale,
                                  int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (dtype == LAB_F32)
    lab_launch(embed_position_kernel<float>, dim3(tokens), dim3(kThreads), 0, stream, out,
               (const float*)table, (const float*)pos_table, ids, positions, hidden, vocab, max_positions, scale);
  else
    lab_launch(embed_position_kernel<__nv_bfloat16>, dim3(tokens), dim3(kThreads), 0, stream, out,
               (const __nv_bfloat16*)table, (const __nv_bfloat16*)pos_table, ids, positions, hidden, vocab,
               max_positions, scale);
  LAB_LAUNCH_CHECK();
}

LAB_EXPORT int lab_stream_norm_add(float* x, void* copy, const float* a, int a_splits, const void* bias, const void* w,
                                   int tokens, int hidden, float eps, const void* w_next, int dtype,
                                   cudaStream_t stream) {
  if (tokens <= 0) return 0;
  const long long stride = (long long)tokens * hidden;
  const size_t smem = (size_t)hidden * sizeof(float);
  if (smem > 160 * 1024) return (int)cudaErrorInvalidValue;
  const int threads = tokens <= 64 ? (hidden >= 1024 ? 1024 : (hidden + 31) / 32 * 32) : kThreads;
  if (dtype == LAB_F32) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(stream_norm_add_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    lab_launch(stream_norm_add_kernel<float>, dim3(tokens), dim3(threads), smem, stream, x, (float*)copy, a, a_splits,
               stride, (const float*)bias, (const float*)w, hidden, eps, (const float*)w_next);
  } else {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(stream_norm_add_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    lab_launch(stream_norm_add_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), smem, stream, x, (__nv_bfloat16*)copy,
               a, a_splits, stride, (const __nv_bfloat16*)bias, (const __nv_bfloat16*)w, hidden, eps,
               (const __nv_bfloat16*)w_next);
  }
  LAB_LAUNCH_CHECK();
}

LAB_EXPORT int lab_stream_round(void* out, const float* x, long long n, int dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (dtype == LAB_F32)
    lab_launch(stream_round_kernel<float>, dim3(blocks_for(n)), dim3(kThreads), 0, stream, (float*)out, x, n);
  else
    lab_launch(stream_round_kernel<__nv_bfloat16>, dim3(blocks_for(n)), dim3(kThreads), 0, stream, (__nv_bfloat16*)out, x, n);
  LAB_LAUNCH_CHECK();
}

LAB_EXPORT int lab_weighted_sum(float* out, const float* a, int a_splits, const float* b, int b_splits, long long n,
                                float ca, float cb, cudaStream_t stream) {
  if (n <= 0) return 0;
  lab_launch(weighted_sum_kernel, dim3(blocks_for(n)), dim3(kThreads), 0, stream, out, a, a_splits, b, b_splits, n, ca, cb);
  LAB_LAUNCH_CHECK();
}

LAB_EXPORT int lab_stream_concat(void* out, const float* x, const float* x0, long long tokens, int hidden, int dtype,
                                 cudaStream_t stream) {
  const long long n = tokens * 2 * hidden;
  if (n <= 0) return 0;
  if (dtype == LAB_F32)
    lab_launch(concat_kernel<float>, dim3(blocks_for(n)), dim3(kThreads), 0, stream, (float*)out, x, x0, tokens, hidden);
  else
    lab_launch(concat_kernel<__nv_bfloat16>, dim3(blocks_for(n)), dim3(kThreads), 0, stream, (__nv_bfloat16*)out, x, x0,
               tokens, hidden);
  LAB_LAUNCH_CHECK();
}

LAB_EXPORT int lab_softcap(float* logits, long long n, float cap, cudaStream_t stream) {
  if (n <= 0) return 0;
  lab_launch(softcap_kernel, dim3(blocks_for(n)), dim3(kThreads), 0, stream, logits, n, cap);
  LAB_LAUNCH_CHECK();
}
