// Routed feed-forward layers (a mixture of experts): the router's choice, the layout of the chosen
// (token, expert) pairs in rows grouped by expert, and the weighted sum of the experts' results.
//
//   scores  s = softmax(z) over all experts, z the router's logits in 32-bit
//   choice  the `top` largest scores of a token (ties: the smaller index)
//   weights the chosen scores over their sum (+ 1e-20), or (renorm 0) the chosen scores as they are
//   out[t]  = sum over the chosen of weight * expert's result  (+ sigmoid(g_t) * shared expert's result)
//
// The grouped matrix products between these kernels read rows through `row_src` and pick a tile's matrix
// by `tile_group` (see the product kernels): pair (t, k) lies at row pos_of[t * top + k] of the grouped
// layout, every expert's rows start on a tile border, unused rows are marked -1.  Where a pair lands inside
// its expert's rows depends on timing; no result does: the sum over a token's experts runs in the order of
// its choice.
#include "common.cuh"

namespace {
constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

// One warp per token.  logits [tokens, ld]: the experts' logits at columns [0, E); column `gate_col` (if
// >= 0) holds the logit of the shared expert's gate.
__global__ void __launch_bounds__(kThreads) moe_route_kernel(int* __restrict__ chosen, float* __restrict__ weight,
                                                             float* __restrict__ shared_gate,
                                                             const float* __restrict__ logits, int ld, int tokens,
                                                             int E, int top, int gate_col, int renorm) {
  extern __shared__ float scores[];      // [kWarps][E]
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * kWarps + warp;
  if (t >= tokens) return;
  float* s = scores + (size_t)warp * E;
  const float* z = logits + (size_t)t * ld;
  float big = -INFINITY;
  for (int e = lane; e < E; e += 32) big = fmaxf(big, z[e]);
  big = warp_max(big);
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) {
    const float v = expf(z[e] - big);
    s[e] = v;
    sum += v;
  }
  sum = warp_sum(sum);
  __syncwarp();
  float total = 0.f;
  // A score that is no number (a row of padding may hold anything) counts as -1, below every real score and
  // above the mark of a taken expert (-3), so that every choice names an expert that exists.
  for (int k = 0; k < top; ++k) {
    float best = -2.f;
    int at = E;
    for (int e = lane; e < E; e += 32) {
      const float v = s[e] >= 0.f || s[e] == -3.f ? s[e] : -1.f;
      if (v > best) { best = v; at = e; }       // ascending e: the first of equals stays
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    const float score = best >= 0.f ? best / sum : 0.f;
    total += score;
    if (lane == 0) {
      chosen[(size_t)t * top + k] = min(at, E - 1);
      weight[(size_t)t * top + k] = score;
      if (at < E) s[at] = -3.f;      // taken
    }
    __syncwarp();
  }
  __syncwarp();
  if (renorm) {
    const float inv = 1.f / (total + 1e-20f);
    for (int k = lane; k < top; k += 32) weight[(size_t)t * top + k] *= inv;
  }
  if (lane == 0 && shared_gate != nullptr) shared_gate[t] = gate_col >= 0 ? 1.f / (1.f + expf(-z[gate_col])) : 1.f;
}

// One CTA lays the pairs out: counts per expert, every expert's first row on a border of `tile` rows, the
// expert of every tile (-1 beyond the last used tile), and every pair's row.
__global__ void __launch_bounds__(1024) moe_align_kernel(int* __restrict__ row_src, int* __restrict__ tile_group,
                                                         int* __restrict__ pos_of, const int* __restrict__ chosen,
                                                         int pairs, int E, int tile, int rows_cap) {
  extern __shared__ int counts[];        // [E] counts, then [E] first rows, then [E] cursors
  int* start = counts + E;
  int* cursor = start + E;
  pdl_trigger();
  pdl_wait();
  const int tid = threadIdx.x;
  for (int e = tid; e < E; e += blockDim.x) counts[e] = cursor[e] = 0;
  for (int i = tid; i < rows_cap; i += blockDim.x) row_src[i] = -1;
  __syncthreads();
  for (int i = tid; i < pairs; i += blockDim.x) {
    const int e = chosen[i];
    if (e >= 0 && e < E) atomicAdd(&counts[e], 1);
  }
  __syncthreads();
  if (tid == 0) {
    int at = 0;
    for (int e = 0; e < E; ++e) {
      start[e] = at;
      const int tiles = (counts[e] + tile - 1) / tile;
      for (int j = 0; j < tiles; ++j) tile_group[at / tile + j] = e;
      at += tiles * tile;
    }
    for (int j = at / tile; j < rows_cap / tile; ++j) tile_group[j] = -1;
  }
  __syncthreads();
  for (int i = tid; i < pairs; i += blockDim.x) {
    const int e = chosen[i];
    if (e < 0 || e >= E) {
      pos_of[i] = -1;
      continue;
    }
    const int at = start[e] + atomicAdd(&cursor[e], 1);
    pos_of[i] = at;
    row_src[at] = i;
  }
}

// rows of the grouped layout as a matrix of their own (for products that cannot gather): out[r] = x[row_src[r] / top],
// zeros where row_src is -1.  grid (rows); 16 bytes a thread where the rows allow it (`vec`).
template <typename T>
__global__ void __launch_bounds__(128) moe_gather_kernel(T* __restrict__ out, const T* __restrict__ x,
                                                         const int* __restrict__ row_src, int top, int width, int ldx,
                                                         int vec) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x, src = row_src[r];
  T* dst = out + (size_t)r * width;
  const T* row = src < 0 ? nullptr : x + (size_t)(src / top) * ldx;
  if (vec) {
    constexpr int PER = 16 / sizeof(T);
    for (int i = threadIdx.x; i < width / PER; i += 128)
      reinterpret_cast<uint4*>(dst)[i] = row ? reinterpret_cast<const uint4*>(row)[i] : make_uint4(0, 0, 0, 0);
    return;
  }
  for (int i = threadIdx.x; i < width; i += 128) dst[i] = row ? row[i] : from_f32<T>(0.f);
}

// out[t] = sum_k weight[t, k] * y[pos_of[t, k]] (+ shared_gate[t] * shared[t]), all 32-bit.  grid (tokens).
__global__ void __launch_bounds__(kThreads) moe_combine_kernel(float* __restrict__ out, const float* __restrict__ y,
                                                               const int* __restrict__ pos_of,
                                                               const float* __restrict__ weight,
                                                               const float* __restrict__ shared,
                                                               const float* __restrict__ shared_gate, int top,
                                                               int width) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const float g = shared != nullptr ? (shared_gate != nullptr ? shared_gate[t] : 1.f) : 0.f;
  for (int i = threadIdx.x; i < width; i += kThreads) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k) {
      const int at = pos_of[(size_t)t * top + k];
      if (at >= 0) acc = fmaf(weight[(size_t)t * top + k], y[(size_t)at * width + i], acc);
    }
    if (shared != nullptr) acc = fmaf(g, shared[(size_t)t * width + i], acc);
    out[(size_t)t * width + i] = acc;
  }
}
}  // namespace

LAB_EXPORT int lab_moe_route(int* chosen, float* weight, float* shared_gate, const float* logits, int ld, int tokens,
                             int E, int top, int gate_col, int renorm, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (E <= 0 || top <= 0 || top > E || (size_t)kWarps * E * sizeof(float) > 48 * 1024) return (int)cudaErrorInvalidValue;
  lab_launch(moe_route_kernel, dim3((tokens + kWarps - 1) / kWarps), dim3(kThreads), sizeof(float) * kWarps * E, stream,
             chosen, weight, shared_gate, logits, ld, tokens, E, top, gate_col, renorm);
  LAB_LAUNCH_CHECK();
}

// rows_cap: rows of the grouped layout, a multiple of `tile` and at least pairs + E * (tile - 1) rounded up to it.
LAB_EXPORT int lab_moe_align(int* row_src, int* tile_group, int* pos_of, const int* chosen, int pairs, int E, int tile,
                             int rows_cap, cudaStream_t stream) {
  if (pairs <= 0) return 0;
  if (tile <= 0 || rows_cap % tile || rows_cap < pairs + E * (tile - 1) || (size_t)3 * E * sizeof(int) > 48 * 1024)
    return (int)cudaErrorInvalidValue;
  lab_launch(moe_align_kernel, dim3(1), dim3(1024), sizeof(int) * 3 * E, stream, row_src, tile_group, pos_of, chosen,
             pairs, E, tile, rows_cap);
  LAB_LAUNCH_CHECK();
}

LAB_EXPORT int lab_moe_gather(void* out, const void* x, const int* row_src, int rows, int top, int width, int ldx,
                              int dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  const int per = dtype == LAB_F32 ? 4 : 8;
  const int vec = width % per == 0 && ldx % per == 0 && ((((uintptr_t)out) | ((uintptr_t)x)) & 15) == 0;
  if (dtype == LAB_F32)
    lab_launch(moe_gather_kernel<float>, dim3(rows), dim3(128), 0, stream, (float*)out, (const float*)x, row_src, top,
               width, ldx, vec);
  else
    lab_launch(moe_gather_kernel<__nv_bfloat16>, dim3(rows), dim3(128), 0, stream, (__nv_bfloat16*)out,
               (const __nv_bfloat16*)x, row_src, top, width, ldx, vec);
  LAB_LAUNCH_CHECK();
}

LAB_EXPORT int lab_moe_combine(float* out, const float* y, const int* pos_of, const float* weight, const float* shared,
                               const float* shared_gate, int tokens, int top, int width, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  lab_launch(moe_combine_kernel, dim3(tokens), dim3(kThreads), 0, stream, out, y, pos_of, weight, shared, shared_gate, top,
             width);
  LAB_LAUNCH_CHECK();
}
