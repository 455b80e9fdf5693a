// Plain matrix product on the ordinary arithmetic units (no tensor cores, no reduced
// precision): the matrix product of the 32-bit path, and the yardstick the tensor-core
// kernels are tested against.
//
//   out[m, n] = OutT( sum_k x[m, k] * w[n, k]  (+ bias[n]) )          w is [out, in]
//   gated:      out[m, n] = T( silu(g) * u ),  g = x . w[n], u = x . w[inter + n]   (32-bit, one rounding)
//
// The sum over k runs in ascending order with one fused multiply-add per term, so an
// output element does not depend on how the rows were batched.  Formulas:
// rust/engine/src/runner/model/qwen2/kernels.rs:156-178, 393-418 (linear, bias in 32-bit,
// one rounding), 422-448 (gate/up with the SiLU product), 1469-1486 (SiLU).
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, PAD = 4;

template <typename T, typename OutT, bool GATED>
__global__ void __launch_bounds__(256) gemm_plain_kernel(OutT* __restrict__ out, const T* __restrict__ x,
                                                         const T* __restrict__ w, const T* __restrict__ bias, int M,
                                                         int N, int K, int ldx, int ldo, long long batch_x,
                                                         long long batch_w, long long batch_o, int gelu,
                                                         const int* __restrict__ row_src, int row_div,
                                                         const int* __restrict__ tile_group, float gate_limit) {
  pdl_trigger();
  pdl_wait();
  // a batch of products of one shape (blockIdx.z): operand b lies b * batch_* elements further on
  x += blockIdx.z * batch_x;
  w += blockIdx.z * batch_w;
  out += blockIdx.z * batch_o;
  // grouped rows: every tile of BM rows meets the matrix of its own group (tile_group[tile], -1: a tile without
  // rows), batch_w elements apart; row m reads x's row row_src[m] / row_div (-1: a row of padding, zeros)
  if (tile_group != nullptr) {
    const int group = tile_group[blockIdx.y];
    if (group < 0) return;
    w += (long long)group * batch_w;
  }
  __shared__ float xs[BK][BM + PAD];
  __shared__ float ws[GATED ? 2 : 1][BK][BN + PAD];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[GATED ? 2 : 1][4][4];
#pragma unroll
  for (int g = 0; g < (GATED ? 2 : 1); ++g)
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[g][i][j] = 0.f;

  const int lr = tid >> 2, lk = (tid & 3) * 4;  // this thread loads row lr, k in [lk, lk + 4)
  int m = m0 + lr;                              // the row of x this thread loads
  if (row_src != nullptr && m < M) {
    const int src = row_src[m];
    m = src < 0 ? M : src / row_div;
  }
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int k = k0 + lk + e;
      xs[lk + e][lr] = (m < M && k < K) ? to_f32<T>(x[(size_t)m * ldx + k]) : 0.f;
      const int n = n0 + lr;
      ws[0][lk + e][lr] = (n < N && k < K) ? to_f32<T>(w[(size_t)n * K + k]) : 0.f;
      if (GATED) ws[GATED ? 1 : 0][lk + e][lr] = (n < N && k < K) ? to_f32<T>(w[(size_t)(N + n) * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[4], b[GATED ? 2 : 1][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[k][ty * 4 + i];
#pragma unroll
      for (int g = 0; g < (GATED ? 2 : 1); ++g)
#pragma unroll
        for (int j = 0; j < 4; ++j) b[g][j] = ws[g][k][tx * 4 + j];
#pragma unroll
      for (int g = 0; g < (GATED ? 2 : 1); ++g)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[g][i][j] = fmaf(a[i], b[g][j], acc[g][i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v;
      if (GATED) {
        const float g = acc[0][i][j], u = acc[GATED ? 1 : 0][i][j];
        v = gate_pair(g, u, gate_limit);
      } else {
        v = acc[0][i][j] + (bias ? to_f32<T>(bias[n]) : 0.f);
        if (gelu) v = lab_act(v, gelu);      // the activation after the bias, before the rounding
      }
      out[(size_t)m * ldo + n] = from_f32<OutT>(v);
    }
  }
}

// Per-head products for few tokens (a decode step): out[t, h, n] = sum_k w[h, n, k] * x[t, h, k].  A warp
// forms one output column for every token: it reads the weight row once, lanes over k, and finishes each
// token's sum with a shuffle tree; the tokens' inputs of the head wait in shared memory.  The 64 x 64 tiles
// above walk K in steps of 16 behind a barrier each, which costs a memory latency per step.
constexpr int HF_TOKENS = 16;
template <typename T, typename OutT>
__global__ void __launch_bounds__(256) gemm_heads_few_kernel(OutT* __restrict__ out, const T* __restrict__ x,
                                                             const T* __restrict__ w, int M, int N, int K, int ldx,
                                                             int ldo, long long head_x, long long head_o) {
  extern __shared__ float hf_x[];      // [M][K]
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < M * K; i += 256) hf_x[i] = to_f32<T>(x[(size_t)(i / K) * ldx + h * head_x + i % K]);
  __syncthreads();
  const int n = blockIdx.x * 8 + warp;
  if (n >= N) return;
  const T* row = w + ((size_t)h * N + n) * K;
  float acc[HF_TOKENS];
#pragma unroll
  for (int t = 0; t < HF_TOKENS; ++t) acc[t] = 0.f;
  for (int k = lane; k < K; k += 32) {
    const float wv = to_f32<T>(row[k]);
#pragma unroll
    for (int t = 0; t < HF_TOKENS; ++t)
      if (t < M) acc[t] = fmaf(wv, hf_x[t * K + k], acc[t]);
  }
#pragma unroll
  for (int t = 0; t < HF_TOKENS; ++t) {
    if (t >= M) break;
    const float v = warp_sum(acc[t]);
    if (lane == 0) out[(size_t)t * ldo + h * head_o + n] = from_f32<OutT>(v);
  }
}

template <typename T, typename OutT>
int launch_heads_few(void* out, const void* x, const void* w, int M, int N, int K, int ldx, int ldo, int heads,
                     long long head_x, long long head_o, cudaStream_t stream) {
  return (int)lab_launch(gemm_heads_few_kernel<T, OutT>, dim3((N + 7) / 8, heads), dim3(256),
                         sizeof(float) * (size_t)M * K, stream, (OutT*)out, (const T*)x, (const T*)w, M, N, K, ldx, ldo,
                         head_x, head_o);
}

// Grouped rows for few rows (a decode step's pairs of token and expert): the tiles above would walk K in steps
// of 16 behind a barrier each for a handful of live rows.  Here a CTA takes one tile of the layout and 16 (gated)
// or 32 output columns; a warp reads its four weight rows once, 16 bytes a lane where the rows allow it, for up
// to GF_ROWS live rows of the tile, whose inputs wait in shared memory in 32-bit; each row's sums close with a
// shuffle tree.  More live rows take further passes.  Rows whose source is -1 stay unwritten.
constexpr int GF_ROWS = 8;      // live rows a pass takes
constexpr int GF_KC = 1024;     // inputs of a row that wait in shared memory at a time
constexpr int GF_TILE_MAX = 128;

template <typename T> struct Vec16;
template <> struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float* v) {
    const float4 q = *reinterpret_cast<const float4*>(p);
    v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
  }
};
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) {
    const uint4 q = *reinterpret_cast<const uint4*>(p);
    const uint32_t u[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(u[i] << 16);
      v[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    }
  }
};

template <typename T, typename OutT, bool GATED>
__global__ void __launch_bounds__(256) gemm_grouped_few_kernel(OutT* __restrict__ out, const T* __restrict__ x,
                                                               const T* __restrict__ w, int M, int N, int K, int ldx,
                                                               int ldo, long long group_w,
                                                               const int* __restrict__ row_src, int row_div,
                                                               int gather, const int* __restrict__ tile_group,
                                                               int tile, int vec, float gate_limit) {
  __shared__ float xs[GF_ROWS][GF_KC];
  __shared__ int live_row[GF_TILE_MAX], live_x[GF_TILE_MAX];
  __shared__ int n_live_s;
  pdl_trigger();
  pdl_wait();
  const int group = tile_group[blockIdx.y];
  if (group < 0) return;
  w += (long long)group * group_w;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, m0 = blockIdx.y * tile;
  // the tile's live rows in their order: a thread a row, places from the warps' ballots
  __shared__ int warp_live[GF_TILE_MAX / 32];
  const int my_src = (tid < tile && m0 + tid < M) ? row_src[m0 + tid] : -1;
  const unsigned ballot = __ballot_sync(0xffffffffu, my_src >= 0);
  if (tid < GF_TILE_MAX && lane == 0) warp_live[warp] = __popc(ballot);
  __syncthreads();
  if (tid < GF_TILE_MAX) {
    int at = __popc(ballot & ((1u << lane) - 1u)), all = 0;
#pragma unroll
    for (int i = 0; i < GF_TILE_MAX / 32; ++i) {
      if (i < warp) at += warp_live[i];
      all += warp_live[i];
    }
    if (my_src >= 0) {
      live_row[at] = m0 + tid;
      live_x[at] = gather ? my_src / row_div : m0 + tid;
    }
    if (tid == 0) n_live_s = all;
  }
  __syncthreads();
  const int n_live = n_live_s;
  // the warp's four weight rows: gate and up of two neighbouring columns, or four neighbouring columns
  constexpr int NR = 4;
  const int n0 = (blockIdx.x * 8 + warp) * (GATED ? 2 : NR);
  int col[NR];
  const T* wrow[NR];
#pragma unroll
  for (int r = 0; r < NR; ++r) {
    col[r] = GATED ? n0 + (r >> 1) : n0 + r;
    const int c = col[r] < N ? col[r] : 0;        // a row beyond the last reads row 0; its sums are dropped
    wrow[r] = w + (size_t)(GATED && (r & 1) ? N + c : c) * K;
  }
  const bool any = n0 < N;
  for (int r0 = 0; r0 < n_live; r0 += GF_ROWS) {
    const int rows = min(GF_ROWS, n_live - r0);
    float acc[NR][GF_ROWS];
#pragma unroll
    for (int r = 0; r < NR; ++r)
#pragma unroll
      for (int t = 0; t < GF_ROWS; ++t) acc[r][t] = 0.f;
    for (int k0 = 0; k0 < K; k0 += GF_KC) {
      const int kc = min(GF_KC, K - k0);
      __syncthreads();      // whoever still read the inputs before is done
      for (int t = 0; t < rows; ++t) {
        const T* src = x + (size_t)live_x[r0 + t] * ldx + k0;
        for (int k = tid; k < kc; k += 256) xs[t][k] = to_f32<T>(src[k]);
      }
      __syncthreads();
      if (!any) continue;
      if (vec) {
        constexpr int V = Vec16<T>::N;
        for (int k = lane * V; k < kc; k += 32 * V) {
          float wv[NR][V];
#pragma unroll
          for (int r = 0; r < NR; ++r) Vec16<T>::load(wrow[r] + k0 + k, wv[r]);
#pragma unroll
          for (int t = 0; t < GF_ROWS; ++t) {
            if (t < rows) {
#pragma unroll
              for (int e = 0; e < V; ++e) {
                const float xv = xs[t][k + e];
#pragma unroll
                for (int r = 0; r < NR; ++r) acc[r][t] = fmaf(wv[r][e], xv, acc[r][t]);
              }
            }
          }
        }
      } else {
        for (int k = lane; k < kc; k += 32) {
          float wv[NR];
#pragma unroll
          for (int r = 0; r < NR; ++r) wv[r] = to_f32<T>(wrow[r][k0 + k]);
#pragma unroll
          for (int t = 0; t < GF_ROWS; ++t)
            if (t < rows) {
              const float xv = xs[t][k];
#pragma unroll
              for (int r = 0; r < NR; ++r) acc[r][t] = fmaf(wv[r], xv, acc[r][t]);
            }
        }
      }
    }
    if (!any) continue;
#pragma unroll
    for (int t = 0; t < GF_ROWS; ++t) {
      if (t >= rows) break;
      float v[NR];
#pragma unroll
      for (int r = 0; r < NR; ++r) v[r] = warp_sum(acc[r][t]);
      if (lane != 0) continue;
      OutT* dst = out + (size_t)live_row[r0 + t] * ldo;
      if (GATED) {
#pragma unroll
        for (int c = 0; c < NR / 2; ++c)
          if (col[2 * c] < N) dst[col[2 * c]] = from_f32<OutT>(gate_pair(v[2 * c], v[2 * c + 1], gate_limit));
      } else {
#pragma unroll
        for (int r = 0; r < NR; ++r)
          if (col[r] < N) dst[col[r]] = from_f32<OutT>(v[r]);
      }
    }
  }
}

template <typename T, typename OutT>
int launch_grouped_few(void* out, const void* x, const void* w, int M, int N, int K, int ldx, int ldo, int gated,
                       long long group_w, const int* row_src, int row_div, int gather, const int* tile_group, int tile,
                       cudaStream_t stream, float gate_limit) {
  constexpr int V = 16 / (int)sizeof(T);
  const int vec = K % V == 0 && ((uintptr_t)w & 15) == 0;
  const int cols = gated ? 16 : 32;      // 8 warps, four weight rows each
  dim3 grid((N + cols - 1) / cols, (M + tile - 1) / tile);
  if (gated)
    return (int)lab_launch(gemm_grouped_few_kernel<T, OutT, true>, grid, dim3(256), 0, stream, (OutT*)out, (const T*)x,
                           (const T*)w, M, N, K, ldx, ldo, group_w, row_src, row_div, gather, tile_group, tile, vec,
                           gate_limit);
  return (int)lab_launch(gemm_grouped_few_kernel<T, OutT, false>, grid, dim3(256), 0, stream, (OutT*)out, (const T*)x,
                         (const T*)w, M, N, K, ldx, ldo, group_w, row_src, row_div, gather, tile_group, tile, vec, 0.f);
}

template <typename T, typename OutT>
int launch(void* out, const void* x, const void* w, const void* bias, int M, int N, int K, int ldx, int ldo, int gated,
           cudaStream_t stream, int batch = 1, long long batch_x = 0, long long batch_w = 0, long long batch_o = 0,
           const int* row_src = nullptr, int row_div = 1, const int* tile_group = nullptr, float gate_limit = 0.f) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM, batch);
  if (gated == 1)
    return (int)lab_launch(gemm_plain_kernel<T, OutT, true>, grid, dim3(256), 0, stream, (OutT*)out, (const T*)x,
                           (const T*)w, (const T*)nullptr, M, N, K, ldx, ldo, batch_x, batch_w, batch_o, 0, row_src,
                           row_div, tile_group, gate_limit);
  return (int)lab_launch(gemm_plain_kernel<T, OutT, false>, grid, dim3(256), 0, stream, (OutT*)out, (const T*)x,
                         (const T*)w, (const T*)bias, M, N, K, ldx, ldo, batch_x, batch_w, batch_o,
                         gated >= 2 ? gated - 1 : 0, row_src, row_div, tile_group, 0.f);
}
}  // namespace

// N is the number of output columns; with gated == 1, w holds 2 N rows (gate rows, then up rows); gated == 2 is
// the plain product with GELU (tanh form) after the bias, 3 with the square of relu.
LAB_EXPORT int lab_gemm_plain(void* out, const void* x, const void* w, const void* bias, int M, int N, int K, int ldx,
                              int ldo, int gated, int dtype, int out_f32, float gate_limit, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (dtype == LAB_F32)
    return launch<float, float>(out, x, w, bias, M, N, K, ldx, ldo, gated, stream, 1, 0, 0, 0, nullptr, 1, nullptr, gate_limit);
  if (out_f32)
    return launch<__nv_bfloat16, float>(out, x, w, bias, M, N, K, ldx, ldo, gated, stream, 1, 0, 0, 0, nullptr, 1, nullptr,
                                        gate_limit);
  return launch<__nv_bfloat16, __nv_bfloat16>(out, x, w, bias, M, N, K, ldx, ldo, gated, stream, 1, 0, 0, 0, nullptr, 1,
                                              nullptr, gate_limit);
}

// `batch` products of one shape in one launch: out_b[m, n] = sum_k x_b[m, k] * w_b[n, k], operand b lying
// b * batch_* elements after operand 0 (heads side by side in a row: batch_x = the head's width).
LAB_EXPORT int lab_gemm_plain_batched(void* out, const void* x, const void* w, int M, int N, int K, int ldx, int ldo,
                                      int batch, long long batch_x, long long batch_w, long long batch_o, int dtype,
                                      int out_f32, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || batch <= 0) return 0;
  if (batch > 65535) return (int)cudaErrorInvalidValue;
  if (M <= HF_TOKENS && (size_t)M * K * sizeof(float) <= 48 * 1024 && batch_w == (long long)N * K) {
    if (dtype == LAB_F32)
      return launch_heads_few<float, float>(out, x, w, M, N, K, ldx, ldo, batch, batch_x, batch_o, stream);
    if (out_f32)
      return launch_heads_few<__nv_bfloat16, float>(out, x, w, M, N, K, ldx, ldo, batch, batch_x, batch_o, stream);
    return launch_heads_few<__nv_bfloat16, __nv_bfloat16>(out, x, w, M, N, K, ldx, ldo, batch, batch_x, batch_o, stream);
  }
  if (dtype == LAB_F32)
    return launch<float, float>(out, x, w, nullptr, M, N, K, ldx, ldo, 0, stream, batch, batch_x, batch_w, batch_o);
  if (out_f32)
    return launch<__nv_bfloat16, float>(out, x, w, nullptr, M, N, K, ldx, ldo, 0, stream, batch, batch_x, batch_w,
                                        batch_o);
  return launch<__nv_bfloat16, __nv_bfloat16>(out, x, w, nullptr, M, N, K, ldx, ldo, 0, stream, batch, batch_x, batch_w,
                                              batch_o);
}

// Rows grouped by the matrix they meet (routed experts): tile t of lab_gemm_plain_group_rows() rows meets the
// matrix tile_group[t] of `w` (matrices group_w elements apart; -1: the tile holds no rows and is skipped); row m of
// the product reads x's row row_src[m] / row_div (row_src null: row m itself; -1: padding, read as zeros).
// M counts the rows of the grouped layout (out has that many); x must hold every row that row_src names.
LAB_EXPORT int lab_gemm_plain_group_rows() { return BM; }
LAB_EXPORT int lab_gemm_plain_grouped(void* out, const void* x, const void* w, int M, int N, int K, int ldx, int ldo,
                                      int gated, long long group_w, const int* row_src, int row_div,
                                      const int* tile_group, int dtype, int out_f32, float gate_limit,
                                      cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (tile_group == nullptr || row_div < 1) return (int)cudaErrorInvalidValue;
  if (dtype == LAB_F32)
    return launch<float, float>(out, x, w, nullptr, M, N, K, ldx, ldo, gated, stream, 1, 0, group_w, 0, row_src, row_div,
                                tile_group, gate_limit);
  if (out_f32)
    return launch<__nv_bfloat16, float>(out, x, w, nullptr, M, N, K, ldx, ldo, gated, stream, 1, 0, group_w, 0, row_src,
                                        row_div, tile_group, gate_limit);
  return launch<__nv_bfloat16, __nv_bfloat16>(out, x, w, nullptr, M, N, K, ldx, ldo, gated, stream, 1, 0, group_w, 0,
                                              row_src, row_div, tile_group, gate_limit);
}

// The same product for few rows (a decode step): tile t of `tile` rows (at most 128) meets matrix tile_group[t];
// only rows whose row_src is not -1 are formed and written.  gather: row m reads x's row row_src[m] / row_div,
// else x's row m.
LAB_EXPORT int lab_gemm_plain_grouped_few(void* out, const void* x, const void* w, int M, int N, int K, int ldx,
                                          int ldo, int gated, long long group_w, const int* row_src, int row_div,
                                          int gather, const int* tile_group, int tile, int dtype, int out_f32,
                                          float gate_limit, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (tile_group == nullptr || row_src == nullptr || row_div < 1 || tile < 1 || tile > GF_TILE_MAX || K <= 0)
    return (int)cudaErrorInvalidValue;
  if ((M + tile - 1) / tile > 65535) return (int)cudaErrorInvalidValue;
  if (dtype == LAB_F32)
    return launch_grouped_few<float, float>(out, x, w, M, N, K, ldx, ldo, gated, group_w, row_src, row_div, gather,
                                            tile_group, tile, stream, gate_limit);
  if (out_f32)
    return launch_grouped_few<__nv_bfloat16, float>(out, x, w, M, N, K, ldx, ldo, gated, group_w, row_src, row_div,
                                                    gather, tile_group, tile, stream, gate_limit);
  return launch_grouped_few<__nv_bfloat16, __nv_bfloat16>(out, x, w, M, N, K, ldx, ldo, gated, group_w, row_src,
                                                          row_div, gather, tile_group, tile, stream, gate_limit);
}
