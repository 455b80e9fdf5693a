// A residual made of several streams (hyper-connections), kept in 32-bit floats whatever the storage type T:
// X [tokens, S, hidden].  A sublayer reads one mix of the streams and writes back into all of them:
//
//     u      = sum_s c_in[s] X[s]                      what the sublayer's norm reads
//     h      = u / rms(u) * w                          w one number for all coordinates, or one per coordinate
//     X'[r]  = sum_s mix[s, r] X[s] + c_out[r] * y     all streams at once from the old ones; y the sublayer's result
//
//   hyper_expand      X[t, s] = x[t] for every s (the streams start as copies of the embedding output)
//   hyper_read_norm   h of all rows, or of gathered rows (the model's last norm reads the plain sum: c_in null)
//   hyper_write       X <- X' with y a 32-bit product or split-K partial products summed in ascending order;
//                     with c_in / w of the next sublayer also that sublayer's h, in the same pass
//   normed_sum        y = sum_i c_i * a_i / rms(a_i) * w_i over one or two products (whole or partial), 32-bit:
//                     the result of mixers that run side by side and are normed before their sum
//   scale_rows        logits <- logits * c
//
// The coefficients are 32-bit.  S is at most kMaxStreams.
#include "common.cuh"

namespace {
constexpr int kThreads = 256;
constexpr int kMaxStreams = 8;

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

__global__ void __launch_bounds__(kThreads) hyper_expand_kernel(float* __restrict__ X, const float* __restrict__ x,
                                                                int S, int hidden) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < hidden; i += kThreads) {
    const float v = x[(size_t)t * hidden + i];
    for (int s = 0; s < S; ++s) X[((size_t)t * S + s) * hidden + i] = v;
  }
}

struct HyperCoef {
  float c_in[kMaxStreams];                  // of the sublayer that reads next
  float c_out[kMaxStreams];
  float mix[kMaxStreams * kMaxStreams];     // [from, to]
};

// the norm's weight at coordinate i: one number for all, or one each
template <typename T>
__device__ __forceinline__ float weight_at(const T* __restrict__ w, int scalar, int i) {
  return to_f32(w[scalar ? 0 : i]);
}

template <typename T>
__global__ void __launch_bounds__(kThreads) hyper_read_norm_kernel(T* __restrict__ out, const float* __restrict__ X,
                                                                   const float* __restrict__ c_in,
                                                                   const T* __restrict__ w, int w_scalar,
                                                                   const int* __restrict__ rows, int n_in, int S,
                                                                   int hidden, float eps) {
  extern __shared__ float row[];      // [hidden]
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  int t = blockIdx.x;
  if (rows != nullptr) {
    t = rows[blockIdx.x];
    if (t < 0 || t >= n_in) {
      if (threadIdx.x == 0) lab_set_error(LAB_ERR_ROW_RANGE);
      t = min(max(t, 0), n_in - 1);
    }
  }
  const float* x = X + (size_t)t * S * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += kThreads) {
    float u = 0.f;
    for (int s = 0; s < S; ++s) u = fmaf(c_in != nullptr ? c_in[s] : 1.f, x[(size_t)s * hidden + i], u);
    row[i] = u;
    ss += u * u;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += kThreads)
    out[(size_t)blockIdx.x * hidden + i] = from_f32<T>(row[i] * inv * weight_at(w, w_scalar, i));
}

// SMAX bounds the streams the instance serves (2, 4 or kMaxStreams): the loops over streams unroll to it, and the
// instances for few streams keep few registers, so that more rows are in flight on an SM.
template <typename T, int SMAX>
__global__ void __launch_bounds__(kThreads, SMAX <= 4 ? 5 : 3) hyper_write_kernel(float* __restrict__ X, T* __restrict__ out,
                                                               const float* __restrict__ y, int y_splits,
                                                               long long split_stride, const float* __restrict__ mix,
                                                               const float* __restrict__ c_out,
                                                               const float* __restrict__ c_in_next,
                                                               const T* __restrict__ w_next, int w_scalar, int S,
                                                               int hidden, float eps) {
  extern __shared__ float row[];      // [hidden]: the next sublayer's u
  __shared__ float scratch[32];
  __shared__ HyperCoef coef;
  pdl_trigger();
  for (int i = threadIdx.x; i < S * S; i += kThreads) coef.mix[i] = mix[i];
  for (int i = threadIdx.x; i < S; i += kThreads) {
    coef.c_out[i] = c_out[i];
    coef.c_in[i] = c_in_next != nullptr ? c_in_next[i] : 0.f;
  }
  pdl_wait();
  __syncthreads();
  const int t = blockIdx.x;
  float* x = X + (size_t)t * S * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += kThreads) {
    const float yi = sum_splits(y, y_splits, split_stride, (size_t)t * hidden + i);
    float old[SMAX];
#pragma unroll
    for (int s = 0; s < SMAX; ++s) old[s] = s < S ? x[(size_t)s * hidden + i] : 0.f;
    float u = 0.f;
#pragma unroll
    for (int r = 0; r < SMAX; ++r) {
      if (r >= S) break;
      float v = 0.f;
#pragma unroll
      for (int s = 0; s < SMAX; ++s)
        if (s < S) v = fmaf(coef.mix[s * S + r], old[s], v);
      v = fmaf(coef.c_out[r], yi, v);
      x[(size_t)r * hidden + i] = v;
      u = fmaf(coef.c_in[r], v, u);
    }
    if (out != nullptr) {
      row[i] = u;
      ss += u * u;
    }
  }
  if (out == nullptr) return;
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += kThreads)
    out[(size_t)t * hidden + i] = from_f32<T>(row[i] * inv * weight_at(w_next, w_scalar, i));
}

template <typename T>
__global__ void __launch_bounds__(kThreads) normed_sum_kernel(float* __restrict__ out, const float* __restrict__ a,
                                                              int a_splits, const T* __restrict__ wa, float ca,
                                                              const float* __restrict__ b, int b_splits,
                                                              const T* __restrict__ wb, float cb,
                                                              long long split_stride, int hidden, float eps) {
  extern __shared__ float rows[];      // [2][hidden]
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  float sa = 0.f, sb = 0.f;
  for (int i = threadIdx.x; i < hidden; i += kThreads) {
    const float va = sum_splits(a, a_splits, split_stride, (size_t)t * hidden + i);
    rows[i] = va;
    sa += va * va;
    if (b != nullptr) {
      const float vb = sum_splits(b, b_splits, split_stride, (size_t)t * hidden + i);
      rows[hidden + i] = vb;
      sb += vb * vb;
    }
  }
  sa = block_sum(sa, scratch);
  const float ia = 1.0f / sqrtf(sa / (float)hidden + eps);
  float ib = 0.f;
  if (b != nullptr) {
    sb = block_sum(sb, scratch);
    ib = 1.0f / sqrtf(sb / (float)hidden + eps);
  }
  for (int i = threadIdx.x; i < hidden; i += kThreads) {
    float v = ca * (rows[i] * ia * to_f32(wa[i]));
    if (b != nullptr) v += cb * (rows[hidden + i] * ib * to_f32(wb[i]));
    out[(size_t)t * hidden + i] = v;
  }
}

__global__ void __launch_bounds__(kThreads) scale_rows_kernel(float* __restrict__ x, long long n, float c) {
  pdl_trigger();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * kThreads + threadIdx.x; i < n; i += (long long)gridDim.x * kThreads)
    x[i] *= c;
}

template <typename K>
void allow_smem(K kernel, size_t smem) {
  if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
}

template <typename T, int SMAX>
int launch_write(float* X, void* out, const float* y, int y_splits, const float* mix, const float* c_out,
                 const float* c_in_next, const void* w_next, int w_scalar, int tokens, int S, int hidden, float eps,
                 cudaStream_t stream) {
  const size_t smem = (size_t)hidden * sizeof(float);
  allow_smem(hyper_write_kernel<T, SMAX>, smem);
  return (int)lab_launch(hyper_write_kernel<T, SMAX>, dim3(tokens), dim3(kThreads), smem, stream, X, (T*)out, y, y_splits,
                         (long long)tokens * hidden, mix, c_out, c_in_next, (const T*)w_next, w_scalar, S, hidden, eps);
}

template <typename T>
int launch_write_for(int S, float* X, void* out, const float* y, int y_splits, const float* mix, const float* c_out,
                     const float* c_in_next, const void* w_next, int w_scalar, int tokens, int hidden, float eps,
                     cudaStream_t stream) {
  if (S <= 2)
    return launch_write<T, 2>(X, out, y, y_splits, mix, c_out, c_in_next, w_next, w_scalar, tokens, S, hidden, eps, stream);
  if (S <= 4)
    return launch_write<T, 4>(X, out, y, y_splits, mix, c_out, c_in_next, w_next, w_scalar, tokens, S, hidden, eps, stream);
  return launch_write<T, kMaxStreams>(X, out, y, y_splits, mix, c_out, c_in_next, w_next, w_scalar, tokens, S, hidden, eps,
                                      stream);
}
}  // namespace

LAB_EXPORT int lab_hyper_max_streams() { return kMaxStreams; }

LAB_EXPORT int lab_hyper_expand(float* X, const float* x, int tokens, int S, int hidden, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (S < 1 || S > kMaxStreams) return (int)cudaErrorInvalidValue;
  lab_launch(hyper_expand_kernel, dim3(tokens), dim3(kThreads), 0, stream, X, x, S, hidden);
  LAB_LAUNCH_CHECK();
}

LAB_EXPORT int lab_hyper_read_norm(void* out, const float* X, const float* c_in, const void* w, int w_scalar,
                                   const int* rows, int n_out, int n_in, int S, int hidden, float eps, int dtype,
                                   cudaStream_t stream) {
  if (n_out <= 0) return 0;
  const size_t smem = (size_t)hidden * sizeof(float);
  if (S < 1 || S > kMaxStreams || smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  if (dtype == LAB_F32) {
    allow_smem(hyper_read_norm_kernel<float>, smem);
    lab_launch(hyper_read_norm_kernel<float>, dim3(n_out), dim3(kThreads), smem, stream, (float*)out, X, c_in,
               (const float*)w, w_scalar, rows, n_in, S, hidden, eps);
  } else {
    allow_smem(hyper_read_norm_kernel<__nv_bfloat16>, smem);
    lab_launch(hyper_read_norm_kernel<__nv_bfloat16>, dim3(n_out), dim3(kThreads), smem, stream, (__nv_bfloat16*)out, X,
               c_in, (const __nv_bfloat16*)w, w_scalar, rows, n_in, S, hidden, eps);
  }
  LAB_LAUNCH_CHECK();
}

// out / c_in_next / w_next null: the write alone.
LAB_EXPORT int lab_hyper_write(float* X, void* out, const float* y, int y_splits, const float* mix, const float* c_out,
                               const float* c_in_next, const void* w_next, int w_scalar, int tokens, int S, int hidden,
                               float eps, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  const size_t smem = (size_t)hidden * sizeof(float);
  if (S < 1 || S > kMaxStreams || smem > 200 * 1024 || y_splits < 1) return (int)cudaErrorInvalidValue;
  if (dtype == LAB_F32)
    return launch_write_for<float>(S, X, out, y, y_splits, mix, c_out, c_in_next, w_next, w_scalar, tokens, hidden, eps,
                                   stream);
  return launch_write_for<__nv_bfloat16>(S, X, out, y, y_splits, mix, c_out, c_in_next, w_next, w_scalar, tokens, hidden,
                                         eps, stream);
}

LAB_EXPORT int lab_normed_sum(float* out, const float* a, int a_splits, const void* wa, float ca, const float* b,
                              int b_splits, const void* wb, float cb, int tokens, int hidden, float eps, int dtype,
                              cudaStream_t stream) {
  if (tokens <= 0) return 0;
  const size_t smem = (size_t)2 * hidden * sizeof(float);
  if (smem > 200 * 1024 || a_splits < 1 || (b != nullptr && b_splits < 1)) return (int)cudaErrorInvalidValue;
  const long long stride = (long long)tokens * hidden;
  if (dtype == LAB_F32) {
    allow_smem(normed_sum_kernel<float>, smem);
    lab_launch(normed_sum_kernel<float>, dim3(tokens), dim3(kThreads), smem, stream, out, a, a_splits, (const float*)wa,
               ca, b, b_splits, (const float*)wb, cb, stride, hidden, eps);
  } else {
    allow_smem(normed_sum_kernel<__nv_bfloat16>, smem);
    lab_launch(normed_sum_kernel<__nv_bfloat16>, dim3(tokens), dim3(kThreads), smem, stream, out, a, a_splits,
               (const __nv_bfloat16*)wa, ca, b, b_splits, (const __nv_bfloat16*)wb, cb, stride, hidden, eps);
  }
  LAB_LAUNCH_CHECK();
}

LAB_EXPORT int lab_scale_rows(float* x, long long n, float c, cudaStream_t stream) {
  if (n <= 0) return 0;
  const long long blocks = (n + kThreads - 1) / kThreads;
  lab_launch(scale_rows_kernel, dim3((int)(blocks < 148 * 8 ? blocks : 148 * 8)), dim3(kThreads), 0, stream, x, n, c);
  LAB_LAUNCH_CHECK();
}
