// A state-space mixer whose decay differs per channel and per entry of the state (selective scan):
//
//   S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n        A = -exp(A_log), dt = softplus(dt_pre + dt_bias)
//   y_c      = sum_n S[c, n] C_n + D_c x_c,   out_c = y_c * silu(z_c)
//
// x, z and dt_pre have one number per channel and token, B and C one per state entry and token (shared by
// all channels).  S [channels, N] per request is 32-bit, starts at zero and is carried from token to token;
// everything here is 32-bit, the output is rounded once for the output projection.
//
// Kernels: the causal convolution of x with the request's last inputs kept between steps (+ SiLU), and
// the walk.  The walk is sequential in tokens; a CTA takes 16 channels of one request, 8 lanes a channel,
// each lane a share of the state's entries in registers.  A chunk of tokens waits in shared memory while the
// next one arrives there (cp.async); step sizes are formed once per channel and token before the chunk is
// walked.  From token to token passes only the state's own update: every lane leaves its share of the sum
// over the state in shared memory, and the sums, the skip term and the gate are formed after the chunk, a
// thread per channel and token.
#include "common.cuh"

namespace {
constexpr int kThreads = 256;

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// ---- causal convolution over the last `taps` inputs of every channel, then SiLU -------------------
struct ConvParams {
  const float* proj;     // [tokens, ld]; the convolution's inputs at columns [conv_at, conv_at + channels)
  int ld, conv_at, channels, taps;
  float* kept;           // [slots, taps - 1, channels]: the request's last inputs, oldest first
  const int* row_req;
  const int* q_start;
  const int* state_slot;
  int n_slots;
};

// grid (rows, blocks of channels).  out32 [tokens, channels] floats; out_t the same rounded to T (or null).
template <typename T>
__global__ void __launch_bounds__(kThreads) conv_silu_kernel(float* __restrict__ out32, T* __restrict__ out_t,
                                                             const T* __restrict__ taps_w, const T* __restrict__ taps_b,
                                                             ConvParams p) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, r = p.row_req[t], first = p.q_start[r], slot = p.state_slot[r];
  const int K = p.taps, C = p.channels;
  const int c = blockIdx.y * kThreads + threadIdx.x;
  if (c >= C) return;
  if (slot == -1) {       // a row of padding
    out32[(size_t)t * C + c] = 0.f;
    if (out_t != nullptr) out_t[(size_t)t * C + c] = from_f32<T>(0.f);
    return;
  }
  if (slot < 0 || slot >= p.n_slots) {
    lab_set_error(LAB_ERR_PAGE_RANGE);
    return;
  }
  const float* kept = p.kept + (size_t)slot * (K - 1) * C;
  float acc = to_f32(taps_b[c]);
  for (int jj = 0; jj < K; ++jj) {
    const int src = t - (K - 1) + jj;       // the last tap meets the row itself
    const float u = src >= first ? p.proj[(size_t)src * p.ld + p.conv_at + c]
                                 : kept[(size_t)((K - 1) + (src - first)) * C + c];
    acc = fmaf(to_f32(taps_w[(size_t)c * K + jj]), u, acc);
  }
  const float v = silu_f(acc);
  out32[(size_t)t * C + c] = v;
  if (out_t != nullptr) out_t[(size_t)t * C + c] = from_f32<T>(v);
}

// grid (requests, blocks of channels), after every row of the step has read the kept inputs.  A thread walks
// the kept rows of its one channel oldest first: what it overwrites it has already moved.
__global__ void __launch_bounds__(kThreads) conv_keep_inputs_kernel(ConvParams p) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const int first = p.q_start[r], n = p.q_start[r + 1] - first, slot = p.state_slot[r];
  if (n <= 0 || slot == -1) return;
  if (slot < 0 || slot >= p.n_slots) {
    if (threadIdx.x == 0) lab_set_error(LAB_ERR_PAGE_RANGE);
    return;
  }
  const int K1 = p.taps - 1, C = p.channels;
  float* kept = p.kept + (size_t)slot * K1 * C;
  const int c = blockIdx.y * kThreads + threadIdx.x;
  if (c >= C) return;
  for (int i = 0; i < K1; ++i) {
    const int s = n - K1 + i;               // the step's row that becomes kept row i
    kept[(size_t)i * C + c] = s >= 0 ? p.proj[(size_t)(first + s) * p.ld + p.conv_at + c] : kept[(size_t)(i + n) * C + c];
  }
}

// ---- the walk ----------------------------------------------------------------------------------------
constexpr int WC = 16;        // channels a CTA takes
constexpr int WL = 8;         // lanes a channel: lane l holds the state entries l, l + 8, ...
constexpr int WT = 32;        // tokens a chunk
constexpr int WTHREADS = WC * WL;

struct ScanParams {
  const float* x;        // [tokens, ld_x] after the convolution and SiLU
  const float* dt_pre;   // [tokens, ld_dt] the step sizes before bias and softplus
  const float* bc;       // [tokens, ld_bc]: B at columns [b_at, b_at + N), C at [c_at, c_at + N)
  const float* z;        // [tokens, ld_z] the gate's input
  float* state;          // [slots, channels, N]
  const int* q_start;
  const int* state_slot;
  int ld_x, ld_dt, ld_bc, ld_z, b_at, c_at, channels, N, n_slots, write, ld_out;
};

// 4 bytes from global to shared memory without a register in between; waited for by cp_async_wait_all.
__device__ __forceinline__ void cp_async_f32(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src)
               : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }

// Floats of one chunk's inputs as they arrive: dt_pre, x, z [WT][WC] each, then B and C [WT][N] each.
__host__ __device__ inline int scan_chunk_floats(int N) { return 3 * WT * WC + 2 * WT * N; }

template <typename T, int R>
__global__ void __launch_bounds__(WTHREADS) selective_scan_kernel(T* __restrict__ out, const T* __restrict__ a_log,
                                                                  const T* __restrict__ skip,
                                                                  const T* __restrict__ dt_bias, ScanParams p) {
  extern __shared__ float smem[];
  const int N = p.N, chunk_floats = scan_chunk_floats(N);
  float* s_in = smem;                          // two chunks of inputs: one walked, one arriving
  float* s_dx = smem + 2 * chunk_floats;       // [WT][WC] step size times x
  float* s_part = s_dx + WT * WC;              // [WT][WC][WL] every lane's share of the sum over the state
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.y, c0 = blockIdx.x * WC;
  const int first = p.q_start[r], n = p.q_start[r + 1] - first, slot = p.state_slot[r];
  if (n <= 0) return;
  const int tid = threadIdx.x, ch = tid / WL, l = tid % WL, c = c0 + ch;
  const bool live = c < p.channels;
  if (slot == -1) {       // rows of padding leave zeros
    for (int i = tid; i < n * WC; i += WTHREADS)
      if (c0 + i % WC < p.channels) out[(size_t)(first + i / WC) * p.ld_out + c0 + i % WC] = from_f32<T>(0.f);
    return;
  }
  if (slot < 0 || slot >= p.n_slots) {
    if (tid == 0) lab_set_error(LAB_ERR_PAGE_RANGE);
    return;
  }
  // a chunk's inputs set out for shared memory; channels beyond the last read nothing and stay unused
  auto fetch = [&](int t0, float* buf) {
    const int nt = min(WT, n - t0);
    float *b_dt = buf, *b_x = buf + WT * WC, *b_z = buf + 2 * WT * WC, *b_b = buf + 3 * WT * WC, *b_c = b_b + WT * N;
    for (int i = tid; i < nt * WC; i += WTHREADS) {
      const int cc = c0 + i % WC;
      if (cc >= p.channels) continue;
      const size_t row = (size_t)(first + t0 + i / WC);
      cp_async_f32(b_dt + i, p.dt_pre + row * p.ld_dt + cc);
      cp_async_f32(b_x + i, p.x + row * p.ld_x + cc);
      cp_async_f32(b_z + i, p.z + row * p.ld_z + cc);
    }
    for (int i = tid; i < nt * N; i += WTHREADS) {
      const float* row = p.bc + (size_t)(first + t0 + i / N) * p.ld_bc + i % N;
      cp_async_f32(b_b + i, row + p.b_at);
      cp_async_f32(b_c + i, row + p.c_at);
    }
  };
  fetch(0, s_in);
  float S[R], A[R];
  float* st = p.state + ((size_t)slot * p.channels + (live ? c : 0)) * N;
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int e = i * WL + l;
    const bool has = live && e < N;
    S[i] = has ? st[e] : 0.f;
    A[i] = has ? -expf(to_f32(a_log[(size_t)c * N + e])) : 0.f;
  }
  int which = 0;
  for (int t0 = 0; t0 < n; t0 += WT, which ^= 1) {
    const int nt = min(WT, n - t0);
    float* buf = s_in + which * chunk_floats;
    float *b_dt = buf, *b_x = buf + WT * WC, *b_z = buf + 2 * WT * WC, *b_b = buf + 3 * WT * WC, *b_c = b_b + WT * N;
    cp_async_wait_all();
    __syncthreads();       // the chunk is here; the chunk before has been written out, its buffer is free
    if (t0 + WT < n) fetch(t0 + WT, s_in + (which ^ 1) * chunk_floats);
    // step sizes once per channel and token
    for (int i = tid; i < nt * WC; i += WTHREADS) {
      const int cc = c0 + i % WC;
      float dt = 0.f, dx = 0.f;
      if (cc < p.channels) {
        dt = softplus_f(b_dt[i] + to_f32(dt_bias[cc]));
        dx = dt * b_x[i];
      }
      b_dt[i] = dt;
      s_dx[i] = dx;
    }
    __syncthreads();
    // the walk: nothing but the state's own update passes from token to token
#pragma unroll 4
    for (int tt = 0; tt < nt; ++tt) {
      const float dt = b_dt[tt * WC + ch], dx = s_dx[tt * WC + ch];
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < R; ++i) {
        const int e = i * WL + l;
        if (e < N) {
          // expf, not a power of two with A scaled: a slow decay's error of one more unit in the last place
          // comes with the same sign at every token and adds up over the state's memory
          S[i] = fmaf(expf(dt * A[i]), S[i], dx * b_b[tt * N + e]);
          acc = fmaf(S[i], b_c[tt * N + e], acc);
        }
      }
      s_part[tt * WTHREADS + tid] = acc;
    }
    __syncthreads();
    // the sum over the lanes (in their order), the skip term and the gate, a thread per channel and token
    for (int i = tid; i < nt * WC; i += WTHREADS) {
      const int cc = c0 + i % WC;
      if (cc >= p.channels) continue;
      const float4 lo = *reinterpret_cast<const float4*>(s_part + (size_t)i * WL);
      const float4 hi = *reinterpret_cast<const float4*>(s_part + (size_t)i * WL + 4);
      const float acc = ((lo.x + hi.x) + (lo.z + hi.z)) + ((lo.y + hi.y) + (lo.w + hi.w));
      out[(size_t)(first + t0 + i / WC) * p.ld_out + cc] =
          from_f32<T>(fmaf(to_f32(skip[cc]), b_x[i], acc) * silu_f(b_z[i]));
    }
  }
  if (p.write && live) {
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int e = i * WL + l;
      if (e < N) st[e] = S[i];
    }
  }
}

template <typename T, int R>
int launch_scan(void* out, const void* a_log, const void* skip, const void* dt_bias, const ScanParams& p, int requests,
                cudaStream_t stream) {
  const size_t smem = sizeof(float) * ((size_t)2 * scan_chunk_floats(p.N) + (size_t)WT * WC + (size_t)WT * WC * WL);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(selective_scan_kernel<T, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return (int)lab_launch(selective_scan_kernel<T, R>, dim3((p.channels + WC - 1) / WC, requests), dim3(WTHREADS), smem,
                         stream, (T*)out, (const T*)a_log, (const T*)skip, (const T*)dt_bias, p);
}

template <typename T>
int pick_scan(void* out, const void* a_log, const void* skip, const void* dt_bias, const ScanParams& p, int requests,
              cudaStream_t stream) {
  const int per_lane = (p.N + WL - 1) / WL;
  if (per_lane <= 1) return launch_scan<T, 1>(out, a_log, skip, dt_bias, p, requests, stream);
  if (per_lane <= 2) return launch_scan<T, 2>(out, a_log, skip, dt_bias, p, requests, stream);
  if (per_lane <= 3) return launch_scan<T, 3>(out, a_log, skip, dt_bias, p, requests, stream);
  if (per_lane <= 4) return launch_scan<T, 4>(out, a_log, skip, dt_bias, p, requests, stream);
  if (per_lane <= 8) return launch_scan<T, 8>(out, a_log, skip, dt_bias, p, requests, stream);
  if (per_lane <= 16) return launch_scan<T, 16>(out, a_log, skip, dt_bias, p, requests, stream);
  if (per_lane <= 32) return launch_scan<T, 32>(out, a_log, skip, dt_bias, p, requests, stream);
  return (int)cudaErrorInvalidValue;
}
}  // namespace

// The largest state (entries per channel) the walk takes.
LAB_EXPORT int lab_selective_scan_max_state() { return 32 * WL; }

LAB_EXPORT int lab_conv_silu(float* out32, void* out_t, const float* proj, int ld, int conv_at, int channels, int taps,
                             const void* taps_w, const void* taps_b, float* kept, const int* row_req,
                             const int* q_start, const int* state_slot, int tokens, int requests, int n_slots,
                             int write, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (taps < 1 || channels <= 0) return (int)cudaErrorInvalidValue;
  ConvParams p;
  p.proj = proj; p.ld = ld; p.conv_at = conv_at; p.channels = channels; p.taps = taps; p.kept = kept;
  p.row_req = row_req; p.q_start = q_start; p.state_slot = state_slot; p.n_slots = n_slots;
  const int c_blocks = (channels + kThreads - 1) / kThreads;
  if (c_blocks > 65535) return (int)cudaErrorInvalidValue;
  cudaError_t e;
  if (dtype == LAB_F32)
    e = lab_launch(conv_silu_kernel<float>, dim3(tokens, c_blocks), dim3(kThreads), 0, stream, out32, (float*)nullptr,
                   (const float*)taps_w, (const float*)taps_b, p);
  else
    e = lab_launch(conv_silu_kernel<__nv_bfloat16>, dim3(tokens, c_blocks), dim3(kThreads), 0, stream, out32,
                   (__nv_bfloat16*)out_t, (const __nv_bfloat16*)taps_w, (const __nv_bfloat16*)taps_b, p);
  if (e != cudaSuccess) return (int)e;
  if (write && taps > 1)
    return (int)lab_launch(conv_keep_inputs_kernel, dim3(requests, c_blocks), dim3(kThreads), 0, stream, p);
  return 0;
}

LAB_EXPORT int lab_selective_scan(void* out, int ld_out, const float* x, int ld_x, const float* dt_pre, int ld_dt,
                                  const float* bc, int ld_bc, int b_at, int c_at, const float* z, int ld_z,
                                  const void* a_log, const void* skip, const void* dt_bias, float* state,
                                  const int* q_start, const int* state_slot, int requests, int channels, int N,
                                  int n_slots, int write, int dtype, cudaStream_t stream) {
  if (requests <= 0) return 0;
  if (channels <= 0 || N <= 0 || N > 32 * WL) return (int)cudaErrorInvalidValue;
  ScanParams p;
  p.x = x; p.dt_pre = dt_pre; p.bc = bc; p.z = z; p.state = state; p.q_start = q_start; p.state_slot = state_slot;
  p.ld_x = ld_x; p.ld_dt = ld_dt; p.ld_bc = ld_bc; p.ld_z = ld_z; p.b_at = b_at; p.c_at = c_at; p.channels = channels;
  p.N = N; p.n_slots = n_slots; p.write = write; p.ld_out = ld_out;
  if (requests > 65535) return (int)cudaErrorInvalidValue;
  if (dtype == LAB_F32) return pick_scan<float>(out, a_log, skip, dt_bias, p, requests, stream);
  return pick_scan<__nv_bfloat16>(out, a_log, skip, dt_bias, p, requests, stream);
}
