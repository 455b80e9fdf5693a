// A matrix memory with exponential gates (the mLSTM cell), around the framework's recurrence kernel.
// Per head, with log input gate i_t, log forget gate f_t and a running maximum m (m_0 = 0):
//
//     m_t = max(f_t + m_{t-1}, i_t)
//     S_t = exp(f_t + m_{t-1} - m_t) S_{t-1} + exp(i_t - m_t) k_t v_t^T          S [keys, values]
//     n_t = exp(f_t + m_{t-1} - m_t) n_{t-1} + exp(i_t - m_t) k_t
//     o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + floor)
//
// n rides along as one more column of S: the values get a column of ones (and zeros up to `vpad` columns a
// head, which keeps rows 16-byte aligned), so the recurrence S <- a S + (s k) v^T, o = S^T q of
// `decay_scan` forms S^T q and n . q together.  Here:
//
//   memory_gates      per row, parallel: i = cap tanh((z_i + b_i) / cap), f = logsigmoid(cap tanh((z_f + b_f) / cap));
//                     the values copied with their column of ones
//   memory_stabilize  per request and head, over the step's rows in order: m, the decay a_t and the key scale
//                     s_t of every row; m of the request's last row goes back to its state slot
//   memory_finish     per row: o_t with q's scale, each head over its root mean square, the weight, the sigmoid
//                     gate, rounded to T for the output projection; zeros for rows of padding (state slot -1)
//
// All of it is 32-bit; T says how the weights are stored and how the last result is rounded.
#include "common.cuh"

namespace {
constexpr int kThreads = 256;

__device__ __forceinline__ float log_sigmoid_f(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

struct GateParams {
  const float* proj;      // [tokens, ld]
  int ld, v_at, i_at, f_at;
  int H, V, vpad;
  float cap;
};

template <typename T>
__global__ void __launch_bounds__(kThreads) memory_gates_kernel(float* __restrict__ gates, float* __restrict__ v_out,
                                                                const T* __restrict__ b_i, const T* __restrict__ b_f,
                                                                GateParams p) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const float* row = p.proj + (size_t)t * p.ld;
  for (int h = threadIdx.x; h < p.H; h += kThreads) {
    const float zi = row[p.i_at + h] + to_f32(b_i[h]), zf = row[p.f_at + h] + to_f32(b_f[h]);
    gates[((size_t)t * 2) * p.H + h] = p.cap * tanhf(zi / p.cap);
    gates[((size_t)t * 2 + 1) * p.H + h] = log_sigmoid_f(p.cap * tanhf(zf / p.cap));
  }
  const int W = p.H * p.vpad;
  for (int i = threadIdx.x; i < W; i += kThreads) {
    const int h = i / p.vpad, e = i - h * p.vpad;
    v_out[(size_t)t * W + i] = e < p.V ? row[p.v_at + h * p.V + e] : (e == p.V ? 1.f : 0.f);
  }
}

// One warp per (request, head) walks the request's rows 32 at a time: every lane loads one row's gates, all lanes
// follow the chain m <- max(f + m, i) through the 32 rows (the same operations in the same order as a walk row
// by row, so a row's m does not depend on how the sequence was cut), each lane keeps the m before and after its
// own row and forms that row's two exponentials.
// decay[t, h] and scale[t, h] leave as rows of [tokens, 2, H] (over the gates).
__global__ void __launch_bounds__(kThreads) memory_stabilize_kernel(float* __restrict__ gates, float* __restrict__ m_out,
                                                                    float* __restrict__ m_state,
                                                                    const int* __restrict__ q_start,
                                                                    const int* __restrict__ state_slot, int requests,
                                                                    int n_slots, int H, int write) {
  __shared__ __align__(16) float chunk_gates[kThreads / 32][64];      // per warp: 32 forget gates, then 32 input gates
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pair = blockIdx.x * (kThreads / 32) + warp;
  if (pair >= requests * H) return;
  const int r = pair / H, h = pair - r * H;
  const int t0 = q_start[r], n = q_start[r + 1] - t0, slot = state_slot[r];
  if (n <= 0 || slot == -1) return;
  if (slot < 0 || slot >= n_slots) {
    if (lane == 0) lab_set_error(LAB_ERR_PAGE_RANGE);
    return;
  }
  // Lanes beyond the request's rows hold (f, i) = (0, -inf), which leaves m as it is: every chunk walks all 32
  // lanes, so the chain unrolls and its shuffles are issued ahead of it.  Rows come in groups of kAhead chunks:
  // the next group's gates are loaded before the current group's chains, which hides the loads' latency.
  constexpr int kAhead = 4;
  float* mine = chunk_gates[warp];
  float m = m_state[(size_t)slot * H + h];
  float gi[kAhead], gf[kAhead], gi_next[kAhead], gf_next[kAhead];
  auto load = [&](int first, float (&to_i)[kAhead], float (&to_f)[kAhead]) {
#pragma unroll
    for (int k = 0; k < kAhead; ++k) {
      const int row = first + k * 32 + lane;
      const bool in = row < n;
      to_i[k] = in ? gates[(size_t)(t0 + row) * 2 * H + h] : -INFINITY;
      to_f[k] = in ? gates[(size_t)(t0 + row) * 2 * H + H + h] : 0.f;
    }
  };
  load(0, gi, gf);
  for (int c = 0; c < n; c += kAhead * 32) {
    load(c + kAhead * 32, gi_next, gf_next);
#pragma unroll
    for (int k = 0; k < kAhead; ++k) {
      // the chunk's gates go through shared memory: every lane reads all 32 pairs, four at a time, ahead of the
      // chain (shuffles would put their latency on it)
      __syncwarp();
      mine[lane] = gf[k];
      mine[32 + lane] = gi[k];
      __syncwarp();
      float carried_mine = 0.f, m_mine = 0.f;
#pragma unroll
      for (int j4 = 0; j4 < 8; ++j4) {
        const float4 f4 = reinterpret_cast<const float4*>(mine)[j4];
        const float4 i4 = reinterpret_cast<const float4*>(mine + 32)[j4];
        const float fs[4] = {f4.x, f4.y, f4.z, f4.w}, is[4] = {i4.x, i4.y, i4.z, i4.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float carried = fs[e] + m;
          m = fmaxf(carried, is[e]);
          if (4 * j4 + e == lane) carried_mine = carried, m_mine = m;
        }
      }
      const int row = c + k * 32 + lane;
      if (row < n) {
        float* g = gates + (size_t)(t0 + row) * 2 * H;
        g[h] = expf(carried_mine - m_mine);       // decay of the state
        g[H + h] = expf(gi[k] - m_mine);          // scale of the new key
        m_out[(size_t)(t0 + row) * H + h] = m_mine;
      }
    }
#pragma unroll
    for (int k = 0; k < kAhead; ++k) gi[k] = gi_next[k], gf[k] = gf_next[k];
  }
  if (write && lane == 0) m_state[(size_t)slot * H + h] = m;
}

// One warp per (row, head).
template <typename T>
__global__ void __launch_bounds__(kThreads) memory_finish_kernel(T* __restrict__ out, int ld_out,
                                                                 const float* __restrict__ o, const float* __restrict__ m,
                                                                 const float* __restrict__ gate, int ld_g,
                                                                 const T* __restrict__ w, int tokens, int H, int V,
                                                                 int vpad, float q_scale, float floor_, float eps,
                                                                 float mult, const int* __restrict__ row_req,
                                                                 const int* __restrict__ state_slot) {
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long pair = (long long)blockIdx.x * (kThreads / 32) + warp;
  if (pair >= (long long)tokens * H) return;
  const int t = (int)(pair / H), h = (int)(pair - (long long)t * H);
  if (state_slot[row_req[t]] == -1) {      // a row of padding: the recurrence left nothing for it
    for (int e = lane; e < V; e += 32) out[(size_t)t * ld_out + h * V + e] = from_f32<T>(0.f);
    return;
  }
  const float* oh = o + ((size_t)t * H + h) * vpad;
  const float nq = oh[V] * q_scale;
  const float den = fmaxf(fabsf(nq), expf(-m[(size_t)t * H + h])) + floor_;
  float ss = 0.f;
  for (int e = lane; e < V; e += 32) {
    const float y = oh[e] * q_scale / den;
    ss += y * y;
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)V + eps);
  for (int e = lane; e < V; e += 32) {
    const int c = h * V + e;
    const float y = oh[e] * q_scale / den * inv * to_f32(w[c]);
    const float gz = gate[(size_t)t * ld_g + c];
    out[(size_t)t * ld_out + c] = from_f32<T>(y / (1.f + expf(-gz)) * mult);
  }
}
}  // namespace

// gates [tokens, 2, H] (log input gate, log forget gate), v_out [tokens, H * vpad].
LAB_EXPORT int lab_memory_gates(float* gates, float* v_out, const float* proj, int ld, int v_at, int i_at, int f_at,
                                const void* b_i, const void* b_f, int tokens, int H, int V, int vpad, float cap, int dtype,
                                cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (H <= 0 || V <= 0 || vpad <= V || !(cap > 0.f)) return (int)cudaErrorInvalidValue;
  GateParams p;
  p.proj = proj; p.ld = ld; p.v_at = v_at; p.i_at = i_at; p.f_at = f_at; p.H = H; p.V = V; p.vpad = vpad; p.cap = cap;
  if (dtype == LAB_F32)
    lab_launch(memory_gates_kernel<float>, dim3(tokens), dim3(kThreads), 0, stream, gates, v_out, (const float*)b_i,
               (const float*)b_f, p);
  else
    lab_launch(memory_gates_kernel<__nv_bfloat16>, dim3(tokens), dim3(kThreads), 0, stream, gates, v_out,
               (const __nv_bfloat16*)b_i, (const __nv_bfloat16*)b_f, p);
  LAB_LAUNCH_CHECK();
}

// gates [tokens, 2, H]: in, the log gates; out, the decay and the key's scale of every row.  m_out [tokens, H].
LAB_EXPORT int lab_memory_stabilize(float* gates, float* m_out, float* m_state, const int* q_start, const int* state_slot,
                                    int requests, int n_slots, int H, int write, cudaStream_t stream) {
  if (requests <= 0) return 0;
  const int warps = kThreads / 32;
  lab_launch(memory_stabilize_kernel, dim3((requests * H + warps - 1) / warps), dim3(kThreads), 0, stream, gates, m_out,
             m_state, q_start, state_slot, requests, n_slots, H, write);
  LAB_LAUNCH_CHECK();
}

LAB_EXPORT int lab_memory_finish(void* out, int ld_out, const float* o, const float* m, const float* gate, int ld_g,
                                 const void* w, int tokens, int H, int V, int vpad, float q_scale, float floor_, float eps,
                                 float mult, const int* row_req, const int* state_slot, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  const long long pairs = (long long)tokens * H;
  const int blocks = (int)((pairs + kThreads / 32 - 1) / (kThreads / 32));
  if (dtype == LAB_F32)
    lab_launch(memory_finish_kernel<float>, dim3(blocks), dim3(kThreads), 0, stream, (float*)out, ld_out, o, m, gate, ld_g,
               (const float*)w, tokens, H, V, vpad, q_scale, floor_, eps, mult, row_req, state_slot);
  else
    lab_launch(memory_finish_kernel<__nv_bfloat16>, dim3(blocks), dim3(kThreads), 0, stream, (__nv_bfloat16*)out, ld_out,
               o, m, gate, ld_g, (const __nv_bfloat16*)w, tokens, H, V, vpad, q_scale, floor_, eps, mult, row_req, state_slot);
  LAB_LAUNCH_CHECK();
}
