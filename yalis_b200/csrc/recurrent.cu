// Mixers that keep a matrix per head instead of keys and values: linear recurrences
// over a float32 state S [dim, vdim] per (request, head),
//
//   S <- diag(g_t) S                      g_t: a constant per head, a scalar per token, or a vector over dim
//   u  = beta_t (v_t - S^T k_t)           (delta rule)        or   u = v_t   (plain outer-product write)
//   S <- S + k_t u^T
//   o_t = S^T q_t                         (the read-out sees the token's own write)
//
// with the short causal convolution that feeds some of them and the per-head norm and gate
// that follow them.  Everything here is float32 arithmetic whatever the model's dtype; the
// state and the convolution's tail live in the per-request slot memory of the cache manager.
//
// The columns of S are independent of one another (column j only ever meets v_j), so a thread
// owns 16 rows of one column in registers, the lanes that share a column sit in one warp, and
// a block walks the tokens of one request in order: a portion of a prompt and a single
// decoded token are the same loop, and the result for a token does not depend on how the
// request was cut into steps or on what else is in the batch.
#include "common.cuh"

namespace {

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }

// ---- short causal convolution over time, per channel, then silu -----------------------------------
//   y_t[c] = sum_j w[c][K-1-j] x_(t-j)[c],  x before the request's start = 0
// The last K-1 inputs of every request are kept in its slot: tail[c][0..K-2], oldest first.
constexpr int kMaxTaps = 16;

template <typename T>
__global__ void short_conv_silu_kernel(const T* __restrict__ x, int x_stride, const float* __restrict__ w,
                                       const float* __restrict__ tail, size_t slot_stride,
                                       const int32_t* __restrict__ req_of_token, const int32_t* __restrict__ q_start,
                                       const int32_t* __restrict__ slots, float* __restrict__ out, int out_stride,
                                       int channels, int taps) {
  pdl_launch_dependents();
  pdl_wait();
  const int n = blockIdx.x;
  const int req = req_of_token[n];
  if (req < 0) return;
  const int i = n - q_start[req];                 // index of the token in its request's portion
  const float* tl = tail + (size_t)slots[req] * slot_stride;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
    float acc = 0.f;
    for (int j = taps - 1; j >= 0; --j) {         // oldest input first: a fixed order of additions
      float xv;
      if (i - j >= 0) xv = to_f32<T>(x[(size_t)(n - j) * x_stride + c]);
      else xv = tl[(size_t)c * (taps - 1) + (taps - 1 + i - j)];
      acc = __fmaf_rn(w[(size_t)c * taps + (taps - 1 - j)], xv, acc);
    }
    out[(size_t)n * out_stride + c] = silu_exact(acc);
  }
}

// After the step: the tail becomes the last K-1 inputs the request has seen.
template <typename T>
__global__ void short_conv_tail_kernel(const T* __restrict__ x, int x_stride, float* __restrict__ tail,
                                       size_t slot_stride, const int32_t* __restrict__ q_start,
                                       const int32_t* __restrict__ slots, int channels, int taps) {
  pdl_launch_dependents();
  pdl_wait();
  const int req = blockIdx.x;
  const int a = q_start[req], q_len = q_start[req + 1] - a;
  if (q_len <= 0) return;
  float* tl = tail + (size_t)slots[req] * slot_stride;
  const int keep = taps - 1;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
    float nv[kMaxTaps];
#pragma unroll
    for (int m = 0; m < kMaxTaps; ++m) {
      if (m < keep) {
        const int i = q_len - keep + m;           // index in the portion of the input that lands at place m
        nv[m] = i >= 0 ? to_f32<T>(x[(size_t)(a + i) * x_stride + c]) : tl[(size_t)c * keep + (m + q_len)];
      }
    }
#pragma unroll
    for (int m = 0; m < kMaxTaps; ++m)
      if (m < keep) tl[(size_t)c * keep + m] = nv[m];
  }
}

// ---- the recurrence ------------------------------------------------------------------------------
constexpr int kScanThreads = 128;
constexpr int kRows = 16;            // rows of a column a thread keeps

struct ScanParams {
  const float* q; int q_stride;      // [N, kv_heads * dim]
  const float* k; int k_stride;
  const float* v; int v_stride;      // [N, heads * vdim]
  const float* decay_const;          // DECAY 0: [heads]
  const void* a_raw; int a_stride;   // DECAY 1: [N, heads]; DECAY 2: [N, heads * dim]  (model dtype)
  const float* a_log;                // [heads]
  const float* dt_bias;              // [heads] or [heads * dim]
  const void* b_raw; int b_stride;   // DELTA: [N, heads]  (model dtype)
  float* state; size_t slot_stride;  // per slot: [heads][vdim][dim_padded]
  float* out; int out_stride;        // [N, heads * vdim]
  const int32_t* q_start; const int32_t* slots;
  int heads, kv_heads, dim, dim_padded, vdim, lanes, tile;
  int normalize; float q_scale, unit_eps;
};

// DECAY: 0 constant per head, 1 scalar per token and head, 2 vector per token, head and key channel.
template <typename T, bool DELTA, int DECAY>
__global__ void __launch_bounds__(kScanThreads) state_scan_kernel(const ScanParams p) {
  extern __shared__ __align__(16) float sm[];
  pdl_launch_dependents();
  pdl_wait();
  const int req = blockIdx.z, h = blockIdx.y;
  const int t_begin = p.q_start[req], q_len = p.q_start[req + 1] - t_begin;
  if (q_len <= 0) return;
  const int L = p.lanes, cols = kScanThreads / L, width = kRows * L;
  const int tid = threadIdx.x, l = tid % L, c = tid / L;
  const int j = blockIdx.x * cols + c;
  const bool live = j < p.vdim;
  const int kvh = h / (p.heads / p.kv_heads);
  const int D = p.dim, Dp = p.dim_padded, V = p.vdim, TT = p.tile;
  float* qs = sm;                                  // [TT][width]
  float* ks = qs + (size_t)TT * width;
  float* gv = ks + (size_t)TT * width;             // DECAY 2 only
  float* vs = gv + (DECAY == 2 ? (size_t)TT * width : 0);   // [TT][cols]
  float* bs = vs + (size_t)TT * cols;              // beta [TT]
  float* gs = bs + TT;                             // scalar decay [TT]

  float* sp = p.state + (size_t)p.slots[req] * p.slot_stride + ((size_t)h * V + (live ? j : 0)) * Dp;
  float S[kRows];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int d = (i * L + l) * 4;
    float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
    if (live && d < Dp) x = *reinterpret_cast<const float4*>(sp + d);
    S[4 * i] = x.x; S[4 * i + 1] = x.y; S[4 * i + 2] = x.z; S[4 * i + 3] = x.w;
  }
  const float exp_a = DECAY != 0 ? expf(p.a_log[h]) : 0.f;
  const float g_const = DECAY == 0 ? p.decay_const[h] : 1.f;
  const T* a_raw = reinterpret_cast<const T*>(p.a_raw);
  const T* b_raw = reinterpret_cast<const T*>(p.b_raw);

  for (int t0 = 0; t0 < q_len; t0 += TT) {
    const int tt = min(TT, q_len - t0);
    __syncthreads();
    for (int e = tid; e < tt * width; e += kScanThreads) {
      const int t = e / width, d = e - t * width;
      const size_t n = (size_t)(t_begin + t0 + t);
      const bool in = d < D;
      qs[e] = in ? p.q[n * p.q_stride + (size_t)kvh * D + d] : 0.f;
      ks[e] = in ? p.k[n * p.k_stride + (size_t)kvh * D + d] : 0.f;
      if (DECAY == 2) {
        float g = 1.f;
        if (in) {
          const float a = to_f32<T>(a_raw[n * p.a_stride + (size_t)h * D + d]) + p.dt_bias[(size_t)h * D + d];
          g = expf(-exp_a * softplus_f(a));
        }
        gv[e] = g;
      }
    }
    for (int e = tid; e < tt * cols; e += kScanThreads) {
      const int t = e / cols, cc = e - t * cols;
      const int jj = blockIdx.x * cols + cc;
      vs[e] = jj < V ? p.v[(size_t)(t_begin + t0 + t) * p.v_stride + (size_t)h * V + jj] : 0.f;
    }
    if (tid < tt) {
      const size_t n = (size_t)(t_begin + t0 + tid);
      if (DELTA) bs[tid] = sigmoid_f(to_f32<T>(b_raw[n * p.b_stride + h]));
      if (DECAY == 1) gs[tid] = expf(-exp_a * softplus_f(to_f32<T>(a_raw[n * p.a_stride + h]) + p.dt_bias[h]));
    }
    __syncthreads();
    if (p.normalize) {
      // q and k of every token to unit length (q then scaled); a warp per token, sums in a fixed order
      for (int t = tid >> 5; t < tt; t += kScanThreads / 32) {
        float sq = 0.f, sk = 0.f;
        for (int d = tid & 31; d < D; d += 32) {
          const float a = qs[t * width + d], b = ks[t * width + d];
          sq = __fmaf_rn(a, a, sq);
          sk = __fmaf_rn(b, b, sk);
        }
        sq = warp_sum(sq);
        sk = warp_sum(sk);
        const float rq = p.q_scale / sqrtf(sq + p.unit_eps), rk = 1.0f / sqrtf(sk + p.unit_eps);
        for (int d = tid & 31; d < D; d += 32) {
          qs[t * width + d] *= rq;
          ks[t * width + d] *= rk;
        }
      }
      __syncthreads();
    }
    for (int t = 0; t < tt; ++t) {
      float kr[kRows], qr[kRows];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int d = (i * L + l) * 4;
        const float4 a = *reinterpret_cast<const float4*>(ks + (size_t)t * width + d);
        const float4 b = *reinterpret_cast<const float4*>(qs + (size_t)t * width + d);
        kr[4 * i] = a.x; kr[4 * i + 1] = a.y; kr[4 * i + 2] = a.z; kr[4 * i + 3] = a.w;
        qr[4 * i] = b.x; qr[4 * i + 1] = b.y; qr[4 * i + 2] = b.z; qr[4 * i + 3] = b.w;
      }
      if (DECAY == 2) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float4 g = *reinterpret_cast<const float4*>(gv + (size_t)t * width + (i * L + l) * 4);
          S[4 * i] *= g.x; S[4 * i + 1] *= g.y; S[4 * i + 2] *= g.z; S[4 * i + 3] *= g.w;
        }
      } else {
        const float g = DECAY == 1 ? gs[t] : g_const;
#pragma unroll
        for (int r = 0; r < kRows; ++r) S[r] *= g;
      }
      float u = vs[t * cols + c];
      if (DELTA) {
        float dot = 0.f;
#pragma unroll
        for (int r = 0; r < kRows; ++r) dot = __fmaf_rn(S[r], kr[r], dot);
        for (int o = 1; o < L; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        u = bs[t] * (u - dot);
      }
      float o_acc = 0.f;
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        S[r] = __fmaf_rn(kr[r], u, S[r]);
        o_acc = __fmaf_rn(S[r], qr[r], o_acc);
      }
      for (int o = 1; o < L; o <<= 1) o_acc += __shfl_xor_sync(0xffffffffu, o_acc, o);
      if (live && l == 0) p.out[(size_t)(t_begin + t0 + t) * p.out_stride + (size_t)h * V + j] = o_acc;
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int d = (i * L + l) * 4;
      if (d < Dp) *reinterpret_cast<float4*>(sp + d) = make_float4(S[4 * i], S[4 * i + 1], S[4 * i + 2], S[4 * i + 3]);
    }
  }
}

// ---- per-head norm, weight and gate of a mixer's read-out ---------------------------------------------
//   y[n, h, :] = o / sqrt(mean(o^2) + eps) * weight * act(gate[n, h, :]) * out_scale
// GATE: 0 none, 1 silu, 2 sigmoid.
template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, int o_stride, const float* __restrict__ weight,
                                      const T* __restrict__ gate, int gate_stride, int gate_kind, T* __restrict__ y,
                                      int y_stride, const int32_t* __restrict__ req_of_token, int vdim, float eps,
                                      float out_scale) {
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const int n = blockIdx.x, h = blockIdx.y;
  if (req_of_token[n] < 0) return;
  const float* op = o + (size_t)n * o_stride + (size_t)h * vdim;
  float ss = 0.f;
  for (int d = threadIdx.x; d < vdim; d += blockDim.x) ss = __fmaf_rn(op[d], op[d], ss);
  ss = block_sum(ss, scratch);
  const float r = 1.0f / sqrtf(ss / (float)vdim + eps);
  for (int d = threadIdx.x; d < vdim; d += blockDim.x) {
    float val = op[d] * r;
    if (weight) val *= weight[d];
    if (gate_kind) {
      const float z = to_f32<T>(gate[(size_t)n * gate_stride + (size_t)h * vdim + d]);
      val *= gate_kind == 1 ? silu_exact(z) : sigmoid_f(z);
    }
    y[(size_t)n * y_stride + (size_t)h * vdim + d] = from_f32<T>(val * out_scale);
  }
}

}  // namespace

YALIS_API int yalis_short_conv_silu(const void* x, int dtype, int x_stride, const float* w, float* tail,
                                    int64_t slot_stride, const int32_t* req_of_token, const int32_t* q_start,
                                    const int32_t* slots, float* out, int out_stride, int n_tokens, int n_requests,
                                    int channels, int taps, cudaStream_t stream) {
  if (n_tokens <= 0) return YALIS_OK;
  if (taps < 1 || taps > kMaxTaps || channels <= 0) return YALIS_ERR_SHAPE;
  const int by = (channels + 127) / 128;
  YALIS_DISPATCH_DTYPE(dtype, T, {
    int st = yalis_launch(short_conv_silu_kernel<T>, dim3(n_tokens, by), dim3(128), 0, stream, (const T*)x, x_stride, w,
                          (const float*)tail, (size_t)slot_stride, req_of_token, q_start, slots, out, out_stride,
                          channels, taps);
    if (st != YALIS_OK || taps == 1) return st;
    return yalis_launch(short_conv_tail_kernel<T>, dim3(n_requests, by), dim3(128), 0, stream, (const T*)x, x_stride,
                        tail, (size_t)slot_stride, q_start, slots, channels, taps);
  });
  return YALIS_OK;
}

// Lanes that share a column of the state: the smallest power of two with 16 * lanes >= dim.
YALIS_API int yalis_state_scan_lanes(int dim) {
  int lanes = 1;
  while (lanes * kRows < dim) lanes <<= 1;
  return lanes;
}

YALIS_API int yalis_state_scan(const float* q, int q_stride, const float* k, int k_stride, const float* v, int v_stride,
                               const float* decay_const, const void* a_raw, int a_stride, const float* a_log,
                               const float* dt_bias, const void* b_raw, int b_stride, int raw_dtype, float* state,
                               int64_t slot_stride, float* out, int out_stride, const int32_t* q_start,
                               const int32_t* slots, int n_requests, int heads, int kv_heads, int dim, int vdim,
                               int delta, int decay_kind, int normalize, float q_scale, float unit_eps,
                               cudaStream_t stream) {
  if (n_requests <= 0) return YALIS_OK;
  if (dim <= 0 || vdim <= 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads || heads > 65535 || n_requests > 65535)
    return YALIS_ERR_SHAPE;
  const int lanes = yalis_state_scan_lanes(dim);
  if (lanes > 32) return YALIS_ERR_SHAPE;           // dim <= 512
  if (decay_kind < 0 || decay_kind > 2 || (decay_kind == 0 && !decay_const) || (decay_kind != 0 && (!a_raw || !a_log || !dt_bias)) ||
      (delta && !b_raw))
    return YALIS_ERR_SHAPE;
  const int dim_padded = (dim + 3) & ~3;
  if ((slot_stride & 3) || ((uintptr_t)state & 15)) return YALIS_ERR_ALIGN;
  const int cols = kScanThreads / lanes, width = kRows * lanes;
  const size_t per_token = ((decay_kind == 2 ? 3 : 2) * (size_t)width + cols + 2) * sizeof(float);
  int tile = (int)((40 * 1024) / per_token);
  tile = tile > 16 ? 16 : (tile < 1 ? 1 : tile);
  ScanParams p;
  p.q = q; p.q_stride = q_stride; p.k = k; p.k_stride = k_stride; p.v = v; p.v_stride = v_stride;
  p.decay_const = decay_const; p.a_raw = a_raw; p.a_stride = a_stride; p.a_log = a_log; p.dt_bias = dt_bias;
  p.b_raw = b_raw; p.b_stride = b_stride; p.state = state; p.slot_stride = (size_t)slot_stride; p.out = out;
  p.out_stride = out_stride; p.q_start = q_start; p.slots = slots; p.heads = heads; p.kv_heads = kv_heads;
  p.dim = dim; p.dim_padded = dim_padded; p.vdim = vdim; p.lanes = lanes; p.tile = tile; p.normalize = normalize;
  p.q_scale = q_scale; p.unit_eps = unit_eps;
  const dim3 grid((vdim + cols - 1) / cols, heads, n_requests);
  const size_t smem = per_token * tile;
#define YALIS_SCAN(DELTA, DECAY) \
  return yalis_launch(state_scan_kernel<T, DELTA, DECAY>, grid, dim3(kScanThreads), smem, stream, p)
  YALIS_DISPATCH_DTYPE(raw_dtype, T, {
    if (delta && decay_kind == 1) YALIS_SCAN(true, 1);
    if (delta && decay_kind == 2) YALIS_SCAN(true, 2);
    if (delta && decay_kind == 0) YALIS_SCAN(true, 0);
    if (decay_kind == 0) YALIS_SCAN(false, 0);
    if (decay_kind == 1) YALIS_SCAN(false, 1);
    YALIS_SCAN(false, 2);
  });
#undef YALIS_SCAN
  return YALIS_OK;
}

YALIS_API int yalis_head_norm_gate(const float* o, int o_stride, const float* weight, const void* gate, int gate_stride,
                                   int gate_kind, void* y, int y_stride, int dtype, const int32_t* req_of_token,
                                   int n_tokens, int heads, int vdim, float eps, float out_scale, cudaStream_t stream) {
  if (n_tokens <= 0) return YALIS_OK;
  if (heads <= 0 || heads > 65535 || vdim <= 0 || gate_kind < 0 || gate_kind > 2 || (gate_kind && !gate)) return YALIS_ERR_SHAPE;
  const int threads = vdim <= 32 ? 32 : (vdim <= 64 ? 64 : 128);
  YALIS_DISPATCH_DTYPE(dtype, T,
                       return yalis_launch(head_norm_gate_kernel<T>, dim3(n_tokens, heads), dim3(threads), 0, stream, o,
                                           o_stride, weight, (const T*)gate, gate_stride, gate_kind, (T*)y, y_stride,
                                           req_of_token, vdim, eps, out_scale));
  return YALIS_OK;
}
