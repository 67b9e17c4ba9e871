// Attention over a latent: every token keeps ONE row [c (r) | k_rot (p)] for all heads, where c is a normed
// low-rank projection of the layer's input and k_rot a rotated key part that all heads share.  A head's keys
// and values are linear maps of c (k_h = Uk_h c, v_h = Uv_h c), so they are never formed: with
// a_h = Uk_h^T q_h ("absorbed" queries, r wide)
//
//     score_h(i, j) = (a_h(i) . c(j) + q_rot_h(i) . k_rot(j)) * scale
//     out_h(i)      = Uv_h  sum_j softmax_j(score_h(i, j)) c(j)
//
// which is attention with one key/value head of width r + p whose values are the first r sizes of the keys.
// The pieces here: `latent_prepare` (norm of c, rotation of k_rot and of the queries' rotated parts, page
// write), `head_project` (the per-head maps Uk^T and Uv on the CUDA cores, float32 in k order, with an optional
// sigmoid gate on the result), and the attention itself in two forms: an exact one (float32 path, twin of the
// other) and a tensor-core one (bfloat16 pages).  Scores, weights and sums are float32 in every form.
#include "common.cuh"


namespace {

// ---- prepare -----------------------------------------------------------------------------------------------
struct LatentPrep {
  const void* src; int src_stride;    // [N, ...] model dtype: heads [plain d | rotated p] at q_off, [c r | k_rot p] at kv_off
  int q_off, kv_off;                  // kv_off < 0: this layer reads another layer's rows and writes none
  int heads, d, r, p;
  const float* norm_w; float eps;     // scale of the norm over c
  const float* inv_freq; int rot_dims; int interleaved; float magnitude;   // inv_freq null: no rotation
  float* qc;                          // [N, heads, r + p] float32: this kernel fills the last p of every head
  void* pool;                         // [pages, 1, page_size, r + p] model dtype, or null
  const int32_t* block_table; int table_width, page_size, num_pages;
  const int32_t* positions; const int32_t* req_of_token;
  int32_t* bad_page;
};

// The first rot_dims of src[0..p) turned by position * inv_freq (pairs (2i, 2i+1) or (i, i + rot_dims / 2)),
// the rest copied.  One warp.
template <typename T, typename TO>
__device__ __forceinline__ void rotate_part(const T* __restrict__ src, TO* __restrict__ dst, int p, int pos,
                                            const LatentPrep& a, int lane) {
  const int half = a.inv_freq ? a.rot_dims >> 1 : 0;
  for (int i = lane; i < half; i += 32) {
    float sn, cs, o1, o2;
    sincosf((float)pos * a.inv_freq[i], &sn, &cs);
    sn *= a.magnitude;
    cs *= a.magnitude;
    const int i1 = a.interleaved ? 2 * i : i, i2 = a.interleaved ? 2 * i + 1 : i + half;
    rotate_pair(to_f32<T>(src[i1]), to_f32<T>(src[i2]), cs, sn, o1, o2);
    dst[i1] = from_f32<TO>(o1);
    dst[i2] = from_f32<TO>(o2);
  }
  for (int i = 2 * half + lane; i < p; i += 32) dst[i] = from_f32<TO>(to_f32<T>(src[i]));
}

// One warp per job of a token: jobs [0, heads) rotate a head's query part, job `heads` makes the token's row.
template <typename T>
__global__ void latent_prepare_kernel(const LatentPrep a) {
  pdl_launch_dependents();
  pdl_wait();
  const int n = blockIdx.x, job = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (job > a.heads) return;
  const int req = a.req_of_token[n];
  if (req < 0) return;
  const int pos = a.positions[n];
  const T* row = reinterpret_cast<const T*>(a.src) + (size_t)n * a.src_stride;
  if (job < a.heads) {
    rotate_part<T, float>(row + a.q_off + (size_t)job * (a.d + a.p) + a.d,
                          a.qc + ((size_t)n * a.heads + job) * (a.r + a.p) + a.r, a.p, pos, a, lane);
    return;
  }
  if (a.kv_off < 0 || a.pool == nullptr) return;
  const int page_idx = pos / a.page_size;
  const int page = page_idx < a.table_width ? a.block_table[(size_t)req * a.table_width + page_idx] : -1;
  if (page < 0 || page >= a.num_pages) {
    if (lane == 0 && a.bad_page) atomicOr(a.bad_page, YALIS_FLAG_BAD_PAGE);
    return;
  }
  T* dst = reinterpret_cast<T*>(a.pool) + ((size_t)page * a.page_size + (pos - page_idx * a.page_size)) * (a.r + a.p);
  const T* s = row + a.kv_off;
  float ss = 0.f;
  for (int i = lane; i < a.r; i += 32) {
    const float x = to_f32<T>(s[i]);
    ss = __fmaf_rn(x, x, ss);
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)a.r + a.eps);
  for (int i = lane; i < a.r; i += 32) dst[i] = from_f32<T>(to_f32<T>(s[i]) * inv * a.norm_w[i]);
  rotate_part<T, T>(s + a.r, dst + a.r, a.p, pos, a, lane);
}

// ---- per-head linear maps -------------------------------------------------------------------------------------
// out[n, h, o] = sum_k w[h, o, k] x[n, h, k]   (optionally times sigmoid(gate[n, h * O + o])), float32 sums in k
// order per lane and a fixed butterfly across lanes.  Block (n, h); a warp per output.
template <typename T, typename TX, typename TO>
__global__ void head_project_kernel(const TX* __restrict__ x, long xs_n, long xs_h, const T* __restrict__ w, int O, int K,
                                    TO* __restrict__ out, long os_n, long os_h, const T* __restrict__ gate, long gs_n,
                                    const int32_t* __restrict__ req_of_token) {
  extern __shared__ float xs[];
  pdl_launch_dependents();
  pdl_wait();
  const int n = blockIdx.x, h = blockIdx.y;
  if (req_of_token && req_of_token[n] < 0) return;
  const TX* xp = x + (size_t)n * xs_n + (size_t)h * xs_h;
  for (int k = threadIdx.x; k < K; k += blockDim.x) xs[k] = to_f32<TX>(xp[k]);
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const T* wh = w + (size_t)h * O * K;
  for (int o = warp; o < O; o += warps) {
    const T* wr = wh + (size_t)o * K;
    float acc = 0.f;
    for (int k = lane; k < K; k += 32) acc = __fmaf_rn(to_f32<T>(wr[k]), xs[k], acc);
    acc = warp_sum(acc);
    if (lane == 0) {
      if (gate) acc *= 1.0f / (1.0f + expf(-to_f32<T>(gate[(size_t)n * gs_n + (size_t)h * O + o])));
      out[(size_t)n * os_n + (size_t)h * os_h + o] = from_f32<TO>(acc);
    }
  }
}

// y[n, c] = x[n, c] * sigmoid(g[n, c])  (x float32 or model dtype, y model dtype)
template <typename T, typename TX>
__global__ void sigmoid_gate_kernel(const TX* __restrict__ x, long xs, const T* __restrict__ g, long gs,
                                    T* __restrict__ y, long ys, int rows, int cols) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t total = (size_t)rows * cols;
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
    const size_t r = e / cols, c = e - r * cols;
    const float v = to_f32<TX>(x[r * xs + c]) / (1.0f + expf(-to_f32<T>(g[r * gs + c])));
    y[r * ys + c] = from_f32<T>(v);
  }
}

// ---- the exact attention -----------------------------------------------------------------------------------------
constexpr int kWarps = 4;
constexpr int kMaxPerLane = 20;   // r + p <= 640

// Block (token, head).  Each warp walks every fourth visible row in ascending order with an online softmax; the
// four partial results are merged in warp order, so a (position, head) has one order of sums whatever the step.
template <typename T>
__global__ void latent_attention_exact_kernel(const float* __restrict__ qc, float* __restrict__ out,
                                              const T* __restrict__ pool, const int32_t* __restrict__ positions,
                                              const int32_t* __restrict__ req_of_token,
                                              const int32_t* __restrict__ block_table, int table_width, int page_size,
                                              int num_pages, int heads, int r, int p, float scale, int window) {
  extern __shared__ float smem[];   // [kWarps][r] sums, then m[kWarps], l[kWarps]
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const int req = req_of_token[t];
  if (req < 0) return;
  const int pos = positions[t];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int w = r + p;
  float qr[kMaxPerLane], acc[kMaxPerLane];
  const float* qp = qc + ((size_t)t * heads + h) * w;
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int d = lane + 32 * i;
    qr[i] = d < w ? qp[d] : 0.f;
    acc[i] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int32_t* bt = block_table + (size_t)req * table_width;
  for (int j = lo + warp; j <= pos; j += kWarps) {
    const int pi = j / page_size;
    const int page = pi < table_width ? bt[pi] : -1;
    if (page < 0 || page >= num_pages) continue;
    const T* row = pool + ((size_t)page * page_size + (j - pi * page_size)) * w;
    float x[kMaxPerLane];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      const int d = lane + 32 * i;
      x[i] = d < w ? to_f32<T>(row[d]) : 0.f;
      dot = __fmaf_rn(qr[i], x[i], dot);
    }
    const float s = warp_sum(dot) * scale;
    const float m_new = fmaxf(m, s);
    const float corr = expf(m - m_new);
    const float pr = expf(s - m_new);
    l = l * corr + pr;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) acc[i] = acc[i] * corr + pr * x[i];
    m = m_new;
  }
  float* acc_s = smem;
  float* m_s = smem + kWarps * r;
  float* l_s = m_s + kWarps;
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int d = lane + 32 * i;
    if (d < r) acc_s[warp * r + d] = acc[i];
  }
  if (lane == 0) {
    m_s[warp] = m;
    l_s[warp] = l;
  }
  __syncthreads();
  float mm = -INFINITY;
#pragma unroll
  for (int k = 0; k < kWarps; ++k) mm = fmaxf(mm, m_s[k]);
  float ll = 0.f, wgt[kWarps];
#pragma unroll
  for (int k = 0; k < kWarps; ++k) {
    wgt[k] = (m_s[k] == -INFINITY) ? 0.f : expf(m_s[k] - mm);
    ll += l_s[k] * wgt[k];
  }
  float* op = out + ((size_t)t * heads + h) * r;
  for (int d = threadIdx.x; d < r; d += blockDim.x) {
    float o = 0.f;
#pragma unroll
    for (int k = 0; k < kWarps; ++k) o += acc_s[k * r + d] * wgt[k];
    op[d] = ll > 0.f ? o / ll : 0.f;
  }
}

}  // namespace

YALIS_API int yalis_latent_prepare(const void* src, int dtype, int src_stride, int q_off, int kv_off, int heads, int d,
                                   int r, int p, const float* norm_w, float eps, const float* inv_freq, int rot_dims,
                                   int interleaved, float magnitude, float* qc, void* pool,
                                   const int32_t* block_table, int table_width, int page_size, int num_pages,
                                   const int32_t* positions, const int32_t* req_of_token, int n_tokens,
                                   int32_t* bad_page, cudaStream_t stream) {
  if (n_tokens <= 0) return YALIS_OK;
  if (heads <= 0 || heads > 65535 || d < 0 || r <= 0 || p < 0) return YALIS_ERR_SHAPE;
  if (inv_freq && (rot_dims <= 0 || (rot_dims & 1) || rot_dims > p)) return YALIS_ERR_SHAPE;
  LatentPrep a;
  a.src = src; a.src_stride = src_stride; a.q_off = q_off; a.kv_off = kv_off; a.heads = heads; a.d = d; a.r = r; a.p = p;
  a.norm_w = norm_w; a.eps = eps; a.inv_freq = inv_freq; a.rot_dims = rot_dims; a.interleaved = interleaved;
  a.magnitude = magnitude; a.qc = qc; a.pool = pool; a.block_table = block_table; a.table_width = table_width;
  a.page_size = page_size; a.num_pages = num_pages; a.positions = positions; a.req_of_token = req_of_token;
  a.bad_page = bad_page;
  const int warps = 4;
  const dim3 grid(n_tokens, (heads + 1 + warps - 1) / warps);
  YALIS_DISPATCH_DTYPE(dtype, T, return yalis_launch(latent_prepare_kernel<T>, grid, dim3(32 * warps), 0, stream, a));
  return YALIS_OK;
}

// x_dtype / out_dtype: float32 or the model dtype `dtype` of w and gate.
YALIS_API int yalis_head_project(const void* x, int x_dtype, long xs_n, long xs_h, const void* w, int dtype, int heads,
                                 int O, int K, void* out, int out_dtype, long os_n, long os_h, const void* gate,
                                 long gs_n, const int32_t* req_of_token, int n_tokens, cudaStream_t stream) {
  if (n_tokens <= 0) return YALIS_OK;
  if (heads <= 0 || heads > 65535 || O <= 0 || K <= 0 || K > 12288) return YALIS_ERR_SHAPE;
  const dim3 grid(n_tokens, heads), block(128);
  const size_t smem = (size_t)K * sizeof(float);
#define YALIS_HP(T, TX, TO)                                                                                         \
  return yalis_launch(head_project_kernel<T, TX, TO>, grid, block, smem, stream, (const TX*)x, xs_n, xs_h, (const T*)w, \
                      O, K, (TO*)out, os_n, os_h, (const T*)gate, gs_n, req_of_token)
  if (dtype == YALIS_F32 && x_dtype == YALIS_F32 && out_dtype == YALIS_F32) YALIS_HP(float, float, float);
  if (dtype == YALIS_BF16 && x_dtype == YALIS_BF16 && out_dtype == YALIS_F32) YALIS_HP(__nv_bfloat16, __nv_bfloat16, float);
  if (dtype == YALIS_BF16 && x_dtype == YALIS_F32 && out_dtype == YALIS_BF16) YALIS_HP(__nv_bfloat16, float, __nv_bfloat16);
  if (dtype == YALIS_BF16 && x_dtype == YALIS_F32 && out_dtype == YALIS_F32) YALIS_HP(__nv_bfloat16, float, float);
#undef YALIS_HP
  return YALIS_ERR_DTYPE;
}

YALIS_API int yalis_sigmoid_gate(const void* x, int x_dtype, long xs, const void* g, long gs, void* y, long ys, int dtype,
                                 int rows, int cols, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return YALIS_OK;
  const size_t total = (size_t)rows * cols;
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  if (dtype == YALIS_F32 && x_dtype == YALIS_F32)
    return yalis_launch(sigmoid_gate_kernel<float, float>, dim3(blocks), dim3(256), 0, stream, (const float*)x, xs,
                        (const float*)g, gs, (float*)y, ys, rows, cols);
  if (dtype == YALIS_BF16 && x_dtype == YALIS_F32)
    return yalis_launch(sigmoid_gate_kernel<__nv_bfloat16, float>, dim3(blocks), dim3(256), 0, stream, (const float*)x, xs,
                        (const __nv_bfloat16*)g, gs, (__nv_bfloat16*)y, ys, rows, cols);
  if (dtype == YALIS_BF16 && x_dtype == YALIS_BF16)
    return yalis_launch(sigmoid_gate_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(blocks), dim3(256), 0, stream,
                        (const __nv_bfloat16*)x, xs, (const __nv_bfloat16*)g, gs, (__nv_bfloat16*)y, ys, rows, cols);
  return YALIS_ERR_DTYPE;
}

YALIS_API int yalis_latent_attention_exact(const float* qc, float* out, const void* pool, int dtype,
                                           const int32_t* positions, const int32_t* req_of_token,
                                           const int32_t* block_table, int table_width, int page_size, int num_pages,
                                           int n_tokens, int heads, int r, int p, float scale, int window,
                                           cudaStream_t stream) {
  if (n_tokens <= 0) return YALIS_OK;
  if (heads <= 0 || heads > 65535 || r <= 0 || p < 0 || r + p > 32 * kMaxPerLane) return YALIS_ERR_SHAPE;
  const size_t smem = ((size_t)kWarps * r + 2 * kWarps) * sizeof(float);
  const dim3 grid(n_tokens, heads);
  YALIS_DISPATCH_DTYPE(dtype, T,
                       return yalis_launch(latent_attention_exact_kernel<T>, grid, dim3(kWarps * 32), smem, stream, qc, out,
                                           (const T*)pool, positions, req_of_token, block_table, table_width, page_size,
                                           num_pages, heads, r, p, scale, window));
  return YALIS_OK;
}
