// Gated delta rule with one decay per key channel, as a recurrent mixer with per-sequence state.
//
// Per token and head (S is [d, e], 32-bit, carried from token to token):
//     S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
// with q, k unit vectors per head (q also times d^-1/2) made from projections that pass a short
// causal convolution over time and SiLU, beta = sigmoid(.), g = exp(-exp(A) softplus(a + bias)).
// A column of S (one value channel) never meets another column, so the scan runs one column per
// group of 8 lanes, the column's d rows spread over the lanes' registers, sequentially over the
// tokens of a sequence and in parallel over sequences, heads and columns.
//
// Four kernels, all taking packed rows of several sequences (prompts, chunks, single tokens):
//   delta_prepare    convolution + SiLU, unit norms, beta, decays                (a block a token)
//   delta_conv_tail  the last taps-1 convolution inputs of every sequence -> its state
//   delta_scan       the recurrence; reads and writes S in the state
//   delta_out_norm   o / rms(o) * w * sigmoid(gate) per head, to the activation type
// State of a slot (32-bit): [heads][e][DP] for S (DP = d rounded up to the scan's row count), then
// [channels][taps-1] convolution inputs.  A fresh slot is all zeros.
// Everything that enters the recurrence is computed and kept in 32-bit.
#include "common.cuh"

namespace ek {

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

struct DeltaShape {
  int heads, kv_heads, dim, vdim, taps;
  int rank_a, rank_g;          // inner sizes of the low-rank decay and gate projections
  // columns of a projected row: [q | k | v | beta | a1 | g1]
  __host__ __device__ int cq() const { return kv_heads * dim; }
  __host__ __device__ int cv() const { return heads * vdim; }
  __host__ __device__ int channels() const { return 2 * cq() + cv(); }
  __host__ __device__ int off_beta() const { return channels(); }
  __host__ __device__ int off_a() const { return channels() + heads; }
  __host__ __device__ int off_g() const { return off_a() + rank_a; }
  __host__ __device__ int row() const { return off_g() + rank_g; }
};

// grid: tokens.  proj [T, >= row()] 32-bit.  conv_w [channels][taps] (last column: the current
// token).  a2t [rank_a][heads * dim], dt_bias [heads * dim], a_log [heads].
// Outputs (32-bit): qn, kn [T, kv_heads * dim]; vc [T, heads * vdim]; beta [T, heads];
// decay [T, heads * dim].
__global__ void __launch_bounds__(256)
delta_prepare_kernel(float* __restrict__ qn, float* __restrict__ kn, float* __restrict__ vc,
                     float* __restrict__ beta, float* __restrict__ decay,
                     const float* __restrict__ proj, int proj_stride, const float* __restrict__ conv_w,
                     const float* __restrict__ a2t, const float* __restrict__ dt_bias,
                     const float* __restrict__ a_log, const float* __restrict__ state,
                     size_t slot_stride, size_t tail_offset, const int* __restrict__ positions,
                     const int* __restrict__ token_slot, DeltaShape sh) {
  extern __shared__ float qk_s[];               // [2 * cq] convolved q and k, then [rank_a]
  __shared__ int n_prev_s;
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, tid = threadIdx.x;
  const int pos = positions[t];
  if (pos < 0) return;
  const int slot = token_slot[t];
  const int K = sh.taps, cq = sh.cq(), nch = sh.channels();
  if (tid == 0) {
    int n = 0;                                  // predecessors of this token inside the step
    while (n < K - 1 && t - n - 1 >= 0 && token_slot[t - n - 1] == slot && positions[t - n - 1] == pos - n - 1) ++n;
    n_prev_s = n;
  }
  float* a1_s = qk_s + 2 * cq;
  const float* row = proj + (size_t)t * proj_stride;
  for (int r = tid; r < sh.rank_a; r += blockDim.x) a1_s[r] = row[sh.off_a() + r];
  __syncthreads();
  const int n_prev = n_prev_s;
  const float* tail = state + (size_t)slot * slot_stride + tail_offset;
  for (int c = tid; c < nch; c += blockDim.x) {
    const float* w = conv_w + (size_t)c * K;
    float acc = w[K - 1] * row[c];
    for (int j = 1; j < K; ++j) {
      const float x = j <= n_prev ? proj[(size_t)(t - j) * proj_stride + c]
                                  : tail[(size_t)c * (K - 1) + (n_prev - j + K - 1)];
      acc = fmaf(w[K - 1 - j], x, acc);
    }
    const float y = acc * sigmoid_f(acc);
    if (c < 2 * cq) qk_s[c] = y;
    else vc[(size_t)t * sh.cv() + (c - 2 * cq)] = y;
  }
  __syncthreads();
  // unit vectors per head: a warp a head
  const int warp = tid >> 5, lane = tid & 31, nwarps = blockDim.x >> 5;
  const float q_scale = rsqrtf((float)sh.dim);
  for (int hh = warp; hh < 2 * sh.kv_heads; hh += nwarps) {
    const float* x = qk_s + (size_t)hh * sh.dim;
    float ss = 0.f;
    for (int i = lane; i < sh.dim; i += 32) ss += x[i] * x[i];
    ss = warp_sum(ss);
    const bool is_q = hh < sh.kv_heads;
    const float f = rsqrtf(ss + 1e-6f) * (is_q ? q_scale : 1.f);
    float* dst = (is_q ? qn : kn) + (size_t)t * cq + (size_t)(is_q ? hh : hh - sh.kv_heads) * sh.dim;
    for (int i = lane; i < sh.dim; i += 32) dst[i] = x[i] * f;
  }
  for (int h = tid; h < sh.heads; h += blockDim.x)
    beta[(size_t)t * sh.heads + h] = sigmoid_f(row[sh.off_beta() + h]);
  const int nd = sh.heads * sh.dim;
  for (int c = tid; c < nd; c += blockDim.x) {
    float a = dt_bias[c];
    for (int r = 0; r < sh.rank_a; ++r) a = fmaf(a2t[(size_t)r * nd + c], a1_s[r], a);
    decay[(size_t)t * nd + c] = expf(-expf(a_log[c / sh.dim]) * softplus_f(a));
  }
}

// grid: sequences.  After the step the state's tail holds the last taps-1 inputs of the sequence.
__global__ void delta_conv_tail_kernel(float* __restrict__ state, size_t slot_stride, size_t tail_offset,
                                       const float* __restrict__ proj, int proj_stride,
                                       const int* __restrict__ cu_seqlens, const int* __restrict__ positions,
                                       const int* __restrict__ token_slot, int channels, int taps) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x;
  const int start = cu_seqlens[b], n = cu_seqlens[b + 1] - start;
  if (n <= 0 || positions[start] < 0) return;
  float* tail = state + (size_t)token_slot[start] * slot_stride + tail_offset;
  const int keep = taps - 1;
  for (int c = threadIdx.x; c < channels; c += blockDim.x) {
    float* tc = tail + (size_t)c * keep;
    for (int m = 0; m < keep; ++m) {
      const int from_step = n - keep + m;       // row of the step that lands at place m
      tc[m] = from_step >= 0 ? proj[(size_t)(start + from_step) * proj_stride + c] : tc[m + n];
    }
  }
}

constexpr int kScanCols = 32;        // columns of S a block takes
constexpr int kScanLanes = 8;        // lanes that share a column
constexpr int kScanChunk = 8;        // tokens fetched into shared memory at a time

// grid (sequences, heads, column tiles); 256 threads = 32 columns x 8 lanes; a lane holds RPL
// consecutive rows of its column.
template <int RPL>
__global__ void __launch_bounds__(kScanCols* kScanLanes)
delta_scan_kernel(float* __restrict__ out, const float* __restrict__ qn, const float* __restrict__ kn,
                  const float* __restrict__ vc, const float* __restrict__ beta,
                  const float* __restrict__ decay, float* __restrict__ state, size_t slot_stride,
                  const int* __restrict__ cu_seqlens, const int* __restrict__ positions,
                  const int* __restrict__ token_slot, DeltaShape sh) {
  constexpr int DP = RPL * kScanLanes;          // rows held (>= dim; rows past dim stay zero)
  constexpr int LDS = RPL + 4;                  // a lane's stretch in shared memory, padded
  constexpr int ROW = kScanLanes * LDS;
  __shared__ __align__(16) float q_s[kScanChunk][ROW];
  __shared__ __align__(16) float k_s[kScanChunk][ROW];
  __shared__ __align__(16) float g_s[kScanChunk][ROW];
  __shared__ float v_s[kScanChunk][kScanCols];
  __shared__ float o_s[kScanChunk][kScanCols];
  __shared__ float b_s[kScanChunk];
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int start = cu_seqlens[b], n = cu_seqlens[b + 1] - start;
  if (n <= 0 || positions[start] < 0) return;
  const int slot = token_slot[start];
  const int cl = tid / kScanLanes, lr = tid % kScanLanes;
  const int col = blockIdx.z * kScanCols + cl;
  const bool live = col < sh.vdim;
  const int kvh = h / (sh.heads / sh.kv_heads);
  const int cq = sh.cq(), cv = sh.cv(), nd = sh.heads * sh.dim;

  float S[RPL];
  float* sp = state + (size_t)slot * slot_stride + ((size_t)h * sh.vdim + (live ? col : 0)) * DP + lr * RPL;
#pragma unroll
  for (int i = 0; i < RPL; i += 4) {
    const float4 x = live ? *reinterpret_cast<const float4*>(sp + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    S[i] = x.x; S[i + 1] = x.y; S[i + 2] = x.z; S[i + 3] = x.w;
  }

  for (int c0 = 0; c0 < n; c0 += kScanChunk) {
    const int nt = min(kScanChunk, n - c0);
    for (int idx = tid; idx < kScanChunk * DP; idx += kScanCols * kScanLanes) {
      const int tt = idx / DP, r = idx % DP;
      const bool ok = tt < nt && r < sh.dim;
      const size_t rowi = (size_t)(start + c0 + tt);
      const int at = (r / RPL) * LDS + r % RPL;
      q_s[tt][at] = ok ? qn[rowi * cq + (size_t)kvh * sh.dim + r] : 0.f;
      k_s[tt][at] = ok ? kn[rowi * cq + (size_t)kvh * sh.dim + r] : 0.f;
      g_s[tt][at] = ok ? decay[rowi * nd + (size_t)h * sh.dim + r] : 1.f;
    }
    for (int idx = tid; idx < kScanChunk * kScanCols; idx += kScanCols * kScanLanes) {
      const int tt = idx / kScanCols, c = idx % kScanCols;
      const int gc = blockIdx.z * kScanCols + c;
      v_s[tt][c] = (tt < nt && gc < sh.vdim) ? vc[(size_t)(start + c0 + tt) * cv + (size_t)h * sh.vdim + gc] : 0.f;
    }
    if (tid < kScanChunk) b_s[tid] = tid < nt ? beta[(size_t)(start + c0 + tid) * sh.heads + h] : 0.f;
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float* kk = &k_s[tt][lr * LDS];
      const float* gg = &g_s[tt][lr * LDS];
      const float* qq = &q_s[tt][lr * LDS];
      float part = 0.f;
#pragma unroll
      for (int i = 0; i < RPL; i += 4) {
        const float4 g4 = *reinterpret_cast<const float4*>(gg + i);
        const float4 k4 = *reinterpret_cast<const float4*>(kk + i);
        S[i] *= g4.x; S[i + 1] *= g4.y; S[i + 2] *= g4.z; S[i + 3] *= g4.w;
        part = fmaf(S[i], k4.x, part);
        part = fmaf(S[i + 1], k4.y, part);
        part = fmaf(S[i + 2], k4.z, part);
        part = fmaf(S[i + 3], k4.w, part);
      }
      part += __shfl_xor_sync(0xffffffffu, part, 1);
      part += __shfl_xor_sync(0xffffffffu, part, 2);
      part += __shfl_xor_sync(0xffffffffu, part, 4);
      const float u = b_s[tt] * (v_s[tt][cl] - part);
      float po = 0.f;
#pragma unroll
      for (int i = 0; i < RPL; i += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(kk + i);
        const float4 q4 = *reinterpret_cast<const float4*>(qq + i);
        S[i] = fmaf(k4.x, u, S[i]);
        S[i + 1] = fmaf(k4.y, u, S[i + 1]);
        S[i + 2] = fmaf(k4.z, u, S[i + 2]);
        S[i + 3] = fmaf(k4.w, u, S[i + 3]);
        po = fmaf(S[i], q4.x, po);
        po = fmaf(S[i + 1], q4.y, po);
        po = fmaf(S[i + 2], q4.z, po);
        po = fmaf(S[i + 3], q4.w, po);
      }
      po += __shfl_xor_sync(0xffffffffu, po, 1);
      po += __shfl_xor_sync(0xffffffffu, po, 2);
      po += __shfl_xor_sync(0xffffffffu, po, 4);
      if (lr == 0) o_s[tt][cl] = po;
    }
    __syncthreads();
    for (int idx = tid; idx < nt * kScanCols; idx += kScanCols * kScanLanes) {
      const int tt = idx / kScanCols, c = idx % kScanCols;
      const int gc = blockIdx.z * kScanCols + c;
      if (gc < sh.vdim) out[(size_t)(start + c0 + tt) * cv + (size_t)h * sh.vdim + gc] = o_s[tt][c];
    }
    // (the next chunk's loads touch q_s, k_s, g_s, v_s, b_s only, and o_s is next written after
    // the barrier that follows those loads)
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < RPL; i += 4)
      *reinterpret_cast<float4*>(sp + i) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
  }
}

// grid: tokens.  y[t, h, j] = o[t, h, j] / rms_j(o[t, h, :]) * w[j] * sigmoid(sum_r g2t[r][h, j] g1[t, r]).
template <typename T>
__global__ void __launch_bounds__(256)
delta_out_norm_kernel(T* __restrict__ y, const float* __restrict__ o, const float* __restrict__ proj,
                      int proj_stride, const float* __restrict__ g2t, const float* __restrict__ w,
                      float eps, const int* __restrict__ positions, DeltaShape sh) {
  extern __shared__ float g1_s[];               // [rank_g]
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, tid = threadIdx.x;
  const int cv = sh.cv();
  if (positions[t] < 0) {
    for (int c = tid; c < cv; c += blockDim.x) y[(size_t)t * cv + c] = from_f<T>(0.f);
    return;
  }
  for (int r = tid; r < sh.rank_g; r += blockDim.x) g1_s[r] = proj[(size_t)t * proj_stride + sh.off_g() + r];
  __syncthreads();
  const int warp = tid >> 5, lane = tid & 31, nwarps = blockDim.x >> 5;
  for (int h = warp; h < sh.heads; h += nwarps) {
    const float* x = o + (size_t)t * cv + (size_t)h * sh.vdim;
    float ss = 0.f;
    for (int j = lane; j < sh.vdim; j += 32) ss += x[j] * x[j];
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)sh.vdim + eps);
    for (int j = lane; j < sh.vdim; j += 32) {
      const int c = h * sh.vdim + j;
      float gate = 0.f;
      for (int r = 0; r < sh.rank_g; ++r) gate = fmaf(g2t[(size_t)r * cv + c], g1_s[r], gate);
      y[(size_t)t * cv + c] = from_f<T>(x[j] * inv * w[j] * sigmoid_f(gate));
    }
  }
}

static bool shape_ok(const DeltaShape& sh) {
  return sh.heads > 0 && sh.kv_heads > 0 && sh.heads % sh.kv_heads == 0 && sh.dim > 0 && sh.vdim > 0 &&
         sh.taps >= 1 && sh.rank_a > 0 && sh.rank_g > 0 && sh.heads <= 65535;
}

}  // namespace ek

// Rows of S the scan holds for a key size `dim` (the state's [heads][vdim][rows] uses it); 0: too large.
EK_EXPORT int ek_delta_state_rows(int dim) {
  if (dim <= 0 || dim > 256) return 0;
  if (dim <= 32) return 32;
  if (dim <= 64) return 64;
  if (dim <= 128) return 128;
  return 256;
}

EK_EXPORT int ek_delta_prepare(float* qn, float* kn, float* vc, float* beta, float* decay,
                               const float* proj, int proj_stride, const float* conv_w, const float* a2t,
                               const float* dt_bias, const float* a_log, const float* state,
                               long long slot_stride, long long tail_offset, const int* positions,
                               const int* token_slot, int n_tokens, int heads, int kv_heads, int dim,
                               int vdim, int taps, int rank_a, int rank_g, cudaStream_t stream) {
  using namespace ek;
  if (n_tokens <= 0) return 0;
  DeltaShape sh{heads, kv_heads, dim, vdim, taps, rank_a, rank_g};
  if (!shape_ok(sh) || proj_stride < sh.row()) return EK_ERR_ARG;
  const size_t smem = (size_t)(2 * sh.cq() + rank_a) * sizeof(float);
  if (smem > 200 * 1024) return EK_ERR_ARG;
  if (smem > 40 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(delta_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  delta_prepare_kernel<<<n_tokens, 256, smem, stream>>>(qn, kn, vc, beta, decay, proj, proj_stride, conv_w,
                                                        a2t, dt_bias, a_log, state, (size_t)slot_stride,
                                                        (size_t)tail_offset, positions, token_slot, sh);
  EK_RETURN_LAUNCH_STATUS();
}

EK_EXPORT int ek_delta_conv_tail(float* state, long long slot_stride, long long tail_offset,
                                 const float* proj, int proj_stride, const int* cu_seqlens,
                                 const int* positions, const int* token_slot, int n_seqs, int channels,
                                 int taps, cudaStream_t stream) {
  if (n_seqs <= 0 || taps <= 1) return 0;
  if (channels <= 0 || proj_stride < channels) return EK_ERR_ARG;
  ek::delta_conv_tail_kernel<<<n_seqs, 256, 0, stream>>>(state, (size_t)slot_stride, (size_t)tail_offset,
                                                         proj, proj_stride, cu_seqlens, positions,
                                                         token_slot, channels, taps);
  EK_RETURN_LAUNCH_STATUS();
}

EK_EXPORT int ek_delta_scan(float* out, const float* qn, const float* kn, const float* vc,
                            const float* beta, const float* decay, float* state, long long slot_stride,
                            const int* cu_seqlens, const int* positions, const int* token_slot,
                            int n_seqs, int heads, int kv_heads, int dim, int vdim, cudaStream_t stream) {
  using namespace ek;
  if (n_seqs <= 0) return 0;
  DeltaShape sh{heads, kv_heads, dim, vdim, 1, 1, 1};
  // S is read and written four values at a time: every slot's S must start on a 16-byte boundary
  if (!shape_ok(sh) || slot_stride % 4 || ((uintptr_t)state & 15)) return EK_ERR_ARG;
  dim3 grid(n_seqs, heads, (vdim + kScanCols - 1) / kScanCols);
  if (grid.z > 65535) return EK_ERR_ARG;
  const int rows = ek_delta_state_rows(dim);
#define EK_SCAN(RPL)                                                                                 \
  delta_scan_kernel<RPL><<<grid, kScanCols * kScanLanes, 0, stream>>>(                               \
      out, qn, kn, vc, beta, decay, state, (size_t)slot_stride, cu_seqlens, positions, token_slot, sh)
  switch (rows) {
    case 32: EK_SCAN(4); break;
    case 64: EK_SCAN(8); break;
    case 128: EK_SCAN(16); break;
    case 256: EK_SCAN(32); break;
    default: return EK_ERR_ARG;
  }
#undef EK_SCAN
  EK_RETURN_LAUNCH_STATUS();
}

#define EK_INSTANTIATE(SUFFIX, T)                                                                    \
  EK_EXPORT int ek_delta_out_norm_##SUFFIX(void* y, const float* o, const float* proj, int proj_stride, \
                                           const float* g2t, const float* w, float eps,              \
                                           const int* positions, int n_tokens, int heads,            \
                                           int kv_heads, int dim, int vdim, int taps, int rank_a,    \
                                           int rank_g, cudaStream_t stream) {                        \
    using namespace ek;                                                                              \
    if (n_tokens <= 0) return 0;                                                                     \
    DeltaShape sh{heads, kv_heads, dim, vdim, taps, rank_a, rank_g};                                 \
    if (!shape_ok(sh) || proj_stride < sh.row() || rank_g > 8192) return EK_ERR_ARG;                 \
    delta_out_norm_kernel<T><<<n_tokens, 256, rank_g * sizeof(float), stream>>>(                     \
        (T*)y, o, proj, proj_stride, g2t, w, eps, positions, sh);                                    \
    EK_RETURN_LAUNCH_STATUS();                                                                       \
  }

EK_INSTANTIATE(f32, float)
EK_INSTANTIATE(bf16, ek::bf16)
