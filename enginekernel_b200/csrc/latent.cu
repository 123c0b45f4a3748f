// Latent attention: what stands between the projections and the attention kernels.
//
// A token's keys and values of all heads are functions of one latent vector c (size C) and one
// rotated key part r (size R) shared by the heads:  k_h = [W_uk,h c ; r],  v_h = W_uv,h c.  Only
// [c ; r] is cached, one row of D >= C + R values per token (padded with zeros to the row length
// the attention kernels take), and attention runs in the absorbed form
//     score_h(i, j) = (W_uk,h^T q_h,flat)(i) . c(j) + q_h,rot(i) . r(j),
//     out_h(i)      = W_uv,h sum_j p_h(i, j) c(j),
// that is: attention with ONE key head whose keys and values are both the cached rows, H query
// heads of size D, followed by a product per head.  Two kernels:
//   latent_prepare   norms of the two latents (32-bit), rotation of r, cache write, per token
//   head_linear      out[t, h, :] = W_h in[t, h, :] per head: the value up-projection, and - with the
//                    rotated tail - the absorbed query [W_uk,h^T q_h,flat ; rot(q_h,rot) ; 0]
// Norms, angles and rotations are computed in 32-bit; T is the activation / cache type.
#include "common.cuh"

namespace ek {

// One block per token.  proj[t] = [dq (QR) | dkv latent (C) | key rot part (R)] in 32-bit.
//   cq[t, :QR]   = gain_q  * dq / rms(dq)                      (type T, feeds the q up-projection)
//   page row     = [gain_kv * lat / rms(lat) | rot(r) | 0..]   (type T, D values)
// cos/sin: [positions, rot_dims / 2] in 32-bit (any factor on them is already in the tables);
// dimension i < rot_dims/2 of r turns with dimension i + rot_dims/2, the rest of r passes.
template <typename T>
__global__ void latent_prepare_kernel(T* __restrict__ cq, const float* __restrict__ proj, int proj_stride,
                                      const float* __restrict__ gain_q, const float* __restrict__ gain_kv,
                                      float eps, const float* __restrict__ cos_t,
                                      const float* __restrict__ sin_t, int rot_dims,
                                      const int* __restrict__ positions, const int* __restrict__ token_slot,
                                      T* __restrict__ pages, const int* __restrict__ block_table,
                                      int table_stride, int QR, int C, int R, int D, int write_cache) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, tid = threadIdx.x;
  const float* row = proj + (size_t)t * proj_stride;
  const int pos = positions[t];

  float ssq = 0.f;
  for (int i = tid; i < QR; i += blockDim.x) ssq += row[i] * row[i];
  ssq = block_sum(ssq, scratch);
  const float inv_q = rsqrtf(ssq / (float)QR + eps);
  for (int i = tid; i < QR; i += blockDim.x)
    cq[(size_t)t * QR + i] = from_f<T>(row[i] * inv_q * gain_q[i]);

  if (!write_cache || pos < 0) return;            // (uniform over the block)
  const float* lat = row + QR;
  float ssk = 0.f;
  for (int i = tid; i < C; i += blockDim.x) ssk += lat[i] * lat[i];
  ssk = block_sum(ssk, scratch);
  const float inv_k = rsqrtf(ssk / (float)C + eps);
  const int slot = token_slot[t];
  const int page = block_table[(size_t)slot * table_stride + pos / EK_PAGE];
  T* dst = pages + ((size_t)page * EK_PAGE + (pos & (EK_PAGE - 1))) * (size_t)D;
  for (int i = tid; i < C; i += blockDim.x) dst[i] = from_f<T>(lat[i] * inv_k * gain_kv[i]);
  const float* r = lat + C;
  const int half = rot_dims / 2;
  for (int i = tid; i < R; i += blockDim.x) {
    float v = r[i];
    if (i < half) {
      const float c = cos_t[(size_t)pos * half + i], s = sin_t[(size_t)pos * half + i];
      v = r[i] * c - r[i + half] * s;
    } else if (i < rot_dims) {
      const float c = cos_t[(size_t)pos * half + i - half], s = sin_t[(size_t)pos * half + i - half];
      v = r[i] * c + r[i - half] * s;
    }
    dst[C + i] = from_f<T>(v);
  }
  for (int i = C + R + tid; i < D; i += blockDim.x) dst[i] = from_f<T>(0.f);
}

constexpr int kHeadTokens = 8;       // tokens a block of the per-head products takes
constexpr int kHeadOuts = 32;        // output values a block takes ...
constexpr int kHeadSlices = 4;       // ... each summed by this many threads over a quarter of the inputs
constexpr int kHeadThreads = kHeadOuts * kHeadSlices;

// out[t, h, o] = sum_i w[h, i, o] * in[t, h, i]   for o < n_out, i < n_in.
// w is laid out [heads, n_in, n_out] (neighbouring threads read neighbouring weights); w == null
// skips the product.  grid (token tiles, heads, output tiles of 32); a warp takes a quarter of the
// inputs for the tile's 32 outputs and the four warps' sums meet in shared memory, so that with few
// tokens the chain of loads is short and the weights are spread over many blocks.  If rot_dims >= 0
// the block with blockIdx.z == 0 also writes the rotated tail: out[t, h, n_out + i] =
// rot(in[t, h, n_in + i]) for i < R and zeros up to out_head_stride (the absorbed query).
template <typename T>
__global__ void __launch_bounds__(kHeadThreads)
head_linear_kernel(T* __restrict__ out, int out_row_stride, int out_head_stride,
                   const T* __restrict__ in, int in_row_stride, int in_head_stride,
                   const T* __restrict__ w, int n_tokens, int n_in, int n_out, int R, int rot_dims,
                   const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                   const int* __restrict__ positions) {
  extern __shared__ float in_s[];               // [kHeadTokens][n_in + R]
  __shared__ float part_s[kHeadSlices][kHeadTokens][kHeadOuts];
  pdl_launch_dependents();
  pdl_wait();
  const int t0 = blockIdx.x * kHeadTokens, h = blockIdx.y, tid = threadIdx.x;
  const int nt = min(kHeadTokens, n_tokens - t0);
  const int width = n_in + (rot_dims >= 0 ? R : 0);
  for (int idx = tid; idx < kHeadTokens * width; idx += kHeadThreads) {
    const int tt = idx / width, i = idx % width;
    in_s[idx] = tt < nt ? to_f<T>(in[(size_t)(t0 + tt) * in_row_stride + (size_t)h * in_head_stride + i]) : 0.f;
  }
  __syncthreads();
  if (w != nullptr) {
    const int slice = tid / kHeadOuts, oo = tid % kHeadOuts;
    const int o = blockIdx.z * kHeadOuts + oo;
    const int per = (n_in + kHeadSlices - 1) / kHeadSlices;
    const int i0 = slice * per, i1 = min(n_in, i0 + per);
    float acc[kHeadTokens];
#pragma unroll
    for (int tt = 0; tt < kHeadTokens; ++tt) acc[tt] = 0.f;
    if (o < n_out) {
      const T* wp = w + (size_t)h * n_in * n_out + o;
#pragma unroll 8
      for (int i = i0; i < i1; ++i) {
        const float wv = to_f<T>(wp[(size_t)i * n_out]);
#pragma unroll
        for (int tt = 0; tt < kHeadTokens; ++tt) acc[tt] = fmaf(wv, in_s[tt * width + i], acc[tt]);
      }
    }
#pragma unroll
    for (int tt = 0; tt < kHeadTokens; ++tt) part_s[slice][tt][oo] = acc[tt];
    __syncthreads();
    for (int idx = tid; idx < nt * kHeadOuts; idx += kHeadThreads) {
      const int tt = idx / kHeadOuts, o2 = blockIdx.z * kHeadOuts + idx % kHeadOuts;
      if (o2 < n_out) {
        float v = 0.f;
#pragma unroll
        for (int sl = 0; sl < kHeadSlices; ++sl) v += part_s[sl][tt][idx % kHeadOuts];
        out[(size_t)(t0 + tt) * out_row_stride + (size_t)h * out_head_stride + o2] = from_f<T>(v);
      }
    }
  }
  if (rot_dims >= 0 && blockIdx.z == 0) {
    const int half = rot_dims / 2;
    const int tail = out_head_stride - n_out;
    for (int idx = tid; idx < nt * tail; idx += kHeadThreads) {
      const int tt = idx / tail, i = idx % tail;
      float v = 0.f;
      if (i < R) {
        const float* r = in_s + tt * width + n_in;
        const int pos = max(positions[t0 + tt], 0);
        v = r[i];
        if (i < half) {
          const float c = cos_t[(size_t)pos * half + i], s = sin_t[(size_t)pos * half + i];
          v = r[i] * c - r[i + half] * s;
        } else if (i < rot_dims) {
          const float c = cos_t[(size_t)pos * half + i - half], s = sin_t[(size_t)pos * half + i - half];
          v = r[i] * c + r[i - half] * s;
        }
      }
      out[(size_t)(t0 + tt) * out_row_stride + (size_t)h * out_head_stride + n_out + i] = from_f<T>(v);
    }
  }
}

template <typename T>
static int launch_head_linear(T* out, int out_row_stride, int out_head_stride, const T* in,
                              int in_row_stride, int in_head_stride, const T* w, int n_tokens,
                              int heads, int n_in, int n_out, int R, int rot_dims, const float* cos_t,
                              const float* sin_t, const int* positions, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (heads <= 0 || heads > 65535 || n_in <= 0 || n_out <= 0 || R < 0 || rot_dims > R ||
      (rot_dims >= 0 && (rot_dims % 2 || out_head_stride < n_out + R || !positions ||
                         (rot_dims > 0 && (!cos_t || !sin_t)))))
    return EK_ERR_ARG;
  const int width = n_in + (rot_dims >= 0 ? R : 0);
  const size_t smem = (size_t)kHeadTokens * width * sizeof(float);
  if (smem > 200 * 1024) return EK_ERR_ARG;
  if (smem > 40 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(head_linear_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid((n_tokens + kHeadTokens - 1) / kHeadTokens, heads, w ? (n_out + kHeadOuts - 1) / kHeadOuts : 1);
  if (grid.z > 65535) return EK_ERR_ARG;
  head_linear_kernel<T><<<grid, kHeadThreads, smem, stream>>>(
      out, out_row_stride, out_head_stride, in, in_row_stride, in_head_stride, w, n_tokens, n_in, n_out,
      R, rot_dims, cos_t, sin_t, positions);
  EK_RETURN_LAUNCH_STATUS();
}

}  // namespace ek

#define EK_INSTANTIATE(SUFFIX, T)                                                                     \
  EK_EXPORT int ek_latent_prepare_##SUFFIX(                                                           \
      void* cq, const float* proj, int proj_stride, const float* gain_q, const float* gain_kv,        \
      float eps, const float* cos_t, const float* sin_t, int rot_dims, const int* positions,          \
      const int* token_slot, void* pages, const int* block_table, int table_stride, int n_tokens,     \
      int QR, int C, int R, int D, int write_cache, cudaStream_t stream) {                            \
    using namespace ek;                                                                               \
    if (n_tokens <= 0) return 0;                                                                      \
    if (QR <= 0 || C <= 0 || R < 0 || D < C + R || rot_dims < 0 || rot_dims > R || rot_dims % 2 ||    \
        proj_stride < QR + C + R)                                                                     \
      return EK_ERR_ARG;                                                                              \
    latent_prepare_kernel<T><<<n_tokens, 128, 0, stream>>>(                                           \
        (T*)cq, proj, proj_stride, gain_q, gain_kv, eps, cos_t, sin_t, rot_dims, positions,           \
        token_slot, (T*)pages, block_table, table_stride, QR, C, R, D, write_cache);                  \
    EK_RETURN_LAUNCH_STATUS();                                                                        \
  }                                                                                                   \
  EK_EXPORT int ek_head_linear_##SUFFIX(                                                              \
      void* out, int out_row_stride, int out_head_stride, const void* in, int in_row_stride,          \
      int in_head_stride, const void* w, int n_tokens, int heads, int n_in, int n_out, int R,         \
      int rot_dims, const float* cos_t, const float* sin_t, const int* positions,                     \
      cudaStream_t stream) {                                                                          \
    return ek::launch_head_linear<T>((T*)out, out_row_stride, out_head_stride, (const T*)in,          \
                                     in_row_stride, in_head_stride, (const T*)w, n_tokens, heads,     \
                                     n_in, n_out, R, rot_dims, cos_t, sin_t, positions, stream);      \
  }

EK_INSTANTIATE(f32, float)
EK_INSTANTIATE(bf16, ek::bf16)
