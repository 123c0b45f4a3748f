// Several residual streams (hyper-connections): instead of one stream x a token carries n
// copies x_0 .. x_{n-1}, [T, n, W] in 32-bit.  A sublayer reads one mixture of them,
//     u = sum_s in[s] * x_s,
// and its output y is written back into all of them at once from the old values,
//     x_t <- sum_s mix[s, t] * x_s + out[t] * y        (mix is indexed [from, to]).
// One kernel does the write of the sublayer before, the read for the sublayer after and the RMS norm
// of what was read (gain * u * rsqrt(mean(u^2) + eps), the row kept in shared memory meanwhile), so
// the streams make one round trip through memory per sublayer and the mixture none.  Everything is
// computed in 32-bit; y arrives, and the normed mixture leaves, in the activation type T.
#include "common.cuh"

namespace ek {

constexpr int kMaxStreams = 8;

struct StreamCoefficients {
  float in[kMaxStreams];
  float out[kMaxStreams];
  float mix[kMaxStreams * kMaxStreams];
};

// streams[t, s, :] = x[t, :] for every s.
__global__ void hc_broadcast_kernel(float* __restrict__ streams, const float* __restrict__ x,
                                    int n, int width) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t t = blockIdx.x;
  const float* src = x + t * width;
  float* dst = streams + t * n * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = src[i];
    for (int s = 0; s < n; ++s) dst[(size_t)s * width + i] = v;
  }
}

// If y != null: the write with (mix, out) of the sublayer before, in place.  Then, if u != null:
// u[t, :] = sum_s in[s] * x_s, and if normed != null: normed[t, :] = gain * u / rms(u).  Coefficient
// tensors are device pointers ([n], [n], [n, n], 32-bit); any of write_mix / write_out / read_in may
// be null when the matching half is not asked for.
// NS: the number of streams rounded up to 2, 4 or 8 (the copies a thread holds in registers).
template <typename T, int NS>
__global__ void hc_step_kernel(float* __restrict__ streams, const T* __restrict__ y,
                               const float* __restrict__ write_mix, const float* __restrict__ write_out,
                               const float* __restrict__ read_in, float* __restrict__ u, int n,
                               int width, const float* __restrict__ gain, float eps,
                               T* __restrict__ normed) {
  __shared__ StreamCoefficients c;
  __shared__ float scratch[33];
  extern __shared__ __align__(16) float u_s[];  // [width] when the norm is asked for
  float ss = 0.f;
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x < n) {
    c.in[threadIdx.x] = read_in ? read_in[threadIdx.x] : 1.f;
    c.out[threadIdx.x] = write_out ? write_out[threadIdx.x] : 0.f;
  }
  if (y != nullptr)
    for (int i = threadIdx.x; i < n * n; i += blockDim.x) c.mix[i] = write_mix[i];
  __syncthreads();
  const size_t t = blockIdx.x;
  float* xs = streams + t * n * width;
  // V values a thread and step: four (16-byte accesses) when rows allow, else one
  const int V = (width % 4 == 0) ? 4 : 1;
  for (int i0 = threadIdx.x * V; i0 < width; i0 += blockDim.x * V) {
    float x[NS][4];
#pragma unroll
    for (int s = 0; s < NS; ++s) {
      if (s < n) {
        if (V == 4) {
          const float4 v = *reinterpret_cast<const float4*>(xs + (size_t)s * width + i0);
          x[s][0] = v.x; x[s][1] = v.y; x[s][2] = v.z; x[s][3] = v.w;
        } else {
          x[s][0] = xs[(size_t)s * width + i0];
          x[s][1] = x[s][2] = x[s][3] = 0.f;
        }
      } else {
        x[s][0] = x[s][1] = x[s][2] = x[s][3] = 0.f;
      }
    }
    if (y != nullptr) {
      float yv[4] = {0.f, 0.f, 0.f, 0.f};
      if (V == 4) {
        const float4 v = Vec4<T>::load(y + t * width + i0);
        yv[0] = v.x; yv[1] = v.y; yv[2] = v.z; yv[3] = v.w;
      } else {
        yv[0] = to_f<T>(y[t * width + i0]);
      }
      float nx[NS][4];
#pragma unroll
      for (int to = 0; to < NS; ++to) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float a = 0.f;
#pragma unroll
          for (int s = 0; s < NS; ++s)
            if (s < n && to < n) a += c.mix[s * n + to] * x[s][j];
          nx[to][j] = to < n ? a + c.out[to] * yv[j] : 0.f;
        }
        if (to < n) {
          if (V == 4) *reinterpret_cast<float4*>(xs + (size_t)to * width + i0) = make_float4(nx[to][0], nx[to][1], nx[to][2], nx[to][3]);
          else xs[(size_t)to * width + i0] = nx[to][0];
        }
      }
#pragma unroll
      for (int s = 0; s < NS; ++s)
#pragma unroll
        for (int j = 0; j < 4; ++j) x[s][j] = nx[s][j];
    }
    if (u != nullptr || normed != nullptr) {
      float a[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int s = 0; s < NS; ++s)
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (s < n) a[j] += c.in[s] * x[s][j];
      if (u != nullptr) {
        if (V == 4) *reinterpret_cast<float4*>(u + t * width + i0) = make_float4(a[0], a[1], a[2], a[3]);
        else u[t * width + i0] = a[0];
      }
      if (normed != nullptr) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (j < V) { u_s[i0 + j] = a[j]; ss += a[j] * a[j]; }
      }
    }
  }
  if (normed != nullptr) {
    ss = block_sum(ss, scratch);                 // (its barriers also publish u_s)
    const float inv = rsqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x)
      normed[t * width + i] = from_f<T>(u_s[i] * inv * gain[i]);
  }
}

}  // namespace ek

EK_EXPORT int ek_hc_broadcast(float* streams, const float* x, int n_tokens, int n, int width,
                              cudaStream_t stream) {
  using namespace ek;
  if (n_tokens <= 0) return 0;
  if (n < 1 || n > kMaxStreams || width <= 0) return EK_ERR_ARG;
  hc_broadcast_kernel<<<n_tokens, 256, 0, stream>>>(streams, x, n, width);
  EK_RETURN_LAUNCH_STATUS();
}

#define EK_INSTANTIATE(SUFFIX, T)                                                                   \
  EK_EXPORT int ek_hc_step_##SUFFIX(float* streams, const void* y, const float* write_mix,          \
                                    const float* write_out, const float* read_in, float* u,         \
                                    int n_tokens, int n, int width, const float* gain, float eps,   \
                                    void* normed, cudaStream_t stream) {                            \
    using namespace ek;                                                                             \
    if (n_tokens <= 0) return 0;                                                                    \
    if (n < 1 || n > kMaxStreams || width <= 0 || (y && (!write_mix || !write_out)) ||              \
        (normed && !gain))                                                                          \
      return EK_ERR_ARG;                                                                            \
    const size_t smem = normed ? (size_t)width * sizeof(float) : 0;                                 \
    if (smem > 200 * 1024) return EK_ERR_ARG;                                                       \
    if (smem > 40 * 1024) {                                                                         \
      cudaError_t e = cudaFuncSetAttribute(hc_step_kernel<T, 2>,                                    \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e == cudaSuccess)                                                                         \
        e = cudaFuncSetAttribute(hc_step_kernel<T, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                 (int)smem);                                                        \
      if (e == cudaSuccess)                                                                         \
        e = cudaFuncSetAttribute(hc_step_kernel<T, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                 (int)smem);                                                        \
      if (e != cudaSuccess) return (int)e;                                                          \
    }                                                                                               \
    if (n <= 2)                                                                                     \
      hc_step_kernel<T, 2><<<n_tokens, 256, smem, stream>>>(streams, (const T*)y, write_mix,        \
                                                            write_out, read_in, u, n, width, gain,  \
                                                            eps, (T*)normed);                       \
    else if (n <= 4)                                                                                \
      hc_step_kernel<T, 4><<<n_tokens, 256, smem, stream>>>(streams, (const T*)y, write_mix,        \
                                                            write_out, read_in, u, n, width, gain,  \
                                                            eps, (T*)normed);                       \
    else                                                                                            \
      hc_step_kernel<T, 8><<<n_tokens, 256, smem, stream>>>(streams, (const T*)y, write_mix,        \
                                                            write_out, read_in, u, n, width, gain,  \
                                                            eps, (T*)normed);                       \
    EK_RETURN_LAUNCH_STATUS();                                                                      \
  }

EK_INSTANTIATE(f32, float)
EK_INSTANTIATE(bf16, ek::bf16)
