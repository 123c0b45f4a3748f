// Several residual streams (hyper-connections): instead of one stream x a token carries n
// copies x_0 .. x_{n-1}, [T, n, W] in 32-bit.  A sublayer reads one mixture of them,
//     u = sum_s in[s] * x_s,
// and its output y is written back into all of them at once from the old values,
//     x_t <- sum_s mix[s, t] * x_s + out[t] * y        (mix is indexed [from, to]).
// One kernel does the write of the sublayer before and the read for the sublayer after, so the
// streams make one round trip through memory per sublayer.  Everything is computed in 32-bit; y
// arrives in the activation type T.
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
// u[t, :] = sum_s in[s] * x_s.  Coefficient tensors are device pointers ([n], [n], [n, n], 32-bit);
// any of write_mix / write_out / read_in may be null when the matching half is not asked for.
template <typename T>
__global__ void hc_step_kernel(float* __restrict__ streams, const T* __restrict__ y,
                               const float* __restrict__ write_mix, const float* __restrict__ write_out,
                               const float* __restrict__ read_in, float* __restrict__ u, int n,
                               int width) {
  __shared__ StreamCoefficients c;
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
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float x[kMaxStreams];
#pragma unroll
    for (int s = 0; s < kMaxStreams; ++s) x[s] = s < n ? xs[(size_t)s * width + i] : 0.f;
    if (y != nullptr) {
      const float yv = to_f<T>(y[t * width + i]);
      float nx[kMaxStreams];
#pragma unroll
      for (int to = 0; to < kMaxStreams; ++to) {
        float a = 0.f;
        if (to < n) {
#pragma unroll
          for (int s = 0; s < kMaxStreams; ++s)
            if (s < n) a += c.mix[s * n + to] * x[s];
          a += c.out[to] * yv;
          xs[(size_t)to * width + i] = a;
        }
        nx[to] = a;
      }
#pragma unroll
      for (int s = 0; s < kMaxStreams; ++s) x[s] = nx[s];
    }
    if (u != nullptr) {
      float a = 0.f;
#pragma unroll
      for (int s = 0; s < kMaxStreams; ++s)
        if (s < n) a += c.in[s] * x[s];
      u[t * width + i] = a;
    }
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
                                    int n_tokens, int n, int width, cudaStream_t stream) {          \
    using namespace ek;                                                                             \
    if (n_tokens <= 0) return 0;                                                                    \
    if (n < 1 || n > kMaxStreams || width <= 0 || (y && (!write_mix || !write_out)))                \
      return EK_ERR_ARG;                                                                            \
    hc_step_kernel<T><<<n_tokens, 256, 0, stream>>>(streams, (const T*)y, write_mix, write_out,     \
                                                    read_in, u, n, width);                          \
    EK_RETURN_LAUNCH_STATUS();                                                                      \
  }

EK_INSTANTIATE(f32, float)
EK_INSTANTIATE(bf16, ek::bf16)
