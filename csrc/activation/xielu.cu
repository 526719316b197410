// Elementwise activations of the feed-forward layers, for bf16 or fp32 activations, evaluated in fp32:
//
//   xIELU        : z > 0 :  a_pos * z^2 + z / 2          a_pos = softplus(p)
//                  z <= 0:  a_neg * (exp(z) - 1 - z) + z / 2,   a_neg = 1/2 + softplus(q)
//                  (the caller passes a_pos and a_neg; they depend on two learned numbers only)
//   gated SiLU   : out = silu(gate) * up on a packed [rows, 2F] activation (gate first) of either type
//                  (csrc/swiglu/swiglu.cu is the bf16-only training kernel with a backward).
//   squared ReLU : max(z, 0)^2
//   clamped gate : g' = min(gate, limit), u' = clamp(up, -limit, limit); out = g' sigmoid(alpha g') (u' + 1), packed like
//                  the gated SiLU
//   gated GELU   : out = gelu_tanh(gate) * up, packed like the gated SiLU
//   sigmoid gate : y *= sigmoid(z) in place, z a strided view of pre-activation gates
// Reference: none (the reference has no model code).
#include "../common/dtype.cuh"

namespace llmctl {

template <typename T>
__global__ void __launch_bounds__(256)
xielu_kernel(const T* __restrict__ z, T* __restrict__ out, long long n, float a_pos, float a_neg) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float v = to_f32(z[i]);
    const float r = v > 0.f ? a_pos * v * v + 0.5f * v : a_neg * (expm1f(v) - v) + 0.5f * v;
    out[i] = from_f32<T>(r);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
gated_silu_kernel(const T* __restrict__ gu, long long ld, T* __restrict__ out, int rows, int F) {
  const long long n = static_cast<long long>(rows) * F;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / F;
    const int c = static_cast<int>(i % F);
    const float g = to_f32(gu[r * ld + c]), u = to_f32(gu[r * ld + F + c]);
    out[i] = from_f32<T>(g / (1.f + expf(-g)) * u);
  }
}

// tanh form of GELU on the gate of a packed [gate | up] activation: 0.5 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3))) * up
template <typename T>
__global__ void __launch_bounds__(256)
gated_gelu_tanh_kernel(const T* __restrict__ gu, long long ld, T* __restrict__ out, int rows, int F) {
  const long long n = static_cast<long long>(rows) * F;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / F;
    const int c = static_cast<int>(i % F);
    const float g = to_f32(gu[r * ld + c]), u = to_f32(gu[r * ld + F + c]);
    out[i] = from_f32<T>(0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g))) * u);
  }
}

// y[r, c] *= sigmoid(z[r, c]) in place; z is a strided view (row stride ldz) of pre-activation gates
template <typename T>
__global__ void __launch_bounds__(256)
sigmoid_gate_kernel(T* __restrict__ y, const T* __restrict__ z, long long ldz, int rows, int F) {
  const long long n = static_cast<long long>(rows) * F;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / F;
    const int c = static_cast<int>(i % F);
    y[i] = from_f32<T>(to_f32(y[i]) / (1.f + expf(-to_f32(z[r * ldz + c]))));
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
gated_clamped_kernel(const T* __restrict__ gu, long long ld, T* __restrict__ out, int rows, int F, float limit, float alpha) {
  const long long n = static_cast<long long>(rows) * F;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / F;
    const int c = static_cast<int>(i % F);
    const float g = fminf(to_f32(gu[r * ld + c]), limit);
    const float u = fminf(fmaxf(to_f32(gu[r * ld + F + c]), -limit), limit);
    out[i] = from_f32<T>(g / (1.f + expf(-alpha * g)) * (u + 1.f));
  }
}

template <typename T>
__global__ void __launch_bounds__(256) relu_squared_kernel(const T* __restrict__ z, T* __restrict__ out, long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float v = fmaxf(to_f32(z[i]), 0.f);
    out[i] = from_f32<T>(v * v);
  }
}

static inline int grid_for(long long n) {
  long long b = (n + 255) / 256;
  if (b > kNumSMs * 16) b = kNumSMs * 16;
  return static_cast<int>(b);
}

}  // namespace llmctl

using namespace llmctl;

LLMCTL_API int llmctl_xielu(const void* z, void* out, int is_fp32, long long n, float a_pos, float a_neg, void* stream) {
  LLMCTL_BEGIN();
  if (n == 0) return 0;
  LLMCTL_DISPATCH_DTYPE(is_fp32, T, (xielu_kernel<T><<<grid_for(n), 256, 0, (cudaStream_t)stream>>>((const T*)z, (T*)out, n, a_pos, a_neg)));
  LLMCTL_RETURN_LAST();
}

LLMCTL_API int llmctl_gated_silu(const void* gate_up, long long ld, void* out, int is_fp32, int rows, int F, void* stream) {
  LLMCTL_BEGIN();
  LLMCTL_REQUIRE(ld >= 2LL * F);
  if (rows == 0 || F == 0) return 0;
  LLMCTL_DISPATCH_DTYPE(is_fp32, T, (gated_silu_kernel<T><<<grid_for(static_cast<long long>(rows) * F), 256, 0, (cudaStream_t)stream>>>(
                                        (const T*)gate_up, ld, (T*)out, rows, F)));
  LLMCTL_RETURN_LAST();
}

LLMCTL_API int llmctl_gated_gelu_tanh(const void* gate_up, long long ld, void* out, int is_fp32, int rows, int F, void* stream) {
  LLMCTL_BEGIN();
  LLMCTL_REQUIRE(ld >= 2LL * F);
  if (rows == 0 || F == 0) return 0;
  LLMCTL_DISPATCH_DTYPE(is_fp32, T, (gated_gelu_tanh_kernel<T><<<grid_for(static_cast<long long>(rows) * F), 256, 0, (cudaStream_t)stream>>>(
                                        (const T*)gate_up, ld, (T*)out, rows, F)));
  LLMCTL_RETURN_LAST();
}

LLMCTL_API int llmctl_sigmoid_gate(void* y, const void* z, long long ldz, int is_fp32, int rows, int F, void* stream) {
  LLMCTL_BEGIN();
  LLMCTL_REQUIRE(ldz >= F);
  if (rows == 0 || F == 0) return 0;
  LLMCTL_DISPATCH_DTYPE(is_fp32, T, (sigmoid_gate_kernel<T><<<grid_for(static_cast<long long>(rows) * F), 256, 0, (cudaStream_t)stream>>>(
                                        (T*)y, (const T*)z, ldz, rows, F)));
  LLMCTL_RETURN_LAST();
}

LLMCTL_API int llmctl_gated_clamped(const void* gate_up, long long ld, void* out, int is_fp32, int rows, int F, float limit, float alpha,
                                    void* stream) {
  LLMCTL_BEGIN();
  LLMCTL_REQUIRE(ld >= 2LL * F && limit > 0.f);
  if (rows == 0 || F == 0) return 0;
  LLMCTL_DISPATCH_DTYPE(is_fp32, T, (gated_clamped_kernel<T><<<grid_for(static_cast<long long>(rows) * F), 256, 0, (cudaStream_t)stream>>>(
                                        (const T*)gate_up, ld, (T*)out, rows, F, limit, alpha)));
  LLMCTL_RETURN_LAST();
}

LLMCTL_API int llmctl_relu_squared(const void* z, void* out, int is_fp32, long long n, void* stream) {
  LLMCTL_BEGIN();
  if (n == 0) return 0;
  LLMCTL_DISPATCH_DTYPE(is_fp32, T, (relu_squared_kernel<T><<<grid_for(n), 256, 0, (cudaStream_t)stream>>>((const T*)z, (T*)out, n)));
  LLMCTL_RETURN_LAST();
}
