// Gate of a gated feed-forward: out[t, i] = act(gu[t, 2i]) * gu[t, 2i + 1], computed in float32 and
// rounded once.  act 0: silu(g) = g / (1 + exp(-g)) (SwiGLU); act 1: the tanh form of gelu,
// 0.5 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3))).  gu is the [T, 2I] output of the packed
// gate/up projection, whose rows 2i and 2i + 1 are gate_i and up_i.
#include "common.cuh"
using namespace arle;

__device__ __forceinline__ float gelu_tanh_f(float g) {
  return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
}

template <typename T, int ACT>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter, size_t total, int out_stride) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / inter;
    const int i = (int)(idx - t * inter);
    const float g = to_f32(gu[t * 2 * (size_t)inter + 2 * i]);
    const float u = to_f32(gu[t * 2 * (size_t)inter + 2 * i + 1]);
    out[t * out_stride + i] = from_f32<T>((ACT == 0 ? g / (1.0f + expf(-g)) : gelu_tanh_f(g)) * u);
  }
}

// Eight elements per thread and step for bfloat16 rows whose width is a multiple of 8.
template <int ACT>
__global__ void silu_mul_bf16_vec_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int inter,
                                         size_t total8, int out_stride) {
  pdl_launch_dependents();
  pdl_wait();
  const int i8 = inter >> 3;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total8; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / i8;
    const int c = (int)(idx - t * i8);
    const uint4 a4 = *reinterpret_cast<const uint4*>(gu + t * 2 * (size_t)inter + 16 * c);       // pairs 0..3
    const uint4 b4 = *reinterpret_cast<const uint4*>(gu + t * 2 * (size_t)inter + 16 * c + 8);   // pairs 4..7
    const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a4);
    const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b4);
    uint4 o4;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const __nv_bfloat162 p0 = k < 2 ? a2[2 * k] : b2[2 * k - 4], p1 = k < 2 ? a2[2 * k + 1] : b2[2 * k - 3];
      const float ga = __low2float(p0), gb = __low2float(p1);
      // fast exponential and division (a few ulp of float32, far below the bfloat16 rounding that follows):
      // with the exact ones the kernel was bound by arithmetic, not by memory
      if (ACT == 0)
        o2[k] = __floats2bfloat162_rn(__fdividef(ga, 1.0f + __expf(-ga)) * __high2float(p0),
                                      __fdividef(gb, 1.0f + __expf(-gb)) * __high2float(p1));
      else
        o2[k] = __floats2bfloat162_rn(gelu_tanh_f(ga) * __high2float(p0), gelu_tanh_f(gb) * __high2float(p1));
    }
    *reinterpret_cast<uint4*>(out + t * (size_t)out_stride + 8 * c) = o4;
  }
}

template <int ACT>
static int act_mul_launch(const void* gu, void* out, int dtype, int num_tokens, int inter, int out_stride, cudaStream_t s) {
  const size_t total = (size_t)num_tokens * inter;
  const int threads = 256;
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 32) blocks = 148 * 32;
  if (dtype == 1 && inter % 8 == 0 && out_stride % 8 == 0 && ((uintptr_t)gu & 15) == 0 && ((uintptr_t)out & 15) == 0) {
    const size_t total8 = total / 8;
    size_t b8 = (total8 + threads - 1) / threads;
    if (b8 > 148 * 32) b8 = 148 * 32;
    launch_kernel(silu_mul_bf16_vec_kernel<ACT>, dim3((int)b8), dim3(threads), 0, s, 1, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, inter, total8, out_stride);
    return launch_status();
  }
  if (dtype == 0)
    launch_kernel(silu_mul_kernel<float, ACT>, dim3((int)blocks), dim3(threads), 0, s, 1, (const float*)gu, (float*)out, inter, total, out_stride);
  else if (dtype == 1)
    launch_kernel(silu_mul_kernel<__nv_bfloat16, ACT>, dim3((int)blocks), dim3(threads), 0, s, 1, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, inter, total, out_stride);
  else
    return ARLE_E_BADARG;
  return launch_status();
}

ARLE_API int arle_silu_mul(const void* gu, void* out, int dtype, int num_tokens, int inter, cudaStream_t s) {
  if (num_tokens <= 0) return 0;
  if (inter <= 0) return ARLE_E_BADARG;
  return act_mul_launch<0>(gu, out, dtype, num_tokens, inter, inter, s);
}

// act: 0 silu, 1 gelu (tanh form); out_stride: elements between rows of out (inter when it is contiguous)
ARLE_API int arle_act_mul(const void* gu, void* out, int dtype, int num_tokens, int inter, int act, int out_stride,
                          cudaStream_t s) {
  if (num_tokens <= 0) return 0;
  if (inter <= 0 || (act != 0 && act != 1) || out_stride < inter) return ARLE_E_BADARG;
  return act == 0 ? act_mul_launch<0>(gu, out, dtype, num_tokens, inter, out_stride, s)
                  : act_mul_launch<1>(gu, out, dtype, num_tokens, inter, out_stride, s);
}

// A gated unit with clamped inputs: g = min(gate, limit), u = clamp(up, -limit, limit),
// out = g * sigmoid(alpha * g) * (u + 1); float32 arithmetic, rounded once.  gate_up [T, 2I] with (gate_i, up_i) in
// columns 2i and 2i + 1.
template <typename T>
__global__ void clamped_glu_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter, size_t total, int out_stride, float limit,
                                   float alpha) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / inter;
    const int i = (int)(idx - t * inter);
    const float g = fminf(to_f32(gu[t * 2 * inter + 2 * i]), limit);
    const float u = fminf(fmaxf(to_f32(gu[t * 2 * inter + 2 * i + 1]), -limit), limit);
    out[t * (size_t)out_stride + i] = from_f32<T>(g / (1.0f + expf(-alpha * g)) * (u + 1.0f));
  }
}

// The same, four results a thread: inter and out_stride multiples of 4, both bases on boundaries of their accesses.
template <typename T>
__global__ void clamped_glu_vec_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter4, size_t total4, int out_stride, float limit,
                                       float alpha) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total4; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / inter4;
    const int i = (int)(idx - t * inter4) * 4;
    float in[8], res[4];
    load_vec<T, 8>(gu + t * 8 * inter4 + 2 * i, in);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float g = fminf(in[2 * j], limit);
      const float u = fminf(fmaxf(in[2 * j + 1], -limit), limit);
      res[j] = g / (1.0f + expf(-alpha * g)) * (u + 1.0f);
    }
    store_vec<T, 4>(out + t * (size_t)out_stride + i, res);
  }
}

ARLE_API int arle_clamped_glu(const void* gu, void* out, int dtype, int num_tokens, int inter, int out_stride, float limit, float alpha,
                              cudaStream_t s) {
  if (num_tokens <= 0) return 0;
  if (inter <= 0 || out_stride < inter || !(limit > 0.f)) return ARLE_E_BADARG;
  const size_t elem = dtype == 0 ? sizeof(float) : sizeof(__nv_bfloat16);
  if ((dtype == 0 || dtype == 1) && inter % 4 == 0 && out_stride % 4 == 0 && vec_aligned<8>(gu, elem) && vec_aligned<4>(out, elem)) {
    const size_t total4 = (size_t)num_tokens * (inter / 4);
    size_t blocks = (total4 + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    if (dtype == 0)
      launch_kernel(clamped_glu_vec_kernel<float>, dim3((int)blocks), dim3(256), 0, s, 1, (const float*)gu, (float*)out, inter / 4, total4,
                    out_stride, limit, alpha);
    else
      launch_kernel(clamped_glu_vec_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(256), 0, s, 1, (const __nv_bfloat16*)gu,
                    (__nv_bfloat16*)out, inter / 4, total4, out_stride, limit, alpha);
    return launch_status();
  }
  const size_t total = (size_t)num_tokens * inter;
  size_t blocks = (total + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  if (dtype == 0)
    launch_kernel(clamped_glu_kernel<float>, dim3((int)blocks), dim3(256), 0, s, 1, (const float*)gu, (float*)out, inter, total, out_stride,
                  limit, alpha);
  else if (dtype == 1)
    launch_kernel(clamped_glu_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(256), 0, s, 1, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out,
                  inter, total, out_stride, limit, alpha);
  else
    return ARLE_E_BADARG;
  return launch_status();
}
