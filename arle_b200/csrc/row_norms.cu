// Norms of plain rows (not the residual) and the sum of normed branches.
//
//  * rms_rows: out[t, :] = x[t, :] / sqrt(mean(x[t, :]^2) + eps) * weight, x float32 or in the activation type, rows of a
//    wider buffer allowed on both sides.  The norm of a small latent between two projections.  Narrow rows (up to 1,024
//    numbers) take a warp each, so that a step of few tokens with a latent of a hundred numbers is not one thread block
//    of idle warps per row; wider rows a block.
//  * normed_sum: out[t, :] = sum_m scale_m * (x_m[t, :] + bias_m) / sqrt(mean((x_m[t, :] + bias_m)^2) + eps) * weight_m over
//    up to four members: mixers that stand side by side and whose outputs are each normed over the model width before
//    they are added.  A member's output bias (that of its last projection) may be added here, before the norm, so that
//    it costs no pass of its own.  A block per token, float32 arithmetic, one rounding at the end.
//  * bias_add: x[t, c] += bias[c] in place (rows of a wider buffer allowed).
//
// The reduction order depends on the row length alone.
#include "common.cuh"
using namespace arle;

constexpr int kMaxMembers = 4;

template <typename TI, typename TO>
__global__ void rms_rows_warp_kernel(const TI* __restrict__ x, int x_stride, const float* __restrict__ weight, TO* __restrict__ out,
                                     int out_stride, int n, float eps, int num_rows) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= num_rows) return;
  const TI* xr = x + (size_t)t * x_stride;
  float ss = 0.f;
  for (int c = lane; c < n; c += 32) {
    const float v = to_f32(xr[c]);
    ss += v * v;
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)n + eps);
  TO* orow = out + (size_t)t * out_stride;
  for (int c = lane; c < n; c += 32) orow[c] = from_f32<TO>(to_f32(xr[c]) * inv * (weight ? weight[c] : 1.0f));
}

template <typename TI, typename TO>
__global__ void rms_rows_block_kernel(const TI* __restrict__ x, int x_stride, const float* __restrict__ weight, TO* __restrict__ out,
                                      int out_stride, int n, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[33];
  const int t = blockIdx.x;
  const TI* xr = x + (size_t)t * x_stride;
  float ss = 0.f;
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    const float v = to_f32(xr[c]);
    ss += v * v;
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)n + eps);
  TO* orow = out + (size_t)t * out_stride;
  for (int c = threadIdx.x; c < n; c += blockDim.x) orow[c] = from_f32<TO>(to_f32(xr[c]) * inv * (weight ? weight[c] : 1.0f));
}

template <typename TI, typename TO>
static int launch_rms_rows(const void* x, int x_stride, const float* weight, void* out, int out_stride, int num_rows, int n, float eps,
                           cudaStream_t s) {
  if (n <= 1024) {
    const int warps = 4;
    launch_kernel(rms_rows_warp_kernel<TI, TO>, dim3((num_rows + warps - 1) / warps), dim3(warps * 32), 0, s, 1, (const TI*)x, x_stride,
                  weight, (TO*)out, out_stride, n, eps, num_rows);
  } else {
    launch_kernel(rms_rows_block_kernel<TI, TO>, dim3(num_rows), dim3(256), 0, s, 1, (const TI*)x, x_stride, weight, (TO*)out, out_stride,
                  n, eps);
  }
  return launch_status();
}

// in_dtype / out_dtype: 0 float32, 1 bfloat16 (float32 in, bfloat16 out is allowed; the reverse is not).
ARLE_API int arle_rms_rows(const void* x, int in_dtype, int x_stride, const float* weight, void* out, int out_dtype, int out_stride,
                           int num_rows, int n, float eps, cudaStream_t s) {
  if (num_rows <= 0) return 0;
  if (n <= 0) return ARLE_E_BADARG;
  if (in_dtype == 0 && out_dtype == 0) return launch_rms_rows<float, float>(x, x_stride, weight, out, out_stride, num_rows, n, eps, s);
  if (in_dtype == 0 && out_dtype == 1) return launch_rms_rows<float, __nv_bfloat16>(x, x_stride, weight, out, out_stride, num_rows, n, eps, s);
  if (in_dtype == 1 && out_dtype == 1)
    return launch_rms_rows<__nv_bfloat16, __nv_bfloat16>(x, x_stride, weight, out, out_stride, num_rows, n, eps, s);
  return ARLE_E_BADARG;
}

struct NormedSumArgs {
  const void* x[kMaxMembers];
  const float* bias[kMaxMembers];
  const float* weight[kMaxMembers];
  int stride[kMaxMembers];
  float scale[kMaxMembers];
  int members;
};

template <typename T>
__global__ void normed_sum_kernel(NormedSumArgs a, T* __restrict__ out, int out_stride, int hidden, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[33];
  const int t = blockIdx.x;
  float inv[kMaxMembers];
#pragma unroll
  for (int m = 0; m < kMaxMembers; ++m) {
    inv[m] = 0.f;
    if (m < a.members) {
      const T* xr = (const T*)a.x[m] + (size_t)t * a.stride[m];
      const float* b = a.bias[m];
      float ss = 0.f;
      for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float v = to_f32(xr[c]) + (b ? b[c] : 0.f);
        ss += v * v;
      }
      inv[m] = a.scale[m] / sqrtf(block_sum(ss, red) / (float)hidden + eps);
    }
  }
  T* orow = out + (size_t)t * out_stride;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float y = 0.f;
#pragma unroll
    for (int m = 0; m < kMaxMembers; ++m) {
      if (m < a.members) {
        const T* xr = (const T*)a.x[m] + (size_t)t * a.stride[m];
        const float v = to_f32(xr[c]) + (a.bias[m] ? a.bias[m][c] : 0.f);
        y = fmaf(v * inv[m], a.weight[m][c], y);
      }
    }
    orow[c] = from_f32<T>(y);
  }
}

// xs, biases, weights: arrays of `members` device pointers (a bias may be null); strides and scales arrays of as many numbers.
ARLE_API int arle_normed_sum(const void* const* xs, const int* strides, const float* const* biases, const float* const* weights,
                             const float* scales, int members, void* out, int dtype, int out_stride, int num_tokens, int hidden, float eps,
                             cudaStream_t s) {
  if (num_tokens <= 0) return 0;
  if (members <= 0 || members > kMaxMembers || hidden <= 0) return ARLE_E_UNSUPPORTED;
  NormedSumArgs a = {};
  a.members = members;
  for (int m = 0; m < members; ++m) {
    if (!xs[m] || !weights[m]) return ARLE_E_BADARG;
    a.x[m] = xs[m];
    a.bias[m] = biases ? biases[m] : nullptr;
    a.weight[m] = weights[m];
    a.stride[m] = strides[m];
    a.scale[m] = scales[m];
  }
  const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  if (dtype == 0)
    launch_kernel(normed_sum_kernel<float>, dim3(num_tokens), dim3(threads), 0, s, 1, a, (float*)out, out_stride, hidden, eps);
  else if (dtype == 1)
    launch_kernel(normed_sum_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(threads), 0, s, 1, a, (__nv_bfloat16*)out, out_stride, hidden, eps);
  else
    return ARLE_E_BADARG;
  return launch_status();
}

template <typename T>
__global__ void bias_add_kernel(T* __restrict__ x, int x_stride, const float* __restrict__ bias, int n) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= n) return;
  T* p = x + (size_t)blockIdx.x * x_stride + c;
  *p = from_f32<T>(to_f32(*p) + bias[c]);
}

ARLE_API int arle_bias_add(void* x, int dtype, int x_stride, const float* bias, int num_rows, int n, cudaStream_t s) {
  if (num_rows <= 0) return 0;
  if (n <= 0 || !bias) return ARLE_E_BADARG;
  const int cb = (n + 255) / 256;
  if (cb > 65535) return ARLE_E_UNSUPPORTED;
  if (dtype == 0)
    launch_kernel(bias_add_kernel<float>, dim3(num_rows, cb), dim3(256), 0, s, 1, (float*)x, x_stride, bias, n);
  else if (dtype == 1)
    launch_kernel(bias_add_kernel<__nv_bfloat16>, dim3(num_rows, cb), dim3(256), 0, s, 1, (__nv_bfloat16*)x, x_stride, bias, n);
  else
    return ARLE_E_BADARG;
  return launch_status();
}
