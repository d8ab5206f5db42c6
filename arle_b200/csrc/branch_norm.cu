// A norm that stands on a branch's OUTPUT instead of its input:
//
//     resid[t, :] += branch[t, :] * rsqrt(mean(branch[t, :]^2) + eps) * weight          (float32)
//     copy[t, :]   = resid[t, :] in the activation type                                  (when asked for)
//
// The sublayers of such a block read the residual as it is, so in bfloat16 the rounded copy that the next
// sublayer reads is written in the same pass.  Without a branch the kernel only writes the copy (the rows a
// model's first block reads).  One block per row, the row staged in shared memory; the reduction order depends on
// the row length alone.
#include "common.cuh"
using namespace arle;

template <typename TA>
__global__ void branch_norm_add_kernel(float* __restrict__ resid, const TA* __restrict__ branch, int branch_stride,
                                       const float* __restrict__ weight, TA* __restrict__ copy, int hidden, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float xs[];
  __shared__ float red[33];
  const int t = blockIdx.x;
  float* xr = resid + (size_t)t * hidden;
  float inv = 0.f;
  if (branch) {
    const TA* br = branch + (size_t)t * branch_stride;
    float ss = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
      const float x = to_f32(br[c]);
      xs[c] = x;
      ss += x * x;
    }
    const float total = block_sum(ss, red);
    inv = 1.0f / sqrtf(total / (float)hidden + eps);
  }
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float x = xr[c];
    if (branch) {
      x += xs[c] * inv * weight[c];
      xr[c] = x;
    }
    if (copy) copy[(size_t)t * hidden + c] = from_f32<TA>(x);
  }
}

// The same with four numbers a thread and access (hidden and branch_stride multiples of 4, bases on the accesses'
// boundaries); the branch's numbers stay in shared memory between the two passes as above.
template <typename TA>
__global__ void branch_norm_add_vec_kernel(float* __restrict__ resid, const TA* __restrict__ branch, int branch_stride,
                                           const float* __restrict__ weight, TA* __restrict__ copy, int hidden, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float xs[];
  __shared__ float red[33];
  const int t = blockIdx.x;
  float* xr = resid + (size_t)t * hidden;
  float inv = 0.f;
  if (branch) {
    const TA* br = branch + (size_t)t * branch_stride;
    float ss = 0.f;
    for (int c = threadIdx.x * 4; c < hidden; c += blockDim.x * 4) {
      float x[4];
      load_vec<TA, 4>(br + c, x);
      store_vec<float, 4>(xs + c, x);
      ss += x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
    }
    const float total = block_sum(ss, red);
    inv = 1.0f / sqrtf(total / (float)hidden + eps);
  }
  for (int c = threadIdx.x * 4; c < hidden; c += blockDim.x * 4) {
    float x[4];
    load_vec<float, 4>(xr + c, x);
    if (branch) {
      float b[4], w[4];
      load_vec<float, 4>(xs + c, b);              // written by this thread
      load_vec<float, 4>(weight + c, w);
#pragma unroll
      for (int i = 0; i < 4; ++i) x[i] += b[i] * inv * w[i];
      store_vec<float, 4>(xr + c, x);
    }
    if (copy) store_vec<TA, 4>(copy + (size_t)t * hidden + c, x);
  }
}

template <typename TA>
static int launch_branch_norm(float* resid, const void* branch, int branch_stride, const float* weight, void* copy, int num_tokens,
                              int hidden, float eps, cudaStream_t s) {
  const size_t smem = (size_t)hidden * sizeof(float);
  const bool vec = hidden % 4 == 0 && branch_stride % 4 == 0 && vec_aligned<4>(resid, sizeof(float)) && vec_aligned<4>(weight, sizeof(float)) &&
                   vec_aligned<4>(branch, sizeof(TA)) && vec_aligned<4>(copy, sizeof(TA));
  auto kernel = vec ? branch_norm_add_vec_kernel<TA> : branch_norm_add_kernel<TA>;
  if (smem > 40 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int per = vec ? 4 : 1;
  const int threads = hidden >= 2048 * per ? 512 : (hidden >= 512 * per ? 256 : 128);
  launch_kernel(kernel, dim3(num_tokens), dim3(threads), smem, s, 1, resid, (const TA*)branch, branch_stride, weight, (TA*)copy, hidden, eps);
  return launch_status();
}

// resid float32 [T, hidden] contiguous; branch [T, hidden] in the activation type (row stride given) or null;
// weight float32 [hidden]; copy [T, hidden] contiguous in the activation type or null.
ARLE_API int arle_branch_norm_add(float* resid, const void* branch, int branch_stride, const float* weight, void* copy, int dtype,
                                  int num_tokens, int hidden, float eps, cudaStream_t s) {
  if (num_tokens <= 0) return 0;
  if (hidden <= 0 || (branch && !weight)) return ARLE_E_BADARG;
  if (!branch && !copy) return 0;
  if ((size_t)hidden * sizeof(float) > 160 * 1024) return ARLE_E_UNSUPPORTED;
  if (dtype == 0) return launch_branch_norm<float>(resid, branch, branch_stride, weight, copy, num_tokens, hidden, eps, s);
  if (dtype == 1) return launch_branch_norm<__nv_bfloat16>(resid, branch, branch_stride, weight, copy, num_tokens, hidden, eps, s);
  return ARLE_E_BADARG;
}

// The same sum followed at once by the NEXT sublayer's norm, for blocks that norm a sublayer's input and its output:
//
//     resid[t, :] += branch[t, :] * rsqrt(mean(branch[t, :]^2) + eps) * weight          (float32)
//     out[t, :]    = resid[t, :] * rsqrt(mean(resid[t, :]^2) + next_eps) * next_weight   (activation type)
//
// One pass over the residual instead of two kernels with a round trip between them.  A thread meets the same numbers
// in all three loops, so the row in shared memory needs no barrier of its own.
template <typename TA, int VEC>
__global__ void branch_norm_add_norm_kernel(float* __restrict__ resid, const TA* __restrict__ branch, int branch_stride,
                                            const float* __restrict__ weight, const float* __restrict__ next_weight, TA* __restrict__ out,
                                            int hidden, float eps, float next_eps) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float xs[];
  __shared__ float red[33];
  const int t = blockIdx.x;
  float* xr = resid + (size_t)t * hidden;
  const TA* br = branch + (size_t)t * branch_stride;
  float ss = 0.f;
  for (int c = threadIdx.x * VEC; c < hidden; c += blockDim.x * VEC) {
    float x[VEC];
    load_vec<TA, VEC>(br + c, x);
    store_vec<float, VEC>(xs + c, x);
#pragma unroll
    for (int i = 0; i < VEC; ++i) ss += x[i] * x[i];
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)hidden + eps);
  ss = 0.f;
  for (int c = threadIdx.x * VEC; c < hidden; c += blockDim.x * VEC) {
    float x[VEC], b[VEC], w[VEC];
    load_vec<float, VEC>(xr + c, x);
    load_vec<float, VEC>(xs + c, b);
    load_vec<float, VEC>(weight + c, w);
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      x[i] += b[i] * inv * w[i];
      ss += x[i] * x[i];
    }
    store_vec<float, VEC>(xr + c, x);
    store_vec<float, VEC>(xs + c, x);
  }
  const float inv2 = 1.0f / sqrtf(block_sum(ss, red) / (float)hidden + next_eps);
  for (int c = threadIdx.x * VEC; c < hidden; c += blockDim.x * VEC) {
    float x[VEC], w[VEC];
    load_vec<float, VEC>(xs + c, x);
    load_vec<float, VEC>(next_weight + c, w);
#pragma unroll
    for (int i = 0; i < VEC; ++i) x[i] = x[i] * inv2 * w[i];
    store_vec<TA, VEC>(out + (size_t)t * hidden + c, x);
  }
}

template <typename TA>
static int launch_branch_norm_norm(float* resid, const void* branch, int branch_stride, const float* weight, const float* next_weight,
                                   void* out, int num_tokens, int hidden, float eps, float next_eps, cudaStream_t s) {
  const size_t smem = (size_t)hidden * sizeof(float);
  const bool vec = hidden % 4 == 0 && branch_stride % 4 == 0 && vec_aligned<4>(resid, sizeof(float)) && vec_aligned<4>(weight, sizeof(float)) &&
                   vec_aligned<4>(next_weight, sizeof(float)) && vec_aligned<4>(branch, sizeof(TA)) && vec_aligned<4>(out, sizeof(TA));
  auto kernel = vec ? branch_norm_add_norm_kernel<TA, 4> : branch_norm_add_norm_kernel<TA, 1>;
  if (smem > 40 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int per = vec ? 4 : 1;
  const int threads = hidden >= 2048 * per ? 512 : (hidden >= 512 * per ? 256 : 128);
  launch_kernel(kernel, dim3(num_tokens), dim3(threads), smem, s, 1, resid, (const TA*)branch, branch_stride, weight, next_weight, (TA*)out,
                hidden, eps, next_eps);
  return launch_status();
}

// resid float32 [T, hidden] contiguous; branch [T, hidden] in the activation type (row stride given); weight, next_weight float32
// [hidden]; out [T, hidden] contiguous in the activation type.
ARLE_API int arle_branch_norm_add_norm(float* resid, const void* branch, int branch_stride, const float* weight, const float* next_weight,
                                       void* out, int dtype, int num_tokens, int hidden, float eps, float next_eps, cudaStream_t s) {
  if (num_tokens <= 0) return 0;
  if (hidden <= 0 || !branch || !weight || !next_weight || !out) return ARLE_E_BADARG;
  if ((size_t)hidden * sizeof(float) > 160 * 1024) return ARLE_E_UNSUPPORTED;
  if (dtype == 0) return launch_branch_norm_norm<float>(resid, branch, branch_stride, weight, next_weight, out, num_tokens, hidden, eps, next_eps, s);
  if (dtype == 1)
    return launch_branch_norm_norm<__nv_bfloat16>(resid, branch, branch_stride, weight, next_weight, out, num_tokens, hidden, eps, next_eps, s);
  return ARLE_E_BADARG;
}
