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

// resid float32 [T, hidden] contiguous; branch [T, hidden] in the activation type (row stride given) or null;
// weight float32 [hidden]; copy [T, hidden] contiguous in the activation type or null.
ARLE_API int arle_branch_norm_add(float* resid, const void* branch, int branch_stride, const float* weight, void* copy, int dtype,
                                  int num_tokens, int hidden, float eps, cudaStream_t s) {
  if (num_tokens <= 0) return 0;
  if (hidden <= 0 || (branch && !weight)) return ARLE_E_BADARG;
  if (!branch && !copy) return 0;
  const size_t smem = (size_t)hidden * sizeof(float);
  if (smem > 160 * 1024) return ARLE_E_UNSUPPORTED;
  const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  if (dtype == 0) {
    if (smem > 40 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(branch_norm_add_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    launch_kernel(branch_norm_add_kernel<float>, dim3(num_tokens), dim3(threads), smem, s, 1, resid, (const float*)branch, branch_stride,
                  weight, (float*)copy, hidden, eps);
  } else if (dtype == 1) {
    if (smem > 40 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(branch_norm_add_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    launch_kernel(branch_norm_add_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(threads), smem, s, 1, resid, (const __nv_bfloat16*)branch,
                  branch_stride, weight, (__nv_bfloat16*)copy, hidden, eps);
  } else {
    return ARLE_E_BADARG;
  }
  return launch_status();
}
