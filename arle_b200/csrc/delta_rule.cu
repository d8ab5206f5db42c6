// The gated delta rule: a matrix memory per head that forgets by a scalar decay and is corrected towards the value
// of the current key,
//
//     S <- g_t S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t          (S: dim x vdim, float32)
//
// so the read-out sees the current token's write.  q and k are brought to unit length per head first,
// x / sqrt(sum x^2 + unit_eps), and q is multiplied by q_scale.  Everything is float32 arithmetic whatever the
// activation type; the memory lives in the request's slot of the cache manager's state arena.
//
//  * delta_gates: beta = sigmoid(z_b), g = exp(-exp(A_log) * softplus(z_a + dt_bias)) from the float32 sums
//    [T, 2 * heads] (the betas' sums, then the decays').
//  * delta_scan: a block per (row of the step, head, tile of columns).  A column of S (dim numbers, stored contiguously:
//    the memory is kept transposed, [head][column][dim]) is held by `lpc` lanes, EPL numbers a lane.  Per token the
//    lanes form their parts of S_old . k and S_old . q, add both by shuffles in one round, and since
//    S^T q = g S_old^T q + u (k . q) the read-out needs no second round; k . q is formed once per token while
//    16 tokens are staged in shared memory (where the unit lengths are applied).  The split of a column depends on
//    dim alone, so a token's sums have one order whatever the cutting or the batch.
#include "common.cuh"
using namespace arle;

__global__ void delta_gates_kernel(const float* __restrict__ pre, int pre_stride, const float* __restrict__ a_log,
                                   const float* __restrict__ dt_bias, float* __restrict__ beta, float* __restrict__ decay, int H,
                                   size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / H;
    const int h = (int)(idx - t * H);
    const float zb = pre[t * pre_stride + h];
    const float za = pre[t * pre_stride + H + h] + dt_bias[h];
    const float sp = za > 20.f ? za : log1pf(expf(za));
    beta[idx] = 1.0f / (1.0f + expf(-zb));
    decay[idx] = expf(-expf(a_log[h]) * sp);
  }
}

ARLE_API int arle_delta_gates(const float* pre, int pre_stride, const float* a_log, const float* dt_bias, float* beta, float* decay,
                              int num_tokens, int H, cudaStream_t s) {
  if (num_tokens <= 0) return 0;
  if (H <= 0) return ARLE_E_BADARG;
  const size_t total = (size_t)num_tokens * H;
  size_t blocks = (total + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  launch_kernel(delta_gates_kernel, dim3((int)blocks), dim3(256), 0, s, 1, pre, pre_stride, a_log, dt_bias, beta, decay, H, total);
  return launch_status();
}

constexpr int kDeltaChunk = 16;
constexpr int kDeltaThreads = 256;

template <typename T, int EPL>
__global__ void __launch_bounds__(kDeltaThreads) delta_scan_kernel(
    const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, int q_stride, int k_stride, int v_stride,
    const float* __restrict__ beta, const float* __restrict__ decay, float* __restrict__ state, long slot_stride,
    const int* __restrict__ q_indptr, const int* __restrict__ state_slots, float* __restrict__ out, int H, int kq_heads, int dim,
    int vdim, float q_scale, float unit_eps, int lpc) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float sm[];
  const int cpb = kDeltaThreads / lpc;                   // columns of S a block holds
  const int dpad = lpc * EPL;                            // a token's q or k in shared memory, padded with zeros
  float* qs = sm;                                        // [chunk][dpad]
  float* ksm = qs + kDeltaChunk * dpad;                  // [chunk][dpad]
  float* vs = ksm + kDeltaChunk * dpad;                  // [chunk][cpb]
  float* gs = vs + kDeltaChunk * cpb;                    // [chunk] decay
  float* bs = gs + kDeltaChunk;                          // [chunk] beta
  float* kq = bs + kDeltaChunk;                          // [chunk] k . q
  const int r = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * cpb;
  const int g = h / (H / kq_heads);
  const int cl = threadIdx.x / lpc, part = threadIdx.x % lpc;
  const int e0 = part * EPL;
  const int beg = q_indptr[r], end = q_indptr[r + 1];
  const bool col_live = c0 + cl < vdim;
  float* sp = state + (size_t)state_slots[r] * slot_stride + (size_t)h * vdim * dim + (size_t)(c0 + cl) * dim;
  float S[EPL];
#pragma unroll
  for (int i = 0; i < EPL; ++i) S[i] = (col_live && e0 + i < dim) ? sp[e0 + i] : 0.f;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  for (int t0 = beg; t0 < end; t0 += kDeltaChunk) {
    const int n = min(kDeltaChunk, end - t0);
    __syncthreads();
    // a warp per staged token: unit lengths of q and k, their product
    for (int tt = warp; tt < n; tt += kDeltaThreads / 32) {
      const T* qp = q + (size_t)(t0 + tt) * q_stride + (size_t)g * dim;
      const T* kp = k + (size_t)(t0 + tt) * k_stride + (size_t)g * dim;
      float sq = 0.f, sk = 0.f, qk = 0.f;
      for (int e = lane; e < dim; e += 32) {
        const float qv = to_f32(qp[e]), kv = to_f32(kp[e]);
        sq = fmaf(qv, qv, sq);
        sk = fmaf(kv, kv, sk);
        qk = fmaf(qv, kv, qk);
      }
      sq = warp_sum(sq);
      sk = warp_sum(sk);
      qk = warp_sum(qk);
      const float iq = q_scale / sqrtf(sq + unit_eps), ik = 1.0f / sqrtf(sk + unit_eps);
      for (int e = lane; e < dpad; e += 32) {
        const bool in = e < dim;
        qs[tt * dpad + e] = in ? to_f32(qp[e]) * iq : 0.f;
        ksm[tt * dpad + e] = in ? to_f32(kp[e]) * ik : 0.f;
      }
      if (lane == 0) kq[tt] = qk * iq * ik;
    }
    for (int idx = threadIdx.x; idx < n * cpb; idx += kDeltaThreads) {
      const int tt = idx / cpb, cc = idx - tt * cpb;
      vs[idx] = c0 + cc < vdim ? to_f32(v[(size_t)(t0 + tt) * v_stride + (size_t)h * vdim + c0 + cc]) : 0.f;
    }
    if (threadIdx.x < n) {
      gs[threadIdx.x] = decay[(size_t)(t0 + threadIdx.x) * H + h];
      bs[threadIdx.x] = beta[(size_t)(t0 + threadIdx.x) * H + h];
    }
    __syncthreads();
    for (int tt = 0; tt < n; ++tt) {
      const float gt = gs[tt];
      const float4* kt = reinterpret_cast<const float4*>(ksm + tt * dpad + e0);
      const float4* qt = reinterpret_cast<const float4*>(qs + tt * dpad + e0);
      float kk[EPL];
      float pk = 0.f, pq = 0.f;
#pragma unroll
      for (int i = 0; i < EPL / 4; ++i) {
        const float4 kv = kt[i], qv = qt[i];
        kk[4 * i] = kv.x; kk[4 * i + 1] = kv.y; kk[4 * i + 2] = kv.z; kk[4 * i + 3] = kv.w;
        pk = fmaf(S[4 * i], kv.x, pk); pk = fmaf(S[4 * i + 1], kv.y, pk); pk = fmaf(S[4 * i + 2], kv.z, pk); pk = fmaf(S[4 * i + 3], kv.w, pk);
        pq = fmaf(S[4 * i], qv.x, pq); pq = fmaf(S[4 * i + 1], qv.y, pq); pq = fmaf(S[4 * i + 2], qv.z, pq); pq = fmaf(S[4 * i + 3], qv.w, pq);
      }
      for (int o = lpc >> 1; o > 0; o >>= 1) {
        pk += __shfl_xor_sync(0xffffffffu, pk, o);
        pq += __shfl_xor_sync(0xffffffffu, pq, o);
      }
      const float u = bs[tt] * (vs[tt * cpb + cl] - gt * pk);
#pragma unroll
      for (int i = 0; i < EPL; ++i) S[i] = fmaf(gt, S[i], kk[i] * u);
      if (part == 0 && col_live) out[((size_t)(t0 + tt) * H + h) * vdim + c0 + cl] = fmaf(gt, pq, u * kq[tt]);
    }
  }
  if (end > beg) {
#pragma unroll
    for (int i = 0; i < EPL; ++i)
      if (col_live && e0 + i < dim) sp[e0 + i] = S[i];
  }
}

template <typename T, int EPL>
static int launch_delta(const void* q, const void* k, const void* v, int q_stride, int k_stride, int v_stride, const float* beta,
                        const float* decay, float* state, long slot_stride, const int* q_indptr, const int* state_slots, float* out,
                        int R, int H, int kq_heads, int dim, int vdim, float q_scale, float unit_eps, cudaStream_t s) {
  int lpc = 1;
  while (lpc * EPL < dim) lpc <<= 1;
  const int cpb = kDeltaThreads / lpc;
  const size_t smem = ((size_t)2 * kDeltaChunk * lpc * EPL + (size_t)kDeltaChunk * cpb + 3 * kDeltaChunk) * sizeof(float);
  if (smem > 200 * 1024) return ARLE_E_UNSUPPORTED;
  if (smem > 40 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(delta_scan_kernel<T, EPL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid((vdim + cpb - 1) / cpb, H, R);
  launch_kernel(delta_scan_kernel<T, EPL>, dim3(grid), dim3(kDeltaThreads), smem, s, 1, (const T*)q, (const T*)k, (const T*)v, q_stride,
                k_stride, v_stride, beta, decay, state, slot_stride, q_indptr, state_slots, out, H, kq_heads, dim, vdim, q_scale, unit_eps,
                lpc);
  return launch_status();
}

// q, k [T, kq_heads*dim] and v [T, H*vdim] in the activation type (row strides given); beta, decay float32 [T, H]; state:
// float32, a slot every slot_stride numbers, [H][vdim][dim] at its start; out float32 [T, H, vdim].
ARLE_API int arle_delta_scan(const void* q, const void* k, const void* v, int dtype, int q_stride, int k_stride, int v_stride,
                             const float* beta, const float* decay, float* state, long slot_stride, const int* q_indptr,
                             const int* state_slots, float* out, int R, int H, int kq_heads, int dim, int vdim, float q_scale,
                             float unit_eps, cudaStream_t s) {
  if (R <= 0) return 0;
  if (H <= 0 || kq_heads <= 0 || H % kq_heads || dim <= 0 || vdim <= 0 || H > 65535 || R > 65535) return ARLE_E_BADARG;
  if (dim > 32 * 16) return ARLE_E_UNSUPPORTED;
#define ARLE_DELTA(TT, E) \
  return launch_delta<TT, E>(q, k, v, q_stride, k_stride, v_stride, beta, decay, state, slot_stride, q_indptr, state_slots, out, R, H, \
                             kq_heads, dim, vdim, q_scale, unit_eps, s)
  if (dtype == 0) {
    if (dim <= 128) ARLE_DELTA(float, 4);
    if (dim <= 256) ARLE_DELTA(float, 8);
    ARLE_DELTA(float, 16);
  }
  if (dtype == 1) {
    if (dim <= 128) ARLE_DELTA(__nv_bfloat16, 4);
    if (dim <= 256) ARLE_DELTA(__nv_bfloat16, 8);
    ARLE_DELTA(__nv_bfloat16, 16);
  }
#undef ARLE_DELTA
  return ARLE_E_BADARG;
}
