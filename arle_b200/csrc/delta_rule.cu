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
//    the memory is kept transposed, [head][column][dim]) is held by LPC lanes, EPL numbers a lane in groups of four
//    (group i of lane p is numbers 4 (i LPC + p) ...: neighbouring lanes read neighbouring 16 bytes of the memory and of
//    the staged k and q).  Per token the lanes form their parts of S_old . k and S_old . q, add both by shuffles in one
//    round, and since S^T q = g S_old^T q + u (k . q) the read-out needs no second round.  16 tokens are staged in shared
//    memory at a time as they are; their unit lengths are three sums a token (q . q, k . k, q . k) and enter as factors
//    of the two products and of u.  Eight lanes a column (sixteen numbers a lane at dim 128) cost a third of the
//    instructions of thirty-two lanes with four numbers.  The split of a column depends on dim alone, so a token's sums
//    have one order whatever the cutting or the batch.
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

// LONG: the step has rows of many tokens (a chunk's loads asked for at once, a full chunk's tokens unrolled); without it the
// kernel is the short form for steps of single tokens, which needs fewer registers.
template <typename T, int EPL, int LPC, bool LONG>
__global__ void __launch_bounds__(256) delta_scan_kernel(
    const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, int q_stride, int k_stride, int v_stride,
    const float* __restrict__ beta, const float* __restrict__ decay, float* __restrict__ state, long slot_stride,
    const int* __restrict__ q_indptr, const int* __restrict__ state_slots, float* __restrict__ out, int H, int kq_heads, int dim,
    int vdim, float q_scale, float unit_eps) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float sm[];
  constexpr int DPAD = LPC * EPL;                        // a token's q or k in shared memory, zeros past dim
  constexpr int ROW = DPAD + 4;                          // its row there: sixteen rows are read side by side for the sums
  constexpr int NG = EPL / 4;                            // groups of four numbers a lane holds
  const int nthreads = blockDim.x;                       // 64, 128 or 256
  const int cpb = nthreads / LPC;                        // columns of S a block holds
  float* qs = sm;                                        // [chunk][ROW]
  float* ksm = qs + kDeltaChunk * ROW;                   // [chunk][ROW]
  float* vs = ksm + kDeltaChunk * ROW;                   // [chunk][cpb]
  float* gs = vs + kDeltaChunk * cpb;                    // [chunk] decay
  float* bs = gs + kDeltaChunk;                          // [chunk] beta
  float* kq = bs + kDeltaChunk;                          // [chunk] k . q of the unit vectors (q's scale included)
  float* iqs = kq + kDeltaChunk;                         // [chunk] q_scale / |q|
  float* iks = iqs + kDeltaChunk;                        // [chunk] 1 / |k|
  float* psum = iks + kDeltaChunk;                       // [3][8 warps][chunk] partial sums
  const int r = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * cpb;
  const int g = h / (H / kq_heads);
  const int cl = threadIdx.x / LPC, part = threadIdx.x % LPC;
  const int beg = q_indptr[r], end = q_indptr[r + 1];
  const bool col_live = c0 + cl < vdim;
  float* sp = state + (size_t)state_slots[r] * slot_stride + (size_t)h * vdim * dim + (size_t)(c0 + cl) * dim;
  const bool vec_state = dim % 4 == 0 && ((uintptr_t)sp & 15) == 0;
  float S[EPL];
#pragma unroll
  for (int i = 0; i < NG; ++i) {
    const int e = 4 * (i * LPC + part);
    if (col_live && vec_state && e < dim) {
      const float4 x = *reinterpret_cast<const float4*>(sp + e);
      S[4 * i] = x.x; S[4 * i + 1] = x.y; S[4 * i + 2] = x.z; S[4 * i + 3] = x.w;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) S[4 * i + j] = (col_live && e + j < dim) ? sp[e + j] : 0.f;
    }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = nthreads >> 5;
  const int stt = threadIdx.x & (kDeltaChunk - 1), sseg = threadIdx.x >> 4, nseg = nthreads >> 4;   // the sums: a token, a share of dim

  for (int t0 = beg; t0 < end; t0 += kDeltaChunk) {
    const int n = min(kDeltaChunk, end - t0);
    __syncthreads();
    for (int e = threadIdx.x; e < DPAD; e += nthreads) {
      const bool in = e < dim;
      const T* qp = q + (size_t)t0 * q_stride + (size_t)g * dim + e;
      const T* kp = k + (size_t)t0 * k_stride + (size_t)g * dim + e;
      if constexpr (LONG) {      // all of the chunk's loads are asked for before the first is used: one wait for memory a chunk
        T qv[kDeltaChunk], kv[kDeltaChunk];
#pragma unroll
        for (int tt = 0; tt < kDeltaChunk; ++tt) {
          const bool on = in && tt < n;
          qv[tt] = on ? qp[(size_t)tt * q_stride] : from_f32<T>(0.f);
          kv[tt] = on ? kp[(size_t)tt * k_stride] : from_f32<T>(0.f);
        }
#pragma unroll
        for (int tt = 0; tt < kDeltaChunk; ++tt) {
          qs[tt * ROW + e] = to_f32(qv[tt]);
          ksm[tt * ROW + e] = to_f32(kv[tt]);
        }
      } else {
        for (int tt = 0; tt < n; ++tt) {
          qs[tt * ROW + e] = in ? to_f32(qp[(size_t)tt * q_stride]) : 0.f;
          ksm[tt * ROW + e] = in ? to_f32(kp[(size_t)tt * k_stride]) : 0.f;
        }
      }
    }
    for (int idx = threadIdx.x; idx < n * cpb; idx += nthreads) {
      const int tt = idx / cpb, cc = idx - tt * cpb;
      vs[idx] = c0 + cc < vdim ? to_f32(v[(size_t)(t0 + tt) * v_stride + (size_t)h * vdim + c0 + cc]) : 0.f;
    }
    if (threadIdx.x < n) {
      gs[threadIdx.x] = decay[(size_t)(t0 + threadIdx.x) * H + h];
      bs[threadIdx.x] = beta[(size_t)(t0 + threadIdx.x) * H + h];
    }
    __syncthreads();
    {
      float sq = 0.f, sk = 0.f, qk = 0.f;
      if (stt < n)
        for (int e = sseg; e < dim; e += nseg) {
          const float qv = qs[stt * ROW + e], kv = ksm[stt * ROW + e];
          sq = fmaf(qv, qv, sq);
          sk = fmaf(kv, kv, sk);
          qk = fmaf(qv, kv, qk);
        }
      sq += __shfl_xor_sync(0xffffffffu, sq, 16);          // a warp holds two shares of each of the sixteen tokens
      sk += __shfl_xor_sync(0xffffffffu, sk, 16);
      qk += __shfl_xor_sync(0xffffffffu, qk, 16);
      if (lane < kDeltaChunk) {
        psum[(0 * 8 + warp) * kDeltaChunk + lane] = sq;
        psum[(1 * 8 + warp) * kDeltaChunk + lane] = sk;
        psum[(2 * 8 + warp) * kDeltaChunk + lane] = qk;
      }
    }
    __syncthreads();
    if (threadIdx.x < n) {
      float sq = 0.f, sk = 0.f, qk = 0.f;
      for (int w = 0; w < nwarps; ++w) {
        sq += psum[(0 * 8 + w) * kDeltaChunk + threadIdx.x];
        sk += psum[(1 * 8 + w) * kDeltaChunk + threadIdx.x];
        qk += psum[(2 * 8 + w) * kDeltaChunk + threadIdx.x];
      }
      const float iq = q_scale / sqrtf(sq + unit_eps), ik = 1.0f / sqrtf(sk + unit_eps);
      iqs[threadIdx.x] = iq;
      iks[threadIdx.x] = ik;
      kq[threadIdx.x] = qk * iq * ik;
    }
    __syncthreads();
    auto step = [&](int tt) {
      const float gt = gs[tt], ik = iks[tt];
      const float4* kt = reinterpret_cast<const float4*>(ksm + tt * ROW) + part;
      const float4* qt = reinterpret_cast<const float4*>(qs + tt * ROW) + part;
      float kk[EPL];
      float pk0 = 0.f, pk1 = 0.f, pk2 = 0.f, pk3 = 0.f, pq0 = 0.f, pq1 = 0.f, pq2 = 0.f, pq3 = 0.f;
#pragma unroll
      for (int i = 0; i < NG; ++i) {
        const float4 kv = kt[i * LPC], qv = qt[i * LPC];
        kk[4 * i] = kv.x; kk[4 * i + 1] = kv.y; kk[4 * i + 2] = kv.z; kk[4 * i + 3] = kv.w;
        pk0 = fmaf(S[4 * i], kv.x, pk0); pk1 = fmaf(S[4 * i + 1], kv.y, pk1); pk2 = fmaf(S[4 * i + 2], kv.z, pk2); pk3 = fmaf(S[4 * i + 3], kv.w, pk3);
        pq0 = fmaf(S[4 * i], qv.x, pq0); pq1 = fmaf(S[4 * i + 1], qv.y, pq1); pq2 = fmaf(S[4 * i + 2], qv.z, pq2); pq3 = fmaf(S[4 * i + 3], qv.w, pq3);
      }
      float pk = (pk0 + pk1) + (pk2 + pk3), pq = (pq0 + pq1) + (pq2 + pq3);
#pragma unroll
      for (int o = LPC >> 1; o > 0; o >>= 1) {
        pk += __shfl_xor_sync(0xffffffffu, pk, o);
        pq += __shfl_xor_sync(0xffffffffu, pq, o);
      }
      const float u = bs[tt] * (vs[tt * cpb + cl] - gt * (ik * pk));
      const float uk = u * ik;
#pragma unroll
      for (int i = 0; i < EPL; ++i) S[i] = fmaf(gt, S[i], kk[i] * uk);
      if (part == 0 && col_live) out[((size_t)(t0 + tt) * H + h) * vdim + c0 + cl] = fmaf(gt * iqs[tt], pq, u * kq[tt]);
    };
    if (LONG && n == kDeltaChunk) {                      // a full chunk unrolled: a token's loads from shared memory run ahead of
#pragma unroll                                          // the tokens before it, whose sums wait on one another
      for (int tt = 0; tt < kDeltaChunk; ++tt) step(tt);
    } else {
      for (int tt = 0; tt < n; ++tt) step(tt);
    }
  }
  if (end > beg && col_live) {
#pragma unroll
    for (int i = 0; i < NG; ++i) {
      const int e = 4 * (i * LPC + part);
      if (vec_state && e < dim) {
        *reinterpret_cast<float4*>(sp + e) = make_float4(S[4 * i], S[4 * i + 1], S[4 * i + 2], S[4 * i + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (e + j < dim) sp[e + j] = S[4 * i + j];
      }
    }
  }
}

template <typename T, int EPL, int LPC, bool LONG>
static int launch_delta(const void* q, const void* k, const void* v, int q_stride, int k_stride, int v_stride, const float* beta,
                        const float* decay, float* state, long slot_stride, const int* q_indptr, const int* state_slots, float* out,
                        int R, int H, int kq_heads, int dim, int vdim, float q_scale, float unit_eps, cudaStream_t s) {
  // 128 threads a block while the step's blocks are few; twice the columns share the staging of a head's q and k once the
  // SMs are full
  int threads = 128;
  while (threads < 256 && (long)((vdim + threads / LPC - 1) / (threads / LPC)) * H * R > 4L * 148) threads <<= 1;
  const int cpb = threads / LPC;
  const size_t smem = ((size_t)2 * kDeltaChunk * (LPC * EPL + 4) + (size_t)kDeltaChunk * cpb + 5 * kDeltaChunk + 3 * 8 * kDeltaChunk) * sizeof(float);
  if (smem > 200 * 1024) return ARLE_E_UNSUPPORTED;
  if (smem > 40 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(delta_scan_kernel<T, EPL, LPC, LONG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid((vdim + cpb - 1) / cpb, H, R);
  launch_kernel(delta_scan_kernel<T, EPL, LPC, LONG>, dim3(grid), dim3(threads), smem, s, 1, (const T*)q, (const T*)k, (const T*)v, q_stride,
                k_stride, v_stride, beta, decay, state, slot_stride, q_indptr, state_slots, out, H, kq_heads, dim, vdim, q_scale, unit_eps);
  return launch_status();
}

// q, k [T, kq_heads*dim] and v [T, H*vdim] in the activation type (row strides given); beta, decay float32 [T, H]; state:
// float32, a slot every slot_stride numbers, [H][vdim][dim] at its start; out float32 [T, H, vdim]; num_tokens: T, all rows'.
ARLE_API int arle_delta_scan(const void* q, const void* k, const void* v, int dtype, int q_stride, int k_stride, int v_stride,
                             const float* beta, const float* decay, float* state, long slot_stride, const int* q_indptr,
                             const int* state_slots, float* out, int num_tokens, int R, int H, int kq_heads, int dim, int vdim,
                             float q_scale, float unit_eps, cudaStream_t s) {
  if (R <= 0 || num_tokens <= 0) return 0;
  if (H <= 0 || kq_heads <= 0 || H % kq_heads || dim <= 0 || vdim <= 0 || H > 65535 || R > 65535) return ARLE_E_BADARG;
  if (dim > 512) return ARLE_E_UNSUPPORTED;
  const bool long_rows = num_tokens >= 2 * R + kDeltaChunk;       // some row has a full chunk, or nearly
#define ARLE_DELTA(TT, E, L)                                                                                                           \
  return long_rows ? launch_delta<TT, E, L, true>(q, k, v, q_stride, k_stride, v_stride, beta, decay, state, slot_stride, q_indptr,     \
                                                  state_slots, out, R, H, kq_heads, dim, vdim, q_scale, unit_eps, s)                    \
                   : launch_delta<TT, E, L, false>(q, k, v, q_stride, k_stride, v_stride, beta, decay, state, slot_stride, q_indptr,    \
                                                   state_slots, out, R, H, kq_heads, dim, vdim, q_scale, unit_eps, s)
#define ARLE_DELTA_BY_DIM(TT)          \
  if (dim <= 8) ARLE_DELTA(TT, 4, 2);   \
  if (dim <= 32) ARLE_DELTA(TT, 4, 8);  \
  if (dim <= 64) ARLE_DELTA(TT, 8, 8);  \
  if (dim <= 128) ARLE_DELTA(TT, 16, 8); \
  if (dim <= 256) ARLE_DELTA(TT, 32, 8); \
  ARLE_DELTA(TT, 16, 32)
  if (dtype == 0) {
    ARLE_DELTA_BY_DIM(float);
  }
  if (dtype == 1) {
    ARLE_DELTA_BY_DIM(__nv_bfloat16);
  }
#undef ARLE_DELTA_BY_DIM
#undef ARLE_DELTA
  return ARLE_E_BADARG;
}
