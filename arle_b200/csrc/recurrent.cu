// Recurrent mixers whose memory is one matrix per head with a scalar decay per token:
//
//     S_t = a_t S_(t-1) + b_t k_t v_t^T,        o_t = S_t^T q_t          (S: dim x vcols, float32)
//
// a_t and b_t are one number per (token, head), prepared in float32 by the mixer's own gate kernel.  The matrix
// memory of xLSTM (a = exp(f + m_(t-1) - m_t), b = exp(i - m_t), and a column of ones beside v that carries the
// normaliser n_t) and the state-space recurrence of Mamba-2 (a = exp(-exp(A_log) dt), b = dt, k = B, q = C shared
// by the heads of a group) are both this recurrence, so they share decay_scan.  Everything here is float32
// arithmetic whatever the activation type; the state lives in the request's slot of the cache manager's state
// arena and is carried from step to step.
//
//  * decay_scan: a block per (row of the step, head, tile of columns).  A column of S (dim numbers, stored
//    contiguously: the state is kept transposed, [head][column][dim]) is held by `lpc` lanes, EPL numbers a lane;
//    the lanes add their parts of o_t by shuffles; a thread holds one column, or four that share its loads of k and q.
//    q, k, b v and a of 16 tokens are staged in shared memory, then the 16 steps run from there, while the next 16 tokens'
//    numbers are already on their way into registers.  The split of a column depends on dim alone, so a token's sums have one order
//    whatever the cutting or the batch.
//  * mlstm_gates: the log gates of the matrix LSTM (soft-capped), its running maximum m (carried in the state),
//    and from them a_t, b_t and exp(-m_t); the gates of 128 tokens are evaluated side by side, the maximum runs
//    through them in order.
//  * mlstm_out: o / (max(|n . q|, exp(-m)) + 1e-6), each head divided by its root mean square, times the weight,
//    times sigmoid(gate).
//  * ssm_gates: dt = softplus(dt_raw + bias), a = exp(-exp(A_log) dt), b = dt.
//  * conv_silu: a causal convolution per channel over a row's tokens (the last tap is the current token's; before
//    a request's first token stand zeros), bias, silu; the last taps - 1 inputs of every request live in its
//    state slot, are read by the first tokens of the next portion and are brought up to date by a second launch.
//  * gated_group_norm: (y + D x) * silu(z), RMS-normed in equal parts of the row, times a weight.
#include "common.cuh"
using namespace arle;

constexpr int kScanChunk = 16;
constexpr int kScanThreads = 256;

// AHEAD: the variant that asks for the next chunk while this one's steps run (steps of prompt portions; it holds more registers,
// which a step of decoded tokens, bound by reading and writing the memories, pays for in blocks per SM).
template <typename T, int EPL, int CPT, bool AHEAD>
__global__ void __launch_bounds__(kScanThreads) decay_scan_kernel(
    const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, int q_stride, int k_stride, int v_stride,
    const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ state, long slot_stride,
    const int* __restrict__ q_indptr, const int* __restrict__ state_slots, float* __restrict__ out, int H, int kq_heads,
    int dim, int vdim, int ones_col, float q_scale, int lpc, int ab_stride, int act) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float sm[];
  const int cpb = kScanThreads / lpc * CPT;              // columns of S a block holds: CPT to a thread
  const int dpad = lpc * EPL;                            // a token's q or k in shared memory, padded with zeros to the lanes' shares
  float* qs = sm;                                        // [chunk][dpad]
  float* ksm = qs + kScanChunk * dpad;                   // [chunk][dpad]
  float* vs = ksm + kScanChunk * dpad;                   // [chunk][cpb], already times b
  float* as = vs + kScanChunk * cpb;                     // [chunk]
  const int r = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * cpb;
  const int vcols = vdim + ones_col;
  const int g = h / (H / kq_heads);
  const int cl0 = threadIdx.x / lpc * CPT, part = threadIdx.x % lpc;      // the thread's first column inside the block
  const int e0 = part * EPL;
  const int beg = q_indptr[r], end = q_indptr[r + 1];
  float* sp = state + (size_t)state_slots[r] * slot_stride + (size_t)h * vcols * dim;
  float S[CPT][EPL];
#pragma unroll
  for (int j = 0; j < CPT; ++j)
#pragma unroll
    for (int i = 0; i < EPL; ++i) S[j][i] = (c0 + cl0 + j < vcols && e0 + i < dim) ? sp[(size_t)(c0 + cl0 + j) * dim + e0 + i] : 0.f;

  // Rows of more than one chunk: the NEXT chunk's q, k, v, a and b are asked for before this chunk's steps run and wait in
  // registers (as they lie in memory) until the steps are done; the chain of steps then never waits for memory.  A thread
  // holds at most NQ numbers of q and of k (16 tokens x 32 lanes x EPL / 256 threads) and NV of v.
  constexpr int NQ = 2 * EPL;
  constexpr int NV = 2;
  constexpr bool PRE = AHEAD;
  const bool pre = PRE && end - beg > kScanChunk;       // a row of one chunk (a decoded token) has nothing to ask for ahead
  const bool vpre = pre && kScanChunk * cpb <= NV * kScanThreads;
  const int dshift = __ffs(dpad) - 1;                    // dpad is a power of two
  T rq[PRE ? NQ : 1], rk[PRE ? NQ : 1], rv[NV];
  float rb[NV], ra = 0.f;
  auto ask = [&](int t0, int n) {
#pragma unroll
    for (int i = 0; i < NQ; ++i) {
      const int idx = threadIdx.x + i * kScanThreads;
      const int tt = idx >> dshift, e = idx & (dpad - 1);
      const bool in = idx < n * dpad && e < dim;
      rq[i] = in ? q[(size_t)(t0 + tt) * q_stride + (size_t)g * dim + e] : from_f32<T>(0.f);
      rk[i] = in ? k[(size_t)(t0 + tt) * k_stride + (size_t)g * dim + e] : from_f32<T>(0.f);
    }
    if (vpre) {
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int idx = threadIdx.x + i * kScanThreads;
        const int tt = idx / cpb, c = c0 + idx - tt * cpb;
        const bool in = idx < n * cpb;
        rv[i] = (in && c < vdim) ? v[(size_t)(t0 + tt) * v_stride + (size_t)h * vdim + c] : from_f32<T>(0.f);
        rb[i] = (in && b) ? b[(size_t)(t0 + tt) * ab_stride + h] : 1.f;
      }
    }
    if (threadIdx.x < n) ra = a[(size_t)(t0 + threadIdx.x) * ab_stride + h];
  };
  if (pre) ask(beg, kScanChunk);

  for (int t0 = beg; t0 < end; t0 += kScanChunk) {
    const int n = min(kScanChunk, end - t0);
    __syncthreads();
    if (pre) {
#pragma unroll
      for (int i = 0; i < NQ; ++i) {
        const int idx = threadIdx.x + i * kScanThreads;
        if (idx < n * dpad) {
          float qv = to_f32(rq[i]), kv = to_f32(rk[i]);  // zero past dim
          if (act) {
            qv = qv / (1.0f + expf(-qv));
            kv = kv / (1.0f + expf(-kv));
          }
          qs[idx] = qv * q_scale;
          ksm[idx] = kv;
        }
      }
      if (threadIdx.x < n) as[threadIdx.x] = ra;
    } else {
      for (int idx = threadIdx.x; idx < n * dpad; idx += kScanThreads) {
        const int tt = idx / dpad, e = idx - tt * dpad;
        const bool in = e < dim;
        float qv = in ? to_f32(q[(size_t)(t0 + tt) * q_stride + (size_t)g * dim + e]) : 0.f;
        float kv = in ? to_f32(k[(size_t)(t0 + tt) * k_stride + (size_t)g * dim + e]) : 0.f;
        if (act) {
          qv = qv / (1.0f + expf(-qv));
          kv = kv / (1.0f + expf(-kv));
        }
        qs[idx] = qv * q_scale;
        ksm[idx] = kv;
      }
      if (threadIdx.x < n) as[threadIdx.x] = a[(size_t)(t0 + threadIdx.x) * ab_stride + h];
    }
    if (vpre) {
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int idx = threadIdx.x + i * kScanThreads;
        if (idx < n * cpb) {
          const int tt = idx / cpb, c = c0 + idx - tt * cpb;
          float vv = c < vdim ? to_f32(rv[i]) : (c == vdim && ones_col ? 1.f : 0.f);
          if (act && c < vdim) vv = vv / (1.0f + expf(-vv));
          vs[idx] = rb[i] * vv;
        }
      }
    } else {
      for (int idx = threadIdx.x; idx < n * cpb; idx += kScanThreads) {
        const int tt = idx / cpb, cc = idx - tt * cpb;
        const int c = c0 + cc;
        float vv = c < vdim ? to_f32(v[(size_t)(t0 + tt) * v_stride + (size_t)h * vdim + c]) : (c == vdim && ones_col ? 1.f : 0.f);
        if (act && c < vdim) vv = vv / (1.0f + expf(-vv));
        vs[idx] = b ? b[(size_t)(t0 + tt) * ab_stride + h] * vv : vv;
      }
    }
    __syncthreads();
    if (pre && t0 + kScanChunk < end) ask(t0 + kScanChunk, min(kScanChunk, end - t0 - kScanChunk));
    for (int tt = 0; tt < n; ++tt) {
      const float at = as[tt];
      float bv[CPT], p[CPT];
#pragma unroll
      for (int j = 0; j < CPT; ++j) {
        bv[j] = vs[tt * cpb + cl0 + j];
        p[j] = 0.f;
      }
      const float4* kt = reinterpret_cast<const float4*>(ksm + tt * dpad + e0);
      const float4* qt = reinterpret_cast<const float4*>(qs + tt * dpad + e0);
#pragma unroll
      for (int i = 0; i < EPL / 4; ++i) {
        const float4 kv = kt[i], qv = qt[i];
#pragma unroll
        for (int j = 0; j < CPT; ++j) {
          S[j][4 * i] = fmaf(at, S[j][4 * i], bv[j] * kv.x);
          p[j] = fmaf(S[j][4 * i], qv.x, p[j]);
          S[j][4 * i + 1] = fmaf(at, S[j][4 * i + 1], bv[j] * kv.y);
          p[j] = fmaf(S[j][4 * i + 1], qv.y, p[j]);
          S[j][4 * i + 2] = fmaf(at, S[j][4 * i + 2], bv[j] * kv.z);
          p[j] = fmaf(S[j][4 * i + 2], qv.z, p[j]);
          S[j][4 * i + 3] = fmaf(at, S[j][4 * i + 3], bv[j] * kv.w);
          p[j] = fmaf(S[j][4 * i + 3], qv.w, p[j]);
        }
      }
      for (int o = lpc >> 1; o > 0; o >>= 1) {
#pragma unroll
        for (int j = 0; j < CPT; ++j) p[j] += __shfl_xor_sync(0xffffffffu, p[j], o);
      }
      if (part == 0) {
        float* op = out + ((size_t)(t0 + tt) * H + h) * vcols + c0 + cl0;
#pragma unroll
        for (int j = 0; j < CPT; ++j)
          if (c0 + cl0 + j < vcols) op[j] = p[j];
      }
    }
  }
#pragma unroll
  for (int j = 0; j < CPT; ++j)
#pragma unroll
    for (int i = 0; i < EPL; ++i)
      if (c0 + cl0 + j < vcols && e0 + i < dim) sp[(size_t)(c0 + cl0 + j) * dim + e0 + i] = S[j][i];
}

template <typename T, int EPL, int CPT>
static int launch_scan_as(const void* q, const void* k, const void* v, int q_stride, int k_stride, int v_stride, const float* a,
                          const float* b, float* state, long slot_stride, const int* q_indptr, const int* state_slots, float* out,
                          int R, int H, int kq_heads, int dim, int vdim, int ones_col, float q_scale, int lpc, int ab_stride, int act, bool ahead,
                          cudaStream_t s) {
  const int cpb = kScanThreads / lpc * CPT;
  const int vcols = vdim + ones_col;
  const size_t smem = ((size_t)2 * kScanChunk * lpc * EPL + (size_t)kScanChunk * cpb + kScanChunk) * sizeof(float);
  if (smem > 200 * 1024) return ARLE_E_UNSUPPORTED;
  // four numbers a lane (columns of up to 128) gain from asking ahead; eight a lane were measured slower with it
  auto kernel = (ahead && EPL == 4) ? decay_scan_kernel<T, EPL, CPT, EPL == 4> : decay_scan_kernel<T, EPL, CPT, false>;
  if (smem > 40 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid((vcols + cpb - 1) / cpb, H, R);
  launch_kernel(kernel, dim3(grid), dim3(kScanThreads), smem, s, 1, (const T*)q, (const T*)k, (const T*)v,
                q_stride, k_stride, v_stride, a, b, state, slot_stride, q_indptr, state_slots, out, H, kq_heads, dim, vdim, ones_col,
                q_scale, lpc, ab_stride, act);
  return launch_status();
}

// Four columns to a thread (they share the loads of k and q) where that still leaves a block for every SM; one otherwise.
// A column's arithmetic is the same either way.
template <typename T, int EPL>
static int launch_scan(const void* q, const void* k, const void* v, int q_stride, int k_stride, int v_stride, const float* a,
                       const float* b, float* state, long slot_stride, const int* q_indptr, const int* state_slots, float* out,
                       int R, int H, int kq_heads, int dim, int vdim, int ones_col, float q_scale, int ab_stride, int act, bool ahead, cudaStream_t s) {
  int lpc = 1;
  while (lpc * EPL < dim) lpc <<= 1;
  const int wide = kScanThreads / lpc * 4;
  const long blocks_wide = (long)((vdim + ones_col + wide - 1) / wide) * H * R;
  if (blocks_wide >= 148)
    return launch_scan_as<T, EPL, 4>(q, k, v, q_stride, k_stride, v_stride, a, b, state, slot_stride, q_indptr, state_slots, out, R, H,
                                     kq_heads, dim, vdim, ones_col, q_scale, lpc, ab_stride, act, ahead, s);
  return launch_scan_as<T, EPL, 1>(q, k, v, q_stride, k_stride, v_stride, a, b, state, slot_stride, q_indptr, state_slots, out, R, H,
                                   kq_heads, dim, vdim, ones_col, q_scale, lpc, ab_stride, act, ahead, s);
}

// q, k [T, kq_heads*dim] and v [T, H*vdim] in the activation type (row strides given); a, b float32 [T, H] (ab_stride = H), or
// one number a head for all tokens (ab_stride = 0: a float32 [H], b float32 [H] or null for ones: a memory with a constant
// decay per head); act 1: silu on q, k and v as they are staged; long_rows: the step's rows are mostly longer than a chunk of
// 16 tokens (a hint: the variant that asks for the next chunk ahead is launched); state: float32,
// a slot every slot_stride numbers, [H][vdim + ones_col][dim] at its start; out float32 [T, H, vdim + ones_col].
ARLE_API int arle_decay_scan(const void* q, const void* k, const void* v, int dtype, int q_stride, int k_stride, int v_stride,
                             const float* a, const float* b, float* state, long slot_stride, const int* q_indptr,
                             const int* state_slots, float* out, int R, int H, int kq_heads, int dim, int vdim, int ones_col,
                             float q_scale, int ab_stride, int act, int long_rows, cudaStream_t s) {
  if (R <= 0) return 0;
  if (!a || (ab_stride != 0 && ab_stride != H) || (act != 0 && act != 1)) return ARLE_E_BADARG;
  if (H <= 0 || kq_heads <= 0 || H % kq_heads || dim <= 0 || vdim <= 0 || H > 65535 || R > 65535) return ARLE_E_BADARG;
  if (dim > 32 * 16) return ARLE_E_UNSUPPORTED;
#define ARLE_SCAN(TT, E) \
  return launch_scan<TT, E>(q, k, v, q_stride, k_stride, v_stride, a, b, state, slot_stride, q_indptr, state_slots, out, R, H, \
                            kq_heads, dim, vdim, ones_col, q_scale, ab_stride, act, long_rows != 0, s)
  // numbers of a column a lane holds: 4 up to 128 (eight at 128, with 16 lanes a column, measured 1.25 to 2 times slower)
  if (dtype == 0) {
    if (dim <= 128) ARLE_SCAN(float, 4);
    if (dim <= 256) ARLE_SCAN(float, 8);
    ARLE_SCAN(float, 16);
  }
  if (dtype == 1) {
    if (dim <= 128) ARLE_SCAN(__nv_bfloat16, 4);
    if (dim <= 256) ARLE_SCAN(__nv_bfloat16, 8);
    ARLE_SCAN(__nv_bfloat16, 16);
  }
#undef ARLE_SCAN
  return ARLE_E_BADARG;
}

// ------------------------------------------------------------------------------------------------ matrix LSTM
__device__ __forceinline__ float log_sigmoid(float z) { return z >= 0.f ? -log1pf(expf(-z)) : z - log1pf(expf(z)); }

constexpr int kGateChunk = 128;

// pre: float32 [T, 2H], the input gates' sums before the bias, then the forget gates'.  m lives at state[slot][m_off + h].
__global__ void __launch_bounds__(kGateChunk) mlstm_gates_kernel(const float* __restrict__ pre, int pre_stride,
                                                                  const float* __restrict__ bias_i, const float* __restrict__ bias_f,
                                                                  float cap, const int* __restrict__ q_indptr,
                                                                  const int* __restrict__ state_slots, float* __restrict__ state,
                                                                  long slot_stride, long m_off, float* __restrict__ a,
                                                                  float* __restrict__ b, float* __restrict__ floor_, int H) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float gi[kGateChunk], gf[kGateChunk], mprev[kGateChunk], mnew[kGateChunk];
  const int r = blockIdx.y, h = blockIdx.x;
  const int beg = q_indptr[r], end = q_indptr[r + 1];
  float* mp = state + (size_t)state_slots[r] * slot_stride + m_off + h;
  float m = *mp;                                   // read by every thread, used by thread 0
  const float bi = bias_i ? bias_i[h] : 0.f, bf = bias_f ? bias_f[h] : 0.f;
  for (int t0 = beg; t0 < end; t0 += kGateChunk) {
    const int n = min(kGateChunk, end - t0);
    const int tt = threadIdx.x;
    float i_t = 0.f, f_t = 0.f;
    if (tt < n) {
      const float* p = pre + (size_t)(t0 + tt) * pre_stride;
      i_t = cap * tanhf((p[h] + bi) / cap);
      f_t = log_sigmoid(cap * tanhf((p[H + h] + bf) / cap));
      gi[tt] = i_t;
      gf[tt] = f_t;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int j = 0; j < n; ++j) {
        mprev[j] = m;
        m = fmaxf(gf[j] + m, gi[j]);
        mnew[j] = m;
      }
    }
    __syncthreads();
    if (tt < n) {
      const size_t o = (size_t)(t0 + tt) * H + h;
      a[o] = expf(f_t + mprev[tt] - mnew[tt]);
      b[o] = expf(i_t - mnew[tt]);
      floor_[o] = expf(-mnew[tt]);
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) *mp = m;
}

ARLE_API int arle_mlstm_gates(const float* pre, int pre_stride, const float* bias_i, const float* bias_f, float cap,
                              const int* q_indptr, const int* state_slots, float* state, long slot_stride, long m_off, float* a,
                              float* b, float* floor_, int R, int H, cudaStream_t s) {
  if (R <= 0) return 0;
  if (H <= 0 || R > 65535 || !(cap > 0.f)) return ARLE_E_BADARG;
  launch_kernel(mlstm_gates_kernel, dim3(H, R), dim3(kGateChunk), 0, s, 1, pre, pre_stride, bias_i, bias_f, cap, q_indptr, state_slots,
                state, slot_stride, m_off, a, b, floor_, H);
  return launch_status();
}

template <typename T>
__global__ void mlstm_out_kernel(const float* __restrict__ num, const float* __restrict__ floor_, const T* __restrict__ gate,
                                 int gate_stride, const float* __restrict__ weight, float eps, T* __restrict__ out, int out_stride,
                                 int H, int vdim) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[33];
  const int t = blockIdx.x, h = blockIdx.y;
  const float* np = num + ((size_t)t * H + h) * (vdim + 1);
  const float inv_den = 1.0f / (fmaxf(fabsf(np[vdim]), floor_[(size_t)t * H + h]) + 1e-6f);
  float ss = 0.f;
  for (int c = threadIdx.x; c < vdim; c += blockDim.x) {
    const float o = np[c] * inv_den;
    ss += o * o;
  }
  const float total = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(total / (float)vdim + eps);
  for (int c = threadIdx.x; c < vdim; c += blockDim.x) {
    const float o = np[c] * inv_den * inv * weight[h * vdim + c];
    const float gz = to_f32(gate[(size_t)t * gate_stride + h * vdim + c]);
    out[(size_t)t * out_stride + h * vdim + c] = from_f32<T>(o / (1.0f + expf(-gz)));
  }
}

ARLE_API int arle_mlstm_out(const float* num, const float* floor_, const void* gate, int dtype, int gate_stride, const float* weight,
                            float eps, void* out, int out_stride, int num_tokens, int H, int vdim, cudaStream_t s) {
  if (num_tokens <= 0) return 0;
  if (H <= 0 || H > 65535 || vdim <= 0) return ARLE_E_BADARG;
  const int threads = vdim >= 256 ? 128 : (vdim >= 64 ? 64 : 32);
  if (dtype == 0)
    launch_kernel(mlstm_out_kernel<float>, dim3(num_tokens, H), dim3(threads), 0, s, 1, num, floor_, (const float*)gate, gate_stride,
                  weight, eps, (float*)out, out_stride, H, vdim);
  else if (dtype == 1)
    launch_kernel(mlstm_out_kernel<__nv_bfloat16>, dim3(num_tokens, H), dim3(threads), 0, s, 1, num, floor_, (const __nv_bfloat16*)gate,
                  gate_stride, weight, eps, (__nv_bfloat16*)out, out_stride, H, vdim);
  else
    return ARLE_E_BADARG;
  return launch_status();
}

// ------------------------------------------------------------------------------------------------ state space
__global__ void ssm_gates_kernel(const float* __restrict__ dt_raw, int dt_stride, const float* __restrict__ dt_bias,
                                 const float* __restrict__ a_log, float* __restrict__ a, float* __restrict__ b, int H, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / H;
    const int h = (int)(idx - t * H);
    const float z = dt_raw[t * dt_stride + h] + dt_bias[h];
    const float dt = z > 20.f ? z : log1pf(expf(z));
    a[idx] = expf(-expf(a_log[h]) * dt);
    b[idx] = dt;
  }
}

ARLE_API int arle_ssm_gates(const float* dt_raw, int dt_stride, const float* dt_bias, const float* a_log, float* a, float* b,
                            int num_tokens, int H, cudaStream_t s) {
  if (num_tokens <= 0) return 0;
  if (H <= 0) return ARLE_E_BADARG;
  const size_t total = (size_t)num_tokens * H;
  size_t blocks = (total + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  launch_kernel(ssm_gates_kernel, dim3((int)blocks), dim3(256), 0, s, 1, dt_raw, dt_stride, dt_bias, a_log, a, b, H, total);
  return launch_status();
}

// x: the convolution's input channels of this step's tokens [T, C] (row stride given); the request's last taps - 1 inputs
// at state[slot][conv_off + c * (taps - 1) + j], oldest first.
template <typename T>
__global__ void conv_silu_kernel(const T* __restrict__ x, int x_stride, const float* __restrict__ w, const float* __restrict__ bias,
                                 const float* __restrict__ state, long slot_stride, long conv_off, const int* __restrict__ q_indptr,
                                 const int* __restrict__ row_of_token, const int* __restrict__ state_slots, T* __restrict__ out,
                                 int out_stride, int C, int taps) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int r = row_of_token[t];
  const int beg = q_indptr[r];
  const int local = t - beg;
  const float* st = state + (size_t)state_slots[r] * slot_stride + conv_off + (size_t)c * (taps - 1);
  float acc = bias ? bias[c] : 0.f;
  for (int j = 0; j < taps; ++j) {
    const int src = local - (taps - 1) + j;
    const float xv = src >= 0 ? to_f32(x[(size_t)(beg + src) * x_stride + c]) : st[src + taps - 1];
    acc = fmaf(w[(size_t)c * taps + j], xv, acc);
  }
  out[(size_t)t * out_stride + c] = from_f32<T>(acc / (1.0f + expf(-acc)));
}

template <typename T>
__global__ void conv_state_kernel(const T* __restrict__ x, int x_stride, float* __restrict__ state, long slot_stride, long conv_off,
                                  const int* __restrict__ q_indptr, const int* __restrict__ state_slots, int C, int taps) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int beg = q_indptr[r], n = q_indptr[r + 1] - beg;
  if (n <= 0) return;
  float* st = state + (size_t)state_slots[r] * slot_stride + conv_off + (size_t)c * (taps - 1);
  for (int j = 0; j < taps - 1; ++j) {                 // ascending: st[j] is written after st[j + n] was read
    const int src = n + j - (taps - 1);                // index among this step's tokens of the row
    st[j] = src >= 0 ? to_f32(x[(size_t)(beg + src) * x_stride + c]) : st[src + taps - 1];
  }
}

ARLE_API int arle_conv_silu(const void* x, int dtype, int x_stride, const float* w, const float* bias, float* state, long slot_stride,
                            long conv_off, const int* q_indptr, const int* row_of_token, const int* state_slots, void* out,
                            int out_stride, int num_tokens, int R, int C, int taps, cudaStream_t s) {
  if (num_tokens <= 0) return 0;
  if (C <= 0 || taps <= 0 || R <= 0) return ARLE_E_BADARG;
  const int threads = 128;
  const int cb = (C + threads - 1) / threads;
  if (cb > 65535) return ARLE_E_UNSUPPORTED;
  if (dtype == 0) {
    launch_kernel(conv_silu_kernel<float>, dim3(num_tokens, cb), dim3(threads), 0, s, 1, (const float*)x, x_stride, w, bias,
                  (const float*)state, slot_stride, conv_off, q_indptr, row_of_token, state_slots, (float*)out, out_stride, C, taps);
    if (taps > 1)
      launch_kernel(conv_state_kernel<float>, dim3(R, cb), dim3(threads), 0, s, 1, (const float*)x, x_stride, state, slot_stride,
                    conv_off, q_indptr, state_slots, C, taps);
  } else if (dtype == 1) {
    launch_kernel(conv_silu_kernel<__nv_bfloat16>, dim3(num_tokens, cb), dim3(threads), 0, s, 1, (const __nv_bfloat16*)x, x_stride, w,
                  bias, (const float*)state, slot_stride, conv_off, q_indptr, row_of_token, state_slots, (__nv_bfloat16*)out,
                  out_stride, C, taps);
    if (taps > 1)
      launch_kernel(conv_state_kernel<__nv_bfloat16>, dim3(R, cb), dim3(threads), 0, s, 1, (const __nv_bfloat16*)x, x_stride, state,
                    slot_stride, conv_off, q_indptr, state_slots, C, taps);
  } else {
    return ARLE_E_BADARG;
  }
  return launch_status();
}

// y float32 [T, inner]; x, z in the activation type (row strides given); skip[head] with head = column / vdim (or no skip);
// the row in `parts` equal parts, each divided by its own root mean square.
template <typename T>
__global__ void gated_group_norm_kernel(const float* __restrict__ y, const T* __restrict__ x, int x_stride,
                                        const float* __restrict__ skip, int vdim, const T* __restrict__ z, int z_stride,
                                        const float* __restrict__ weight, float eps, T* __restrict__ out, int out_stride, int inner,
                                        int parts) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[33];
  const int t = blockIdx.x, part = blockIdx.y;
  const int width = inner / parts, c0 = part * width;
  const float* yr = y + (size_t)t * inner;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const int c = c0 + i;
    float val = yr[c];
    if (skip) val = fmaf(skip[c / vdim], to_f32(x[(size_t)t * x_stride + c]), val);
    const float g = to_f32(z[(size_t)t * z_stride + c]);
    val *= g / (1.0f + expf(-g));
    ss += val * val;
  }
  const float total = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(total / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const int c = c0 + i;
    float val = yr[c];
    if (skip) val = fmaf(skip[c / vdim], to_f32(x[(size_t)t * x_stride + c]), val);
    const float g = to_f32(z[(size_t)t * z_stride + c]);
    val *= g / (1.0f + expf(-g));
    out[(size_t)t * out_stride + c] = from_f32<T>(val * inv * weight[c]);
  }
}

ARLE_API int arle_gated_group_norm(const float* y, const void* x, int dtype, int x_stride, const float* skip, int vdim, const void* z,
                                   int z_stride, const float* weight, float eps, void* out, int out_stride, int num_tokens, int inner,
                                   int parts, cudaStream_t s) {
  if (num_tokens <= 0) return 0;
  if (inner <= 0 || parts <= 0 || inner % parts || parts > 65535 || vdim <= 0) return ARLE_E_BADARG;
  const int width = inner / parts;
  const int threads = width >= 1024 ? 256 : (width >= 256 ? 128 : 64);
  if (dtype == 0)
    launch_kernel(gated_group_norm_kernel<float>, dim3(num_tokens, parts), dim3(threads), 0, s, 1, y, (const float*)x, x_stride, skip,
                  vdim, (const float*)z, z_stride, weight, eps, (float*)out, out_stride, inner, parts);
  else if (dtype == 1)
    launch_kernel(gated_group_norm_kernel<__nv_bfloat16>, dim3(num_tokens, parts), dim3(threads), 0, s, 1, y, (const __nv_bfloat16*)x,
                  x_stride, skip, vdim, (const __nv_bfloat16*)z, z_stride, weight, eps, (__nv_bfloat16*)out, out_stride, inner, parts);
  else
    return ARLE_E_BADARG;
  return launch_status();
}
