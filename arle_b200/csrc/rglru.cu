// The recurrent block with a real-gated linear recurrent unit, and the general short causal convolution.
//
//  * causal_conv: out[t, c] = act(out_bias[c] + sum_j w[c, j] * in[t - (taps - 1) + j, c]) over the tokens of t's row,
//    in = x + in_bias for tokens of the request and zero before its first; act is nothing or silu; the output may be
//    float32 whatever the input's type.  The request's last taps - 1 inputs (with in_bias already added) live in its
//    state slot at conv_off + c * (taps - 1) + j, oldest first, are read by the first tokens of the next portion and are
//    brought up to date by a second launch.
//  * rglru_scan: per channel c of a row's tokens, with z the gates' sums before their biases (a block-diagonal
//    product of u that the caller ran; [T, blocks, 2 * bs]: a block's recurrence gates, then its input gates),
//        r = sigmoid(z_r + b_r), i = sigmoid(z_i + b_i), log a = -c_decay * r * softplus(lam), a = exp(log a),
//        S_t = a S_(t-1) + sqrt(1 - a^2) * i * u_t,   out = S_t * act(y_t + y_bias)   (act: the tanh form of gelu)
//    all in float32; S lives in the request's state slot.  A thread holds one channel and `seg_len` consecutive tokens:
//    it runs them from a zero state, the segments' (product of a, end state) pairs are chained in order through shared
//    memory, and the tokens are run again from the true incoming state; 32 channels x up to 32 segments a block, or 16
//    channels x up to 64 segments for long rows of a narrow model.
#include "common.cuh"
using namespace arle;

template <typename TI, typename TO>
__global__ void causal_conv_kernel(const TI* __restrict__ x, int x_stride, const float* __restrict__ in_bias, const float* __restrict__ w,
                                   const float* __restrict__ out_bias, int act, const float* __restrict__ state, long slot_stride,
                                   long conv_off, const int* __restrict__ q_indptr, const int* __restrict__ row_of_token,
                                   const int* __restrict__ state_slots, TO* __restrict__ out, int out_stride, int C, int taps) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int r = row_of_token[t];
  const int beg = q_indptr[r];
  const int local = t - beg;
  const float* st = state + (size_t)state_slots[r] * slot_stride + conv_off + (size_t)c * (taps - 1);
  const float ib = in_bias ? in_bias[c] : 0.f;
  float acc = out_bias ? out_bias[c] : 0.f;
  for (int j = 0; j < taps; ++j) {
    const int src = local - (taps - 1) + j;
    const float xv = src >= 0 ? to_f32(x[(size_t)(beg + src) * x_stride + c]) + ib : st[src + taps - 1];
    acc = fmaf(w[(size_t)c * taps + j], xv, acc);
  }
  if (act == 1) acc = acc / (1.0f + expf(-acc));
  out[(size_t)t * out_stride + c] = from_f32<TO>(acc);
}

template <typename TI>
__global__ void causal_conv_state_kernel(const TI* __restrict__ x, int x_stride, const float* __restrict__ in_bias, float* __restrict__ state,
                                         long slot_stride, long conv_off, const int* __restrict__ q_indptr,
                                         const int* __restrict__ state_slots, int C, int taps) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int beg = q_indptr[r], n = q_indptr[r + 1] - beg;
  if (n <= 0) return;
  float* st = state + (size_t)state_slots[r] * slot_stride + conv_off + (size_t)c * (taps - 1);
  const float ib = in_bias ? in_bias[c] : 0.f;
  for (int j = 0; j < taps - 1; ++j) {                 // ascending: st[j] is written after st[j + n] was read
    const int src = n + j - (taps - 1);                // index among this step's tokens of the row
    st[j] = src >= 0 ? to_f32(x[(size_t)(beg + src) * x_stride + c]) + ib : st[src + taps - 1];
  }
}

template <typename TI, typename TO>
static int launch_conv(const void* x, int x_stride, const float* in_bias, const float* w, const float* out_bias, int act, float* state,
                       long slot_stride, long conv_off, const int* q_indptr, const int* row_of_token, const int* state_slots, void* out,
                       int out_stride, int num_tokens, int R, int C, int taps, cudaStream_t s) {
  const int threads = 128;
  const int cb = (C + threads - 1) / threads;
  if (cb > 65535) return ARLE_E_UNSUPPORTED;
  launch_kernel(causal_conv_kernel<TI, TO>, dim3(num_tokens, cb), dim3(threads), 0, s, 1, (const TI*)x, x_stride, in_bias, w, out_bias, act,
                (const float*)state, slot_stride, conv_off, q_indptr, row_of_token, state_slots, (TO*)out, out_stride, C, taps);
  if (taps > 1)
    launch_kernel(causal_conv_state_kernel<TI>, dim3(R, cb), dim3(threads), 0, s, 1, (const TI*)x, x_stride, in_bias, state, slot_stride,
                  conv_off, q_indptr, state_slots, C, taps);
  return launch_status();
}

// dtype: of x; out_dtype: of out (float32 from bfloat16 inputs is allowed, the reverse is not).  act: 0 none, 1 silu.
ARLE_API int arle_causal_conv(const void* x, int dtype, int x_stride, const float* in_bias, const float* w, const float* out_bias, int act,
                              float* state, long slot_stride, long conv_off, const int* q_indptr, const int* row_of_token,
                              const int* state_slots, void* out, int out_dtype, int out_stride, int num_tokens, int R, int C, int taps,
                              cudaStream_t s) {
  if (num_tokens <= 0) return 0;
  if (C <= 0 || taps <= 0 || R <= 0 || (act != 0 && act != 1)) return ARLE_E_BADARG;
#define ARLE_CONV(TI, TO) \
  return launch_conv<TI, TO>(x, x_stride, in_bias, w, out_bias, act, state, slot_stride, conv_off, q_indptr, row_of_token, state_slots, \
                             out, out_stride, num_tokens, R, C, taps, s)
  if (dtype == 0 && out_dtype == 0) ARLE_CONV(float, float);
  if (dtype == 1 && out_dtype == 1) ARLE_CONV(__nv_bfloat16, __nv_bfloat16);
  if (dtype == 1 && out_dtype == 0) ARLE_CONV(__nv_bfloat16, float);
#undef ARLE_CONV
  return ARLE_E_BADARG;
}

// ------------------------------------------------------------------------------------------------ the recurrence
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }
// 0.5 z (1 + tanh(w)) with w = sqrt(2 / pi) (z + 0.044715 z^3), written as z / (1 + exp(-2 w)): the same function, one
// exponential and one division.
__device__ __forceinline__ float gelu_tanh_f32(float z) {
  return z / (1.0f + expf(-1.5957691216057308f * (z + 0.044715f * z * z * z)));
}

constexpr int kLruThreads = 1024;      // CH channels x up to 1,024 / CH segments a block
constexpr int kLruMaxSeg = 8;          // tokens a thread holds at a time

// CH: 32 channels a block (a warp's lanes); 16 channels and up to 64 segments for rows of more than 256 tokens when the
// step's blocks are so few that twice as many still run at once (a single prompt of a narrow model).
template <typename T, int CH>
__global__ void __launch_bounds__(kLruThreads) rglru_scan_kernel(const float* __restrict__ z, const T* __restrict__ u, const T* __restrict__ y, int y_stride,
                                  const float* __restrict__ bias_r, const float* __restrict__ bias_i, const float* __restrict__ lam,
                                  const float* __restrict__ y_bias, float c_decay, float* __restrict__ state, long slot_stride,
                                  const int* __restrict__ q_indptr, const int* __restrict__ state_slots, T* __restrict__ out,
                                  int out_stride, int width, int bs) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float seg_a[kLruThreads / CH][CH + 1], seg_b[kLruThreads / CH][CH + 1];
  const int r = blockIdx.y;
  const int c = blockIdx.x * CH + threadIdx.x;
  const int seg = threadIdx.y, nseg = blockDim.y;
  const bool live = c < width;
  const int beg = q_indptr[r], end = q_indptr[r + 1];
  float* sp = state + (size_t)state_slots[r] * slot_stride + c;
  float S = live ? *sp : 0.f;
  const int blk = live ? c / bs : 0, cin = live ? c - blk * bs : 0;
  const size_t zr_at = (size_t)blk * 2 * bs + cin, zi_at = zr_at + bs;       // within a token's 2 * width sums
  const float br = live ? bias_r[c] : 0.f, bi = live ? bias_i[c] : 0.f, yb = live && y_bias ? y_bias[c] : 0.f;
  const float sp_lam = live ? softplus_f(lam[c]) : 0.f;
  const int span = nseg * kLruMaxSeg;
  for (int t0 = beg; t0 < end; t0 += span) {
    const int mine = t0 + seg * kLruMaxSeg;
    float a[kLruMaxSeg], b[kLruMaxSeg];
    float A = 1.f, B = 0.f;
#pragma unroll
    for (int j = 0; j < kLruMaxSeg; ++j) {
      const int t = mine + j;
      a[j] = 1.f;
      b[j] = 0.f;
      if (live && t < end) {
        const float* zt = z + (size_t)t * 2 * width;
        const float rg = 1.0f / (1.0f + expf(-(zt[zr_at] + br)));
        const float ig = 1.0f / (1.0f + expf(-(zt[zi_at] + bi)));
        const float log_a = -c_decay * rg * sp_lam;
        const float at = 1.0f + expm1f(log_a);      // rounded to nearest also next to 1, where a biased last bit would add up over a long row
        a[j] = at;
        b[j] = sqrtf(-expm1f(2.0f * log_a)) * ig * to_f32(u[(size_t)t * width + c]);      // sqrt(1 - a^2), exact near a = 1
      }
      A *= a[j];
      B = fmaf(a[j], B, b[j]);
    }
    if (nseg > 1) {
      seg_a[seg][threadIdx.x] = A;
      seg_b[seg][threadIdx.x] = B;
      __syncthreads();
      float Sin = S;
      for (int g = 0; g < seg; ++g) Sin = fmaf(seg_a[g][threadIdx.x], Sin, seg_b[g][threadIdx.x]);
      float Send = Sin;
      for (int g = seg; g < nseg; ++g) Send = fmaf(seg_a[g][threadIdx.x], Send, seg_b[g][threadIdx.x]);
      __syncthreads();
      S = Sin;
#pragma unroll
      for (int j = 0; j < kLruMaxSeg; ++j) {
        const int t = mine + j;
        if (live && t < end) {
          S = fmaf(a[j], S, b[j]);
          const float yv = gelu_tanh_f32(to_f32(y[(size_t)t * y_stride + c]) + yb);
          out[(size_t)t * out_stride + c] = from_f32<T>(S * yv);
        }
      }
      S = Send;                                       // every segment's thread carries the state after the whole span
    } else {
#pragma unroll
      for (int j = 0; j < kLruMaxSeg; ++j) {
        const int t = mine + j;
        if (live && t < end) {
          S = fmaf(a[j], S, b[j]);
          const float yv = gelu_tanh_f32(to_f32(y[(size_t)t * y_stride + c]) + yb);
          out[(size_t)t * out_stride + c] = from_f32<T>(S * yv);
        }
      }
    }
  }
  if (live && seg == 0 && end > beg) *sp = S;
}

// z float32 [T, 2 * width] contiguous ([blocks][recurrence gates bs | input gates bs] per token); u [T, width] contiguous and
// y, out [T, width] in the activation type (row strides given); biases, lam float32 [width]; state: float32, a slot every
// slot_stride numbers, the channels' states at its start.  max_q_len: the most tokens any row of the step has.
ARLE_API int arle_rglru_scan(const float* z, const void* u, const void* y, int dtype, int y_stride, const float* bias_r,
                             const float* bias_i, const float* lam, const float* y_bias, float c_decay, float* state, long slot_stride,
                             const int* q_indptr, const int* state_slots, void* out, int out_stride, int R, int width, int blocks,
                             int max_q_len, cudaStream_t s) {
  if (R <= 0) return 0;
  if (width <= 0 || blocks <= 0 || width % blocks || R > 65535) return ARLE_E_BADARG;
  // 16 channels a block only where the row is long and twice the blocks still run at once
  const int ch = max_q_len > 32 * kLruMaxSeg && (long)((width + 31) / 32) * R * 2 <= 148 ? 16 : 32;
  int nseg = 1;
  while (nseg < kLruThreads / ch && nseg * kLruMaxSeg < max_q_len) nseg <<= 1;
  dim3 grid((width + ch - 1) / ch, R), block(ch, nseg);
#define ARLE_LRU(TT, CH) \
  launch_kernel(rglru_scan_kernel<TT, CH>, dim3(grid), dim3(block), 0, s, 1, z, (const TT*)u, (const TT*)y, y_stride, bias_r, bias_i, lam, \
                y_bias, c_decay, state, slot_stride, q_indptr, state_slots, (TT*)out, out_stride, width, width / blocks)
  if (dtype == 0 && ch == 32)
    ARLE_LRU(float, 32);
  else if (dtype == 0)
    ARLE_LRU(float, 16);
  else if (dtype == 1 && ch == 32)
    ARLE_LRU(__nv_bfloat16, 32);
  else if (dtype == 1)
    ARLE_LRU(__nv_bfloat16, 16);
  else
    return ARLE_E_BADARG;
#undef ARLE_LRU
  return launch_status();
}
