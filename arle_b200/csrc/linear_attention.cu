// Gated linear attention: a recurrent mixer with a matrix state per head,
//
//     S_t = diag(alpha_t) S_(t-1) + k_t v_t^T          S: [dim, vdim], float32, one per (request, head)
//     o_t = S_t^T q_t
//
// with a decay alpha_t in (0, 1) per key channel.  Three kernels:
//
//  * gla_decay: alpha[t, c] = sigmoid(z)^(1/tau), z = b[c] + sum_r low[t, r] * w2[c, r], the second
//    half of a low-rank gate (low = W_a1 x comes from the packed input projection).  Evaluated as
//    exp(-softplus(-z) / tau) in float32; a block takes sixteen tokens and 256 channels, r ascending.
//  * gla_scan: the recurrence over this step's tokens of every request row, from the state that the
//    request's slot holds, which is left updated.  Float32 throughout; q, k, v are read in the
//    activation type.  One block of 128 threads per (columns of vdim, head, row); a thread keeps four
//    consecutive key channels of each of four columns of S in registers (up to 32 consecutive lanes share a
//    column; the state is stored [vdim][dim], so a column's lanes read one contiguous run), the step's
//    q, k, alpha and v are staged in shared memory a chunk of tokens at a time, and o_t[j] is the sum
//    over the column's lanes.  The order of every sum depends on (dim, vdim) only: a token's result
//    does not depend on how the prompt was cut or on what else is in the batch.
//  * gla_out: per head, o / sqrt(mean(o^2) + eps) * weight (shared by the heads), times silu(gate) (or sigmoid(gate)),
//    times a constant, rounded once into the activation type (a row of a wider buffer may be given).
#include "common.cuh"
using namespace arle;

constexpr int kScanThreads = 128;
constexpr int kScanCpt = 4;                      // columns of the state a thread keeps
constexpr int kDecayTokens = 16;                 // tokens a block of the decay kernel takes
constexpr int kDecayBatch = 16;                  // weights a thread asks for before it uses the first

// w2t is the second matrix of the gate transposed, [rank][channels]: consecutive threads read consecutive floats.
template <typename T>
__global__ void __launch_bounds__(256) gla_decay_kernel(const T* __restrict__ low, int low_stride, const float* __restrict__ w2t,
                                                        const float* __restrict__ bias, float inv_tau, float* __restrict__ alpha,
                                                        int num_tokens, int channels, int rank) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float lo_s[];                // [kDecayTokens][rank]
  const int t0 = blockIdx.x * kDecayTokens;
  const int n = min(kDecayTokens, num_tokens - t0);
  for (int i = threadIdx.x; i < kDecayTokens * rank; i += blockDim.x) {
    const int tt = i / rank, r = i - tt * rank;
    lo_s[i] = tt < n ? to_f32(low[(size_t)(t0 + tt) * low_stride + r]) : 0.f;
  }
  __syncthreads();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  float z[kDecayTokens];
#pragma unroll
  for (int tt = 0; tt < kDecayTokens; ++tt) z[tt] = 0.f;
  for (int r0 = 0; r0 < rank; r0 += kDecayBatch) {
    float w[kDecayBatch];
#pragma unroll
    for (int i = 0; i < kDecayBatch; ++i) w[i] = r0 + i < rank ? w2t[(size_t)(r0 + i) * channels + c] : 0.f;
#pragma unroll
    for (int i = 0; i < kDecayBatch; ++i) {
      if (r0 + i >= rank) break;
#pragma unroll
      for (int tt = 0; tt < kDecayTokens; ++tt) z[tt] = fmaf(lo_s[tt * rank + r0 + i], w[i], z[tt]);
    }
  }
  const float b = bias ? bias[c] : 0.f;
#pragma unroll
  for (int tt = 0; tt < kDecayTokens; ++tt) {
    if (tt >= n) break;
    const float y = -(z[tt] + b);                // softplus(y) = log(1 + e^y), the stable way
    const float sp = y > 0.f ? y + log1pf(expf(-y)) : log1pf(expf(y));
    alpha[(size_t)(t0 + tt) * channels + c] = expf(-sp * inv_tau);
  }
}

// Four elements as they lie in memory (converted only when they are staged: a conversion right after its load would
// make every load wait for the one before it).
__device__ __forceinline__ float4 load_raw4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ uint2 load_raw4(const __nv_bfloat16* p) { return *reinterpret_cast<const uint2*>(p); }
__device__ __forceinline__ float4 widen4(float4 u) { return u; }
__device__ __forceinline__ float4 widen4(uint2 u) {
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x), b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
  return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
template <typename T, bool VEC> struct Raw4 { using type = float4; };
template <> struct Raw4<__nv_bfloat16, true> { using type = uint2; };

// DPT: consecutive key channels that a thread keeps of each of its kScanCpt columns of the state (4 up to 128
// channels, then 8, 16).  LPC: lanes that share a column (a power of two; LPC * DPT >= dim).  VEC: four channels
// at a time can be fetched with one aligned load.  A chunk of CHUNK tokens is staged in shared memory; while it is
// worked on, the next chunk's q, k, alpha and v are already on their way into registers.  Every number of q, k and
// alpha that a thread reads from shared memory serves four columns: with one column a thread the kernel was bound by
// shared-memory bandwidth.
template <typename T, int DPT, int LPC, bool VEC>
__global__ void __launch_bounds__(kScanThreads) gla_scan_kernel(
    const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, int in_stride,
    const float* __restrict__ alpha, float* __restrict__ state, const int* __restrict__ q_indptr,
    const int* __restrict__ state_slots, float* __restrict__ out, int heads, int dim, int vdim, float q_scale) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int CPT = kScanCpt;
  constexpr int COLS = kScanThreads / LPC * CPT; // columns a block takes
  constexpr int DSPAN = DPT * LPC;               // dim rounded up; channels past dim hold zeros
  constexpr int PAD = DPT == 4 ? 4 : DPT + 4;    // floats a thread's channels take in shared memory: 16-byte rows, spread over the banks
  constexpr int DPAD = PAD * LPC;
  constexpr int CHUNK = DSPAN >= 512 ? 4 : (DSPAN >= 256 ? 8 : 16);
  constexpr int QUADS = CHUNK * DSPAN / 4;       // groups of four channels in a chunk
  constexpr int QPT = (QUADS + kScanThreads - 1) / kScanThreads;
  constexpr int VPT = (CHUNK * COLS + kScanThreads - 1) / kScanThreads;
  __shared__ __align__(16) float qs[CHUNK * DPAD], ks[CHUNK * DPAD], as[CHUNK * DPAD];
  __shared__ __align__(16) float vs[CHUNK * COLS];
  const int r = blockIdx.z, h = blockIdx.y, j0 = blockIdx.x * COLS;
  const int l = threadIdx.x & (LPC - 1), jl = threadIdx.x / LPC;
  const int jb = j0 + jl * CPT;                  // this thread's first column
  const int t_begin = q_indptr[r], t_end = q_indptr[r + 1];
  // the state of a head is kept as [vdim][dim]: a thread's channels of a column are contiguous
  float* S_g = state + (((size_t)state_slots[r] * heads + h) * vdim) * dim + l * DPT;
  const bool vec_state = (dim & 3) == 0;
  float S[CPT][DPT];
#pragma unroll
  for (int cc = 0; cc < CPT; ++cc) {
    const bool col_ok = jb + cc < vdim;
    const float* sp = S_g + (size_t)(col_ok ? jb + cc : 0) * dim;
#pragma unroll
    for (int i = 0; i < DPT; i += 4) {
      const int c = l * DPT + i;
      if (vec_state) {
        float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
        if (col_ok && c < dim) u = *reinterpret_cast<const float4*>(sp + i);
        S[cc][i] = u.x, S[cc][i + 1] = u.y, S[cc][i + 2] = u.z, S[cc][i + 3] = u.w;
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) S[cc][i + e] = (col_ok && c + e < dim) ? sp[i + e] : 0.f;
      }
    }
  }
  const size_t hq = (size_t)h * dim, hv = (size_t)h * vdim;
  const size_t a_stride = (size_t)heads * dim;
  using RawT = typename Raw4<T, VEC>::type;
  RawT rq[QPT], rk[QPT];
  float4 ra[QPT];
  T rv[VPT];

  // The chunk's numbers into registers; nothing waits on them yet.  Loads are unconditional (a place outside the
  // chunk reads the row's first token instead and is zeroed when staged), so that they are all under way at once.
  auto fetch = [&](int t0, int n) {
#pragma unroll
    for (int u = 0; u < QPT; ++u) {
      const int idx = threadIdx.x + u * kScanThreads;
      const int tt = idx / (DSPAN / 4), c = (idx - tt * (DSPAN / 4)) * 4;
      const bool ok = idx < QUADS && tt < n && c < dim;
      const size_t row = ok ? (size_t)(t0 + tt) : (size_t)t_begin;
      const int cs = ok ? c : 0;
      if constexpr (VEC) {
        rq[u] = load_raw4(q + row * in_stride + hq + cs);
        rk[u] = load_raw4(k + row * in_stride + hq + cs);
        ra[u] = *reinterpret_cast<const float4*>(alpha + row * a_stride + hq + cs);
      } else {
        float4 fq = make_float4(0.f, 0.f, 0.f, 0.f), fk = fq, fa = fq;
        float* pq = &fq.x; float* pk = &fk.x; float* pa = &fa.x;
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (cs + e < dim) {
            pq[e] = to_f32(q[row * in_stride + hq + cs + e]);
            pk[e] = to_f32(k[row * in_stride + hq + cs + e]);
            pa[e] = alpha[row * a_stride + hq + cs + e];
          }
        *reinterpret_cast<float4*>(&rq[u]) = fq;
        *reinterpret_cast<float4*>(&rk[u]) = fk;
        ra[u] = fa;
      }
    }
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
      const int idx = threadIdx.x + u * kScanThreads;
      const int tt = idx / COLS, c = idx - tt * COLS;
      const bool ok = idx < CHUNK * COLS && tt < n && j0 + c < vdim;
      rv[u] = v[(ok ? (size_t)(t0 + tt) : (size_t)t_begin) * in_stride + hv + (ok ? j0 + c : 0)];
    }
  };
  auto stage = [&](int n) {                      // registers to shared memory, widened, q scaled on the way
#pragma unroll
    for (int u = 0; u < QPT; ++u) {
      const int idx = threadIdx.x + u * kScanThreads;
      const int tt = idx / (DSPAN / 4), c = (idx - tt * (DSPAN / 4)) * 4;
      const int at = tt * DPAD + (c / DPT) * PAD + (c % DPT);
      if (idx >= QUADS) continue;
      const bool ok = tt < n && c < dim;
      const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
      const float4 fq = widen4(rq[u]), fk = widen4(rk[u]);
      *reinterpret_cast<float4*>(qs + at) = ok ? make_float4(fq.x * q_scale, fq.y * q_scale, fq.z * q_scale, fq.w * q_scale) : z;
      *reinterpret_cast<float4*>(ks + at) = ok ? fk : z;
      *reinterpret_cast<float4*>(as + at) = ok ? ra[u] : z;
    }
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
      const int idx = threadIdx.x + u * kScanThreads;
      const int tt = idx / COLS, c = idx - tt * COLS;
      if (idx < CHUNK * COLS) vs[idx] = (tt < n && j0 + c < vdim) ? to_f32(rv[u]) : 0.f;
    }
  };

  if (t_begin < t_end) fetch(t_begin, min(CHUNK, t_end - t_begin));
  for (int t0 = t_begin; t0 < t_end; t0 += CHUNK) {
    const int n = min(CHUNK, t_end - t0);
    __syncthreads();                             // the chunk before has been read by everyone
    stage(n);
    __syncthreads();
    if (t0 + CHUNK < t_end) fetch(t0 + CHUNK, min(CHUNK, t_end - t0 - CHUNK));
#pragma unroll 4
    for (int tt = 0; tt < n; ++tt) {
      const float4 v4 = *reinterpret_cast<const float4*>(vs + tt * COLS + jl * CPT);
      const float vj[CPT] = {v4.x, v4.y, v4.z, v4.w};
      const float4* qt = reinterpret_cast<const float4*>(qs + tt * DPAD + l * PAD);
      const float4* kt = reinterpret_cast<const float4*>(ks + tt * DPAD + l * PAD);
      const float4* at = reinterpret_cast<const float4*>(as + tt * DPAD + l * PAD);
      float o[CPT];
#pragma unroll
      for (int cc = 0; cc < CPT; ++cc) o[cc] = 0.f;
#pragma unroll
      for (int i = 0; i < DPT / 4; ++i) {
        const float4 a4 = at[i], k4 = kt[i], q4 = qt[i];
#pragma unroll
        for (int cc = 0; cc < CPT; ++cc) {
          S[cc][4 * i] = fmaf(a4.x, S[cc][4 * i], k4.x * vj[cc]);
          S[cc][4 * i + 1] = fmaf(a4.y, S[cc][4 * i + 1], k4.y * vj[cc]);
          S[cc][4 * i + 2] = fmaf(a4.z, S[cc][4 * i + 2], k4.z * vj[cc]);
          S[cc][4 * i + 3] = fmaf(a4.w, S[cc][4 * i + 3], k4.w * vj[cc]);
          const float lo = fmaf(S[cc][4 * i], q4.x, S[cc][4 * i + 1] * q4.y);
          const float hi = fmaf(S[cc][4 * i + 2], q4.z, S[cc][4 * i + 3] * q4.w);
          o[cc] += lo + hi;
        }
      }
      // the four columns' sums over the LPC lanes: two exchanges halve what a lane holds, then a butterfly
      int mine = 0;                              // the column whose sum this lane ends up with
      float b;
      if (LPC >= 4) {
        const bool up = (l & (LPC / 2)) != 0, up2 = (l & (LPC / 4)) != 0;
        const float r0 = __shfl_xor_sync(0xffffffffu, up ? o[0] : o[2], LPC / 2);
        const float r1 = __shfl_xor_sync(0xffffffffu, up ? o[1] : o[3], LPC / 2);
        const float a0 = (up ? o[2] : o[0]) + r0, a1 = (up ? o[3] : o[1]) + r1;
        const float r2 = __shfl_xor_sync(0xffffffffu, up2 ? a0 : a1, LPC / 4);
        b = (up2 ? a1 : a0) + r2;
        mine = (up ? 2 : 0) + (up2 ? 1 : 0);
#pragma unroll
        for (int w = LPC / 8; w > 0; w >>= 1) b += __shfl_xor_sync(0xffffffffu, b, w);
        if ((l & (LPC / 4 - 1)) == 0 && jb + mine < vdim) out[(size_t)(t0 + tt) * heads * vdim + hv + jb + mine] = b;
      } else {
#pragma unroll
        for (int cc = 0; cc < CPT; ++cc) {
          float x = o[cc];
#pragma unroll
          for (int w = LPC >> 1; w > 0; w >>= 1) x += __shfl_xor_sync(0xffffffffu, x, w);
          if (l == 0 && jb + cc < vdim) out[(size_t)(t0 + tt) * heads * vdim + hv + jb + cc] = x;
        }
      }
    }
  }
#pragma unroll
  for (int cc = 0; cc < CPT; ++cc) {
    const bool col_ok = jb + cc < vdim;
    float* sp = S_g + (size_t)(col_ok ? jb + cc : 0) * dim;
#pragma unroll
    for (int i = 0; i < DPT; i += 4) {
      const int c = l * DPT + i;
      if (vec_state) {
        if (col_ok && c < dim) *reinterpret_cast<float4*>(sp + i) = make_float4(S[cc][i], S[cc][i + 1], S[cc][i + 2], S[cc][i + 3]);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (col_ok && c + e < dim) sp[i + e] = S[cc][i + e];
      }
    }
  }
}

__device__ __forceinline__ void store4(float* p, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, float a, float b, float c, float d) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
}

template <typename T, bool VEC4>
__global__ void gla_out_kernel(const float* __restrict__ o, const T* __restrict__ gate, int gate_stride,
                               const float* __restrict__ weight, float eps, float scale, T* __restrict__ out,
                               int out_stride, int heads, int vdim, long long units, int sigmoid_gate) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= units) return;
  const long long t = unit / heads;
  const int h = (int)(unit - t * heads);
  const float* src = o + ((size_t)t * heads + h) * vdim;
  float ss = 0.f;
  if constexpr (VEC4) {                          // vdim a multiple of 4, rows on 16-byte (8-byte for bfloat16) boundaries
    const T* gp = gate ? gate + (size_t)t * gate_stride + (size_t)h * vdim : nullptr;
    T* op = out + (size_t)t * out_stride + (size_t)h * vdim;
    for (int e = lane * 4; e < vdim; e += 128) {
      const float4 x = *reinterpret_cast<const float4*>(src + e);
      ss += (x.x * x.x + x.y * x.y) + (x.z * x.z + x.w * x.w);
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)vdim + eps);
    for (int e = lane * 4; e < vdim; e += 128) {
      const float4 x = *reinterpret_cast<const float4*>(src + e);
      float y[4] = {x.x * inv, x.y * inv, x.z * inv, x.w * inv};
      if (weight) {
        const float4 w = *reinterpret_cast<const float4*>(weight + e);
        y[0] *= w.x, y[1] *= w.y, y[2] *= w.z, y[3] *= w.w;
      }
      if (gp) {
        const float4 g = widen4(load_raw4(gp + e));
        if (sigmoid_gate) {
          y[0] *= 1.0f / (1.0f + expf(-g.x)), y[1] *= 1.0f / (1.0f + expf(-g.y));
          y[2] *= 1.0f / (1.0f + expf(-g.z)), y[3] *= 1.0f / (1.0f + expf(-g.w));
        } else {
          y[0] *= g.x / (1.0f + expf(-g.x)), y[1] *= g.y / (1.0f + expf(-g.y));
          y[2] *= g.z / (1.0f + expf(-g.z)), y[3] *= g.w / (1.0f + expf(-g.w));
        }
      }
      store4(op + e, y[0] * scale, y[1] * scale, y[2] * scale, y[3] * scale);
    }
  } else {
    for (int e = lane; e < vdim; e += 32) ss += src[e] * src[e];
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)vdim + eps);
    for (int e = lane; e < vdim; e += 32) {
      float y = src[e] * inv;
      if (weight) y *= weight[e];
      if (gate) {
        const float g = to_f32(gate[(size_t)t * gate_stride + (size_t)h * vdim + e]);
        y *= (sigmoid_gate ? 1.0f : g) / (1.0f + expf(-g));
      }
      out[(size_t)t * out_stride + (size_t)h * vdim + e] = from_f32<T>(y * scale);
    }
  }
}

ARLE_API int arle_gla_decay(const void* low, int dtype, int low_stride, const float* w2t, const float* bias, float tau,
                            float* alpha, int num_tokens, int channels, int rank, cudaStream_t s) {
  if (num_tokens <= 0) return 0;
  if (channels <= 0 || rank <= 0 || !(tau > 0.f) || rank > 1024) return ARLE_E_BADARG;
  const int threads = 256;
  dim3 grid((num_tokens + kDecayTokens - 1) / kDecayTokens, (channels + threads - 1) / threads);
  if (grid.y > 65535) return ARLE_E_UNSUPPORTED;
  const size_t smem = (size_t)kDecayTokens * rank * sizeof(float);
  if (dtype == 0)
    launch_kernel(gla_decay_kernel<float>, grid, dim3(threads), smem, s, 1, (const float*)low, low_stride, w2t, bias, 1.0f / tau, alpha,
                  num_tokens, channels, rank);
  else if (dtype == 1)
    launch_kernel(gla_decay_kernel<__nv_bfloat16>, grid, dim3(threads), smem, s, 1, (const __nv_bfloat16*)low, low_stride, w2t, bias,
                  1.0f / tau, alpha, num_tokens, channels, rank);
  else
    return ARLE_E_BADARG;
  return launch_status();
}

namespace {

template <typename T, int DPT, int LPC>
int scan_launch(const void* q, const void* k, const void* v, int in_stride, const float* alpha, float* state, const int* q_indptr,
                const int* state_slots, float* out, int rows, int heads, int dim, int vdim, float q_scale, cudaStream_t s) {
  constexpr int COLS = kScanThreads / LPC * kScanCpt;
  dim3 grid((vdim + COLS - 1) / COLS, heads, rows);
  const size_t eb = sizeof(T) * 4;               // bytes of four elements of q or k
  const bool vec = dim % 4 == 0 && in_stride % 4 == 0 && ((uintptr_t)q % eb) == 0 && ((uintptr_t)k % eb) == 0 &&
                   ((uintptr_t)alpha % 16) == 0;
  if (vec)
    launch_kernel(gla_scan_kernel<T, DPT, LPC, true>, grid, dim3(kScanThreads), 0, s, 1, (const T*)q, (const T*)k, (const T*)v,
                  in_stride, alpha, state, q_indptr, state_slots, out, heads, dim, vdim, q_scale);
  else
    launch_kernel(gla_scan_kernel<T, DPT, LPC, false>, grid, dim3(kScanThreads), 0, s, 1, (const T*)q, (const T*)k, (const T*)v,
                  in_stride, alpha, state, q_indptr, state_slots, out, heads, dim, vdim, q_scale);
  return launch_status();
}

// The split of the key channels among threads depends on dim alone, so the order of a token's sums does too: four
// channels a thread up to 128 channels (as many lanes as that takes, a power of two), then 8 and 16 on 32 lanes.
template <typename T>
int scan_dispatch(const void* q, const void* k, const void* v, int in_stride, const float* alpha, float* state,
                  const int* q_indptr, const int* state_slots, float* out, int rows, int heads, int dim, int vdim, float q_scale,
                  cudaStream_t s) {
#define ARLE_SCAN(D, L) \
  return scan_launch<T, D, L>(q, k, v, in_stride, alpha, state, q_indptr, state_slots, out, rows, heads, dim, vdim, q_scale, s)
  if (dim <= 4) ARLE_SCAN(4, 1);
  if (dim <= 8) ARLE_SCAN(4, 2);
  if (dim <= 16) ARLE_SCAN(4, 4);
  if (dim <= 32) ARLE_SCAN(4, 8);
  if (dim <= 64) ARLE_SCAN(4, 16);
  if (dim <= 128) ARLE_SCAN(4, 32);
  if (dim <= 256) ARLE_SCAN(8, 32);
  if (dim <= 512) ARLE_SCAN(16, 32);
#undef ARLE_SCAN
  return ARLE_E_UNSUPPORTED;
}

}  // namespace

ARLE_API int arle_gla_scan(const void* q, const void* k, const void* v, int dtype, int in_stride, const float* alpha,
                           float* state, const int* q_indptr, const int* state_slots, float* out, int rows, int heads,
                           int dim, int vdim, float q_scale, int max_q_len, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (heads <= 0 || dim <= 0 || vdim <= 0 || max_q_len <= 0) return ARLE_E_BADARG;
  if (dim > 512 || heads > 65535 || rows > 65535) return ARLE_E_UNSUPPORTED;
  if (dtype == 0)
    return scan_dispatch<float>(q, k, v, in_stride, alpha, state, q_indptr, state_slots, out, rows, heads, dim, vdim, q_scale, s);
  if (dtype == 1)
    return scan_dispatch<__nv_bfloat16>(q, k, v, in_stride, alpha, state, q_indptr, state_slots, out, rows, heads, dim, vdim, q_scale, s);
  return ARLE_E_BADARG;
}

ARLE_API int arle_gla_out(const float* o, const void* gate, int dtype, int gate_stride, const float* weight, float eps,
                          float scale, void* out, int out_stride, int num_tokens, int heads, int vdim, int sigmoid_gate, cudaStream_t s) {
  if (num_tokens <= 0) return 0;
  if (heads <= 0 || vdim <= 0) return ARLE_E_BADARG;
  const long long units = (long long)num_tokens * heads;
  const int warps = 8;
  const long long blocks = (units + warps - 1) / warps;
  if (blocks > 0x7fffffffLL) return ARLE_E_UNSUPPORTED;
  const size_t eb = dtype == 0 ? 16 : 8;         // bytes of four elements of gate and out
  const bool vec = vdim % 4 == 0 && gate_stride % 4 == 0 && out_stride % 4 == 0 && ((uintptr_t)o % 16) == 0 &&
                   ((uintptr_t)gate % eb) == 0 && ((uintptr_t)out % eb) == 0 && ((uintptr_t)weight % 16) == 0;
  if (dtype == 0) {
    auto kern = vec ? gla_out_kernel<float, true> : gla_out_kernel<float, false>;
    launch_kernel(kern, dim3((unsigned)blocks), dim3(warps * 32), 0, s, 1, o, (const float*)gate, gate_stride, weight, eps, scale,
                  (float*)out, out_stride, heads, vdim, units, sigmoid_gate);
  } else if (dtype == 1) {
    auto kern = vec ? gla_out_kernel<__nv_bfloat16, true> : gla_out_kernel<__nv_bfloat16, false>;
    launch_kernel(kern, dim3((unsigned)blocks), dim3(warps * 32), 0, s, 1, o, (const __nv_bfloat16*)gate, gate_stride, weight, eps,
                  scale, (__nv_bfloat16*)out, out_stride, heads, vdim, units, sigmoid_gate);
  } else {
    return ARLE_E_BADARG;
  }
  return launch_status();
}
