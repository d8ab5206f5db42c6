// Rotation first, norm after it: the preparation of attention designs that bring q and k to unit root mean square
// (per head, with or without a weight) AFTER the rotary encoding, and whose values may have another width than
// their keys.
//
// Input is the packed projection qkv[t, :] = [q heads (hd each) | k heads (hd each) | v heads (vd each)] (row stride
// given).  One warp handles one (token, head):
//   q head: rotate the first rotary_dim numbers (number i with i + rotary_dim/2, angle position * inv_freq[i]),
//           x <- x / sqrt(mean(x^2) + eps) (* weight), store in place
//   k head: the same, stored into k_cache at the token's slot
//   v head: copied into v_cache at the token's slot
// With norm_first the norm (and its weight) comes BEFORE the rotation instead: x <- x / sqrt(mean(x^2) + eps) * weight, then
// the first rotary_dim numbers turn.
// Everything between load and store is float32; the angle is evaluated with sincosf in float32.
// Cache layout: keys [page][kv_head][slot_in_page][hd], values [page][kv_head][slot_in_page][vd]; slot_mapping[t] is
// page * page_size + slot_in_page, negative = do not store.  nkv = 0: the rows hold q only.
#include "common.cuh"
using namespace arle;

constexpr int kPostWarps = 4;
constexpr int kPostMaxHead = 256;

template <typename T>
__global__ void attention_prep_post_kernel(T* __restrict__ qkv, int row_stride, const int* __restrict__ positions,
                                           const int* __restrict__ slot_mapping, const float* __restrict__ q_weight,
                                           const float* __restrict__ k_weight, float eps, const float* __restrict__ inv_freq,
                                           int rotary_dim, T* __restrict__ k_cache, T* __restrict__ v_cache, int nq, int nkv, int hd,
                                           int vd, int page_size, int num_tokens, int norm_first) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float bufs[kPostWarps][kPostMaxHead];
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = nq + 2 * nkv;
  const long long unit = (long long)blockIdx.x * kPostWarps + w;
  if (unit >= (long long)num_tokens * heads) return;
  const int t = (int)(unit / heads), h = (int)(unit % heads);
  const int kind = h < nq ? 0 : (h < nq + nkv ? 1 : 2);
  const int kvh = kind == 1 ? h - nq : h - nq - nkv;
  T* src = qkv + (size_t)t * row_stride + (kind < 2 ? (size_t)h * hd : (size_t)(nq + nkv) * hd + (size_t)kvh * vd);

  size_t cache_base = 0;
  bool store = false;
  if (kind != 0) {
    const int slot = slot_mapping[t];
    if (slot >= 0) {
      const int page = slot / page_size, off = slot - page * page_size;
      cache_base = (((size_t)page * nkv + kvh) * page_size + off) * (kind == 1 ? hd : vd);
      store = true;
    }
  }
  if (kind == 2) {
    if (store)
      for (int e = lane; e < vd; e += 32) v_cache[cache_base + e] = src[e];
    return;
  }
  float* buf = bufs[w];
  for (int e = lane; e < hd; e += 32) buf[e] = to_f32(src[e]);
  __syncwarp();
  const float* wt = kind == 0 ? q_weight : k_weight;
  if (norm_first && eps >= 0.f) {
    float s0 = 0.f;
    for (int e = lane; e < hd; e += 32) s0 += buf[e] * buf[e];
    s0 = warp_sum(s0);
    const float inv0 = 1.0f / sqrtf(s0 / (float)hd + eps);
    for (int e = lane; e < hd; e += 32) buf[e] = buf[e] * inv0 * (wt ? wt[e] : 1.0f);
    __syncwarp();
  }
  const float pos = (float)positions[t];
  const int half = rotary_dim >> 1;
  float ss = 0.f;
  float o[kPostMaxHead / 32];
#pragma unroll
  for (int i = 0; i < kPostMaxHead / 32; ++i) {
    const int e = lane + 32 * i;
    float x = 0.f;
    if (e < hd) {
      if (e < rotary_dim) {
        const int f = e < half ? e : e - half;
        float sn, cs;
        sincosf(pos * inv_freq[f], &sn, &cs);
        x = e < half ? buf[e] * cs - buf[e + half] * sn : buf[e] * cs + buf[e - half] * sn;
      } else {
        x = buf[e];
      }
    }
    o[i] = x;
    ss += x * x;
  }
  ss = warp_sum(ss);
  const float inv = (eps >= 0.f && !norm_first) ? 1.0f / sqrtf(ss / (float)hd + eps) : 1.0f;
  if (norm_first) wt = nullptr;
#pragma unroll
  for (int i = 0; i < kPostMaxHead / 32; ++i) {
    const int e = lane + 32 * i;
    if (e < hd) {
      const float y = o[i] * inv * (wt ? wt[e] : 1.0f);
      if (kind == 0)
        src[e] = from_f32<T>(y);
      else if (store)
        k_cache[cache_base + e] = from_f32<T>(y);
    }
  }
}

// eps < 0: no norm (rotation and stores only).
ARLE_API int arle_attention_prep_post(void* qkv, int dtype, int row_stride, const int* positions, const int* slot_mapping,
                                      const float* q_weight, const float* k_weight, float eps, const float* inv_freq, int rotary_dim,
                                      void* k_cache, void* v_cache, int nq, int nkv, int hd, int vd, int page_size, int num_tokens,
                                      int norm_first, cudaStream_t s) {
  if (num_tokens <= 0) return 0;
  if (hd <= 0 || hd > kPostMaxHead || vd <= 0 || nq <= 0 || nkv < 0 || page_size <= 0) return ARLE_E_UNSUPPORTED;
  if (rotary_dim < 0 || rotary_dim % 2 || rotary_dim > hd || (rotary_dim && !inv_freq)) return ARLE_E_BADARG;
  if (nkv > 0 && (!slot_mapping || !k_cache || !v_cache)) return ARLE_E_BADARG;
  const long long units = (long long)num_tokens * (nq + 2 * nkv);
  const long long blocks = (units + kPostWarps - 1) / kPostWarps;
  if (blocks > 0x7fffffffLL) return ARLE_E_UNSUPPORTED;
  if (dtype == 0)
    launch_kernel(attention_prep_post_kernel<float>, dim3((unsigned)blocks), dim3(kPostWarps * 32), 0, s, 1, (float*)qkv, row_stride,
                  positions, slot_mapping, q_weight, k_weight, eps, inv_freq, rotary_dim, (float*)k_cache, (float*)v_cache, nq, nkv, hd,
                  vd, page_size, num_tokens, norm_first);
  else if (dtype == 1)
    launch_kernel(attention_prep_post_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(kPostWarps * 32), 0, s, 1, (__nv_bfloat16*)qkv,
                  row_stride, positions, slot_mapping, q_weight, k_weight, eps, inv_freq, rotary_dim, (__nv_bfloat16*)k_cache,
                  (__nv_bfloat16*)v_cache, nq, nkv, hd, vd, page_size, num_tokens, norm_first);
  else
    return ARLE_E_BADARG;
  return launch_status();
}
