// A feed-forward of routed experts.
//
//  * moe_select: from a token's float32 router sums z: scores s = sigmoid(z); choice scores s + correction; the experts
//    stand in `groups` equal groups of neighbours, a group's score is the sum of its two largest choice scores (its one
//    score when a group is a single expert), only experts of the `keep` best groups can be chosen (the others count as
//    minus infinity); the `top` largest choice scores are chosen and weighted with s * scale (no renormalisation).
//    Ties go to the lower index.  One thread per token, everything float32.  `mode` bit 0: the scores are a softmax
//    over all experts instead of sigmoids; bit 1: a group's score is its largest choice score alone; bit 2: the sums z
//    themselves are the choice scores and the weights are the softmax over the chosen sums alone (times scale).
//  * moe_plan: sorts the step's (token, choice) pairs by expert (counts, offsets, a place for every pair) and lists
//    the tiles of 64 places that the grouped product runs, one block of 1,024 threads; nothing goes through the host,
//    so the step can be captured in a graph.  The order of the pairs inside an expert's run is whatever the
//    atomics gave; no result depends on it, since every place is computed alone.
//  * moe_gemm: C[place, :] = A[row(place), :] . W[expert(place)]^T in tiles of 64 x 64, float32 sums with k ascending
//    (the per-expert twin of the plain product).  `rows` maps a place to its row of A (the token of the pair) or is
//    absent (A is already in place order).
//    In bfloat16 with aligned rows the same product runs on the tensor cores (moe_gemm_mma: tiles of 64 places x 128
//    columns, mma.sync with float32 sums, operands brought in by cp.async in three stages), and a step of few pairs
//    (decoding) runs it as one dot product a warp (moe_gemv: every chosen expert's rows are streamed once, 16 bytes
//    a lane and load), since a tile of 64 places would be all but empty.
//  * moe_combine: out[t] = sum_k weight[t, k] * Y[place(t, k)] (k ascending) + sigmoid(gate[t]) * shared[t].
#include "common.cuh"
#include "mma_utils.cuh"
using namespace arle;

__global__ void moe_select_kernel(const float* __restrict__ z, int z_stride, const float* __restrict__ correction,
                                  float* __restrict__ scratch, int E, int top, int groups, int keep, float scale,
                                  int mode, int* __restrict__ ids, float* __restrict__ wts, int num_tokens) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= num_tokens) return;
  const float* zr = z + (size_t)t * z_stride;
  float* ch = scratch + (size_t)t * (E + groups);       // choice scores, then the groups' scores
  float* gs = ch + E;
  float zmax = -INFINITY, zsum = 1.f;
  if (mode & 1) {
    for (int e = 0; e < E; ++e) zmax = fmaxf(zmax, zr[e]);
    zsum = 0.f;
    for (int e = 0; e < E; ++e) zsum += expf(zr[e] - zmax);
  }
  for (int e = 0; e < E; ++e)
    ch[e] = ((mode & 4) ? zr[e] : (mode & 1) ? expf(zr[e] - zmax) / zsum : 1.0f / (1.0f + expf(-zr[e]))) + (correction ? correction[e] : 0.f);
  const int per = E / groups;
  for (int g = 0; g < groups; ++g) {
    float b1 = -INFINITY, b2 = -INFINITY;
    for (int i = 0; i < per; ++i) {
      const float v = ch[g * per + i];
      if (v > b1) {
        b2 = b1;
        b1 = v;
      } else if (v > b2) {
        b2 = v;
      }
    }
    gs[g] = (per > 1 && !(mode & 2)) ? b1 + b2 : b1;
  }
  if (keep < groups) {
    // the groups that are not kept: all but the `keep` best
    for (int it = 0; it < keep; ++it) {
      int bi = -1;
      float bv = -INFINITY;
      for (int g = 0; g < groups; ++g) {
        const float v = gs[g];
        if (v != INFINITY && (bi < 0 || v > bv)) {
          bv = v;
          bi = g;
        }
      }
      gs[bi] = INFINITY;                                // marks a kept group
    }
    for (int g = 0; g < groups; ++g)
      if (gs[g] != INFINITY)
        for (int i = 0; i < per; ++i) ch[g * per + i] = -INFINITY;
  }
  for (int it = 0; it < top; ++it) {
    int bi = -1;
    float bv = -INFINITY;
    for (int e = 0; e < E; ++e) {
      const float v = ch[e];
      if (v != INFINITY && (bi < 0 || v > bv)) {
        bv = v;
        bi = e;
      }
    }
    ch[bi] = INFINITY;                                  // taken
    ids[(size_t)t * top + it] = bi;
    wts[(size_t)t * top + it] = (mode & 4) ? zr[bi] : (mode & 1) ? scale * (expf(zr[bi] - zmax) / zsum) : scale / (1.0f + expf(-zr[bi]));
  }
  if (mode & 4) {                                       // softmax over the chosen sums, in choice order
    float* wr = wts + (size_t)t * top;
    float cm = -INFINITY, cs = 0.f;
    for (int it = 0; it < top; ++it) cm = fmaxf(cm, wr[it]);
    for (int it = 0; it < top; ++it) cs += expf(wr[it] - cm);
    for (int it = 0; it < top; ++it) wr[it] = scale * (expf(wr[it] - cm) / cs);
  }
}

ARLE_API int arle_moe_select(const float* z, int z_stride, const float* correction, float* scratch, int E, int top, int groups,
                             int keep, float scale, int mode, int* ids, float* wts, int num_tokens, cudaStream_t s) {
  if (num_tokens <= 0) return 0;
  if (E <= 0 || top <= 0 || groups <= 0 || E % groups || keep <= 0 || keep > groups || top > keep * (E / groups)) return ARLE_E_BADARG;
  launch_kernel(moe_select_kernel, dim3((num_tokens + 63) / 64), dim3(64), 0, s, 1, z, z_stride, correction, scratch, E, top, groups,
                keep, scale, mode, ids, wts, num_tokens);
  return launch_status();
}

constexpr int kMoeTile = 64;
constexpr int kMoeMaxExperts = 1024;

// plan (int32): [0, E] offsets of the experts' runs; [E + 1] tiles in use; then per tile (expert, first place, places).
__global__ void __launch_bounds__(1024) moe_plan_kernel(const int* __restrict__ ids, int pairs, int top, int E, int* __restrict__ plan,
                                                        int* __restrict__ place_of_pair, int* __restrict__ row_of_place, int max_tiles) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ int count[kMoeMaxExperts], offset[kMoeMaxExperts + 1], cursor[kMoeMaxExperts];
  for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = cursor[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) atomicAdd(&count[ids[p]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0, tiles = 0;
    int* tt = plan + E + 2;
    for (int e = 0; e < E; ++e) {
      offset[e] = at;
      plan[e] = at;
      for (int r0 = 0; r0 < count[e] && tiles < max_tiles; r0 += kMoeTile, ++tiles) {
        tt[3 * tiles] = e;
        tt[3 * tiles + 1] = at + r0;
        tt[3 * tiles + 2] = min(kMoeTile, count[e] - r0);
      }
      at += count[e];
    }
    offset[E] = at;
    plan[E] = at;
    plan[E + 1] = tiles;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = ids[p];
    const int place = offset[e] + atomicAdd(&cursor[e], 1);
    place_of_pair[p] = place;
    row_of_place[place] = p / top;
  }
}

ARLE_API int arle_moe_plan_ints(int E, int pairs) { return E + 2 + 3 * (pairs / kMoeTile + E + 1); }

ARLE_API int arle_moe_plan(const int* ids, int pairs, int top, int E, int* plan, int* place_of_pair, int* row_of_place,
                           cudaStream_t s) {
  if (pairs <= 0) return 0;
  if (E <= 0 || E > kMoeMaxExperts || top <= 0) return ARLE_E_UNSUPPORTED;
  launch_kernel(moe_plan_kernel, dim3(1), dim3(1024), 0, s, 1, ids, pairs, top, E, plan, place_of_pair, row_of_place,
                pairs / kMoeTile + E + 1);
  return launch_status();
}

constexpr int GM = 64, GN = 64, GK = 16;

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256) moe_gemm_kernel(const TA* __restrict__ A, int lda, const int* __restrict__ rows,
                                                       const TW* __restrict__ W, int ldw, long w_expert, TC* __restrict__ C, int ldc,
                                                       const int* __restrict__ plan, int E, int N, int K) {
  pdl_launch_dependents();
  pdl_wait();
  const int tile = blockIdx.y;
  if (tile >= plan[E + 1]) return;
  const int* tt = plan + E + 2 + 3 * tile;
  const int expert = tt[0], p0 = tt[1], M = tt[2];
  __shared__ float As[GK][GM + 4];
  __shared__ float Ws[GK][GN + 4];
  __shared__ int arow[GM];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int n0 = blockIdx.x * GN;
  if (tid < GM) arow[tid] = tid < M ? (rows ? rows[p0 + tid] : p0 + tid) : -1;
  __syncthreads();
  W += (size_t)expert * w_expert;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += GK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = tid + i * 256;
      const int r = idx >> 4, c = idx & 15;
      const int gn = n0 + r, gk = k0 + c;
      const int ar = arow[r];
      As[c][r] = (ar >= 0 && gk < K) ? to_f32(A[(size_t)ar * lda + gk]) : 0.f;
      Ws[c][r] = (gn < N && gk < K) ? to_f32(W[(size_t)gn * ldw + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn < N) C[(size_t)(p0 + m) * ldc + gn] = from_f32<TC>(acc[i][j]);
    }
  }
}

constexpr int TM = 64, TN = 128, TK = 32, TPITCH = 40, kStages = 3;

// A tile of 64 rows x 128 columns of C = A . W^T on the tensor cores: row r of the tile is row arow[r] of A (-1: none) and
// row crow0 + r of C; M rows are live.  Three stages of cp.async, one barrier a stage, eight warps of 32 x 32, mma.sync with float32 sums.
template <typename TC>
__device__ __forceinline__ void mma_tile_64x128(const __nv_bfloat16* __restrict__ A, int lda, const int* arow, const __nv_bfloat16* __restrict__ W,
                                                int ldw, TC* __restrict__ C, int ldc, size_t crow0, int M, int n0, int N, int K,
                                                __nv_bfloat16 (*As)[TM * TPITCH], __nv_bfloat16 (*Ws)[TN * TPITCH]) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = warp & 1, wn = warp >> 1;
  auto load = [&](int stage, int k0) {
    {
      const int r = tid >> 2, c = (tid & 3) * 8;
      const int ar = arow[r];
      const bool ok = ar >= 0 && k0 + c < K;
      cp_async16(smem_u32(&As[stage][r * TPITCH + c]), ok ? A + (size_t)ar * lda + k0 + c : A, ok ? 16 : 0);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int id = tid + i * 256;
      const int r = id >> 2, c = (id & 3) * 8;
      const bool ok = n0 + r < N && k0 + c < K;
      cp_async16(smem_u32(&Ws[stage][r * TPITCH + c]), ok ? W + (size_t)(n0 + r) * ldw + k0 + c : W, ok ? 16 : 0);
    }
  };
  float acc[2][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;
  const int nk = (K + TK - 1) / TK;
  load(0, 0);
  cp_commit();
  if (nk > 1) load(1, TK);
  cp_commit();
  for (int kt = 0; kt < nk; ++kt) {
    const int st = kt % kStages;
    cp_wait<1>();                             // stage kt has landed (one younger group may still be under way)
    __syncthreads();                          // and every warp has finished with the stage that is filled next
    if (kt + 2 < nk) load((kt + 2) % kStages, (kt + 2) * TK);
    cp_commit();
#pragma unroll
    for (int kk = 0; kk < TK / 16; ++kk) {
      uint32_t a[2][4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
        ldsm_x4(smem_u32(&As[st][(wm * 32 + mt * 16 + (lane & 15)) * TPITCH + kk * 16 + (lane >> 4) * 8]), a[mt][0], a[mt][1], a[mt][2],
                a[mt][3]);
#pragma unroll
      for (int nb = 0; nb < 2; ++nb) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(smem_u32(&Ws[st][(wn * 32 + nb * 16 + (lane >> 4) * 8 + (lane & 7)) * TPITCH + kk * 16 + ((lane >> 3) & 1) * 8]), b0, b1,
                b2, b3);
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
          mma_bf16(acc[mt][2 * nb], a[mt], b0, b1);
          mma_bf16(acc[mt][2 * nb + 1], a[mt], b2, b3);
        }
      }
    }
  }
  cp_wait<0>();
  const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int m = wm * 32 + mt * 16 + g + half * 8;
        const int col = n0 + wn * 32 + nt * 8 + 2 * t4;
        if (m >= M) continue;
        TC* cp = C + (crow0 + m) * ldc + col;
        if (col < N) cp[0] = from_f32<TC>(acc[mt][nt][2 * half]);
        if (col + 1 < N) cp[1] = from_f32<TC>(acc[mt][nt][2 * half + 1]);
      }
}

__global__ void __launch_bounds__(256) moe_gemm_mma_kernel(const __nv_bfloat16* __restrict__ A, int lda, const int* __restrict__ rows,
                                                           const __nv_bfloat16* __restrict__ W, int ldw, long w_expert,
                                                           __nv_bfloat16* __restrict__ C, int ldc, const int* __restrict__ plan, int E,
                                                           int N, int K) {
  pdl_launch_dependents();
  pdl_wait();
  const int tile = blockIdx.y;
  if (tile >= plan[E + 1]) return;
  const int* tt = plan + E + 2 + 3 * tile;
  const int expert = tt[0], p0 = tt[1], M = tt[2];
  __shared__ __align__(16) __nv_bfloat16 As[kStages][TM * TPITCH];
  __shared__ __align__(16) __nv_bfloat16 Ws[kStages][TN * TPITCH];
  __shared__ int arow[TM];
  if (threadIdx.x < TM) arow[threadIdx.x] = (int)threadIdx.x < M ? (rows ? rows[p0 + threadIdx.x] : p0 + (int)threadIdx.x) : -1;
  __syncthreads();
  mma_tile_64x128(A, lda, arow, W + (size_t)expert * w_expert, ldw, C, ldc, (size_t)p0, M, blockIdx.x * TN, N, K, As, Ws);
}

// The same tile for one matrix per head, heads side by side in the rows of A and C (see arle_gemm_heads): grid (column
// tiles, row tiles, heads).
template <typename TC>
__global__ void __launch_bounds__(256) gemm_heads_mma_kernel(const __nv_bfloat16* __restrict__ A, int lda, int a_head,
                                                             const __nv_bfloat16* __restrict__ W, int ldw, long w_head,
                                                             TC* __restrict__ C, int ldc, int c_head, int M, int N, int K) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ __align__(16) __nv_bfloat16 As[kStages][TM * TPITCH];
  __shared__ __align__(16) __nv_bfloat16 Ws[kStages][TN * TPITCH];
  __shared__ int arow[TM];
  const int m0 = blockIdx.y * TM, head = blockIdx.z;
  if (threadIdx.x < TM) arow[threadIdx.x] = m0 + (int)threadIdx.x < M ? m0 + (int)threadIdx.x : -1;
  __syncthreads();
  mma_tile_64x128(A + (size_t)head * a_head, lda, arow, W + (size_t)head * w_head, ldw, C + (size_t)head * c_head, ldc, (size_t)m0,
                  min(TM, M - m0), blockIdx.x * TN, N, K, As, Ws);
}

// bfloat16 A and W, K and every stride a multiple of 8 elements, bases on 16-byte boundaries; C bfloat16 or (c_dtype 0) float32.
ARLE_API int arle_gemm_heads_mma(const void* A, const void* W, void* C, int c_dtype, int M, int N, int K, int heads, int lda, int ldw, int ldc,
                                 int a_head, long w_head, int c_head, cudaStream_t s) {
  if (M <= 0 || N <= 0 || heads <= 0) return 0;
  if (K <= 0) return ARLE_E_BADARG;
  if (K % 8 || lda % 8 || ldw % 8 || a_head % 8 || w_head % 8 || ((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return ARLE_E_UNSUPPORTED;
  dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM, heads);
  if (grid.y > 65535 || heads > 65535) return ARLE_E_UNSUPPORTED;
  if (c_dtype == 0)
    launch_kernel(gemm_heads_mma_kernel<float>, dim3(grid), dim3(256), 0, s, 1, (const __nv_bfloat16*)A, lda, a_head, (const __nv_bfloat16*)W,
                  ldw, w_head, (float*)C, ldc, c_head, M, N, K);
  else
    launch_kernel(gemm_heads_mma_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, s, 1, (const __nv_bfloat16*)A, lda, a_head,
                  (const __nv_bfloat16*)W, ldw, w_head, (__nv_bfloat16*)C, ldc, c_head, M, N, K);
  return launch_status();
}

// One warp per (place, output column): the dot product of the place's row of A with one row of its expert's matrix,
// eight elements a lane and load (K a multiple of 8, rows on 16-byte boundaries).
__global__ void __launch_bounds__(256) moe_gemv_kernel(const __nv_bfloat16* __restrict__ A, int lda, const int* __restrict__ rows,
                                                       const __nv_bfloat16* __restrict__ W, int ldw, long w_expert,
                                                       __nv_bfloat16* __restrict__ C, int ldc, const int* __restrict__ plan, int E, int N,
                                                       int K) {
  pdl_launch_dependents();
  pdl_wait();
  const int place = blockIdx.y;
  if (place >= plan[E]) return;
  const int lane = threadIdx.x & 31;
  const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (n >= N) return;
  int expert = 0;
  while (expert + 1 < E && plan[expert + 1] <= place) ++expert;
  const __nv_bfloat16* a = A + (size_t)(rows ? rows[place] : place) * lda;
  const __nv_bfloat16* w = W + (size_t)expert * w_expert + (size_t)n * ldw;
  float acc = 0.f;
  for (int k = lane * 8; k < K; k += 256) {
    const uint4 av = *reinterpret_cast<const uint4*>(a + k);
    const uint4 wv = *reinterpret_cast<const uint4*>(w + k);
    const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&av);
    const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      acc = fmaf(__low2float(a2[i]), __low2float(w2[i]), acc);
      acc = fmaf(__high2float(a2[i]), __high2float(w2[i]), acc);
    }
  }
  acc = warp_sum(acc);
  if (lane == 0) C[(size_t)place * ldc + n] = __float2bfloat16_rn(acc);
}

// dtype: type of A and C; w_dtype: type of W [E][N][K] (an expert every w_expert elements).  pairs: places in all.
// fast: bfloat16 operands with aligned rows may take the tensor-core tiles or, for few pairs, the dot products.
ARLE_API int arle_moe_gemm(const void* A, int lda, const int* rows, const void* W, int ldw, long w_expert, void* C, int ldc,
                           int dtype, int w_dtype, const int* plan, int E, int pairs, int N, int K, int fast, cudaStream_t s) {
  if (pairs <= 0 || N <= 0) return 0;
  if (K <= 0 || E <= 0) return ARLE_E_BADARG;
  const int max_tiles = pairs / kMoeTile + E + 1;
  if (max_tiles > 65535) return ARLE_E_UNSUPPORTED;
  if (fast && dtype == 1 && w_dtype == 1 && K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0 && w_expert % 8 == 0 &&
      ((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0) {
    if (pairs <= 128) {
      launch_kernel(moe_gemv_kernel, dim3((N + 7) / 8, pairs), dim3(256), 0, s, 1, (const __nv_bfloat16*)A, lda, rows,
                    (const __nv_bfloat16*)W, ldw, w_expert, (__nv_bfloat16*)C, ldc, plan, E, N, K);
    } else {
      launch_kernel(moe_gemm_mma_kernel, dim3((N + TN - 1) / TN, max_tiles), dim3(256), 0, s, 1, (const __nv_bfloat16*)A, lda, rows,
                    (const __nv_bfloat16*)W, ldw, w_expert, (__nv_bfloat16*)C, ldc, plan, E, N, K);
    }
    return launch_status();
  }
  dim3 grid((N + GN - 1) / GN, max_tiles);
  if (dtype == 0 && w_dtype == 0)
    launch_kernel(moe_gemm_kernel<float, float, float>, dim3(grid), dim3(256), 0, s, 1, (const float*)A, lda, rows, (const float*)W, ldw,
                  w_expert, (float*)C, ldc, plan, E, N, K);
  else if (dtype == 0 && w_dtype == 1)
    launch_kernel(moe_gemm_kernel<float, __nv_bfloat16, float>, dim3(grid), dim3(256), 0, s, 1, (const float*)A, lda, rows,
                  (const __nv_bfloat16*)W, ldw, w_expert, (float*)C, ldc, plan, E, N, K);
  else if (dtype == 1 && w_dtype == 1)
    launch_kernel(moe_gemm_kernel<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>, dim3(grid), dim3(256), 0, s, 1, (const __nv_bfloat16*)A,
                  lda, rows, (const __nv_bfloat16*)W, ldw, w_expert, (__nv_bfloat16*)C, ldc, plan, E, N, K);
  else
    return ARLE_E_BADARG;
  return launch_status();
}

template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ y, int y_stride, const int* __restrict__ place_of_pair,
                                   const float* __restrict__ wts, int top, const T* __restrict__ shared, int shared_stride,
                                   const float* __restrict__ gate, int gate_stride, T* __restrict__ out, int out_stride, int width) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  float g = 1.f;
  if (shared && gate) g = 1.0f / (1.0f + expf(-gate[(size_t)t * gate_stride]));
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k)
      acc = fmaf(wts[(size_t)t * top + k], to_f32(y[(size_t)place_of_pair[(size_t)t * top + k] * y_stride + c]), acc);
    if (shared) acc = fmaf(g, to_f32(shared[(size_t)t * shared_stride + c]), acc);
    out[(size_t)t * out_stride + c] = from_f32<T>(acc);
  }
}

ARLE_API int arle_moe_combine(const void* y, int y_stride, const int* place_of_pair, const float* wts, int top, const void* shared,
                              int shared_stride, const float* gate, int gate_stride, void* out, int out_stride, int dtype,
                              int num_tokens, int width, cudaStream_t s) {
  if (num_tokens <= 0) return 0;
  if (width <= 0 || top <= 0) return ARLE_E_BADARG;
  const int threads = width >= 1024 ? 256 : 128;
  if (dtype == 0)
    launch_kernel(moe_combine_kernel<float>, dim3(num_tokens), dim3(threads), 0, s, 1, (const float*)y, y_stride, place_of_pair, wts, top,
                  (const float*)shared, shared_stride, gate, gate_stride, (float*)out, out_stride, width);
  else if (dtype == 1)
    launch_kernel(moe_combine_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(threads), 0, s, 1, (const __nv_bfloat16*)y, y_stride,
                  place_of_pair, wts, top, (const __nv_bfloat16*)shared, shared_stride, gate, gate_stride, (__nv_bfloat16*)out,
                  out_stride, width);
  else
    return ARLE_E_BADARG;
  return launch_status();
}
