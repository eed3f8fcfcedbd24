// Mixture of experts: router, grouping of (token, chosen expert) pairs by expert, the experts' two
// matrix products as grouped products over that order, and the weighted sum back per token.
//
//   route:   z = W_router x in 32-bit (one warp per expert row, lane-strided k in a fixed order, butterfly sum);
//            scores = sigmoid(z) or softmax(z); the `top` largest (lowest index among equals); weights are
//            the chosen scores, optionally divided by their sum.  Optionally the choice goes by
//            score + correction[e] (the weights stay the scores), only experts of the `keep` best of `groups`
//            equal groups of neighbouring experts can be chosen (a group's score: its largest choice score),
//            and the weights are multiplied by a constant.  Extra rows (a shared expert's gate) are
//            dotted the same way and leave sigmoid(row . x).
//   align:   pairs p = token * top + slot are laid out expert by expert, each expert's run padded to whole
//            tiles of MOE_BM rows with -1, with the expert of every tile and the number of tiles used
//            (optionally also the row of every pair and where each expert's run begins).
//            Launch sizes depend on the batch's shape only: blocks beyond the tiles used leave at once.
//   gemm:    out[p, n] = sum_k a(p, k) * w[expert(p), n, k], one accumulator per output taking its
//            products in ascending k, so a pair's result depends on nothing else in the batch.
//            a(p, k) = A[p / a_row_div, k] (* pair weight, rounded to the storage type): the weight
//            multiplies the expert's INPUT.  GATED: w holds gate rows [0, N) and up rows [N, 2N) and
//            out = silu(gate) * up.
//   gemv:    the same two products for a handful of pairs in bf16, bound by the bytes of the chosen
//            experts' matrices (no padded tiles).
//   gather:  the pairs' input rows expert by expert at a common stride, for one batched library product
//            over all experts.
//   combine: y[token] = sum over slots of out[row of (token, slot)] (ascending slot, 32-bit)
//            (+ gate[token] * shared[token]).
#include "common.cuh"

#define MOE_BM 16
#define MOE_BN 64
#define MOE_BK 16
#define MOE_ROUTE_THREADS 512

// TPB tokens a block share every pass over a router row (a prompt's tokens would otherwise each pull the
// whole router through the L2 cache); a token's sums are formed in the same order whatever TPB is: lane l
// adds the products k = l, l + 32, ... into four partial sums by (k / 32) % 4, then ((p0 + p1) + (p2 + p3)),
// then the butterfly over the lanes.
template <typename T, int TPB>
__global__ void __launch_bounds__(MOE_ROUTE_THREADS)
moe_route_kernel(int* __restrict__ ids_out, float* __restrict__ weights_out, float* __restrict__ gate_out,
                 const T* __restrict__ x, long long x_stride, const float* __restrict__ router,
                 const float* __restrict__ gate_rows, int tokens, int E, int R, int K, int top, int score_mode,
                 int renormalize, const float* __restrict__ correction, int groups, int keep, float weight_scale) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_MOE_ROUTE);
  extern __shared__ __align__(16) unsigned char route_smem[];
  T* xs = reinterpret_cast<T*>(route_smem);                                   // [TPB][K]
  float* scores = reinterpret_cast<float*>(route_smem + (size_t)TPB * K * sizeof(T));   // [TPB][E + R]
  float* choices = scores + (size_t)TPB * (E + R);                                      // [TPB][E + 2 * groups]
  const int token0 = blockIdx.x * TPB;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = MOE_ROUTE_THREADS / 32;
  for (int i = threadIdx.x; i < TPB * K; i += MOE_ROUTE_THREADS) {
    const int t = i / K, k = i % K;
    xs[i] = token0 + t < tokens ? x[(size_t)(token0 + t) * x_stride + k] : from_float<T>(0.0f);
  }
  __syncthreads();
  for (int e = warp; e < E + R; e += nwarps) {
    const float* w = e < E ? router + (size_t)e * K : gate_rows + (size_t)(e - E) * K;
    float part[TPB][4];
#pragma unroll
    for (int t = 0; t < TPB; ++t) part[t][0] = part[t][1] = part[t][2] = part[t][3] = 0.0f;
    int k = lane;
    for (; k + 96 < K; k += 128) {
      const float w0 = w[k], w1 = w[k + 32], w2 = w[k + 64], w3 = w[k + 96];
#pragma unroll
      for (int t = 0; t < TPB; ++t) {
        const T* xt = xs + (size_t)t * K;
        part[t][0] = fmaf(w0, to_float(xt[k]), part[t][0]);
        part[t][1] = fmaf(w1, to_float(xt[k + 32]), part[t][1]);
        part[t][2] = fmaf(w2, to_float(xt[k + 64]), part[t][2]);
        part[t][3] = fmaf(w3, to_float(xt[k + 96]), part[t][3]);
      }
    }
    for (int j = 0; k < K; k += 32, ++j) {
      const float wk = w[k];
#pragma unroll
      for (int t = 0; t < TPB; ++t) {
        const float prod_x = to_float(xs[(size_t)t * K + k]);
        if (j == 0) part[t][0] = fmaf(wk, prod_x, part[t][0]);
        else if (j == 1) part[t][1] = fmaf(wk, prod_x, part[t][1]);
        else part[t][2] = fmaf(wk, prod_x, part[t][2]);
      }
    }
#pragma unroll
    for (int t = 0; t < TPB; ++t) {
      const float acc = warp_sum((part[t][0] + part[t][1]) + (part[t][2] + part[t][3]));
      if (lane == 0) scores[t * (E + R) + e] = acc;
    }
  }
  __syncthreads();
  if (warp >= TPB || token0 + warp >= tokens) return;
  const int token = token0 + warp;                    // warp t finishes token t of the block
  float* sc = scores + warp * (E + R);
  for (int r = lane; r < R; r += 32) gate_out[(size_t)token * R + r] = 1.0f / (1.0f + expf(-sc[E + r]));
  if (score_mode == 0) {
    for (int e = lane; e < E; e += 32) sc[e] = 1.0f / (1.0f + expf(-sc[e]));
  } else {
    float m = -INFINITY;
    for (int e = lane; e < E; e += 32) m = fmaxf(m, sc[e]);
    m = warp_max(m);
    float sum = 0.0f;
    for (int e = lane; e < E; e += 32) { const float p = expf(sc[e] - m); sc[e] = p; sum += p; }
    sum = warp_sum(sum);
    for (int e = lane; e < E; e += 32) sc[e] = sc[e] / sum;
  }
  __syncwarp();
  // what the choice goes by: the scores, with the correction when there is one
  float* ch = choices + warp * (E + 2 * groups);
  for (int e = lane; e < E; e += 32) ch[e] = correction != nullptr ? sc[e] + correction[e] : sc[e];
  __syncwarp();
  auto arg_max = [&](const float* values, int count, float& best, int& best_i) {
    best = -INFINITY;
    best_i = 0x7fffffff;
    for (int i = lane; i < count; i += 32) {
      const float v = values[i];
      if (v > best) { best = v; best_i = i; }   // ascending i: the lowest index among equals stays
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (best_i == 0x7fffffff) best_i = 0;       // nothing but minus infinity or NaN: stay inside the arrays
  };
  if (keep < groups) {
    // a group's score is its largest choice score; experts outside the `keep` best groups cannot be chosen
    const int per = E / groups;
    float* gs = ch + E;
    float* kept = gs + groups;
    for (int g = lane; g < groups; g += 32) {
      float m = -INFINITY;
      for (int e = g * per; e < (g + 1) * per; ++e) m = fmaxf(m, ch[e]);
      gs[g] = m;
      kept[g] = 0.0f;
    }
    __syncwarp();
    for (int n = 0; n < keep; ++n) {
      float best; int best_g;
      arg_max(gs, groups, best, best_g);
      if (lane == 0) { gs[best_g] = -INFINITY; kept[best_g] = 1.0f; }
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32)
      if (kept[e / per] == 0.0f) ch[e] = -INFINITY;
    __syncwarp();
  }
  float chosen_sum = 0.0f;
  for (int slot = 0; slot < top; ++slot) {
    float best; int best_e;
    arg_max(ch, E, best, best_e);
    const float weight = sc[best_e];
    if (lane == 0) {
      ids_out[(size_t)token * top + slot] = best_e;
      weights_out[(size_t)token * top + slot] = weight;
      ch[best_e] = -INFINITY;
    }
    chosen_sum += weight;
    __syncwarp();
  }
  if (lane == 0 && (renormalize || weight_scale != 1.0f))
    for (int slot = 0; slot < top; ++slot) {
      float w = weights_out[(size_t)token * top + slot];
      if (renormalize) w /= chosen_sum;
      weights_out[(size_t)token * top + slot] = w * weight_scale;
    }
}

template <typename T, int TPB>
static int launch_moe_route(int* ids_out, float* weights_out, float* gate_out, const void* x, long long x_stride,
                            const float* router, const float* gate_rows, int tokens, int E, int R, int K, int top,
                            int score_mode, int renormalize, const float* correction, int groups, int keep,
                            float weight_scale, cudaStream_t stream) {
  const size_t smem = (size_t)TPB * K * sizeof(T) + (size_t)TPB * (2 * E + R + 2 * groups) * sizeof(float);
  KVB_REQUIRE(smem <= 200 * 1024, "moe_route: the tokens' rows and scores do not fit in shared memory");
  if (smem > 48 * 1024)
    KVB_CHECK_CUDA(cudaFuncSetAttribute(moe_route_kernel<T, TPB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  KVB_CHECK_CUDA(kvb_launch((moe_route_kernel<T, TPB>), dim3((tokens + TPB - 1) / TPB), dim3(MOE_ROUTE_THREADS), smem,
                            stream, true, ids_out, weights_out, gate_out, (const T*)x, x_stride, router, gate_rows,
                            tokens, E, R, K, top, score_mode, renormalize, correction, groups, keep, weight_scale));
  return 0;
}

extern "C" int kvb_moe_route(int* ids_out, float* weights_out, float* gate_out, const void* x, long long x_stride,
                             const float* router, const float* gate_rows, int tokens, int E, int R, int K, int top,
                             int score_mode, int renormalize, const float* correction, int groups, int keep,
                             float weight_scale, int dtype, cudaStream_t stream) {
  if (tokens == 0) return 0;
  KVB_REQUIRE(E > 0 && K > 0 && top > 0 && top <= E, "moe_route: need 0 < top <= experts");
  KVB_REQUIRE(groups > 0 && E % groups == 0 && keep > 0 && keep <= groups && (long long)keep * (E / groups) >= top,
              "moe_route: the kept groups of experts must hold the experts to choose");
  KVB_REQUIRE(R >= 0 && (R == 0 || (gate_rows != nullptr && gate_out != nullptr)), "moe_route: gate rows need their weights and output");
  KVB_REQUIRE(score_mode == 0 || score_mode == 1, "moe_route: unknown score function");
  // a prompt's tokens go eight a block; a few tokens one a block, for the parallelism
  const bool many = tokens >= 256 && (size_t)8 * K * (dtype == KVB_F32 ? 4 : 2) <= 96 * 1024;
  int rc;
  if (dtype == KVB_F32)
    rc = many ? launch_moe_route<float, 8>(ids_out, weights_out, gate_out, x, x_stride, router, gate_rows, tokens, E, R, K, top, score_mode, renormalize, correction, groups, keep, weight_scale, stream)
              : launch_moe_route<float, 1>(ids_out, weights_out, gate_out, x, x_stride, router, gate_rows, tokens, E, R, K, top, score_mode, renormalize, correction, groups, keep, weight_scale, stream);
  else
    rc = many ? launch_moe_route<bf16, 8>(ids_out, weights_out, gate_out, x, x_stride, router, gate_rows, tokens, E, R, K, top, score_mode, renormalize, correction, groups, keep, weight_scale, stream)
              : launch_moe_route<bf16, 1>(ids_out, weights_out, gate_out, x, x_stride, router, gate_rows, tokens, E, R, K, top, score_mode, renormalize, correction, groups, keep, weight_scale, stream);
  if (rc) return rc;
  KVB_CHECK_LAUNCH();
  return 0;
}

// sorted [capacity] (capacity = MOE_BM * min(pairs, ceil((pairs + experts * (MOE_BM - 1)) / MOE_BM))),
// tile_expert [capacity / MOE_BM], meta[0] = tiles used.
__global__ void __launch_bounds__(1024)
moe_align_kernel(int* __restrict__ sorted, int* __restrict__ tile_expert, int* __restrict__ meta,
                 int* __restrict__ row_of_pair, int* __restrict__ expert_begin,
                 const int* __restrict__ ids, int pairs, int E, int capacity, int* status) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_MOE_ALIGN);
  extern __shared__ int ismem[];
  int* counts = ismem;        // [E]
  int* offsets = ismem + E;   // [E]
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
  for (int i = threadIdx.x; i < capacity; i += blockDim.x) sorted[i] = -1;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = ids[p];
    if (e >= 0 && e < E) atomicAdd(&counts[e], 1);
    else atomicOr(status, KVB_STATUS_BAD_TOKEN);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < E; ++e) {
      offsets[e] = at;
      const int tiles = (counts[e] + MOE_BM - 1) / MOE_BM;
      for (int t = 0; t < tiles; ++t) tile_expert[at / MOE_BM + t] = e;
      at += tiles * MOE_BM;
      counts[e] = 0;   // becomes the fill cursor
    }
    meta[0] = at / MOE_BM;
    if (expert_begin != nullptr) {   // where each expert's (padded) run of rows begins, and the end of the last
      for (int e = 0; e < E; ++e) expert_begin[e] = offsets[e];
      expert_begin[E] = at;
    }
  }
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = ids[p];
    if (e >= 0 && e < E) {
      const int row = offsets[e] + atomicAdd(&counts[e], 1);
      sorted[row] = p;
      if (row_of_pair != nullptr) row_of_pair[p] = row;
    } else if (row_of_pair != nullptr) {
      row_of_pair[p] = -1;
    }
  }
}

extern "C" int kvb_moe_align(int* sorted, int* tile_expert, int* meta, int* row_of_pair, int* expert_begin,
                             const int* ids, int pairs, int E, int capacity, cudaStream_t stream) {
  if (pairs == 0) return 0;
  KVB_REQUIRE(E > 0 && E <= 8192, "moe_align: between 1 and 8192 experts");
  // tiles used: one per started run of MOE_BM pairs of an expert, so at most one per pair
  const long long padded = (pairs + (long long)E * (MOE_BM - 1) + MOE_BM - 1) / MOE_BM;
  KVB_REQUIRE(capacity % MOE_BM == 0 && capacity / MOE_BM >= (padded < pairs ? padded : pairs),
              "moe_align: the sorted list is too short");
  int* status = kvb_status_word();
  KVB_REQUIRE(status != nullptr, "moe_align: no status word");
  KVB_CHECK_CUDA(kvb_launch((moe_align_kernel), dim3(1), dim3(1024), (size_t)2 * E * sizeof(int), stream, true,
                            sorted, tile_expert, meta, row_of_pair, expert_begin, ids, pairs, E, capacity, status));
  KVB_CHECK_LAUNCH();
  return 0;
}

extern "C" int kvb_moe_tile_rows() { return MOE_BM; }

template <typename T>
__device__ __forceinline__ float moe_silu(float x);
template <>
__device__ __forceinline__ float moe_silu<float>(float x) { return x / (1.0f + expf(-x)); }
template <>
__device__ __forceinline__ float moe_silu<bf16>(float x) { return kvb_silu_for_bf16(x); }

template <typename T, bool GATED>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(T* __restrict__ out, const T* __restrict__ a, long long a_stride, int a_row_div,
                const float* __restrict__ pair_weight, const T* __restrict__ w, const int* __restrict__ sorted,
                const int* __restrict__ tile_expert, const int* __restrict__ meta, int N, int K) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_MOE_GEMM);
  if ((int)blockIdx.x >= meta[0]) return;
  __shared__ float as[MOE_BK][MOE_BM + 1];
  __shared__ float ws[GATED ? 2 : 1][MOE_BK][MOE_BN + 4];
  __shared__ int pair_of[MOE_BM];
  const int expert = tile_expert[blockIdx.x];
  if (threadIdx.x < MOE_BM) pair_of[threadIdx.x] = sorted[blockIdx.x * MOE_BM + threadIdx.x];
  __syncthreads();
  const int n0 = blockIdx.y * MOE_BN;
  const size_t rows_per_expert = (size_t)(GATED ? 2 : 1) * N;
  const T* we = w + (size_t)expert * rows_per_expert * K;
  const int r = threadIdx.x >> 4, c0 = (threadIdx.x & 15) * 4;
  float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f}, acc_up[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  // this thread's element of the A tile: row a_r, column a_k of every slab
  const int a_r = threadIdx.x >> 4, a_k = threadIdx.x & 15;
  const int a_pair = pair_of[a_r];
  const T* a_row = a_pair >= 0 ? a + (size_t)(a_pair / a_row_div) * a_stride : nullptr;
  const float a_scale = (a_pair >= 0 && pair_weight != nullptr) ? pair_weight[a_pair] : 1.0f;
  for (int k0 = 0; k0 < K; k0 += MOE_BK) {
    {
      const int k = k0 + a_k;
      float v = 0.0f;
      if (a_row != nullptr && k < K) {
        v = to_float(a_row[k]);
        if (pair_weight != nullptr) v = to_float(from_float<T>(v * a_scale));
      }
      as[a_k][a_r] = v;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = threadIdx.x + i * 256;
      const int row = idx >> 4, kk = idx & 15;
      const int n = n0 + row, k = k0 + kk;
      const bool ok = n < N && k < K;
      ws[0][kk][row] = ok ? to_float(we[(size_t)n * K + k]) : 0.0f;
      if (GATED) ws[1][kk][row] = ok ? to_float(we[(size_t)(N + n) * K + k]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < MOE_BK; ++kk) {
      const float av = as[kk][r];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[j] = fmaf(av, ws[0][kk][c0 + j], acc[j]);
        if (GATED) acc_up[j] = fmaf(av, ws[1][kk][c0 + j], acc_up[j]);
      }
    }
    __syncthreads();
  }
  const int pair = pair_of[r];
  if (pair < 0) return;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int n = n0 + c0 + j;
    if (n >= N) continue;
    float v = acc[j];
    if (GATED) {
      // as the separate kernels would: both products rounded, the activation rounded, then the product
      const float g = to_float(from_float<T>(acc[j])), u = to_float(from_float<T>(acc_up[j]));
      v = to_float(from_float<T>(moe_silu<T>(g))) * u;
    }
    out[(size_t)pair * N + n] = from_float<T>(v);
  }
}

extern "C" int kvb_moe_gemm(void* out, const void* a, long long a_stride, int a_row_div, const float* pair_weight,
                            const void* w, const int* sorted, const int* tile_expert, const int* meta, int max_tiles,
                            int N, int K, int gated, int dtype, cudaStream_t stream) {
  if (max_tiles == 0) return 0;
  KVB_REQUIRE(N > 0 && K > 0 && a_row_div > 0, "moe_gemm: empty product");
  dim3 grid(max_tiles, (N + MOE_BN - 1) / MOE_BN);
  KVB_REQUIRE(grid.y <= 65535, "moe_gemm: too many output columns for one launch");
#define KVB_MOE_GEMM(T_, G_)                                                                                  \
  KVB_CHECK_CUDA(kvb_launch((moe_gemm_kernel<T_, G_>), grid, dim3(256), 0, stream, true, (T_*)out, (const T_*)a, \
                            a_stride, a_row_div, pair_weight, (const T_*)w, sorted, tile_expert, meta, N, K))
  if (dtype == KVB_F32) { if (gated) KVB_MOE_GEMM(float, true); else KVB_MOE_GEMM(float, false); }
  else { if (gated) KVB_MOE_GEMM(bf16, true); else KVB_MOE_GEMM(bf16, false); }
#undef KVB_MOE_GEMM
  KVB_CHECK_LAUNCH();
  return 0;
}

// Decode-sized batches in bf16: one pass over each chosen expert's matrices.  grid (N / 32, pairs): a block
// holds the pair's input row (weighted and rounded) in shared memory; each of its 8 warps owns 4 output
// columns (GATED: the 4 gate rows and the 4 up rows) and walks K in 16-byte loads, lane-strided, the four
// rows' loads in flight together; a butterfly sums the lanes.  No tile is padded with rows that are not
// there, so the kernel is bound by the weights it reads.
#define MOE_GEMV_COLS 32
template <bool GATED>
__global__ void __launch_bounds__(256)
moe_gemv_kernel(bf16* __restrict__ out, const bf16* __restrict__ a, long long a_stride, int a_row_div,
                const float* __restrict__ pair_weight, const bf16* __restrict__ w, const int* __restrict__ ids,
                int E, int N, int K, int* status) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_MOE_GEMM);
  extern __shared__ __align__(16) unsigned char gemv_smem[];
  bf16* xs = reinterpret_cast<bf16*>(gemv_smem);
  const int pair = blockIdx.y;
  const int expert = ids[pair];
  if (expert < 0 || expert >= E) {
    if (threadIdx.x == 0) atomicOr(status, KVB_STATUS_BAD_TOKEN);
    return;
  }
  const bf16* row = a + (size_t)(pair / a_row_div) * a_stride;
  const float scale = pair_weight != nullptr ? pair_weight[pair] : 1.0f;
  for (int k = threadIdx.x * 8; k < K; k += 256 * 8) {
    Vec16<bf16> v;
    v.load(row + k);
    if (pair_weight != nullptr) {
#pragma unroll
      for (int j = 0; j < 8; ++j) v.set(j, v.get(j) * scale);
    }
    v.store(xs + k);
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * MOE_GEMV_COLS + warp * 4;
  const bf16* we = w + (size_t)expert * (GATED ? 2 : 1) * N * K;
  constexpr int ROWS = GATED ? 8 : 4;
  const bf16* rows[ROWS];
  float acc[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const int n = min(n0 + (r & 3), N - 1) + (r >= 4 ? N : 0);
    rows[r] = we + (size_t)n * K;
    acc[r] = 0.0f;
  }
  for (int k = lane * 8; k < K; k += 32 * 8) {
    Vec16<bf16> x, wv[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) wv[r].load(rows[r] + k);
    x.load(xs + k);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float xv = x.get(j);
#pragma unroll
      for (int r = 0; r < ROWS; ++r) acc[r] = fmaf(wv[r].get(j), xv, acc[r]);
    }
  }
#pragma unroll
  for (int r = 0; r < ROWS; ++r) acc[r] = warp_sum(acc[r]);
  if (lane < 4 && n0 + lane < N) {
    float v = lane == 0 ? acc[0] : lane == 1 ? acc[1] : lane == 2 ? acc[2] : acc[3];
    if (GATED) {
      const float u = lane == 0 ? acc[4 % ROWS] : lane == 1 ? acc[5 % ROWS] : lane == 2 ? acc[6 % ROWS] : acc[7 % ROWS];
      const float g = to_float(from_float<bf16>(v));
      v = to_float(from_float<bf16>(moe_silu<bf16>(g))) * to_float(from_float<bf16>(u));
    }
    out[(size_t)pair * N + n0 + lane] = from_float<bf16>(v);
  }
}

extern "C" int kvb_moe_gemv(void* out, const void* a, long long a_stride, int a_row_div, const float* pair_weight,
                            const void* w, const int* ids, int pairs, int E, int N, int K, int gated,
                            cudaStream_t stream) {
  if (pairs == 0) return 0;
  KVB_REQUIRE(N > 0 && K > 0 && K % 8 == 0 && a_stride % 8 == 0 && a_row_div > 0, "moe_gemv: K and the row stride must be multiples of 8");
  KVB_REQUIRE(aligned16(a) && aligned16(w), "moe_gemv: operands must be 16-byte aligned");
  KVB_REQUIRE(pairs <= 65535, "moe_gemv: too many pairs for one launch");
  const size_t smem = (size_t)K * sizeof(bf16);
  KVB_REQUIRE(smem <= 200 * 1024, "moe_gemv: an input row does not fit in shared memory");
  int* status = kvb_status_word();
  KVB_REQUIRE(status != nullptr, "moe_gemv: no status word");
  dim3 grid((N + MOE_GEMV_COLS - 1) / MOE_GEMV_COLS, pairs);
#define KVB_MOE_GEMV(G_)                                                                                       \
  do {                                                                                                         \
    if (smem > 48 * 1024)                                                                                      \
      KVB_CHECK_CUDA(cudaFuncSetAttribute(moe_gemv_kernel<G_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    KVB_CHECK_CUDA(kvb_launch((moe_gemv_kernel<G_>), grid, dim3(256), smem, stream, true, (bf16*)out, (const bf16*)a, \
                              a_stride, a_row_div, pair_weight, (const bf16*)w, ids, E, N, K, status));        \
  } while (0)
  if (gated) KVB_MOE_GEMV(true); else KVB_MOE_GEMV(false);
#undef KVB_MOE_GEMV
  KVB_CHECK_LAUNCH();
  return 0;
}

// The same for a few hundred pairs: the pairs of one expert share one pass over its matrices.  grid (N / 128,
// 2 * tiles): a block takes one half (8 rows) of a tile of the grouped order (moe_align), holds those pairs'
// input rows in shared memory and gives each warp 2 output columns (GATED: 2 gate and 2 up rows) for all
// 8 rows, 8 such groups of 16 columns one after the other; a weight vector is loaded once and used for every
// row, the staged rows for 128 columns.  (Four columns a warp cost 176 registers and left one block a
// multiprocessor; one group of columns a block spent more bytes on staging the rows than on weights.)
#define MOE_GEMV_ROWS 8
#define MOE_GEMV_ROWS_CPW 2                                  // output columns a warp (GATED: that many gate and up rows)
#define MOE_GEMV_ROWS_COLS (8 * MOE_GEMV_ROWS_CPW)           // output columns of one group: 8 warps
#define MOE_GEMV_ROWS_GROUPS 8                               // groups of columns a block walks with the rows it staged
template <bool GATED>
__global__ void __launch_bounds__(256)
moe_gemv_rows_kernel(bf16* __restrict__ out, const bf16* __restrict__ a, long long a_stride, int a_row_div,
                     const float* __restrict__ pair_weight, const bf16* __restrict__ w,
                     const int* __restrict__ sorted, const int* __restrict__ tile_expert,
                     const int* __restrict__ meta, int N, int K) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_MOE_GEMM);
  extern __shared__ __align__(16) unsigned char gemv_smem[];
  bf16* xs = reinterpret_cast<bf16*>(gemv_smem);            // [MOE_GEMV_ROWS][K]
  __shared__ int pair_of[MOE_GEMV_ROWS];
  const int tile = blockIdx.y >> 1, half = blockIdx.y & 1;
  if (tile >= meta[0]) return;
  const int first = sorted[tile * MOE_BM + half * MOE_GEMV_ROWS];
  if (first < 0) return;                                     // a run fills its tiles from the front
  if (threadIdx.x < MOE_GEMV_ROWS) pair_of[threadIdx.x] = sorted[tile * MOE_BM + half * MOE_GEMV_ROWS + threadIdx.x];
  __syncthreads();
  const int expert = tile_expert[tile];
  for (int i = threadIdx.x * 8; i < MOE_GEMV_ROWS * K; i += 256 * 8) {
    const int r = i / K, k = i % K;
    const int pair = pair_of[r];
    Vec16<bf16> v;
    if (pair >= 0) {
      v.load(a + (size_t)(pair / a_row_div) * a_stride + k);
      if (pair_weight != nullptr) {
        const float scale = pair_weight[pair];
#pragma unroll
        for (int j = 0; j < 8; ++j) v.set(j, v.get(j) * scale);
      }
    } else {
      v.raw = make_uint4(0, 0, 0, 0);
    }
    v.store(xs + i);
  }
  __syncthreads();
  constexpr int CPW = MOE_GEMV_ROWS_CPW;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bf16* we = w + (size_t)expert * (GATED ? 2 : 1) * N * K;
  constexpr int COLS = GATED ? 2 * CPW : CPW;
  // the staged rows serve MOE_GEMV_ROWS_GROUPS groups of columns, one after the other
  for (int group = 0; group < MOE_GEMV_ROWS_GROUPS; ++group) {
  const int n0 = (blockIdx.x * MOE_GEMV_ROWS_GROUPS + group) * MOE_GEMV_ROWS_COLS + warp * CPW;
  if (n0 >= N) break;                                        // uniform over the warp
  const bf16* cols[COLS];
  float acc[COLS][MOE_GEMV_ROWS];
#pragma unroll
  for (int c = 0; c < COLS; ++c) {
    const int n = min(n0 + (c % CPW), N - 1) + (c >= CPW ? N : 0);
    cols[c] = we + (size_t)n * K;
#pragma unroll
    for (int r = 0; r < MOE_GEMV_ROWS; ++r) acc[c][r] = 0.0f;
  }
  for (int k = lane * 8; k < K; k += 32 * 8) {
    Vec16<bf16> wv[COLS];
#pragma unroll
    for (int c = 0; c < COLS; ++c) wv[c].load(cols[c] + k);
#pragma unroll
    for (int r = 0; r < MOE_GEMV_ROWS; ++r) {
      Vec16<bf16> x;
      x.load(xs + (size_t)r * K + k);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xv = x.get(j);
#pragma unroll
        for (int c = 0; c < COLS; ++c) acc[c][r] = fmaf(wv[c].get(j), xv, acc[c][r]);
      }
    }
  }
#pragma unroll
  for (int c = 0; c < COLS; ++c)
#pragma unroll
    for (int r = 0; r < MOE_GEMV_ROWS; ++r) acc[c][r] = warp_sum(acc[c][r]);
  // lane (r, c) = (lane / CPW, lane % CPW) of the first 8 * CPW lanes writes one output
  const int r = lane / CPW, c = lane % CPW;
  float v = 0.0f, u = 0.0f;
#pragma unroll
  for (int rr = 0; rr < MOE_GEMV_ROWS; ++rr)
#pragma unroll
    for (int cc = 0; cc < CPW; ++cc)
      if (rr == r && cc == c) {
        v = acc[cc][rr];
        if (GATED) u = acc[(cc + CPW) % COLS][rr];
      }
  const int pair = lane < MOE_GEMV_ROWS * CPW ? pair_of[r] : -1;
  if (pair >= 0 && n0 + c < N) {
    if (GATED) {
      const float g = to_float(from_float<bf16>(v));
      v = to_float(from_float<bf16>(moe_silu<bf16>(g))) * to_float(from_float<bf16>(u));
    }
    out[(size_t)pair * N + n0 + c] = from_float<bf16>(v);
  }
  }
}

extern "C" int kvb_moe_gemv_rows(void* out, const void* a, long long a_stride, int a_row_div, const float* pair_weight,
                                 const void* w, const int* sorted, const int* tile_expert, const int* meta,
                                 int max_tiles, int N, int K, int gated, cudaStream_t stream) {
  if (max_tiles == 0) return 0;
  KVB_REQUIRE(N > 0 && K > 0 && K % 8 == 0 && a_stride % 8 == 0 && a_row_div > 0, "moe_gemv_rows: K and the row stride must be multiples of 8");
  KVB_REQUIRE(aligned16(a) && aligned16(w), "moe_gemv_rows: operands must be 16-byte aligned");
  KVB_REQUIRE(2 * (long long)max_tiles <= 65535, "moe_gemv_rows: too many tiles for one launch");
  const size_t smem = (size_t)MOE_GEMV_ROWS * K * sizeof(bf16);
  KVB_REQUIRE(smem <= 200 * 1024, "moe_gemv_rows: the input rows do not fit in shared memory");
  const int block_cols = MOE_GEMV_ROWS_COLS * MOE_GEMV_ROWS_GROUPS;
  dim3 grid((N + block_cols - 1) / block_cols, 2 * max_tiles);
#define KVB_MOE_GEMV_ROWS(G_)                                                                                 \
  do {                                                                                                        \
    if (smem > 48 * 1024)                                                                                     \
      KVB_CHECK_CUDA(cudaFuncSetAttribute(moe_gemv_rows_kernel<G_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    KVB_CHECK_CUDA(kvb_launch((moe_gemv_rows_kernel<G_>), grid, dim3(256), smem, stream, true, (bf16*)out,     \
                              (const bf16*)a, a_stride, a_row_div, pair_weight, (const bf16*)w, sorted,        \
                              tile_expert, meta, N, K));                                                       \
  } while (0)
  if (gated) KVB_MOE_GEMV_ROWS(true); else KVB_MOE_GEMV_ROWS(false);
#undef KVB_MOE_GEMV_ROWS
  KVB_CHECK_LAUNCH();
  return 0;
}

// Rows in the grouped order for batched library products: expert e owns rows [e * C, (e + 1) * C) of `out`;
// row e * C + j holds weight(p) * a[p / a_row_div] for the j-th pair p of the expert (sorted[expert_begin[e] + j]),
// zeros beyond the expert's pairs.  row_of_pair[p] is set to the row that pair p got.
template <typename T, bool VEC>
__global__ void moe_gather_kernel(T* __restrict__ out, const T* __restrict__ a, long long a_stride, int a_row_div,
                                  const float* __restrict__ pair_weight, const int* __restrict__ sorted,
                                  const int* __restrict__ expert_begin, int C, int* __restrict__ row_of_pair, int K) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_MOE_GATHER);
  const int e = blockIdx.x / C, j = blockIdx.x % C;
  const int at = expert_begin[e] + j;
  const int pair = at < expert_begin[e + 1] ? sorted[at] : -1;
  T* dst = out + (size_t)blockIdx.x * K;
  constexpr int N = VEC ? Vec16<T>::N : 1;
  if (pair < 0) {
    for (int k = threadIdx.x * N; k < K; k += blockDim.x * N) {
      if (VEC) *reinterpret_cast<uint4*>(dst + k) = make_uint4(0, 0, 0, 0);
      else dst[k] = from_float<T>(0.0f);
    }
    return;
  }
  if (threadIdx.x == 0) row_of_pair[pair] = blockIdx.x;
  const T* src = a + (size_t)(pair / a_row_div) * a_stride;
  const float scale = pair_weight != nullptr ? pair_weight[pair] : 1.0f;
  for (int k = threadIdx.x * N; k < K; k += blockDim.x * N) {
    if (VEC) {
      Vec16<T> v;
      v.load(src + k);
      if (pair_weight != nullptr) {
#pragma unroll
        for (int i = 0; i < Vec16<T>::N; ++i) v.set(i, v.get(i) * scale);
      }
      v.store(dst + k);
    } else {
      dst[k] = pair_weight != nullptr ? from_float<T>(to_float(src[k]) * scale) : src[k];
    }
  }
}

extern "C" int kvb_moe_gather(void* out, const void* a, long long a_stride, int a_row_div, const float* pair_weight,
                              const int* sorted, const int* expert_begin, int E, int C, int* row_of_pair, int K,
                              int dtype, cudaStream_t stream) {
  if (E == 0 || C == 0) return 0;
  KVB_REQUIRE(K > 0 && a_row_div > 0 && row_of_pair != nullptr, "moe_gather: empty rows");
  const int esize = dtype == KVB_F32 ? 4 : 2;
  const bool vec = ((size_t)K * esize) % 16 == 0 && ((size_t)a_stride * esize) % 16 == 0 && aligned16(out) && aligned16(a);
  const long long rows = (long long)E * C;
  KVB_REQUIRE(rows < (1ll << 31), "moe_gather: too many rows");
#define KVB_GATHER(T_, V_)                                                                                  \
  KVB_CHECK_CUDA(kvb_launch((moe_gather_kernel<T_, V_>), dim3((int)rows), dim3(128), 0, stream, true, (T_*)out, \
                            (const T_*)a, a_stride, a_row_div, pair_weight, sorted, expert_begin, C, row_of_pair, K))
  if (dtype == KVB_F32) { if (vec) KVB_GATHER(float, true); else KVB_GATHER(float, false); }
  else { if (vec) KVB_GATHER(bf16, true); else KVB_GATHER(bf16, false); }
#undef KVB_GATHER
  KVB_CHECK_LAUNCH();
  return 0;
}

template <typename T, bool VEC>
__global__ void moe_combine_kernel(T* __restrict__ out, const T* __restrict__ expert_out, int top,
                                   const int* __restrict__ row_of_pair, const float* __restrict__ pair_weight,
                                   const T* __restrict__ shared, const float* __restrict__ gate, int gate_stride,
                                   int width, long long total_vecs) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_MOE_COMBINE);
  constexpr int N = VEC ? Vec16<T>::N : 1;
  const int per_row = width / N;
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < total_vecs; v += step) {
    const long long token = v / per_row;
    const int col = (int)(v % per_row) * N;
    float acc[N];
#pragma unroll
    for (int j = 0; j < N; ++j) acc[j] = 0.0f;
    for (int slot = 0; slot < top; ++slot) {
      const long long pair = token * top + slot;
      const long long row = row_of_pair != nullptr ? row_of_pair[pair] : pair;
      if (row < 0) continue;
      const float w = pair_weight != nullptr ? pair_weight[pair] : 1.0f;
      const T* src = expert_out + (size_t)row * width + col;
      if (VEC) {
        Vec16<T> x;
        x.load(src);
#pragma unroll
        for (int j = 0; j < N; ++j) acc[j] += pair_weight != nullptr ? w * x.get(j) : x.get(j);
      } else {
        acc[0] += pair_weight != nullptr ? w * to_float(src[0]) : to_float(src[0]);
      }
    }
    if (shared != nullptr) {
      const float g = gate != nullptr ? gate[(size_t)token * gate_stride] : 1.0f;
      const T* src = shared + (size_t)token * width + col;
      if (VEC) {
        Vec16<T> x;
        x.load(src);
#pragma unroll
        for (int j = 0; j < N; ++j) acc[j] += gate != nullptr ? g * x.get(j) : x.get(j);
      } else {
        acc[0] += gate != nullptr ? g * to_float(src[0]) : to_float(src[0]);
      }
    }
    T* dst = out + (size_t)token * width + col;
    if (VEC) {
      Vec16<T> y;
#pragma unroll
      for (int j = 0; j < N; ++j) y.set(j, acc[j]);
      y.store(dst);
    } else {
      dst[0] = from_float<T>(acc[0]);
    }
  }
}

extern "C" int kvb_moe_combine(void* out, const void* expert_out, int tokens, int top, const int* row_of_pair,
                               const float* pair_weight, const void* shared, const float* gate, int gate_stride,
                               int width, int dtype, cudaStream_t stream) {
  if (tokens == 0) return 0;
  KVB_REQUIRE(width > 0 && top >= 0, "moe_combine: empty rows");
  const int esize = dtype == KVB_F32 ? 4 : 2;
  const bool vec = ((size_t)width * esize) % 16 == 0 && aligned16(out) && aligned16(expert_out) &&
                   (shared == nullptr || aligned16(shared));
  const long long total = (long long)tokens * (width / (vec ? 16 / esize : 1));
  const int threads = 256;
  const long long wanted = (total + threads - 1) / threads;
  const long long resident = (long long)(kvb_sm_count() > 0 ? kvb_sm_count() : 1) * 16;
  const int blocks = (int)(wanted < resident ? wanted : resident);
#define KVB_COMBINE(T_, V_)                                                                                   \
  KVB_CHECK_CUDA(kvb_launch((moe_combine_kernel<T_, V_>), dim3(blocks), dim3(threads), 0, stream, true, (T_*)out, \
                            (const T_*)expert_out, top, row_of_pair, pair_weight, (const T_*)shared, gate,     \
                            gate_stride, width, total))
  if (dtype == KVB_F32) { if (vec) KVB_COMBINE(float, true); else KVB_COMBINE(float, false); }
  else { if (vec) KVB_COMBINE(bf16, true); else KVB_COMBINE(bf16, false); }
#undef KVB_COMBINE
  KVB_CHECK_LAUNCH();
  return 0;
}

KVB_TRACE_TU(moe)
