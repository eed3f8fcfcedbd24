// Mixers that carry a matrix-valued state per request and head instead of cached keys and values.
// Everything between the projections and the output projection is 32-bit: decays, step sizes, unit
// norms, the state, the read-out and the norm behind it.
//
//   state_scan: per (request, head) a state S [D, V] (32-bit, one row of `state` per state slot) runs
//   over the request's tokens of this step in order.
//     decay per key channel (gated linear attention):
//         S <- diag(a_t) S + k_t v_t^T,                 o_t = S^T q_t
//         with a_t = sigmoid(z_t)^(1/tau) and q_t scaled by `q_scale`, both formed here from the projections;
//     delta rule with one decay per head:
//         S <- g_t S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t
//         with q_t, k_t, v_t, beta_t, g_t as `conv_prepare` left them (32-bit).
//   A thread owns one column of S (all D rows, or D / RSPLIT of them with its RSPLIT - 1 neighbours) in
//   registers; columns never exchange anything, so any cut of a request into steps gives the same bits.
//   The tokens' vectors go through shared memory a batch at a time, shared by the block's columns.
//
//   conv_prepare (delta rule): a short causal convolution over time per channel on the q, k and v
//   projections (taps [channels, C], the last tap on the current token; the C - 1 inputs in front of a
//   portion come from the request's state row), SiLU, q and k made unit vectors per head (q also times
//   `q_scale`), beta = sigmoid(b), g = exp(-exp(A_log) softplus(a + dt_bias)).  conv_state_update then
//   moves the last C - 1 inputs of every request into its state row.
//
//   gated_rms_norm: out[t, h, :] = o[t, h, :] / rms(o[t, h, :]) * weight * silu(gate[t, h, :]) * scale.
#include "common.cuh"

#define SCAN_MAX_THREADS 256

template <typename T>
__device__ __forceinline__ float load_as_float(const T* p, long long i) { return to_float(p[i]); }

struct ScanParams {
  // per token and head: q, k [D] and v [V] at base + t * token_stride + h * head_stride (head h of q and k
  // reads head h / kv_share)
  const void* q; const void* k; const void* v; const void* z;
  long long q_token, q_head, k_token, k_head, v_token, v_head, z_token, z_head;
  const float* beta; const float* gate;     // [T, H] with row stride bg_stride (delta rule)
  long long bg_stride;
  float* out;                               // [T, H, V]
  float* state;                             // [slots, state_stride]; this mixer's S at state_offset, [H, D, V]
  long long state_stride, state_offset;
  const int* query_start; const int* state_slots;
  int heads, kv_share, D, V;
  float q_scale, inv_tau;
  int batch;                                // tokens a trip through shared memory holds
};

// MODE 0: decay per key channel; MODE 1: delta rule.  DREG rows a thread; RSPLIT threads a column.
template <typename TIN, int MODE, int DREG, int RSPLIT>
__global__ void __launch_bounds__(SCAN_MAX_THREADS)
state_scan_kernel(ScanParams p) {
  KVB_KERNEL_PROLOGUE(MODE == 0 ? KVB_TAG_GLA_SCAN : KVB_TAG_DELTA_SCAN);
  extern __shared__ float smem[];
  constexpr int DP = DREG * RSPLIT;           // rows covered (>= D; rows beyond D stay zero)
  const int req = blockIdx.x, h = blockIdx.y;
  const int cols = blockDim.x / RSPLIT;       // columns this block owns
  const int col = blockIdx.z * cols + threadIdx.x / RSPLIT;
  const int part = threadIdx.x % RSPLIT;      // which DREG rows of the column
  const int row0 = part * DREG;
  const int begin = p.query_start[req], end = p.query_start[req + 1];
  const int D = p.D, V = p.V;
  const bool live = col < V;
  float* qs = smem;                           // [batch][DP]
  float* ks = qs + (size_t)p.batch * DP;
  float* as = ks + (size_t)p.batch * DP;      // MODE 0: decays [batch][DP]; MODE 1: beta, gate [batch][2]
  float* vs = as + (size_t)p.batch * (MODE == 0 ? DP : 2);   // [batch][cols]

  float* S_global = p.state + (size_t)p.state_slots[req] * p.state_stride + p.state_offset + (size_t)h * D * V;
  float S[DREG];
#pragma unroll
  for (int i = 0; i < DREG; ++i) S[i] = (live && row0 + i < D) ? S_global[(size_t)(row0 + i) * V + col] : 0.0f;

  const TIN* qg = (const TIN*)p.q; const TIN* kg = (const TIN*)p.k; const TIN* vg = (const TIN*)p.v;
  const TIN* zg = (const TIN*)p.z;
  const int kvh = h / p.kv_share;
  for (int t0 = begin; t0 < end; t0 += p.batch) {
    const int nb = min(p.batch, end - t0);
    __syncthreads();
    for (int e = threadIdx.x; e < nb * DP; e += blockDim.x) {
      const int tt = e / DP, i = e % DP;
      const long long t = t0 + tt;
      float qv = 0.0f, kv = 0.0f, av = 1.0f;
      if (i < D) {
        qv = load_as_float(qg, t * p.q_token + (long long)kvh * p.q_head + i) * p.q_scale;
        kv = load_as_float(kg, t * p.k_token + (long long)kvh * p.k_head + i);
        if (MODE == 0) {
          // sigmoid(z)^(1/tau) = exp(log_sigmoid(z) / tau); log_sigmoid(z) = min(z, 0) - log1p(exp(-|z|))
          const float zv = load_as_float(zg, t * p.z_token + (long long)h * p.z_head + i);
          av = expf((fminf(zv, 0.0f) - log1pf(expf(-fabsf(zv)))) * p.inv_tau);
        }
      }
      qs[e] = qv; ks[e] = kv;
      if (MODE == 0) as[e] = av;
    }
    for (int e = threadIdx.x; e < nb * cols; e += blockDim.x) {
      const int tt = e / cols, c = blockIdx.z * cols + e % cols;
      vs[e] = c < V ? load_as_float(vg, (long long)(t0 + tt) * p.v_token + (long long)h * p.v_head + c) : 0.0f;
    }
    if (MODE == 1)
      for (int e = threadIdx.x; e < nb; e += blockDim.x) {
        as[2 * e] = p.beta[(size_t)(t0 + e) * p.bg_stride + h];
        as[2 * e + 1] = p.gate[(size_t)(t0 + e) * p.bg_stride + h];
      }
    __syncthreads();
    for (int tt = 0; tt < nb; ++tt) {
      const float* q = qs + (size_t)tt * DP + row0;
      const float* k = ks + (size_t)tt * DP + row0;
      const float v = vs[tt * cols + threadIdx.x / RSPLIT];
      float o0 = 0.0f, o1 = 0.0f, o2 = 0.0f, o3 = 0.0f;
      if (MODE == 0) {
        const float* a = as + (size_t)tt * DP + row0;
#pragma unroll
        for (int i = 0; i < DREG; i += 4) {
          const float4 a4 = *reinterpret_cast<const float4*>(a + i);
          const float4 k4 = *reinterpret_cast<const float4*>(k + i);
          const float4 q4 = *reinterpret_cast<const float4*>(q + i);
          S[i] = fmaf(k4.x, v, a4.x * S[i]);         o0 = fmaf(S[i], q4.x, o0);
          S[i + 1] = fmaf(k4.y, v, a4.y * S[i + 1]); o1 = fmaf(S[i + 1], q4.y, o1);
          S[i + 2] = fmaf(k4.z, v, a4.z * S[i + 2]); o2 = fmaf(S[i + 2], q4.z, o2);
          S[i + 3] = fmaf(k4.w, v, a4.w * S[i + 3]); o3 = fmaf(S[i + 3], q4.w, o3);
        }
      } else {
        const float beta = as[2 * tt], g = as[2 * tt + 1];
        float d0 = 0.0f, d1 = 0.0f, d2 = 0.0f, d3 = 0.0f;
#pragma unroll
        for (int i = 0; i < DREG; i += 4) {
          const float4 k4 = *reinterpret_cast<const float4*>(k + i);
          S[i] *= g; S[i + 1] *= g; S[i + 2] *= g; S[i + 3] *= g;
          d0 = fmaf(S[i], k4.x, d0); d1 = fmaf(S[i + 1], k4.y, d1);
          d2 = fmaf(S[i + 2], k4.z, d2); d3 = fmaf(S[i + 3], k4.w, d3);
        }
        float dot = (d0 + d1) + (d2 + d3);
#pragma unroll
        for (int m = 1; m < RSPLIT; m <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, m);
        const float u = beta * (v - dot);
#pragma unroll
        for (int i = 0; i < DREG; i += 4) {
          const float4 k4 = *reinterpret_cast<const float4*>(k + i);
          const float4 q4 = *reinterpret_cast<const float4*>(q + i);
          S[i] = fmaf(k4.x, u, S[i]);         o0 = fmaf(S[i], q4.x, o0);
          S[i + 1] = fmaf(k4.y, u, S[i + 1]); o1 = fmaf(S[i + 1], q4.y, o1);
          S[i + 2] = fmaf(k4.z, u, S[i + 2]); o2 = fmaf(S[i + 2], q4.z, o2);
          S[i + 3] = fmaf(k4.w, u, S[i + 3]); o3 = fmaf(S[i + 3], q4.w, o3);
        }
      }
      float o = (o0 + o1) + (o2 + o3);
#pragma unroll
      for (int m = 1; m < RSPLIT; m <<= 1) o += __shfl_xor_sync(0xffffffffu, o, m);
      if (live && part == 0) p.out[((size_t)(t0 + tt) * p.heads + h) * V + col] = o;
    }
  }
  if (live)
#pragma unroll
    for (int i = 0; i < DREG; ++i)
      if (row0 + i < D) S_global[(size_t)(row0 + i) * V + col] = S[i];
}

template <typename TIN, int MODE>
static int launch_state_scan(const ScanParams& p_in, int num_reqs, cudaStream_t stream) {
  ScanParams p = p_in;
  const int D = p.D, V = p.V;
  int dreg = 16, rsplit = 1;
  while (dreg < D && dreg < 128) dreg *= 2;
  while (dreg * rsplit < D) rsplit *= 2;
  KVB_REQUIRE(rsplit <= 4, "state_scan: keys wider than 512 entries");
  const int dp = dreg * rsplit;
  // columns a block: all of the head's up to the thread limit, in whole warps
  int cols = ((V + 31) / 32) * 32;
  if (cols * rsplit > SCAN_MAX_THREADS) cols = SCAN_MAX_THREADS / rsplit;
  const int chunks = (V + cols - 1) / cols;
  const size_t per_token = ((size_t)dp * (MODE == 0 ? 3 : 2) + (MODE == 0 ? 0 : 2) + cols) * sizeof(float);
  int batch = (int)((40 * 1024) / per_token);
  batch = batch < 1 ? 1 : batch > 32 ? 32 : batch;
  p.batch = batch;
  const size_t smem = per_token * batch;
  const dim3 grid(num_reqs, p.heads, chunks), block(cols * rsplit);
  cudaError_t err = cudaErrorInvalidValue;
#define SCAN_CASE(DR, RS)                                                                                     \
  if (dreg == DR && rsplit == RS)                                                                             \
    err = kvb_launch((state_scan_kernel<TIN, MODE, DR, RS>), grid, block, smem, stream, true, p)
  SCAN_CASE(16, 1); SCAN_CASE(32, 1); SCAN_CASE(64, 1); SCAN_CASE(128, 1); SCAN_CASE(128, 2); SCAN_CASE(128, 4);
#undef SCAN_CASE
  KVB_CHECK_CUDA(err);
  KVB_CHECK_LAUNCH();
  return 0;
}

// Decay per key channel.  q, k, v: columns of the projected rows (row stride `row_stride`, heads side by side);
// z [T, H * D] (row stride z_stride): the decay's logits.
extern "C" int kvb_gla_scan(float* out, const void* q, const void* k, const void* v, long long row_stride,
                            const void* z, long long z_stride, float* state, long long state_stride,
                            long long state_offset, const int* query_start, const int* state_slots, int num_reqs,
                            int heads, int D, int V, float q_scale, float tau, int dtype, cudaStream_t stream) {
  if (num_reqs == 0) return 0;
  KVB_REQUIRE(heads > 0 && D > 0 && V > 0 && tau > 0.0f, "gla_scan: bad sizes");
  KVB_REQUIRE(heads <= 65535 && num_reqs > 0, "gla_scan: too many heads");
  ScanParams p = {};
  p.q = q; p.k = k; p.v = v; p.z = z;
  p.q_token = p.k_token = p.v_token = row_stride; p.q_head = p.k_head = D; p.v_head = V;
  p.z_token = z_stride; p.z_head = D;
  p.out = out; p.state = state; p.state_stride = state_stride; p.state_offset = state_offset;
  p.query_start = query_start; p.state_slots = state_slots;
  p.heads = heads; p.kv_share = 1; p.D = D; p.V = V; p.q_scale = q_scale; p.inv_tau = 1.0f / tau;
  return dtype == KVB_F32 ? launch_state_scan<float, 0>(p, num_reqs, stream) : launch_state_scan<bf16, 0>(p, num_reqs, stream);
}

// Delta rule.  prepared [T, 2 * G * D + H * V + 2 * H] 32-bit as conv_prepare leaves it: q, k (G heads), v, beta, gate.
extern "C" int kvb_delta_scan(float* out, const float* prepared, float* state, long long state_stride,
                              long long state_offset, const int* query_start, const int* state_slots, int num_reqs,
                              int heads, int kv_heads, int D, int V, cudaStream_t stream) {
  if (num_reqs == 0) return 0;
  KVB_REQUIRE(heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && D > 0 && V > 0, "delta_scan: bad sizes");
  KVB_REQUIRE(heads <= 65535, "delta_scan: too many heads");
  const long long width = 2LL * kv_heads * D + (long long)heads * V + 2LL * heads;
  ScanParams p = {};
  p.q = prepared; p.k = prepared + (size_t)kv_heads * D; p.v = prepared + 2 * (size_t)kv_heads * D;
  p.q_token = p.k_token = p.v_token = width; p.q_head = p.k_head = D; p.v_head = V;
  p.out = out; p.state = state; p.state_stride = state_stride; p.state_offset = state_offset;
  p.query_start = query_start; p.state_slots = state_slots;
  p.heads = heads; p.kv_share = heads / kv_heads; p.D = D; p.V = V; p.q_scale = 1.0f; p.inv_tau = 0.0f;
  p.beta = prepared + 2 * (size_t)kv_heads * D + (size_t)heads * V;
  p.gate = p.beta + heads;
  p.bg_stride = width;
  return launch_state_scan<float, 1>(p, num_reqs, stream);
}

// ---- short convolution, activations, unit vectors, step sizes --------------------------------------------------
#define CP_THREADS 128
#define CP_MAX_TAPS 8

template <typename T>
__global__ void __launch_bounds__(CP_THREADS)
conv_prepare_kernel(float* __restrict__ out, long long out_stride, const T* __restrict__ rows, long long row_stride,
                    const T* __restrict__ taps, int num_taps, const float* __restrict__ state, long long state_stride,
                    long long state_offset, const int* __restrict__ req_index, const int* __restrict__ query_start,
                    const int* __restrict__ state_slots, const T* __restrict__ a_log, const T* __restrict__ dt_bias,
                    int heads, int kv_heads, int D, int V, int b_col, int a_col, float q_scale, float unit_eps) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_CONV_PREPARE);
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int req = req_index[t];
  const int first = query_start[req];                 // the portion's first token row
  const int back = t - first;                         // tokens of the portion in front of this one
  const float* held = state + (size_t)state_slots[req] * state_stride + state_offset;   // [channels, taps - 1]
  const int vectors = 2 * kv_heads + heads;
  const T* row = rows + (size_t)t * row_stride;
  float* orow = out + (size_t)t * out_stride;
  for (int n = blockIdx.y * (CP_THREADS / 32) + warp; n < vectors; n += gridDim.y * (CP_THREADS / 32)) {
    const bool unit = n < 2 * kv_heads;
    const int len = unit ? D : V;
    const int c0 = unit ? n * D : 2 * kv_heads * D + (n - 2 * kv_heads) * V;     // first channel of the vector
    float ss = 0.0f;
    for (int i = lane; i < len; i += 32) {
      const int c = c0 + i;
      float acc = 0.0f;
      for (int j = 0; j < num_taps; ++j) {
        const int ago = num_taps - 1 - j;             // tap j reads the input `ago` tokens back
        float x;
        if (ago <= back) x = to_float(rows[(size_t)(t - ago) * row_stride + c]);
        else x = held[(size_t)c * (num_taps - 1) + (num_taps - 1) - (ago - back)];
        acc = fmaf(to_float(taps[(size_t)c * num_taps + j]), x, acc);
      }
      const float y = acc / (1.0f + expf(-acc));
      orow[c] = y;                                    // unit vectors are scaled below
      ss = fmaf(y, y, ss);
    }
    if (unit) {
      const float inv = (n < kv_heads ? q_scale : 1.0f) / sqrtf(warp_sum(ss) + unit_eps);
      __syncwarp();
      for (int i = lane; i < len; i += 32) orow[c0 + i] *= inv;
    }
  }
  if (blockIdx.y == 0) {
    float* extra = orow + 2 * (size_t)kv_heads * D + (size_t)heads * V;
    for (int h = threadIdx.x; h < heads; h += CP_THREADS) {
      const float b = to_float(row[b_col + h]);
      const float a = to_float(row[a_col + h]) + to_float(dt_bias[h]);
      const float softplus = fmaxf(a, 0.0f) + log1pf(expf(-fabsf(a)));
      extra[h] = 1.0f / (1.0f + expf(-b));
      extra[heads + h] = expf(-expf(to_float(a_log[h])) * softplus);
    }
  }
}

// The last taps - 1 inputs of each request, counted over what it held and what this step brought.
template <typename T>
__global__ void conv_state_update_kernel(float* __restrict__ state, long long state_stride, long long state_offset,
                                         const T* __restrict__ rows, long long row_stride, int channels, int keep,
                                         const int* __restrict__ query_start, const int* __restrict__ state_slots) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_CONV_PREPARE);
  const int req = blockIdx.x;
  const int begin = query_start[req], n = query_start[req + 1] - begin;
  float* held = state + (size_t)state_slots[req] * state_stride + state_offset;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
    float fresh[CP_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < CP_MAX_TAPS; ++j) {
      if (j < keep) {
        const int ago = keep - 1 - j;                 // new entry j is the input `ago` tokens before the portion's end
        fresh[j] = ago < n ? to_float(rows[(size_t)(begin + n - 1 - ago) * row_stride + c])
                           : held[(size_t)c * keep + (j + n)];
      }
    }
#pragma unroll
    for (int j = 0; j < CP_MAX_TAPS; ++j)
      if (j < keep) held[(size_t)c * keep + j] = fresh[j];
  }
}

extern "C" int kvb_conv_prepare(float* out, const void* rows, long long row_stride, const void* taps, int num_taps,
                                float* state, long long state_stride, long long state_offset, const int* req_index,
                                const int* query_start, const int* state_slots, const void* a_log, const void* dt_bias,
                                int tokens, int num_reqs, int heads, int kv_heads, int D, int V, int b_col, int a_col,
                                float q_scale, float unit_eps, int dtype, cudaStream_t stream) {
  if (tokens == 0) return 0;
  KVB_REQUIRE(num_taps >= 1 && num_taps <= CP_MAX_TAPS + 1, "conv_prepare: 1 to 9 taps");
  KVB_REQUIRE(heads > 0 && kv_heads > 0 && D > 0 && V > 0, "conv_prepare: bad sizes");
  const int vectors = 2 * kv_heads + heads;
  const long long out_stride = 2LL * kv_heads * D + (long long)heads * V + 2LL * heads;
  int groups = (vectors + CP_THREADS / 32 - 1) / (CP_THREADS / 32);
  if (tokens >= 512 || groups > 65535) groups = 1;     // many tokens: a block a token walks its vectors
  const int channels = 2 * kv_heads * D + heads * V;
  const int update_blocks = (channels + 255) / 256 > 65535 ? 65535 : (channels + 255) / 256;
  if (dtype == KVB_F32) {
    KVB_CHECK_CUDA(kvb_launch((conv_prepare_kernel<float>), dim3(tokens, groups), dim3(CP_THREADS), 0, stream, true,
        out, out_stride, (const float*)rows, row_stride, (const float*)taps, num_taps, (const float*)state, state_stride,
        state_offset, req_index, query_start, state_slots, (const float*)a_log, (const float*)dt_bias, heads, kv_heads,
        D, V, b_col, a_col, q_scale, unit_eps));
    if (num_taps > 1)
      KVB_CHECK_CUDA(kvb_launch((conv_state_update_kernel<float>), dim3(num_reqs, update_blocks), dim3(256), 0, stream,
          true, state, state_stride, state_offset, (const float*)rows, row_stride, channels, num_taps - 1, query_start,
          state_slots));
  } else {
    KVB_CHECK_CUDA(kvb_launch((conv_prepare_kernel<bf16>), dim3(tokens, groups), dim3(CP_THREADS), 0, stream, true,
        out, out_stride, (const bf16*)rows, row_stride, (const bf16*)taps, num_taps, (const float*)state, state_stride,
        state_offset, req_index, query_start, state_slots, (const bf16*)a_log, (const bf16*)dt_bias, heads, kv_heads,
        D, V, b_col, a_col, q_scale, unit_eps));
    if (num_taps > 1)
      KVB_CHECK_CUDA(kvb_launch((conv_state_update_kernel<bf16>), dim3(num_reqs, update_blocks), dim3(256), 0, stream,
          true, state, state_stride, state_offset, (const bf16*)rows, row_stride, channels, num_taps - 1, query_start,
          state_slots));
  }
  KVB_CHECK_LAUNCH();
  return 0;
}

// ---- the norm and the gate behind the read-out -------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(CP_THREADS)
gated_rms_norm_kernel(T* __restrict__ out, long long out_stride, const float* __restrict__ o,
                      const T* __restrict__ gate, long long gate_stride, const T* __restrict__ weight, long long vectors,
                      int heads, int V, float eps, float scale) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_GATED_NORM);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (long long n = (long long)blockIdx.x * (CP_THREADS / 32) + warp; n < vectors;
       n += (long long)gridDim.x * (CP_THREADS / 32)) {
    const long long t = n / heads;
    const int h = (int)(n % heads);
    const float* src = o + n * V;
    const T* g = gate + t * gate_stride + (long long)h * V;
    T* dst = out + t * out_stride + (long long)h * V;
    float ss = 0.0f;
    for (int i = lane; i < V; i += 32) { const float v = src[i]; ss = fmaf(v, v, ss); }
    const float inv = scale / sqrtf(warp_sum(ss) / (float)V + eps);
    for (int i = lane; i < V; i += 32) {
      const float gv = to_float(g[i]);
      dst[i] = from_float<T>(src[i] * inv * to_float(weight[i]) * (gv / (1.0f + expf(-gv))));
    }
  }
}

extern "C" int kvb_gated_rms_norm(void* out, long long out_stride, const float* o, const void* gate,
                                  long long gate_stride, const void* weight, int tokens, int heads, int V, float eps,
                                  float scale, int dtype, cudaStream_t stream) {
  const long long vectors = (long long)tokens * heads;
  if (vectors == 0) return 0;
  KVB_REQUIRE(V > 0, "gated_rms_norm: bad width");
  const long long wanted = (vectors + CP_THREADS / 32 - 1) / (CP_THREADS / 32);
  const long long resident = (long long)(kvb_sm_count() > 0 ? kvb_sm_count() : 1) * 16;
  const int blocks = (int)(wanted < resident ? wanted : resident);
  if (dtype == KVB_F32)
    KVB_CHECK_CUDA(kvb_launch((gated_rms_norm_kernel<float>), dim3(blocks), dim3(CP_THREADS), 0, stream, true,
        (float*)out, out_stride, o, (const float*)gate, gate_stride, (const float*)weight, vectors, heads, V, eps, scale));
  else
    KVB_CHECK_CUDA(kvb_launch((gated_rms_norm_kernel<bf16>), dim3(blocks), dim3(CP_THREADS), 0, stream, true,
        (bf16*)out, out_stride, o, (const bf16*)gate, gate_stride, (const bf16*)weight, vectors, heads, V, eps, scale));
  KVB_CHECK_LAUNCH();
  return 0;
}

KVB_TRACE_TU(recurrence)
