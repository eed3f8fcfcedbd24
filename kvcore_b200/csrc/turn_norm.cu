// Between the projections and the attention of a mixer whose q and k are turned in neighbouring pairs and
// then divided by their root mean square, whose key and value widths differ, and whose heads are gated.
//
//   turn_norm_kv_write: q [H, D] and k [G, D] of a token's projected row.  The first `rot` entries of every
//   head turn by the token's position: entries 2i and 2i+1 form a pair (u, v) -> (u cos a - v sin a,
//   v cos a + u sin a) with a = position * inv_freq[i]; the rest pass unchanged.  After the turn each head is
//   divided by sqrt(mean(x^2) + eps) (`norm`; a weight [D] per side multiplies it when given).  q goes back in
//   place; k and the values [G, V] go side by side into the token's cached row [G * D | G * V].  Positions,
//   angles, sums and scaling are 32-bit; one rounding at the store.
//
//   head_gate: out[t, h, :] = o[t, h, :] * sigmoid(gate[t, h]) * scale, o 32-bit, one gate per head (no gate:
//   the scale alone).
//
//   embed_scaled: the 32-bit stream's first value, table[id] * scale.
//
//   Two optional steps of turn_norm_kv_write: a query temperature, q times
//   1 + coef * ln(floor((position + 1) / every) + 1); and value mixing, the cached values become
//   (1 - lambda) v + lambda v_first with v_first another layer's values of the same token (rows of a tensor of
//   their own) and lambda one 32-bit number.
//
//   gelu_mul: out[t, j] = gelu_tanh(z[t, j]) * rows[t, column + j].
#include "common.cuh"

#define TN_THREADS 128

template <typename T>
__global__ void __launch_bounds__(TN_THREADS)
turn_norm_kv_write_kernel(T* __restrict__ rows, long long row_stride, const float* __restrict__ inv_freq, int rot,
                          const T* __restrict__ q_weight, const T* __restrict__ k_weight, int norm, float eps,
                          const int* __restrict__ positions, const int* __restrict__ req_index,
                          const int* __restrict__ table, int table_stride, T* __restrict__ cache, int page_size,
                          int num_pages, int write, int q_heads, int k_heads, int D, int v_width, int per_block,
                          float temp_coef, int temp_every, const T* __restrict__ mix_values, long long mix_stride,
                          const float* __restrict__ mix_weight, int* status) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_TURN_NORM);
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  T* row = rows + (size_t)t * row_stride;
  const int pos = positions[t];
  const float fpos = (float)pos;
  // the query temperature of this position (1 without one)
  const float temperature = temp_every > 0 ? 1.0f + temp_coef * logf((float)((pos + 1) / temp_every + 1)) : 1.0f;
  T* dst = nullptr;
  if (write) {
    const int page = table[(size_t)req_index[t] * table_stride + pos / page_size];
    if (page <= 0 || page >= num_pages) {
      if (threadIdx.x == 0 && blockIdx.y == 0) atomicOr(status, KVB_STATUS_BAD_PAGE);
    } else {
      dst = cache + ((size_t)page * page_size + pos % page_size) * ((size_t)k_heads * D + v_width);
    }
  }
  const int vectors = q_heads + (write ? k_heads : 0);
  const int pairs = (D + 1) / 2;
  const int group_end = min(vectors, (int)(blockIdx.y + 1) * per_block);
  for (int n = blockIdx.y * per_block + warp; n < group_end; n += TN_THREADS / 32) {
    const bool is_q = n < q_heads;
    const T* vec = row + (size_t)n * D;
    const T* w = is_q ? q_weight : k_weight;
    T* o = is_q ? row + (size_t)n * D : (dst == nullptr ? nullptr : dst + (size_t)(n - q_heads) * D);
    // two passes over the head's pairs: the turn is computed again in the second (cheaper than keeping a head of
    // any size in registers; the angle's sine and cosine are the cost, and a lane has few pairs)
    float ss = 0.0f;
    for (int pair = lane; pair < pairs; pair += 32) {
      const int e = 2 * pair;
      float u = to_float(vec[e]);
      float v = e + 1 < D ? to_float(vec[e + 1]) : 0.0f;
      if (e + 1 < rot) {
        float s, c;
        sincosf(fpos * inv_freq[pair], &s, &c);
        const float tu = u * c - v * s, tv = v * c + u * s;
        u = tu; v = tv;
      }
      ss = fmaf(u, u, ss);
      ss = fmaf(v, v, ss);
    }
    float inv = norm ? 1.0f / sqrtf(warp_sum(ss) / (float)D + eps) : 1.0f;
    if (is_q) inv *= temperature;
    if (o == nullptr) continue;
    for (int pair = lane; pair < pairs; pair += 32) {
      const int e = 2 * pair;
      float u = to_float(vec[e]);
      float v = e + 1 < D ? to_float(vec[e + 1]) : 0.0f;
      if (e + 1 < rot) {
        float s, c;
        sincosf(fpos * inv_freq[pair], &s, &c);
        const float tu = u * c - v * s, tv = v * c + u * s;
        u = tu; v = tv;
      }
      u *= inv; v *= inv;
      if (w != nullptr) { u *= to_float(w[e]); if (e + 1 < D) v *= to_float(w[e + 1]); }
      o[e] = from_float<T>(u);
      if (e + 1 < D) o[e + 1] = from_float<T>(v);
    }
  }
  if (dst != nullptr && blockIdx.y == 0) {
    const T* v = row + (size_t)(q_heads + k_heads) * D;
    T* out = dst + (size_t)k_heads * D;
    if (mix_values != nullptr) {
      const float lam = mix_weight[0];
      const T* first = mix_values + (size_t)t * mix_stride;
      for (int i = threadIdx.x; i < v_width; i += TN_THREADS)
        out[i] = from_float<T>((1.0f - lam) * to_float(v[i]) + lam * to_float(first[i]));
    } else {
      for (int i = threadIdx.x; i < v_width; i += TN_THREADS) out[i] = v[i];
    }
  }
}

extern "C" int kvb_turn_norm_kv_write(void* rows, long long row_stride, const float* inv_freq, int rot,
                                      const void* q_weight, const void* k_weight, int norm, float eps,
                                      const int* positions, const int* req_index, const int* table, int table_stride,
                                      void* cache, int page_size, int num_pages, int write, int tokens, int q_heads,
                                      int k_heads, int D, int v_width, float temp_coef, int temp_every,
                                      const void* mix_values, long long mix_stride, const float* mix_weight,
                                      int dtype, cudaStream_t stream) {
  if (tokens == 0) return 0;
  KVB_REQUIRE(q_heads > 0 && k_heads > 0 && D > 0 && v_width > 0, "turn_norm_kv_write: bad sizes");
  KVB_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= D, "turn_norm_kv_write: the turned entries are an even number within the head");
  KVB_REQUIRE(temp_every >= 0 && (mix_values == nullptr || mix_weight != nullptr),
              "turn_norm_kv_write: the temperature's period is not negative, and mixed values need their weight");
  int* status = kvb_status_word();
  KVB_REQUIRE(status != nullptr, "turn_norm_kv_write: no status word");
  const int vectors = q_heads + (write ? k_heads : 0);
  const int per_block = tokens >= 512 ? ((vectors + 3) / 4) * 4 : TN_THREADS / 32;
  const int groups = (vectors + per_block - 1) / per_block;
  KVB_REQUIRE(groups <= 65535, "turn_norm_kv_write: too many heads a token");
  if (dtype == KVB_F32)
    KVB_CHECK_CUDA(kvb_launch((turn_norm_kv_write_kernel<float>), dim3(tokens, groups), dim3(TN_THREADS), 0, stream, true,
        (float*)rows, row_stride, inv_freq, rot, (const float*)q_weight, (const float*)k_weight, norm, eps, positions,
        req_index, table, table_stride, (float*)cache, page_size, num_pages, write, q_heads, k_heads, D, v_width,
        per_block, temp_coef, temp_every, (const float*)mix_values, mix_stride, mix_weight, status));
  else
    KVB_CHECK_CUDA(kvb_launch((turn_norm_kv_write_kernel<bf16>), dim3(tokens, groups), dim3(TN_THREADS), 0, stream, true,
        (bf16*)rows, row_stride, inv_freq, rot, (const bf16*)q_weight, (const bf16*)k_weight, norm, eps, positions,
        req_index, table, table_stride, (bf16*)cache, page_size, num_pages, write, q_heads, k_heads, D, v_width,
        per_block, temp_coef, temp_every, (const bf16*)mix_values, mix_stride, mix_weight, status));
  KVB_CHECK_LAUNCH();
  return 0;
}

template <typename T>
__global__ void head_gate_kernel(T* __restrict__ out, long long out_stride, const float* __restrict__ o,
                                 const T* __restrict__ gate, long long gate_stride, long long count, int heads, int V,
                                 float scale) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_HEAD_GATE);
  const long long step = (long long)gridDim.x * blockDim.x;
  const int per_token = heads * V;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count; i += step) {
    const long long t = i / per_token;
    const int c = (int)(i % per_token), h = c / V;
    float factor = scale;
    if (gate != nullptr) factor = scale / (1.0f + expf(-to_float(gate[t * gate_stride + h])));
    out[t * out_stride + c] = from_float<T>(o[i] * factor);
  }
}

extern "C" int kvb_head_gate(void* out, long long out_stride, const float* o, const void* gate, long long gate_stride,
                             int tokens, int heads, int V, float scale, int dtype, cudaStream_t stream) {
  const long long count = (long long)tokens * heads * V;
  if (count == 0) return 0;
  const int threads = 256;
  const long long wanted = (count + threads - 1) / threads;
  const long long resident = (long long)(kvb_sm_count() > 0 ? kvb_sm_count() : 1) * 16;
  const int blocks = (int)(wanted < resident ? wanted : resident);
  if (dtype == KVB_F32)
    KVB_CHECK_CUDA(kvb_launch((head_gate_kernel<float>), dim3(blocks), dim3(threads), 0, stream, true, (float*)out,
        out_stride, o, (const float*)gate, gate_stride, count, heads, V, scale));
  else
    KVB_CHECK_CUDA(kvb_launch((head_gate_kernel<bf16>), dim3(blocks), dim3(threads), 0, stream, true, (bf16*)out,
        out_stride, o, (const bf16*)gate, gate_stride, count, heads, V, scale));
  KVB_CHECK_LAUNCH();
  return 0;
}

template <typename T>
__global__ void embed_scaled_kernel(float* __restrict__ out, const T* __restrict__ table, const int* __restrict__ ids,
                                    int vocab, int width, float scale, int* status) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_EMBED_SCALED);
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) atomicOr(status, KVB_STATUS_BAD_TOKEN);
    id = 0;
  }
  const T* src = table + (size_t)id * width;
  float* dst = out + (size_t)t * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = to_float(src[i]) * scale;
}

extern "C" int kvb_embed_scaled(float* out, const void* table, const int* ids, int tokens, int vocab, int width,
                                float scale, int dtype, cudaStream_t stream) {
  if (tokens == 0) return 0;
  KVB_REQUIRE(vocab > 0 && width > 0, "embed_scaled: bad sizes");
  int* status = kvb_status_word();
  KVB_REQUIRE(status != nullptr, "embed_scaled: no status word");
  const int threads = width >= 1024 ? 256 : 128;
  if (dtype == KVB_F32)
    KVB_CHECK_CUDA(kvb_launch((embed_scaled_kernel<float>), dim3(tokens), dim3(threads), 0, stream, true, out,
        (const float*)table, ids, vocab, width, scale, status));
  else
    KVB_CHECK_CUDA(kvb_launch((embed_scaled_kernel<bf16>), dim3(tokens), dim3(threads), 0, stream, true, out,
        (const bf16*)table, ids, vocab, width, scale, status));
  KVB_CHECK_LAUNCH();
  return 0;
}

// out[t, j] = gelu_tanh(z[t, j]) * rows[t, column + j], gelu_tanh(z) = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))),
// in 32-bit with one rounding at the store: the gate of an input that every token brings with it.
template <typename T>
__global__ void gelu_mul_kernel(T* __restrict__ out, const T* __restrict__ z, const T* __restrict__ rows,
                                long long rows_stride, int column, long long count, int dim) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_GELU_MUL);
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count; i += step) {
    const long long t = i / dim;
    const int j = (int)(i - t * dim);
    const float x = to_float(z[i]);
    const float inner = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    const float gelu = 0.5f * x * (1.0f + tanhf(inner));
    out[i] = from_float<T>(gelu * to_float(rows[t * rows_stride + column + j]));
  }
}

extern "C" int kvb_gelu_mul(void* out, const void* z, const void* rows, long long rows_stride, int column, int tokens,
                            int dim, int dtype, cudaStream_t stream) {
  const long long count = (long long)tokens * dim;
  if (count == 0) return 0;
  KVB_REQUIRE(column >= 0 && dim > 0, "gelu_mul: bad sizes");
  const int threads = 256;
  const long long wanted = (count + threads - 1) / threads;
  const long long resident = (long long)(kvb_sm_count() > 0 ? kvb_sm_count() : 1) * 16;
  const int blocks = (int)(wanted < resident ? wanted : resident);
  if (dtype == KVB_F32)
    KVB_CHECK_CUDA(kvb_launch((gelu_mul_kernel<float>), dim3(blocks), dim3(threads), 0, stream, true, (float*)out,
        (const float*)z, (const float*)rows, rows_stride, column, count, dim));
  else
    KVB_CHECK_CUDA(kvb_launch((gelu_mul_kernel<bf16>), dim3(blocks), dim3(threads), 0, stream, true, (bf16*)out,
        (const bf16*)z, (const bf16*)rows, rows_stride, column, count, dim));
  KVB_CHECK_LAUNCH();
  return 0;
}

KVB_TRACE_TU(turn_norm)
