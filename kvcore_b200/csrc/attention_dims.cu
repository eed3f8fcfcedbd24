// Paged attention whose key width and value width differ, general kernel.
//
// What it adds to the plain grouped-query kernel, each a parameter:
//   * DK (width of a query and of a key) and DV (width of a value and of an output row) are separate;
//   * the cache is addressed through strides (page, head, row) given for keys and for values apart, so
//     keys and values may live side by side in one cached row per token, and the values may be the
//     first DV entries of the key rows themselves (a latent cache: one vector a token serves as key
//     and as value);
//   * `maps` score maps per head: query head hq reads value head vh = hq / (group * maps) and key head
//     vh * maps + hq % maps (each map is a softmax of its own over the same values; maps = 1 is plain
//     grouped-query attention);
//   * an optional sink per query head: a logit that joins the softmax's denominator once, unscaled,
//     with no key and no value;
//   * an optional slope per query head: slope * (query position - key position) is taken off the scaled
//     score (a linear bias by distance);
//   * the output is 32-bit or of the cache's type, with token and head strides of its own.
//
// One warp owns one (token, query head) row and walks the keys from the first visible position to the
// token's own in steps of 32: each lane scores one key (a full dot product in ascending order), the warp
// keeps a running maximum and sum in 32-bit, and every lane accumulates its slice of the output.  The
// walk depends on the token's position only, so a row's bits do not depend on batching or cutting.
#include "common.cuh"

#define AD_MAX_DV 512
#define AD_WARPS 4

struct DimsParams {
  void* out; long long out_token_stride, out_head_stride; int out_f32;
  const void* q; long long q_token_stride, q_head_stride;
  const void* k; long long k_page_stride, k_head_stride, k_row_stride;
  const void* v; long long v_page_stride, v_head_stride, v_row_stride;
  const int* table; int table_stride;
  const int* positions; const int* req_index;
  const float* sink;
  const float* slopes;
  int num_rows, HQ, per_value_head, maps, DK, DV, page_size, num_pages, window;
  float scale;
  int* status;
};

template <typename T>
__global__ void __launch_bounds__(AD_WARPS * 32)
attention_dims_rows_kernel(const DimsParams p) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_ATTN_DIMS);
  extern __shared__ float q_smem[];   // [AD_WARPS][DK]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * AD_WARPS + warp;
  if (row >= p.num_rows) return;
  const int token = row / p.HQ, head = row % p.HQ;
  const int vh = head / p.per_value_head;
  const int kh = vh * p.maps + head % p.maps;
  const int pos = p.positions[token];
  const int* pages = p.table + (size_t)p.req_index[token] * p.table_stride;
  const int DK = p.DK, DV = p.DV;
  float* qv = q_smem + warp * DK;
  const T* qrow = (const T*)p.q + (size_t)token * p.q_token_stride + (size_t)head * p.q_head_stride;
  for (int d = lane; d < DK; d += 32) qv[d] = to_float(qrow[d]);
  __syncwarp();

  constexpr int SLICES = AD_MAX_DV / 32;
  float acc[SLICES];
#pragma unroll
  for (int i = 0; i < SLICES; ++i) acc[i] = 0.0f;
  // the sink starts the running maximum and counts once in the sum
  float running_max = -INFINITY, running_sum = 0.0f;
  if (p.sink != nullptr) { running_max = p.sink[head]; running_sum = 1.0f; }
  const int first = p.window > 0 ? max(0, pos - p.window + 1) : 0;
  const float slope = p.slopes != nullptr ? p.slopes[head] : 0.0f;
  const T* kbase = (const T*)p.k + (size_t)kh * p.k_head_stride;
  const T* vbase = (const T*)p.v + (size_t)vh * p.v_head_stride;

  for (int base = first; base <= pos; base += 32) {
    const int key = base + lane;
    const bool valid = key <= pos;
    float score = -INFINITY;
    int page = 0;
    if (valid) {
      page = pages[key / p.page_size];
      if (page <= 0 || page >= p.num_pages) {
        atomicOr(p.status, KVB_STATUS_BAD_PAGE);
        page = 0;
      } else {
        const T* krow = kbase + (size_t)page * p.k_page_stride + (size_t)(key % p.page_size) * p.k_row_stride;
        float dot = 0.0f;
        for (int d = 0; d < DK; ++d) dot = fmaf(to_float(krow[d]), qv[d], dot);
        score = dot * p.scale - slope * (float)(pos - key);
      }
    }
    const float new_max = fmaxf(running_max, warp_max(score));
    const float pr = (score == -INFINITY) ? 0.0f : expf(score - new_max);
    const float correction = (running_max == -INFINITY) ? 0.0f : expf(running_max - new_max);
    running_sum = running_sum * correction + warp_sum(pr);
    running_max = new_max;
#pragma unroll
    for (int i = 0; i < SLICES; ++i) acc[i] *= correction;
    const int count = min(32, pos + 1 - base);
    for (int kk = 0; kk < count; ++kk) {
      const float pk = __shfl_sync(0xffffffffu, pr, kk);
      const int pg = __shfl_sync(0xffffffffu, page, kk);
      if (pg == 0) continue;  // uniform across the warp
      const T* vrow = vbase + (size_t)pg * p.v_page_stride + (size_t)((base + kk) % p.page_size) * p.v_row_stride;
#pragma unroll
      for (int i = 0; i < SLICES; ++i) {
        const int d = lane + 32 * i;
        if (d < DV) acc[i] = fmaf(pk, to_float(vrow[d]), acc[i]);
      }
    }
  }
  const float inv = running_sum > 0.0f ? 1.0f / running_sum : 0.0f;
  const size_t off = (size_t)token * p.out_token_stride + (size_t)head * p.out_head_stride;
#pragma unroll
  for (int i = 0; i < SLICES; ++i) {
    const int d = lane + 32 * i;
    if (d < DV) {
      if (p.out_f32) ((float*)p.out)[off + d] = acc[i] * inv;
      else ((T*)p.out)[off + d] = from_float<T>(acc[i] * inv);
    }
  }
}

extern "C" int kvb_attention_dims_rows(void* out, long long out_token_stride, long long out_head_stride, int out_f32,
                                       const void* q, long long q_token_stride, long long q_head_stride,
                                       const void* k, long long k_page_stride, long long k_head_stride,
                                       long long k_row_stride, const void* v, long long v_page_stride,
                                       long long v_head_stride, long long v_row_stride, const int* table,
                                       int table_stride, const int* positions, const int* req_index,
                                       const float* sink, const float* slopes, int tokens, int HQ, int per_value_head,
                                       int maps, int DK,
                                       int DV, int page_size, int num_pages, float scale, int window, int dtype,
                                       cudaStream_t stream) {
  if (tokens == 0) return 0;
  KVB_REQUIRE(DK > 0 && DK <= 2048, "attention_dims: the key width must be in [1, 2048]");
  KVB_REQUIRE(DV > 0 && DV <= AD_MAX_DV, "attention_dims: the value width must be in [1, 512]");
  KVB_REQUIRE(HQ > 0 && maps > 0 && per_value_head > 0 && per_value_head % maps == 0 && HQ % per_value_head == 0,
              "attention_dims: query heads = value heads x group x maps");
  KVB_REQUIRE(page_size > 0 && num_pages > 1, "attention_dims: empty cache");
  int* status = kvb_status_word();
  KVB_REQUIRE(status != nullptr, "attention_dims: no status word");
  const long long rows = (long long)tokens * HQ;
  KVB_REQUIRE(rows < (1ll << 31), "attention_dims: too many rows");
  DimsParams p;
  p.out = out; p.out_token_stride = out_token_stride; p.out_head_stride = out_head_stride; p.out_f32 = out_f32;
  p.q = q; p.q_token_stride = q_token_stride; p.q_head_stride = q_head_stride;
  p.k = k; p.k_page_stride = k_page_stride; p.k_head_stride = k_head_stride; p.k_row_stride = k_row_stride;
  p.v = v; p.v_page_stride = v_page_stride; p.v_head_stride = v_head_stride; p.v_row_stride = v_row_stride;
  p.table = table; p.table_stride = table_stride; p.positions = positions; p.req_index = req_index;
  p.sink = sink; p.slopes = slopes; p.num_rows = (int)rows; p.HQ = HQ; p.per_value_head = per_value_head; p.maps = maps;
  p.DK = DK; p.DV = DV; p.page_size = page_size; p.num_pages = num_pages; p.window = window; p.scale = scale;
  p.status = status;
  const int blocks = (int)((rows + AD_WARPS - 1) / AD_WARPS);
  const size_t smem = (size_t)AD_WARPS * DK * sizeof(float);
  if (dtype == KVB_F32)
    KVB_CHECK_CUDA(kvb_launch((attention_dims_rows_kernel<float>), dim3(blocks), dim3(AD_WARPS * 32), smem, stream,
                              true, p));
  else
    KVB_CHECK_CUDA(kvb_launch((attention_dims_rows_kernel<bf16>), dim3(blocks), dim3(AD_WARPS * 32), smem, stream,
                              true, p));
  KVB_CHECK_LAUNCH();
  return 0;
}

KVB_TRACE_TU(attention_dims)
