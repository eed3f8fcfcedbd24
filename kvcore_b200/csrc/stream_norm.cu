// RMS norms around the sub-layers of a block that keeps a 32-bit residual stream and norms each
// sub-layer on both sides ("sandwich"): x <- x + norm_after(sublayer(norm_before(x))).
//
//   rms_norm_shift: y = x * rsqrt(mean(x^2) + eps) * w for every row of the stream (32-bit or 16-bit in,
//   the activation type out), optionally followed by a token shift: y_t <- y_t + (y_{t-1} - y_t) * s,
//   element by element, with y_{t-1} the unshifted normed row of the request's token in front.  Inside a
//   step that row is normed again by the block of token t (same reduction, same bits); for the first
//   token of a request's portion it comes from the request's state row, which holds the normed row of
//   the last token of the portion in front (zeros for a new request).  The block of a portion's first
//   token also leaves the portion's last normed row in the state: it is the only block that reads the
//   row, so no other block's write can come between.  Everything is 32-bit up to the store.
//
//   stream_add_norm: X = x + a * rsqrt(mean(a^2) + eps) * w in 32-bit (a: a sub-layer's output), written
//   to `out`; optionally also the depth-weighted average avg = sum_{j<count} c[j] * stack[j] + c[count] * X
//   over the results of all layers in front (stack[j] = [rows, width], 32-bit), summed in ascending j.
//
// One block per row; the reduction tree depends on the width only, so a row's result does not depend
// on the batch or on how a request was cut into steps.
#include "common.cuh"

#define SN_THREADS 256

// Sums of three values over the block at once; all threads get all three.
__device__ __forceinline__ void block_sum3(float& a, float& b, float& c, float (*scratch)[32]) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  a = warp_sum(a); b = warp_sum(b); c = warp_sum(c);
  __syncthreads();
  if (lane == 0) { scratch[0][warp] = a; scratch[1][warp] = b; scratch[2][warp] = c; }
  __syncthreads();
  a = warp_sum(lane < nwarps ? scratch[0][lane] : 0.0f);
  b = warp_sum(lane < nwarps ? scratch[1][lane] : 0.0f);
  c = warp_sum(lane < nwarps ? scratch[2][lane] : 0.0f);
}

// Rows of up to SN_THREADS * SN_KEEP entries are held in registers between the pass that sums the
// squares and the pass that scales and stores: every load of a pass is in flight at once (a small batch is
// bound by the latency of its loads, not by bytes).  Wider rows are read again.
#define SN_KEEP 16

// Four neighbouring entries, loaded and stored as one access.
template <typename T>
struct __align__(4 * sizeof(T)) Quad4 { T v[4]; };

// KEPT: 0 rows of any width, read twice; 1 rows kept in registers; 2 the same with four neighbouring entries a
// thread and access (widths that are multiples of 4, every row on a boundary of four entries).
template <typename IN, typename OUT, typename W, int KEPT>
__global__ void __launch_bounds__(SN_THREADS)
rms_norm_shift_kernel(OUT* __restrict__ out, const IN* __restrict__ x, const W* __restrict__ weight,
                      const W* __restrict__ shift, float* __restrict__ state, const int* __restrict__ req_index,
                      const int* __restrict__ query_start, const int* __restrict__ state_slots, int width,
                      float eps) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_RMS_SHIFT);
  __shared__ float scratch[3][32];
  const int t = blockIdx.x;
  const IN* row = x + (size_t)t * width;
  OUT* orow = out + (size_t)t * width;
  const bool shifting = shift != nullptr;
  bool first = false;
  int last = t;
  float* srow = nullptr;
  if (shifting) {
    const int r = req_index[t];
    first = query_start[r] == t;
    last = query_start[r + 1] - 1;
    srow = state + (size_t)state_slots[r] * width;
  }
  // the row in front inside the step, and (for a portion's first token) the portion's last row
  const IN* prow = shifting && !first ? row - width : nullptr;
  const IN* lrow = first && last != t ? x + (size_t)last * width : nullptr;
  float ss = 0.0f, sp = 0.0f, sl = 0.0f;
  if (KEPT == 2) {
    constexpr int PASSES = SN_KEEP / 4;
    float mine[PASSES][4], before[PASSES][4], final_row[PASSES][4], w[PASSES][4], mix[PASSES][4];
#pragma unroll
    for (int s = 0; s < PASSES; ++s) {
      const int i = (threadIdx.x + s * SN_THREADS) * 4;
      const bool in = i < width;
#pragma unroll
      for (int j = 0; j < 4; ++j) mine[s][j] = w[s][j] = before[s][j] = final_row[s][j] = mix[s][j] = 0.0f;
      if (in) {
        const Quad4<IN> qx = *reinterpret_cast<const Quad4<IN>*>(row + i);
        const Quad4<W> qw = *reinterpret_cast<const Quad4<W>*>(weight + i);
#pragma unroll
        for (int j = 0; j < 4; ++j) { mine[s][j] = to_float(qx.v[j]); w[s][j] = to_float(qw.v[j]); }
        if (shifting) {
          const Quad4<W> qm = *reinterpret_cast<const Quad4<W>*>(shift + i);
#pragma unroll
          for (int j = 0; j < 4; ++j) mix[s][j] = to_float(qm.v[j]);
          if (first) {
            const Quad4<float> qs = *reinterpret_cast<const Quad4<float>*>(srow + i);
#pragma unroll
            for (int j = 0; j < 4; ++j) before[s][j] = qs.v[j];
          } else {
            const Quad4<IN> qp = *reinterpret_cast<const Quad4<IN>*>(prow + i);
#pragma unroll
            for (int j = 0; j < 4; ++j) before[s][j] = to_float(qp.v[j]);
          }
          if (lrow != nullptr) {
            const Quad4<IN> ql = *reinterpret_cast<const Quad4<IN>*>(lrow + i);
#pragma unroll
            for (int j = 0; j < 4; ++j) final_row[s][j] = to_float(ql.v[j]);
          }
        }
      }
    }
#pragma unroll
    for (int s = 0; s < PASSES; ++s)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        ss = fmaf(mine[s][j], mine[s][j], ss);
        if (prow != nullptr) sp = fmaf(before[s][j], before[s][j], sp);
        sl = fmaf(final_row[s][j], final_row[s][j], sl);
      }
    block_sum3(ss, sp, sl, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    const float inv_p = 1.0f / sqrtf(sp / (float)width + eps);
    const float inv_l = 1.0f / sqrtf(sl / (float)width + eps);
#pragma unroll
    for (int s = 0; s < PASSES; ++s) {
      const int i = (threadIdx.x + s * SN_THREADS) * 4;
      if (i >= width) continue;
      Quad4<OUT> result;
      Quad4<float> kept_row;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float y = mine[s][j] * inv * w[s][j];
        float r = y;
        if (shifting) {
          const float in_front = first ? before[s][j] : before[s][j] * inv_p * w[s][j];
          r = y + (in_front - y) * mix[s][j];
          kept_row.v[j] = lrow != nullptr ? final_row[s][j] * inv_l * w[s][j] : y;
        }
        result.v[j] = from_float<OUT>(r);
      }
      if (first) *reinterpret_cast<Quad4<float>*>(srow + i) = kept_row;
      *reinterpret_cast<Quad4<OUT>*>(orow + i) = result;
    }
    return;
  }
  if (KEPT == 1) {
    float mine[SN_KEEP], before[SN_KEEP], final_row[SN_KEEP], w[SN_KEEP], mix[SN_KEEP];
#pragma unroll
    for (int s = 0; s < SN_KEEP; ++s) {
      const int i = threadIdx.x + s * SN_THREADS;
      const bool in = i < width;
      mine[s] = in ? to_float(row[i]) : 0.0f;
      w[s] = in ? to_float(weight[i]) : 0.0f;
      before[s] = 0.0f; final_row[s] = 0.0f; mix[s] = 0.0f;
      if (shifting && in) {
        mix[s] = to_float(shift[i]);
        before[s] = first ? srow[i] : to_float(prow[i]);
        if (lrow != nullptr) final_row[s] = to_float(lrow[i]);
      }
    }
#pragma unroll
    for (int s = 0; s < SN_KEEP; ++s) {
      ss = fmaf(mine[s], mine[s], ss);
      if (prow != nullptr) sp = fmaf(before[s], before[s], sp);
      sl = fmaf(final_row[s], final_row[s], sl);
    }
    block_sum3(ss, sp, sl, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    const float inv_p = 1.0f / sqrtf(sp / (float)width + eps);
    const float inv_l = 1.0f / sqrtf(sl / (float)width + eps);
#pragma unroll
    for (int s = 0; s < SN_KEEP; ++s) {
      const int i = threadIdx.x + s * SN_THREADS;
      if (i >= width) continue;
      const float y = mine[s] * inv * w[s];
      float result = y;
      if (shifting) {
        const float in_front = first ? before[s] : before[s] * inv_p * w[s];
        result = y + (in_front - y) * mix[s];
        if (first) srow[i] = lrow != nullptr ? final_row[s] * inv_l * w[s] : y;
      }
      orow[i] = from_float<OUT>(result);
    }
    return;
  }
  for (int i = threadIdx.x; i < width; i += SN_THREADS) {
    const float v = to_float(row[i]);
    ss = fmaf(v, v, ss);
    if (prow != nullptr) { const float u = to_float(prow[i]); sp = fmaf(u, u, sp); }
    if (lrow != nullptr) { const float u = to_float(lrow[i]); sl = fmaf(u, u, sl); }
  }
  block_sum3(ss, sp, sl, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)width + eps);
  const float inv_p = 1.0f / sqrtf(sp / (float)width + eps);
  const float inv_l = 1.0f / sqrtf(sl / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += SN_THREADS) {
    const float w = to_float(weight[i]);
    const float y = to_float(row[i]) * inv * w;
    float result = y;
    if (shifting) {
      const float before = first ? srow[i] : to_float(prow[i]) * inv_p * w;
      result = y + (before - y) * to_float(shift[i]);
      if (first) srow[i] = lrow != nullptr ? to_float(lrow[i]) * inv_l * w : y;
    }
    orow[i] = from_float<OUT>(result);
  }
}

template <typename IN, typename OUT, typename W>
static cudaError_t launch_rms_norm_shift(void* out, const void* x, const void* w, const void* shift, float* state,
                                         const int* req_index, const int* query_start, const int* slots, int rows,
                                         int width, float eps, cudaStream_t stream) {
  auto on4 = [](const void* p, size_t size) { return (reinterpret_cast<uintptr_t>(p) % (4 * size)) == 0; };
  if (width <= SN_THREADS * SN_KEEP && width % 4 == 0 && on4(out, sizeof(OUT)) && on4(x, sizeof(IN)) &&
      on4(w, sizeof(W)) && (shift == nullptr || (on4(shift, sizeof(W)) && aligned16(state))))
    return kvb_launch((rms_norm_shift_kernel<IN, OUT, W, 2>), dim3(rows), dim3(SN_THREADS), 0, stream, true,
                      (OUT*)out, (const IN*)x, (const W*)w, (const W*)shift, state, req_index, query_start, slots,
                      width, eps);
  if (width <= SN_THREADS * SN_KEEP)
    return kvb_launch((rms_norm_shift_kernel<IN, OUT, W, 1>), dim3(rows), dim3(SN_THREADS), 0, stream, true,
                      (OUT*)out, (const IN*)x, (const W*)w, (const W*)shift, state, req_index, query_start, slots,
                      width, eps);
  return kvb_launch((rms_norm_shift_kernel<IN, OUT, W, 0>), dim3(rows), dim3(SN_THREADS), 0, stream, true,
                    (OUT*)out, (const IN*)x, (const W*)w, (const W*)shift, state, req_index, query_start, slots,
                    width, eps);
}

extern "C" int kvb_rms_norm_shift(void* out, const void* x, const void* weight, const void* shift, float* state,
                                  const int* req_index, const int* query_start, const int* state_slots, int rows,
                                  int width, float eps, int in_dtype, int out_dtype, int weight_dtype,
                                  cudaStream_t stream) {
  if (rows == 0) return 0;
  KVB_REQUIRE(width > 0, "rms_norm_shift: width must be positive");
  KVB_REQUIRE(shift == nullptr || (state != nullptr && req_index != nullptr && query_start != nullptr &&
                                   state_slots != nullptr),
              "rms_norm_shift: a token shift needs the state rows and the batch's request arrays");
  const int code = (in_dtype == KVB_BF16 ? 4 : 0) | (out_dtype == KVB_BF16 ? 2 : 0) | (weight_dtype == KVB_BF16 ? 1 : 0);
  cudaError_t err;
#define KVB_SN_CASE(n, IN, OUT, W)                                                                            \
  case n: err = launch_rms_norm_shift<IN, OUT, W>(out, x, weight, shift, state, req_index, query_start,       \
                                                  state_slots, rows, width, eps, stream); break;
  switch (code) {
    KVB_SN_CASE(0, float, float, float)
    KVB_SN_CASE(1, float, float, bf16)
    KVB_SN_CASE(2, float, bf16, float)
    KVB_SN_CASE(3, float, bf16, bf16)
    KVB_SN_CASE(4, bf16, float, float)
    KVB_SN_CASE(5, bf16, float, bf16)
    KVB_SN_CASE(6, bf16, bf16, float)
    default: err = launch_rms_norm_shift<bf16, bf16, bf16>(out, x, weight, shift, state, req_index, query_start,
                                                           state_slots, rows, width, eps, stream); break;
  }
#undef KVB_SN_CASE
  KVB_CHECK_CUDA(err);
  KVB_CHECK_LAUNCH();
  return 0;
}

// KEPT: 0 rows of any width, read twice; 1 rows up to SN_THREADS * SN_KEEP entries kept in registers; 2 the same
// with four neighbouring entries a thread and access (widths that are multiples of 4, rows on 16-byte boundaries).
template <typename T, typename W, int KEPT>
__global__ void __launch_bounds__(SN_THREADS)
stream_add_norm_kernel(float* out, const float* x, const T* __restrict__ a,
                       const W* __restrict__ weight, int width, float eps, float* __restrict__ avg,
                       const float* __restrict__ stack, long long stack_stride, const W* __restrict__ coeffs,
                       int count, T* __restrict__ rounded) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_ADD_NORM);
  __shared__ float scratch[32];
  const size_t base = (size_t)blockIdx.x * width;
  const T* arow = a + base;
  float ss = 0.0f;
  if (KEPT == 2) {
    constexpr int PASSES = SN_KEEP / 4;
    float mine[PASSES][4], stream[PASSES][4], w[PASSES][4];
#pragma unroll
    for (int s = 0; s < PASSES; ++s) {
      const int i = (threadIdx.x + s * SN_THREADS) * 4;
      if (i < width) {
        const Quad4<T> qa = *reinterpret_cast<const Quad4<T>*>(arow + i);
        const Quad4<float> qx = *reinterpret_cast<const Quad4<float>*>(x + base + i);
        const Quad4<W> qw = *reinterpret_cast<const Quad4<W>*>(weight + i);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          mine[s][j] = to_float(qa.v[j]); stream[s][j] = qx.v[j]; w[s][j] = to_float(qw.v[j]);
          ss = fmaf(mine[s][j], mine[s][j], ss);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) mine[s][j] = stream[s][j] = w[s][j] = 0.0f;
      }
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)width + eps);
#pragma unroll
    for (int s = 0; s < PASSES; ++s)
#pragma unroll
      for (int j = 0; j < 4; ++j) stream[s][j] = stream[s][j] + mine[s][j] * inv * w[s][j];
    if (avg != nullptr) {
#pragma unroll
      for (int s = 0; s < PASSES; ++s)
#pragma unroll
        for (int j = 0; j < 4; ++j) mine[s][j] = 0.0f;
      for (int n = 0; n < count; ++n) {
        const float c = to_float(coeffs[n]);
        const float* result = stack + (size_t)n * stack_stride + base;
#pragma unroll
        for (int s = 0; s < PASSES; ++s) {
          const int i = (threadIdx.x + s * SN_THREADS) * 4;
          if (i < width) {
            const Quad4<float> qr = *reinterpret_cast<const Quad4<float>*>(result + i);
#pragma unroll
            for (int j = 0; j < 4; ++j) mine[s][j] = fmaf(c, qr.v[j], mine[s][j]);
          }
        }
      }
      const float c = to_float(coeffs[count]);
#pragma unroll
      for (int s = 0; s < PASSES; ++s) {
        const int i = (threadIdx.x + s * SN_THREADS) * 4;
        if (i < width) {
          Quad4<float> q;
#pragma unroll
          for (int j = 0; j < 4; ++j) q.v[j] = fmaf(c, stream[s][j], mine[s][j]);
          *reinterpret_cast<Quad4<float>*>(avg + base + i) = q;
        }
      }
    }
#pragma unroll
    for (int s = 0; s < PASSES; ++s) {
      const int i = (threadIdx.x + s * SN_THREADS) * 4;
      if (i < width) {
        Quad4<float> q;
#pragma unroll
        for (int j = 0; j < 4; ++j) q.v[j] = stream[s][j];
        *reinterpret_cast<Quad4<float>*>(out + base + i) = q;
        if (rounded != nullptr) {
          Quad4<T> r;
#pragma unroll
          for (int j = 0; j < 4; ++j) r.v[j] = from_float<T>(stream[s][j]);
          *reinterpret_cast<Quad4<T>*>(rounded + base + i) = r;
        }
      }
    }
    return;
  }
  if (KEPT == 1) {
    float mine[SN_KEEP], stream[SN_KEEP], w[SN_KEEP];
#pragma unroll
    for (int s = 0; s < SN_KEEP; ++s) {
      const int i = threadIdx.x + s * SN_THREADS;
      const bool in = i < width;
      mine[s] = in ? to_float(arow[i]) : 0.0f;
      stream[s] = in ? x[base + i] : 0.0f;
      w[s] = in ? to_float(weight[i]) : 0.0f;
      ss = fmaf(mine[s], mine[s], ss);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)width + eps);
#pragma unroll
    for (int s = 0; s < SN_KEEP; ++s) stream[s] = stream[s] + mine[s] * inv * w[s];
    if (avg != nullptr) {
      // the average in ascending order of the results; the loads of one result are in flight together
#pragma unroll
      for (int s = 0; s < SN_KEEP; ++s) mine[s] = 0.0f;
      for (int j = 0; j < count; ++j) {
        const float c = to_float(coeffs[j]);
        const float* result = stack + (size_t)j * stack_stride + base;
#pragma unroll
        for (int s = 0; s < SN_KEEP; ++s) {
          const int i = threadIdx.x + s * SN_THREADS;
          if (i < width) mine[s] = fmaf(c, result[i], mine[s]);
        }
      }
      const float c = to_float(coeffs[count]);
#pragma unroll
      for (int s = 0; s < SN_KEEP; ++s) {
        const int i = threadIdx.x + s * SN_THREADS;
        if (i < width) avg[base + i] = fmaf(c, stream[s], mine[s]);
      }
    }
#pragma unroll
    for (int s = 0; s < SN_KEEP; ++s) {
      const int i = threadIdx.x + s * SN_THREADS;
      if (i < width) {
        out[base + i] = stream[s];
        if (rounded != nullptr) rounded[base + i] = from_float<T>(stream[s]);
      }
    }
    return;
  }
  for (int i = threadIdx.x; i < width; i += SN_THREADS) {
    const float v = to_float(arow[i]);
    ss = fmaf(v, v, ss);
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += SN_THREADS) {
    const float y = x[base + i] + to_float(arow[i]) * inv * to_float(weight[i]);
    out[base + i] = y;
    if (rounded != nullptr) rounded[base + i] = from_float<T>(y);
    if (avg != nullptr) {
      float sum = 0.0f;
      for (int j = 0; j < count; ++j) sum = fmaf(to_float(coeffs[j]), stack[(size_t)j * stack_stride + base + i], sum);
      avg[base + i] = fmaf(to_float(coeffs[count]), y, sum);
    }
  }
}

extern "C" int kvb_stream_add_norm(float* out, const float* x, const void* a, const void* weight, int rows, int width,
                                   float eps, float* avg, const float* stack, long long stack_stride,
                                   const void* coeffs, int count, void* rounded, int dtype, int weight_dtype,
                                   cudaStream_t stream) {
  if (rows == 0) return 0;
  KVB_REQUIRE(width > 0, "stream_add_norm: width must be positive");
  KVB_REQUIRE(avg == nullptr || (coeffs != nullptr && count >= 0 && (count == 0 || stack != nullptr)),
              "stream_add_norm: the depth average needs its coefficients and the results in front");
  cudaError_t err;
  const bool kept = width <= SN_THREADS * SN_KEEP;
  const bool quads = kept && width % 4 == 0 && aligned16(out) && aligned16(x) && aligned16(a) && aligned16(weight) &&
                     (rounded == nullptr || ((uintptr_t)rounded & 7) == 0) &&
                     (avg == nullptr || (aligned16(avg) && (count == 0 || (aligned16(stack) && stack_stride % 4 == 0))));
#define KVB_AN_LAUNCH(T, W)                                                                                       \
  err = quads                                                                                                     \
      ? kvb_launch((stream_add_norm_kernel<T, W, 2>), dim3(rows), dim3(SN_THREADS), 0, stream, true, out, x,     \
                   (const T*)a, (const W*)weight, width, eps, avg, stack, stack_stride, (const W*)coeffs, count, (T*)rounded)  \
      : kept                                                                                                      \
      ? kvb_launch((stream_add_norm_kernel<T, W, 1>), dim3(rows), dim3(SN_THREADS), 0, stream, true, out, x,     \
                   (const T*)a, (const W*)weight, width, eps, avg, stack, stack_stride, (const W*)coeffs, count, (T*)rounded)  \
      : kvb_launch((stream_add_norm_kernel<T, W, 0>), dim3(rows), dim3(SN_THREADS), 0, stream, true, out, x,     \
                   (const T*)a, (const W*)weight, width, eps, avg, stack, stack_stride, (const W*)coeffs, count, (T*)rounded)
  if (dtype == KVB_F32 && weight_dtype == KVB_F32) KVB_AN_LAUNCH(float, float);
  else if (dtype == KVB_F32) KVB_AN_LAUNCH(float, bf16);
  else if (weight_dtype == KVB_F32) KVB_AN_LAUNCH(bf16, float);
  else KVB_AN_LAUNCH(bf16, bf16);
#undef KVB_AN_LAUNCH
  KVB_CHECK_CUDA(err);
  KVB_CHECK_LAUNCH();
  return 0;
}

KVB_TRACE_TU(stream_norm)
