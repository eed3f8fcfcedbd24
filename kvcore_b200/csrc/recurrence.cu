// Mixers that carry a matrix-valued state per request and head instead of cached keys and values.
// Everything between the projections and the output projection is 32-bit: decays, step sizes, unit
// norms, the state, the read-out and the norm behind it.
//
//   state_scan: per (request, head) a state S [D, V] (32-bit, one row of `state` per state slot) runs
//   over the request's tokens of this step in order.
//     decay per key channel (gated linear attention):
//         S <- diag(a_t) S + k_t v_t^T,                 o_t = S^T q_t
//         with a_t = sigmoid(z_t)^(1/tau) and q_t scaled by `q_scale`, as `gla_prepare` left them (32-bit);
//     delta rule with one decay per head:
//         S <- g_t S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t
//         with q_t, k_t, v_t, beta_t, g_t as `conv_prepare` left them (32-bit).
//     one fixed decay a head (lightning attention):
//         S <- a_h S + k_t v_t^T,                       o_t = S^T q_t
//         with q_t = silu(.) * q_scale, k_t = silu(.) and v_t = silu(.) as `lightning_prepare` left them (32-bit),
//         a_h a constant of the model;
//   S is kept column by column ([H, V, D] in the state row: a column's D rows lie together).  A column is shared
//   by RSPLIT neighbouring lanes (4, 8 or 16 rows each, in registers, loaded and stored as 16-byte pieces); a
//   thread holds those rows of one column or of four neighbouring ones; a block owns 128 / RSPLIT (times four)
//   columns of one (request, head).  The launch picks the shape (see scan_shape).
//   Columns never exchange anything, and a sum over a column's rows is taken in one fixed order (four rows at a
//   time, then a tree over those pieces) whatever the shape, so any cut of a request into steps and any batch it
//   runs in give the same bits.  The tokens' vectors (32-bit: q, k, and the decays or beta and gate) come through
//   two stages of shared memory by cp.async, the next stage in flight while this one is computed; where each
//   thread's copies come from and go to is worked out once, not once a stage.  The read-outs' sums over a
//   column's threads are taken for eight tokens at once, off the chain that carries S from token to token.
//   gla_prepare writes the vectors of the decay-per-channel form (q times its scale, k, a = sigmoid(z)^(1/tau))
//   once a token, so the blocks that share a head do not each take the exponentials.
//
//   conv_prepare (delta rule): a short causal convolution over time per channel on the q, k and v
//   projections (taps [channels, C], the last tap on the current token; the C - 1 inputs in front of a
//   portion come from the request's state row), SiLU, q and k made unit vectors per head (q also times
//   `q_scale`), beta = sigmoid(b), g = exp(-exp(A_log) softplus(a + dt_bias)).  conv_state_update then
//   moves the last C - 1 inputs of every request into its state row.
//
//   gated_rms_norm: out[t, h, :] = o[t, h, :] / rms(o[t, h, :]) * weight * silu(gate[t, h, :]) * scale
//   (or sigmoid(gate) in place of silu(gate)).
#include "common.cuh"

#define SCAN_THREADS 128

__device__ __forceinline__ void scan_copy16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src));
}
__device__ __forceinline__ void scan_copy4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src));
}
__device__ __forceinline__ void scan_copies_done() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }

struct ScanParams {
  // 32-bit vectors per token: q and k [D] of head h / kv_share, and (decay per key channel) the decays a [D]
  // of head h, each at base + t * vec_token + head * D
  const float* q; const float* k; const float* a;
  long long vec_token;
  int vec16;                                // every vector starts on a 16-byte boundary and D is a multiple of 4
  int state16;                              // so does every column of S in the state rows
  const void* v; long long v_token;         // values [V] of head h at v + t * v_token + h * V (elements)
  const float* beta; const float* gate;     // [T, H] with row stride bg_stride (delta rule)
  long long bg_stride;
  float* out;                               // [T, H, V]
  float* state;                             // [slots, state_stride]; this mixer's S at state_offset, [H, V, D]
  long long state_stride, state_offset;
  const int* query_start; const int* state_slots;
  int heads, kv_share, D, V;
};

// MODE 0: decay per key channel; MODE 1: delta rule; MODE 2: one fixed decay a head (p.a[h]).  RSPLIT threads a column of S, DREG rows each; a thread
// holds those rows of CPT neighbouring columns (one load of q, k and the decays then serves CPT columns, and the
// columns' chains of dependent instructions run interleaved); BATCH tokens a stage of shared memory.
template <typename TV, int MODE, int DREG, int RSPLIT, int CPT, int BATCH>
__global__ void __launch_bounds__(SCAN_THREADS)
state_scan_kernel(ScanParams p) {
  KVB_KERNEL_PROLOGUE(MODE == 0 ? KVB_TAG_GLA_SCAN : MODE == 1 ? KVB_TAG_DELTA_SCAN : KVB_TAG_LIGHTNING_SCAN);
  extern __shared__ __align__(16) float smem[];
  constexpr int DP = DREG * RSPLIT;                 // rows covered (>= D; rows beyond D stay zero)
  constexpr int COLS = SCAN_THREADS / RSPLIT * CPT; // columns this block owns
  constexpr int NVEC = MODE == 0 ? 3 : 2;           // q, k (, a)
  constexpr int TOKEN = NVEC * DP + 4;              // floats a token holds in a stage; the last four: beta, gate
  constexpr int STAGE = BATCH * TOKEN;
  constexpr int VPT = (BATCH * COLS + SCAN_THREADS - 1) / SCAN_THREADS;
  constexpr int FPT = (BATCH * NVEC * (DP / 4) + SCAN_THREADS - 1) / SCAN_THREADS;   // 16-byte copies a thread, a stage
  constexpr int J = DREG / 4;
  constexpr int GROUP = BATCH < 8 ? BATCH : 8;      // tokens whose read-outs are summed over the threads together
  float* const vectors = smem;                      // [2][BATCH][TOKEN]
  float* const values = smem + 2 * STAGE;           // [2][BATCH][COLS]

  const int req = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int part = tid % RSPLIT, c = tid / RSPLIT * CPT;
  const int col = blockIdx.z * COLS + c;            // the first of this thread's columns
  const int begin = p.query_start[req], end = p.query_start[req + 1];
  const int D = p.D, V = p.V;
  const int kvh = h / p.kv_share;
  const TV* vg = (const TV*)p.v;

  // Thread `part` of a column holds the column's rows part * DREG .. part * DREG + DREG - 1 as J 16-byte pieces.
  // In shared memory a vector's piece n lies at place (n % J) * RSPLIT + n / J, so that for one j the parts of a
  // column read neighbouring pieces.
  float* const S_head = p.state + (size_t)p.state_slots[req] * p.state_stride + p.state_offset + (size_t)h * V * D;
  float S[CPT][DREG];
#pragma unroll
  for (int cc = 0; cc < CPT; ++cc) {
    const float* S_column = S_head + (size_t)(col + cc < V ? col + cc : 0) * D;
#pragma unroll
    for (int j = 0; j < J; ++j) {
      const int row = part * DREG + 4 * j;
      float4 s4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      if (col + cc < V && row < D) {
        if (p.state16) {
          s4 = *reinterpret_cast<const float4*>(S_column + row);
        } else {
          s4.x = S_column[row];
          if (row + 1 < D) s4.y = S_column[row + 1];
          if (row + 2 < D) s4.z = S_column[row + 2];
          if (row + 3 < D) s4.w = S_column[row + 3];
        }
      }
      S[cc][4 * j] = s4.x; S[cc][4 * j + 1] = s4.y; S[cc][4 * j + 2] = s4.z; S[cc][4 * j + 3] = s4.w;
    }
  }
  auto place = [](int row) { return (((row >> 2) % J) * RSPLIT + (row >> 2) / J) * 4 + (row & 3); };
  if (D < DP)                                       // rows beyond D read zeros whatever the stage holds
    for (int e = tid; e < 2 * BATCH * NVEC * (DP - D); e += SCAN_THREADS) {
      const int slot = e / (DP - D), i = D + e % (DP - D);
      vectors[(slot / NVEC) * TOKEN + (slot % NVEC) * DP + place(i)] = 0.0f;
    }

  // Where this thread's 16-byte copies of a stage come from (for the stage that starts at token 0) and go to:
  // the same for every stage, so the divisions are taken once.
  const float* copy_from[FPT];
  int copy_to[FPT];
  const int pieces = D >> 2, per_token = NVEC * pieces;
  if (p.vec16) {
#pragma unroll
    for (int n = 0; n < FPT; ++n) {
      const int e = tid + n * SCAN_THREADS;
      const int tt = e / per_token, r = e - tt * per_token, vec = r / pieces, i = (r - vec * pieces) << 2;
      const float* base = vec == 0 ? p.q : vec == 1 ? p.k : p.a;
      copy_from[n] = base + (long long)tt * p.vec_token + (long long)(vec == 2 ? h : kvh) * D + i;
      copy_to[n] = tt * TOKEN + vec * DP + place(i);
    }
  }
  auto fetch = [&](int stage, int t0, int nb) {     // the vectors of tokens t0 .. t0 + nb - 1, asynchronously
    float* dst = vectors + stage * STAGE;
    if (p.vec16) {
      const long long shift = (long long)t0 * p.vec_token;
#pragma unroll
      for (int n = 0; n < FPT; ++n)
        if (tid + n * SCAN_THREADS < nb * per_token) scan_copy16(dst + copy_to[n], copy_from[n] + shift);
    } else {
      const int floats = NVEC * D;
      for (int e = tid; e < nb * floats; e += SCAN_THREADS) {
        const int tt = e / floats, r = e - tt * floats, vec = r / D, i = r - vec * D;
        const float* base = vec == 0 ? p.q : vec == 1 ? p.k : p.a;
        scan_copy4(dst + tt * TOKEN + vec * DP + place(i),
                   base + (long long)(t0 + tt) * p.vec_token + (long long)(vec == 2 ? h : kvh) * D + i);
      }
    }
    if (MODE == 1)
      for (int e = tid; e < 2 * nb; e += SCAN_THREADS) {
        const int tt = e >> 1;
        scan_copy4(dst + tt * TOKEN + NVEC * DP + (e & 1),
                   ((e & 1) ? p.gate : p.beta) + (size_t)(t0 + tt) * p.bg_stride + h);
      }
  };
  // This block's columns of v pass through registers, as they were stored: a conversion at the load would wait
  // for the load at the top of every stage.
  TV held[VPT];
  auto load_values = [&](int t0, int nb) {
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int e = tid + j * SCAN_THREADS, tt = e / COLS, cc = blockIdx.z * COLS + e % COLS;
      if (tt < nb && cc < V) held[j] = vg[(long long)(t0 + tt) * p.v_token + (long long)h * V + cc];
    }
  };
  auto store_values = [&](int stage, int nb) {
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int e = tid + j * SCAN_THREADS, tt = e / COLS, cc = blockIdx.z * COLS + e % COLS;
      if (e < BATCH * COLS) values[stage * BATCH * COLS + e] = (tt < nb && cc < V) ? to_float(held[j]) : 0.0f;
    }
  };
  const float head_decay = MODE == 2 ? p.a[h] : 0.0f;
  // One token: the state's step and this thread's part of the read-out of each of its columns.  A sum over a
  // column's rows is taken piece by piece (four rows, in order), and the pieces are added as a tree over their
  // numbers (n with n ^ 1, then with n ^ 2, ...): inside a thread for the pieces it holds, by shuffles between the
  // threads of a column.  The result has the same bits for every DREG and CPT, so a launch may pick both by how
  // many columns it has.
  auto own = [&](const float (&piece)[J]) {         // the pieces this thread holds
    float sum = piece[0];
    if constexpr (J == 2) sum = piece[0] + piece[1];
    if constexpr (J == 4) sum = (piece[0] + piece[1]) + (piece[2] + piece[3]);
    return sum;
  };
  // The sums over the column's threads of the read-out are left to the caller, who takes them for all tokens of
  // a stage at once: those shuffles do not wait for one another, and the state's step does not wait for them.
  auto token = [&](const float* q, const float* vs, float (&o_own)[CPT]) {
    const float* k = q + DP;
    float v[CPT];
    if constexpr (CPT == 4) {
      const float4 v4 = *reinterpret_cast<const float4*>(vs);
      v[0] = v4.x; v[1] = v4.y; v[2] = v4.z; v[3] = v4.w;
    } else {
#pragma unroll
      for (int cc = 0; cc < CPT; ++cc) v[cc] = vs[cc];
    }
    float4 k4[J], q4[J];
#pragma unroll
    for (int j = 0; j < J; ++j) {
      k4[j] = *reinterpret_cast<const float4*>(k + (j * RSPLIT + part) * 4);
      q4[j] = *reinterpret_cast<const float4*>(q + (j * RSPLIT + part) * 4);
    }
    float o[CPT][J];
    if (MODE == 0) {
      const float* a = k + DP;
#pragma unroll
      for (int j = 0; j < J; ++j) {
        const float4 a4 = *reinterpret_cast<const float4*>(a + (j * RSPLIT + part) * 4);
#pragma unroll
        for (int cc = 0; cc < CPT; ++cc) {
          float* s = &S[cc][4 * j];
          s[0] = fmaf(k4[j].x, v[cc], a4.x * s[0]);
          s[1] = fmaf(k4[j].y, v[cc], a4.y * s[1]);
          s[2] = fmaf(k4[j].z, v[cc], a4.z * s[2]);
          s[3] = fmaf(k4[j].w, v[cc], a4.w * s[3]);
          o[cc][j] = fmaf(s[3], q4[j].w, fmaf(s[2], q4[j].z, fmaf(s[1], q4[j].y, s[0] * q4[j].x)));
        }
      }
    } else if (MODE == 2) {
#pragma unroll
      for (int j = 0; j < J; ++j) {
#pragma unroll
        for (int cc = 0; cc < CPT; ++cc) {
          float* s = &S[cc][4 * j];
          s[0] = fmaf(k4[j].x, v[cc], head_decay * s[0]);
          s[1] = fmaf(k4[j].y, v[cc], head_decay * s[1]);
          s[2] = fmaf(k4[j].z, v[cc], head_decay * s[2]);
          s[3] = fmaf(k4[j].w, v[cc], head_decay * s[3]);
          o[cc][j] = fmaf(s[3], q4[j].w, fmaf(s[2], q4[j].z, fmaf(s[1], q4[j].y, s[0] * q4[j].x)));
        }
      }
    } else {
      const float beta = q[NVEC * DP], g = q[NVEC * DP + 1];
      float dot[CPT];
#pragma unroll
      for (int cc = 0; cc < CPT; ++cc) {
        float d[J];
#pragma unroll
        for (int j = 0; j < J; ++j) {
          float* s = &S[cc][4 * j];
          s[0] *= g; s[1] *= g; s[2] *= g; s[3] *= g;
          d[j] = fmaf(s[3], k4[j].w, fmaf(s[2], k4[j].z, fmaf(s[1], k4[j].y, s[0] * k4[j].x)));
        }
        dot[cc] = own(d);
      }
#pragma unroll
      for (int m = 1; m < RSPLIT; m <<= 1)
#pragma unroll
        for (int cc = 0; cc < CPT; ++cc) dot[cc] += __shfl_xor_sync(0xffffffffu, dot[cc], m);
#pragma unroll
      for (int cc = 0; cc < CPT; ++cc) {
        const float u = beta * (v[cc] - dot[cc]);
#pragma unroll
        for (int j = 0; j < J; ++j) {
          float* s = &S[cc][4 * j];
          s[0] = fmaf(k4[j].x, u, s[0]);
          s[1] = fmaf(k4[j].y, u, s[1]);
          s[2] = fmaf(k4[j].z, u, s[2]);
          s[3] = fmaf(k4[j].w, u, s[3]);
          o[cc][j] = fmaf(s[3], q4[j].w, fmaf(s[2], q4[j].z, fmaf(s[1], q4[j].y, s[0] * q4[j].x)));
        }
      }
    }
#pragma unroll
    for (int cc = 0; cc < CPT; ++cc) o_own[cc] = own(o[cc]);
  };
  const bool out16 = CPT == 4 && (V & 3) == 0 && ((uintptr_t)p.out & 15) == 0;
  auto write_out = [&](float* at, const float (&sum)[CPT]) {      // the thread with part 0 writes its columns
    if (part != 0) return;
    if (CPT == 4 && out16 && col < V) {
      *reinterpret_cast<float4*>(at) = make_float4(sum[0], sum[1], sum[2], sum[3]);
      return;
    }
#pragma unroll
    for (int cc = 0; cc < CPT; ++cc)
      if (col + cc < V) at[cc] = sum[cc];
  };

  if (begin < end) {
    fetch(0, begin, min(BATCH, end - begin));
    load_values(begin, min(BATCH, end - begin));
    store_values(0, min(BATCH, end - begin));
  }
  scan_copies_done();
  __syncthreads();
  int stage = 0;
  const size_t out_token = (size_t)p.heads * V;
  for (int t0 = begin; t0 < end; t0 += BATCH, stage ^= 1) {
    const int nb = min(BATCH, end - t0);
    const int next = t0 + BATCH, next_nb = min(BATCH, end - next);
    if (next < end) {
      fetch(stage ^ 1, next, next_nb);
      load_values(next, next_nb);
    }
    const float* st = vectors + stage * STAGE;
    const float* vs = values + stage * BATCH * COLS + c;
    float* out_at = p.out + ((size_t)t0 * p.heads + h) * V + (col < V ? col : 0);
    if (nb == BATCH) {                                // a full stage: nothing to ask between its tokens
#pragma unroll
      for (int g = 0; g < BATCH; g += GROUP) {
        float sums[GROUP][CPT];
#pragma unroll
        for (int tt = 0; tt < GROUP; ++tt) token(st + (g + tt) * TOKEN, vs + (g + tt) * COLS, sums[tt]);
#pragma unroll
        for (int m = 1; m < RSPLIT; m <<= 1)
#pragma unroll
          for (int tt = 0; tt < GROUP; ++tt)
#pragma unroll
            for (int cc = 0; cc < CPT; ++cc) sums[tt][cc] += __shfl_xor_sync(0xffffffffu, sums[tt][cc], m);
#pragma unroll
        for (int tt = 0; tt < GROUP; ++tt) write_out(out_at + (g + tt) * out_token, sums[tt]);
      }
    } else {
      for (int tt = 0; tt < nb; ++tt) {
        float sum[CPT];
        token(st + tt * TOKEN, vs + tt * COLS, sum);
#pragma unroll
        for (int m = 1; m < RSPLIT; m <<= 1)
#pragma unroll
          for (int cc = 0; cc < CPT; ++cc) sum[cc] += __shfl_xor_sync(0xffffffffu, sum[cc], m);
        write_out(out_at + tt * out_token, sum);
      }
    }
    if (next < end) store_values(stage ^ 1, next_nb);
    scan_copies_done();
    __syncthreads();
  }
#pragma unroll
  for (int cc = 0; cc < CPT; ++cc) {
    if (col + cc >= V) continue;
    float* S_column = S_head + (size_t)(col + cc) * D;
#pragma unroll
    for (int j = 0; j < J; ++j) {
      const int row = part * DREG + 4 * j;
      if (row < D) {
        if (p.state16) {
          *reinterpret_cast<float4*>(S_column + row) =
              make_float4(S[cc][4 * j], S[cc][4 * j + 1], S[cc][4 * j + 2], S[cc][4 * j + 3]);
        } else {
          S_column[row] = S[cc][4 * j];
          if (row + 1 < D) S_column[row + 1] = S[cc][4 * j + 1];
          if (row + 2 < D) S_column[row + 2] = S[cc][4 * j + 2];
          if (row + 3 < D) S_column[row + 3] = S[cc][4 * j + 3];
        }
      }
    }
  }
}

// Rows of S a thread holds, how many neighbouring columns, and how many tokens a stage.  Sums over a column come
// out with the same bits whatever the choice, so it follows the launch (timed at keys of 128 entries, 2,048 to
// 4,096 columns a request).  A step of single tokens moves every state once and does little else: 8 rows of four
// columns, stages of two tokens (6 KB a block, so that many blocks share an SM).  A step with prompts in it is a
// chain of dependent instructions per token, and the stages' hand-overs cost as much as their tokens: stages of
// 16 tokens; the delta rule, whose chain passes through a sum over the column's threads, 16 rows of one column
// (three shuffles in the chain, not five); the decay per channel, whose chain stays inside a thread, 8 or 4 rows
// of four columns (one load of q, k and the decays serves four columns) while that still fills the SMs, else 4
// rows of one column, which gives four times the warps.
struct ScanShape { int rows, cols; bool brief; };
static long long scan_blocks(int D, long long heads_of_all, int V, int rows, int cols) {
  int rsplit = 1;
  while (rows * rsplit < D) rsplit *= 2;
  const int owned = SCAN_THREADS / rsplit * cols;
  return heads_of_all * ((V + owned - 1) / owned);
}
static ScanShape scan_shape(int mode, int D, long long heads_of_all, int V, bool brief) {
  const long long sms = kvb_sm_count() > 0 ? kvb_sm_count() : 148;
  int least = 4;                                      // 32 threads a column at most
  while (least * 32 < D) least *= 2;
  // tests run every choice on one input and compare the bits
  const char* rows_asked = getenv("KVCORE_SCAN_ROWS");
  const char* cols_asked = getenv("KVCORE_SCAN_COLS");
  const int r = rows_asked ? atoi(rows_asked) : 0, c = cols_asked ? atoi(cols_asked) : 0;
  if ((r == 4 || r == 8 || r == 16) && r >= least) return {r, (c == 4 && r <= 8) ? 4 : 1, false};
  if (c == 4) return {least, least <= 8 ? 4 : 1, brief && least == 8};
  if (c == 1) return {least, 1, false};
  if (brief) return least <= 8 ? ScanShape{8, 4, true} : ScanShape{16, 1, true};
  if (mode == 1) return {16, 1, false};
  if (least <= 8 && scan_blocks(D, heads_of_all, V, 8, 4) >= 2 * sms) return {8, 4, false};
  if (least <= 4 && scan_blocks(D, heads_of_all, V, 4, 4) >= sms) return {4, 4, false};
  return {least, 1, false};
}

template <typename TV, int MODE>
static int launch_state_scan(const ScanParams& p_in, int num_reqs, long long tokens, cudaStream_t stream) {
  ScanParams p = p_in;
  KVB_REQUIRE(p.D <= 512, "state_scan: keys wider than 512 entries");
  const ScanShape shape = scan_shape(MODE, p.D, (long long)num_reqs * p.heads, p.V, tokens <= 2LL * num_reqs);
  const int dreg = shape.rows, cpt = shape.cols;
  int rsplit = 1;
  while (dreg * rsplit < p.D) rsplit *= 2;
  p.vec16 = (p.D % 4 == 0 && p.vec_token % 4 == 0 &&
             ((uintptr_t)p.q | (uintptr_t)p.k | (MODE == 2 ? 0 : (uintptr_t)p.a)) % 16 == 0) ? 1 : 0;
  p.state16 = (p.D % 4 == 0 && p.state_stride % 4 == 0 && p.state_offset % 4 == 0 && (uintptr_t)p.state % 16 == 0) ? 1 : 0;
  const int cols = SCAN_THREADS / rsplit * cpt;
  const dim3 grid(num_reqs, p.heads, (p.V + cols - 1) / cols), block(SCAN_THREADS);
  cudaError_t err = cudaErrorInvalidValue;
#define SCAN_CASE(DR, RS, CP, BRIEF)                                                                          \
  if (dreg == DR && rsplit == RS && cpt == CP && shape.brief == BRIEF) {                                      \
    constexpr int B = BRIEF ? 2 : DR * RS <= 128 ? 16 : 2048 / (DR * RS);                                     \
    const size_t smem = 2 * (size_t)B * ((MODE == 0 ? 3 : 2) * DR * RS + 4 + SCAN_THREADS / RS * CP) * sizeof(float); \
    static bool allowed = false;                      /* more than 48 KB a block is asked for once */         \
    if (smem > 48 * 1024 && !allowed) {                                                                       \
      KVB_CHECK_CUDA(cudaFuncSetAttribute(state_scan_kernel<TV, MODE, DR, RS, CP, B>,                         \
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));           \
      allowed = true;                                                                                         \
    }                                                                                                         \
    err = kvb_launch((state_scan_kernel<TV, MODE, DR, RS, CP, B>), grid, block, smem, stream, true, p);       \
  }
#define SCAN_ROWS(DR, CP, BRIEF)                                                                              \
  SCAN_CASE(DR, 1, CP, BRIEF) SCAN_CASE(DR, 2, CP, BRIEF) SCAN_CASE(DR, 4, CP, BRIEF) SCAN_CASE(DR, 8, CP, BRIEF) \
  SCAN_CASE(DR, 16, CP, BRIEF) SCAN_CASE(DR, 32, CP, BRIEF)
  SCAN_ROWS(4, 1, false) SCAN_ROWS(8, 1, false) SCAN_ROWS(16, 1, false) SCAN_ROWS(4, 4, false) SCAN_ROWS(8, 4, false)
  SCAN_ROWS(16, 1, true) SCAN_ROWS(8, 4, true)
#undef SCAN_ROWS
#undef SCAN_CASE
  KVB_CHECK_CUDA(err);
  KVB_CHECK_LAUNCH();
  return 0;
}

// What the decay-per-channel scan reads, 32-bit [T, 3 * H * D]: q times q_scale, k, and the decays
// a = sigmoid(z)^(1/tau) = exp(log_sigmoid(z) / tau) with log_sigmoid(z) = min(z, 0) - log1p(exp(-|z|)).
template <typename T>
__global__ void __launch_bounds__(256)
gla_prepare_kernel(float* __restrict__ out, const T* __restrict__ q, const T* __restrict__ k, long long row_stride,
                   const T* __restrict__ z, long long z_stride, long long tokens, int width, float q_scale,
                   float inv_tau) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_GLA_PREPARE);
  const long long total = tokens * width;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
    const long long t = e / width;
    const int i = (int)(e - t * width);
    float* row = out + t * 3 * width;
    const float zv = to_float(z[t * z_stride + i]);
    row[i] = to_float(q[t * row_stride + i]) * q_scale;
    row[width + i] = to_float(k[t * row_stride + i]);
    row[2 * width + i] = expf((fminf(zv, 0.0f) - log1pf(expf(-fabsf(zv)))) * inv_tau);
  }
}

// Decay per key channel.  q, k, v: columns of the projected rows (row stride `row_stride`, heads side by side);
// z [T, H * D] (row stride z_stride): the decay's logits; prepared: scratch, 32-bit [T, 3 * H * D].
extern "C" int kvb_gla_scan(float* out, float* prepared, const void* q, const void* k, const void* v,
                            long long row_stride, const void* z, long long z_stride, float* state,
                            long long state_stride, long long state_offset, const int* query_start,
                            const int* state_slots, int tokens, int num_reqs, int heads, int D, int V, float q_scale,
                            float tau, int dtype, cudaStream_t stream) {
  if (num_reqs == 0 || tokens == 0) return 0;
  KVB_REQUIRE(heads > 0 && D > 0 && V > 0 && tau > 0.0f, "gla_scan: bad sizes");
  KVB_REQUIRE(heads <= 65535, "gla_scan: too many heads");
  const int width = heads * D;
  const long long wanted = ((long long)tokens * width + 255) / 256;
  const long long resident = (long long)(kvb_sm_count() > 0 ? kvb_sm_count() : 1) * 16;
  const dim3 grid((unsigned)(wanted < resident ? wanted : resident));
  if (dtype == KVB_F32)
    KVB_CHECK_CUDA(kvb_launch((gla_prepare_kernel<float>), grid, dim3(256), 0, stream, true, prepared, (const float*)q,
        (const float*)k, row_stride, (const float*)z, z_stride, (long long)tokens, width, q_scale, 1.0f / tau));
  else
    KVB_CHECK_CUDA(kvb_launch((gla_prepare_kernel<bf16>), grid, dim3(256), 0, stream, true, prepared, (const bf16*)q,
        (const bf16*)k, row_stride, (const bf16*)z, z_stride, (long long)tokens, width, q_scale, 1.0f / tau));
  ScanParams p = {};
  p.q = prepared; p.k = prepared + width; p.a = prepared + 2 * width; p.vec_token = 3LL * width;
  p.v = v; p.v_token = row_stride;
  p.out = out; p.state = state; p.state_stride = state_stride; p.state_offset = state_offset;
  p.query_start = query_start; p.state_slots = state_slots;
  p.heads = heads; p.kv_share = 1; p.D = D; p.V = V;
  return dtype == KVB_F32 ? launch_state_scan<float, 0>(p, num_reqs, tokens, stream)
                          : launch_state_scan<bf16, 0>(p, num_reqs, tokens, stream);
}

// What the fixed-decay scan reads, 32-bit [T, 2 * H * D + H * V]: silu(q) times q_scale, silu(k), silu(v).
// QUADS: four neighbouring entries a thread, loaded and stored as one piece (widths that are multiples of four,
// rows and pointers on the boundaries of such pieces).
template <typename T>
struct __align__(4 * sizeof(T)) ScanQuad { T v[4]; };

__device__ __forceinline__ float scan_silu(float x) { return __fdividef(x, 1.0f + expf(-x)); }

template <typename T, bool QUADS>
__global__ void __launch_bounds__(256)
lightning_prepare_kernel(float* __restrict__ out, const T* __restrict__ q, const T* __restrict__ k,
                         const T* __restrict__ v, long long row_stride, long long tokens, int width, int vwidth,
                         float q_scale) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_LIGHTNING_PREPARE);
  constexpr int N = QUADS ? 4 : 1;
  const int per_token = (2 * width + vwidth) / N;
  const long long total = tokens * per_token;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
    const long long t = e / per_token;
    const int i = (int)(e - t * per_token) * N;
    const T* src = (i < width ? q + i : i < 2 * width ? k + (i - width) : v + (i - 2 * width)) + t * row_stride;
    const float factor = i < width ? q_scale : 1.0f;
    if (QUADS) {
      const ScanQuad<T> in = *reinterpret_cast<const ScanQuad<T>*>(src);
      ScanQuad<float> y;
#pragma unroll
      for (int j = 0; j < 4; ++j) y.v[j] = scan_silu(to_float(in.v[j])) * factor;
      *reinterpret_cast<ScanQuad<float>*>(out + e * 4) = y;
    } else {
      out[e] = scan_silu(to_float(src[0])) * factor;
    }
  }
}

// One fixed decay a head.  q, k, v: columns of the projected rows (row stride `row_stride`, heads side by side),
// all three passed through SiLU; decay [H] 32-bit; prepared: scratch, 32-bit [T, 2 * H * D + H * V].
extern "C" int kvb_lightning_scan(float* out, float* prepared, const void* q, const void* k, const void* v,
                                  long long row_stride, const float* decay, float* state, long long state_stride,
                                  long long state_offset, const int* query_start, const int* state_slots, int tokens,
                                  int num_reqs, int heads, int D, int V, float q_scale, int dtype,
                                  cudaStream_t stream) {
  if (num_reqs == 0 || tokens == 0) return 0;
  KVB_REQUIRE(heads > 0 && D > 0 && V > 0 && decay != nullptr, "lightning_scan: bad sizes");
  KVB_REQUIRE(heads <= 65535, "lightning_scan: too many heads");
  const int width = heads * D, vwidth = heads * V;
  const long long per_token = 2LL * width + vwidth;
  const size_t piece = 4 * (dtype == KVB_F32 ? sizeof(float) : sizeof(bf16));
  const bool quads = width % 4 == 0 && vwidth % 4 == 0 && row_stride % 4 == 0 && aligned16(prepared) &&
                     ((uintptr_t)q | (uintptr_t)k | (uintptr_t)v) % piece == 0;
  const long long wanted = ((long long)tokens * per_token / (quads ? 4 : 1) + 255) / 256;
  const long long resident = (long long)(kvb_sm_count() > 0 ? kvb_sm_count() : 1) * 16;
  const dim3 grid((unsigned)(wanted < resident ? wanted : resident));
#define KVB_LP_LAUNCH(T_, Q_)                                                                                  \
  KVB_CHECK_CUDA(kvb_launch((lightning_prepare_kernel<T_, Q_>), grid, dim3(256), 0, stream, true, prepared,    \
      (const T_*)q, (const T_*)k, (const T_*)v, row_stride, (long long)tokens, width, vwidth, q_scale))
  if (dtype == KVB_F32) { if (quads) KVB_LP_LAUNCH(float, true); else KVB_LP_LAUNCH(float, false); }
  else { if (quads) KVB_LP_LAUNCH(bf16, true); else KVB_LP_LAUNCH(bf16, false); }
#undef KVB_LP_LAUNCH
  ScanParams p = {};
  p.q = prepared; p.k = prepared + width; p.a = decay; p.vec_token = per_token;
  p.v = prepared + 2 * width; p.v_token = per_token;
  p.out = out; p.state = state; p.state_stride = state_stride; p.state_offset = state_offset;
  p.query_start = query_start; p.state_slots = state_slots;
  p.heads = heads; p.kv_share = 1; p.D = D; p.V = V;
  return launch_state_scan<float, 2>(p, num_reqs, tokens, stream);
}

// Delta rule.  prepared [T, 2 * G * D + H * V + 2 * H] 32-bit as conv_prepare leaves it: q, k (G heads), v, beta, gate.
extern "C" int kvb_delta_scan(float* out, const float* prepared, float* state, long long state_stride,
                              long long state_offset, const int* query_start, const int* state_slots, int tokens,
                              int num_reqs, int heads, int kv_heads, int D, int V, cudaStream_t stream) {
  if (num_reqs == 0) return 0;
  KVB_REQUIRE(heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && D > 0 && V > 0, "delta_scan: bad sizes");
  KVB_REQUIRE(heads <= 65535, "delta_scan: too many heads");
  const long long width = 2LL * kv_heads * D + (long long)heads * V + 2LL * heads;
  ScanParams p = {};
  p.q = prepared; p.k = prepared + (size_t)kv_heads * D; p.a = prepared; p.vec_token = width;
  p.v = prepared + 2 * (size_t)kv_heads * D; p.v_token = width;
  p.out = out; p.state = state; p.state_stride = state_stride; p.state_offset = state_offset;
  p.query_start = query_start; p.state_slots = state_slots;
  p.heads = heads; p.kv_share = heads / kv_heads; p.D = D; p.V = V;
  p.beta = prepared + 2 * (size_t)kv_heads * D + (size_t)heads * V;
  p.gate = p.beta + heads;
  p.bg_stride = width;
  return launch_state_scan<float, 1>(p, num_reqs, tokens, stream);
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
                      int heads, int V, float eps, float scale, int sigmoid_gate) {
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
      const float sig = 1.0f / (1.0f + expf(-gv));
      dst[i] = from_float<T>(src[i] * inv * to_float(weight[i]) * (sigmoid_gate ? sig : gv * sig));
    }
  }
}

// The same for vectors of more than a thousand entries (one norm over all heads of a token): a block a vector.
template <typename T>
__global__ void __launch_bounds__(1024)
gated_rms_norm_wide_kernel(T* __restrict__ out, long long out_stride, const float* __restrict__ o,
                           const T* __restrict__ gate, long long gate_stride, const T* __restrict__ weight, int heads,
                           int V, float eps, float scale, int sigmoid_gate) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_GATED_NORM);
  __shared__ float scratch[32];
  const long long n = blockIdx.x;
  const long long t = n / heads;
  const int h = (int)(n % heads);
  const float* src = o + n * V;
  const T* g = gate + t * gate_stride + (long long)h * V;
  T* dst = out + t * out_stride + (long long)h * V;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) { const float v = src[i]; ss = fmaf(v, v, ss); }
  const float inv = scale / sqrtf(block_sum(ss, scratch) / (float)V + eps);
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float gv = to_float(g[i]);
    const float sig = 1.0f / (1.0f + expf(-gv));
    dst[i] = from_float<T>(src[i] * inv * to_float(weight[i]) * (sigmoid_gate ? sig : gv * sig));
  }
}

extern "C" int kvb_gated_rms_norm(void* out, long long out_stride, const float* o, const void* gate,
                                  long long gate_stride, const void* weight, int tokens, int heads, int V, float eps,
                                  float scale, int sigmoid_gate, int dtype, cudaStream_t stream) {
  const long long vectors = (long long)tokens * heads;
  if (vectors == 0) return 0;
  KVB_REQUIRE(V > 0, "gated_rms_norm: bad width");
  if (V > 1024 && vectors <= 0x7fffffffLL) {
    // the threads of a block follow the width alone, so a vector's sum does not depend on the batch
    const int wide_threads = V >= 4096 ? 1024 : V >= 2048 ? 512 : 256;
    if (dtype == KVB_F32)
      KVB_CHECK_CUDA(kvb_launch((gated_rms_norm_wide_kernel<float>), dim3((unsigned)vectors), dim3(wide_threads), 0, stream, true,
          (float*)out, out_stride, o, (const float*)gate, gate_stride, (const float*)weight, heads, V, eps, scale,
          sigmoid_gate));
    else
      KVB_CHECK_CUDA(kvb_launch((gated_rms_norm_wide_kernel<bf16>), dim3((unsigned)vectors), dim3(wide_threads), 0, stream, true,
          (bf16*)out, out_stride, o, (const bf16*)gate, gate_stride, (const bf16*)weight, heads, V, eps, scale,
          sigmoid_gate));
    KVB_CHECK_LAUNCH();
    return 0;
  }
  const long long wanted = (vectors + CP_THREADS / 32 - 1) / (CP_THREADS / 32);
  const long long resident = (long long)(kvb_sm_count() > 0 ? kvb_sm_count() : 1) * 16;
  const int blocks = (int)(wanted < resident ? wanted : resident);
  if (dtype == KVB_F32)
    KVB_CHECK_CUDA(kvb_launch((gated_rms_norm_kernel<float>), dim3(blocks), dim3(CP_THREADS), 0, stream, true,
        (float*)out, out_stride, o, (const float*)gate, gate_stride, (const float*)weight, vectors, heads, V, eps, scale, sigmoid_gate));
  else
    KVB_CHECK_CUDA(kvb_launch((gated_rms_norm_kernel<bf16>), dim3(blocks), dim3(CP_THREADS), 0, stream, true,
        (bf16*)out, out_stride, o, (const bf16*)gate, gate_stride, (const bf16*)weight, vectors, heads, V, eps, scale, sigmoid_gate));
  KVB_CHECK_LAUNCH();
  return 0;
}

KVB_TRACE_TU(recurrence)
