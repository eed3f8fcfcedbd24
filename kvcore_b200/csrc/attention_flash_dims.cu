// Paged flash attention for bf16 on tensor cores (mma.sync m16n8k16, fp32 accumulate) when the width of
// a query/key (DK) and the width of a value (DV) differ: the tensor-core form of attention_dims.cu, with the
// same parameters (strides of keys and values given apart, several score maps a value head, values that
// may be the first entries of the key rows, a sink per query head, a slope per query head times the distance
// between query and key taken off the score, 32-bit or bf16 output).
//
// A block of 4 warps works on one (request, key head, slice of the value width) and one tile of query
// rows; a row is a (token, query head of the key head's group) pair, so the heads that share a key head
// reuse every K/V tile.  Two shapes of one kernel body:
//   * TILE (prompt portions, many heads a key head): 64 rows a block, 16 a warp; every warp scores all
//     keys of a K tile.
//   * SPLIT (at most 16 or 32 rows a key head: decode): the warps form RG row groups of 16 rows (RG = 1 or 2)
//     times 4 / RG key groups; a key group takes its share of every K tile's keys, and the key groups of a
//     row group merge their partial (max, sum, output) through shared memory.
// In both, the key range of a request may be cut into `num_splits` contiguous chunks (one block each);
// partial results then go to scratch and a second kernel combines them.
//
// DK is a runtime multiple of 16: the query tile stays in shared memory and its fragments are fetched
// for every k-step, so no register array depends on DK (a latent cache has keys of several hundred
// entries).  The value width a block accumulates, DVB, is a template parameter (its accumulators are
// registers); a wider DV is cut into slices of DVB, each a block of its own that scores the keys again.
// When the values are the leading entries of the key rows, no value tile is loaded: the products read
// the K tile's columns.  K/V tiles are gathered row by row through the block table with 16-byte cp.async
// copies into padded shared-memory rows, double buffered.  Scores, softmax and accumulation are 32-bit.
#include "common.cuh"

#define FD_THREADS 128
#define FD_PAD 8

struct FlashDimsParams {
  void* out; long long out_token_stride, out_head_stride; int out_f32;
  const bf16* q; long long q_token_stride, q_head_stride;
  const bf16* k; long long k_page_stride, k_head_stride, k_row_stride;
  const bf16* v; long long v_page_stride, v_head_stride, v_row_stride;
  const int* table; int table_stride;
  const int* query_start; const int* context_lens;
  const float* sink;
  const float* slopes;
  int num_reqs, KH, G, maps, DK, DV, page_size, num_pages, window, v_in_k, vsplit, tiles;
  float scale_log2;
  int num_splits;
  float* partial_o;   // [slot][TILE_M][DVB]
  float* partial_ml;  // [slot][TILE_M][2]
  int* status;
};

__device__ __forceinline__ void fd_cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;  // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void fd_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void fd_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void fd_ldmatrix_x4(unsigned (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void fd_ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void fd_mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned fd_pack(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const unsigned*>(&v);
}

// Element offsets of every key row (and value row) of a tile inside the cache, or -1: zero-fill.
template <int KEYS>
__device__ __forceinline__ void fd_lookup_rows(long long* k_rows, long long* v_rows, const FlashDimsParams& p,
                                               const int* pages, int kh, int vh, int v_col, int key0, int key_lo,
                                               int key_hi) {
  if (threadIdx.x >= KEYS) return;
  const int key = key0 + threadIdx.x;
  long long ko = -1, vo = -1;
  if (key >= key_lo && key < key_hi) {
    const int page = pages[key / p.page_size];
    if (page > 0 && page < p.num_pages) {
      const int slot = key % p.page_size;
      ko = (long long)page * p.k_page_stride + (long long)kh * p.k_head_stride + (long long)slot * p.k_row_stride;
      vo = (long long)page * p.v_page_stride + (long long)vh * p.v_head_stride + (long long)slot * p.v_row_stride + v_col;
    } else if (page != 0) {
      atomicOr(p.status, KVB_STATUS_BAD_PAGE);
    }
  }
  k_rows[threadIdx.x] = ko;
  v_rows[threadIdx.x] = vo;
}

template <int DVB, int KEYS>
__device__ __forceinline__ void fd_load_tile(bf16* ks, bf16* vs, const FlashDimsParams& p, const long long* k_rows,
                                             const long long* v_rows, int krow, int v_cols) {
  const int kchunks = p.DK / 8;
  for (int i = threadIdx.x; i < KEYS * kchunks; i += FD_THREADS) {
    const int row = i / kchunks, chunk = i % kchunks;
    const long long base = k_rows[row];
    fd_cp_async16(ks + row * krow + chunk * 8, p.k + (base >= 0 ? base + chunk * 8 : 0), base >= 0);
  }
  if (!p.v_in_k) {
    constexpr int VROW = DVB + FD_PAD;
    constexpr int vchunks = DVB / 8;
    for (int i = threadIdx.x; i < KEYS * vchunks; i += FD_THREADS) {
      const int row = i / vchunks, chunk = i % vchunks;
      const long long base = v_rows[row];
      const bool valid = base >= 0 && chunk * 8 < v_cols;   // columns beyond the value width read as zeros
      fd_cp_async16(vs + row * VROW + chunk * 8, p.v + (valid ? base + chunk * 8 : 0), valid);
    }
  }
}

template <int DVB, int KEYS, int RG>      // RG: row groups of the few-row form (1 or 2), 0 for 64-row tiles
__global__ void __launch_bounds__(FD_THREADS)
flash_dims_kernel(const FlashDimsParams p) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_FLASH_DIMS);
  constexpr bool SPLIT = RG > 0;
  constexpr int KG = SPLIT ? 4 / RG : 1;             // key groups of warps
  constexpr int TILE_M = SPLIT ? 16 * RG : 64;
  constexpr int VROW = DVB + FD_PAD;
  constexpr int DBLOCKS = DVB / 8;
  constexpr int WARP_KEYS = KEYS / KG;
  constexpr int NB = WARP_KEYS / 8;
  static_assert(NB >= 2 && NB % 2 == 0, "a warp scores at least 16 keys of a tile");
  const int DK = p.DK, krow = DK + FD_PAD, ksteps = DK / 16;

  extern __shared__ __align__(16) unsigned char smem_raw[];
  long long* k_rows = reinterpret_cast<long long*>(smem_raw);     // [2][KEYS]
  long long* v_rows = k_rows + 2 * KEYS;                            // [2][KEYS]
  bf16* qs = reinterpret_cast<bf16*>(v_rows + 2 * KEYS);            // [TILE_M][krow]
  bf16* ks = qs + TILE_M * krow;                                    // [2][KEYS][krow]
  bf16* vs = ks + 2 * KEYS * krow;                                  // [2][KEYS][VROW] unless the values are in the keys

  const int req = blockIdx.z;
  const int kh = blockIdx.y / p.vsplit, slice = blockIdx.y % p.vsplit;
  const int vh = kh / p.maps, map = kh % p.maps;
  const int tile = p.tiles - 1 - (int)(blockIdx.x / p.num_splits);   // heaviest (latest) query tiles first
  const int split = blockIdx.x % p.num_splits;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_begin = p.query_start[req];
  const int q_len = p.query_start[req + 1] - q_begin;
  const int context = p.context_lens[req];
  const int rows_total = q_len * p.G;
  const int row0 = tile * TILE_M;
  if (row0 >= rows_total) return;  // whole block: this request has fewer rows
  const int* pages = p.table + (size_t)req * p.table_stride;
  const int v_col = slice * DVB;                // first value column of this block
  const int v_cols = min(DVB, p.DV - v_col);    // value columns of this block that exist

  const int last_row = min(row0 + TILE_M, rows_total) - 1;
  const int first_pos = context + row0 / p.G;
  const int last_pos = context + last_row / p.G;
  int key_lo = p.window > 0 ? max(0, first_pos - p.window + 1) : 0;
  int key_hi = last_pos + 1;
  if (p.num_splits > 1) {
    const int base = (key_lo / KEYS) * KEYS;
    const int tiles = (key_hi - base + KEYS - 1) / KEYS;
    const int per = (tiles + p.num_splits - 1) / p.num_splits;
    const int lo = base + split * per * KEYS;
    key_hi = min(key_hi, lo + per * KEYS);
    key_lo = max(key_lo, lo);
  }
  const int tile_begin = key_lo / KEYS;
  const int tile_end = key_hi > key_lo ? (key_hi + KEYS - 1) / KEYS : tile_begin;

  // ---- Q tile into shared memory ---------------------------------------------------------------
  {
    const int chunks = DK / 8;
    for (int i = threadIdx.x; i < TILE_M * chunks; i += FD_THREADS) {
      const int r = i / chunks, chunk = i % chunks;
      const int flat = row0 + r;
      const bool valid = flat < rows_total;
      const int token = q_begin + (valid ? flat / p.G : 0);
      const int head = (vh * p.G + (valid ? flat % p.G : 0)) * p.maps + map;
      fd_cp_async16(qs + r * krow + chunk * 8,
                    p.q + (size_t)token * p.q_token_stride + (size_t)head * p.q_head_stride + chunk * 8, valid);
    }
  }
  fd_commit();
  if (tile_begin < tile_end) {
    fd_lookup_rows<KEYS>(k_rows, v_rows, p, pages, kh, vh, v_col, tile_begin * KEYS, key_lo, key_hi);
    if (tile_begin + 1 < tile_end)
      fd_lookup_rows<KEYS>(k_rows + KEYS, v_rows + KEYS, p, pages, kh, vh, v_col, (tile_begin + 1) * KEYS, key_lo, key_hi);
    __syncthreads();
    fd_load_tile<DVB, KEYS>(ks, vs, p, k_rows, v_rows, krow, v_cols);
  }
  fd_commit();
  fd_wait<1>();
  __syncthreads();

  const int wrow = SPLIT ? (warp % (SPLIT ? RG : 1)) * 16 : warp * 16;  // first row of this warp inside the block's tile
  int row_pos[2];
  bool row_valid[2];
  int row_head[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int flat = row0 + wrow + (lane >> 2) + 8 * h;
    row_valid[h] = flat < rows_total;
    row_pos[h] = context + (row_valid[h] ? flat / p.G : 0);
    row_head[h] = (vh * p.G + (row_valid[h] ? flat % p.G : 0)) * p.maps + map;
  }

  // the row's slope, in units of the base-2 exponent like the scores
  float row_slope[2] = {0.0f, 0.0f};
  if (p.slopes != nullptr) {
#pragma unroll
    for (int h = 0; h < 2; ++h) row_slope[h] = p.slopes[row_head[h]] * 1.4426950408889634f;
  }
  float o[DBLOCKS][4];
#pragma unroll
  for (int j = 0; j < DBLOCKS; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;
  float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.0f, 0.0f};
  // the sink joins the denominator once: in the first chunk of keys, and (SPLIT) in the first key group only
  if (p.sink != nullptr && split == 0 && (!SPLIT || warp / (SPLIT ? RG : 1) == 0)) {
#pragma unroll
    for (int h = 0; h < 2; ++h)
      if (row_valid[h]) {
        row_max[h] = p.sink[row_head[h]] * 1.4426950408889634f;
        row_sum[h] = (lane & 3) == 0 ? 1.0f : 0.0f;   // the row's sum is spread over the 4 lanes of a quad
      }
  }

  for (int t = tile_begin; t < tile_end; ++t) {
    const int buf = (t - tile_begin) & 1;
    bf16* kt = ks + buf * KEYS * krow;
    if (t + 1 < tile_end)
      fd_load_tile<DVB, KEYS>(ks + (buf ^ 1) * KEYS * krow, vs + (buf ^ 1) * KEYS * VROW, p,
                              k_rows + (buf ^ 1) * KEYS, v_rows + (buf ^ 1) * KEYS, krow, v_cols);
    fd_commit();
    fd_wait<1>();
    __syncthreads();  // tile t has landed; the row offsets of tile t (slot buf) are spent
    if (t + 2 < tile_end)
      fd_lookup_rows<KEYS>(k_rows + buf * KEYS, v_rows + buf * KEYS, p, pages, kh, vh, v_col, (t + 2) * KEYS, key_lo, key_hi);

    const int wkey = SPLIT ? (warp / (SPLIT ? RG : 1)) * WARP_KEYS : 0;  // first key of the tile this warp scores
    float s[NB][4];
#pragma unroll
    for (int j = 0; j < NB; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
#pragma unroll 4
    for (int k = 0; k < ksteps; ++k) {
      unsigned qf[4];
      fd_ldmatrix_x4(qf, qs + (wrow + (lane & 7) + 8 * ((lane >> 3) & 1)) * krow + k * 16 + 8 * (lane >> 4));
#pragma unroll
      for (int j = 0; j < NB; j += 2) {
        unsigned kb[4];
        const int key = wkey + j * 8 + (lane & 7) + 8 * (lane >> 4);
        fd_ldmatrix_x4(kb, kt + key * krow + k * 16 + 8 * ((lane >> 3) & 1));
        fd_mma(s[j], qf, kb[0], kb[1]);
        fd_mma(s[j + 1], qf, kb[2], kb[3]);
      }
    }
    // mask and online softmax (base-2 exponent)
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < NB; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int h = e >> 1;
        const int key = t * KEYS + wkey + j * 8 + (lane & 3) * 2 + (e & 1);
        const bool seen = row_valid[h] && key >= key_lo && key < key_hi && key <= row_pos[h] &&
                          (p.window <= 0 || key > row_pos[h] - p.window);
        const float v = seen ? fmaf(s[j][e], p.scale_log2, -row_slope[h] * (float)(row_pos[h] - key)) : -INFINITY;
        s[j][e] = v;
        tile_max[h] = fmaxf(tile_max[h], v);
      }
    }
    float correction[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float m = tile_max[h];
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
      const float new_max = fmaxf(row_max[h], m);
      correction[h] = (row_max[h] == -INFINITY) ? 0.0f : exp2f(row_max[h] - new_max);
      row_max[h] = new_max;
      row_sum[h] *= correction[h];
    }
#pragma unroll
    for (int j = 0; j < DBLOCKS; ++j) {
      o[j][0] *= correction[0]; o[j][1] *= correction[0];
      o[j][2] *= correction[1]; o[j][3] *= correction[1];
    }
#pragma unroll
    for (int j = 0; j < NB; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int h = e >> 1;
        const float pv = (s[j][e] == -INFINITY) ? 0.0f : exp2f(s[j][e] - row_max[h]);
        s[j][e] = pv;
        row_sum[h] += pv;
      }
    }
    // O += P V over this warp's keys, 16 keys per step; the values are a tile of their own or columns of K
    const bf16* vt = p.v_in_k ? kt + v_col : vs + buf * KEYS * VROW;
    const int vpitch = p.v_in_k ? krow : VROW;
#pragma unroll
    for (int kk = 0; kk < NB / 2; ++kk) {
      unsigned pa[4];
      pa[0] = fd_pack(s[2 * kk][0], s[2 * kk][1]);
      pa[1] = fd_pack(s[2 * kk][2], s[2 * kk][3]);
      pa[2] = fd_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      pa[3] = fd_pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int j = 0; j < DBLOCKS; j += 2) {
        unsigned vb[4];
        const int key = wkey + kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
        fd_ldmatrix_x4_trans(vb, vt + key * vpitch + j * 8 + 8 * (lane >> 4));
        fd_mma(o[j], pa, vb[0], vb[1]);
        fd_mma(o[j + 1], pa, vb[2], vb[3]);
      }
    }
    __syncthreads();  // everyone is done with this buffer before it is refilled
  }
  fd_wait<0>();

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    row_sum[h] += __shfl_xor_sync(0xffffffffu, row_sum[h], 1);
    row_sum[h] += __shfl_xor_sync(0xffffffffu, row_sum[h], 2);
  }
  const size_t slot = ((((size_t)req * p.KH + kh) * p.vsplit + slice) * p.tiles + tile) * p.num_splits + split;

  if (!SPLIT) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      if (!row_valid[h]) continue;
      const int r = wrow + (lane >> 2) + 8 * h;
      if (p.num_splits > 1) {
        float* dst = p.partial_o + (slot * TILE_M + r) * DVB + (lane & 3) * 2;
#pragma unroll
        for (int j = 0; j < DBLOCKS; ++j) { dst[j * 8] = o[j][2 * h]; dst[j * 8 + 1] = o[j][2 * h + 1]; }
        if ((lane & 3) == 0) {
          p.partial_ml[(slot * TILE_M + r) * 2 + 0] = row_max[h];
          p.partial_ml[(slot * TILE_M + r) * 2 + 1] = row_sum[h];
        }
        continue;
      }
      const int token = q_begin + (row0 + r) / p.G;
      const float inv = row_sum[h] > 0.0f ? 1.0f / row_sum[h] : 0.0f;
      const size_t off = (size_t)token * p.out_token_stride + (size_t)row_head[h] * p.out_head_stride + v_col;
#pragma unroll
      for (int j = 0; j < DBLOCKS; ++j) {
        const int c = j * 8 + (lane & 3) * 2;
        if (c >= v_cols) continue;           // value widths are multiples of 8: a pair is inside or outside
        if (p.out_f32)
          *reinterpret_cast<float2*>((float*)p.out + off + c) = make_float2(o[j][2 * h] * inv, o[j][2 * h + 1] * inv);
        else
          *reinterpret_cast<unsigned*>((bf16*)p.out + off + c) = fd_pack(o[j][2 * h] * inv, o[j][2 * h + 1] * inv);
      }
    }
    return;
  }

  // ---- SPLIT: merge the key groups of every row group (each saw other keys of the same 16 rows) ---------
  __syncthreads();
  float* merge_o = reinterpret_cast<float*>(ks);            // [4 warps][16 rows][DVB]
  float* merge_ml = merge_o + 4 * 16 * DVB;                 // [4 warps][16 rows][2]
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = (lane >> 2) + 8 * h;
#pragma unroll
    for (int j = 0; j < DBLOCKS; ++j) {
      float* dst = merge_o + ((size_t)(warp * 16 + r)) * DVB + j * 8 + (lane & 3) * 2;
      dst[0] = o[j][2 * h];
      dst[1] = o[j][2 * h + 1];
    }
    if ((lane & 3) == 0) {
      merge_ml[(warp * 16 + r) * 2 + 0] = row_max[h];
      merge_ml[(warp * 16 + r) * 2 + 1] = row_sum[h];
    }
  }
  __syncthreads();
  constexpr int GROUPS = SPLIT ? RG : 1;
  for (int i = threadIdx.x; i < TILE_M * DVB; i += FD_THREADS) {
    const int r = i / DVB, d = i % DVB;
    if (r >= rows_total || d >= v_cols) continue;
    const int group = r / 16, rr = r % 16;     // the row's warps are group, group + GROUPS, ...
    float m = -INFINITY;
#pragma unroll
    for (int kg = 0; kg < KG; ++kg) m = fmaxf(m, merge_ml[((kg * GROUPS + group) * 16 + rr) * 2]);
    float total = 0.0f, acc = 0.0f;
#pragma unroll
    for (int kg = 0; kg < KG; ++kg) {
      const int w = kg * GROUPS + group;
      const float mw = merge_ml[(w * 16 + rr) * 2];
      const float f = (mw == -INFINITY) ? 0.0f : exp2f(mw - m);
      total += merge_ml[(w * 16 + rr) * 2 + 1] * f;
      acc += merge_o[((size_t)(w * 16 + rr)) * DVB + d] * f;
    }
    if (p.num_splits == 1) {
      const int token = q_begin + r / p.G;
      const int head = (vh * p.G + r % p.G) * p.maps + map;
      const size_t off = (size_t)token * p.out_token_stride + (size_t)head * p.out_head_stride + v_col + d;
      const float value = total > 0.0f ? acc / total : 0.0f;
      if (p.out_f32) ((float*)p.out)[off] = value;
      else ((bf16*)p.out)[off] = __float2bfloat16_rn(value);
    } else {
      p.partial_o[(slot * TILE_M + r) * DVB + d] = acc;
      if (d == 0) {
        p.partial_ml[(slot * TILE_M + r) * 2 + 0] = m;
        p.partial_ml[(slot * TILE_M + r) * 2 + 1] = total;
      }
    }
  }
}

// Merge the splits of every (request, key head, value slice, query tile, row); one thread per output element.
template <int DVB>
__global__ void flash_dims_combine_kernel(const FlashDimsParams p, int tile_m) {
  KVB_KERNEL_PROLOGUE(KVB_TAG_FLASH_DIMS_COMBINE);
  const int req = blockIdx.z;
  const int kh = blockIdx.y / p.vsplit, slice = blockIdx.y % p.vsplit;
  const int vh = kh / p.maps, map = kh % p.maps;
  const int q_begin = p.query_start[req];
  const int rows_total = (p.query_start[req + 1] - q_begin) * p.G;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int flat = (int)(i / DVB), d = (int)(i % DVB);
  const int v_col = slice * DVB;
  if (flat >= rows_total || flat >= p.tiles * tile_m || v_col + d >= p.DV) return;
  const int tile = flat / tile_m, r = flat % tile_m;
  const size_t base = ((((size_t)req * p.KH + kh) * p.vsplit + slice) * p.tiles + tile) * p.num_splits;
  float m = -INFINITY, total = 0.0f, acc = 0.0f;
  for (int s = 0; s < p.num_splits; ++s) {
    const float ms = p.partial_ml[((base + s) * tile_m + r) * 2];
    const float ls = p.partial_ml[((base + s) * tile_m + r) * 2 + 1];
    const float os = p.partial_o[((base + s) * tile_m + r) * DVB + d];
    if (ms == -INFINITY) continue;
    if (ms > m) {
      const float keep = (m == -INFINITY) ? 0.0f : exp2f(m - ms);
      total *= keep;
      acc *= keep;
      m = ms;
    }
    const float f = exp2f(ms - m);
    total += ls * f;
    acc += os * f;
  }
  const int token = q_begin + flat / p.G;
  const int head = (vh * p.G + flat % p.G) * p.maps + map;
  const size_t off = (size_t)token * p.out_token_stride + (size_t)head * p.out_head_stride + v_col + d;
  const float value = total > 0.0f ? acc / total : 0.0f;
  if (p.out_f32) ((float*)p.out)[off] = value;
  else ((bf16*)p.out)[off] = __float2bfloat16_rn(value);
}

template <int DVB, int KEYS, int RG>
static int fd_launch_shape(const FlashDimsParams& p, int max_rows, cudaStream_t stream) {
  constexpr bool SPLIT = RG > 0;
  constexpr int TILE_M = SPLIT ? 16 * RG : 64;
  const int krow = p.DK + FD_PAD;
  size_t smem = 4 * KEYS * sizeof(long long) + (size_t)(TILE_M + 2 * KEYS) * krow * sizeof(bf16);
  if (!p.v_in_k) smem += (size_t)2 * KEYS * (DVB + FD_PAD) * sizeof(bf16);
  if (SPLIT) {
    const size_t merge = 4 * KEYS * sizeof(long long) + (size_t)TILE_M * krow * sizeof(bf16) +
                         (size_t)(4 * 16 * DVB + 4 * 16 * 2) * sizeof(float);
    if (smem < merge) smem = merge;
  }
  KVB_REQUIRE(smem <= 227 * 1024, "flash_dims: the tiles do not fit in shared memory");
  static size_t configured = 0;   // grows only; the first call of a size is never inside a graph capture
  if (smem > configured) {
    KVB_CHECK_CUDA(cudaFuncSetAttribute(flash_dims_kernel<DVB, KEYS, RG>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  dim3 grid(p.tiles * p.num_splits, p.KH * p.vsplit, p.num_reqs);
  KVB_CHECK_CUDA(kvb_launch((flash_dims_kernel<DVB, KEYS, RG>), dim3(grid), dim3(FD_THREADS), smem, stream, true, p));
  KVB_CHECK_LAUNCH();
  if (p.num_splits > 1) {
    const long long elements = (long long)(max_rows < p.tiles * TILE_M ? max_rows : p.tiles * TILE_M) * DVB;
    dim3 cgrid((unsigned)((elements + 127) / 128), p.KH * p.vsplit, p.num_reqs);
    KVB_CHECK_CUDA(kvb_launch((flash_dims_combine_kernel<DVB>), dim3(cgrid), dim3(128), 0, stream, true, p, TILE_M));
    KVB_CHECK_LAUNCH();
  }
  return 0;
}

template <int DVB>
static int fd_launch(const FlashDimsParams& p, int row_groups, int max_rows, cudaStream_t stream) {
  if (row_groups == 1) return fd_launch_shape<DVB, 64, 1>(p, max_rows, stream);
  if (row_groups == 2) return fd_launch_shape<DVB, 64, 2>(p, max_rows, stream);
  // tiles of 64 keys while three blocks of them fit a multiprocessor's shared memory, else tiles of 32
  size_t wide = 4 * 64 * sizeof(long long) + (size_t)(64 + 2 * 64) * (p.DK + FD_PAD) * sizeof(bf16);
  if (!p.v_in_k) wide += (size_t)2 * 64 * (DVB + FD_PAD) * sizeof(bf16);
  if (wide > 75 * 1024) return fd_launch_shape<DVB, 32, 0>(p, max_rows, stream);
  return fd_launch_shape<DVB, 64, 0>(p, max_rows, stream);
}

// The value width a block accumulates for a value width DV, and the number of slices (0: not taken).
extern "C" int kvb_flash_dims_block_width(int DV, int* slices) {
  static const int widths[] = {32, 64, 96, 128, 192, 256};
  if (DV <= 0 || DV % 8) { if (slices) *slices = 0; return 0; }
  const int count = (DV + 255) / 256;
  const int each = (DV + count - 1) / count;
  for (int w : widths)
    if (w >= each && (long long)w * count >= DV) { if (slices) *slices = count; return w; }
  if (slices) *slices = 0;
  return 0;
}

// Scratch floats for `num_splits` chunks of keys: partial outputs, then partial (max, sum).
extern "C" long long kvb_flash_dims_scratch_floats(int num_reqs, int KH, int DV, int max_rows, int num_splits) {
  if (num_splits <= 1) return 0;
  int slices = 0;
  const int dvb = kvb_flash_dims_block_width(DV, &slices);
  const int tile_m = max_rows <= 16 ? 16 : max_rows <= 32 ? 32 : 64;
  const long long tiles = (max_rows + tile_m - 1) / tile_m;
  return (long long)num_reqs * KH * slices * tiles * num_splits * tile_m * (dvb + 2);
}

extern "C" int kvb_flash_dims_attention(void* out, long long out_token_stride, long long out_head_stride, int out_f32,
                                        const void* q, long long q_token_stride, long long q_head_stride,
                                        const void* k, long long k_page_stride, long long k_head_stride,
                                        long long k_row_stride, const void* v, long long v_page_stride,
                                        long long v_head_stride, long long v_row_stride, const int* table,
                                        int table_stride, const int* query_start, const int* context_lens,
                                        const float* sink, const float* slopes, int num_reqs, int max_query_len,
                                        int value_heads,
                                        int group, int maps, int DK, int DV, int page_size, int num_pages,
                                        float scale, int window, int num_splits, float* scratch,
                                        cudaStream_t stream) {
  if (num_reqs == 0) return 0;
  KVB_REQUIRE(DK >= 16 && DK % 16 == 0 && DK <= 1024, "flash_dims: the key width must be a multiple of 16 up to 1024");
  int slices = 0;
  const int dvb = kvb_flash_dims_block_width(DV, &slices);
  KVB_REQUIRE(dvb > 0 && DV <= 1024, "flash_dims: the value width must be a multiple of 8 up to 1024");
  KVB_REQUIRE(value_heads > 0 && group > 0 && maps > 0, "flash_dims: bad head counts");
  KVB_REQUIRE(page_size > 0 && num_pages > 1, "flash_dims: empty cache");
  KVB_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && q_token_stride % 8 == 0 && q_head_stride % 8 == 0 &&
              k_page_stride % 8 == 0 && k_head_stride % 8 == 0 && k_row_stride % 8 == 0 && v_page_stride % 8 == 0 &&
              v_head_stride % 8 == 0 && v_row_stride % 8 == 0,
              "flash_dims: q and the cache rows must lie on 16-byte boundaries");
  KVB_REQUIRE(out_f32 ? (out_token_stride % 2 == 0 && out_head_stride % 2 == 0 && ((uintptr_t)out & 7) == 0)
                      : (out_token_stride % 2 == 0 && out_head_stride % 2 == 0 && ((uintptr_t)out & 3) == 0),
              "flash_dims: output rows must lie on boundaries of a pair of values");
  FlashDimsParams p;
  p.out = out; p.out_token_stride = out_token_stride; p.out_head_stride = out_head_stride; p.out_f32 = out_f32;
  p.q = (const bf16*)q; p.q_token_stride = q_token_stride; p.q_head_stride = q_head_stride;
  p.k = (const bf16*)k; p.k_page_stride = k_page_stride; p.k_head_stride = k_head_stride; p.k_row_stride = k_row_stride;
  p.v = (const bf16*)v; p.v_page_stride = v_page_stride; p.v_head_stride = v_head_stride; p.v_row_stride = v_row_stride;
  p.table = table; p.table_stride = table_stride; p.query_start = query_start; p.context_lens = context_lens;
  p.sink = sink; p.slopes = slopes; p.num_reqs = num_reqs; p.KH = value_heads * maps; p.G = group; p.maps = maps; p.DK = DK; p.DV = DV;
  p.page_size = page_size; p.num_pages = num_pages; p.window = window;
  // the values are columns of the key tile when they are the leading entries of the very rows that serve as keys
  p.v_in_k = (k == v && maps == 1 && k_page_stride == v_page_stride && k_head_stride == v_head_stride &&
              k_row_stride == v_row_stride && slices * dvb <= DK) ? 1 : 0;
  p.vsplit = slices;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = kvb_status_word();
  KVB_REQUIRE(p.status != nullptr, "flash_dims: no status word");
  const int max_rows = max_query_len * group;
  const int row_groups = max_rows <= 16 ? 1 : max_rows <= 32 ? 2 : 0;   // the few-row form, or 64-row tiles
  p.tiles = row_groups ? 1 : (max_rows + 63) / 64;
  p.num_splits = num_splits < 1 ? 1 : num_splits;
  KVB_REQUIRE(p.num_splits <= KVB_MAX_SPLITS, "flash_dims: at most 1024 splits");
  KVB_REQUIRE(p.num_splits == 1 || scratch != nullptr, "flash_dims: splits need scratch memory");
  KVB_REQUIRE(num_reqs <= 65535 && p.KH * p.vsplit <= 65535, "flash_dims: batch too large for one launch");
  p.partial_o = scratch;
  const int tile_m = row_groups ? 16 * row_groups : 64;
  p.partial_ml = scratch == nullptr ? nullptr
      : scratch + (size_t)num_reqs * p.KH * p.vsplit * p.tiles * p.num_splits * tile_m * dvb;
  switch (dvb) {
    case 32: return fd_launch<32>(p, row_groups, max_rows, stream);
    case 64: return fd_launch<64>(p, row_groups, max_rows, stream);
    case 96: return fd_launch<96>(p, row_groups, max_rows, stream);
    case 128: return fd_launch<128>(p, row_groups, max_rows, stream);
    case 192: return fd_launch<192>(p, row_groups, max_rows, stream);
    default: return fd_launch<256>(p, row_groups, max_rows, stream);
  }
}

KVB_TRACE_TU(attention_flash_dims)
