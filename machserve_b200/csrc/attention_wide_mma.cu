// Tensor-core (mma.sync m16n8k16, bfloat16) paged attention for the mixers of attention_wide.cu: keys and values of
// different widths, values that are the first columns of the keys' own plane (a latent cache), an optional sink per head.
//
// A block of four warps attends 16 query rows: 16 consecutive rows of one sequence with one head (a tile of a prompt's
// portion), or, HEADS, up to 16 query heads of one token that share a key head (a decoding row: the heads of a group, or
// all heads over a latent cache, fill the tensor core's 16 rows).  Wide values do not fit one warp's registers, so the
// warps divide the work of a tile of 64 keys twice: for S = Q K^T each warp takes 16 of the keys (over all dk), for
// O += P V each warp takes a quarter of the value columns (over all 64 keys); the probabilities cross between the two
// through shared memory, and the row maxima through a small array.  Keys come in by 16-byte asynchronous copies through
// the block table; with a latent cache the value tile IS the key tile.  Scores, maxima, sums and O are float32; Q, K,
// V and P enter the tensor core as bfloat16.  Exponentials are 2^x with the scale folded in.
// With `splits` > 1 (decoding rows, to fill the GPU) split s takes the key tiles s, s + splits, ... and leaves
// (O, m, l) in scratch memory; a second kernel merges the splits in order and adds the sink.  Nothing waits on another
// block.  dk a multiple of 16; dv and the value rows' stride multiples of 8; dv <= 512.
#include "attention_mma.cuh"
#include "launch.cuh"

#define AWM_KT 64
#define AWM_ROWS 16
#define AWM_WARPS 4

// DVW: value columns a warp owns (the block covers 4 * DVW >= dv).
template <int DVW, bool SEPARATE_V, bool HEADS>
__global__ void __launch_bounds__(AWM_WARPS * 32)
attention_wide_mma_kernel(const float* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
                          const __nv_bfloat16* __restrict__ v_pages, __nv_bfloat16* __restrict__ out,
                          const float* __restrict__ sinks, const int* __restrict__ positions, const int* __restrict__ slots,
                          const int* __restrict__ block_table, int max_pages, int num_pages, const int* __restrict__ unit_row0,
                          const int* __restrict__ unit_rows, int hq, int hkv, int dk, int dv, int vw, int page_size, int window,
                          float scale_log2, int splits, float* __restrict__ scratch) {
  constexpr int DVP = 4 * DVW;
  extern __shared__ __align__(16) unsigned char awm_smem[];
  const int ks_stride = dk + 8;          // elements of a row of the Q and K tiles
  constexpr int VS = DVP + 8;            // elements of a row of a separate V tile
  constexpr int PS = AWM_KT + 8;         // elements of a row of P
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(awm_smem);                 // [16][dk + 8]
  __nv_bfloat16* k_s = q_s + AWM_ROWS * ks_stride;                                  // [64][dk + 8] (+ slack: V columns past dk)
  __nv_bfloat16* v_s = SEPARATE_V ? k_s + AWM_KT * ks_stride + DVP : k_s;           // [64][DVP + 8] or the key tile
  __nv_bfloat16* p_s = (SEPARATE_V ? v_s + AWM_KT * VS : k_s + AWM_KT * ks_stride + DVP);  // [16][64 + 8]
  float* red = reinterpret_cast<float*>(p_s + AWM_ROWS * PS);                       // [4][16]
  const int v_stride = SEPARATE_V ? VS : ks_stride;

  ms_pdl_trigger();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int groups = hq / hkv;
  const int split = blockIdx.x % splits, item = blockIdx.x / splits;
  int row0, live, kvh, head0, seq, pos0;
  ms_pdl_wait();
  if (HEADS) {  // item = (unit, kv head, chunk of 16 heads of its group)
    const int per_kv = (groups + AWM_ROWS - 1) / AWM_ROWS;
    const int unit = item / (hkv * per_kv), rem = item - unit * (hkv * per_kv);
    kvh = rem / per_kv;
    const int g0 = (rem - kvh * per_kv) * AWM_ROWS;
    head0 = kvh * groups + g0;
    live = min(AWM_ROWS, groups - g0);
    row0 = unit_row0 ? unit_row0[unit] : unit;
    if (row0 < 0) return;
  } else {  // item = (tile of rows, head)
    const int unit = item / hq;
    head0 = item - unit * hq;
    kvh = head0 / groups;
    row0 = unit_row0[unit];
    live = unit_rows[unit];
    if (live <= 0) return;
  }
  seq = slots[row0];
  if (seq < 0) return;
  pos0 = positions[row0];
  const int last_pos = HEADS ? pos0 : pos0 + live - 1;
  const int lo_key = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
  // the two rows this thread holds in every accumulator: r0 = lane / 4 and r0 + 8; their ranges of visible keys
  int lo[2], hi[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = (lane >> 2) + 8 * i;
    const int p = HEADS ? pos0 : pos0 + r;
    hi[i] = r < live ? p : -1;
    lo[i] = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
  }

  // Q: float32 rows -> bfloat16 tile (rows past `live` are zero)
  for (int e = threadIdx.x; e < AWM_ROWS * dk; e += blockDim.x) {
    const int r = e / dk, d = e - r * dk;
    float v = 0.f;
    if (r < live) v = HEADS ? q[((size_t)row0 * hq + head0 + r) * dk + d] : q[((size_t)(row0 + r) * hq + head0) * dk + d];
    q_s[r * ks_stride + d] = __float2bfloat16_rn(v);
  }

  float o[DVW / 8][4];
#pragma unroll
  for (int j = 0; j < DVW / 8; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[j][i] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  const int* table = block_table + (size_t)seq * max_pages;
  const int mat = lane >> 3, within = lane & 7, col = 2 * (lane & 3);
  const int k_chunks = dk / 8, v_chunks = (dv + 7) / 8;  // 16-byte pieces of a key row, of a value row
  const int first_tile = lo_key / AWM_KT, last_tile = last_pos / AWM_KT;

#pragma unroll 1
  for (int tile = first_tile + split; tile <= last_tile; tile += splits) {
    const int key0 = tile * AWM_KT;
    __syncthreads();  // the tile before has been read (and Q has been written)
    for (int c = threadIdx.x; c < AWM_KT * k_chunks; c += blockDim.x) {
      const int j = c / k_chunks, piece = c - j * k_chunks;
      const int key = key0 + j;
      bool ok = key >= lo_key && key <= last_pos;
      size_t at = 0;
      if (ok) {
        const int page = table[key / page_size];
        ok = page >= 0 && page < num_pages;
        at = ((size_t)(ok ? page : 0) * hkv + kvh) * page_size + key % page_size;
      }
      ms_cp_async16(k_s + j * ks_stride + piece * 8, k_pages + at * dk + piece * 8, ok);
    }
    if (SEPARATE_V) {
      for (int c = threadIdx.x; c < AWM_KT * (DVP / 8); c += blockDim.x) {
        const int j = c / (DVP / 8), piece = c - j * (DVP / 8);
        const int key = key0 + j;
        bool ok = key >= lo_key && key <= last_pos && piece < v_chunks;
        size_t at = 0;
        if (ok) {
          const int page = table[key / page_size];
          ok = page >= 0 && page < num_pages;
          at = ((size_t)(ok ? page : 0) * hkv + kvh) * page_size + key % page_size;
        }
        ms_cp_async16(v_s + j * VS + piece * 8, v_pages + at * vw + piece * 8, ok);
      }
    }
    ms_cp_async_commit();
    ms_cp_async_wait<0>();
    __syncthreads();

    // S for this warp's 16 keys (rows [16 * warp, 16 * warp + 16) of the tile), over all dk
    float s[2][4];
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) s[n][i] = 0.f;
    const int krow0 = 16 * warp;
#pragma unroll 2
    for (int ks = 0; ks < dk / 16; ++ks) {
      unsigned a[4], b[4];
      ms_ldmatrix_x4(a[0], a[1], a[2], a[3], q_s + (within + 8 * (mat & 1)) * ks_stride + ks * 16 + 8 * (mat >> 1));
      ms_ldmatrix_x4(b[0], b[1], b[2], b[3], k_s + (krow0 + within + 8 * (mat >> 1)) * ks_stride + ks * 16 + 8 * (mat & 1));
      ms_mma_bf16(s[0], a, b[0], b[1]);
      ms_mma_bf16(s[1], a, b[2], b[3]);
    }
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = i >> 1;
        const int key = key0 + krow0 + n * 8 + col + (i & 1);
        const bool ok = key >= lo[r] && key <= hi[r];
        s[n][i] = ok ? s[n][i] * scale_log2 : -INFINITY;
        mx[r] = fmaxf(mx[r], s[n][i]);
      }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    }
    if ((lane & 3) == 0) {
      red[warp * AWM_ROWS + (lane >> 2)] = mx[0];
      red[warp * AWM_ROWS + (lane >> 2) + 8] = mx[1];
    }
    __syncthreads();
    float corr[2], mu[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = (lane >> 2) + 8 * r;
      float t = fmaxf(fmaxf(red[row], red[AWM_ROWS + row]), fmaxf(red[2 * AWM_ROWS + row], red[3 * AWM_ROWS + row]));
      const float m_new = fmaxf(m[r], t);
      mu[r] = m_new == -INFINITY ? 0.f : m_new;  // nothing visible yet: any finite reference works
      corr[r] = ms_exp2(m[r] - mu[r]);            // 0 when the old maximum was -inf
      m[r] = m_new;
      l[r] *= corr[r];
    }
    {
      float p[2][4];
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          p[n][i] = ms_exp2(s[n][i] - mu[i >> 1]);
          l[i >> 1] += p[n][i];  // (this warp's keys only: the warps' sums meet at the end)
        }
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        const int c = krow0 + n * 8 + col;
        *reinterpret_cast<unsigned*>(p_s + (lane >> 2) * PS + c) = ms_pack_bf16(p[n][0], p[n][1]);
        *reinterpret_cast<unsigned*>(p_s + ((lane >> 2) + 8) * PS + c) = ms_pack_bf16(p[n][2], p[n][3]);
      }
    }
    __syncthreads();
    // O += P V for this warp's value columns [warp * DVW, warp * DVW + DVW), over the tile's 64 keys
#pragma unroll
    for (int j = 0; j < DVW / 8; ++j) {
      o[j][0] *= corr[0];
      o[j][1] *= corr[0];
      o[j][2] *= corr[1];
      o[j][3] *= corr[1];
    }
#pragma unroll
    for (int kk = 0; kk < AWM_KT / 16; ++kk) {
      unsigned pa[4];
      ms_ldmatrix_x4(pa[0], pa[1], pa[2], pa[3], p_s + (within + 8 * (mat & 1)) * PS + kk * 16 + 8 * (mat >> 1));
#pragma unroll
      for (int jj = 0; jj < DVW / 16; ++jj) {
        unsigned b[4];
        ms_ldmatrix_x4_trans(b[0], b[1], b[2], b[3],
                             v_s + (kk * 16 + within + 8 * (mat & 1)) * v_stride + warp * DVW + (2 * jj + (mat >> 1)) * 8);
        ms_mma_bf16(o[2 * jj], pa, b[0], b[1]);
        ms_mma_bf16(o[2 * jj + 1], pa, b[2], b[3]);
      }
    }
  }

  // the warps' sums of a row meet
  __syncthreads();
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
  }
  if ((lane & 3) == 0) {
    red[warp * AWM_ROWS + (lane >> 2)] = l[0];
    red[warp * AWM_ROWS + (lane >> 2) + 8] = l[1];
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = (lane >> 2) + 8 * r;
    l[r] = (red[row] + red[AWM_ROWS + row]) + (red[2 * AWM_ROWS + row] + red[3 * AWM_ROWS + row]);
  }

  if (splits > 1) {  // (O, m, l) of this split: [item][split][16][DVP + 2]
    float* mine = scratch + ((size_t)item * splits + split) * AWM_ROWS * (DVP + 2);
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = (lane >> 2) + 8 * r;
      float* dst = mine + (size_t)row * (DVP + 2);
#pragma unroll
      for (int j = 0; j < DVW / 8; ++j) {
        dst[warp * DVW + j * 8 + col] = o[j][2 * r];
        dst[warp * DVW + j * 8 + col + 1] = o[j][2 * r + 1];
      }
      if (warp == 0 && (lane & 3) == 0) {
        dst[DVP] = m[r];
        dst[DVP + 1] = l[r];
      }
    }
    return;
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = (lane >> 2) + 8 * r;
    if (row >= live) continue;
    const int head = HEADS ? head0 + row : head0;
    const int token = HEADS ? row0 : row0 + row;
    float sum = l[r];
    float f = 1.f;
    if (sinks) {  // exp(sink) joins the denominator: against the reference m (or as the reference, if it is larger)
      const float s2 = sinks[head] * MS_LOG2E;
      const float top = fmaxf(m[r], s2);
      f = ms_exp2(m[r] - top);
      sum = sum * f + ms_exp2(s2 - top);
    }
    const float inv = sum > 0.f ? f / sum : 0.f;
    __nv_bfloat16* dst = out + ((size_t)token * hq + head) * dv;
#pragma unroll
    for (int j = 0; j < DVW / 8; ++j) {
      const int d = warp * DVW + j * 8 + col;
      if (d < dv) *reinterpret_cast<unsigned*>(dst + d) = ms_pack_bf16(o[j][2 * r] * inv, o[j][2 * r + 1] * inv);
    }
  }
}

// Merges the splits of the decoding rows in split order and adds the sink: one block per item, a thread per column.
__global__ void attention_wide_mma_merge_kernel(const float* __restrict__ scratch, __nv_bfloat16* __restrict__ out,
                                                const float* __restrict__ sinks, const int* __restrict__ slots,
                                                const int* __restrict__ unit_row0, int hq, int hkv, int dv, int dvp, int splits) {
  ms_pdl_trigger();
  ms_pdl_wait();
  const int groups = hq / hkv;
  const int per_kv = (groups + AWM_ROWS - 1) / AWM_ROWS;
  const int item = blockIdx.x;
  const int unit = item / (hkv * per_kv), rem = item - unit * (hkv * per_kv);
  const int kvh = rem / per_kv, g0 = (rem - kvh * per_kv) * AWM_ROWS;
  const int live = min(AWM_ROWS, groups - g0);
  const int token = unit_row0 ? unit_row0[unit] : unit;
  if (token < 0 || slots[token] < 0) return;
  const float* base = scratch + (size_t)item * splits * AWM_ROWS * (dvp + 2);
  for (int row = 0; row < live; ++row) {
    const int head = kvh * groups + g0 + row;
    float top = sinks ? sinks[head] * MS_LOG2E : -INFINITY;
    for (int s = 0; s < splits; ++s) top = fmaxf(top, base[((size_t)s * AWM_ROWS + row) * (dvp + 2) + dvp]);
    float sum = sinks ? ms_exp2(sinks[head] * MS_LOG2E - top) : 0.f;
    for (int s = 0; s < splits; ++s) {
      const float* p = base + ((size_t)s * AWM_ROWS + row) * (dvp + 2);
      sum += p[dvp + 1] * ms_exp2(p[dvp] - top);
    }
    const float inv = sum > 0.f ? 1.f / sum : 0.f;
    for (int d = threadIdx.x; d < dv; d += blockDim.x) {
      float acc = 0.f;
      for (int s = 0; s < splits; ++s) {
        const float* p = base + ((size_t)s * AWM_ROWS + row) * (dvp + 2);
        acc += p[d] * ms_exp2(p[dvp] - top);
      }
      out[((size_t)token * hq + head) * dv + d] = __float2bfloat16_rn(acc * inv);
    }
  }
}

static size_t awm_smem_bytes(int dk, int dvp, bool separate_v) {
  size_t elems = (size_t)AWM_ROWS * (dk + 8) + (size_t)AWM_KT * (dk + 8) + dvp + (size_t)AWM_ROWS * (AWM_KT + 8);
  if (separate_v) elems += (size_t)AWM_KT * (dvp + 8);
  return elems * 2 + 4 * AWM_ROWS * sizeof(float) + 16;
}

MS_API int ms_attention_wide_mma_supports(int dk, int dv, int vw, int separate_v) {
  if (dk <= 0 || dk % 16 || dv <= 0 || dv % 8 || dv > 512 || vw % 8 || vw < dv) return 0;
  const int dvp = dv <= 64 ? 64 : dv <= 128 ? 128 : dv <= 256 ? 256 : 512;
  return awm_smem_bytes(dk, dvp, separate_v != 0) <= 200 * 1024;
}

// float32 words of scratch memory for `items` items (tokens x key heads x chunks of 16 heads) cut into `splits`
MS_API long long ms_attention_wide_mma_scratch_words(int items, int dv, int splits) {
  const int dvp = dv <= 64 ? 64 : dv <= 128 ? 128 : dv <= 256 ? 256 : 512;
  return splits > 1 ? (long long)items * splits * AWM_ROWS * (dvp + 2) : 0;
}

template <int DVW>
static int awm_launch(bool separate_v, bool heads, unsigned blocks, size_t smem, cudaStream_t stream, const float* q,
                      const __nv_bfloat16* k_pages, const __nv_bfloat16* v_pages, __nv_bfloat16* out, const float* sinks,
                      const int* positions, const int* slots, const int* block_table, int max_pages, int num_pages,
                      const int* unit_row0, const int* unit_rows, int hq, int hkv, int dk, int dv, int vw, int page_size, int window,
                      float scale_log2, int splits, float* scratch) {
#define MS_AWM_GO(SV, H)                                                                                                   \
  do {                                                                                                                     \
    auto kern = attention_wide_mma_kernel<DVW, SV, H>;                                                                     \
    static size_t configured = 0;                                                                                          \
    if (smem > configured) {                                                                                               \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                  \
      MS_REQUIRE(e == cudaSuccess, "attention_wide_mma: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e)); \
      configured = smem;                                                                                                   \
    }                                                                                                                      \
    MS_LAUNCH_RESULT("attention_wide_mma",                                                                                 \
                     ms_launch(kern, dim3(blocks), dim3(AWM_WARPS * 32), smem, stream, 1, true, q, k_pages, v_pages, out, sinks, \
                               positions, slots, block_table, max_pages, num_pages, unit_row0, unit_rows, hq, hkv, dk, dv, vw,    \
                               page_size, window, scale_log2, splits, scratch));                                           \
  } while (0)
  if (separate_v && heads) MS_AWM_GO(true, true);
  else if (separate_v) MS_AWM_GO(true, false);
  else if (heads) MS_AWM_GO(false, true);
  else MS_AWM_GO(false, false);
#undef MS_AWM_GO
  return 0;
}

// q float32 [tokens, hq*dk]; out bfloat16 [tokens, hq*dv]; k pages [pages, hkv, page, dk]; v pages [pages, hkv, page, vw]
// (the same pointer as k_pages for a latent cache: the values are the keys' first dv columns).
// heads == 0: `units` tiles of rows, tile u = rows [unit_row0[u], unit_row0[u] + unit_rows[u]) of one sequence, at most
// 16 each (a tile of no rows does nothing).  heads != 0: `units` decoding rows, row unit_row0[u] (or u, without a list;
// -1: none), each cut into `splits` runs of key tiles; scratch as ms_attention_wide_mma_scratch_words says.
MS_API int ms_attention_wide_mma(const float* q, const void* k_pages, const void* v_pages, void* out, const float* sinks,
                                 const int* positions, const int* slots, const int* block_table, int max_pages, int num_pages,
                                 const int* unit_row0, const int* unit_rows, int units, int heads, int hq, int hkv, int dk, int dv,
                                 int vw, int page_size, int window, float scale, int splits, float* scratch, cudaStream_t stream) {
  if (units == 0) return 0;
  const bool separate_v = k_pages != v_pages;
  MS_REQUIRE(units > 0 && hq > 0 && hkv > 0 && hq % hkv == 0, "attention_wide_mma: bad sizes units=%d hq=%d hkv=%d", units, hq, hkv);
  MS_REQUIRE(ms_attention_wide_mma_supports(dk, dv, vw, separate_v), "attention_wide_mma: widths dk=%d dv=%d (rows of %d) are not covered",
             dk, dv, vw);
  MS_REQUIRE(separate_v || vw == dk, "attention_wide_mma: values inside the keys' plane have the keys' row stride");
  MS_REQUIRE(page_size > 0 && max_pages > 0 && num_pages > 0, "attention_wide_mma: bad cache sizes");
  MS_REQUIRE(heads || (unit_row0 && unit_rows && splits == 1), "attention_wide_mma: tiles of rows need their lists and are not split");
  MS_REQUIRE(splits >= 1 && (splits == 1 || scratch), "attention_wide_mma: %d splits without scratch memory", splits);
  MS_REQUIRE(((uintptr_t)k_pages | (uintptr_t)v_pages) % 16 == 0, "attention_wide_mma: the pages must be 16-byte aligned");
  const int groups = hq / hkv;
  const int dvp = dv <= 64 ? 64 : dv <= 128 ? 128 : dv <= 256 ? 256 : 512;
  const unsigned items = heads ? (unsigned)units * hkv * ((groups + AWM_ROWS - 1) / AWM_ROWS) : (unsigned)units * hq;
  const size_t smem = awm_smem_bytes(dk, dvp, separate_v);
  const float scale_log2 = scale * MS_LOG2E;
#define MS_AWM_ARGS separate_v, heads != 0, items * (unsigned)splits, smem, stream, q, (const __nv_bfloat16*)k_pages,         \
                    (const __nv_bfloat16*)v_pages, (__nv_bfloat16*)out, sinks, positions, slots, block_table, max_pages, num_pages, \
                    unit_row0, unit_rows, hq, hkv, dk, dv, vw, page_size, window, scale_log2, splits, scratch
  int rc;
  if (dvp == 64) rc = awm_launch<16>(MS_AWM_ARGS);
  else if (dvp == 128) rc = awm_launch<32>(MS_AWM_ARGS);
  else if (dvp == 256) rc = awm_launch<64>(MS_AWM_ARGS);
  else rc = awm_launch<128>(MS_AWM_ARGS);
#undef MS_AWM_ARGS
  if (rc) return rc;
  if (splits > 1)
    MS_LAUNCH_RESULT("attention_wide_mma_merge",
                     ms_launch(attention_wide_mma_merge_kernel, dim3(items), dim3(128), 0, stream, 1, true, (const float*)scratch,
                               (__nv_bfloat16*)out, sinks, slots, unit_row0, hq, hkv, dv, dvp, splits));
  return 0;
}
