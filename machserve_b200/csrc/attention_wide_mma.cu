// Tensor-core (mma.sync m16n8k16, bfloat16) paged attention for the mixers of attention_wide.cu: keys and values of
// different widths, values that are the first columns of the keys' own plane (a latent cache), an optional sink per head.
//
// A block of four warps attends 16 * MT query rows: consecutive rows of one sequence with one head (a tile of a prompt's
// portion; MT = 4, 2 or 1 as the value columns leave registers, so that a tile of keys is staged once for up to 64 rows),
// or, HEADS, up to 16 query heads of one token that share a key head (a decoding row: the heads of a group, or all heads
// over a latent cache, fill the tensor core's 16 rows).  Wide values do not fit one warp's registers, so the
// warps divide the work of a tile of 64 keys twice: for S = Q K^T each warp takes its 16 or 8 of the keys (over all dk),
// for O += P V each warp takes its share of the value columns (over all 64 keys); the probabilities cross between the two
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

// NW: warps of a block, 4, or 8 for decoding rows where the values are 256 or more columns wide (half the accumulators
// a warp, twice the warps an SM).  DVW: value columns a warp owns (the block covers NW * DVW >= dv).
// MT: tiles of 16 query rows a block attends.  A warp takes 64 / NW keys of a tile in the score phase.
__device__ __forceinline__ float awm_tanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void awm_ldmatrix_x2(unsigned& r0, unsigned& r1, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(ms_smem_addr(p)));
}

template <int DVW, int MT, int NW, bool SEPARATE_V, bool HEADS>
__global__ void __launch_bounds__(NW * 32)
attention_wide_mma_kernel(const float* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
                          const __nv_bfloat16* __restrict__ v_pages, __nv_bfloat16* __restrict__ out,
                          const float* __restrict__ sinks, const int* __restrict__ positions, const int* __restrict__ slots,
                          const int* __restrict__ block_table, int max_pages, int num_pages, const int* __restrict__ unit_row0,
                          const int* __restrict__ unit_rows, int hq, int hkv, int dk, int dv, int vw, int page_size, int window,
                          float scale_log2, int splits, float* __restrict__ scratch, int stages, MsScoreExtras ex) {
  constexpr int DVP = NW * DVW;
  constexpr int ROWS = AWM_ROWS * MT;
  constexpr int KW = AWM_KT / NW;  // keys of a tile a warp scores: 16 or 8
  constexpr int NS = KW / 8;       // tiles of 8 keys among them
  extern __shared__ __align__(16) unsigned char awm_smem[];
  const int ks_stride = dk + 8;          // elements of a row of the Q and K tiles
  constexpr int VS = DVP + 8;            // elements of a row of a separate V tile
  constexpr int PS = AWM_KT + 8;         // elements of a row of P
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(awm_smem);                 // [16][dk + 8]
  const int k_elems = AWM_KT * ks_stride, v_elems = AWM_KT * VS;                    // elements of a key tile, of a value tile
  __nv_bfloat16* k_ring = q_s + ROWS * ks_stride;                                   // [stages][64][dk + 8] (+ slack: V columns past dk)
  __nv_bfloat16* v_ring = SEPARATE_V ? k_ring + stages * k_elems + DVP : k_ring;    // [stages][64][DVP + 8], or the key tiles
  __nv_bfloat16* p_s = (SEPARATE_V ? v_ring + stages * v_elems : k_ring + stages * k_elems + DVP);  // [ROWS][64 + 8]
  float* red = reinterpret_cast<float*>(p_s + ROWS * PS);                           // [NW][ROWS]
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
  int lo_key = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
  if (ex.chunk > 0) lo_key = max(lo_key, pos0 / ex.chunk * ex.chunk);  // (later rows of the tile begin there or later)
  // the two rows this thread holds in every accumulator of a tile of 16 rows: lane / 4 and lane / 4 + 8; their
  // ranges of visible keys
  int lo[MT][2], hi[MT][2];
#pragma unroll
  for (int t = 0; t < MT; ++t)
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = t * AWM_ROWS + (lane >> 2) + 8 * i;
      const int p = HEADS ? pos0 : pos0 + r;
      hi[t][i] = r < live ? p : -1;
      lo[t][i] = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
      if (ex.chunk > 0) lo[t][i] = max(lo[t][i], p / ex.chunk * ex.chunk);
    }

  const float inv_cap = ex.softcap > 0.f ? 1.f / ex.softcap : 0.f;
  float o[MT][DVW / 8][4];
  float m[MT][2], l[MT][2];
#pragma unroll
  for (int t = 0; t < MT; ++t) {
#pragma unroll
    for (int j = 0; j < DVW / 8; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) o[t][j][i] = 0.f;
    m[t][0] = m[t][1] = -INFINITY;
    l[t][0] = l[t][1] = 0.f;
  }
  const int live_tiles = (live + AWM_ROWS - 1) / AWM_ROWS;  // tiles of 16 rows with a live row

  const int* table = block_table + (size_t)seq * max_pages;
  const int mat = lane >> 3, within = lane & 7, col = 2 * (lane & 3);
  const int k_chunks = dk / 8, v_chunks = (dv + 7) / 8;  // 16-byte pieces of a key row, of a value row
  const int first_tile = lo_key / AWM_KT, last_tile = last_pos / AWM_KT;

  // A tile's copy: two (or four) threads a key row, each its share of the row's 16-byte pieces; one page look-up a thread and tile.
  constexpr int TPR = NW / 2;  // threads a row
  auto request = [&](int tile, int buf) {
    const int j = threadIdx.x / TPR, key = tile * AWM_KT + j;
    bool ok = key >= lo_key && key <= last_pos;
    size_t at = 0;
    if (ok) {
      const int page = table[key / page_size];
      ok = page >= 0 && page < num_pages;
      at = ((size_t)(ok ? page : 0) * hkv + kvh) * page_size + key % page_size;
    }
    __nv_bfloat16* kd = k_ring + buf * k_elems + j * ks_stride;
    const __nv_bfloat16* ksrc = k_pages + at * dk;
    for (int piece = threadIdx.x % TPR; piece < k_chunks; piece += TPR) ms_cp_async16(kd + piece * 8, ksrc + piece * 8, ok);
    if (SEPARATE_V) {
      __nv_bfloat16* vd = v_ring + buf * v_elems + j * VS;
      const __nv_bfloat16* vsrc = v_pages + at * vw;
      for (int piece = threadIdx.x % TPR; piece < DVP / 8; piece += TPR) ms_cp_async16(vd + piece * 8, vsrc + piece * 8, ok && piece < v_chunks);
    }
    ms_cp_async_commit();
  };

  if (first_tile + split <= last_tile) request(first_tile + split, 0);  // (on its way while the queries are brought in)
  // Q: float32 rows -> bfloat16 tile (rows past `live` are zero)
  for (int e = threadIdx.x; e < ROWS * dk; e += blockDim.x) {
    const int r = e / dk, d = e - r * dk;
    float v = 0.f;
    if (r < live) v = HEADS ? q[((size_t)row0 * hq + head0 + r) * dk + d] : q[((size_t)(row0 + r) * hq + head0) * dk + d];
    q_s[r * ks_stride + d] = __float2bfloat16_rn(v);
  }
  __syncthreads();  // Q has been written
  int it = 0;
#pragma unroll 1
  for (int tile = first_tile + split; tile <= last_tile; tile += splits, ++it) {
    const int key0 = tile * AWM_KT;
    const int buf = stages == 2 ? (it & 1) : 0;
    const bool more = tile + splits <= last_tile;
    if (stages == 2 && more) {  // the next tile is on its way while this one is attended
      request(tile + splits, buf ^ 1);
      ms_cp_async_wait<1>();
    } else {
      ms_cp_async_wait<0>();
    }
    __syncthreads();
    const __nv_bfloat16* k_s = k_ring + buf * k_elems;
    const __nv_bfloat16* v_s = SEPARATE_V ? v_ring + buf * v_elems : k_s;

    // S for this warp's KW keys (rows [KW * warp, KW * warp + KW) of the tile), over all dk, for every tile of rows
    float s[MT][NS][4];
#pragma unroll
    for (int t = 0; t < MT; ++t)
#pragma unroll
      for (int n = 0; n < NS; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) s[t][n][i] = 0.f;
    const int krow0 = KW * warp;
#pragma unroll 2
    for (int ks = 0; ks < dk / 16; ++ks) {
      unsigned b[4];
      if (NS == 2)
        ms_ldmatrix_x4(b[0], b[1], b[2], b[3], k_s + (krow0 + within + 8 * (mat >> 1)) * ks_stride + ks * 16 + 8 * (mat & 1));
      else
        awm_ldmatrix_x2(b[0], b[1], k_s + (krow0 + within) * ks_stride + ks * 16 + 8 * (mat & 1));
#pragma unroll
      for (int t = 0; t < MT; ++t) {
        if (t >= live_tiles) continue;
        unsigned a[4];
        ms_ldmatrix_x4(a[0], a[1], a[2], a[3], q_s + (t * AWM_ROWS + within + 8 * (mat & 1)) * ks_stride + ks * 16 + 8 * (mat >> 1));
        ms_mma_bf16(s[t][0], a, b[0], b[1]);
        if (NS == 2) ms_mma_bf16(s[t][NS - 1], a, b[2], b[3]);
      }
    }
#pragma unroll
    for (int t = 0; t < MT; ++t) {
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int n = 0; n < NS; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int r = i >> 1;
          const int key = key0 + krow0 + n * 8 + col + (i & 1);
          const bool ok = key >= lo[t][r] && key <= hi[t][r];
          float sc = -INFINITY;
          if (ok) {
            sc = s[t][n][i] * scale_log2;
            if (ex.softcap > 0.f || ex.dist_bias) {  // back to natural units: the cap and the bias are not scaled
              sc *= 0.6931471805599453f;
              if (ex.softcap > 0.f) sc = ex.softcap * awm_tanh(sc * inv_cap);  // (P is rounded to bfloat16 right after)
              if (ex.dist_bias) {
                const int head = HEADS ? head0 + t * AWM_ROWS + (lane >> 2) + 8 * r : head0;
                sc += ex.dist_bias[(size_t)head * ex.dist_len + min(hi[t][r] - key, ex.dist_len - 1)];
              }
              sc *= MS_LOG2E;
            }
          }
          s[t][n][i] = sc;
          mx[r] = fmaxf(mx[r], s[t][n][i]);
        }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      }
      if ((lane & 3) == 0) {
        red[warp * ROWS + t * AWM_ROWS + (lane >> 2)] = mx[0];
        red[warp * ROWS + t * AWM_ROWS + (lane >> 2) + 8] = mx[1];
      }
    }
    __syncthreads();
    float corr[MT][2];
#pragma unroll
    for (int t = 0; t < MT; ++t) {
      float mu[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int row = t * AWM_ROWS + (lane >> 2) + 8 * r;
        float top = red[row];
#pragma unroll
        for (int w = 1; w < NW; ++w) top = fmaxf(top, red[w * ROWS + row]);
        const float m_new = fmaxf(m[t][r], top);
        mu[r] = m_new == -INFINITY ? 0.f : m_new;  // nothing visible yet: any finite reference works
        corr[t][r] = ms_exp2(m[t][r] - mu[r]);      // 0 when the old maximum was -inf
        m[t][r] = m_new;
        l[t][r] *= corr[t][r];
      }
      float p[NS][4];
#pragma unroll
      for (int n = 0; n < NS; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          p[n][i] = ms_exp2(s[t][n][i] - mu[i >> 1]);
          l[t][i >> 1] += p[n][i];  // (this warp's keys only: the warps' sums meet at the end)
        }
#pragma unroll
      for (int n = 0; n < NS; ++n) {
        const int c = krow0 + n * 8 + col;
        *reinterpret_cast<unsigned*>(p_s + (t * AWM_ROWS + (lane >> 2)) * PS + c) = ms_pack_bf16(p[n][0], p[n][1]);
        *reinterpret_cast<unsigned*>(p_s + (t * AWM_ROWS + (lane >> 2) + 8) * PS + c) = ms_pack_bf16(p[n][2], p[n][3]);
      }
    }
    __syncthreads();
    // O += P V for this warp's value columns [warp * DVW, warp * DVW + DVW), over the tile's 64 keys
#pragma unroll
    for (int t = 0; t < MT; ++t)
#pragma unroll
      for (int j = 0; j < DVW / 8; ++j) {
        o[t][j][0] *= corr[t][0];
        o[t][j][1] *= corr[t][0];
        o[t][j][2] *= corr[t][1];
        o[t][j][3] *= corr[t][1];
      }
#pragma unroll
    for (int kk = 0; kk < AWM_KT / 16; ++kk) {
      unsigned pa[MT][4];
#pragma unroll
      for (int t = 0; t < MT; ++t)
        ms_ldmatrix_x4(pa[t][0], pa[t][1], pa[t][2], pa[t][3],
                       p_s + (t * AWM_ROWS + within + 8 * (mat & 1)) * PS + kk * 16 + 8 * (mat >> 1));
#pragma unroll
      for (int jj = 0; jj < DVW / 16; ++jj) {
        unsigned b[4];
        ms_ldmatrix_x4_trans(b[0], b[1], b[2], b[3],
                             v_s + (kk * 16 + within + 8 * (mat & 1)) * v_stride + warp * DVW + (2 * jj + (mat >> 1)) * 8);
#pragma unroll
        for (int t = 0; t < MT; ++t) {
          if (t >= live_tiles) continue;
          ms_mma_bf16(o[t][2 * jj], pa[t], b[0], b[1]);
          ms_mma_bf16(o[t][2 * jj + 1], pa[t], b[2], b[3]);
        }
      }
    }
    __syncthreads();  // the tile, P and the maxima have been read
    if (stages != 2 && more) request(tile + splits, 0);
  }

  // the warps' sums of a row meet
  __syncthreads();
#pragma unroll
  for (int t = 0; t < MT; ++t) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      l[t][r] += __shfl_xor_sync(0xffffffffu, l[t][r], 1);
      l[t][r] += __shfl_xor_sync(0xffffffffu, l[t][r], 2);
    }
    if ((lane & 3) == 0) {
      red[warp * ROWS + t * AWM_ROWS + (lane >> 2)] = l[t][0];
      red[warp * ROWS + t * AWM_ROWS + (lane >> 2) + 8] = l[t][1];
    }
  }
  __syncthreads();
#pragma unroll
  for (int t = 0; t < MT; ++t)
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = t * AWM_ROWS + (lane >> 2) + 8 * r;
      float sum = red[row];
#pragma unroll
      for (int w = 1; w < NW; ++w) sum += red[w * ROWS + row];  // in warp order
      l[t][r] = sum;
    }

  if (splits > 1) {  // (O, m, l) of this split: [item][split][16][DVP + 2]  (decoding rows: one tile of 16 rows)
    float* mine = scratch + ((size_t)item * splits + split) * AWM_ROWS * (DVP + 2);
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = (lane >> 2) + 8 * r;
      float* dst = mine + (size_t)row * (DVP + 2);
#pragma unroll
      for (int j = 0; j < DVW / 8; ++j) {
        dst[warp * DVW + j * 8 + col] = o[0][j][2 * r];
        dst[warp * DVW + j * 8 + col + 1] = o[0][j][2 * r + 1];
      }
      if (warp == 0 && (lane & 3) == 0) {
        dst[DVP] = m[0][r];
        dst[DVP + 1] = l[0][r];
      }
    }
    return;
  }
#pragma unroll
  for (int t = 0; t < MT; ++t)
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = t * AWM_ROWS + (lane >> 2) + 8 * r;
      if (row >= live) continue;
      const int head = HEADS ? head0 + row : head0;
      const int token = HEADS ? row0 : row0 + row;
      float sum = l[t][r];
      float f = 1.f;
      if (sinks) {  // exp(sink) joins the denominator: against the reference m (or as the reference, if it is larger)
        const float s2 = sinks[head] * MS_LOG2E;
        const float top = fmaxf(m[t][r], s2);
        f = ms_exp2(m[t][r] - top);
        sum = sum * f + ms_exp2(s2 - top);
      }
      const float inv = sum > 0.f ? f / sum : 0.f;
      __nv_bfloat16* dst = out + ((size_t)token * hq + head) * dv;
#pragma unroll
      for (int j = 0; j < DVW / 8; ++j) {
        const int d = warp * DVW + j * 8 + col;
        if (d < dv) *reinterpret_cast<unsigned*>(dst + d) = ms_pack_bf16(o[t][j][2 * r] * inv, o[t][j][2 * r + 1] * inv);
      }
    }
}

// Merges the splits of the decoding rows in split order and adds the sink: one block per (item, row of the item); a warp
// makes the splits' weights once (at most 32 splits), then a thread per value column sums the splits in order.
__global__ void __launch_bounds__(128)
attention_wide_mma_merge_kernel(const float* __restrict__ scratch, __nv_bfloat16* __restrict__ out,
                                const float* __restrict__ sinks, const int* __restrict__ slots,
                                const int* __restrict__ unit_row0, int hq, int hkv, int dv, int dvp, int splits) {
  __shared__ float w_s[36];  // (four zeros behind the 32: the sums below go four splits at a time)
  ms_pdl_trigger();
  ms_pdl_wait();
  const int groups = hq / hkv;
  const int per_kv = (groups + AWM_ROWS - 1) / AWM_ROWS;
  const int item = blockIdx.x / AWM_ROWS, row = blockIdx.x - item * AWM_ROWS;
  const int unit = item / (hkv * per_kv), rem = item - unit * (hkv * per_kv);
  const int kvh = rem / per_kv, g0 = (rem - kvh * per_kv) * AWM_ROWS;
  if (row >= min(AWM_ROWS, groups - g0)) return;
  const int token = unit_row0 ? unit_row0[unit] : unit;
  if (token < 0 || slots[token] < 0) return;
  const int head = kvh * groups + g0 + row;
  const float* base = scratch + ((size_t)item * splits * AWM_ROWS + row) * (dvp + 2);  // split s: + s * 16 * (dvp + 2)
  const size_t step = (size_t)AWM_ROWS * (dvp + 2);
  if (threadIdx.x < 32) {
    const int sp = threadIdx.x;
    const float ms = sp < splits ? base[sp * step + dvp] : -INFINITY;
    const float ls = sp < splits ? base[sp * step + dvp + 1] : 0.f;
    const float s2 = sinks ? sinks[head] * MS_LOG2E : -INFINITY;
    const float top = fmaxf(ms_warp_max(ms), s2);
    const float w = ls > 0.f ? ms_exp2(ms - top) : 0.f;
    float sum = ls * w;
    // (in split order: the sum must not depend on how the shuffles pair the lanes)
    float total = 0.f;
    for (int i = 0; i < splits; ++i) total += __shfl_sync(0xffffffffu, sum, i);
    if (sinks) total += ms_exp2(s2 - top);
    w_s[sp] = total > 0.f ? w / total : 0.f;
    if (sp < 4) w_s[32 + sp] = 0.f;
  }
  __syncthreads();
  for (int d = threadIdx.x; d < dv; d += blockDim.x) {
    float acc = 0.f;
    for (int sp = 0; sp < splits; sp += 4) {  // four loads in flight; added in split order
      float v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = sp + u < splits ? base[(sp + u) * step + d] : 0.f;
#pragma unroll
      for (int u = 0; u < 4; ++u) acc += w_s[sp + u] * v[u];
    }
    out[((size_t)token * hq + head) * dv + d] = __float2bfloat16_rn(acc);
  }
}

static int awm_dvp(int dv) { return dv <= 64 ? 64 : dv <= 128 ? 128 : dv <= 256 ? 256 : 512; }
// tiles of 16 rows a block of four warps attends when the rows are a portion's: as many as leave the value columns their
// registers.  (Decoding rows at 256 or more value columns take blocks of eight warps: measured at latents of 256 and 512,
// 64 rows under a window of 1,024 went from 55, 121 and 158 us to 45, 86 and 114; portions with eight warps and twice the
// rows a block were slower, 795 against 570 us at the smallest: one block of 180 registers a thread per SM.)
static int awm_row_tiles(int dvp) { return dvp <= 128 ? 4 : dvp == 256 ? 2 : 1; }

static size_t awm_smem_bytes(int dk, int dvp, bool separate_v, int rows, int stages = 1) {
  size_t elems = (size_t)rows * (dk + 8) + (size_t)stages * AWM_KT * (dk + 8) + dvp + (size_t)rows * (AWM_KT + 8);
  if (separate_v) elems += (size_t)stages * AWM_KT * (dvp + 8);
  return elems * 2 + 8 * rows * sizeof(float) + 16;
}

MS_API int ms_attention_wide_mma_supports(int dk, int dv, int vw, int separate_v) {
  if (dk <= 0 || dk % 16 || dv <= 0 || dv % 8 || dv > 512 || vw % 8 || vw < dv) return 0;
  const int dvp = awm_dvp(dv);
  return awm_smem_bytes(dk, dvp, separate_v != 0, AWM_ROWS * awm_row_tiles(dvp)) <= 200 * 1024;
}

// rows of a portion that one block attends (the tiles of the work lists have at most this many rows)
MS_API int ms_attention_wide_mma_tile_rows(int dv) { return AWM_ROWS * awm_row_tiles(awm_dvp(dv)); }

// float32 words of scratch memory for `items` items (tokens x key heads x chunks of 16 heads) cut into `splits`
MS_API long long ms_attention_wide_mma_scratch_words(int items, int dv, int splits) {
  return splits > 1 ? (long long)items * splits * AWM_ROWS * (awm_dvp(dv) + 2) : 0;
}

template <int DVW, int MT, int DVW_H, int NW_H>
static int awm_launch(bool separate_v, bool heads, unsigned blocks, size_t smem, cudaStream_t stream, const float* q,
                      const __nv_bfloat16* k_pages, const __nv_bfloat16* v_pages, __nv_bfloat16* out, const float* sinks,
                      const int* positions, const int* slots, const int* block_table, int max_pages, int num_pages,
                      const int* unit_row0, const int* unit_rows, int hq, int hkv, int dk, int dv, int vw, int page_size, int window,
                      float scale_log2, int splits, float* scratch, int stages, MsScoreExtras ex) {
#define MS_AWM_GO(W, M, N, SV, H)                                                                                              \
  do {                                                                                                                     \
    auto kern = attention_wide_mma_kernel<W, M, N, SV, H>;                                                                  \
    static size_t configured = 0;                                                                                          \
    if (smem > configured) {                                                                                               \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                  \
      MS_REQUIRE(e == cudaSuccess, "attention_wide_mma: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e)); \
      configured = smem;                                                                                                   \
    }                                                                                                                      \
    MS_LAUNCH_RESULT("attention_wide_mma",                                                                                 \
                     ms_launch(kern, dim3(blocks), dim3(N * 32), smem, stream, 1, true, q, k_pages, v_pages, out, sinks, \
                               positions, slots, block_table, max_pages, num_pages, unit_row0, unit_rows, hq, hkv, dk, dv, vw,    \
                               page_size, window, scale_log2, splits, scratch, stages, ex));                                \
  } while (0)
  if (separate_v && heads) MS_AWM_GO(DVW_H, 1, NW_H, true, true);
  else if (separate_v) MS_AWM_GO(DVW, MT, 4, true, false);
  else if (heads) MS_AWM_GO(DVW_H, 1, NW_H, false, true);
  else MS_AWM_GO(DVW, MT, 4, false, false);
#undef MS_AWM_GO
  return 0;
}

// q float32 [tokens, hq*dk]; out bfloat16 [tokens, hq*dv]; k pages [pages, hkv, page, dk]; v pages [pages, hkv, page, vw]
// (the same pointer as k_pages for a latent cache: the values are the keys' first dv columns).
// heads == 0: `units` tiles of rows, tile u = rows [unit_row0[u], unit_row0[u] + unit_rows[u]) of one sequence, at most
// ms_attention_wide_mma_tile_rows(dv) each (a tile of no rows does nothing).  heads != 0: `units` decoding rows, row
// unit_row0[u] (or u, without a list; -1: none), each cut into `splits` runs of key tiles; scratch as
// ms_attention_wide_mma_scratch_words says.
static int awm_entry(const float* q, const void* k_pages, const void* v_pages, void* out, const float* sinks,
                     const int* positions, const int* slots, const int* block_table, int max_pages, int num_pages,
                     const int* unit_row0, const int* unit_rows, int units, int heads, int hq, int hkv, int dk, int dv,
                     int vw, int page_size, int window, float scale, int splits, float* scratch, MsScoreExtras ex, cudaStream_t stream) {
  if (units == 0) return 0;
  MS_REQUIRE(ex.dist_bias == nullptr || ex.dist_len > 0, "attention_wide_mma: a distance bias without entries");
  const bool separate_v = k_pages != v_pages;
  MS_REQUIRE(units > 0 && hq > 0 && hkv > 0 && hq % hkv == 0, "attention_wide_mma: bad sizes units=%d hq=%d hkv=%d", units, hq, hkv);
  MS_REQUIRE(ms_attention_wide_mma_supports(dk, dv, vw, separate_v), "attention_wide_mma: widths dk=%d dv=%d (rows of %d) are not covered",
             dk, dv, vw);
  MS_REQUIRE(separate_v || vw == dk, "attention_wide_mma: values inside the keys' plane have the keys' row stride");
  MS_REQUIRE(page_size > 0 && max_pages > 0 && num_pages > 0, "attention_wide_mma: bad cache sizes");
  MS_REQUIRE(heads || (unit_row0 && unit_rows && splits == 1), "attention_wide_mma: tiles of rows need their lists and are not split");
  MS_REQUIRE(splits >= 1 && splits <= 32 && (splits == 1 || scratch), "attention_wide_mma: %d splits (1 to 32, with scratch memory)", splits);
  MS_REQUIRE(((uintptr_t)k_pages | (uintptr_t)v_pages) % 16 == 0, "attention_wide_mma: the pages must be 16-byte aligned");
  const int groups = hq / hkv;
  const int dvp = awm_dvp(dv);
  const unsigned items = heads ? (unsigned)units * hkv * ((groups + AWM_ROWS - 1) / AWM_ROWS) : (unsigned)units * hq;
  const int rows = heads ? AWM_ROWS : AWM_ROWS * awm_row_tiles(dvp);
  // two places for key tiles (the next one is copied while this one is attended) while two blocks still fit an SM
  const int stages = awm_smem_bytes(dk, dvp, separate_v, rows, 2) <= 100 * 1024 ? 2 : 1;
  const size_t smem = awm_smem_bytes(dk, dvp, separate_v, rows, stages);
  const float scale_log2 = scale * MS_LOG2E;
#define MS_AWM_ARGS separate_v, heads != 0, items * (unsigned)splits, smem, stream, q, (const __nv_bfloat16*)k_pages,         \
                    (const __nv_bfloat16*)v_pages, (__nv_bfloat16*)out, sinks, positions, slots, block_table, max_pages, num_pages, \
                    unit_row0, unit_rows, hq, hkv, dk, dv, vw, page_size, window, scale_log2, splits, scratch, stages, ex
  int rc;
  if (dvp == 64) rc = awm_launch<16, 4, 16, 4>(MS_AWM_ARGS);
  else if (dvp == 128) rc = awm_launch<32, 4, 32, 4>(MS_AWM_ARGS);
  else if (dvp == 256) rc = awm_launch<64, 2, 32, 8>(MS_AWM_ARGS);
  else rc = awm_launch<128, 1, 64, 8>(MS_AWM_ARGS);
#undef MS_AWM_ARGS
  if (rc) return rc;
  if (splits > 1)
    MS_LAUNCH_RESULT("attention_wide_mma_merge",
                     ms_launch(attention_wide_mma_merge_kernel, dim3(items * AWM_ROWS), dim3(128), 0, stream, 1, true, (const float*)scratch,
                               (__nv_bfloat16*)out, sinks, slots, unit_row0, hq, hkv, dv, dvp, splits));
  return 0;
}

MS_API int ms_attention_wide_mma(const float* q, const void* k_pages, const void* v_pages, void* out, const float* sinks,
                                 const int* positions, const int* slots, const int* block_table, int max_pages, int num_pages,
                                 const int* unit_row0, const int* unit_rows, int units, int heads, int hq, int hkv, int dk, int dv,
                                 int vw, int page_size, int window, float scale, int splits, float* scratch, cudaStream_t stream) {
  return awm_entry(q, k_pages, v_pages, out, sinks, positions, slots, block_table, max_pages, num_pages, unit_row0, unit_rows, units,
                   heads, hq, hkv, dk, dv, vw, page_size, window, scale, splits, scratch, MsScoreExtras{0.f, nullptr, 0, 0}, stream);
}

// The same with a soft cap, a bias by head and distance, and a mask by chunks (common.cuh, MsScoreExtras).
MS_API int ms_attention_wide_mma_scored(const float* q, const void* k_pages, const void* v_pages, void* out, const float* sinks,
                                        const int* positions, const int* slots, const int* block_table, int max_pages, int num_pages,
                                        const int* unit_row0, const int* unit_rows, int units, int heads, int hq, int hkv, int dk,
                                        int dv, int vw, int page_size, int window, float scale, int splits, float* scratch,
                                        float softcap, const float* dist_bias, int dist_len, int chunk, cudaStream_t stream) {
  return awm_entry(q, k_pages, v_pages, out, sinks, positions, slots, block_table, max_pages, num_pages, unit_row0, unit_rows, units,
                   heads, hq, hkv, dk, dv, vw, page_size, window, scale, splits, scratch,
                   MsScoreExtras{softcap, dist_bias, dist_len, chunk}, stream);
}
