// Exact paged attention for mixers whose keys and values differ in width, whose softmax has a sink, or whose values
// are a column range of the keys' own plane (a latent cache): float32 queries, float32 or bfloat16 cache.
//
//   score(i, j) = scale * q_i . k_j over dk coordinates, for the keys j in [max(0, p_i - window + 1), p_i]
//   weight(i, j) = exp(score - m) / (sum_j exp(score - m) + exp(sink_h - m))      (the sink term only when sinks are given;
//                                                                                  it has no value and is not scaled)
//   out_i = sum_j weight(i, j) * v_j[0:dv]
// k pages are [pages, hkv, page, dk]; v pages are [pages, hkv, page, vw] with vw >= dv (vw = dk and the same pointer for
// a latent cache whose values are the first dv coordinates of its keys).  Any dk; dv up to 512.
//
// The arithmetic of a row depends on its position alone, as in the exact kernel for equal widths: the keys are cut into
// tiles of 32 at absolute multiples of 32, warp w of W takes the tiles first + w, first + w + W, ... in ascending order
// with an online softmax, and the W partial results are merged in warp order.  R rows share a block and every tile it
// stages: R consecutive rows of the step with one head (portions of prompts; rows of one sequence whose ranges of keys
// begin in the same tile go through the tiles together), or, HEADS, up to R query heads of one token that share a key
// head (decoding).  A row's result is the same bits in either form and beside any other rows.
// Keys are staged in shared memory 64 coordinates at a time (a lane then owns one key of the tile); values are read
// as they lie, a few keys at a time, each value serving all R rows.
#include "common.cuh"

#define AW_KC 64

template <typename TC, int W, int NACC, int R, bool HEADS>
__global__ void __launch_bounds__(W * 32)
attention_wide_kernel(const float* __restrict__ q, const TC* __restrict__ k_pages, const TC* __restrict__ v_pages,
                      TC* __restrict__ out, const float* __restrict__ sinks, const int* __restrict__ positions,
                      const int* __restrict__ slots, const int* __restrict__ block_table, int max_pages, int num_pages,
                      int tokens, int hq, int hkv, int dk, int dv, int vw, int page_size, int window, float scale, MsScoreExtras ex) {
  extern __shared__ __align__(16) float aw_smem[];
  float* q_s = aw_smem;                                  // [R][dk]
  float* k_all = q_s + (size_t)R * dk;                   // [W][32][AW_KC + 1]
  float* part = k_all + (size_t)W * 32 * (AW_KC + 1);    // [W][R][dv + 2]
  const int groups = hq / hkv;
  int tok0, tok_step, head0, head_step, live_rows, kvh;
  if (HEADS) {
    const int per_kv = (groups + R - 1) / R;
    const int t = blockIdx.x / (hkv * per_kv), rem = blockIdx.x - t * (hkv * per_kv);
    kvh = rem / per_kv;
    const int g0 = (rem - kvh * per_kv) * R;
    tok0 = t; tok_step = 0; head0 = kvh * groups + g0; head_step = 1;
    live_rows = min(R, groups - g0);
  } else {
    const int group = blockIdx.x / hq, h = blockIdx.x - group * hq;
    kvh = h / groups;
    tok0 = group * R; tok_step = 1; head0 = h; head_step = 0;
    live_rows = min(R, tokens - tok0);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* my_k = k_all + (size_t)warp * 32 * (AW_KC + 1);

  int seq[R], pos[R], first[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    seq[r] = r < live_rows ? slots[tok0 + r * tok_step] : -1;
    pos[r] = seq[r] >= 0 ? positions[tok0 + r * tok_step] : -1;
    first[r] = (window > 0 && pos[r] - window + 1 > 0) ? pos[r] - window + 1 : 0;
    if (ex.chunk > 0 && pos[r] >= 0) first[r] = max(first[r], pos[r] / ex.chunk * ex.chunk);
  }
  for (int e = threadIdx.x; e < R * dk; e += blockDim.x) {
    const int r = e / dk, d = e - r * dk;
    q_s[e] = r < live_rows ? q[((size_t)(tok0 + r * tok_step) * hq + head0 + r * head_step) * dk + d] : 0.f;
  }
  __syncthreads();

  float m[R], l[R], acc[R][NACC];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    m[r] = -INFINITY;
    l[r] = 0.f;
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[r][i] = 0.f;
  }

  // runs of rows that share their tiles: the same sequence and the same first tile
  unsigned done = 0;
#pragma unroll 1
  for (int lead = 0; lead < R; ++lead) {
    if ((done >> lead) & 1u) continue;
    int lead_seq = -1, lead_tile = 0;
#pragma unroll
    for (int r = 0; r < R; ++r)
      if (r == lead) {
        lead_seq = seq[r];
        lead_tile = first[r] / 32;
      }
    unsigned run = 0;
    int lo_key = 0x7fffffff, hi_pos = -1;
#pragma unroll
    for (int r = 0; r < R; ++r)
      if (r >= lead && seq[r] == lead_seq && first[r] / 32 == lead_tile && !((done >> r) & 1u)) {
        run |= 1u << r;
        lo_key = min(lo_key, first[r]);
        hi_pos = max(hi_pos, pos[r]);
      }
    done |= run;
    if (lead_seq < 0) continue;  // rows without a request
    const int* table = block_table + (size_t)lead_seq * max_pages;
#pragma unroll 1
    for (int tile = lead_tile + warp; tile * 32 <= hi_pos; tile += W) {
      const int key = tile * 32 + lane;
      long long base = -1;  // this lane's key: its row in the [page][head][slot] arrays
      if (key >= lo_key && key <= hi_pos) {
        const int page = table[key / page_size];
        if (page >= 0 && page < num_pages) base = (long long)(((size_t)page * hkv + kvh) * page_size + key % page_size);
      }
      float dot[R];
#pragma unroll
      for (int r = 0; r < R; ++r) dot[r] = 0.f;
#pragma unroll 1
      for (int d0 = 0; d0 < dk; d0 += AW_KC) {
        const int clen = min(AW_KC, dk - d0);
        __syncwarp();  // the piece before has been read
        for (int j0 = 0; j0 < 32; j0 += 8) {
          long long b[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) b[u] = __shfl_sync(0xffffffffu, base, j0 + u);
          for (int d = lane; d < clen; d += 32) {
            float kv[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) kv[u] = b[u] >= 0 ? ms_to_float(k_pages[(size_t)b[u] * dk + d0 + d]) : 0.f;
#pragma unroll
            for (int u = 0; u < 8; ++u) my_k[(j0 + u) * (AW_KC + 1) + d] = kv[u];
          }
        }
        __syncwarp();
        const float* kr = my_k + lane * (AW_KC + 1);
        const float* qd = q_s + d0;
        // each row's own chain of sums, coordinate by coordinate in ascending order
        if ((dk & 3) == 0) {
          for (int d = 0; d < clen; d += 4) {
            const float k0 = kr[d], k1 = kr[d + 1], k2 = kr[d + 2], k3 = kr[d + 3];
#pragma unroll
            for (int r = 0; r < R; ++r) {
              const float4 qv = *reinterpret_cast<const float4*>(qd + r * dk + d);
              dot[r] = fmaf(qv.x, k0, dot[r]);
              dot[r] = fmaf(qv.y, k1, dot[r]);
              dot[r] = fmaf(qv.z, k2, dot[r]);
              dot[r] = fmaf(qv.w, k3, dot[r]);
            }
          }
        } else {
          for (int d = 0; d < clen; ++d) {
            const float kd = kr[d];
#pragma unroll
            for (int r = 0; r < R; ++r) dot[r] = fmaf(qd[r * dk + d], kd, dot[r]);
          }
        }
      }
      float pr[R];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        pr[r] = 0.f;
        if (!((run >> r) & 1u) || tile * 32 > pos[r]) continue;  // (the same for the whole warp)
        const bool valid = base >= 0 && key >= first[r] && key <= pos[r];
        float sc = -INFINITY;
        if (valid) {
          sc = dot[r] * scale;
          if (ex.softcap > 0.f) sc = ex.softcap * tanhf(sc / ex.softcap);
          if (ex.dist_bias) sc += ex.dist_bias[(size_t)(head0 + r * head_step) * ex.dist_len + min(pos[r] - key, ex.dist_len - 1)];
        }
        const float tile_max = ms_warp_max(sc);
        const float m_new = fmaxf(m[r], tile_max);
        pr[r] = (valid && m_new > -INFINITY) ? expf(sc - m_new) : 0.f;
        const float corr = (m[r] == -INFINITY) ? 0.f : expf(m[r] - m_new);
        l[r] = l[r] * corr + ms_warp_sum(pr[r]);
#pragma unroll
        for (int i = 0; i < NACC; ++i) acc[r][i] *= corr;
        m[r] = m_new;
      }
      // the values key by key in ascending order; a value serves all rows (a row that does not see the key has weight 0)
      constexpr int U = NACC <= 4 ? 8 : (NACC <= 8 ? 4 : 2);
      for (int j0 = 0; j0 < 32; j0 += U) {
        long long b[U];
        float vj[U][NACC];
#pragma unroll
        for (int u = 0; u < U; ++u) b[u] = __shfl_sync(0xffffffffu, base, j0 + u);
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
          for (int i = 0; i < NACC; ++i) {
            const int d = lane + 32 * i;
            vj[u][i] = (b[u] >= 0 && d < dv) ? ms_to_float(v_pages[(size_t)b[u] * vw + d]) : 0.f;
          }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (b[u] < 0) continue;  // (the same for the whole warp)
#pragma unroll
          for (int r = 0; r < R; ++r) {
            const float pj = __shfl_sync(0xffffffffu, pr[r], j0 + u);
#pragma unroll
            for (int i = 0; i < NACC; ++i) acc[r][i] = fmaf(pj, vj[u][i], acc[r][i]);
          }
        }
      }
    }
  }

  // every row's partial results of all warps, then warp r merges row r (and r + W, ...) in warp order
  const int pw = dv + 2;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    float* p = part + ((size_t)warp * R + r) * pw;
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
      const int d = lane + 32 * i;
      if (d < dv) p[d] = acc[r][i];
    }
    if (lane == 0) {
      p[dv] = m[r];
      p[dv + 1] = l[r];
    }
  }
  __syncthreads();
  for (int r = warp; r < R; r += W) {
    const int t = tok0 + r * tok_step, h = head0 + r * head_step;
    if (r >= live_rows || slots[t] < 0) continue;
    const bool has_sink = sinks != nullptr;
    const float sink = has_sink ? sinks[h] : -INFINITY;
    float mm = sink;
    for (int w = 0; w < W; ++w) mm = fmaxf(mm, part[((size_t)w * R + r) * pw + dv]);
    float f[W], ll = 0.f;
    for (int w = 0; w < W; ++w) {
      const float* p = part + ((size_t)w * R + r) * pw;
      f[w] = p[dv + 1] > 0.f ? expf(p[dv] - mm) : 0.f;
      ll += p[dv + 1] * f[w];
    }
    if (has_sink) ll += expf(sink - mm);
    const float inv = ll > 0.f ? 1.f / ll : 0.f;
    for (int d = lane; d < dv; d += 32) {
      float o = 0.f;
      for (int w = 0; w < W; ++w) o += part[((size_t)w * R + r) * pw + d] * f[w];
      out[((size_t)t * hq + h) * dv + d] = ms_from_float<TC>(o * inv);
    }
  }
}

template <typename TC, int W, int NACC, int R, bool HEADS>
static int launch_attention_wide_form(const float* q, const void* k_pages, const void* v_pages, void* out, const float* sinks,
                                      const int* positions, const int* slots, const int* block_table, int max_pages, int num_pages,
                                      int tokens, int hq, int hkv, int dk, int dv, int vw, int page_size, int window, float scale,
                                      MsScoreExtras ex, cudaStream_t stream) {
  const int groups = hq / hkv;
  const size_t smem = ((size_t)R * dk + (size_t)W * 32 * (AW_KC + 1) + (size_t)W * R * (dv + 2)) * sizeof(float);
  MS_REQUIRE(smem <= 200 * 1024, "attention_wide: keys of %d coordinates need %zu bytes of shared memory", dk, smem);
  const unsigned blocks = HEADS ? (unsigned)tokens * (unsigned)hkv * (unsigned)((groups + R - 1) / R)
                                : (unsigned)((tokens + R - 1) / R) * (unsigned)hq;
  auto kern = attention_wide_kernel<TC, W, NACC, R, HEADS>;
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    MS_REQUIRE(e == cudaSuccess, "attention_wide: cannot get shared memory: %s", cudaGetErrorString(e));
    configured = smem;
  }
  kern<<<blocks, W * 32, smem, stream>>>(q, (const TC*)k_pages, (const TC*)v_pages, (TC*)out, sinks, positions, slots, block_table,
                                         max_pages, num_pages, tokens, hq, hkv, dk, dv, vw, page_size, window, scale, ex);
  MS_LAUNCH_CHECK("attention_wide");
  return 0;
}

// Rows of portions: R consecutive rows a block.  Rows alone in their sequences: the heads of a group share a block, R of
// them, or, when that would leave most SMs without a block (few rows, few key heads), every head gets a block of its
// own: a row's arithmetic is the same in every form, so the choice changes no bit of the result.
template <typename TC, int W, int NACC, int R>
static int launch_attention_wide(const float* q, const void* k_pages, const void* v_pages, void* out, const float* sinks,
                                 const int* positions, const int* slots, const int* block_table, int max_pages, int num_pages,
                                 int tokens, int hq, int hkv, int dk, int dv, int vw, int page_size, int window, float scale,
                                 MsScoreExtras ex, bool heads, cudaStream_t stream) {
#define MS_AW_ARGS q, k_pages, v_pages, out, sinks, positions, slots, block_table, max_pages, num_pages, tokens, hq, hkv, dk, dv, vw, \
                   page_size, window, scale, ex, stream
  if (!heads) return launch_attention_wide_form<TC, W, NACC, R, false>(MS_AW_ARGS);
  const int groups = hq / hkv;
  int sms = 148;
  {
    static int cached = 0;
    if (!cached) {
      int dev = 0;
      if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&cached, cudaDevAttrMultiProcessorCount, dev);
      if (cached <= 0) cached = 148;
    }
    sms = cached;
  }
  if (groups > 1 && (long long)tokens * hkv * ((groups + R - 1) / R) < 2LL * sms)
    return launch_attention_wide_form<TC, W, NACC, 1, true>(MS_AW_ARGS);
  return launch_attention_wide_form<TC, W, NACC, R, true>(MS_AW_ARGS);
#undef MS_AW_ARGS
}

// q [tokens, hq*dk] float32; out [tokens, hq*dv] in the cache's type.  window <= 0: every earlier key is visible.
// share_rows: the step has rows that follow one another in a sequence, and R consecutive rows share a block; else the
// query heads of a token that share a key head do.  sinks: float32 [hq] or null.
static int attention_wide_entry(const float* q, const void* k_pages, const void* v_pages, void* out, int cache_dtype,
                                const float* sinks, const int* positions, const int* slots, const int* block_table, int max_pages,
                                int num_pages, int tokens, int hq, int hkv, int dk, int dv, int vw, int page_size, int window,
                                float scale, MsScoreExtras ex, int share_rows, cudaStream_t stream) {
  if (tokens == 0) return 0;
  MS_REQUIRE(ex.dist_bias == nullptr || ex.dist_len > 0, "attention_wide: a distance bias without entries");
  MS_REQUIRE(tokens > 0 && hq > 0 && hkv > 0 && hq % hkv == 0, "attention_wide: bad head counts hq=%d hkv=%d", hq, hkv);
  MS_REQUIRE(dk > 0 && dv > 0 && dv <= 512 && vw >= dv, "attention_wide: widths dk=%d dv=%d (of %d) are not covered", dk, dv, vw);
  MS_REQUIRE(page_size > 0 && max_pages > 0 && num_pages > 0, "attention_wide: bad cache sizes");
  const bool heads = !(share_rows && tokens > 1);
#define MS_AW_CASE(TC)                                                                                                  \
  do {                                                                                                                  \
    if (dv <= 64)                                                                                                       \
      return launch_attention_wide<TC, 8, 2, 8>(q, k_pages, v_pages, out, sinks, positions, slots, block_table, max_pages, num_pages, \
                                                tokens, hq, hkv, dk, dv, vw, page_size, window, scale, ex, heads, stream);          \
    if (dv <= 128)                                                                                                      \
      return launch_attention_wide<TC, 4, 4, 8>(q, k_pages, v_pages, out, sinks, positions, slots, block_table, max_pages, num_pages, \
                                                tokens, hq, hkv, dk, dv, vw, page_size, window, scale, ex, heads, stream);          \
    if (dv <= 256)                                                                                                      \
      return launch_attention_wide<TC, 4, 8, 4>(q, k_pages, v_pages, out, sinks, positions, slots, block_table, max_pages, num_pages, \
                                                tokens, hq, hkv, dk, dv, vw, page_size, window, scale, ex, heads, stream);          \
    return launch_attention_wide<TC, 4, 16, 2>(q, k_pages, v_pages, out, sinks, positions, slots, block_table, max_pages, num_pages, \
                                               tokens, hq, hkv, dk, dv, vw, page_size, window, scale, ex, heads, stream);           \
  } while (0)
  if (cache_dtype == MS_F32)
    MS_AW_CASE(float);
  else if (cache_dtype == MS_BF16)
    MS_AW_CASE(__nv_bfloat16);
#undef MS_AW_CASE
  MS_REQUIRE(false, "attention_wide: unknown cache dtype %d", cache_dtype);
  return 0;
}

MS_API int ms_attention_wide(const float* q, const void* k_pages, const void* v_pages, void* out, int cache_dtype,
                             const float* sinks, const int* positions, const int* slots, const int* block_table, int max_pages,
                             int num_pages, int tokens, int hq, int hkv, int dk, int dv, int vw, int page_size, int window,
                             float scale, int share_rows, cudaStream_t stream) {
  return attention_wide_entry(q, k_pages, v_pages, out, cache_dtype, sinks, positions, slots, block_table, max_pages, num_pages, tokens,
                              hq, hkv, dk, dv, vw, page_size, window, scale, MsScoreExtras{0.f, nullptr, 0, 0}, share_rows, stream);
}

// The same with what may come between the scaled score and the softmax (common.cuh, MsScoreExtras): a soft cap
// softcap * tanh(score / softcap), a learned bias by head and distance dist_bias[h][min(i - j, dist_len - 1)] (float32
// [hq, dist_len], not scaled), and a mask by chunks: position i sees the keys j <= i of its own chunk floor(i / chunk) only.
MS_API int ms_attention_wide_scored(const float* q, const void* k_pages, const void* v_pages, void* out, int cache_dtype,
                                    const float* sinks, const int* positions, const int* slots, const int* block_table, int max_pages,
                                    int num_pages, int tokens, int hq, int hkv, int dk, int dv, int vw, int page_size, int window,
                                    float scale, float softcap, const float* dist_bias, int dist_len, int chunk, int share_rows,
                                    cudaStream_t stream) {
  return attention_wide_entry(q, k_pages, v_pages, out, cache_dtype, sinks, positions, slots, block_table, max_pages, num_pages, tokens,
                              hq, hkv, dk, dv, vw, page_size, window, scale, MsScoreExtras{softcap, dist_bias, dist_len, chunk}, share_rows,
                              stream);
}
