// Query/key norm over the whole projection, a query temperature by position, and the write of keys and values
// into their pages: what stands between the q|k|v product and the attention of a mixer that has no rotation.
//
// For every row t of proj [T, ld] = [q (qw) | k (kw) | v (vw)], float32:
//   q' = q / sqrt(mean(q^2) + eps) * wq * temp(p),  temp(p) = 1 + coef * ln(floor((p + 1) / every) + 1)
//   k' = k / sqrt(mean(k^2) + eps) * wk             (the means run over all qw, all kw elements: every head at once)
// q' goes to q_out [T, qw] in float32 (and, rounded, to q_half if that is given); k' and v go to the pages of the row's request at its position, in the
// cache's type.  Keys and values may have different widths per head (dk, dv): k pages are [pages, G, page, dk],
// v pages [pages, G, page, dv].  Rows without a request (slot < 0) are passed over.  With coef == 0 there is no
// temperature.  All arithmetic is float32; the sums of a row happen in an order that depends on the widths alone.
#include "launch.cuh"

template <typename TC, bool VEC>
__global__ void __launch_bounds__(256)
qk_norm_store_kernel(const float* __restrict__ proj, int ld, const float* __restrict__ wq, const float* __restrict__ wk,
                     float eps, float coef, int every, const int* __restrict__ positions, const int* __restrict__ slots,
                     const int* __restrict__ block_table, int max_pages, int num_pages, int page_size,
                     float* __restrict__ q_out, __nv_bfloat16* __restrict__ q_half, TC* __restrict__ k_pages, TC* __restrict__ v_pages, int qw, int groups,
                     int dk, int dv, int store) {
  __shared__ float scratch[33];
  ms_pdl_trigger();
  ms_pdl_wait();
  const int t = blockIdx.x;
  const int slot = slots[t];
  if (slot < 0) return;
  const int pos = positions[t];
  const float* row = proj + (size_t)t * ld;
  const int kw = groups * dk, vw = groups * dv;
  // (four elements at a time where the row, the widths and the weights allow 16-byte accesses; the order of a row's
  // additions depends on the widths and that alignment alone)
  const bool vec = VEC && (qw % 4 == 0) && (kw % 4 == 0);
  float ss = 0.f, sk = 0.f;
  if (vec) {
    for (int c = threadIdx.x * 4; c < qw; c += blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(row + c);
      ss += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
    }
    if (store)
      for (int c = threadIdx.x * 4; c < kw; c += blockDim.x * 4) {
        const float4 v = *reinterpret_cast<const float4*>(row + qw + c);
        sk += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
      }
  } else {
    for (int c = threadIdx.x; c < qw; c += blockDim.x) ss += row[c] * row[c];
    if (store)
      for (int c = threadIdx.x; c < kw; c += blockDim.x) sk += row[qw + c] * row[qw + c];
  }
  const float q_inv = 1.f / sqrtf(ms_block_sum(ss, scratch) / (float)qw + eps);
  const float temp = coef != 0.f ? 1.f + coef * logf((float)((pos + 1) / every + 1)) : 1.f;
  if (vec) {
    for (int c = threadIdx.x * 4; c < qw; c += blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(row + c), w = *reinterpret_cast<const float4*>(wq + c);
      const float4 o = make_float4(v.x * q_inv * w.x * temp, v.y * q_inv * w.y * temp, v.z * q_inv * w.z * temp, v.w * q_inv * w.w * temp);
      *reinterpret_cast<float4*>(q_out + (size_t)t * qw + c) = o;
      if (q_half) {
        uint2 u;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
        h[0] = __floats2bfloat162_rn(o.x, o.y);
        h[1] = __floats2bfloat162_rn(o.z, o.w);
        *reinterpret_cast<uint2*>(q_half + (size_t)t * qw + c) = u;
      }
    }
  } else {
    for (int c = threadIdx.x; c < qw; c += blockDim.x) {
      const float o = row[c] * q_inv * wq[c] * temp;
      q_out[(size_t)t * qw + c] = o;
      if (q_half) q_half[(size_t)t * qw + c] = __float2bfloat16_rn(o);
    }
  }
  if (!store) return;
  const float k_inv = 1.f / sqrtf(ms_block_sum(sk, scratch) / (float)kw + eps);
  const int page = block_table[(size_t)slot * max_pages + pos / page_size];
  if (page < 0 || page >= num_pages) return;
  const size_t at = (size_t)page * groups * page_size + pos % page_size;  // + g * page_size: the row of the (page, head) arrays
  for (int c = threadIdx.x; c < kw; c += blockDim.x) {
    const int g = c / dk, e = c - g * dk;
    k_pages[(at + (size_t)g * page_size) * dk + e] = ms_from_float<TC>(row[qw + c] * k_inv * wk[c]);
  }
  for (int c = threadIdx.x; c < vw; c += blockDim.x) {
    const int g = c / dv, e = c - g * dv;
    v_pages[(at + (size_t)g * page_size) * dv + e] = ms_from_float<TC>(row[qw + kw + c]);
  }
}

MS_API int ms_qk_norm_store(const float* proj, int ld, const float* wq, const float* wk, float eps, float coef, int every,
                            const int* positions, const int* slots, const int* block_table, int max_pages, int num_pages,
                            int page_size, float* q_out, void* q_half, void* k_pages, void* v_pages, int cache_dtype, int tokens, int qw,
                            int groups, int dk, int dv, int store, cudaStream_t stream) {
  if (tokens == 0) return 0;
  MS_REQUIRE(tokens > 0 && qw > 0 && groups > 0 && dk > 0 && dv > 0 && every > 0, "qk_norm_store: bad sizes");
  MS_REQUIRE(ld >= qw + (store ? groups * (dk + dv) : 0), "qk_norm_store: rows of %d elements do not hold q, k and v", ld);
  MS_REQUIRE(!store || (max_pages > 0 && num_pages > 0 && page_size > 0 && k_pages && v_pages), "qk_norm_store: no cache to write");
  const bool vec = ld % 4 == 0 && ((uintptr_t)proj | (uintptr_t)wq | (uintptr_t)q_out) % 16 == 0;
#define MS_QKN(TC, V)                                                                                                      \
  MS_LAUNCH_RESULT("qk_norm_store", ms_launch(qk_norm_store_kernel<TC, V>, dim3(tokens), dim3(256), 0, stream, 1, true, proj, ld, wq, \
                                              wk, eps, coef, every, positions, slots, block_table, max_pages, num_pages, page_size,  \
                                              q_out, (__nv_bfloat16*)q_half, (TC*)k_pages, (TC*)v_pages, qw, groups, dk, dv, store))
  if (cache_dtype == MS_F32) {
    if (vec) MS_QKN(float, true); else MS_QKN(float, false);
  } else if (cache_dtype == MS_BF16) {
    if (vec) MS_QKN(__nv_bfloat16, true); else MS_QKN(__nv_bfloat16, false);
  } else {
    MS_REQUIRE(false, "qk_norm_store: unknown cache dtype %d", cache_dtype);
  }
#undef MS_QKN
  return 0;
}
