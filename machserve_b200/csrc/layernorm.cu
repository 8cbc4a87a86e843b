// Residual add + layer norm with weight and bias, for one or two norms of the same rows.
//
// y = (x - mean) / sqrt(var + eps) * w + b with var the mean of the squared deviations, all in float32.
// x = residual + (delta_a + delta_b): up to two deltas (a parallel layer hands on its mixer's and its feed-forward's)
// are summed first and then added to the stream.  Without `rows`, x is written back to `residual`.  With `rows`,
// output row i is made from input row rows[i] and nothing is written back.
// Two norms that read the same rows (the two norms of a parallel layer) share mean and variance: with a second
// weight, bias and output the kernel writes both.
// One block per output row; the row is kept in shared memory between the passes (mean, deviations, output), so the
// stream is read once.  The additions of a row happen in an order that depends on d alone.
#include "launch.cuh"

template <typename TO>
__global__ void __launch_bounds__(256)
add_layernorm_kernel(float* __restrict__ residual, const void* __restrict__ delta_a, int a_bf16,
                     const void* __restrict__ delta_b, int b_bf16, const float* __restrict__ w1,
                     const float* __restrict__ b1, TO* __restrict__ out1, const float* __restrict__ w2,
                     const float* __restrict__ b2, TO* __restrict__ out2, const int* __restrict__ rows, int d, float eps) {
  extern __shared__ float row_s[];  // [d]
  __shared__ float scratch[33];
  ms_pdl_trigger();
  ms_pdl_wait();
  const int orow = blockIdx.x;
  const int irow = rows ? rows[orow] : orow;
  float* r = residual + (size_t)irow * d;
  const bool any = delta_a != nullptr || delta_b != nullptr;
  float sum = 0.f;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float v = r[c];
    if (any) {
      float add = 0.f;
      if (delta_a)
        add = a_bf16 ? __bfloat162float(((const __nv_bfloat16*)delta_a)[(size_t)irow * d + c]) : ((const float*)delta_a)[(size_t)irow * d + c];
      if (delta_b)
        add += b_bf16 ? __bfloat162float(((const __nv_bfloat16*)delta_b)[(size_t)irow * d + c]) : ((const float*)delta_b)[(size_t)irow * d + c];
      v += add;
      if (!rows) r[c] = v;
    }
    row_s[c] = v;
    sum += v;
  }
  const float mean = ms_block_sum(sum, scratch) / (float)d;
  float ss = 0.f;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    const float dev = row_s[c] - mean;
    ss += dev * dev;
  }
  const float inv = 1.f / sqrtf(ms_block_sum(ss, scratch) / (float)d + eps);
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    const float n = (row_s[c] - mean) * inv;
    out1[(size_t)orow * d + c] = ms_from_float<TO>(n * w1[c] + b1[c]);
    if (out2) out2[(size_t)orow * d + c] = ms_from_float<TO>(n * w2[c] + b2[c]);
  }
}

// The same for widths that are a multiple of 4 and at most 8192 with 16-byte aligned rows: four elements per thread
// and iteration, the summed row kept in registers between the passes.  The order of a row's additions still
// depends on d (and the block size, which d determines) alone.
#define LN_VEC_THREADS 256
#define LN_VEC_GROUPS 8  // groups of 4 elements a thread keeps: d <= 256 * 8 * 4

__device__ __forceinline__ float4 ln_load4(const void* p, int bf16, size_t i) {
  if (bf16) {
    const uint2 u = *reinterpret_cast<const uint2*>((const __nv_bfloat16*)p + i);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
    const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
    return make_float4(a.x, a.y, b.x, b.y);
  }
  return *reinterpret_cast<const float4*>((const float*)p + i);
}
__device__ __forceinline__ void ln_store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void ln_store4(__nv_bfloat16* p, float4 v) {
  uint2 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
  h[0] = __floats2bfloat162_rn(v.x, v.y);
  h[1] = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = u;
}

template <typename TO>
__global__ void __launch_bounds__(LN_VEC_THREADS)
add_layernorm_vec_kernel(float* __restrict__ residual, const void* __restrict__ delta_a, int a_bf16,
                         const void* __restrict__ delta_b, int b_bf16, const float* __restrict__ w1,
                         const float* __restrict__ b1, TO* __restrict__ out1, const float* __restrict__ w2,
                         const float* __restrict__ b2, TO* __restrict__ out2, const int* __restrict__ rows, int d, float eps) {
  __shared__ float scratch[33];
  ms_pdl_trigger();
  ms_pdl_wait();
  const int orow = blockIdx.x;
  const int irow = rows ? rows[orow] : orow;
  float* r = residual + (size_t)irow * d;
  const int ngroups = d / 4;
  float4 v[LN_VEC_GROUPS];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < LN_VEC_GROUPS; ++i) {
    const int gi = threadIdx.x + i * blockDim.x;
    if (gi < ngroups) {
      v[i] = *reinterpret_cast<const float4*>(r + gi * 4);
      if (delta_a || delta_b) {
        float4 add = make_float4(0.f, 0.f, 0.f, 0.f);
        if (delta_a) add = ln_load4(delta_a, a_bf16, (size_t)irow * d + gi * 4);
        if (delta_b) {
          const float4 o = ln_load4(delta_b, b_bf16, (size_t)irow * d + gi * 4);
          add.x += o.x; add.y += o.y; add.z += o.z; add.w += o.w;
        }
        v[i].x += add.x; v[i].y += add.y; v[i].z += add.z; v[i].w += add.w;
        if (!rows) *reinterpret_cast<float4*>(r + gi * 4) = v[i];
      }
      sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
  }
  const float mean = ms_block_sum(sum, scratch) / (float)d;
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < LN_VEC_GROUPS; ++i) {
    const int gi = threadIdx.x + i * blockDim.x;
    if (gi < ngroups) {
      v[i].x -= mean; v[i].y -= mean; v[i].z -= mean; v[i].w -= mean;
      ss += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
    }
  }
  const float inv = 1.f / sqrtf(ms_block_sum(ss, scratch) / (float)d + eps);
#pragma unroll
  for (int i = 0; i < LN_VEC_GROUPS; ++i) {
    const int gi = threadIdx.x + i * blockDim.x;
    if (gi < ngroups) {
      const float4 n = make_float4(v[i].x * inv, v[i].y * inv, v[i].z * inv, v[i].w * inv);
      const float4 wa = *reinterpret_cast<const float4*>(w1 + gi * 4), ba = *reinterpret_cast<const float4*>(b1 + gi * 4);
      ln_store4(out1 + (size_t)orow * d + gi * 4, make_float4(n.x * wa.x + ba.x, n.y * wa.y + ba.y, n.z * wa.z + ba.z, n.w * wa.w + ba.w));
      if (out2) {
        const float4 wb = *reinterpret_cast<const float4*>(w2 + gi * 4), bb = *reinterpret_cast<const float4*>(b2 + gi * 4);
        ln_store4(out2 + (size_t)orow * d + gi * 4, make_float4(n.x * wb.x + bb.x, n.y * wb.y + bb.y, n.z * wb.z + bb.z, n.w * wb.w + bb.w));
      }
    }
  }
}

MS_API int ms_add_layernorm(float* residual, const void* delta_a, int a_dtype, const void* delta_b, int b_dtype,
                            const float* w1, const float* b1, void* out1, const float* w2, const float* b2, void* out2,
                            int out_dtype, const int* rows, int n_out, int d, float eps, cudaStream_t stream) {
  if (n_out == 0) return 0;
  MS_REQUIRE(n_out > 0 && d > 0 && d <= 12000, "add_layernorm: bad sizes n_out=%d d=%d", n_out, d);
  MS_REQUIRE(w1 && b1 && out1 && (!out2 || (w2 && b2)), "add_layernorm: a norm without weight, bias or output");
  const uintptr_t all = (uintptr_t)residual | (uintptr_t)delta_a | (uintptr_t)delta_b | (uintptr_t)w1 | (uintptr_t)b1 | (uintptr_t)out1 |
                        (uintptr_t)w2 | (uintptr_t)b2 | (uintptr_t)out2;
  if (d % 4 == 0 && d <= 4 * LN_VEC_THREADS * LN_VEC_GROUPS && all % 16 == 0 && (out_dtype == MS_F32 || out_dtype == MS_BF16)) {
    int vt = ((d / 4 + 31) / 32) * 32;  // (a function of d alone)
    vt = vt > LN_VEC_THREADS ? LN_VEC_THREADS : vt;
    if (out_dtype == MS_F32)
      MS_LAUNCH_RESULT("add_layernorm",
                       ms_launch(add_layernorm_vec_kernel<float>, dim3(n_out), dim3(vt), 0, stream, 1, true, residual, delta_a,
                                 (int)(a_dtype == MS_BF16), delta_b, (int)(b_dtype == MS_BF16), w1, b1, (float*)out1, w2, b2,
                                 (float*)out2, rows, d, eps));
    else
      MS_LAUNCH_RESULT("add_layernorm",
                       ms_launch(add_layernorm_vec_kernel<__nv_bfloat16>, dim3(n_out), dim3(vt), 0, stream, 1, true, residual,
                                 delta_a, (int)(a_dtype == MS_BF16), delta_b, (int)(b_dtype == MS_BF16), w1, b1,
                                 (__nv_bfloat16*)out1, w2, b2, (__nv_bfloat16*)out2, rows, d, eps));
    return 0;
  }
  const int threads = d >= 256 ? 256 : ((d + 31) / 32) * 32;
  const size_t smem = (size_t)d * sizeof(float);
  if (out_dtype == MS_F32)
    MS_LAUNCH_RESULT("add_layernorm",
                     ms_launch(add_layernorm_kernel<float>, dim3(n_out), dim3(threads), smem, stream, 1, true, residual, delta_a,
                               (int)(a_dtype == MS_BF16), delta_b, (int)(b_dtype == MS_BF16), w1, b1, (float*)out1, w2, b2,
                               (float*)out2, rows, d, eps));
  else if (out_dtype == MS_BF16)
    MS_LAUNCH_RESULT("add_layernorm",
                     ms_launch(add_layernorm_kernel<__nv_bfloat16>, dim3(n_out), dim3(threads), smem, stream, 1, true, residual,
                               delta_a, (int)(a_dtype == MS_BF16), delta_b, (int)(b_dtype == MS_BF16), w1, b1,
                               (__nv_bfloat16*)out1, w2, b2, (__nv_bfloat16*)out2, rows, d, eps));
  else
    MS_REQUIRE(false, "add_layernorm: unknown out dtype %d", out_dtype);
  return 0;
}

// out[t, 0:d] = residual[t] + (delta_a[t] + delta_b[t]); out[t, d:2d] = other[t]: the two streams side by side, in
// the type a matrix product reads, for a product over both (the entry of a pass of a looped run of layers).
template <typename TO>
__global__ void concat_streams_kernel(const float* __restrict__ residual, const void* __restrict__ delta_a, int a_bf16,
                                      const void* __restrict__ delta_b, int b_bf16, const float* __restrict__ other,
                                      TO* __restrict__ out, int d, size_t total) {
  ms_pdl_trigger();
  ms_pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t t = i / d;
  const int c = (int)(i - t * d);
  float v = residual[i];
  float add = 0.f;
  if (delta_a) add = a_bf16 ? __bfloat162float(((const __nv_bfloat16*)delta_a)[i]) : ((const float*)delta_a)[i];
  if (delta_b) add += b_bf16 ? __bfloat162float(((const __nv_bfloat16*)delta_b)[i]) : ((const float*)delta_b)[i];
  if (delta_a || delta_b) v += add;
  out[t * 2 * d + c] = ms_from_float<TO>(v);
  out[t * 2 * d + d + c] = ms_from_float<TO>(other[i]);
}

MS_API int ms_concat_streams(const float* residual, const void* delta_a, int a_dtype, const void* delta_b, int b_dtype,
                             const float* other, void* out, int out_dtype, int rows, int d, cudaStream_t stream) {
  if (rows == 0) return 0;
  MS_REQUIRE(rows > 0 && d > 0, "concat_streams: bad sizes rows=%d d=%d", rows, d);
  const size_t total = (size_t)rows * d;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (out_dtype == MS_F32)
    MS_LAUNCH_RESULT("concat_streams", ms_launch(concat_streams_kernel<float>, dim3(blocks), dim3(256), 0, stream, 1, true, residual,
                                                 delta_a, (int)(a_dtype == MS_BF16), delta_b, (int)(b_dtype == MS_BF16), other,
                                                 (float*)out, d, total));
  else if (out_dtype == MS_BF16)
    MS_LAUNCH_RESULT("concat_streams", ms_launch(concat_streams_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, 1, true,
                                                 residual, delta_a, (int)(a_dtype == MS_BF16), delta_b, (int)(b_dtype == MS_BF16),
                                                 other, (__nv_bfloat16*)out, d, total));
  else
    MS_REQUIRE(false, "concat_streams: unknown out dtype %d", out_dtype);
  return 0;
}
