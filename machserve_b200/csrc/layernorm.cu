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

MS_API int ms_add_layernorm(float* residual, const void* delta_a, int a_dtype, const void* delta_b, int b_dtype,
                            const float* w1, const float* b1, void* out1, const float* w2, const float* b2, void* out2,
                            int out_dtype, const int* rows, int n_out, int d, float eps, cudaStream_t stream) {
  if (n_out == 0) return 0;
  MS_REQUIRE(n_out > 0 && d > 0 && d <= 12000, "add_layernorm: bad sizes n_out=%d d=%d", n_out, d);
  MS_REQUIRE(w1 && b1 && out1 && (!out2 || (w2 && b2)), "add_layernorm: a norm without weight, bias or output");
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
