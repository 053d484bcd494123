// Element-wise kernels around the float32 residual stream for blocks that norm a branch's OUTPUT:
//   token shift   y_t = x_t + (x_{t-1} - x_t) * mu, the previous row of a request's first token coming from
//                 (and its last row going to) per-request state;
//   norm-and-add  h += y / sqrt(mean(y^2) + eps) * w;
//   soft cap      z = cap * tanh(z / cap);
//   tanh of a column slice.
// Statistics, the mix and the sum are float32; only what feeds a matrix product is rounded.
#include "common.cuh"

// ---------------------------------------------------------------------------------
// Token shift. One block per token. `mu` == nullptr: a plain conversion of x to TA.
// The block of a request's FIRST token of the step reads the request's state row (the last row of the
// step before, zeros after admission) and then replaces it by the request's LAST row of this step: the
// same thread reads and writes a column, so no other block touches the row meanwhile.
// ---------------------------------------------------------------------------------
template <typename TA>
__global__ void token_shift_kernel(const float* __restrict__ x, const float* __restrict__ mu,
                                   float* __restrict__ state, const int* __restrict__ token_req,
                                   const int* __restrict__ q_start, const int* __restrict__ n_new,
                                   const int* __restrict__ slot_ids, TA* __restrict__ out, int width) {
  const int t = blockIdx.x;
  const float* xr = x + (size_t)t * width;
  TA* o = out + (size_t)t * width;
  if (mu == nullptr) {
    for (int c = threadIdx.x; c < width; c += blockDim.x) o[c] = from_float<TA>(xr[c]);
    return;
  }
  const int r = token_req[t];
  const int first = q_start[r];
  if (t != first) {
    const float* pr = xr - width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
      const float v = xr[c];
      o[c] = from_float<TA>(v + (pr[c] - v) * mu[c]);
    }
    return;
  }
  float* st = state + (size_t)slot_ids[r] * width;
  const float* last = x + (size_t)(first + n_new[r] - 1) * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = xr[c], p = st[c];
    o[c] = from_float<TA>(v + (p - v) * mu[c]);
    st[c] = last[c];
  }
}

LLMRS_API int llmrs_token_shift(const float* x, const float* mu, float* state, const int* token_req,
                                const int* q_start, const int* n_new, const int* slot_ids, void* out,
                                int out_dtype, int n_tokens, int width, cudaStream_t stream) {
  LLMRS_REQUIRE(n_tokens >= 0 && width > 0, "token_shift: bad sizes");
  LLMRS_REQUIRE(mu == nullptr || (state && token_req && q_start && n_new && slot_ids),
                "token_shift: a shift needs the state and the step's index arrays");
  if (n_tokens == 0) return 0;
  const int threads = width >= 1024 ? 256 : 128;
  if (out_dtype == LLMRS_F32)
    token_shift_kernel<float><<<n_tokens, threads, 0, stream>>>(x, mu, state, token_req, q_start, n_new, slot_ids,
                                                                 (float*)out, width);
  else if (out_dtype == LLMRS_BF16)
    token_shift_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(x, mu, state, token_req, q_start, n_new,
                                                                         slot_ids, (__nv_bfloat16*)out, width);
  else
    return llmrs_fail("token_shift: unknown dtype %d", out_dtype);
  return llmrs_launch_status("token_shift");
}

// ---------------------------------------------------------------------------------
// h[t] += y[t] / sqrt(mean(y[t]^2) + eps) * w. One block per row; y is read twice (the second time
// from the L1/L2). `w` is the factor itself (a weight stored around zero has had its 1 added at load).
// ---------------------------------------------------------------------------------
template <typename TY>
__global__ void outnorm_add_kernel(float* __restrict__ h, const TY* __restrict__ y, const float* __restrict__ w,
                                   int width, float eps) {
  __shared__ float red[33];
  const TY* yr = y + (size_t)blockIdx.x * width;
  float* hr = h + (size_t)blockIdx.x * width;
  float ss = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = to_float(yr[c]);
    ss += v * v;
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x) hr[c] += to_float(yr[c]) * inv * w[c];
}

LLMRS_API int llmrs_outnorm_add(float* h, const void* y, int y_dtype, const float* w, int n_rows, int width,
                                float eps, cudaStream_t stream) {
  LLMRS_REQUIRE(n_rows >= 0 && width > 0, "outnorm_add: bad sizes");
  if (n_rows == 0) return 0;
  const int threads = width >= 1024 ? 256 : 128;
  if (y_dtype == LLMRS_F32)
    outnorm_add_kernel<float><<<n_rows, threads, 0, stream>>>(h, (const float*)y, w, width, eps);
  else if (y_dtype == LLMRS_BF16)
    outnorm_add_kernel<__nv_bfloat16><<<n_rows, threads, 0, stream>>>(h, (const __nv_bfloat16*)y, w, width, eps);
  else
    return llmrs_fail("outnorm_add: unknown dtype %d", y_dtype);
  return llmrs_launch_status("outnorm_add");
}

// ---------------------------------------------------------------------------------
// z = cap * tanh(z / cap), in place, float32.
// ---------------------------------------------------------------------------------
__global__ void softcap_kernel(float* __restrict__ z, long long n, float cap) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) z[i] = cap * tanhf(z[i] / cap);
}

LLMRS_API int llmrs_softcap(float* z, long long n, float cap, cudaStream_t stream) {
  LLMRS_REQUIRE(n >= 0 && cap > 0.f, "softcap: bad arguments");
  if (n == 0) return 0;
  softcap_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(z, n, cap);
  return llmrs_launch_status("softcap");
}

// ---------------------------------------------------------------------------------
// out[t, c] = tanh(in[t, c]) for c < cols, `in` with a row stride (a slice of a wider product).
// ---------------------------------------------------------------------------------
template <typename TI, typename TO>
__global__ void tanh_slice_kernel(const TI* __restrict__ in, long long in_stride, TO* __restrict__ out, int rows,
                                  int cols) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)rows * cols) return;
  const int t = (int)(i / cols), c = (int)(i % cols);
  out[i] = from_float<TO>(tanhf(to_float(in[(size_t)t * in_stride + c])));
}

LLMRS_API int llmrs_tanh_slice(const void* in, int in_dtype, long long in_stride, void* out, int out_dtype, int rows,
                               int cols, cudaStream_t stream) {
  LLMRS_REQUIRE(rows >= 0 && cols > 0, "tanh_slice: bad sizes");
  if (rows == 0) return 0;
  const unsigned grid = (unsigned)(((long long)rows * cols + 255) / 256);
  if (in_dtype == LLMRS_F32 && out_dtype == LLMRS_F32)
    tanh_slice_kernel<float, float><<<grid, 256, 0, stream>>>((const float*)in, in_stride, (float*)out, rows, cols);
  else if (in_dtype == LLMRS_BF16 && out_dtype == LLMRS_BF16)
    tanh_slice_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, stream>>>(
        (const __nv_bfloat16*)in, in_stride, (__nv_bfloat16*)out, rows, cols);
  else if (in_dtype == LLMRS_F32 && out_dtype == LLMRS_BF16)
    tanh_slice_kernel<float, __nv_bfloat16><<<grid, 256, 0, stream>>>((const float*)in, in_stride,
                                                                     (__nv_bfloat16*)out, rows, cols);
  else
    return llmrs_fail("tanh_slice: unsupported types %d -> %d", in_dtype, out_dtype);
  return llmrs_launch_status("tanh_slice");
}

// ---------------------------------------------------------------------------------
// The two norms between the branches of a block that norms a branch before AND after it, in one pass over a row:
//   h[t] += y[t] / sqrt(mean(y[t]^2) + eps) * w_out            (the norm on the branch's output and the residual sum)
//   out[t] = h[t] / sqrt(mean(h[t]^2) + eps) * w_next          (the norm ahead of the next branch; w_next null: none)
// One block per row; the row's new values wait in shared memory for their statistics.
// ---------------------------------------------------------------------------------
template <typename TY, typename TO>
__global__ void outnorm_add_norm_kernel(float* __restrict__ h, const TY* __restrict__ y,
                                        const float* __restrict__ w_out, const float* __restrict__ w_next,
                                        TO* __restrict__ out, int width, float eps) {
  extern __shared__ float row[];
  __shared__ float red[33];
  const TY* yr = y + (size_t)blockIdx.x * width;
  float* hr = h + (size_t)blockIdx.x * width;
  float ss = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = to_float(yr[c]);
    ss += v * v;
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)width + eps);
  ss = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = hr[c] + to_float(yr[c]) * inv * w_out[c];
    hr[c] = v;
    row[c] = v;
    ss += v * v;
  }
  const float inv2 = 1.0f / sqrtf(block_sum(ss, red) / (float)width + eps);
  TO* o = out + (size_t)blockIdx.x * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) o[c] = from_float<TO>(row[c] * inv2 * w_next[c]);
}

LLMRS_API int llmrs_outnorm_add_norm(float* h, const void* y, int y_dtype, const float* w_out, const float* w_next,
                                     void* out, int out_dtype, int n_rows, int width, float eps,
                                     cudaStream_t stream) {
  LLMRS_REQUIRE(n_rows >= 0 && width > 0 && width <= 12288, "outnorm_add_norm: rows of 1 to 12288, got %d", width);
  LLMRS_REQUIRE(w_next != nullptr && out != nullptr, "outnorm_add_norm: the second norm needs its weight and output");
  if (n_rows == 0) return 0;
  const int threads = width >= 1024 ? 256 : 128;
  const size_t smem = (size_t)width * sizeof(float);
#define LLMRS_OAN(TY, TO)                                                                                       \
  outnorm_add_norm_kernel<TY, TO><<<n_rows, threads, smem, stream>>>(h, (const TY*)y, w_out, w_next, (TO*)out, \
                                                                     width, eps)
  if (y_dtype == LLMRS_F32 && out_dtype == LLMRS_F32) LLMRS_OAN(float, float);
  else if (y_dtype == LLMRS_BF16 && out_dtype == LLMRS_BF16) LLMRS_OAN(__nv_bfloat16, __nv_bfloat16);
  else if (y_dtype == LLMRS_F32 && out_dtype == LLMRS_BF16) LLMRS_OAN(float, __nv_bfloat16);
  else return llmrs_fail("outnorm_add_norm: unsupported types %d -> %d", y_dtype, out_dtype);
#undef LLMRS_OAN
  return llmrs_launch_status("outnorm_add_norm");
}

// ---------------------------------------------------------------------------------
// out[t] = x[t] / sqrt(mean(x[t]^2) + eps) * w for rows of activations (a column slice of a wider product: x has a
// row stride), statistics in float32. One block per row.
// ---------------------------------------------------------------------------------
template <typename T>
__global__ void rmsnorm_rows_kernel(const T* __restrict__ x, long long x_stride, const float* __restrict__ w,
                                    T* __restrict__ out, int width, float eps) {
  __shared__ float red[33];
  const T* xr = x + (size_t)blockIdx.x * x_stride;
  float ss = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = to_float(xr[c]);
    ss += v * v;
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)width + eps);
  T* o = out + (size_t)blockIdx.x * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) o[c] = from_float<T>(to_float(xr[c]) * inv * w[c]);
}

LLMRS_API int llmrs_rmsnorm_rows(const void* x, long long x_stride, int dtype, const float* w, void* out, int n_rows,
                                 int width, float eps, cudaStream_t stream) {
  LLMRS_REQUIRE(n_rows >= 0 && width > 0 && x_stride >= width, "rmsnorm_rows: bad sizes");
  if (n_rows == 0) return 0;
  const int threads = width >= 1024 ? 256 : 128;
  if (dtype == LLMRS_F32)
    rmsnorm_rows_kernel<float><<<n_rows, threads, 0, stream>>>((const float*)x, x_stride, w, (float*)out, width, eps);
  else if (dtype == LLMRS_BF16)
    rmsnorm_rows_kernel<__nv_bfloat16><<<n_rows, threads, 0, stream>>>((const __nv_bfloat16*)x, x_stride, w,
                                                                       (__nv_bfloat16*)out, width, eps);
  else
    return llmrs_fail("rmsnorm_rows: unknown dtype %d", dtype);
  return llmrs_launch_status("rmsnorm_rows");
}
