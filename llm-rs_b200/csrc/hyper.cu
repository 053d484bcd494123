// Hyper-connections: the residual stream is S copies x_1 .. x_S per token ([tokens, S, width], float32). A sublayer
//
//   reads    u = sum_s in[s] x_s                      and gets  norm(u) = u / sqrt(mean(u^2) + eps) * g  (ONE number g)
//   writes   x_t <- sum_s mix[s, t] x_s + out[t] * y  for all t at once from the old streams (mix is [from, to])
//
// and the model's output is the sum of the streams. Everything is float32; only the normed u is rounded to the
// activation type. One kernel does a sublayer's write and the NEXT sublayer's read and norm in one pass over the
// token's streams (either half may be absent: the first read has no write before it, the last write of a model is
// folded into the sum of the streams, which only the wanted rows need). in, out, mix and g stay on the device.
//
//   hyper_step    [write of (y, mix, out)] then [read with in_next, norm with g_next -> u_out]; a block per token
//   hyper_leave   sum of the streams of the given rows, after a pending write if there is one, as float32 rows
//   scaled_sum    out = a * sa + b * sb, float32 (two branches that run side by side)
#include "common.cuh"

constexpr int HY_MAXS = 16, HY_THREADS = 256;

struct HyperParams {
  float mix[HY_MAXS][HY_MAXS], out[HY_MAXS], in[HY_MAXS];
};

// SMAX: the streams the unrolled loops are built for (the next of 2, 4, 8, 16 at or above S).
template <typename TY, typename TA, int SMAX>
__global__ void __launch_bounds__(HY_THREADS)
hyper_step_kernel(float* __restrict__ x, const TY* __restrict__ y, const float* __restrict__ mix,
                  const float* __restrict__ out, const float* __restrict__ in_next, const float* __restrict__ g_next,
                  TA* __restrict__ u_out, int S, int width, float eps) {
  extern __shared__ float u_row[];      // [width], only with a read
  __shared__ float red[33];
  __shared__ HyperParams p;
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < S * S; i += HY_THREADS) p.mix[i / S][i % S] = y ? mix[i] : 0.f;
  for (int i = threadIdx.x; i < S; i += HY_THREADS) {
    p.out[i] = y ? out[i] : 0.f;
    p.in[i] = in_next ? in_next[i] : 0.f;
  }
  __syncthreads();
  float* xt = x + (size_t)t * S * width;
  float ss = 0.f;
  for (int c = threadIdx.x; c < width; c += HY_THREADS) {
    float xs[SMAX];
#pragma unroll
    for (int s = 0; s < SMAX; ++s) xs[s] = s < S ? xt[(size_t)s * width + c] : 0.f;
    if (y) {
      const float yv = to_float(y[(size_t)t * width + c]);
      float nx[SMAX];
#pragma unroll
      for (int r = 0; r < SMAX; ++r) {
        float a = p.out[r] * yv;
#pragma unroll
        for (int s = 0; s < SMAX; ++s) a = fmaf(p.mix[s][r], xs[s], a);
        nx[r] = a;
      }
#pragma unroll
      for (int r = 0; r < SMAX; ++r)
        if (r < S) xt[(size_t)r * width + c] = xs[r] = nx[r];
    }
    if (in_next) {
      float u = 0.f;
#pragma unroll
      for (int s = 0; s < SMAX; ++s) u = fmaf(p.in[s], xs[s], u);
      u_row[c] = u;
      ss = fmaf(u, u, ss);
    }
  }
  if (!in_next) return;
  const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)width + eps) * g_next[0];
  for (int c = threadIdx.x; c < width; c += HY_THREADS) u_out[(size_t)t * width + c] = from_float<TA>(u_row[c] * inv);
}

// x: [tokens, S, width] float32, changed in place when y is given. y: [tokens, width] (float32 or the activation
// type, `y_dtype`), null: no write. in_next null: no read (u_out unused). u_out: [tokens, width] of `act_dtype`.
LLMRS_API int llmrs_hyper_step(float* x, const void* y, int y_dtype, const float* mix, const float* out,
                               const float* in_next, const float* g_next, void* u_out, int act_dtype, int n_tokens,
                               int S, int width, float eps, cudaStream_t stream) {
  LLMRS_REQUIRE(n_tokens >= 0 && width > 0 && S >= 1 && S <= HY_MAXS, "hyper_step: %d streams of width %d (1..%d streams)",
                S, width, HY_MAXS);
  LLMRS_REQUIRE(y != nullptr || in_next != nullptr, "hyper_step: neither a write nor a read");
  LLMRS_REQUIRE(y == nullptr || (mix != nullptr && out != nullptr), "hyper_step: a write needs mix and out");
  LLMRS_REQUIRE(in_next == nullptr || (g_next != nullptr && u_out != nullptr), "hyper_step: a read needs g and u_out");
  LLMRS_REQUIRE(width <= 48 * 1024, "hyper_step: width %d is too large", width);
  if (n_tokens == 0) return 0;
  const size_t smem = in_next ? (size_t)width * sizeof(float) : 0;
#define LLMRS_HY_LAUNCH_S(TY, TA, SMAX)                                                                              \
  do {                                                                                                                 \
    static size_t configured = 40 * 1024;                                                                              \
    if (smem > configured) {                                                                                           \
      cudaError_t e = cudaFuncSetAttribute(hyper_step_kernel<TY, TA, SMAX>,                                            \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                    \
      if (e != cudaSuccess) return llmrs_fail("hyper_step: shared memory %zu: %s", smem, cudaGetErrorString(e));       \
      configured = smem;                                                                                               \
    }                                                                                                                  \
    hyper_step_kernel<TY, TA, SMAX><<<n_tokens, HY_THREADS, smem, stream>>>(x, (const TY*)y, mix, out, in_next, g_next, \
                                                                            (TA*)u_out, S, width, eps);                \
  } while (0)
#define LLMRS_HY_LAUNCH(TY, TA)                     \
  do {                                              \
    if (S <= 2) LLMRS_HY_LAUNCH_S(TY, TA, 2);       \
    else if (S <= 4) LLMRS_HY_LAUNCH_S(TY, TA, 4);  \
    else if (S <= 8) LLMRS_HY_LAUNCH_S(TY, TA, 8);  \
    else LLMRS_HY_LAUNCH_S(TY, TA, 16);             \
  } while (0)
  const bool y32 = y == nullptr || y_dtype == LLMRS_F32;
  if (!y32 && y_dtype != LLMRS_BF16) return llmrs_fail("hyper_step: unknown y dtype %d", y_dtype);
  if (act_dtype == LLMRS_F32) {
    if (y32) LLMRS_HY_LAUNCH(float, float);
    else LLMRS_HY_LAUNCH(__nv_bfloat16, float);
  } else if (act_dtype == LLMRS_BF16) {
    if (y32) LLMRS_HY_LAUNCH(float, __nv_bfloat16);
    else LLMRS_HY_LAUNCH(__nv_bfloat16, __nv_bfloat16);
  } else {
    return llmrs_fail("hyper_step: unknown dtype %d", act_dtype);
  }
#undef LLMRS_HY_LAUNCH
#undef LLMRS_HY_LAUNCH_S
  return llmrs_launch_status("hyper_step");
}

template <typename TY>
__global__ void __launch_bounds__(HY_THREADS)
hyper_leave_kernel(const float* __restrict__ x, const TY* __restrict__ y, const float* __restrict__ mix,
                   const float* __restrict__ out, const int* __restrict__ rows, float* __restrict__ sum, int S,
                   int width) {
  // sum_t (sum_s mix[s, t] x_s + out[t] y) = sum_s (sum_t mix[s, t]) x_s + (sum_t out[t]) y
  __shared__ float ws[HY_MAXS], wy;
  if (threadIdx.x < S) {
    float a = 1.0f;
    if (y) {
      a = 0.f;
      for (int r = 0; r < S; ++r) a += mix[threadIdx.x * S + r];
    }
    ws[threadIdx.x] = a;
  }
  if (threadIdx.x == 32) {
    float a = 0.f;
    if (y) for (int r = 0; r < S; ++r) a += out[r];
    wy = a;
  }
  __syncthreads();
  const int i = blockIdx.x, t = rows ? rows[i] : i;
  const float* xt = x + (size_t)t * S * width;
  for (int c = threadIdx.x; c < width; c += HY_THREADS) {
    float a = y ? wy * to_float(y[(size_t)t * width + c]) : 0.f;
    for (int s = 0; s < S; ++s) a = fmaf(ws[s], xt[(size_t)s * width + c], a);
    sum[(size_t)i * width + c] = a;
  }
}

// sum: float32 [n_rows, width] = the sum of the streams of row rows[i] (null: row i), after the write of (y, mix, out)
// when y is given; x itself is left as it is.
LLMRS_API int llmrs_hyper_leave(const float* x, const void* y, int y_dtype, const float* mix, const float* out,
                                const int* rows, float* sum, int n_rows, int S, int width, cudaStream_t stream) {
  LLMRS_REQUIRE(n_rows >= 0 && width > 0 && S >= 1 && S <= HY_MAXS, "hyper_leave: %d streams of width %d", S, width);
  LLMRS_REQUIRE(y == nullptr || (mix != nullptr && out != nullptr), "hyper_leave: a write needs mix and out");
  if (n_rows == 0) return 0;
  if (y == nullptr || y_dtype == LLMRS_F32)
    hyper_leave_kernel<float><<<n_rows, HY_THREADS, 0, stream>>>(x, (const float*)y, mix, out, rows, sum, S, width);
  else if (y_dtype == LLMRS_BF16)
    hyper_leave_kernel<__nv_bfloat16><<<n_rows, HY_THREADS, 0, stream>>>(x, (const __nv_bfloat16*)y, mix, out, rows,
                                                                         sum, S, width);
  else
    return llmrs_fail("hyper_leave: unknown y dtype %d", y_dtype);
  return llmrs_launch_status("hyper_leave");
}

__global__ void scaled_sum_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out,
                                  long long n, float sa, float sb) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    out[i] = fmaf(a[i], sa, b[i] * sb);
}

LLMRS_API int llmrs_scaled_sum(const float* a, const float* b, float* out, long long n, float sa, float sb,
                               cudaStream_t stream) {
  LLMRS_REQUIRE(n >= 0, "scaled_sum: bad size");
  if (n == 0) return 0;
  const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
  scaled_sum_kernel<<<blocks, 256, 0, stream>>>(a, b, out, n, sa, sb);
  return llmrs_launch_status("scaled_sum");
}
