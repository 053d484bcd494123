// Two small kernels: an embedding with a hashed table of token pairs, and the PolyNorm activation.
//
//   bigram embedding   h[t] = E[id_t] * scale + B[(id_(t-1) * mul_prev + id_t * mul_cur) mod buckets], and for a sequence's
//                      first token row number `buckets` of B (its last row). The token before a step's first token of a
//                      request is per-request state (one float per slot, exact for ids below 2^24), read and then
//                      replaced by the request's last token of the step by the block of that first token. The result
//                      is written `copies` times side by side (streams of a hyper-connected residual).
//   poly_norm          out = a N(z) + b N(z^2) + c N(z^3) + e per row, powers element by element, N(v) = v /
//                      sqrt(mean(v^2) + eps) over the row; the four numbers come from the device. Sums in float32.
#include "common.cuh"

template <typename TW>
__global__ void bigram_embedding_kernel(const TW* __restrict__ table, const TW* __restrict__ pairs,
                                        const int* __restrict__ ids, const int* __restrict__ token_req,
                                        const int* __restrict__ q_start, const int* __restrict__ n_new,
                                        const int* __restrict__ cached_len, const int* __restrict__ slot_ids,
                                        float* __restrict__ prev_state, float* __restrict__ out, int hidden, int vocab,
                                        int copies, float scale, int buckets, long long mul_prev, long long mul_cur) {
  __shared__ int s_prev;
  const int t = blockIdx.x;
  auto clamp_id = [&](int id) { return id < 0 ? 0 : (id >= vocab ? vocab - 1 : id); };
  const int id = clamp_id(ids[t]);
  if (threadIdx.x == 0) {
    int prev = -1;
    if (pairs) {
      const int req = token_req[t], first = q_start[req];
      if (t > first) {
        prev = clamp_id(ids[t - 1]);
      } else {
        float* st = prev_state + slot_ids[req];
        if (cached_len[req] > 0) prev = (int)*st;
        *st = (float)clamp_id(ids[first + n_new[req] - 1]);
      }
    }
    s_prev = prev;
  }
  __syncthreads();
  const TW* row = table + (size_t)id * hidden;
  const TW* pair = nullptr;
  if (pairs) {
    const long long b = s_prev < 0 ? buckets : ((long long)s_prev * mul_prev + (long long)id * mul_cur) % buckets;
    pair = pairs + (size_t)b * hidden;
  }
  float* o = out + (size_t)t * copies * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = to_float(row[i]) * scale;
    if (pair) v += to_float(pair[i]);
    for (int s = 0; s < copies; ++s) o[(size_t)s * hidden + i] = v;
  }
}

// table: [vocab, hidden]; pairs: [buckets + 1, hidden] of the same type, or null (no pair table: prev_state unused);
// prev_state: float32 [slots]; out: float32 [tokens, copies, hidden].
LLMRS_API int llmrs_bigram_embedding(const void* table, const void* pairs, int table_dtype, const int* ids,
                                     const int* token_req, const int* q_start, const int* n_new,
                                     const int* cached_len, const int* slot_ids, float* prev_state, float* out,
                                     int n_tokens, int hidden, int vocab, int copies, float scale, int buckets,
                                     long long mul_prev, long long mul_cur, cudaStream_t stream) {
  LLMRS_REQUIRE(n_tokens >= 0 && hidden > 0 && vocab > 0 && copies >= 1, "bigram_embedding: bad sizes");
  LLMRS_REQUIRE(pairs == nullptr || (buckets >= 1 && prev_state != nullptr && mul_prev >= 0 && mul_cur >= 0),
                "bigram_embedding: a pair table needs buckets >= 1, multipliers >= 0 and the state");
  LLMRS_REQUIRE(vocab <= (1 << 24), "bigram_embedding: vocabulary %d does not fit the state's float", vocab);
  if (n_tokens == 0) return 0;
  const int threads = hidden >= 1024 ? 256 : 128;
#define LLMRS_BE_LAUNCH(T)                                                                                          \
  bigram_embedding_kernel<T><<<n_tokens, threads, 0, stream>>>((const T*)table, (const T*)pairs, ids, token_req,    \
                                                               q_start, n_new, cached_len, slot_ids, prev_state,    \
                                                               out, hidden, vocab, copies, scale, buckets, mul_prev, \
                                                               mul_cur)
  if (table_dtype == LLMRS_F32) LLMRS_BE_LAUNCH(float);
  else if (table_dtype == LLMRS_BF16) LLMRS_BE_LAUNCH(__nv_bfloat16);
  else return llmrs_fail("bigram_embedding: unknown table dtype %d", table_dtype);
#undef LLMRS_BE_LAUNCH
  return llmrs_launch_status("bigram_embedding");
}

constexpr int PN_THREADS = 256;

template <typename T>
__global__ void __launch_bounds__(PN_THREADS)
poly_norm_kernel(const T* __restrict__ z, const float* __restrict__ coeff, T* __restrict__ out, int width, float eps) {
  __shared__ float red[33];
  const T* zr = z + (size_t)blockIdx.x * width;
  T* o = out + (size_t)blockIdx.x * width;
  float s2 = 0.f, s4 = 0.f, s6 = 0.f;
  for (int c = threadIdx.x; c < width; c += PN_THREADS) {
    const float v = to_float(zr[c]), v2 = v * v;
    s2 += v2;
    s4 = fmaf(v2, v2, s4);
    s6 = fmaf(v2 * v2, v2, s6);
  }
  s2 = block_sum(s2, red);
  s4 = block_sum(s4, red);
  s6 = block_sum(s6, red);
  const float w = (float)width;
  const float a = coeff[0] / sqrtf(s2 / w + eps), b = coeff[1] / sqrtf(s4 / w + eps), c3 = coeff[2] / sqrtf(s6 / w + eps);
  const float e = coeff[3];
  for (int c = threadIdx.x; c < width; c += PN_THREADS) {
    const float v = to_float(zr[c]), v2 = v * v;
    o[c] = from_float<T>(fmaf(a, v, fmaf(b, v2, fmaf(c3, v2 * v, e))));
  }
}

// z, out: [rows, width] contiguous of `dtype`; coeff: float32 [4] on the device (a, b, c, e).
LLMRS_API int llmrs_poly_norm(const void* z, const float* coeff, void* out, int n_rows, int width, float eps, int dtype,
                              cudaStream_t stream) {
  LLMRS_REQUIRE(n_rows >= 0 && width > 0, "poly_norm: bad sizes");
  if (n_rows == 0) return 0;
  if (dtype == LLMRS_F32)
    poly_norm_kernel<float><<<n_rows, PN_THREADS, 0, stream>>>((const float*)z, coeff, (float*)out, width, eps);
  else if (dtype == LLMRS_BF16)
    poly_norm_kernel<__nv_bfloat16><<<n_rows, PN_THREADS, 0, stream>>>((const __nv_bfloat16*)z, coeff,
                                                                       (__nv_bfloat16*)out, width, eps);
  else
    return llmrs_fail("poly_norm: unknown dtype %d", dtype);
  return llmrs_launch_status("poly_norm");
}
